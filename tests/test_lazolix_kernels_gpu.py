"""Each mechanism of the Lazolix decoder alone, kernel against the plain implementation, with inputs
made so that a fault shows: a query that looks hard at ONE key (the oldest the window still shows, the
one behind it, a page's first and last slot, far back among hundreds), sinks that weigh as much as the
keys, in prompt portions and in single decoded rows; pages that were given back are filled with NaN."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_lazolix as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def close(got, want, tol, what):
    got, want = got.double().cpu(), want.double()
    err = float((got - want).abs().max() / want.abs().max().clamp(min=1e-30))
    assert torch.isfinite(got).all() and err <= tol, (what, err)


def paged(rows, P, order, first_live=0):
    """rows [T, F] of one sequence -> pages [n, P, F] at the places ``order`` names; NaN where nothing was
    written, zero behind the last token of a page, and NaN again in whole pages before token ``first_live``
    (given back to the pool), whose table entries become -1."""
    T, F = rows.shape
    n = -(-T // P)
    pages = torch.full((max(order) + 1, P, F), float("nan"), dtype=rows.dtype)
    table = []
    for b in range(n):
        if (b + 1) * P <= first_live:
            table.append(-1)
            continue
        part = rows[b * P:(b + 1) * P]
        pages[order[b], :part.shape[0]] = part
        pages[order[b], part.shape[0]:] = 0.0
        table.append(order[b])
    return pages, table


def shuffled(n, base):
    return [base + (7 * b + 3) % n for b in range(n)] if math.gcd(7, n) == 1 else [base + n - 1 - b for b in range(n)]


def layer_case(g, H, D, E, R, dtype):
    """Per-head matrices and sinks of one layer."""
    uk = torch.randn(H * D, R, generator=g) / math.sqrt(R)
    uv = torch.randn(H * E, R, generator=g) / math.sqrt(R)
    sink = torch.randn(H, generator=g)
    sink[0] = 4.0                                    # on head 0 the sink outweighs most keys
    return uk.to(dtype).double(), uv.to(dtype).double(), sink.double()


def sequence_case(g, T, H, D, R, uk, before, window, P, dtype):
    """Latents and queries of one sequence in which chosen rows look hard at one key."""
    latent = torch.randn(T, R, generator=g).to(dtype).double()
    q = torch.randn(T, H, D, generator=g)
    k = (latent @ uk.T).view(T, H, D)
    w = window or T
    spikes = {T - 1: T - w, T - 2: T - 2 - w, before: before - w + 1, before + 1: before + 1 - w,
              before + 2: ((before + 2) // P) * P, T - 3: 17 if not window else (T - 3) // P * P - 1,
              T - 4: max(0, T - 4 - w + 1) // P * P + P - 1}
    for n, (row, key) in enumerate(spikes.items()):
        if 0 <= key <= row < T and row >= before:
            h = n % H
            q[row, h] = 9.0 * math.sqrt(D) * k[key, h].float() / k[key, h].norm()
    return latent, q.double()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,D,E,R,P,window", [(3, 24, 40, 48, 8, 21), (4, 64, 48, 120, 16, 90), (5, 16, 8, 80, 16, None),
                                              (2, 32, 32, 136, 8, 1), (9, 8, 16, 20, 8, 70), (1, 20, 12, 28, 32, 300)])
def test_window_and_sink_in_the_latent_space(dtype, tol, H, D, E, R, P, window):
    """Two sequences in one launch, as the mixer runs them: a portion of 37 rows behind 300 cached tokens and a
    single decoded row at position 333 of another; queries carried into the latent space, one key/value head
    whose value is the key itself.  Pages the window has passed are gone."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(H * 100 + D)
    lens = [(300, 37), (333, 1)]
    scale = 1.0 / math.sqrt(D)
    qs, pages_all, table, want = [], [], [], []
    base = 0
    uk, uv, sink = layer_case(g, H, D, E, R, dtype)
    for before, now in lens:
        T = before + now
        latent, q = sequence_case(g, T, H, D, R, uk, before, window, P, dtype)
        full = plain.windowed_sink_attention(q, latent, uk, uv, sink, scale, window)
        want.append(full[before:])
        # the query in the latent space: q_h U_k[h], rounded as the engine stores it
        qa = torch.einsum("thd,hdr->thr", q[before:], uk.view(H, D, R)).to(dtype)
        qs.append(qa)
        n = -(-T // P)
        pg, row = paged(latent, P, shuffled(n, base), first_live=max(0, before - window + 1) if window else 0)
        pages_all.append(pg[base:])
        table.append(row)
        base += n
    pages = torch.cat(pages_all).to(dtype).to(DEV)
    width = max(len(r) for r in table)
    bt = i32([r + [-1] * (width - len(r)) for r in table])
    Tn = sum(now for _, now in lens)
    qd = torch.cat(qs).reshape(Tn, H * R).to(DEV).contiguous()
    positions = [p for before, now in lens for p in range(before, before + now)]
    for single in ((False, True) if dtype == torch.bfloat16 else (False,)):
        out = torch.full((Tn, H * R), float("nan"), dtype=dtype, device=DEV)
        ops.attention_window_bias(qd, out, pages, bt, i32([0, 37, 38]), i32(positions), 2, H, 1, R, R, scale, window or 0,
                                  None, None, single_rows=single, other_rows=True, bias=None, record=R, value_offset=0,
                                  sink=sink.float().to(DEV))
        got = torch.einsum("thr,her->the", out.double().cpu().view(Tn, H, R), uv.view(H, E, R))
        # the rounding of the latent-space queries is not the plain implementation's: a looser 32-bit bound
        close(got, torch.cat(want), max(tol, 5e-5) if dtype == torch.float32 else tol, ("single rows apart", single))


@pytest.mark.parametrize("H,R,P,window", [(3, 48, 8, 21), (16, 512, 16, 100), (20, 136, 16, 64), (40, 64, 32, 1), (8, 256, 16, None),
                                          (6, 128, 16, 90)])
@pytest.mark.parametrize("max_context", [1, 4096])
def test_single_rows_behind_a_window_on_the_tensor_cores(H, R, P, window, max_context):
    """Sequences of 1 to 2500 tokens that each bring their last row: all heads against the shared latents, keys
    cut into one slice or many, a sink per head.  One head looks hard at the oldest key the window shows, the next
    at the one behind it (which must not count); pages the window has passed hold NaN."""
    from allpaca_b200 import ops
    from allpaca_b200.parts import Workspace
    g = torch.Generator().manual_seed(H + R)
    lens = [1, 64, 65, 130, 700, 2500]
    scale = 1.0 / math.sqrt(R)
    sink = torch.randn(H, generator=g)
    sink[H - 1] = 3.0
    qs, table, pages_all, want = [], [], [], []
    base = 0
    for n in lens:
        rec = torch.randn(n, R, generator=g).to(torch.bfloat16).double()
        q = torch.randn(H, R, generator=g)
        lo = max(0, n - window) if window else 0
        for h, key in ((n % H, lo), ((n + 1) % H, lo - 1), ((n + 2) % H, n // 2 if not window else lo + (n - 1 - lo) // 2)):
            if 0 <= key < n:
                q[h] = 5.0 * math.sqrt(R) * rec[key].float() / rec[key].norm()
        q = q.to(torch.bfloat16).double()
        s = torch.einsum("hd,nd->hn", q, rec[lo:]) * scale
        top = torch.maximum(s.max(dim=-1).values, sink.double())
        e = torch.exp(s - top[:, None])
        want.append((e / (e.sum(-1) + torch.exp(sink.double() - top))[:, None]) @ rec[lo:])
        npg = -(-n // P)
        pg, row = paged(rec, P, shuffled(npg, base), first_live=lo)
        pages_all.append(pg[base:])
        table.append(row)
        base += npg
        qs.append(q)
    pages = torch.cat(pages_all).to(torch.bfloat16).to(DEV)
    width = max(len(r) for r in table)
    bt = i32([r + [-1] * (width - len(r)) for r in table])
    T = len(lens)
    q = torch.stack(qs).reshape(T, H * R).to(torch.bfloat16).to(DEV).contiguous()
    out = torch.full((T, H * R), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert ops.latent_decode_takes(R, R)
    ops.latent_decode(q, out, pages, bt, i32(list(range(T + 1))), i32([n - 1 for n in lens]), T, H, R, R, scale, None,
                      max_context, Workspace(torch.device(DEV)), window=window or 0, sink=sink.to(DEV))
    got = out.float().cpu().view(T, H, R)
    for s, n in enumerate(lens):
        close(got[s], want[s], 2e-2, ("sequence of", n))


@pytest.mark.parametrize("H,DK,DV,window", [(3, 40, 40, 30), (2, 192, 128, 64), (5, 56, 8, 65), (2, 96, 72, 1), (1, 136, 64, None),
                                            (4, 64, 64, 200)])
def test_prompt_rows_on_per_head_keys_behind_a_window(H, DK, DV, window):
    """Three sequences in one launch: 70 rows behind 130 earlier tokens, one row (left alone), and 129 rows from
    position 0; per-head keys and values lie token after token from the first token a sequence's first row sees.
    Chosen rows look hard at the oldest key they see and at the one behind it."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(H + DK)
    lens = [(130, 70), (40, 1), (0, 129)]
    scale = 1.0 / math.sqrt(DK)
    sink = torch.randn(H, generator=g)
    sink[0] = 3.0
    kvs, qs, want, positions, starts, where = [], [], [], [], [0], []
    base = 0
    for before, now in lens:
        T = before + now
        q = torch.randn(T, H, DK, generator=g)
        k = torch.randn(T, H, DK, generator=g).to(torch.bfloat16).double()
        v = torch.randn(T, H, DV, generator=g).to(torch.bfloat16).double()
        w = window or T
        for n, (row, key) in enumerate({T - 1: T - w, T - 2: T - 2 - w, before: before - w + 1, before + 1: before + 1 - w,
                                        T - 3: 63, before + 5: 64}.items()):
            if 0 <= key <= row < T and row >= before:
                q[row, n % H] = 6.0 * math.sqrt(DK) * k[key, n % H].float() / k[key, n % H].norm()
        q = q.to(torch.bfloat16).double()
        s = torch.einsum("ihd,jhd->hij", q, k) * scale
        i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
        s = s.masked_fill((j > i) | (i - j >= w), float("-inf"))
        top = torch.maximum(s.max(dim=-1).values, sink.double()[:, None])
        e = torch.exp(s - top[..., None])
        p = e / (e.sum(-1) + torch.exp(sink.double()[:, None] - top))[..., None]
        want.append(torch.einsum("hij,jhe->ihe", p, v)[before:])
        qs.append(q[before:])
        positions += list(range(before, T))
        starts.append(starts[-1] + now)
        lo = max(0, before - w + 1)
        if now > 1:
            kvs.append(torch.cat([k, v], dim=-1).reshape(T, H * (DK + DV))[lo:])
            where.append([-7] * lo + list(range(base, base + T - lo)))
            base += T - lo
        else:
            where.append([])
    width = max(len(w) for w in where)
    wh = i32([w + [-1] * (width - len(w)) for w in where])
    kv = torch.cat(kvs).to(torch.bfloat16).to(DEV).contiguous()
    T = starts[-1]
    q = torch.cat(qs).reshape(T, H * DK).to(torch.bfloat16).to(DEV).contiguous()
    out = torch.full((T, H * DV), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert ops.latent_prefill_takes(DK, DV)
    ops.latent_prefill(q, out, kv, wh, i32(starts), i32(positions), len(lens), H, DK, DV, scale, None, window=window or 0,
                       sink=sink.to(DEV))
    got = out.float().cpu().view(T, H, DV)
    close(got[:70], want[0], 2e-2, "rows behind earlier tokens")
    close(got[71:], want[2], 2e-2, "rows from position 0")
    assert torch.isnan(got[70]).all(), "the row of a sequence that brings one was written"


@pytest.mark.parametrize("window", [0, 5, 40])
def test_gathered_latents_start_where_the_window_starts(window):
    from allpaca_b200 import ops
    P, R = 8, 24
    lens = [(50, 9), (12, 1), (0, 20), (3, 2)]
    g = torch.Generator().manual_seed(window)
    pages_all, table, recs = [], [], []
    base = 0
    for before, now in lens:
        T = before + now
        rec = torch.randn(T, R, generator=g)
        lo = max(0, before - window + 1) if window else 0
        n = -(-T // P)
        pg, row = paged(rec, P, shuffled(n, base), first_live=lo)
        pages_all.append(pg[base:])
        table.append(row)
        recs.append((rec, lo))
        base += n
    pages = torch.cat(pages_all).to(DEV)
    width = max(len(r) for r in table)
    bt = i32([r + [-1] * (width - len(r)) for r in table])
    starts = [0]
    for _, now in lens:
        starts.append(starts[-1] + now)
    total = sum(b + n - lo for (b, n), (_, lo) in zip(lens, recs) if n > 1)
    span = max(b + n for b, n in lens)
    out = torch.full((total, R), float("nan"), device=DEV)
    where = torch.full((len(lens), span), -5, dtype=torch.int32, device=DEV)
    ops.latent_gather(pages, bt, i32(starts), i32([b + n for b, n in lens]), len(lens), out, where, window)
    where = where.cpu()
    for s, ((before, now), (rec, lo)) in enumerate(zip(lens, recs)):
        if now == 1:
            assert (where[s] == -5).all()
            continue
        rows = where[s, lo:before + now]
        assert (where[s, :lo] == -5).all() and rows.tolist() == list(range(int(rows[0]), int(rows[0]) + before + now - lo))
        assert torch.equal(out[rows.long()].cpu(), rec[lo:])


# ---- the stream's kernels ------------------------------------------------------------------------
@pytest.mark.parametrize("W", [64, 42, 7])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh_with_a_pending_addition_and_chosen_rows(W, dtype):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(W)
    T = 13
    x, d = torch.randn(T, W, generator=g), torch.randn(2, T, W, generator=g)
    w, b, alpha = 1 + 0.3 * torch.randn(W, generator=g), torch.randn(W, generator=g), 0.7
    xd = x.to(DEV)
    out = torch.empty(T, W, dtype=dtype, device=DEV)
    ops.add_dyt(xd, w.to(DEV), b.to(DEV), alpha, out, delta=d.to(DEV))
    v = x + d[0] + d[1]
    assert torch.equal(xd.cpu(), v)                                        # the stream took the addition
    want = plain.dynamic_tanh(v.double(), w.double(), b.double(), torch.tensor(alpha, dtype=torch.float64))
    close(out, want, 1e-6 if dtype == torch.float32 else 5e-3, "all rows")
    rows = [11, 0, 5]
    some = torch.empty(3, W, dtype=dtype, device=DEV)
    ops.add_dyt(xd, w.to(DEV), b.to(DEV), alpha, some, rows=i32(rows))
    close(some, want[rows], 1e-6 if dtype == torch.float32 else 5e-3, "chosen rows")
    assert torch.equal(xd.cpu(), v)


@pytest.mark.parametrize("W", [64, 42])
def test_token_shift_across_portions_and_slots(W):
    """Three requests in two steps on four state slots, in another order in the second step; a request that
    starts at position 0 in a slot that holds another's row; a portion of one row."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(W)
    w, b, mix = 1 + 0.3 * torch.randn(W, generator=g), torch.randn(W, generator=g), torch.rand(W, generator=g)
    alpha = 1.3
    seqs = {"a": torch.randn(9, W, generator=g), "b": torch.randn(1, W, generator=g), "c": torch.randn(6, W, generator=g)}
    al = torch.tensor(alpha, dtype=torch.float64)
    want = {r: plain.token_shift(plain.dynamic_tanh(x.double(), w.double(), b.double(), al), mix.double())
            for r, x in seqs.items()}
    state = torch.full((4, W + 3), 99.0, device=DEV)[:, :W]               # rows wider than the state: a strided view
    slot = {"a": 2, "b": 0, "c": 3}

    def run(parts):
        x = torch.cat([seqs[r][lo:hi] for r, lo, hi in parts]).to(DEV)
        starts, positions, seq_of = [0], [], []
        for n, (r, lo, hi) in enumerate(parts):
            starts.append(starts[-1] + hi - lo)
            positions += list(range(lo, hi))
            seq_of += [n] * (hi - lo)
        out = torch.empty(x.shape, device=DEV)
        ops.dyt_shift(x, w.to(DEV), b.to(DEV), alpha, mix.to(DEV), state, i32(starts), i32(positions), i32(seq_of),
                      i32([slot[r] for r, _, _ in parts]), out)
        at = 0
        for r, lo, hi in parts:
            close(out[at:at + hi - lo], want[r][lo:hi], 1e-6, (r, lo, hi))
            at += hi - lo
    run([("a", 0, 4), ("b", 0, 1), ("c", 0, 1)])
    run([("c", 1, 6), ("a", 4, 5)])
    run([("a", 5, 9)])
    slot["b"] = 2                                                          # a's slot, still holding a's last row
    run([("b", 0, 1)])


@pytest.mark.parametrize("W,out_dtype", [(2048, torch.bfloat16), (2048, torch.float32), (2047, torch.float32)])
def test_token_shift_in_a_step_of_many_rows(W, out_dtype):
    """Enough rows for the kernel to walk runs of four rows per thread: portions that start at every offset of a
    run, portions of one, two and three rows, a request that goes on from its state and one that starts anew."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(W)
    w, b, mix = 1 + 0.3 * torch.randn(W, generator=g), torch.randn(W, generator=g), torch.rand(W, generator=g)
    alpha = 0.8
    lengths = [5, 1, 2, 3, 702, 1, 6, 333, 2, 257]                  # 1312 rows
    first = [0, 3, 0, 9, 0, 0, 1, 40, 7, 0]                          # the position of each portion's first row
    x = torch.randn(sum(lengths), W, generator=g)
    before = torch.randn(len(lengths), W, generator=g)               # what each request's state holds
    al = torch.tensor(alpha, dtype=torch.float64)
    state = before.clone().to(DEV)
    starts, positions, seq_of = [0], [], []
    for n, (L, f) in enumerate(zip(lengths, first)):
        starts.append(starts[-1] + L)
        positions += list(range(f, f + L))
        seq_of += [n] * L
    out = torch.empty(x.shape, device=DEV, dtype=out_dtype)
    ops.dyt_shift(x.to(DEV), w.to(DEV), b.to(DEV), alpha, mix.to(DEV), state, i32(starts), i32(positions), i32(seq_of),
                  i32(list(range(len(lengths)))), out)
    for n, (L, f) in enumerate(zip(lengths, first)):
        normed = plain.dynamic_tanh(x[starts[n]:starts[n + 1]].double(), w.double(), b.double(), al)
        prev = torch.cat([torch.zeros(1, W, dtype=torch.float64) if f == 0 else before[n:n + 1].double(), normed[:-1]])
        want = normed + (prev - normed) * mix.double()
        close(out[starts[n]:starts[n + 1]], want, 1e-6 if out_dtype == torch.float32 else 1e-2, ("portion", n))
        close(state[n:n + 1], normed[-1:], 1e-6, ("state", n))


@pytest.mark.parametrize("T,N", [(5, 64), (300, 88), (7, 43), (129, 1)])
@pytest.mark.parametrize("act", ["relu2", "relu", "gelu_tanh", "silu", None])
def test_bias_and_activation_behind_a_product(T, N, act):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(T + N)
    z, bias = 2 * torch.randn(T, N, generator=g), torch.randn(N, generator=g)
    v = (z + bias).double()
    want = {"relu2": torch.relu(v) ** 2, "relu": torch.relu(v), "silu": v * torch.sigmoid(v), None: v,
            "gelu_tanh": 0.5 * v * (1 + torch.tanh((2 / torch.pi) ** 0.5 * (v + 0.044715 * v ** 3)))}[act]
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 1e-2)):
        out = torch.empty(T, N, device=DEV, dtype=dtype)
        ops.bias_act(z.to(DEV), bias.to(DEV), out, act)
        close(out, want, tol, (act, dtype))
    if act == "relu2":                                               # without a bias
        out = torch.empty(T, N, device=DEV)
        ops.bias_act(z.to(DEV), None, out, act)
        close(out, torch.relu(z.double()) ** 2, 2e-6, "no bias")


def test_depth_average_keeps_every_result():
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(3)
    T, W, count = 5, 42, 4
    streams = torch.full((count, T, W), float("nan"), device=DEV)
    x0 = torch.randn(T, W, generator=g)
    x = x0.to(DEV).clone()
    ops.stream_mix(x, None, streams, 0, None)
    kept = [x0.double()]
    assert torch.equal(x.cpu(), x0) and torch.equal(streams[0].cpu(), x0)
    for k in range(1, count):
        delta = torch.randn(1, T, W, generator=g)
        a = torch.randn(k + 1, generator=g)
        before = x.cpu().double()
        ops.stream_mix(x, delta.to(DEV), streams, k, a.to(DEV))
        kept.append(before + delta[0].double())
        close(streams[k], kept[-1], 1e-6, ("result", k))
        close(x, plain.depth_average(kept, a.double()), 1e-6, ("average", k))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("T", [3, 700])
def test_squared_relu_feed_forward_with_biases(dtype, tol, T):
    from allpaca_b200.parts import BuildEnv, PartSpec, Workspace, build
    g = torch.Generator().manual_seed(T)
    W, F = 64, 88
    env = BuildEnv(dtype=dtype, device=torch.device(DEV), workspace=Workspace(torch.device(DEV)))
    part = build("feed_forward", PartSpec("dense_act", {"hidden_size": W, "intermediate_size": F}), env)
    t = {"up": torch.randn(F, W, generator=g) / 8, "up.b": torch.randn(F, generator=g), "down": torch.randn(W, F, generator=g) / 9,
         "down.b": torch.randn(W, generator=g)}
    t = {k: v.to(dtype) for k, v in t.items()}
    part.load({k: v.to(DEV) for k, v in t.items()})
    h = torch.randn(T, W, generator=g).to(dtype)
    got = part.forward(h.to(DEV), None)[0]
    want = plain.dense_feed_forward(h.double(), *(t[k].double() for k in ("up", "up.b", "down", "down.b")))
    close(got, want, tol, "dense feed-forward")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("T,experts,identity,top", [(5, 6, 2, 3), (300, 4, 1, 2), (9, 3, 1, 4), (40, 5, 0, 1), (600, 2, 3, 2), (7, 0, 3, 2), (1030, 7, 2, 3)])
def test_routed_experts_with_corrected_scores_and_identity_experts(dtype, tol, T, experts, identity, top):
    """Few rows (the streaming kernels) and many (in bfloat16 a product per expert on the tensor cores).  The
    corrections are large against the scores, so that they decide the choice; were they to enter the shares,
    the result would be far off."""
    from allpaca_b200 import ops
    from allpaca_b200.parts import BuildEnv, PartSpec, Workspace, build
    g = torch.Generator().manual_seed(T + experts)
    W, F = 64, 24
    env = BuildEnv(dtype=dtype, device=torch.device(DEV), workspace=Workspace(torch.device(DEV)))
    part = build("feed_forward", PartSpec("routed_experts", {
        "hidden_size": W, "expert_size": F, "experts": experts, "identity": identity, "top": top, "activation": "silu",
        "routing": "softmax_all", "router_bias_name": "correction"}), env)
    t = {"router": torch.randn(experts + identity, W, generator=g) / 4, "correction": 0.5 * torch.randn(experts + identity, generator=g)}
    for e in range(experts):
        t.update({f"e{e}.gate": torch.randn(F, W, generator=g) / 8, f"e{e}.up": torch.randn(F, W, generator=g) / 8,
                  f"e{e}.down": torch.randn(W, F, generator=g) / 5})
    t = {k: v.to(dtype) for k, v in t.items()}
    part.load({k: v.to(DEV) for k, v in t.items()})
    h = torch.randn(T, W, generator=g).to(dtype)
    got = part.forward(h.to(DEV), SimpleNamespace(max_query_len=T))[0]
    w = {"m." + k: v.double() for k, v in t.items()}
    want = plain.routed_feed_forward(h.double(), w, "m.", experts, top)
    # a row whose two candidates lie closer than rounding moves them may choose otherwise: judged without such rows
    scores = torch.softmax(h.double() @ w["m.router"].T, dim=-1) + w["m.correction"]
    ranked = scores.sort(dim=-1, descending=True).values
    clear = (ranked[:, top - 1] - ranked[:, top]) > (1e-5 if dtype == torch.float32 else 2e-2) if top < experts + identity \
        else torch.ones(T, dtype=torch.bool)
    assert clear.sum() >= T // 2
    close(got.cpu()[clear], want[clear], tol, "routed feed-forward")
    ops.check_kernel_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["softmax_all", "top_softmax"])
def test_a_row_is_routed_alike_in_a_step_of_many_rows_and_alone(dtype, mode):
    """A step of many rows routes several rows per CTA: every row's experts and shares have the same bits as
    when the row comes in a small step."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(9)
    T, K, E, top = 1027, 136, 11, 3
    rows = torch.randn(T, K, generator=g).to(dtype).to(DEV)
    router = torch.randn(E, K, generator=g).to(dtype).to(DEV)
    bias = (0.1 * torch.randn(E, generator=g)).to(DEV)
    chosen, weight = torch.empty(T, top, dtype=torch.int32, device=DEV), torch.empty(T, top, device=DEV)
    ops.moe_route_rows(rows, router, bias, chosen, weight, mode)
    for lo, hi in ((0, 5), (509, 512), (1024, 1027)):
        c, w = torch.empty(hi - lo, top, dtype=torch.int32, device=DEV), torch.empty(hi - lo, top, device=DEV)
        ops.moe_route_rows(rows[lo:hi].contiguous(), router, bias, c, w, mode)
        assert torch.equal(c, chosen[lo:hi]) and torch.equal(w, weight[lo:hi]), (lo, hi)
    z = rows.double().cpu() @ router.double().cpu().T
    if mode == "softmax_all":
        s = torch.softmax(z, -1)
        want = torch.topk(s + bias.double().cpu(), top, -1).indices
        share = torch.gather(s, 1, want)
        share = share / share.sum(-1, keepdim=True)
    else:
        v, want = torch.topk(z + bias.double().cpu(), top, -1)
        share = torch.softmax(v, -1)
    same = (want == chosen.cpu()).all(-1)
    assert same.float().mean() > 0.99                       # two scores within rounding of one another may swap
    close(weight[same], share[same], 1e-5 if dtype == torch.float32 else 2e-2, mode)
