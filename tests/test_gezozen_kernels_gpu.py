"""Each mechanism of the Gezozen decoder alone, kernel against the plain implementation, with inputs made so that
a fault shows: one key whose score stands out, far away, just inside and just outside the window, at page
borders, under a soft cap that bounds it, in prompt portions and in single decoded rows; rotation of a part of
the head with stretched frequencies; recurrences of every kind carried over portions and slots that change hands,
with a decay that forgets nothing so that the first token stays readable hundreds of tokens on; the norm after a
gated sum; routing by sigmoid scores with shares on the experts' inputs."""
import math

import pytest
import torch

import plain_gezozen as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
F64 = torch.float64


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def close(got, want, tol, what):
    got, want = got.double().cpu(), want.double()
    err = float((got - want).abs().max() / want.abs().max().clamp(min=1e-30))
    assert torch.isfinite(got).all() and err <= tol, (what, err)


def paged(kv, P, order):
    """kv [T, G, D+E] of one sequence -> (pages [n, G, P, D+E], block-table row) with the sequence's pages at the
    places ``order`` names."""
    T, G, F = kv.shape
    n = -(-T // P)
    pages = torch.full((max(order) + 1, G, P, F), float("nan"))
    for b in range(n):
        rows = kv[b * P:(b + 1) * P]
        pages[order[b], :, :rows.shape[0]] = rows.transpose(0, 1)
        pages[order[b], :, rows.shape[0]:] = 0.0
    return pages, order[:n]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,G,D,E,P,window,cap", [(4, 2, 24, 40, 8, 21, 6.0), (2, 2, 64, 64, 16, 72, None),
                                                  (3, 1, 16, 80, 16, None, 2.5), (8, 4, 64, 128, 16, None, 50.0),
                                                  (6, 2, 64, 64, 16, 40, None), (1, 1, 8, 8, 8, 1, 1.0),
                                                  (2, 1, 20, 12, 8, 11, 9.0), (12, 1, 16, 16, 8, 64, 4.0)])
def test_attention_with_a_key_that_stands_out(dtype, tol, H, G, D, E, P, window, cap):
    """Two sequences in one launch: a portion of 37 rows behind 300 cached tokens and a single decoded row at
    position 333 of another.  In each, one key is made to dominate for chosen rows: far back, at a page's first and
    last slot, the oldest key the window still shows and the one just behind it.  The soft cap bounds how far a
    key can dominate, which a kernel that forgot it would not."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(H * 100 + D)
    lens = [(300, 37), (333, 1)]                       # (cached before, rows now)
    scale = 1.0 / math.sqrt(D)
    qs, pages_all, table, want = [], [], [], []
    base = 0
    for s, (before, now) in enumerate(lens):
        T = before + now
        q = torch.randn(T, H, D, generator=g)
        k = torch.randn(T, G, D, generator=g)
        v = torch.randn(T, G, E, generator=g)
        w = window or T
        spikes = {T - 1: T - w, T - 2: T - 2 - w, before: max(0, before - w + 1), before + 1: (before // P) * P,
                  T - 3: ((T - 3 - min(w, T) + 1 + P - 1) // P) * P + P - 1 if w > 2 * P else T - 3}
        for row, key in spikes.items():
            if 0 <= key <= row < T and row >= before:
                k[key] = 0.3 * k[key] + 4.0 * q[row, ::H // G] / q[row, ::H // G].norm(dim=-1, keepdim=True) * math.sqrt(D)
        q, k, v = (t.to(dtype).float() for t in (q, k, v))
        full = plain.attend(q.double(), k.double(), v.double(), scale, cap, window)
        want.append(full[before:])
        qs.append(q[before:])
        n = -(-T // P)
        order = [base + (7 * b + 3) % n for b in range(n)] if math.gcd(7, n) == 1 else [base + n - 1 - b for b in range(n)]
        pg, row = paged(torch.cat([k, v], dim=-1), P, order)
        pages_all.append(pg[base:])
        table.append(row)
        base += n
    pages = torch.cat(pages_all).to(dtype).to(DEV)
    width = max(len(r) for r in table)
    if window:
        # pages the window has passed were given back: their table entries are void, their contents gone
        for s, (before, now) in enumerate(lens):
            for b in range((before - window + 1) // P if before - window + 1 > 0 else 0):
                pages[table[s][b]] = float("nan")
                table[s][b] = -1
    bt = i32([r + [-1] * (width - len(r)) for r in table])
    q = torch.cat(qs).reshape(-1, H * D).to(dtype).to(DEV).contiguous()
    positions = i32([p for before, now in lens for p in range(before, before + now)])
    for single in (False, True):                       # the general kernels for all rows; the decode kernel for the single row
        out = torch.empty(q.shape[0], H * E, dtype=dtype, device=DEV)
        ops.attention_window_bias(q, out, pages, bt, i32([0, 37, 38]), positions, 2, H, G, D, E, scale, window or 0,
                                  bias=None, softcap=cap or 0.0, single_rows=single)
        close(out.float().reshape(-1, H, E), torch.cat(want), tol, ("attention", single))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,G,D,E,P,window,cap", [(4, 2, 64, 128, 16, None, 30.0), (8, 1, 32, 32, 16, 1100, None),
                                                  (2, 2, 24, 40, 8, None, None)])
def test_single_rows_over_key_slices(dtype, tol, H, G, D, E, P, window, cap):
    """Three sequences that bring one row each, at positions 2100, 1500 and 40, with the step's longest context given:
    the decode kernel then shares a sequence's key tiles between the CTAs of a cluster (the short sequence leaves
    most of them without a key).  One key far back, or the oldest the window shows, is made to dominate."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(D + E)
    scale = 1.0 / math.sqrt(D)
    lens = [2101, 1501, 41]
    qs, pages_all, table, want = [], [], [], []
    base = 0
    for T in lens:
        q = torch.randn(T, H, D, generator=g)
        k = torch.randn(T, G, D, generator=g)
        v = torch.randn(T, G, E, generator=g)
        key = max(0, T - window) if window else T // 3
        k[key] = 0.3 * k[key] + 4.0 * q[T - 1, ::H // G] / q[T - 1, ::H // G].norm(dim=-1, keepdim=True) * math.sqrt(D)
        q, k, v = (t.to(dtype).float() for t in (q, k, v))
        want.append(None)
        # the last row alone: it sees all keys (or the window's)
        lo = max(0, T - window) if window else 0
        s = torch.einsum("hd,tgd->htg", q[-1].double(), k[lo:].double())
        s = torch.stack([s[a, :, a // (H // G)] for a in range(H)]) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        w = torch.softmax(s, dim=-1)
        want[-1] = torch.stack([w[a] @ v[lo:, a // (H // G)].double() for a in range(H)])[None]
        qs.append(q[-1:])
        n = -(-T // P)
        order = [base + n - 1 - b for b in range(n)]
        pg, row = paged(torch.cat([k, v], dim=-1), P, order)
        pages_all.append(pg[base:])
        table.append(row)
        base += n
    pages = torch.cat(pages_all).to(dtype).to(DEV)
    width = max(len(r) for r in table)
    bt = i32([r + [-1] * (width - len(r)) for r in table])
    q = torch.cat(qs).reshape(-1, H * D).to(dtype).to(DEV).contiguous()
    out = torch.empty(3, H * E, dtype=dtype, device=DEV)
    ops.attention_window_bias(q, out, pages, bt, i32([0, 1, 2, 3]), i32([n - 1 for n in lens]), 3, H, G, D, E, scale,
                              window or 0, bias=None, softcap=cap or 0.0, single_rows=True, other_rows=False,
                              max_context=max(lens))
    close(out.float().reshape(-1, H, E), torch.cat(want), tol, "single rows over key slices")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,E,dims,scaling", [(4, 2, 24, 40, 8, (4.0, 64, 8.0, 1.0)), (8, 4, 64, 128, 32, None),
                                                  (3, 1, 20, 12, 20, None), (2, 2, 80, 16, 6, (8.0, 32, 4.0, 0.5))])
def test_bias_norm_rotation_and_store(dtype, H, G, D, E, dims, scaling):
    """The stacked projection's sums with their bias, each query and key head over its root mean square times a
    weight the heads share, the first ``dims`` coordinates turned by the position (far positions too), values
    scaled on their way into the page."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(D + dims)
    positions = [0, 1, 7, 8, 200, 4097, 15]
    T, P = len(positions), 8
    qkv = torch.randn(T, (H + G) * D + G * E + 5, generator=g)
    bias = torch.randn((H + G) * D + G * E, generator=g)
    qw, kw = 1 + 0.3 * torch.randn(D, generator=g), 1 + 0.3 * torch.randn(D, generator=g)
    rot = {"base": 5000.0, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    eps, vs = 1e-5, 0.7
    pos = torch.tensor(positions)
    x = qkv[:, :bias.shape[0]].double() + bias.double()
    q = plain.rotate(plain.rms(x[:, :H * D].reshape(T, H, D), eps) * qw.double(), rot, pos)
    k = plain.rotate(plain.rms(x[:, H * D:(H + G) * D].reshape(T, G, D), eps) * kw.double(), rot, pos)
    v = x[:, (H + G) * D:].reshape(T, G, E) * vs
    f, mag = plain.rotary_frequencies(rot)
    table = torch.empty(T, dims // 2, 2, device=DEV)
    ops.rope_table(i32(positions), f.float().to(DEV), table, mag)
    npages = max(positions) // P + 1
    pages = torch.zeros(npages, G, P, D + E, dtype=dtype, device=DEV)
    q_out = torch.empty(T, H * D, dtype=dtype, device=DEV)
    bt = i32([[(3 * b + 1) % npages for b in range(npages)]])
    ops.qk_norm_store(qkv.to(DEV), q_out, pages, i32(positions), i32([0] * T), bt, H, G, D, E, eps, q_weight=qw.to(DEV),
                      k_weight=kw.to(DEV), bias=bias.to(DEV), cos_sin=table, value_scale=vs)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    near = [i for i, p in enumerate(positions) if p < 1000]
    close(q_out.float().reshape(T, H, D)[near], q[near], tol, "queries")
    close(q_out.float().reshape(T, H, D), q, max(tol, 5e-4), "queries at far positions")     # a 32-bit angle of thousands of radians
    for i, p in enumerate(positions):
        rec = pages[(3 * (p // P) + 1) % npages, :, p % P].float().cpu()
        close(rec[:, :D], k[i], max(tol, 5e-4), ("key", p))
        close(rec[:, D:], v[i], tol, ("value", p))


def recurrence_inputs(kind, H, G, D, V, n, g):
    """(tensors by name, the plain read-out before the norm) for a sequence of n rows."""
    t = {"q": torch.randn(n, G * D, generator=g), "k": torch.randn(n, G * D, generator=g),
         "v": torch.randn(n, H * V, generator=g)}
    if kind == "channel":
        t["z"] = 3.0 + 2.0 * torch.randn(n, H * D, generator=g)
    if kind == "head_token":
        t["a"] = torch.randn(n, H, generator=g)
        t["b"] = torch.randn(n, H, generator=g)
    return t


def plain_read(kind, t, H, G, D, V, consts, rot=None, first=0):
    """The read-out of every row, float64, as the design writes the recurrence."""
    n = t["q"].shape[0]
    q, k = t["q"].double().reshape(n, G, D), t["k"].double().reshape(n, G, D)
    v = t["v"].double().reshape(n, H, V)
    if kind == "head":
        pos = torch.arange(first, first + n)
        q, k = plain.rotate(q, rot, pos), plain.rotate(k, rot, pos) * D ** -0.5
        decay = consts["decay"].double()[None, :, None].expand(n, H, D)
    elif kind == "channel":
        q = q * D ** -0.5
        decay = torch.exp(torch.nn.functional.logsigmoid(t["z"].double()) / consts["tau"]).reshape(n, H, D)
    else:
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        forget = torch.exp(-torch.exp(consts["A_log"].double()) *
                           torch.nn.functional.softplus(t["a"].double() + consts["dt_bias"].double()))
        decay = forget[:, :, None].expand(n, H, D)
        beta = torch.sigmoid(t["b"].double())
    S = torch.zeros(H, D, V, dtype=F64)
    out = torch.zeros(n, H, V, dtype=F64)
    rep = H // G
    for i in range(n):
        kt, qt = k[i].repeat_interleave(rep, dim=0), q[i].repeat_interleave(rep, dim=0)
        S = decay[i][:, :, None] * S
        u = v[i]
        if kind == "head_token":
            u = beta[i][:, None] * (v[i] - torch.einsum("hdv,hd->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        out[i] = torch.einsum("hdv,hd->hv", S, qt)
    return out.reshape(n, H * V)


@pytest.mark.parametrize("kind,H,G,D,V", [("head", 3, 3, 16, 8), ("head", 4, 4, 64, 32), ("head", 1, 1, 6, 10),
                                          ("channel", 5, 5, 8, 12), ("channel", 6, 6, 48, 32), ("channel", 2, 2, 40, 24),
                                          ("channel", 1, 1, 130, 7), ("head_token", 3, 1, 16, 24),
                                          ("head_token", 4, 2, 32, 32), ("head_token", 2, 2, 12, 6),
                                          ("head_token", 8, 2, 128, 64)])
def test_recurrences_carried_over_portions_and_slots(kind, H, G, D, V):
    """Two sequences whose portions share steps (a single row beside a long portion, portions of two rows), on
    slots that held something else before; then a slot that changes hands."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(H * 10 + D)
    rot = {"base": 300.0, "dims": D - D % 2 if D < 20 else 16}
    consts = {"decay": torch.tensor([0.9, 0.97, 0.995, 1.0][:H] + [0.99] * max(H - 4, 0)), "tau": 4.0,
              "A_log": torch.log(0.05 + 0.5 * torch.rand(H, generator=g)), "dt_bias": torch.randn(H, generator=g) - 0.5}
    state = torch.full((2, H, D, V), float("nan"), device=DEV)

    def run(parts):
        """parts: (tensors, first position, slot) per sequence of the step."""
        cat = {n: torch.cat([p[0][n] for p in parts]).to(DEV).contiguous() for n in parts[0][0]}
        starts = [0]
        for p in parts:
            starts.append(starts[-1] + p[0]["q"].shape[0])
        positions = [p[1] + i for p in parts for i in range(p[0]["q"].shape[0])]
        y = torch.empty(starts[-1], H * V, device=DEV)
        kw = {}
        if kind == "head":
            f, mag = plain.rotary_frequencies(rot)
            table = torch.empty(starts[-1], rot["dims"] // 2, 2, device=DEV)
            ops.rope_table(i32(positions), f.float().to(DEV), table, mag)
            kw = dict(decay_const=consts["decay"].to(DEV), qk="rotate", cos_sin=table, out_scale=D ** -0.5)
        elif kind == "channel":
            kw = dict(decay_channel=cat["z"], tau=consts["tau"], out_scale=D ** -0.5)
        else:
            kw = dict(decay_head=cat["a"], decay_const=consts["A_log"].to(DEV), dt_bias=consts["dt_bias"].to(DEV),
                      beta=cat["b"], qk="unit", unit_eps=1e-6, out_scale=D ** -0.5)
        ops.linear_scan(cat["q"], cat["k"], cat["v"], y, state, i32(starts), i32(positions), i32([p[2] for p in parts]),
                        len(parts), H, G, D, V, kind, **kw)
        return [y[starts[j]:starts[j + 1]].cpu() for j in range(len(parts))]

    def cut(t, a, b):
        return {n: x[a:b] for n, x in t.items()}
    ta, tb = recurrence_inputs(kind, H, G, D, V, 41, g), recurrence_inputs(kind, H, G, D, V, 9, g)
    ya, yb = [], []
    r = run([(cut(ta, 0, 17), 0, 1), (cut(tb, 0, 1), 0, 0)]); ya.append(r[0]); yb.append(r[1])
    r = run([(cut(tb, 1, 3), 1, 0), (cut(ta, 17, 18), 17, 1)]); yb.append(r[0]); ya.append(r[1])
    r = run([(cut(ta, 18, 41), 18, 1), (cut(tb, 3, 9), 3, 0)]); ya.append(r[0]); yb.append(r[1])
    close(torch.cat(ya), plain_read(kind, ta, H, G, D, V, consts, rot), 3e-5, "recurrence, long sequence")
    close(torch.cat(yb), plain_read(kind, tb, H, G, D, V, consts, rot), 3e-5, "recurrence, short sequence")
    tc = recurrence_inputs(kind, H, G, D, V, 5, g)
    close(run([(tc, 0, 1)])[0], plain_read(kind, tc, H, G, D, V, consts, rot), 3e-5, "recurrence in a slot used before")


def test_a_state_that_forgets_nothing_keeps_the_first_token():
    """Retention with a decay of exactly 1 and keys that are orthogonal to every query but the last: the last row
    reads the FIRST token's value across 600 tokens cut into portions of many sizes; with the decay below 1 it reads
    that value times decay^599."""
    from allpaca_b200 import ops
    D, V, n = 8, 4, 600
    q = torch.zeros(n, D)
    k = torch.zeros(n, D)
    k[:, 1] = 1.0                                      # every key along coordinate 1 ...
    k[0] = 0.0
    k[0, 0] = 1.0                                      # ... but the first, along coordinate 0
    q[:, 2] = 1.0
    q[-1] = 0.0
    q[-1, 0] = 1.0                                     # the last row asks for coordinate 0
    g = torch.Generator().manual_seed(1)
    v = torch.randn(n, V, generator=g)
    for decay in (1.0, 0.995):
        state = torch.full((1, 1, D, V), float("nan"), device=DEV)
        at, got = 0, []
        for m in [1, 2, 64, 1, 1, 333, 2, 100, 96]:
            y = torch.empty(m, V, device=DEV)
            ops.linear_scan(q[at:at + m].to(DEV), k[at:at + m].to(DEV), v[at:at + m].to(DEV), y, state, i32([0, m]),
                            i32(list(range(at, at + m))), i32([0]), 1, 1, 1, D, V, "head",
                            decay_const=torch.tensor([decay], device=DEV))
            got.append(y.cpu())
            at += m
        assert at == n
        got = torch.cat(got)
        close(got[-1], v[0].double() * decay ** (n - 1), 1e-5, ("the first token's value", decay))
        assert float(got[1:-1].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,V,weighted", [(3, 8, True), (6, 32, True), (4, 40, False), (1, 130, True)])
def test_read_out_norm_and_gate(dtype, H, V, weighted):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(V)
    T = 37
    y = torch.randn(T, H * V + 3, generator=g) * 5
    gate = torch.randn(T, 2 * H * V, generator=g)
    w = (1 + 0.3 * torch.randn(V, generator=g)) if weighted else None
    out = torch.empty(T, H * V, dtype=dtype, device=DEV)
    ops.head_norm_gate(y.to(DEV)[:, :H * V], gate.to(DEV)[:, H * V:], w.to(DEV) if weighted else None, 1e-5, out, H, V,
                       out_scale=0.6)
    o = plain.rms(y[:, :H * V].double().reshape(T, H, V), 1e-5) * (w.double() if weighted else 1.0)
    want = o.reshape(T, H * V) * plain.silu(gate[:, H * V:].double()) * 0.6
    close(out, want, 1e-5 if dtype == torch.float32 else 1e-2, "read-out")


@pytest.mark.parametrize("W,groups,S", [(64, 2, 1), (96, 1, 2), (42, 3, 1), (256, 4, 2), (1024, 16, 1), (80, 80, 1)])
def test_norm_after_a_gated_sum(W, groups, S):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(W)
    T, alpha, eps = 19, 2.5, 1e-5
    x = torch.randn(T, W, generator=g)
    delta = torch.randn(S, T, W, generator=g)
    gate = torch.randn(T, W + 8, generator=g)
    gb = torch.randn(W, generator=g)
    w = 1 + 0.2 * torch.randn(W, generator=g)
    want = plain.group_norm(alpha * x.double() + torch.sigmoid(gate[:, :W].double() + gb.double()) * delta.double().sum(0),
                            w.double(), groups, eps)
    xd = x.to(DEV)
    copy = torch.empty(T, W, dtype=torch.bfloat16, device=DEV)
    ops.gated_postnorm(xd, w.to(DEV), groups, eps, alpha=alpha, delta=delta.to(DEV), gate=gate.to(DEV)[:, :W],
                       gate_bias=gb.to(DEV), copy=copy)
    close(xd, want, 1e-5, "the stream")
    close(copy, want, 1e-2, "its copy")
    # chosen rows only, nothing added, the stream left as it is
    rows = [5, 0, 18]
    out = torch.empty(3, W, device=DEV)
    before = xd.clone()
    ops.gated_postnorm(xd, w.to(DEV), groups, eps, rows=i32(rows), out=out)
    close(out, plain.group_norm(before.double().cpu()[rows], w.double(), groups, eps), 1e-5, "chosen rows")
    assert torch.equal(xd, before)


def build_part(kind, name, params, tensors, dtype):
    from allpaca_b200.parts import BuildEnv, PartSpec, Workspace, build
    dev = torch.device(DEV)
    part = build(kind, PartSpec(name, params), BuildEnv(dtype, dev, Workspace(dev)))
    part.load({k: v.to(dtype).to(dev) for k, v in tensors.items()})
    return part


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("W,F,E,top,shared,T", [(72, 40, 6, 2, 24, 150), (128, 64, 9, 3, 64, 5), (40, 24, 5, 1, None, 70),
                                                (64, 96, 4, 4, 8, 1), (128, 32, 12, 12, 48, 700)])
def test_routed_experts_with_shares_on_their_inputs(dtype, tol, W, F, E, top, shared, T):
    g = torch.Generator().manual_seed(W + E)
    w = {"router": torch.randn(E, W, generator=g) * 0.3}
    names = [f"e{e}." for e in range(E)] + (["shared."] if shared else [])
    for n in names:
        f = shared if n == "shared." else F
        w.update({n + "gate": torch.randn(f, W, generator=g) * 0.25, n + "up": torch.randn(f, W, generator=g) * 0.25,
                  n + "down": torch.randn(W, f, generator=g) * 0.2})
    if shared:
        w["shared.sg"] = torch.randn(1, W, generator=g) * 0.2
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    h = torch.randn(T, W, generator=g).to(dtype)
    if dtype == torch.bfloat16 and top < E:
        top = E                                      # rounding may swap two experts with close scores: choose all
    part = build_part("feed_forward", "routed_experts", {
        "hidden_size": W, "expert_size": F, "experts": E, "top": top, "activation": "silu", "routing": "sigmoid",
        "router_bias": False, "weight_on": "input", "shared": {"size": shared, "gate": True} if shared else None}, w, dtype)

    class Step:
        max_query_len = T
    got = part.forward(h.to(DEV), Step()).sum(0)
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": F}}
    if shared:
        mlp["shared"] = {"ff": shared}
    want = plain.routed_feed_forward({"x." + k: v.double() for k, v in w.items()}, "x.", mlp, h.double())
    close(got, want, tol, "routed feed-forward")


def test_sigmoid_routing_chooses_by_score_and_keeps_the_scores():
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(0)
    T, E, K, top = 300, 11, 48, 3
    rows, router = torch.randn(T, K, generator=g), torch.randn(E, K, generator=g)
    rows[:40] *= 0.1                                   # scores in the middle; the other rows' saturate in 32-bit
    chosen = torch.empty(T, top, dtype=torch.int32, device=DEV)
    weight = torch.empty(T, top, device=DEV)
    ops.moe_route_rows(rows.to(DEV), router.to(DEV), None, chosen, weight, "sigmoid")
    s = torch.sigmoid(rows.double() @ router.double().T)
    best = torch.topk(rows.double() @ router.double().T, top, dim=-1)
    assert torch.equal(chosen.cpu().long(), best.indices)
    best = torch.topk(s, top, dim=-1)
    close(weight, best.values, 1e-6, "scores, not renormalised")
