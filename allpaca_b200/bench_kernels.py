"""Times one kernel in isolation, cold in L2, and prints its rate against the roofline.

    python -m allpaca_b200.bench_kernels gemm --m 8 --n 6144 --k 4096 [--splits S] [--partials] [--swiglu]
    python -m allpaca_b200.bench_kernels attention --batch 8 --context 4096
    python -m allpaca_b200.bench_kernels prefill-attention --tokens 2048
    python -m allpaca_b200.bench_kernels latent-decode --batch 8 --context 4096   # single rows in a shared latent
    python -m allpaca_b200.bench_kernels latent-prefill --tokens 2048             # a prompt on per-head keys and values
    python -m allpaca_b200.bench_kernels stream --rows 2048 --width 2048          # norms without statistics, token shift, depth average
    python -m allpaca_b200.bench_kernels recurrent --rows 2048 --seqs 1          # linear-attention recurrences, the norm after a gated sum
    python -m allpaca_b200.bench_kernels versus-reference      # a table: ours against the reference's own kernels

Each call works on the next of several copies of its large operand (together larger than
the 126 MB L2), so every timed launch reads its bytes from HBM.  Times are CUDA events
around ``--iters`` launches after ``--warmup``.  This is the command the summaries under
``profiles/`` were made with (under ``ncu`` with a small ``--iters``).
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch


def _time(fn, iters: int, warmup: int, graph: bool = True) -> float:
    """Microseconds per launch.  The launches are recorded into one CUDA graph and replayed,
    so that the host's launch rate does not bound what is measured."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(warmup + i)
        g.replay()
        torch.cuda.synchronize()
        start.record()
        g.replay()
        stop.record()
    else:
        start.record()
        for i in range(iters):
            fn(warmup + i)
        stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / iters


def bench_gemm(args) -> dict:
    from allpaca_b200 import ops
    M, N, K = args.m, args.n, args.k
    copies = max(2, int(math.ceil(300e6 / (N * K * 2))))
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    S = args.splits or ops.gemm_tc_splits(M, N, K)
    odt = torch.float32 if args.out == "float32" else torch.bfloat16
    kernel = "gemm_tc"
    if (M > 128 and not args.dual and not args.pair and not args.single and (S == 1 or args.whole_tiles)) \
            or args.persistent:
        # the persistent kernel; with --swiglu the rows of w alternate gate and up
        kernel = "gemm_tc_persistent"
        out = torch.empty(M, N // 2 if args.swiglu else N, device="cuda", dtype=odt)
        fn = lambda i: ops.gemm_tc_persistent(a, ws[i % copies], out, pairs=args.swiglu,   # noqa: E731
                                              share_tiles=not args.whole_tiles)
        S = 1
    elif args.pair:
        # a pair of CTAs to a tile of 256 weight rows (cta_group::2); with --swiglu the rows of w alternate
        kernel = "gemm_tc_pair"
        out = torch.empty(M, N // 2 if args.swiglu else N, device="cuda", dtype=odt)
        fn = lambda i: ops.gemm_tc_pair(a, ws[i % copies], out, pairs=args.swiglu,   # noqa: E731
                                        share_tiles=not args.whole_tiles)
        S = 1
    elif args.dual:
        # two weight tiles per CTA
        kernel = "gemm_tc_dual"
        out = torch.empty(M, N, device="cuda", dtype=odt)
        fn = lambda i: ops.gemm_tc_dual(a, ws[i % copies], out)   # noqa: E731
        S = 1
    elif args.residual:
        # few rows: the product adds into the 32-bit residual, writes its bfloat16 copy and the
        # partial sums of squares of its rows (the epilogue of the O and down products of a decode step)
        kernel = "gemm_tc (residual epilogue)"
        out = torch.randn(M, N, device="cuda", dtype=torch.float32)
        xb = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ss = torch.empty(M, ops.gemm_tc_residual_parts(N, S), device="cuda", dtype=torch.float32)
        fn = lambda i: ops.gemm_tc_residual(a, ws[i % copies], out, xb, ss, S)     # noqa: E731
    elif args.swiglu:
        # up to 256 rows: the gated activation in the epilogue of the (cluster) kernel
        out = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
        fn = lambda i: ops.gemm_tc(a, ws[i % copies], out, S, reduce=S > 1, pairs=True)      # noqa: E731
    elif args.partials and S > 1:
        out = torch.empty(S, M, N, device="cuda", dtype=torch.float32)
        fn = lambda i: ops.gemm_tc(a, ws[i % copies], out, S, reduce=False)      # noqa: E731
    else:
        out = torch.empty(M, N, device="cuda", dtype=odt)
        fn = lambda i: ops.gemm_tc(a, ws[i % copies], out, S, reduce=S > 1)       # noqa: E731
    us = _time(fn, args.iters, args.warmup, not args.no_graph)
    ops.check_kernel_status()
    nbytes = N * K * 2 + M * K * 2 + out.numel() * out.element_size()
    flops = 2.0 * M * N * K
    return {"kernel": kernel, "M": M, "N": N, "K": K, "splits": S, "partials": bool(args.partials),
            "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1), "TFLOPs": round(flops / us / 1e6, 1)}


def _paged(batch, context, nkv, hd, P, scattered=False):
    """A cache and block tables: pages in rising order, as a fresh pool hands them out, or
    scattered over the pool (the worst case: one load per page)."""
    pages_per = -(-context // P)
    cache = torch.randn(batch * pages_per, 2, nkv, P, hd, device="cuda", dtype=torch.bfloat16)
    order = torch.randperm(batch * pages_per, device="cuda") if scattered else \
        torch.arange(batch * pages_per, device="cuda")
    return cache, order.to(torch.int32).view(batch, pages_per)


def bench_attention(args) -> dict:
    from allpaca_b200 import ops
    if args.splits:
        forced = args.splits
        ops.decode_splits = lambda *a, **k: forced          # try a slice count other than the plan's
    B, C, nh, nkv, hd, P = args.batch, args.context, args.heads, args.kv_heads, args.head_dim, args.page_size
    per = B * C * 2 * nkv * hd * 2
    copies = max(2, int(math.ceil(300e6 / per)))
    caches = [_paged(B, C, nkv, hd, P, args.scattered_pages) for _ in range(copies)]
    q = torch.randn(B, nh * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    seq = torch.arange(B, device="cuda", dtype=torch.int32)
    start = torch.arange(B + 1, device="cuda", dtype=torch.int32)
    pos = torch.full((B,), C - 1, device="cuda", dtype=torch.int32)
    bufs = {}

    def scratch(name, shape, dtype):
        key = (name, tuple(shape))
        if key not in bufs:
            bufs[key] = torch.empty(shape, device="cuda", dtype=dtype)
        return bufs[key]

    mean = C
    if args.short_context:
        # one long sequence among short ones
        pos[1:] = args.short_context - 1
        mean = (C + (B - 1) * args.short_context) // B
        per = per * mean // C

    def fn(i):
        cache, table = caches[i % copies]
        ops.attention(q, out, cache, table, seq, pos, nh, nkv, hd, 1.0 / math.sqrt(hd), 0, seq_start=start,
                      query_lens=[1] * B, max_context=C, scratch=scratch, use_tma=not args.cp_async,
                      mean_context=0 if args.plan_by_longest else mean)
    us = _time(fn, args.iters, args.warmup, not args.no_graph)
    return {"kernel": "attention_split+merge" if args.cp_async else "attention_split_tma+merge", "batch": B, "context": C, "heads": nh, "kv_heads": nkv,
            "head_dim": hd, "mean_context": mean,
            "splits": ops.decode_splits(B, nh, nkv, C, slots=444 if args.cp_async else 296,
                                        cluster_sizes=() if args.cp_async else (2, 4, 8, 16),
                                        mean_context=0 if args.plan_by_longest else mean),
            "us": round(us, 2),
            "GBps": round(per / us / 1e3, 1)}


def bench_prefill_attention(args) -> dict:
    from allpaca_b200 import ops
    T, nh, nkv, hd, P = args.tokens, args.heads, args.kv_heads, args.head_dim, args.page_size
    cache, table = _paged(1, T, nkv, hd, P, args.scattered_pages)
    q = torch.randn(T, nh * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    seq = torch.zeros(T, device="cuda", dtype=torch.int32)
    start = torch.tensor([0, T], device="cuda", dtype=torch.int32)
    pos = torch.arange(T, device="cuda", dtype=torch.int32)

    def fn(i):
        ops.attention(q, out, cache, table, seq, pos, nh, nkv, hd, 1.0 / math.sqrt(hd), 0, seq_start=start,
                      query_lens=[T], max_context=T, use_tcgen05=not args.mma_sync,
                      wide={"auto": None, "one": False, "two": True}[args.query_tiles])
    us = _time(fn, args.iters, args.warmup, not args.no_graph)
    flops = 4.0 * nh * hd * T * (T + 1) / 2
    return {"kernel": "attention_tile" if args.mma_sync else "attention_tcgen05", "query_tiles": args.query_tiles, "tokens": T, "heads": nh, "kv_heads": nkv, "head_dim": hd,
            "us": round(us, 2), "TFLOPs": round(flops / us / 1e6, 1)}


def bench_latent_decode(args) -> dict:
    """Sequences that bring one row each, all heads against the records ``[latent | rotated key part]`` that
    every head shares (``ops.latent_decode``: the tensor-core kernel and its merge)."""
    from allpaca_b200 import ops
    from allpaca_b200.parts import Workspace
    B, C, nh, R, rot, P = args.batch, args.context, args.heads, args.kv_rank, args.rot_dim, args.page_size
    D = R + rot
    pages_per = -(-C // P)
    per = B * C * D * 2
    copies = max(2, int(math.ceil(300e6 / per)))
    caches = [torch.randn(B * pages_per, P, D, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
    table = torch.arange(B * pages_per, device="cuda", dtype=torch.int32).view(B, pages_per)
    q = torch.randn(B, nh * D, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(B, nh * R, device="cuda", dtype=torch.bfloat16)
    gate = None if args.no_gate else torch.randn(B, nh, device="cuda")
    sink = torch.randn(nh, device="cuda") if args.sink else None
    start = torch.arange(B + 1, device="cuda", dtype=torch.int32)
    pos = torch.full((B,), C - 1, device="cuda", dtype=torch.int32)
    ws = Workspace(torch.device("cuda"))

    def fn(i):
        ops.latent_decode(q, out, caches[i % copies], table, start, pos, B, nh, D, R, 1.0 / math.sqrt(D), gate, C, ws,
                          window=args.window, sink=sink)
    us = _time(fn, args.iters, args.warmup, not args.no_graph)
    seen = min(C, args.window) if args.window > 0 else C              # keys a row reads
    per = B * seen * D * 2
    flops = 2.0 * B * seen * nh * (D + R)
    return {"kernel": "latent_decode+merge", "batch": B, "context": C, "heads": nh, "kv_rank": R, "rot_dim": rot,
            "window": args.window, "sink": bool(args.sink), "us": round(us, 2), "GBps": round(per / us / 1e3, 1), "TFLOPs": round(flops / us / 1e6, 2)}


def bench_latent_prefill(args) -> dict:
    """One prompt on per-head keys and values ``[token][head][key | rotated part | value]`` (what the latent
    mixer's product forms for prompt portions): ``ops.latent_prefill``, or with ``--general`` the tensor-core
    kernel of ``ops.attention_window_bias`` with pages of one token."""
    from allpaca_b200 import ops
    T, nh, dk, dv = args.tokens, args.heads, args.head_dim + args.rot_dim, args.value_dim
    kv = torch.randn(T, nh, 1, dk + dv, device="cuda", dtype=torch.bfloat16)
    where = torch.arange(T, device="cuda", dtype=torch.int32).view(1, T)
    q = torch.randn(T, nh * dk, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, nh * dv, device="cuda", dtype=torch.bfloat16)
    gate = None if args.no_gate else torch.randn(T, nh, device="cuda")
    sink = torch.randn(nh, device="cuda") if args.sink else None
    W = args.window
    start = torch.tensor([0, T], device="cuda", dtype=torch.int32)
    pos = torch.arange(T, device="cuda", dtype=torch.int32)

    def fn(i):
        if args.general:
            ops.attention_window_bias(q, out, kv, where, start, pos, 1, nh, nh, dk, dv, 1.0 / math.sqrt(dk), W, None,
                                      None, single_rows=False, other_rows=True, bias=None, gate=gate, record=dk + dv,
                                      value_offset=dk, sink=sink)
        else:
            ops.latent_prefill(q, out, kv.view(T, nh * (dk + dv)), where, start, pos, 1, nh, dk, dv,
                               1.0 / math.sqrt(dk), gate, window=W, sink=sink)
    us = _time(fn, args.iters, args.warmup, not args.no_graph)
    pairs = T * (T + 1) / 2 if not 0 < W < T else W * (W + 1) / 2 + (T - W) * W      # (row, key) pairs that count
    flops = 2.0 * nh * (dk + dv) * pairs
    return {"kernel": "attention_window_bias_mma" if args.general else "latent_prefill", "tokens": T, "heads": nh, "key_dim": dk, "value_dim": dv,
            "window": W, "sink": bool(args.sink), "us": round(us, 2), "TFLOPs": round(flops / us / 1e6, 1)}


def bench_versus_reference(args) -> dict:
    """The operations of a decode step at the Llama-3.1-8B sizes (8 rows; 2048 keys), and the prompt
    attention of 512 tokens: the reference's own CUDA kernels (32-bit float, its only precision;
    ``baseline/reference_kernels.py``) against this engine's kernel of the same operation in 32-bit
    and in bfloat16 (what serving runs).  Launched from the host one after the other, CUDA events
    around ``--iters`` launches; large operands rotate over copies that together exceed L2."""
    import os
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from allpaca_b200 import ops
    from baseline import reference_kernels
    ref = reference_kernels.load()
    if ref is None:
        return {"unavailable": "the reference's kernels are not built here"}
    H, NH, NKV, HD, INTER, M, KEYS = 4096, 32, 8, 128, 14336, 8, 2048
    rows = []

    def timed(fn):
        return round(_time(fn, args.iters, args.warmup, graph=False), 2)

    def weights(n, k, dtype):
        copies = max(2, int(math.ceil(300e6 / (n * k * torch.empty((), dtype=dtype).element_size()))))
        return [(torch.randn(n, k, device="cuda") * 0.02).to(dtype) for _ in range(min(copies, 8))]

    for name, n, k in (("QKV product", (NH + 2 * NKV) * HD, H), ("O product", H, NH * HD),
                       ("gate and up products + SiLU*up", 2 * INTER, H), ("down product", H, INTER)):
        w32 = weights(n, k, torch.float32)
        a32 = torch.randn(M, k, device="cuda")
        out32 = torch.empty(M, n, device="cuda")
        if name.startswith("gate"):
            act = torch.empty(M, INTER, device="cuda")

            g32, u32 = torch.empty(M, INTER, device="cuda"), torch.empty(M, INTER, device="cuda")

            def theirs(i):
                w = w32[i % len(w32)]
                ref.gemm_nt(a32, w[:INTER], g32)
                ref.gemm_nt(a32, w[INTER:], u32)
                ref.silu_mul(g32, u32, act)

            def ours32(i):
                ops.gemm_simt(a32, w32[i % len(w32)], out32)
                ops.swiglu(out32, act)
        else:
            def theirs(i):
                ref.gemm_nt(a32, w32[i % len(w32)], out32)

            def ours32(i):
                ops.gemm_simt(a32, w32[i % len(w32)], out32)
        t_ref, t32 = timed(theirs), timed(ours32)
        del w32
        w16 = weights(n, k, torch.bfloat16)
        a16 = a32.bfloat16()
        S = ops.gemm_tc_splits(M, n, k)
        if name.startswith("gate"):
            out16 = torch.empty(M, INTER, device="cuda", dtype=torch.bfloat16)

            def ours16(i):
                ops.gemm_tc(a16, w16[i % len(w16)], out16, S, reduce=S > 1, pairs=True)
        else:
            out16 = torch.empty(M, n, device="cuda", dtype=torch.bfloat16)

            def ours16(i):
                ops.gemm_tc(a16, w16[i % len(w16)], out16, S, reduce=S > 1)
        rows.append((f"{name}, {M} x {n} x {k}", t_ref, t32, timed(ours16)))
        del w16
    # norm
    x, w = torch.randn(M, H, device="cuda"), torch.ones(H, device="cuda")
    o32, o16 = torch.empty(M, H, device="cuda"), torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    rows.append((f"RMSNorm, {M} x {H}", timed(lambda i: ref.rmsnorm_rows(x, w, o32, 1e-5)),
                 timed(lambda i: ops.add_rmsnorm(x, w, 1e-5, o32)), timed(lambda i: ops.add_rmsnorm(x, w, 1e-5, o16))))
    # rotation of 8 rows at one position each (the reference: one launch per row, as its decode does)
    q, k = torch.randn(M, NH, HD, device="cuda"), torch.randn(M, NKV, HD, device="cuda")
    qkv = torch.randn(M, (NH + 2 * NKV) * HD, device="cuda")
    pos = torch.arange(100, 100 + M, device="cuda", dtype=torch.int32)
    inv = torch.rand(HD // 2, device="cuda")
    table = torch.empty(M, HD // 2, 2, device="cuda")
    q_out32 = torch.empty(M, NH * HD, device="cuda")
    q_out16 = torch.empty(M, NH * HD, device="cuda", dtype=torch.bfloat16)
    qkv16 = qkv.bfloat16()

    def their_rope(i):
        for r in range(M):
            ref.rope_adjacent(q[r:r + 1], k[r:r + 1], 100 + r, 500000.0)

    def our_rope(out, src):
        def fn(i):
            ops.rope_table(pos, inv, table)
            ops.rope_kv_store(src, out, None, pos, None, None, table, 0, NH, NKV, HD)
        return fn
    rows.append((f"rotation of Q and K, {M} rows", timed(their_rope), timed(our_rope(q_out32, qkv)),
                 timed(our_rope(q_out16, qkv16))))
    # decode attention: 8 sequences of 2048 keys (the reference: one call per sequence)
    kk, vv = torch.randn(M, KEYS, NKV, HD, device="cuda"), torch.randn(M, KEYS, NKV, HD, device="cuda")
    qd = torch.randn(M, 1, NH, HD, device="cuda")
    od = torch.empty_like(qd)

    def their_decode(i):
        for b in range(M):
            ref.attention(qd[b], kk[b], vv[b], od[b], causal=True)
    P = 16
    seq = torch.arange(M, device="cuda", dtype=torch.int32)
    start = torch.arange(M + 1, device="cuda", dtype=torch.int32)
    last = torch.full((M,), KEYS - 1, device="cuda", dtype=torch.int32)
    bufs = {}

    def scratch(name, shape, dtype):
        return bufs.setdefault((name, tuple(shape)), torch.empty(shape, device="cuda", dtype=dtype))

    def our_decode(dtype):
        cache, tbl = _paged(M, KEYS, NKV, HD, P)
        cache = cache.to(dtype)
        qq = torch.randn(M, NH * HD, device="cuda").to(dtype)
        oo = torch.empty_like(qq)
        return lambda i: ops.attention(qq, oo, cache, tbl, seq, last, NH, NKV, HD, HD ** -0.5, 0, seq_start=start,
                                       query_lens=[1] * M, max_context=KEYS, scratch=scratch)
    rows.append((f"decode attention, {M} sequences x {KEYS} keys", timed(their_decode),
                 timed(our_decode(torch.float32)), timed(our_decode(torch.bfloat16))))
    # prompt attention of 512 tokens
    T = 512
    qp, kp, vp = (torch.randn(T, n, HD, device="cuda") for n in (NH, NKV, NKV))
    op = torch.empty_like(qp)

    def our_prompt(dtype):
        cache, tbl = _paged(1, T, NKV, HD, P)
        cache = cache.to(dtype)
        qq = torch.randn(T, NH * HD, device="cuda").to(dtype)
        oo = torch.empty_like(qq)
        ts = torch.zeros(T, device="cuda", dtype=torch.int32)
        st = torch.tensor([0, T], device="cuda", dtype=torch.int32)
        ps = torch.arange(T, device="cuda", dtype=torch.int32)
        return lambda i: ops.attention(qq, oo, cache, tbl, ts, ps, NH, NKV, HD, HD ** -0.5, 0, seq_start=st,
                                       query_lens=[T], max_context=T)
    rows.append((f"prompt attention, {T} tokens, causal", timed(lambda i: ref.attention(qp, kp, vp, op, causal=True)),
                 timed(our_prompt(torch.float32)), timed(our_prompt(torch.bfloat16))))
    ops.check_kernel_status()
    print("| operation | reference kernel (32-bit), us | ours 32-bit, us | ours bfloat16, us | reference / ours bfloat16 |")
    print("|---|---|---|---|---|")
    for name, a, b, c in rows:
        print(f"| {name} | {a} | {b} | {c} | {a / c:.1f}x |")
    return {"rows": [{"operation": n, "reference_us": a, "ours_float32_us": b, "ours_bfloat16_us": c} for n, a, b, c in rows]}


def bench_stream(args) -> dict:
    """The kernels that act on the residual stream element by element (Dynamic Tanh with the pending addition,
    Dynamic Tanh with the mix with the previous token's row, the depth-weighted average over ``--streams`` results,
    bias with the squared ReLU behind a product of ``--ff`` columns), each beside the bytes it must move, and
    ``add_rmsnorm`` on the same rows for comparison."""
    from allpaca_b200 import ops
    T, H, K, F = args.rows, args.width, args.streams, args.ff
    dev = "cuda"
    copies = max(2, int(math.ceil(300e6 / (T * H * 4 * (K + 1)))))
    xs = [torch.randn(T, H, device=dev) for _ in range(copies)]
    deltas = [torch.randn(1, T, H, device=dev) for _ in range(copies)]
    streams = [torch.randn(K + 1, T, H, device=dev) for _ in range(copies)]
    out = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    w, b, shift = torch.randn(H, device=dev), torch.randn(H, device=dev), torch.rand(H, device=dev)
    a = torch.rand(K + 1, device=dev)
    nseq = max(1, args.seqs)
    per = T // nseq
    starts = [i * per for i in range(nseq)] + [T]
    seq_start = torch.tensor(starts, dtype=torch.int32, device=dev)
    token_seq = torch.cat([torch.full((starts[i + 1] - starts[i],), i, dtype=torch.int32) for i in range(nseq)]).to(dev)
    positions = torch.cat([torch.arange(7, 7 + starts[i + 1] - starts[i], dtype=torch.int32) for i in range(nseq)]).to(dev)
    slots = torch.arange(nseq, dtype=torch.int32, device=dev)
    state = torch.zeros(nseq, H, device=dev)
    sums = [torch.randn(T, F, device=dev) for _ in range(max(2, int(math.ceil(300e6 / (T * F * 4)))))]
    act = torch.empty(T, F, device=dev, dtype=torch.bfloat16)
    fb = torch.randn(F, device=dev)
    wb = w.to(torch.bfloat16)
    cases = {
        "add_rmsnorm": (lambda i: ops.add_rmsnorm(xs[i % copies], wb, 1e-6, out, delta=deltas[i % copies]), T * H * 14),
        "add_dyt": (lambda i: ops.add_dyt(xs[i % copies], w, b, 0.7, out, delta=deltas[i % copies]), T * H * 14),
        "dyt_shift": (lambda i: ops.dyt_shift(xs[i % copies], w, b, 0.7, shift, state, seq_start, positions, token_seq,
                                              slots, out), T * H * 6),
        "stream_mix": (lambda i: ops.stream_mix(xs[i % copies], deltas[i % copies], streams[i % copies], K, a),
                       T * H * 4 * (K + 4)),
        "bias_act": (lambda i: ops.bias_act(sums[i % len(sums)], fb, act, "relu2"), T * F * 6),
    }
    E, top = args.experts, args.top
    hb = [torch.randn(T, H, device=dev).to(torch.bfloat16) for _ in range(max(2, int(math.ceil(300e6 / (T * H * 2)))))]
    router = torch.randn(E, H, device=dev).to(torch.bfloat16)
    correction = 0.1 * torch.randn(E, device=dev)
    chosen, share = torch.empty(T, top, dtype=torch.int32, device=dev), torch.empty(T, top, device=dev)
    cases["moe_route_rows"] = (lambda i: ops.moe_route_rows(hb[i % len(hb)], router, correction, chosen, share,
                                                            "softmax_all"), T * H * 2 + E * H * 2)
    res = {"rows": T, "width": H, "streams": K + 1, "ff": F, "seqs": nseq, "experts": E, "top": top}
    for name, (fn, nbytes) in cases.items():
        us = _time(fn, args.iters, args.warmup, not args.no_graph)
        res[name] = {"us": round(us, 2), "MB": round(nbytes / 1e6, 1), "GBps": round(nbytes / us / 1e3, 1)}
    return res


def bench_recurrent(args) -> dict:
    """The linear-attention recurrence in its three kinds (a decay per channel; a fixed decay per head with rotated
    queries and keys; the gated delta rule with unit vectors) on ``--seqs`` sequences of ``--rows`` rows each, beside
    the state-space recurrence of the same state size (``ssm_scan``); and the norm after a gated sum beside
    ``add_rmsnorm`` and ``norm_residual`` on the same rows, each beside the bytes it must move."""
    from allpaca_b200 import ops
    n, S, H, D, V, W = args.rows, max(1, args.seqs), args.heads, args.dim, args.vdim, args.width
    T = n * S
    dev = "cuda"
    copies = max(2, int(math.ceil(300e6 / (T * (3 * H * D + 2 * H * V) * 4))))
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape):
        return torch.randn(*shape, device=dev, generator=g)
    q, k, z = ([rnd(T, H * D) for _ in range(copies)] for _ in range(3))
    v = [rnd(T, H * V) for _ in range(copies)]
    a, b = rnd(T, H), rnd(T, H)
    y = torch.empty(T, H * V, device=dev)
    state = torch.zeros(S, H, D, V, device=dev)
    seq_start = torch.arange(0, T + 1, n, dtype=torch.int32, device=dev)
    positions = torch.cat([torch.arange(7, 7 + n, dtype=torch.int32) for _ in range(S)]).to(dev)
    slots = torch.arange(S, dtype=torch.int32, device=dev)
    token_seq = torch.arange(S, dtype=torch.int32, device=dev).repeat_interleave(n)
    consts = torch.full((H,), 0.99, device=dev)
    a_log, dt_bias = torch.log(0.05 + 0.5 * torch.rand(H, device=dev)), rnd(H)
    table = torch.empty(T, D // 2, 2, device=dev)
    ops.rope_table(positions, torch.pow(10000.0, -torch.arange(D // 2, device=dev) / (D // 2)).float(), table, 1.0)
    common = (y, state, seq_start, positions, slots, S, H, H, D, V)
    io = T * (2 * H * D + 2 * H * V) * 4 + 2 * S * H * D * V * 4
    cases = {
        "la_scan channel": (lambda i: ops.linear_scan(q[i % copies], k[i % copies], v[i % copies], *common, "channel",
                                                      decay_channel=z[i % copies], tau=16.0, out_scale=D ** -0.5),
                            io + T * H * D * 4),
        "la_scan head, rotated": (lambda i: ops.linear_scan(q[i % copies], k[i % copies], v[i % copies], *common, "head",
                                                            decay_const=consts, qk="rotate", cos_sin=table), io),
        "la_scan delta rule": (lambda i: ops.linear_scan(q[i % copies], k[i % copies], v[i % copies], *common,
                                                         "head_token", decay_head=a, decay_const=a_log, dt_bias=dt_bias,
                                                         beta=b, qk="unit", unit_eps=1e-6), io),
    }
    # the state-space recurrence with the same state per head: B and C of D numbers, one group per head
    xbc = [rnd(T, H * V + 2 * H * D) for _ in range(copies)]
    cases["ssm_scan"] = (lambda i: ops.ssm_scan(xbc[i % copies], a, dt_bias, a_log, consts, state, seq_start, positions,
                                                slots, y, S, H, H, D, V), io)
    gate = [rnd(T, H * V) for _ in range(copies)]
    out = torch.empty(T, H * V, device=dev, dtype=torch.bfloat16)
    nw = torch.ones(V, device=dev)
    cases["head_norm_gate"] = (lambda i: ops.head_norm_gate(v[i % copies], gate[i % copies], nw, 1e-6, out, H, V),
                               T * H * V * 10)
    cases["gated_group_rmsnorm"] = (lambda i: ops.gated_group_rmsnorm(v[i % copies], gate[i % copies],
                                                                      torch.ones(H * V, device=dev), 1e-6, out, H),
                                    T * H * V * 10)
    wc = max(2, int(math.ceil(300e6 / (T * W * 12))))
    xs, ds, gs = ([rnd(T, W) for _ in range(wc)] for _ in range(3))
    ds = [d.unsqueeze(0) for d in ds]
    copy = torch.empty(T, W, device=dev, dtype=torch.bfloat16)
    w32, gb = torch.ones(W, device=dev), rnd(W)
    cases["gated_postnorm"] = (lambda i: ops.gated_postnorm(xs[i % wc], w32, args.groups, 1e-6, alpha=2.0, delta=ds[i % wc],
                                                            gate=gs[i % wc], gate_bias=gb, copy=copy), T * W * 18)
    cases["norm_residual"] = (lambda i: ops.norm_residual(xs[i % wc], ds[i % wc], w32, 1e-6, 0.5, copy), T * W * 14)
    cases["add_rmsnorm"] = (lambda i: ops.add_rmsnorm(xs[i % wc], w32.to(torch.bfloat16), 1e-6, copy, delta=ds[i % wc]),
                            T * W * 14)
    res = {"rows_per_seq": n, "seqs": S, "heads": H, "dim": D, "vdim": V, "width": W, "groups": args.groups}
    for name, (fn, nbytes) in cases.items():
        us = _time(fn, args.iters, args.warmup, not args.no_graph)
        res[name] = {"us": round(us, 2), "MB": round(nbytes / 1e6, 1), "GBps": round(nbytes / us / 1e3, 1)}
    return res


def bench_sampling(args) -> dict:
    """The choice of the next token for ``--rows`` rows of logits over ``--vocab`` entries."""
    from allpaca_b200 import ops
    R, V = args.rows, args.vocab
    copies = max(2, int(math.ceil(300e6 / (R * V * 4))))
    logits = [torch.randn(R, V, device="cuda") * args.spread for _ in range(copies)]
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    temp = torch.full((R,), args.temperature, device="cuda")
    top_k = torch.full((R,), args.top_k, dtype=torch.int32, device="cuda")
    top_p = torch.full((R,), args.top_p, device="cuda")
    uniform = torch.rand(R, device="cuda")
    if args.temperature <= 1e-5:
        kernel, fn = "argmax", (lambda i: ops.argmax(logits[i % copies], out))     # noqa: E731
    else:
        kernel = "sample"
        fn = lambda i: ops.sample(logits[i % copies], temp, top_k, top_p, uniform, out)   # noqa: E731
    us = _time(fn, args.iters, args.warmup, not args.no_graph)
    return {"kernel": kernel, "rows": R, "vocab": V, "temperature": args.temperature, "top_k": args.top_k,
            "top_p": args.top_p, "us": round(us, 2), "GBps": round(R * V * 4 / us / 1e3, 1)}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m allpaca_b200.bench_kernels")
    sub = p.add_subparsers(dest="what", required=True)
    for name in ("gemm", "attention", "prefill-attention"):
        s = sub.add_parser(name)
        s.add_argument("--iters", type=int, default=50)
        s.add_argument("--warmup", type=int, default=5)
        s.add_argument("--no-graph", action="store_true", help="launch from the host (for ncu)")
        if name == "gemm":
            s.add_argument("--m", type=int, default=8)
            s.add_argument("--n", type=int, default=4096)
            s.add_argument("--k", type=int, default=4096)
            s.add_argument("--splits", type=int, default=0, help="K slices (0: the kernel's own plan)")
            s.add_argument("--partials", action="store_true", help="write partial sums instead of adding in a cluster")
            s.add_argument("--out", choices=["float32", "bfloat16"], default="bfloat16")
            s.add_argument("--dual", action="store_true", help="more than 64 rows: two weight tiles per CTA")
            s.add_argument("--pair", action="store_true", help="more than 64 rows: a pair of CTAs to a tile (cta_group::2)")
            s.add_argument("--single", action="store_true", help="more than 64 rows: one tile per CTA, not persistent")
            s.add_argument("--persistent", action="store_true", help="the persistent kernel, whatever the plan says")
            s.add_argument("--whole-tiles", action="store_true",
                           help="persistent and pair kernel: never share a tile's K among several CTAs")
            s.add_argument("--swiglu", action="store_true", help="w holds gate and up rows: fused gated activation")
            s.add_argument("--residual", action="store_true",
                           help="few rows: add into a 32-bit residual in the epilogue (with its bfloat16 copy and sums of squares)")
        else:
            s.add_argument("--heads", type=int, default=32)
            s.add_argument("--kv-heads", type=int, default=8)
            s.add_argument("--head-dim", type=int, default=128)
            s.add_argument("--page-size", type=int, default=16)
            s.add_argument("--batch", type=int, default=8)
            s.add_argument("--context", type=int, default=4096)
            s.add_argument("--tokens", type=int, default=2048)
            s.add_argument("--cp-async", action="store_true", help="decode: the cp.async kernel instead of the TMA one")
            s.add_argument("--short-context", type=int, default=0,
                           help="decode: every sequence but the first holds this many keys (0: all hold --context)")
            s.add_argument("--plan-by-longest", action="store_true",
                           help="decode: plan the key slices as if every sequence were as long as the longest")
            s.add_argument("--splits", type=int, default=0, help="key slices (0: the kernel's own plan)")
            s.add_argument("--mma-sync", action="store_true", help="prompt attention with the mma.sync tile kernel")
            s.add_argument("--query-tiles", choices=["auto", "one", "two"], default="auto",
                           help="prompt attention on tcgen05: query tiles to a CTA (auto: by the number of CTAs)")
            s.add_argument("--scattered-pages", action="store_true",
                           help="block tables in random order instead of rising page numbers")
    s = sub.add_parser("sampling")
    s.add_argument("--iters", type=int, default=50)
    s.add_argument("--warmup", type=int, default=5)
    s.add_argument("--no-graph", action="store_true", help="launch from the host (for ncu)")
    s.add_argument("--rows", type=int, default=8)
    s.add_argument("--vocab", type=int, default=128256)
    s.add_argument("--temperature", type=float, default=0.8, help="0: the arg-max kernel")
    s.add_argument("--top-k", type=int, default=40, help="0: off")
    s.add_argument("--top-p", type=float, default=0.95, help="1: off")
    s.add_argument("--spread", type=float, default=3.0, help="standard deviation of the random logits")
    for name in ("latent-decode", "latent-prefill"):
        s = sub.add_parser(name)
        s.add_argument("--iters", type=int, default=50)
        s.add_argument("--warmup", type=int, default=5)
        s.add_argument("--no-graph", action="store_true", help="launch from the host (for ncu)")
        s.add_argument("--heads", type=int, default=16)
        s.add_argument("--kv-rank", type=int, default=512)
        s.add_argument("--rot-dim", type=int, default=64)
        s.add_argument("--head-dim", type=int, default=128, help="unrotated query/key dimensions per head")
        s.add_argument("--value-dim", type=int, default=128)
        s.add_argument("--page-size", type=int, default=16)
        s.add_argument("--batch", type=int, default=8)
        s.add_argument("--context", type=int, default=4096)
        s.add_argument("--tokens", type=int, default=2048)
        s.add_argument("--window", type=int, default=0, help="a row sees its last WINDOW keys only (0: all)")
        s.add_argument("--sink", action="store_true", help="a learned term per head in the softmax's denominator")
        s.add_argument("--no-gate", action="store_true", help="no output gate per head")
        s.add_argument("--general", action="store_true",
                       help="latent-prefill: the general windowed kernel (pages of one token) instead of the one made for it")
    s = sub.add_parser("stream")
    s.add_argument("--iters", type=int, default=50)
    s.add_argument("--warmup", type=int, default=5)
    s.add_argument("--no-graph", action="store_true", help="launch from the host (for ncu)")
    s.add_argument("--rows", type=int, default=2048)
    s.add_argument("--width", type=int, default=2048)
    s.add_argument("--streams", type=int, default=4, help="results before the one the depth average stores")
    s.add_argument("--ff", type=int, default=8192)
    s.add_argument("--seqs", type=int, default=1, help="sequences the rows belong to (one row each: as many as rows)")
    s.add_argument("--experts", type=int, default=18, help="router outputs")
    s.add_argument("--top", type=int, default=4)
    s = sub.add_parser("recurrent")
    s.add_argument("--iters", type=int, default=20)
    s.add_argument("--warmup", type=int, default=3)
    s.add_argument("--no-graph", action="store_true", help="launch from the host (for ncu)")
    s.add_argument("--rows", type=int, default=2048, help="rows of every sequence in the step")
    s.add_argument("--seqs", type=int, default=1)
    s.add_argument("--heads", type=int, default=16)
    s.add_argument("--dim", type=int, default=128)
    s.add_argument("--vdim", type=int, default=128)
    s.add_argument("--width", type=int, default=2048)
    s.add_argument("--groups", type=int, default=4)
    s = sub.add_parser("versus-reference")
    s.add_argument("--iters", type=int, default=20)
    s.add_argument("--warmup", type=int, default=3)
    args = p.parse_args(argv)
    fn = {"gemm": bench_gemm, "attention": bench_attention, "prefill-attention": bench_prefill_attention,
          "sampling": bench_sampling, "versus-reference": bench_versus_reference,
          "stream": bench_stream, "recurrent": bench_recurrent, "latent-decode": bench_latent_decode, "latent-prefill": bench_latent_prefill}[args.what]
    print(json.dumps(fn(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
