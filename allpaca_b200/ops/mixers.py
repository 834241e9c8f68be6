"""Python faces of the kernels of the mixers beyond rotary attention, and of the embedding
with a position vector: argument checks, then one C call each (see ``ops/__init__.py``)."""
from __future__ import annotations

from typing import Optional

import torch

from . import AP_F32, KernelError, _check, call, core, dtype_code, stream_handle


def embed_sinusoid_norm(tokens: torch.Tensor, positions: torch.Tensor, table: torch.Tensor,
                        inv_freq: Optional[torch.Tensor], norm_weight: Optional[torch.Tensor], eps: float,
                        x: torch.Tensor, scale: float = 1.0) -> None:
    """``x[t] = norm(table[tokens[t]] * scale + sinusoid(positions[t]))`` into the 32-bit residual.

    The position vector has ``sin(p * inv_freq[i])`` at entry ``2i`` and the cosine at ``2i + 1``
    (``inv_freq`` None: no position vector); the norm is an RMS norm with the weight vector
    ``norm_weight [H]`` (None: no norm)."""
    _check(tokens, "tokens", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    _check(table, "table", dims=2)
    _check(x, "x", torch.float32, 2)
    T, H = x.shape
    if tokens.shape[0] != T or positions.shape[0] < T or table.shape[1] != H:
        raise KernelError("embed_sinusoid_norm: shapes disagree")
    if inv_freq is not None:
        _check(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] * 2 != H:
            raise KernelError("embed_sinusoid_norm: one frequency per pair of entries is needed")
    if norm_weight is not None:
        _check(norm_weight, "norm_weight", dims=1)
        if norm_weight.shape[0] != H:
            raise KernelError("embed_sinusoid_norm: the norm's weight must have one entry per column")
    call(core(), "ap_embed_sinusoid_norm", tokens.data_ptr(), positions.data_ptr(), table.data_ptr(),
         dtype_code(table.dtype), inv_freq.data_ptr() if inv_freq is not None else 0,
         norm_weight.data_ptr() if norm_weight is not None else 0,
         dtype_code(norm_weight.dtype) if norm_weight is not None else AP_F32, float(eps), float(scale),
         x.data_ptr(), T, H, table.shape[0], stream_handle())


BIAS_KINDS = {None: 0, "log": 1, "linear": 2}


def _kv_pages(cache_layer: torch.Tensor, num_kv_heads: int, record: int, name: str):
    """(P, page stride) of pages ``[pages, nkv, P, record]``; with one key/value head the pages may
    come as ``[pages, P, record]``."""
    if cache_layer.dim() == 3 and num_kv_heads == 1:
        cache_layer = cache_layer.unsqueeze(1)
    if cache_layer.dim() != 4 or cache_layer.shape[1] != num_kv_heads or cache_layer.shape[3] != record:
        raise KernelError(f"{name}: pages {tuple(cache_layer.shape)} are not [pages, {num_kv_heads}, P, {record}]")
    if cache_layer.stride(3) != 1 or cache_layer.stride(2) != record \
            or (num_kv_heads > 1 and cache_layer.stride(1) != cache_layer.shape[2] * record):
        raise KernelError(f"{name}: a page must be contiguous")
    return cache_layer.shape[2], cache_layer.stride(0)


def qk_norm_store(qkv: torch.Tensor, q_out: torch.Tensor, cache_layer: Optional[torch.Tensor],
                  positions: torch.Tensor, token_seq: torch.Tensor, block_table: Optional[torch.Tensor],
                  num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, eps: float,
                  normalise: bool = True, temp_coef: float = 0.0, temp_every: int = 0,
                  q_weight: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None,
                  bias: Optional[torch.Tensor] = None, cos_sin: Optional[torch.Tensor] = None,
                  value_scale: float = 1.0) -> None:
    """Prepare the operands of :func:`attention_window_bias` from the stacked projection
    ``qkv [T, nh*D + nkv*D + nkv*VD (+ more columns that are not read)]``: every query and key head
    rescaled to unit mean square (``normalise``) and multiplied by ``q_weight`` / ``k_weight``
    (32-bit ``[D]``, shared by the heads; None: no weight), queries multiplied by
    ``1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1)`` (``temp_every`` 0: no temperature) into
    ``q_out [T, nh*D]``, keys and values into the pages ``cache_layer [pages, nkv, P, D + VD]``
    (None: not stored).  ``bias`` (32-bit, one number per column of Q, K and V) is added to the sums as they are
    read; ``cos_sin [T, r/2, 2]`` turns the first ``r`` coordinates of every normed query and key head, coordinate
    ``i`` with ``i + r/2``; values are multiplied by ``value_scale`` on their way into the page."""
    if qkv.dim() != 2 or not qkv.is_cuda or qkv.stride(1) != 1:
        raise KernelError("qk_norm_store: qkv must be a CUDA matrix with contiguous rows")
    _check(q_out, "q_out", dims=2)
    T = qkv.shape[0]
    for w, n in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            _check(w, n, torch.float32, 1)
            if w.shape[0] != key_dim:
                raise KernelError(f"qk_norm_store: {n} must have one entry per coordinate of a head")
    if qkv.shape[1] < (num_heads + num_kv_heads) * key_dim + num_kv_heads * value_dim \
            or q_out.shape[0] < T or q_out.shape[1] != num_heads * key_dim:
        raise KernelError(f"qk_norm_store: shapes disagree: qkv {tuple(qkv.shape)}, q_out {tuple(q_out.shape)}")
    _check(positions, "positions", torch.int32, 1)
    rot_dims = 0
    if cos_sin is not None:
        _check(cos_sin, "cos_sin", torch.float32, 3)
        rot_dims = 2 * cos_sin.shape[1]
        if cos_sin.shape[0] < T or cos_sin.shape[2] != 2 or rot_dims > key_dim:
            raise KernelError(f"qk_norm_store: cos_sin {tuple(cos_sin.shape)} is not [T, r/2, 2] with r <= {key_dim}")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.shape[0] != (num_heads + num_kv_heads) * key_dim + num_kv_heads * value_dim:
            raise KernelError("qk_norm_store: the bias must have one entry per column of Q, K and V")
    P, page_stride, cptr, tsptr, btptr, maxb = 1, 0, 0, 0, 0, 0
    if cache_layer is not None:
        if cache_layer.dtype != q_out.dtype:
            raise KernelError("qk_norm_store: the pages must have the queries' type")
        P, page_stride = _kv_pages(cache_layer, num_kv_heads, key_dim + value_dim, "qk_norm_store")
        _check(token_seq, "token_seq", torch.int32, 1)
        _check(block_table, "block_table", torch.int32, 2)
        cptr, tsptr, btptr, maxb = cache_layer.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(), \
            block_table.shape[1]
    call(core(), "ap_qk_norm_store", qkv.data_ptr(), dtype_code(qkv.dtype), qkv.stride(0), q_out.data_ptr(), cptr,
         dtype_code(q_out.dtype), positions.data_ptr(), tsptr, btptr, maxb, T, num_heads, num_kv_heads, key_dim,
         value_dim, P, page_stride, float(eps), 1 if normalise else 0, float(temp_coef), int(temp_every),
         q_weight.data_ptr() if q_weight is not None else 0, k_weight.data_ptr() if k_weight is not None else 0,
         bias.data_ptr() if bias is not None else 0, cos_sin.data_ptr() if cos_sin is not None else 0, rot_dims,
         float(value_scale), stream_handle())


def attention_window_bias(q: torch.Tensor, out: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor,
                          seq_start: torch.Tensor, positions: torch.Tensor, num_seqs: int, num_heads: int,
                          num_kv_heads: int, key_dim: int, value_dim: int, scale: float, window: int = 0,
                          r1: Optional[torch.Tensor] = None, r2: Optional[torch.Tensor] = None,
                          single_rows: bool = False, other_rows: bool = True, bias: Optional[str] = "log",
                          keep_first: int = 0, gate: Optional[torch.Tensor] = None,
                          record: Optional[int] = None, value_offset: Optional[int] = None,
                          sink: Optional[torch.Tensor] = None, softcap: float = 0.0, max_context: int = 0) -> None:
    """Causal attention of ``q [T, nh*D]`` over pages ``[pages, nkv, P, record]`` into
    ``out [T, nh*VD]``: ``score = cap(q.k * scale) - bias_h(distance)`` (``cap(s) = softcap * tanh(s / softcap)``
    where ``softcap`` is positive, else ``s``), over the last ``window`` keys (0: all)
    and, behind a window, the sequence's first ``keep_first`` tokens; ordinary softmax, 32-bit.

    ``bias``: ``"log"``: ``r1[h] * ln(1 + r2[h] * distance)``; ``"linear"``: ``r1[h] * distance``; None: no
    bias (``r1``, ``r2`` 32-bit ``[nh]``; without ``r1`` there is no bias whatever ``bias`` says).
    ``gate`` (32-bit ``[T, nh]``, may be a strided view): head ``h`` of row ``t`` is multiplied by
    ``sigmoid(gate[t, h])``.  A token's record holds its key at 0 and its value at ``value_offset``
    (default: side by side, ``record = D + VD`` and ``value_offset = D``).  ``sink`` (32-bit ``[nh]``): the
    softmax's denominator also holds ``exp(sink[h])``, an extra logit to which no value belongs.

    ``single_rows``: ``"skip"``: sequences that bring one row are left out (the caller serves them
    otherwise); True: sequences that bring one row run on the kernel made for decoding (the query
    heads of a key/value head together, the key tiles spread over the warps); ``other_rows`` says
    whether the step has sequences of another length as well (they run on the general kernel,
    which serves everything when ``single_rows`` is False).  ``max_context`` (0: not known): the longest context
    among the sequences that bring one row; from a thousand visible keys on, the decode kernel shares a
    sequence's key tiles between the CTAs of a cluster."""
    _check(q, "q", dims=2)
    _check(out, "out", q.dtype, 2)
    T = q.shape[0]
    if q.shape[1] != num_heads * key_dim or tuple(out.shape) != (T, num_heads * value_dim):
        raise KernelError("attention_window_bias: q/out do not match the heads")
    if cache_layer.dtype != q.dtype:
        raise KernelError("attention_window_bias: the pages must have the queries' type")
    record = key_dim + value_dim if record is None else int(record)
    value_offset = key_dim if value_offset is None else int(value_offset)
    P, page_stride = _kv_pages(cache_layer, num_kv_heads, record, "attention_window_bias")
    if r1 is None:
        bias = None
    if bias not in BIAS_KINDS:
        raise KernelError(f"attention_window_bias: bias {bias!r} is not known (log, linear, None)")
    gptr, gld = 0, 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.dim() != 2 or gate.shape[0] < T or gate.shape[1] != num_heads \
                or gate.stride(1) != 1 or not gate.is_cuda:
            raise KernelError("attention_window_bias: the gate must be 32-bit [T, heads] with contiguous rows")
        gptr, gld = gate.data_ptr(), gate.stride(0)
    _check(block_table, "block_table", torch.int32, 2)
    _check(seq_start, "seq_start", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    if seq_start.shape[0] < num_seqs + 1 or block_table.shape[0] < num_seqs:
        raise KernelError("attention_window_bias: seq_start or the block table is shorter than the sequences")
    for t, n in ((r1, "r1"), (r2, "r2"), (sink, "sink")):
        if t is not None:
            _check(t, n, torch.float32, 1)
            if t.shape[0] != num_heads:
                raise KernelError(f"attention_window_bias: {n} must have one entry per head")
    call(core(), "ap_attention_window_bias", q.data_ptr(), out.data_ptr(), cache_layer.data_ptr(), dtype_code(q.dtype),
         block_table.data_ptr(), block_table.shape[1], seq_start.data_ptr(), positions.data_ptr(), int(num_seqs), T,
         num_heads, num_kv_heads, key_dim, value_dim, P, page_stride, float(scale), float(softcap or 0.0),
         int(window or 0),
         r1.data_ptr() if r1 is not None else 0, r2.data_ptr() if r2 is not None else 0,
         2 if single_rows == "skip" else (1 if single_rows else 0), 1 if other_rows else 0, record, value_offset, BIAS_KINDS[bias], int(keep_first or 0),
         gptr, gld, sink.data_ptr() if sink is not None else 0, int(max_context or 0), stream_handle())


def latent_prepare(proj: torch.Tensor, q_col: int, q_rank: int, q_weight: Optional[torch.Tensor],
                   q_latent: Optional[torch.Tensor], kv_col: int, kv_rank: int, rot_dim: int, rot_dims: int,
                   kv_weight: Optional[torch.Tensor], cache_layer: Optional[torch.Tensor], positions: torch.Tensor,
                   token_seq: torch.Tensor, block_table: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor],
                   eps: float) -> None:
    """From the stacked down-projections ``proj [T, ...]`` (32-bit): columns ``q_col .. q_col + q_rank``
    RMS-normed with ``q_weight`` into ``q_latent [T, q_rank]``; columns ``kv_col .. kv_col + kv_rank``
    RMS-normed with ``kv_weight`` and the ``rot_dim`` columns behind them rotated (the first ``rot_dims``
    of them, entry ``i`` paired with ``i + rot_dims/2``, by ``cos_sin [T, rot_dims/2, 2]``) into the
    row's page and slot of ``cache_layer [pages, P, kv_rank + rot_dim]`` (None: not stored)."""
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1 or not proj.is_cuda:
        raise KernelError("latent_prepare: proj must be a 32-bit CUDA matrix with contiguous rows")
    T = proj.shape[0]
    qptr = qwptr = cptr = kvwptr = tsptr = btptr = csptr = 0
    P, page_stride, maxb, act = 1, 0, 0, None
    if q_rank > 0:
        _check(q_latent, "q_latent", dims=2)
        _check(q_weight, "q_weight", torch.float32, 1)
        if tuple(q_latent.shape) != (T, q_rank) or q_weight.shape[0] != q_rank or q_col + q_rank > proj.shape[1]:
            raise KernelError("latent_prepare: the query latent's shapes disagree")
        qptr, qwptr, act = q_latent.data_ptr(), q_weight.data_ptr(), q_latent.dtype
    if cache_layer is not None:
        _check(kv_weight, "kv_weight", torch.float32, 1)
        if kv_weight.shape[0] != kv_rank or kv_col + kv_rank + rot_dim > proj.shape[1]:
            raise KernelError("latent_prepare: the key/value latent's shapes disagree")
        if act is not None and cache_layer.dtype != act:
            raise KernelError("latent_prepare: the pages must have the query latent's type")
        act = cache_layer.dtype
        P, page_stride = _kv_pages(cache_layer, 1, kv_rank + rot_dim, "latent_prepare")
        _check(token_seq, "token_seq", torch.int32, 1)
        _check(block_table, "block_table", torch.int32, 2)
        cptr, kvwptr, tsptr, btptr, maxb = cache_layer.data_ptr(), kv_weight.data_ptr(), token_seq.data_ptr(), \
            block_table.data_ptr(), block_table.shape[1]
        if rot_dims > 0:
            _check(cos_sin, "cos_sin", torch.float32, 3)
            if tuple(cos_sin.shape) != (T, rot_dims // 2, 2):
                raise KernelError("latent_prepare: cos_sin must be [T, rot_dims/2, 2]")
            csptr = cos_sin.data_ptr()
    if act is None:
        return
    _check(positions, "positions", torch.int32, 1)
    call(core(), "ap_latent_prepare", proj.data_ptr(), proj.stride(0), int(q_col), int(q_rank), qwptr, qptr,
         int(kv_col), int(kv_rank), int(rot_dim), int(rot_dims), kvwptr, cptr, dtype_code(act), positions.data_ptr(),
         tsptr, btptr, maxb, P, page_stride, csptr, float(eps), T, stream_handle())


def head_project(inp: torch.Tensor, weight: Optional[torch.Tensor], out: torch.Tensor, heads: int, tail: int = 0,
                 tail_dims: int = 0, cos_sin: Optional[torch.Tensor] = None) -> None:
    """``out[t, h, :N] = inp[t, h, :K] @ weight[h]`` for ``weight [heads, K, N]``, every sum 32-bit in
    ascending ``k``.  ``inp [T, heads*(K + tail)]`` and ``out [T, heads*(N + tail)]``: the ``tail``
    numbers behind a head's ``K`` inputs go behind its ``N`` outputs, the first ``tail_dims`` of them
    rotated by ``cos_sin [T, tail_dims/2, 2]`` (entry ``i`` paired with ``i + tail_dims/2``).  With
    ``weight`` None the ``K`` numbers are copied (``out`` has ``inp``'s shape): a rotation alone."""
    if inp.dim() != 2 or not inp.is_cuda or inp.stride(1) != 1:
        raise KernelError("head_project: inp must be a CUDA matrix with contiguous rows (it may be a view of wider rows)")
    _check(out, "out", dims=2)
    T = inp.shape[0]
    if weight is None:
        H = heads
        K = N = inp.shape[1] // H - tail
        if K <= 0:
            raise KernelError("head_project: without a matrix the rows must hold more than the tails")
        weight_ptr, weight_code = 0, dtype_code(out.dtype)
    else:
        _check(weight, "weight", dims=3)
        H, K, N = weight.shape
        weight_ptr, weight_code = weight.data_ptr(), dtype_code(weight.dtype)
    if H != heads or inp.shape[1] != H * (K + tail) or tuple(out.shape) != (T, H * (N + tail)):
        raise KernelError(f"head_project: inp {tuple(inp.shape)}, weight {tuple(weight.shape)} and out "
                          f"{tuple(out.shape)} disagree (tail {tail})")
    csptr = 0
    if tail_dims > 0:
        _check(cos_sin, "cos_sin", torch.float32, 3)
        if tuple(cos_sin.shape) != (T, tail_dims // 2, 2):
            raise KernelError("head_project: cos_sin must be [T, tail_dims/2, 2]")
        csptr = cos_sin.data_ptr()
    call(core(), "ap_head_project", inp.data_ptr(), dtype_code(inp.dtype), inp.stride(0), K + tail, weight_ptr,
         weight_code, out.data_ptr(), dtype_code(out.dtype), out.stride(0), N + tail, T, H, K, N,
         int(tail), int(tail_dims), csptr, stream_handle())


def causal_conv_silu(inp: torch.Tensor, col0: int, weight: torch.Tensor, bias: Optional[torch.Tensor],
                     state: Optional[torch.Tensor], token_seq: torch.Tensor, seq_start: torch.Tensor,
                     positions: torch.Tensor, state_slots: torch.Tensor, out: torch.Tensor, num_seqs: int) -> None:
    """``out[t, c] = silu(bias[c] + sum_j weight[c, j] * in[t - (taps-1) + j, col0 + c])`` per
    sequence, inputs of negative positions being zero; ``state [slots, taps-1, C]`` (32-bit, may be a strided
    view of the slots' rows) supplies the inputs from before the step and is brought up to date."""
    _check(inp, "in", torch.float32, 2)
    _check(weight, "weight", torch.float32, 2)
    _check(out, "out", torch.float32, 2)
    T, C = out.shape
    taps = weight.shape[1]
    if weight.shape[0] != C or inp.shape[0] < T or inp.shape[1] < col0 + C:
        raise KernelError("causal_conv_silu: shapes disagree")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    sptr, sstride = 0, 0
    if taps > 1:
        if state is None or state.dtype != torch.float32 or state.dim() != 3 \
                or tuple(state.shape[1:]) != (taps - 1, C) or state.stride(2) != 1 or state.stride(1) != C:
            raise KernelError("causal_conv_silu: the state must be 32-bit [slots, taps-1, C] with contiguous rows")
        sptr, sstride = state.data_ptr(), state.stride(0)
    for t, n in ((token_seq, "token_seq"), (seq_start, "seq_start"), (positions, "positions"),
                 (state_slots, "state_slots")):
        _check(t, n, torch.int32, 1)
    call(core(), "ap_causal_conv_silu", inp.data_ptr(), inp.stride(0), int(col0), weight.data_ptr(),
         bias.data_ptr() if bias is not None else 0, sptr, sstride, token_seq.data_ptr(), seq_start.data_ptr(),
         positions.data_ptr(), state_slots.data_ptr(), out.data_ptr(), T, int(num_seqs), C, taps, stream_handle())


def ssm_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: Optional[torch.Tensor], a_log: torch.Tensor,
             d_skip: Optional[torch.Tensor], state: torch.Tensor, seq_start: torch.Tensor, positions: torch.Tensor,
             state_slots: torch.Tensor, y: torch.Tensor, num_seqs: int, heads: int, groups: int, state_size: int,
             value_dim: int) -> None:
    """The recurrence of a selective state-space layer with one decay per head, all 32-bit:
    ``dt = softplus(dt_raw + dt_bias)``, ``S = exp(-exp(a_log) dt) S + dt B x^T``,
    ``y = S^T C + d_skip x``.  ``xbc [T, heads*vdim + 2*groups*N]`` holds x, B and C side by side;
    ``dt_raw [T, heads]`` may be a strided view; ``state [slots, heads, N, vdim]`` may be a strided
    view of the slots' rows.  A sequence whose first row has position 0 starts from zero."""
    _check(xbc, "xbc", torch.float32, 2)
    _check(y, "y", torch.float32, 2)
    T = y.shape[0]
    inner = heads * value_dim
    if tuple(xbc.shape) != (T, inner + 2 * groups * state_size) or y.shape[1] != inner:
        raise KernelError("ssm_scan: xbc/y do not match the sizes")
    if dt_raw.dtype != torch.float32 or dt_raw.dim() != 2 or dt_raw.shape[0] < T or dt_raw.shape[1] != heads \
            or dt_raw.stride(1) != 1:
        raise KernelError("ssm_scan: dt_raw must be 32-bit [T, heads] with contiguous rows")
    if state.dtype != torch.float32 or state.dim() != 4 or tuple(state.shape[1:]) != (heads, state_size, value_dim) \
            or not state[0].is_contiguous():
        raise KernelError("ssm_scan: the state must be 32-bit [slots, heads, N, vdim] with contiguous rows")
    for t, n in ((dt_bias, "dt_bias"), (a_log, "a_log"), (d_skip, "d_skip")):
        if t is not None:
            _check(t, n, torch.float32, 1)
            if t.shape[0] != heads:
                raise KernelError(f"ssm_scan: {n} must have one entry per head")
    for t, n in ((seq_start, "seq_start"), (positions, "positions"), (state_slots, "state_slots")):
        _check(t, n, torch.int32, 1)
    call(core(), "ap_ssm_scan", xbc.data_ptr(), xbc.stride(0), dt_raw.data_ptr(), dt_raw.stride(0),
         dt_bias.data_ptr() if dt_bias is not None else 0, a_log.data_ptr(),
         d_skip.data_ptr() if d_skip is not None else 0, state.data_ptr(), state.stride(0), seq_start.data_ptr(),
         positions.data_ptr(), state_slots.data_ptr(), y.data_ptr(), T, int(num_seqs), heads, groups, state_size,
         value_dim, stream_handle())


def gated_group_rmsnorm(y: torch.Tensor, z: torch.Tensor, weight: Optional[torch.Tensor], eps: float,
                        out: torch.Tensor, parts: int) -> None:
    """``out = rmsnorm(y * silu(z)) * weight`` where a row is cut into ``parts`` slices of equal
    length and every slice is normalised on its own; ``y [T, inner]`` 32-bit, ``z`` a 32-bit (strided) view of the
    same shape."""
    _check(y, "y", torch.float32, 2)
    _check(out, "out", dims=2)
    T, inner = y.shape
    if z.dtype != torch.float32 or z.dim() != 2 or z.shape[0] < T or z.shape[1] != inner or z.stride(1) != 1 \
            or tuple(out.shape) != (T, inner):
        raise KernelError("gated_group_rmsnorm: shapes disagree")
    if weight is not None:
        _check(weight, "weight", dims=1)
    call(core(), "ap_gated_group_rmsnorm", y.data_ptr(), z.data_ptr(), z.stride(0),
         weight.data_ptr() if weight is not None else 0, dtype_code(weight.dtype) if weight is not None else AP_F32,
         float(eps), out.data_ptr(), dtype_code(out.dtype), T, inner, int(parts), stream_handle())


def latent_gather(cache_layer: torch.Tensor, block_table: torch.Tensor, seq_start: torch.Tensor,
                  context_lens: torch.Tensor, num_seqs: int, out: torch.Tensor, where: torch.Tensor,
                  window: int = 0) -> None:
    """The records of all tokens (0 to the last of this step) of every sequence that brings several
    rows, from the pages ``cache_layer [pages, P, record]`` into the rows of ``out [total, record]`` in
    sequence order; ``where [num_seqs, width]`` (int32) receives, for token ``j`` of sequence ``s``, its
    row in ``out``.  ``total`` must be the sum of those sequences' context lengths.  Behind a ``window``
    (0: none) only the tokens from ``first - window + 1`` on are gathered, ``first`` being the position of
    the sequence's first row of this step (earlier entries of ``where`` are left alone), and ``total``
    counts those."""
    if cache_layer.dim() != 3 or not cache_layer.is_cuda or not cache_layer[0].is_contiguous():
        raise KernelError("latent_gather: the pages must be [pages, P, record] with contiguous pages")
    _check(out, "out", cache_layer.dtype, 2)
    _check(where, "where", torch.int32, 2)
    _check(block_table, "block_table", torch.int32, 2)
    _check(seq_start, "seq_start", torch.int32, 1)
    _check(context_lens, "context_lens", torch.int32, 1)
    if out.shape[1] != cache_layer.shape[2] or where.shape[0] < num_seqs or seq_start.shape[0] < num_seqs + 1:
        raise KernelError("latent_gather: shapes disagree")
    call(core(), "ap_latent_gather", cache_layer.data_ptr(), dtype_code(cache_layer.dtype), cache_layer.stride(0),
         cache_layer.shape[1], cache_layer.shape[2], block_table.data_ptr(), block_table.shape[1], seq_start.data_ptr(),
         context_lens.data_ptr(), int(num_seqs), out.data_ptr(), where.data_ptr(), where.shape[1], out.shape[0],
         int(window or 0), stream_handle())


def latent_decode_takes(record: int, value_dim: int) -> bool:
    """Whether :func:`latent_decode` takes a record of ``record`` numbers whose first ``value_dim`` are the value."""
    return bool(core().ap_latent_decode_takes(int(record), int(value_dim)))


def latent_decode(q: torch.Tensor, out: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor,
                  seq_start: torch.Tensor, positions: torch.Tensor, num_seqs: int, num_heads: int, record: int,
                  value_dim: int, scale: float, gate: Optional[torch.Tensor], max_context: int, workspace,
                  window: int = 0, sink: Optional[torch.Tensor] = None) -> None:
    """bfloat16 attention of the sequences that bring ONE row over pages ``[pages, P, record]`` whose
    records are every head's key and, in their first ``value_dim`` numbers, every head's value:
    ``q [T, heads*record]`` -> ``out [T, heads*value_dim]`` times ``sigmoid(gate[t, h])`` (rows of other
    sequences are left alone).  All heads of a sequence share the key tiles on the tensor cores; the
    keys are cut into slices by ``max_context`` (the longest context the step may hold), whose partial
    results wait in a buffer taken from ``workspace``.  ``window`` (0: none): a row sees its last ``window``
    keys; ``sink`` (32-bit ``[heads]``): the denominator also holds ``exp(sink[h])``."""
    _check(q, "q", torch.bfloat16, 2)
    _check(out, "out", torch.bfloat16, 2)
    T = q.shape[0]
    if q.shape[1] != num_heads * record or tuple(out.shape) != (T, num_heads * value_dim):
        raise KernelError("latent_decode: q/out do not match the heads")
    if cache_layer.dtype != torch.bfloat16:
        raise KernelError("latent_decode: the pages must be bfloat16")
    P, page_stride = _kv_pages(cache_layer, 1, record, "latent_decode")
    _check(block_table, "block_table", torch.int32, 2)
    _check(seq_start, "seq_start", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    gptr, gld = 0, 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.dim() != 2 or gate.shape[0] < T or gate.shape[1] != num_heads \
                or gate.stride(1) != 1 or not gate.is_cuda:
            raise KernelError("latent_decode: the gate must be 32-bit [T, heads] with contiguous rows")
        gptr, gld = gate.data_ptr(), gate.stride(0)
    if sink is not None:
        _check(sink, "sink", torch.float32, 1)
        if sink.shape[0] != num_heads:
            raise KernelError("latent_decode: the sink must have one entry per head")
    window = int(window or 0)
    if window > 0:
        max_context = min(int(max_context), window + 64)       # no row reads more keys than its window
    lib = core()
    nsplit = int(lib.ap_latent_decode_splits(int(num_seqs), int(num_heads), int(max_context)))
    need = num_seqs * nsplit * num_heads * (value_dim + 2)
    scratch = workspace.get("latent_decode.partial", (need,), torch.float32)
    call(lib, "ap_latent_decode", q.data_ptr(), out.data_ptr(), cache_layer.data_ptr(), block_table.data_ptr(),
         block_table.shape[1], seq_start.data_ptr(), positions.data_ptr(), int(num_seqs), int(num_heads), int(record),
         int(value_dim), P, page_stride, float(scale), gptr, gld, nsplit, scratch.data_ptr(), need, window,
         sink.data_ptr() if sink is not None else 0, stream_handle())


def latent_prefill_takes(key_dim: int, value_dim: int) -> bool:
    """Whether :func:`latent_prefill` takes these head sizes."""
    return bool(core().ap_latent_prefill_takes(int(key_dim), int(value_dim)))


def latent_prefill(q: torch.Tensor, out: torch.Tensor, kv: torch.Tensor, where: torch.Tensor, seq_start: torch.Tensor,
                   positions: torch.Tensor, num_seqs: int, num_heads: int, key_dim: int, value_dim: int, scale: float,
                   gate: Optional[torch.Tensor] = None, window: int = 0, sink: Optional[torch.Tensor] = None) -> None:
    """bfloat16 causal attention of the sequences that bring SEVERAL rows on per-head keys and values
    ``kv [tokens, heads*(key_dim + value_dim)]`` in which a sequence's tokens follow one another from row
    ``where[s, 0]`` on (what :func:`latent_gather` and the product after it leave):
    ``q [T, heads*key_dim]`` -> ``out [T, heads*value_dim]`` times ``sigmoid(gate[t, h])``; rows of sequences
    that bring one row are left alone.  ``window`` (0: none): a row sees its last ``window`` keys, and ``kv``
    holds a sequence's tokens from the first one its first row sees (as :func:`latent_gather` leaves them with
    the same window); ``sink`` (32-bit ``[heads]``): the denominator also holds ``exp(sink[h])``."""
    if sink is not None:
        _check(sink, "sink", torch.float32, 1)
        if sink.shape[0] != num_heads:
            raise KernelError("latent_prefill: the sink must have one entry per head")
    _check(q, "q", torch.bfloat16, 2)
    _check(out, "out", torch.bfloat16, 2)
    _check(kv, "kv", torch.bfloat16, 2)
    _check(where, "where", torch.int32, 2)
    _check(seq_start, "seq_start", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    T = q.shape[0]
    if q.shape[1] != num_heads * key_dim or tuple(out.shape) != (T, num_heads * value_dim) \
            or kv.shape[1] != num_heads * (key_dim + value_dim) or where.shape[0] < num_seqs:
        raise KernelError("latent_prefill: shapes disagree")
    gptr, gld = 0, 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.dim() != 2 or gate.shape[0] < T or gate.shape[1] != num_heads \
                or gate.stride(1) != 1 or not gate.is_cuda:
            raise KernelError("latent_prefill: the gate must be 32-bit [T, heads] with contiguous rows")
        gptr, gld = gate.data_ptr(), gate.stride(0)
    call(core(), "ap_latent_prefill", q.data_ptr(), out.data_ptr(), kv.data_ptr(), where.data_ptr(), where.shape[1],
         seq_start.data_ptr(), positions.data_ptr(), int(num_seqs), T, int(num_heads), int(key_dim), int(value_dim),
         float(scale), gptr, gld, int(window or 0), sink.data_ptr() if sink is not None else 0, stream_handle())
