"""Python faces of the kernels of linear attention in its recurrent form and of the norm that follows a gated sum;
see ``ops/__init__.py``."""
from __future__ import annotations

from typing import Optional

import torch

from . import AP_F32, KernelError, _check, _partials, call, core, dtype_code, stream_handle

DECAY_MODES = {"head": 0, "head_token": 1, "channel": 2}
QK_MODES = {None: 0, "plain": 0, "rotate": 1, "unit": 2}


def _rows32(t: torch.Tensor, name: str, T: int, width: int):
    """(pointer, row stride) of a 32-bit matrix view ``[T, width]`` with contiguous rows (it may be a run of
    columns of a wider matrix)."""
    if t.dtype != torch.float32 or t.dim() != 2 or not t.is_cuda or t.stride(1) != 1 or t.shape[0] < T \
            or t.shape[1] != width:
        raise KernelError(f"linear_scan: {name} must be 32-bit [T, {width}] with contiguous rows, is "
                          f"{tuple(t.shape)} {t.dtype}")
    return t.data_ptr(), t.stride(0)


def linear_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, y: torch.Tensor, state: torch.Tensor,
                seq_start: torch.Tensor, positions: torch.Tensor, state_slots: torch.Tensor, num_seqs: int,
                heads: int, qk_heads: int, key_dim: int, value_dim: int, decay: str,
                decay_channel: Optional[torch.Tensor] = None, tau: float = 1.0,
                decay_head: Optional[torch.Tensor] = None, decay_const: Optional[torch.Tensor] = None,
                dt_bias: Optional[torch.Tensor] = None, beta: Optional[torch.Tensor] = None,
                qk: Optional[str] = None, cos_sin: Optional[torch.Tensor] = None, unit_eps: float = 0.0,
                out_scale: float = 1.0) -> None:
    """Linear attention as a recurrence over each sequence's rows, all 32-bit:
    ``S = diag(a_t) S + k_t u_t^T``, ``y_t = S^T q_t * out_scale`` with a state ``[key_dim, value_dim]`` per head.

    ``q``, ``k`` ``[T, qk_heads * key_dim]``, ``v`` ``[T, heads * value_dim]`` (views of columns of a wider
    32-bit matrix are taken); value head ``h`` reads query/key head ``h // (heads / qk_heads)``.
    ``decay``: ``"head"``: ``a = decay_const[h]``; ``"head_token"``: ``a = exp(-exp(decay_const[h]) *
    softplus(decay_head[t, h] + dt_bias[h]))``; ``"channel"``: ``a[d] = sigmoid(decay_channel[t, h, d])^(1/tau)``.
    ``beta [T, heads]`` (raw): the delta rule, ``u = sigmoid(beta) (v - S^T k)`` on the decayed state; else
    ``u = v``.  ``qk``: ``"rotate"`` turns the first ``2 * cos_sin.shape[1]`` coordinates of every query and key
    head by ``cos_sin [T, r/2, 2]``; ``"unit"`` divides each by ``sqrt(sum x^2 + unit_eps)``.
    ``state [slots, heads, key_dim, value_dim]`` may be a strided view of the slots' rows; a sequence whose first
    row has position 0 starts from zero.  ``q``, ``k``, ``decay_channel``, ``decay_head`` and ``beta`` are scratch:
    a pass before the recurrence turns them into what it reads (rotated or unit vectors, decays, gates) in place."""
    T = y.shape[0]
    if decay not in DECAY_MODES or qk not in QK_MODES:
        raise KernelError(f"linear_scan: decay {decay!r} or qk {qk!r} is not known")
    qp, ldq = _rows32(q, "q", T, qk_heads * key_dim)
    kp, ldk = _rows32(k, "k", T, qk_heads * key_dim)
    vp, ldv = _rows32(v, "v", T, heads * value_dim)
    yp, ldy = _rows32(y, "y", T, heads * value_dim)
    dcp = dcl = dhp = dhl = bp = bl = 0
    if decay == "channel":
        dcp, dcl = _rows32(decay_channel, "decay_channel", T, heads * key_dim)
    if decay == "head_token":
        dhp, dhl = _rows32(decay_head, "decay_head", T, heads)
    if decay in ("head", "head_token"):
        _check(decay_const, "decay_const", torch.float32, 1)
        if decay_const.shape[0] != heads:
            raise KernelError("linear_scan: one decay constant per head is needed")
    if dt_bias is not None:
        _check(dt_bias, "dt_bias", torch.float32, 1)
    if beta is not None:
        bp, bl = _rows32(beta, "beta", T, heads)
    rot = 0
    if QK_MODES[qk] == 1:
        _check(cos_sin, "cos_sin", torch.float32, 3)
        rot = 2 * cos_sin.shape[1]
        if cos_sin.shape[0] < T or cos_sin.shape[2] != 2 or rot > key_dim:
            raise KernelError(f"linear_scan: cos_sin {tuple(cos_sin.shape)} is not [T, r/2, 2] with r <= {key_dim}")
    if state.dtype != torch.float32 or state.dim() != 4 or tuple(state.shape[1:]) != (heads, key_dim, value_dim) \
            or state.stride(3) != 1 or state.stride(2) != value_dim or state.stride(1) != key_dim * value_dim:
        raise KernelError(f"linear_scan: the state must be 32-bit [slots, {heads}, {key_dim}, {value_dim}] with "
                          f"contiguous heads")
    for t, n in ((seq_start, "seq_start"), (positions, "positions"), (state_slots, "state_slots")):
        _check(t, n, torch.int32, 1)
    call(core(), "ap_linear_scan", qp, ldq, kp, ldk, vp, ldv, dcp, dcl, dhp, dhl,
         decay_const.data_ptr() if decay_const is not None else 0, dt_bias.data_ptr() if dt_bias is not None else 0,
         bp, bl, cos_sin.data_ptr() if rot else 0, rot, state.data_ptr(), state.stride(0), seq_start.data_ptr(),
         positions.data_ptr(), state_slots.data_ptr(), yp, ldy, T, int(num_seqs), int(heads), int(qk_heads),
         int(key_dim), int(value_dim), DECAY_MODES[decay], QK_MODES[qk], float(tau), float(unit_eps),
         float(out_scale), stream_handle())


def head_norm_gate(y: torch.Tensor, gate: torch.Tensor, weight: Optional[torch.Tensor], eps: float,
                   out: torch.Tensor, heads: int, value_dim: int, out_scale: float = 1.0) -> None:
    """``out[t, h] = y[t, h] / sqrt(mean(y[t, h]^2) + eps) * weight * silu(gate[t, h]) * out_scale`` per head of
    ``value_dim`` numbers; ``y`` and ``gate`` 32-bit ``[T, heads * value_dim]`` (may be runs of columns of a
    wider matrix), ``weight`` 32-bit ``[value_dim]`` shared by the heads or None."""
    T = out.shape[0]
    _check(out, "out", dims=2)
    yp, ldy = _rows32(y, "y", T, heads * value_dim)
    gp, ldg = _rows32(gate, "gate", T, heads * value_dim)
    if out.shape[1] != heads * value_dim:
        raise KernelError("head_norm_gate: out must be [T, heads * value_dim]")
    if weight is not None:
        _check(weight, "weight", torch.float32, 1)
        if weight.shape[0] != value_dim:
            raise KernelError("head_norm_gate: the weight must have one entry per coordinate of a head")
    call(core(), "ap_head_norm_gate", yp, ldy, gp, ldg, weight.data_ptr() if weight is not None else 0, float(eps),
         float(out_scale), out.data_ptr(), dtype_code(out.dtype), T, int(heads), int(value_dim), stream_handle())


def gated_postnorm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, alpha: float = 1.0,
                   delta: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                   gate_bias: Optional[torch.Tensor] = None, copy: Optional[torch.Tensor] = None,
                   rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> None:
    """The norm after a sum: ``v = alpha * x + sigmoid(gate + gate_bias) * sum(delta)``, then every one of the
    ``groups`` equal runs of ``v`` over its own ``sqrt(mean(run^2) + eps)``, times ``weight``; all 32-bit.

    Without ``rows``: ``x`` (32-bit ``[T, H]``) is overwritten with the result, and ``copy`` (optional, any type)
    receives it too.  With ``rows`` (int32 indices) or ``out`` alone: the chosen (or all) rows are normed into
    ``out`` and ``x`` stays.  ``delta``: 32-bit partial sums ``[S, T, H]`` or ``[T, H]``; ``gate``: 32-bit ``[T, H]``
    raw (may be a run of columns of a wider matrix), ``gate_bias [H]``."""
    _check(x, "x", torch.float32, 2)
    _check(weight, "weight", dims=1)
    T, H = x.shape
    if weight.shape[0] != H:
        raise KernelError("gated_postnorm: the weight must have one entry per column")
    S, dptr, dstride = 0, 0, 0
    if delta is not None:
        dptr, code, S, dstride, dT, dN = _partials(delta, "delta")
        if code != AP_F32 or dT != T or dN != H:
            raise KernelError(f"gated_postnorm: delta {tuple(delta.shape)} {delta.dtype} does not match x {tuple(x.shape)}")
    gptr = gld = 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape[0] < T \
                or gate.shape[1] != H or not gate.is_cuda:
            raise KernelError("gated_postnorm: the gate must be 32-bit [T, H] with contiguous rows")
        gptr, gld = gate.data_ptr(), gate.stride(0)
    if gate_bias is not None:
        _check(gate_bias, "gate_bias", torch.float32, 1)
    update = rows is None and out is None
    target = copy if update else out
    R = T
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        R = rows.shape[0]
    if target is not None:
        _check(target, "out", dims=2)
        if target.shape[0] < R or target.shape[1] != H:
            raise KernelError("gated_postnorm: the output has too few rows or another width")
    elif not update:
        raise KernelError("gated_postnorm: chosen rows need an output")
    call(core(), "ap_gated_postnorm", x.data_ptr(), rows.data_ptr() if rows is not None else 0, R, dptr, S, dstride,
         gptr, gld, gate_bias.data_ptr() if gate_bias is not None else 0, float(alpha), weight.data_ptr(),
         dtype_code(weight.dtype), int(groups), float(eps), 1 if update else 0,
         target.data_ptr() if target is not None else 0, dtype_code(target.dtype) if target is not None else AP_F32,
         H, stream_handle())


def gated_row_add(delta: torch.Tensor, other: torch.Tensor, h: torch.Tensor, g: torch.Tensor) -> None:
    """``delta[t] += sigmoid(h[t] . g) * other[t]``: 32-bit ``delta``, ``other`` ``[T, H]``; ``h [T, H]`` the rows
    the gate is read off, ``g [H]``."""
    _check(delta, "delta", torch.float32, 2)
    _check(other, "other", torch.float32, 2)
    _check(h, "h", dims=2)
    T, H = delta.shape
    g = g.reshape(-1)
    _check(g, "g", dims=1)
    if tuple(other.shape) != (T, H) or tuple(h.shape) != (T, H) or g.shape[0] != H:
        raise KernelError("gated_row_add: shapes disagree")
    call(core(), "ap_gated_row_add", delta.data_ptr(), other.data_ptr(), h.data_ptr(), dtype_code(h.dtype),
         g.data_ptr(), dtype_code(g.dtype), T, H, stream_handle())
