"""Python faces of the kernels that act on the residual stream element by element: a norm without
statistics (Dynamic Tanh), its mix with the previous token's row, the depth-weighted average over
the layers' outputs, and bias with activation behind a product; see ``ops/__init__.py``."""
from __future__ import annotations

from typing import Optional

import torch

from . import AP_F32, KernelError, _check, _partials, call, core, dtype_code, stream_handle

BIAS_ACTIVATIONS = {None: 0, "none": 0, "relu": 1, "relu2": 2, "gelu_tanh": 3, "silu": 4}


def _delta(delta: Optional[torch.Tensor], T: int, H: int, who: str):
    if delta is None:
        return 0, 0, 0
    dptr, code, S, dstride, dT, dN = _partials(delta, "delta")
    if code != AP_F32 or dT != T or dN != H:
        raise KernelError(f"{who}: delta {tuple(delta.shape)} {delta.dtype} does not match x [{T}, {H}]")
    return dptr, S, dstride


def add_dyt(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, alpha: float, out: torch.Tensor,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """``v = x + sum(delta); out = tanh(alpha * v) * weight + bias`` (``weight``, ``bias`` 32-bit ``[H]``).

    Without ``rows`` every row is normed and ``x`` is overwritten with ``v``.  With ``rows`` (int32
    indices) only those rows are normed into ``out[r]`` and ``x`` stays."""
    _check(x, "x", torch.float32, 2)
    _check(weight, "weight", torch.float32, 1)
    _check(bias, "bias", torch.float32, 1)
    _check(out, "out", dims=2)
    T, H = x.shape
    if weight.shape[0] != H or bias.shape[0] != H or out.shape[1] != H:
        raise KernelError("add_dyt: widths disagree")
    dptr, S, dstride = _delta(delta, T, H, "add_dyt")
    R = T
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        R = rows.shape[0]
    if out.shape[0] < R:
        raise KernelError("add_dyt: out has too few rows")
    call(core(), "ap_add_dyt", x.data_ptr(), dptr, S, dstride, weight.data_ptr(), bias.data_ptr(), float(alpha),
         out.data_ptr(), dtype_code(out.dtype), rows.data_ptr() if rows is not None else 0, R, H, stream_handle())


def dyt_shift(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, alpha: float, shift: torch.Tensor,
              state: torch.Tensor, seq_start: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
              state_slots: torch.Tensor, out: torch.Tensor) -> None:
    """``n_t = tanh(alpha * x_t) * weight + bias``; ``out_t = n_t + (n_{t-1} - n_t) * shift`` with the previous
    row of the same sequence (zeros before position 0).  ``state [slots, H]`` (32-bit, rows may be strided)
    holds, per request, the normed row of its last token so far: it supplies ``n_{t-1}`` for a portion's
    first row and receives the portion's last."""
    _check(x, "x", torch.float32, 2)
    T, H = x.shape
    for t, n in ((weight, "weight"), (bias, "bias"), (shift, "shift")):
        _check(t, n, torch.float32, 1)
        if t.shape[0] != H:
            raise KernelError(f"dyt_shift: {n} must have one entry per column")
    _check(out, "out", dims=2)
    if tuple(out.shape) != (T, H):
        raise KernelError("dyt_shift: out must have x's shape")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != H or state.stride(1) != 1 or not state.is_cuda:
        raise KernelError("dyt_shift: the state must be 32-bit [slots, H] with contiguous rows")
    for t, n in ((seq_start, "seq_start"), (positions, "positions"), (token_seq, "token_seq"),
                 (state_slots, "state_slots")):
        _check(t, n, torch.int32, 1)
    call(core(), "ap_dyt_shift", x.data_ptr(), weight.data_ptr(), bias.data_ptr(), float(alpha), shift.data_ptr(),
         state.data_ptr(), state.stride(0), seq_start.data_ptr(), positions.data_ptr(), token_seq.data_ptr(),
         state_slots.data_ptr(), out.data_ptr(), dtype_code(out.dtype), T, H, stream_handle())


def stream_mix(x: torch.Tensor, delta: Optional[torch.Tensor], streams: torch.Tensor, k: int,
               weights: Optional[torch.Tensor]) -> None:
    """``v = x + sum(delta)``; ``streams[k] = v``; ``x = sum_{j <= k} weights[j] * streams[j]`` (32-bit, the sum
    over ``j`` upwards).  ``streams [count, T, H]``; with ``weights`` None the stream is only stored (and ``x``
    becomes ``v``)."""
    _check(x, "x", torch.float32, 2)
    _check(streams, "streams", torch.float32, 3)
    T, H = x.shape
    if tuple(streams.shape[1:]) != (T, H) or not (0 <= k < streams.shape[0]):
        raise KernelError(f"stream_mix: streams {tuple(streams.shape)} do not hold stream {k} of x {tuple(x.shape)}")
    dptr, S, dstride = _delta(delta, T, H, "stream_mix")
    if weights is not None:
        _check(weights, "weights", torch.float32, 1)
        if weights.shape[0] < k + 1:
            raise KernelError("stream_mix: one weight per stream is needed")
    call(core(), "ap_stream_mix", x.data_ptr(), dptr, S, dstride, streams.data_ptr(), streams.stride(0), int(k),
         weights.data_ptr() if weights is not None else 0, x.numel(), stream_handle())


def bias_act(inp: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, activation: Optional[str]) -> None:
    """``out = act(inp + bias)`` for ``inp [T, N]`` (32-bit sums of a product, or 16-bit) and 32-bit ``bias [N]``
    (None: none); ``activation``: ``"relu"``, ``"relu2"`` (the square of relu), ``"gelu_tanh"``, ``"silu"`` or None."""
    _check(inp, "inp", dims=2)
    _check(out, "out", dims=2)
    if activation not in BIAS_ACTIVATIONS:
        raise KernelError(f"bias_act: activation {activation!r} is not known")
    T, N = inp.shape
    if tuple(out.shape) != (T, N):
        raise KernelError("bias_act: out must have inp's shape")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.shape[0] != N:
            raise KernelError("bias_act: one bias per column is needed")
    call(core(), "ap_bias_act", inp.data_ptr(), dtype_code(inp.dtype), bias.data_ptr() if bias is not None else 0,
         out.data_ptr(), dtype_code(out.dtype), T, N, BIAS_ACTIVATIONS[activation], stream_handle())
