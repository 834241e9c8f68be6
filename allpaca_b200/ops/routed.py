"""Python faces of the kernels of feed-forwards beyond the SiLU-gated one: gated activations by
name and a routed feed-forward (mixture of experts); see ``ops/__init__.py``."""
from __future__ import annotations

from typing import Optional

import torch

from . import KernelError, _check, call, core, dtype_code, stream_handle

ACTIVATIONS = {"silu": 0, "relu": 1, "clamped_sigmoid": 2, "gelu_tanh": 3}


def activation_code(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"gated activation {name!r} is not known ({', '.join(sorted(ACTIVATIONS))})") from None


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu", pairs: bool = False,
              limit: float = 0.0, alpha: float = 1.0, shift: float = 0.0,
              row_scale: Optional[torch.Tensor] = None, scale_index: Optional[torch.Tensor] = None) -> None:
    """``out[t, j] = act(gate, up)`` for ``gate_up [T, 2I]`` holding ``[gate | up]`` (or, with
    ``pairs``, gate and up columns alternating).  ``silu``: ``silu(g) u``; ``relu``: ``max(g, 0) u``;
    ``clamped_sigmoid``: ``g' sigmoid(alpha g') (u' + shift)`` with ``g' = min(g, limit)`` and
    ``u' = clamp(u, -limit, limit)``; ``gelu_tanh``: ``0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) u``.
    ``row_scale`` (32-bit): gate and up of row ``t`` are first multiplied by ``row_scale[scale_index[t]]``
    (``scale_index`` int32 or None: ``row_scale[t]``), which is what a scale of the row's input does to both."""
    _check(gate_up, "gate_up", dims=2)
    _check(out, "out", dims=2)
    T, inter = out.shape
    if tuple(gate_up.shape) != (T, 2 * inter):
        raise KernelError("gated_act: out must be [T, I] for gate_up [T, 2I]")
    call(core(), "ap_gated_act", gate_up.data_ptr(), dtype_code(gate_up.dtype), out.data_ptr(), dtype_code(out.dtype),
         T, inter, 1 if pairs else 0, activation_code(activation), float(limit), float(alpha), float(shift),
         row_scale.data_ptr() if row_scale is not None else 0,
         scale_index.data_ptr() if scale_index is not None else 0, stream_handle())


def moe_route(logits: torch.Tensor, bias: Optional[torch.Tensor], chosen: torch.Tensor, weight: torch.Tensor) -> None:
    """Per row of 32-bit ``logits [T, E]`` (plus ``bias [E]``): the ``top`` experts with the largest
    values into ``chosen [T, top]`` (int32, ties to the lower index) and the softmax over those
    values into ``weight [T, top]``."""
    _check(logits, "logits", torch.float32, 2)
    _check(chosen, "chosen", torch.int32, 2)
    _check(weight, "weight", torch.float32, 2)
    T, E = logits.shape
    top = chosen.shape[1]
    if tuple(chosen.shape) != (T, top) or tuple(weight.shape) != (T, top):
        raise KernelError("moe_route: chosen and weight must be [T, top]")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.shape[0] != E:
            raise KernelError("moe_route: one bias per expert is needed")
    call(core(), "ap_moe_route", logits.data_ptr(), bias.data_ptr() if bias is not None else 0, chosen.data_ptr(),
         weight.data_ptr(), T, E, top, stream_handle())


ROUTE_MODES = {"top_softmax": 0, "softmax_all": 1, "sigmoid": 2}


def moe_route_rows(rows: torch.Tensor, router: torch.Tensor, bias: Optional[torch.Tensor], chosen: torch.Tensor,
                   weight: torch.Tensor, mode: str = "top_softmax") -> None:
    """:func:`moe_route` with the router's product inside: the logits of row ``t`` are
    ``z = router [E, K] @ rows[t]`` in 32-bit sums.  ``mode`` ``"top_softmax"``: the ``top`` largest
    ``z + bias``, shares their softmax; ``"softmax_all"``: scores ``s = softmax(z)`` over all experts, the
    ``top`` largest ``s + bias`` chosen, shares ``s_e / (sum of the chosen s + 1e-20)``; ``"sigmoid"``: scores
    ``s = sigmoid(z)``, every output alone, the ``top`` largest ``s + bias`` chosen, shares the chosen ``s`` as they are."""
    if mode not in ROUTE_MODES:
        raise KernelError(f"moe_route_rows: mode {mode!r} is not known ({', '.join(ROUTE_MODES)})")
    _check(rows, "rows", dims=2)
    _check(router, "router", dims=2)
    _check(chosen, "chosen", torch.int32, 2)
    _check(weight, "weight", torch.float32, 2)
    T, K = rows.shape
    E, top = router.shape[0], chosen.shape[1]
    if router.shape[1] != K or tuple(chosen.shape) != (T, top) or tuple(weight.shape) != (T, top):
        raise KernelError("moe_route_rows: shapes disagree")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.shape[0] != E:
            raise KernelError("moe_route_rows: one bias per expert is needed")
    call(core(), "ap_moe_route_rows", rows.data_ptr(), dtype_code(rows.dtype), router.data_ptr(),
         dtype_code(router.dtype), K, bias.data_ptr() if bias is not None else 0, chosen.data_ptr(), weight.data_ptr(),
         T, E, top, ROUTE_MODES[mode], stream_handle())


def moe_max_tiles(pairs: int, experts: int) -> int:
    """Row tiles the grouped products are planned for, whatever the routing."""
    return int(core().ap_moe_max_tiles(int(pairs), int(experts)))


def moe_sort(chosen: torch.Tensor, perm: torch.Tensor, place: torch.Tensor, tiles: torch.Tensor, experts: int,
             offsets: Optional[torch.Tensor] = None, real: Optional[int] = None) -> None:
    """Group the (row, choice) pairs of ``chosen [T, top]`` by expert: ``perm [pairs]`` lists the
    pairs in grouped order, ``place [pairs]`` is each pair's position in it, ``tiles
    [max_tiles + 1, 3]`` the row tiles (expert, first position, rows) with their number last,
    ``offsets [experts + 1]`` (optional) the first position of every expert's pairs.  Only the first
    ``real`` experts (default: all) get row tiles: the others have no weights (identity experts)."""
    _check(chosen, "chosen", torch.int32, 2)
    pairs = chosen.numel()
    for t, n in ((perm, "perm"), (place, "place")):
        _check(t, n, torch.int32, 1)
        if t.shape[0] < pairs:
            raise KernelError(f"moe_sort: {n} is shorter than the pairs")
    _check(tiles, "tiles", torch.int32, 2)
    if tuple(tiles.shape) != (moe_max_tiles(pairs, experts) + 1, 3):
        raise KernelError("moe_sort: tiles must be [max_tiles + 1, 3]")
    if offsets is not None:
        _check(offsets, "offsets", torch.int32, 1)
        if offsets.shape[0] != experts + 1:
            raise KernelError("moe_sort: offsets must have one entry per expert and one more")
    call(core(), "ap_moe_sort", chosen.data_ptr(), perm.data_ptr(), place.data_ptr(), tiles.data_ptr(),
         offsets.data_ptr() if offsets is not None else 0, pairs, int(experts),
         int(experts if real is None else real), stream_handle())


def moe_gather(a: torch.Tensor, out: torch.Tensor, perm: torch.Tensor, top: int) -> None:
    """``out[p] = a[perm[p] // top]``: the rows of 16-bit ``a [T, K]`` in grouped order, ``[pairs, K]``."""
    _check(a, "a", torch.bfloat16, 2)
    _check(out, "out", torch.bfloat16, 2)
    _check(perm, "perm", torch.int32, 1)
    if out.shape[1] != a.shape[1] or out.shape[0] != a.shape[0] * top or perm.shape[0] < out.shape[0]:
        raise KernelError("moe_gather: shapes disagree")
    call(core(), "ap_moe_gather", a.data_ptr(), out.data_ptr(), perm.data_ptr(), int(top), out.shape[0], a.shape[1],
         stream_handle())


def moe_gate_up(a: torch.Tensor, w: torch.Tensor, y: torch.Tensor, perm: torch.Tensor, top: int, tiles: torch.Tensor,
                activation: str, limit: float = 0.0, alpha: float = 1.0, shift: float = 0.0,
                experts: Optional[int] = None, pair_scale: Optional[torch.Tensor] = None) -> None:
    """For every row tile: ``y[p] = act(a[perm[p] // top] W_gate[e]^T, ... W_up[e]^T)`` with
    ``w [E, 2F, K]`` (gate rows, then up rows of each expert) and ``y [pairs, F]``.  ``experts``: the
    number the pairs were sorted by, where that is more than the experts that have weights.  ``pair_scale`` (32-bit
    ``[pairs]`` by pair ``t * top + k``): the pair's input row counts that many times, so both sums are multiplied
    by it before the activation."""
    _check(a, "a", dims=2)
    _check(w, "w", dims=3)
    _check(y, "y", dims=2)
    pairs, F = y.shape
    E, F2, K = w.shape
    if F2 != 2 * F or a.shape[1] != K or pairs != a.shape[0] * top:
        raise KernelError(f"moe_gate_up: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    call(core(), "ap_moe_gate_up", a.data_ptr(), dtype_code(a.dtype), w.data_ptr(), dtype_code(w.dtype), y.data_ptr(),
         dtype_code(y.dtype), perm.data_ptr(), int(top), tiles.data_ptr(), pairs, int(experts or E), F, K,
         activation_code(activation),
         float(limit), float(alpha), float(shift), pair_scale.data_ptr() if pair_scale is not None else 0,
         stream_handle())


def moe_down(y: torch.Tensor, w: torch.Tensor, o: torch.Tensor, tiles: torch.Tensor, experts: Optional[int] = None) -> None:
    """For every row tile: ``o[p] = y[p] W_down[e]^T`` with ``w [E, H, F]``; ``o [pairs, H]`` 32-bit.
    ``experts``: as for :func:`moe_gate_up`."""
    _check(y, "y", dims=2)
    _check(w, "w", dims=3)
    _check(o, "o", torch.float32, 2)
    pairs, F = y.shape
    E, H, F2 = w.shape
    if F2 != F or tuple(o.shape) != (pairs, H):
        raise KernelError(f"moe_down: shapes disagree: y {tuple(y.shape)}, w {tuple(w.shape)}, o {tuple(o.shape)}")
    call(core(), "ap_moe_down", y.data_ptr(), dtype_code(y.dtype), w.data_ptr(), dtype_code(w.dtype), o.data_ptr(),
         tiles.data_ptr(), pairs, int(experts or E), H, F, stream_handle())


def moe_combine(o: torch.Tensor, place: torch.Tensor, weight: torch.Tensor, delta: torch.Tensor,
                chosen: Optional[torch.Tensor] = None, real: int = 0, rows: Optional[torch.Tensor] = None,
                unweighted: bool = False) -> None:
    """``delta[t] = sum_k weight[t, k] * o[place[t * top + k]]`` (32-bit, in the order of k).  With
    ``chosen [T, top]``: a choice of an expert from ``real`` on contributes ``rows[t]``, the row's input
    itself, instead (an identity expert).  ``unweighted``: every weight counts as 1 (``weight`` gives the shape only)."""
    _check(o, "o", torch.float32, 2)
    _check(weight, "weight", torch.float32, 2)
    _check(delta, "delta", torch.float32, 2)
    T, top = weight.shape
    H = o.shape[1]
    if tuple(delta.shape) != (T, H) or o.shape[0] != T * top:
        raise KernelError("moe_combine: shapes disagree")
    cptr = rptr = 0
    rcode = 0
    if chosen is not None:
        _check(chosen, "chosen", torch.int32, 2)
        _check(rows, "rows", dims=2)
        if tuple(chosen.shape) != (T, top) or tuple(rows.shape) != (T, H):
            raise KernelError("moe_combine: chosen must be [T, top] and rows [T, H]")
        cptr, rptr, rcode = chosen.data_ptr(), rows.data_ptr(), dtype_code(rows.dtype)
    call(core(), "ap_moe_combine", o.data_ptr(), place.data_ptr(), 0 if unweighted else weight.data_ptr(),
         delta.data_ptr(), T, H, top,
         cptr, int(real), rptr, rcode, stream_handle())
