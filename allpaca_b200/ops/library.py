"""Loads the CUDA kernel libraries and exposes their C entry points.

The libraries are plain shared objects with `extern "C"` functions that take
device pointers, sizes and a stream; they are called through ctypes with the
pointers of torch tensors.  There is no CPU implementation behind these calls:
if nvcc or a CUDA device is missing the load fails with a clear error.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_void_p, c_int, c_float, c_longlong, c_char_p
from typing import Dict

from ..csrc import build as _build


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or could not be launched."""


_P, _I, _F, _L = c_void_p, c_int, c_float, c_longlong

_CORE_SIGNATURES = {
    "ap_embed_gather": [_P, _P, _I, _P, _I, _I, _I, _F, _P],
    "ap_bias_add": [_P, _I, _P, _I, _I, _I, _P],
    "ap_logit_transform": [_P, _P, _I, _I, _I, _F, _F, _P],
    "ap_add_rmsnorm": [_P, _P, _I, _L, _P, _I, _F, _P, _I, _P, _I, _I, _P],
    "ap_residual_add": [_P, _P, _I, _L, _L, _P],
    "ap_rope_kv_store": [_P, _I, _I, _L, _P, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _L, _P],
    "ap_clear_page_tails": [_P, _I, _L, _L, _I, _I, _I, _I, _P, _P, _P, _I, _P, _I, _P],
    "ap_rope_table": [_P, _P, _P, _I, _I, _F, _P],
    # int ap_norm_residual(x, delta, S, delta_stride, weight, w_dtype, eps, mult, copy, copy_dtype, T, H, stream)
    "ap_norm_residual": [_P, _P, _I, _L, _P, _I, _F, _F, _P, _I, _I, _I, _P],
    "ap_swiglu": [_P, _I, _I, _L, _P, _I, _I, _I, _I, _P],
    "ap_gemm_simt": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _L, _L, _L, _P],
    "ap_argmax": [_P, _L, _I, _I, _P, _P],
    "ap_sample": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P],
    "ap_sample_rows": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P],
    "ap_sample_cluster": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P],
    # int ap_embed_sinusoid_norm(tokens, positions, table, table_dtype, inv_freq, norm_w, norm_dtype, eps, scale,
    #                            x, T, H, V, stream)
    "ap_embed_sinusoid_norm": [_P, _P, _P, _I, _P, _P, _I, _F, _F, _P, _I, _I, _I, _P],
    # int ap_qk_norm_store(in, in_dtype, ld_in, q_out, cache, act_dtype, positions, token_seq, block_table,
    #                      max_blocks, T, nh, nkv, D, VD, P, page_stride, eps, normalise, temp_coef, temp_every,
    #                      q_weight, k_weight, bias, cos_sin, rot_dims, value_scale, stream)
    "ap_qk_norm_store": [_P, _I, _L, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _L, _F, _I, _F, _I, _P, _P, _P,
                         _P, _I, _F, _P],
    # int ap_attention_window_bias(q, out, cache, dtype, block_table, max_blocks, seq_start, positions, nseq, T,
    #                              nh, nkv, D, VD, P, page_stride, scale, softcap, window, r1, r2, single_rows,
    #                              other_rows, record, value_offset, bias_kind, keep_first, gate, gate_ld, sink,
    #                              max_context, stream)
    "ap_attention_window_bias": [_P, _P, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _L, _F, _F, _I, _P, _P, _I, _I,
                                 _I, _I, _I, _I, _P, _L, _P, _I, _P],
    # int ap_latent_prepare(in, ld, q0, Q, q_weight, cq, kv0, R, rot, rot_dims, kv_weight, cache, act_dtype, positions,
    #                       token_seq, block_table, max_blocks, P, page_stride, cos_sin, eps, T, stream)
    "ap_latent_prepare": [_P, _L, _I, _I, _P, _P, _I, _I, _I, _I, _P, _P, _I, _P, _P, _P, _I, _I, _L, _P, _F, _I, _P],
    # int ap_head_project(in, in_dtype, in_ld, in_hs, w, w_dtype, out, out_dtype, out_ld, out_hs, T, H, K, N, tail,
    #                     tail_dims, cos_sin, stream)
    "ap_head_project": [_P, _I, _L, _I, _P, _I, _P, _I, _L, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    # int ap_latent_gather(cache, dtype, page_stride, P, record, block_table, max_blocks, seq_start, context_lens,
    #                      nseq, out, where, width, total, window, stream)
    "ap_latent_gather": [_P, _I, _L, _I, _I, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _P],
    # int ap_latent_decode(q, out, cache, block_table, max_blocks, seq_start, positions, nseq, nh, record, value,
    #                      P, page_stride, scale, gate, gate_ld, nsplit, scratch, scratch_floats, window, sink, stream)
    "ap_latent_decode": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _L, _F, _P, _L, _I, _P, _L, _I, _P, _P],
    "ap_latent_decode_splits": [_I, _I, _I],
    "ap_latent_decode_takes": [_I, _I],
    # int ap_latent_prefill(q, out, kv, where, width, seq_start, positions, nseq, T, nh, key, value, scale, gate,
    #                       gate_ld, window, sink, stream)
    "ap_latent_prefill": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _P, _L, _I, _P, _P],
    "ap_latent_prefill_takes": [_I, _I],
    # int ap_causal_conv_silu(in, ld_in, col0, w, bias, state, state_stride, token_seq, seq_start, positions,
    #                         state_slots, out, T, nseq, C, taps, stream)
    "ap_causal_conv_silu": [_P, _L, _I, _P, _P, _P, _L, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    # int ap_ssm_scan(xbc, ld_xbc, dt_raw, ld_dt, dt_bias, a_log, d_skip, state, state_stride, seq_start, positions,
    #                 state_slots, y, T, nseq, heads, groups, N, vdim, stream)
    "ap_ssm_scan": [_P, _L, _P, _L, _P, _P, _P, _P, _L, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    # int ap_gated_group_rmsnorm(y, z, ld_z, w, w_dtype, eps, out, out_dtype, T, inner, parts, stream)
    "ap_gated_group_rmsnorm": [_P, _P, _L, _P, _I, _F, _P, _I, _I, _I, _I, _P],
    # int ap_gated_act(in, in_dtype, out, out_dtype, T, I, pairs, act, limit, alpha, shift, row_scale, scale_index, stream)
    "ap_gated_act": [_P, _I, _P, _I, _I, _I, _I, _I, _F, _F, _F, _P, _P, _P],
    "ap_moe_route": [_P, _P, _P, _P, _I, _I, _I, _P],
    # int ap_moe_route_rows(rows, rows_dtype, router, router_dtype, K, bias, chosen, weight, T, E, top, mode, stream)
    "ap_moe_route_rows": [_P, _I, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _P],
    "ap_moe_max_tiles": [_I, _I],
    # int ap_moe_sort(chosen, perm, place, tiles, offsets, pairs, E, real, stream)
    "ap_moe_sort": [_P, _P, _P, _P, _P, _I, _I, _I, _P],
    "ap_moe_gather": [_P, _P, _P, _I, _I, _I, _P],
    # int ap_moe_gate_up(a, a_dtype, w, w_dtype, y, y_dtype, perm, top, tiles, pairs, E, F, K, act, limit, alpha,
    #                    shift, pair_scale, stream)
    "ap_moe_gate_up": [_P, _I, _P, _I, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _F, _F, _F, _P, _P],
    # int ap_moe_down(y, y_dtype, w, w_dtype, o, tiles, pairs, E, H, F, stream)
    "ap_moe_down": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _P],
    # int ap_moe_combine(o, place, weight, delta, T, H, top, chosen, real, rows, rows_dtype, stream)
    "ap_moe_combine": [_P, _P, _P, _P, _I, _I, _I, _P, _I, _P, _I, _P],
    # int ap_add_dyt(x, delta, S, delta_stride, w, b, alpha, out, out_dtype, rows, R, H, stream)
    "ap_add_dyt": [_P, _P, _I, _L, _P, _P, _F, _P, _I, _P, _I, _I, _P],
    # int ap_dyt_shift(x, w, b, alpha, shift, state, state_stride, seq_start, positions, token_seq, state_slots,
    #                  out, out_dtype, T, H, stream)
    "ap_dyt_shift": [_P, _P, _P, _F, _P, _P, _L, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    # int ap_stream_mix(x, delta, S, delta_stride, streams, stream_stride, k, weights, n, stream)
    "ap_stream_mix": [_P, _P, _I, _L, _P, _L, _I, _P, _L, _P],
    # int ap_linear_scan(q, ld_q, k, ld_k, v, ld_v, decay_channel, ld_dc, decay_head, ld_dh, decay_const, dt_bias, beta,
    #                    ld_beta, cos_sin, rot_dims, state, state_stride, seq_start, positions, state_slots, y, ld_y,
    #                    T, nseq, heads, qk_heads, D, V, decay_mode, qk_mode, tau, unit_eps, out_scale, stream)
    "ap_linear_scan": [_P, _L, _P, _L, _P, _L, _P, _L, _P, _L, _P, _P, _P, _L, _P, _I, _P, _L, _P, _P, _P, _P, _L,
                       _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _F, _P],
    # int ap_head_norm_gate(y, ld_y, gate, ld_g, w, eps, out_scale, out, out_dtype, T, heads, V, stream)
    "ap_head_norm_gate": [_P, _L, _P, _L, _P, _F, _F, _P, _I, _I, _I, _I, _P],
    # int ap_gated_postnorm(x, rows, R, delta, S, slice_stride, gate, ld_gate, gate_bias, alpha, w, w_dtype, groups,
    #                       eps, update, out, out_dtype, H, stream)
    "ap_gated_postnorm": [_P, _P, _I, _P, _I, _L, _P, _L, _P, _F, _P, _I, _I, _F, _I, _P, _I, _I, _P],
    # int ap_gated_row_add(delta, other, h, h_dtype, g, g_dtype, T, H, stream)
    "ap_gated_row_add": [_P, _P, _P, _I, _P, _I, _I, _I, _P],
    # int ap_bias_act(in, in_dtype, bias, out, out_dtype, T, N, act, stream)
    "ap_bias_act": [_P, _I, _P, _P, _I, _I, _I, _I, _P],
}
_OPTIONAL_CORE_SIGNATURES = {
    # int ap_gemm_tc(a, w, out, out_dtype, M, N, K, lda, ldw, ldc, nsplit, split_stride, reduce, epi,
    #                ss_in, ss_in_parts, inv_width, eps, xb, ldxb, ss_out, ss_out_parts, stream)
    "ap_gemm_tc": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _I, _L, _I, _I, _P, _I, _F, _F, _P, _L, _P, _I, _P],
    "ap_gemm_tc_residual_parts": [_I, _I],
    # int ap_gemm_tc_rope(a, w, M, K, lda, ldw, nsplit, ss_in, ss_in_parts, inv_width, eps, q_out, cache, positions,
    #                     token_seq, block_table, max_blocks, cos_sin, pairing, nh, nkv, hd, P, page_stride, stream)
    "ap_gemm_tc_rope": [_P, _P, _I, _I, _L, _L, _I, _P, _I, _F, _F, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I,
                        _L, _P],
    "ap_gemm_tc_dual": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P],
    "ap_gemm_tc_pair": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _I, _P, _L, _P],
    "ap_gemm_tc_pair_status": [],
    "ap_gemm_tc_pair_reset_status": [],
    "ap_gemm_tc_persistent": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _I, _P, _L, _P],
    "ap_gemm_tc_plan": [_I, _I, _I],
    "ap_gemm_tc_prefers_dual": [_I, _I, _I],
    "ap_gemm_tc_prefers_pair": [_I, _I, _I],
    "ap_gemm_tc_prefers_persistent": [_I, _I, _I],
    "ap_gemm_tc_status": [],
    "ap_gemm_tc_reset_status": [],
}
_ATTN_SIGNATURES = {
    "ap_attention_rows": [_P, _P, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _L, _F, _I, _P],
}

_lock = threading.Lock()
_core = None
_attn: Dict[int, ctypes.CDLL] = {}


def _declare(lib: ctypes.CDLL, signatures, optional=False) -> None:
    for name, args in signatures.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            if optional:
                continue
            raise
        fn.argtypes = args
        fn.restype = c_int
    lib.ap_last_error.restype = c_char_p
    lib.ap_last_error.argtypes = []
    if hasattr(lib, "ap_gemm_tc_persistent_scratch_bytes"):
        lib.ap_gemm_tc_persistent_scratch_bytes.restype = c_longlong
        lib.ap_gemm_tc_persistent_scratch_bytes.argtypes = []


def _require_cuda() -> None:
    import torch
    if not torch.cuda.is_available():
        raise KernelError(
            "no CUDA device is visible: allpaca_b200 runs only on a GPU (sm_100a); "
            "there is no CPU implementation of its kernels")


def core() -> ctypes.CDLL:
    """The library of size-independent kernels, built on first use."""
    global _core
    if _core is None:
        with _lock:
            if _core is None:
                path = _build.build_core()
                lib = ctypes.CDLL(path)
                _declare(lib, _CORE_SIGNATURES)
                _declare(lib, _OPTIONAL_CORE_SIGNATURES, optional=True)
                _core = lib
    return _core


def attention(head_dim: int) -> ctypes.CDLL:
    """The attention library specialised for one head size, built on first use."""
    lib = _attn.get(head_dim)
    if lib is None:
        with _lock:
            lib = _attn.get(head_dim)
            if lib is None:
                path = _build.build_attention(head_dim)
                lib = ctypes.CDLL(path)
                _declare(lib, _ATTN_SIGNATURES)
                for name, args in _OPTIONAL_ATTN_SIGNATURES.items():
                    if hasattr(lib, name):
                        getattr(lib, name).argtypes = args
                        getattr(lib, name).restype = c_int
                _attn[head_dim] = lib
    return lib


_OPTIONAL_ATTN_SIGNATURES: Dict[str, list] = {
    "ap_attention_tc": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _L, _F, _I, _I, _I, _I, _P, _P, _P],
    "ap_attention_tc_tokens_per_tile": [_I, _I],
    "ap_attention_tcgen05": [_P, _P, _P, _L, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _L, _F, _I, _I, _P],
    "ap_attention_tcgen05_supports": [_I, _I, _I, _I],
    "ap_attention_tcgen05_tokens_per_tile": [_I, _I],
    "ap_attention_tcgen05_status": [],
    "ap_attention_tcgen05_wide": [_P, _P, _P, _L, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _L, _F, _I, _I, _P],
    "ap_attention_tcgen05_wide_supports": [_I, _I, _I, _I],
    "ap_attention_tcgen05_wide_tokens_per_cta": [_I, _I],
    "ap_attention_tcgen05_wide_status": [],
    # int ap_attention_decode_tma(q, out, cache, num_pages, block_table, max_blocks, positions, T, nh, nkv, hd, P,
    #                             page_stride, scale, window, nsplit, part_o, part_ml, stream)
    "ap_attention_decode_tma": [_P, _P, _P, _L, _P, _I, _P, _I, _I, _I, _I, _I, _L, _F, _I, _I, _P, _P, _P],
    "ap_attention_decode_tma_supports": [_I, _I, _I, _I],
    "ap_attention_decode_tma_in_cluster": [_I, _I, _I],
    "ap_attention_decode_tma_status": [],
    "ap_attention_decode_tma_slots": [],
}


def call(lib: ctypes.CDLL, name: str, *args) -> None:
    """Call an entry point and raise with the library's own message on failure."""
    global _launches
    rc = getattr(lib, name)(*args)
    _launches += 1
    if rc != 0:
        msg = lib.ap_last_error()
        raise KernelError(f"{name} failed (status {rc}): {msg.decode() if msg else 'no message'}")


_raw_stream = None


def stream_handle() -> int:
    """The CUDA stream torch currently launches on, as the integer the C entry points take."""
    global _raw_stream
    if _raw_stream is None:
        import torch
        fast = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        if fast is not None:
            _raw_stream = lambda: fast(torch.cuda.current_device())          # noqa: E731
        else:
            _raw_stream = lambda: torch.cuda.current_stream().cuda_stream    # noqa: E731
    return _raw_stream()


_launches = 0


def launch_count() -> int:
    """Calls into the kernel libraries so far (each launches one kernel)."""
    return _launches


def add_launches(n: int) -> None:
    """Account for kernels launched by replaying a captured graph."""
    global _launches
    _launches += n
