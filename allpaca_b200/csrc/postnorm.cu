// The norm of a layer that normalises AFTER the sum, with the sublayer's result under a gate:
//
//   v = alpha * x + sigmoid(gate + gate_bias) * sum_s delta[s]        x <- group_rmsnorm(v) * w
//
// group_rmsnorm cuts the row into `groups` equal runs and divides each by its own sqrt(mean(run^2) + eps).
// The same kernel serves a plain grouped RMS norm of chosen rows (no delta, no gate, alpha 1, the stream left as
// it is): the model's last norm.  And gated_row_add: delta[t] += sigmoid(h[t] . g) * other[t], one gate per row.
//
// All 32-bit up to the store; the updated row may also be written in the activation type for the sublayer
// that reads the stream next.  One CTA per row: the row's values wait in shared memory between the pass that
// sums their squares and the pass that scales them; a group's sum is the sum of its warps' parts in a fixed
// order, so a row has the same bits in any batch.
#include "common.cuh"

#define PN_THREADS 256
#define PN_WARPS (PN_THREADS / 32)

// VEC numbers at a time (4: 16-byte accesses where every run starts on such a boundary; else 1)
template <int VEC> __device__ __forceinline__ void pn_load(const float* p, float* v) {
    if constexpr (VEC == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
        v[0] = p[0];
    }
}
template <int VEC> __device__ __forceinline__ void pn_load(const bf16* p, float* v) {
    if constexpr (VEC == 4) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    } else {
        v[0] = __bfloat162float(p[0]);
    }
}
template <int VEC> __device__ __forceinline__ void pn_store(float* p, const float* v) {
    if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else p[0] = v[0];
}
template <int VEC> __device__ __forceinline__ void pn_store(bf16* p, const float* v) {
    if constexpr (VEC == 4) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 t;
        t.x = *reinterpret_cast<const unsigned*>(&a);
        t.y = *reinterpret_cast<const unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = t;
    } else {
        p[0] = __float2bfloat16_rn(v[0]);
    }
}

template <typename TW, typename TO, int VEC>
__global__ void __launch_bounds__(PN_THREADS)
gated_postnorm_kernel(float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ delta, int S,
                      size_t slice_stride, const float* __restrict__ gate, long long ld_gate,
                      const float* __restrict__ gate_bias, float alpha, const TW* __restrict__ w, int groups,
                      float eps, int update, TO* __restrict__ out, int H, int split, int chunk) {
    extern __shared__ __align__(16) float row_s[];          // [H] values, then [units] partial sums
    ap_pdl_trigger();
    ap_pdl_wait();
    const int r = blockIdx.x;
    const size_t t = rows ? (size_t)rows[r] : (size_t)r;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gw = H / groups;
    const int units = groups * split;                        // `split` warps share a group, `chunk` columns each
    float* ss_s = row_s + H;
    float* xr = x + t * H;
    for (int u = warp; u < units; u += PN_WARPS) {
        const int g = u / split, p = u - g * split;
        const int c0 = g * gw + p * chunk, c1 = min(g * gw + (p + 1) * chunk, (g + 1) * gw);
        float ss = 0.f;
        for (int c = c0 + lane * VEC; c < c1; c += 32 * VEC) {
            float v[VEC], d[VEC], e[VEC];
            pn_load<VEC>(xr + c, v);
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[i] *= alpha;
            if (delta) {
                pn_load<VEC>(delta + t * H + c, d);
                for (int s = 1; s < S; ++s) {
                    pn_load<VEC>(delta + s * slice_stride + t * H + c, e);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) d[i] += e[i];
                }
                if (gate) {
                    pn_load<VEC>(gate + t * ld_gate + c, e);
                    if (gate_bias) {
                        float b[VEC];
                        pn_load<VEC>(gate_bias + c, b);
#pragma unroll
                        for (int i = 0; i < VEC; ++i) e[i] += b[i];
                    }
#pragma unroll
                    for (int i = 0; i < VEC; ++i) d[i] *= 1.0f / (1.0f + expf(-e[i]));
                }
#pragma unroll
                for (int i = 0; i < VEC; ++i) v[i] += d[i];
            }
            pn_store<VEC>(row_s + c, v);
#pragma unroll
            for (int i = 0; i < VEC; ++i) ss = fmaf(v[i], v[i], ss);
        }
        ss = ap_warp_sum(ss);
        if (lane == 0) ss_s[u] = ss;
    }
    __syncthreads();
    for (int u = warp; u < units; u += PN_WARPS) {
        const int g = u / split, p = u - g * split;
        const int c0 = g * gw + p * chunk, c1 = min(g * gw + (p + 1) * chunk, (g + 1) * gw);
        float total = 0.f;
        for (int j = 0; j < split; ++j) total += ss_s[g * split + j];
        const float inv = 1.0f / sqrtf(total / (float)gw + eps);
        for (int c = c0 + lane * VEC; c < c1; c += 32 * VEC) {
            float v[VEC], ww[VEC];
            pn_load<VEC>(row_s + c, v);
            pn_load<VEC>(w + c, ww);
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[i] = v[i] * inv * ww[i];
            if (update) pn_store<VEC>(xr + c, v);
            if (out) pn_store<VEC>(out + (size_t)r * H + c, v);
        }
    }
}

AP_EXPORT int ap_gated_postnorm(float* x, const int* rows, int R, const float* delta, int S, long long slice_stride,
                                const float* gate, long long ld_gate, const float* gate_bias, float alpha,
                                const void* w, int w_dtype, int groups, float eps, int update, void* out,
                                int out_dtype, int H, cudaStream_t stream) {
    AP_REQUIRE(R >= 0 && H > 0 && groups > 0 && H % groups == 0, "gated_postnorm: a row of %d does not fall into %d equal parts",
               H, groups);
    AP_REQUIRE(x && w && (update || out), "gated_postnorm: an operand is missing");
    AP_REQUIRE(!(update && rows), "gated_postnorm: chosen rows are normed into `out` only");
    AP_REQUIRE(delta == nullptr || S > 0, "gated_postnorm: partial sums without slices");
    AP_REQUIRE(gate == nullptr || (delta != nullptr && ld_gate >= H), "gated_postnorm: a gate needs a result to act on");
    if (R == 0) return AP_OK;
    const int gw = H / groups;
    const int split = groups >= PN_WARPS ? 1 : PN_WARPS / groups;
    // 16-byte accesses where every warp's run of a group starts on such a boundary in every operand
    const bool vec = gw % 4 == 0 && ((((uintptr_t)x) | ((uintptr_t)delta) | ((uintptr_t)gate) | ((uintptr_t)gate_bias) |
                                     ((uintptr_t)w) | ((uintptr_t)out)) & 15) == 0 && slice_stride % 4 == 0 &&
                     (gate == nullptr || ld_gate % 4 == 0);
    int chunk = (gw + split - 1) / split;
    if (vec) chunk = (chunk + 3) / 4 * 4;
    const size_t smem = ((size_t)H + (size_t)groups * split) * sizeof(float);
    AP_REQUIRE(smem <= 200 * 1024, "gated_postnorm: a row of %d does not fit shared memory", H);
#define LAUNCH_V(TW, TO, VEC)                                                                                       \
    do {                                                                                                            \
        auto kern = gated_postnorm_kernel<TW, TO, VEC>;                                                             \
        if (smem > 48 * 1024) {                                                                                     \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
            AP_REQUIRE(e == cudaSuccess, "gated_postnorm: cannot reserve %zu bytes of shared memory", smem);        \
        }                                                                                                           \
        AP_CHECK_PDL_LAUNCH("gated_postnorm", ap_launch_pdl(kern, dim3((unsigned)R), dim3(PN_THREADS), smem, stream, x, \
                                                            rows, delta, S, (size_t)slice_stride, gate, ld_gate,    \
                                                            gate_bias, alpha, (const TW*)w, groups, eps, update,    \
                                                            (TO*)out, H, split, chunk));                            \
    } while (0)
#define LAUNCH(TW, TO) do { if (vec) LAUNCH_V(TW, TO, 4); else LAUNCH_V(TW, TO, 1); } while (0)
    const int od = out ? out_dtype : AP_F32;
    if (w_dtype == AP_F32 && od == AP_F32) LAUNCH(float, float);
    else if (w_dtype == AP_F32 && od == AP_BF16) LAUNCH(float, bf16);
    else if (w_dtype == AP_BF16 && od == AP_BF16) LAUNCH(bf16, bf16);
    else if (w_dtype == AP_BF16 && od == AP_F32) LAUNCH(bf16, float);
    else AP_REQUIRE(false, "gated_postnorm: unknown dtypes w=%d out=%d", w_dtype, out_dtype);
#undef LAUNCH
#undef LAUNCH_V
    return AP_OK;
}

// delta[t, :] += sigmoid(h[t] . g) * other[t, :]: one CTA per row
template <typename TA, typename TW>
__global__ void __launch_bounds__(PN_THREADS)
gated_row_add_kernel(float* __restrict__ delta, const float* __restrict__ other, const TA* __restrict__ h,
                     const TW* __restrict__ g, int H) {
    __shared__ float scratch[32];
    ap_pdl_trigger();
    ap_pdl_wait();
    const size_t t = blockIdx.x;
    float dot = 0.f;
    for (int c = threadIdx.x; c < H; c += PN_THREADS) dot = fmaf(ap_to_float(h[t * H + c]), ap_to_float(g[c]), dot);
    dot = ap_block_sum(dot, scratch);
    const float s = 1.0f / (1.0f + expf(-dot));
    for (int c = threadIdx.x; c < H; c += PN_THREADS) delta[t * H + c] = fmaf(s, other[t * H + c], delta[t * H + c]);
}

AP_EXPORT int ap_gated_row_add(float* delta, const float* other, const void* h, int h_dtype, const void* g,
                               int g_dtype, int T, int H, cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && H > 0 && delta && other && h && g, "gated_row_add: bad arguments");
    if (T == 0) return AP_OK;
#define LAUNCH(TA, TW)                                                                                              \
    AP_CHECK_PDL_LAUNCH("gated_row_add", ap_launch_pdl(gated_row_add_kernel<TA, TW>, dim3((unsigned)T),             \
                                                       dim3(PN_THREADS), 0, stream, delta, other, (const TA*)h,     \
                                                       (const TW*)g, H))
    if (h_dtype == AP_F32 && g_dtype == AP_F32) LAUNCH(float, float);
    else if (h_dtype == AP_BF16 && g_dtype == AP_BF16) LAUNCH(bf16, bf16);
    else if (h_dtype == AP_BF16 && g_dtype == AP_F32) LAUNCH(bf16, float);
    else AP_REQUIRE(false, "gated_row_add: unsupported dtypes h=%d g=%d", h_dtype, g_dtype);
#undef LAUNCH
    return AP_OK;
}
