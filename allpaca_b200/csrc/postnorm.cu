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

template <typename TW, typename TO>
__global__ void __launch_bounds__(PN_THREADS)
gated_postnorm_kernel(float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ delta, int S,
                      size_t slice_stride, const float* __restrict__ gate, long long ld_gate,
                      const float* __restrict__ gate_bias, float alpha, const TW* __restrict__ w, int groups,
                      float eps, int update, TO* __restrict__ out, int H) {
    extern __shared__ __align__(16) float row_s[];          // [H] values, then [units] partial sums
    ap_pdl_trigger();
    ap_pdl_wait();
    const int r = blockIdx.x;
    const size_t t = rows ? (size_t)rows[r] : (size_t)r;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gw = H / groups;
    const int split = groups >= PN_WARPS ? 1 : PN_WARPS / groups;    // warps that share a group
    const int units = groups * split;
    const int chunk = (gw + split - 1) / split;
    float* ss_s = row_s + H;
    float* xr = x + t * H;
    for (int u = warp; u < units; u += PN_WARPS) {
        const int g = u / split, p = u - g * split;
        const int c0 = g * gw + p * chunk, c1 = min(g * gw + (p + 1) * chunk, (g + 1) * gw);
        float ss = 0.f;
        for (int c = c0 + lane; c < c1; c += 32) {
            float v = alpha * xr[c];
            if (delta) {
                float d = 0.f;
                for (int s = 0; s < S; ++s) d += delta[s * slice_stride + t * H + c];
                if (gate) d *= 1.0f / (1.0f + expf(-(gate[t * ld_gate + c] + (gate_bias ? gate_bias[c] : 0.f))));
                v += d;
            }
            row_s[c] = v;
            ss = fmaf(v, v, ss);
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
        for (int c = c0 + lane; c < c1; c += 32) {
            const float v = row_s[c] * inv * ap_to_float(w[c]);
            if (update) xr[c] = v;
            if (out) out[(size_t)r * H + c] = ap_from_float<TO>(v);
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
    const int split = groups >= PN_WARPS ? 1 : PN_WARPS / groups;
    const size_t smem = ((size_t)H + (size_t)groups * split) * sizeof(float);
    AP_REQUIRE(smem <= 200 * 1024, "gated_postnorm: a row of %d does not fit shared memory", H);
#define LAUNCH(TW, TO)                                                                                              \
    do {                                                                                                            \
        auto kern = gated_postnorm_kernel<TW, TO>;                                                                  \
        if (smem > 48 * 1024) {                                                                                     \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
            AP_REQUIRE(e == cudaSuccess, "gated_postnorm: cannot reserve %zu bytes of shared memory", smem);        \
        }                                                                                                           \
        AP_CHECK_PDL_LAUNCH("gated_postnorm", ap_launch_pdl(kern, dim3((unsigned)R), dim3(PN_THREADS), smem, stream, x, \
                                                            rows, delta, S, (size_t)slice_stride, gate, ld_gate,    \
                                                            gate_bias, alpha, (const TW*)w, groups, eps, update,    \
                                                            (TO*)out, H));                                          \
    } while (0)
    const int od = out ? out_dtype : AP_F32;
    if (w_dtype == AP_F32 && od == AP_F32) LAUNCH(float, float);
    else if (w_dtype == AP_F32 && od == AP_BF16) LAUNCH(float, bf16);
    else if (w_dtype == AP_BF16 && od == AP_BF16) LAUNCH(bf16, bf16);
    else if (w_dtype == AP_BF16 && od == AP_F32) LAUNCH(bf16, float);
    else AP_REQUIRE(false, "gated_postnorm: unknown dtypes w=%d out=%d", w_dtype, out_dtype);
#undef LAUNCH
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
