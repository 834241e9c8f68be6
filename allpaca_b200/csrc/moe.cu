// A routed feed-forward (mixture of experts) and the gated activations of feed-forwards:
//
//   moe_route      per row: the `top` experts with the largest router logits (ties: the lower
//                  index), shares = exp(z_e) / sum over the selected exp(z_s); all 32-bit.  Or
//                  (ROUTE_SOFTMAX_ALL) scores s = softmax(z) over all experts, the `top` largest
//                  s + bias chosen, shares = the chosen s divided by their sum.  Experts from
//                  `real` on are identity experts: no weights, their result is the row's input
//   moe_sort       (row, choice) pairs grouped by expert: a permutation, every pair's place in
//                  it, and a list of row tiles (expert, first place, rows) for the products
//   moe_gate_up    for every tile: y = act(A W_gate[e]^T, A W_up[e]^T), rows gathered by the permutation
//   moe_down       for every tile: o = y W_down[e]^T, 32-bit
//   moe_combine    delta[t] = sum_k weight[t,k] * o[place(t,k)], in the order of k
//   gated_act      the activation alone, for a dense feed-forward whose product left [gate | up]
//
// Activations (g = gate, u = up):
//   0 silu:   g / (1 + exp(-g)) * u
//   1 relu:   max(g, 0) * u
//   2 clamped sigmoid gate: g' = min(g, limit), u' = clamp(u, -limit, limit); g' * sigmoid(alpha g') * (u' + shift)
//
// The products run on the CUDA cores with 32-bit accumulation (every output element one
// thread's sum over k in ascending order), so a row's result does not depend on where the
// sort placed it or on what else is in the batch.  Nothing is decided on the host: counts and
// tiles stay on the device, grids are planned for the worst case and surplus CTAs return.
#include "common.cuh"
#include <float.h>

#define ACT_SILU 0
#define ACT_RELU 1
#define ACT_CLAMPED 2
#define ACT_GELU_TANH 3

__device__ __forceinline__ float gated_activation(float g, float u, int act, float limit, float alpha, float shift) {
    if (act == ACT_RELU) return fmaxf(g, 0.f) * u;
    if (act == ACT_GELU_TANH)        // 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) u
        return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
    if (act == ACT_CLAMPED) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-alpha * g)) * (u + shift);
    }
    return g / (1.0f + expf(-g)) * u;
}

// ---- the activation alone ------------------------------------------------------------
template <typename TI, typename TO>
__global__ void gated_act_kernel(const TI* __restrict__ in, TO* __restrict__ out, int T, int I, int pairs, int act,
                                 float limit, float alpha, float shift, const float* __restrict__ row_scale,
                                 const int* __restrict__ scale_index) {
    ap_pdl_trigger();
    ap_pdl_wait();
    const size_t n = (size_t)T * I;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / I, j = e - t * I;
        const size_t base = t * 2 * (size_t)I;
        const float g = ap_to_float(in[pairs ? base + 2 * j : base + j]);
        const float u = ap_to_float(in[pairs ? base + 2 * j + 1 : base + I + j]);
        // a scale of the row's INPUT: both products are linear in it, so it multiplies both sums
        const float sc = row_scale ? row_scale[scale_index ? scale_index[t] : t] : 1.0f;
        out[e] = ap_from_float<TO>(gated_activation(g * sc, u * sc, act, limit, alpha, shift));
    }
}

AP_EXPORT int ap_gated_act(const void* in, int in_dtype, void* out, int out_dtype, int T, int I, int pairs, int act,
                           float limit, float alpha, float shift, const float* row_scale, const int* scale_index,
                           cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && I > 0 && act >= 0 && act <= 3, "gated_act: bad sizes T=%d I=%d or activation %d", T, I, act);
    if (T == 0) return AP_OK;
    long long blocks = ((long long)T * I + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
#define LAUNCH(TI, TO)                                                                                              \
    AP_CHECK_PDL_LAUNCH("gated_act", ap_launch_pdl(gated_act_kernel<TI, TO>, dim3((unsigned)blocks), dim3(256), 0, stream, \
                                                   (const TI*)in, (TO*)out, T, I, pairs, act, limit, alpha, shift, row_scale, \
                                                   scale_index))
    if (in_dtype == AP_F32 && out_dtype == AP_F32) LAUNCH(float, float);
    else if (in_dtype == AP_F32 && out_dtype == AP_BF16) LAUNCH(float, bf16);
    else if (in_dtype == AP_BF16 && out_dtype == AP_BF16) LAUNCH(bf16, bf16);
    else AP_REQUIRE(false, "gated_act: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
#undef LAUNCH
    return AP_OK;
}

// ---- routing ---------------------------------------------------------------------------
#define ROUTE_MAX_PER_LANE 8          // experts <= 256
#define ROUTE_MAX_TOP 16
#define ROUTE_TOP_SOFTMAX 0           // the `top` largest z + bias; shares: their softmax
#define ROUTE_SOFTMAX_ALL 1           // s = softmax(z) over all; the `top` largest s + bias; shares: their s / sum
#define ROUTE_SIGMOID 2               // s = sigmoid(z), each output alone; the `top` largest s + bias; shares: their s as it is

// One CTA per RPB rows: eight warps, or, for a CTA of one row, a warp per router output (at most 32: a step of
// few rows is a chain of loads per warp, which more warps shorten).  With `rows` the warps first form the rows' router logits: E dot
// products of each row with the router's rows, the experts dealt to the warps in turn, 32-bit sums
// (every lane a strided part of K, 16-byte loads where the types and alignment allow, then a
// butterfly over the lanes: one fixed order per row, whatever the batch and whichever rows share its CTA;
// a part of the router that a warp has loaded meets all RPB rows before the next is loaded, so that a step of
// many rows reads the router RPB times less often); else the logits are read from `logits` [T, E].  The bias is
// added; warp r takes the `top` largest of row r and their shares.
#define ROUTE_THREADS 256            // a CTA of several rows; a CTA of one row has up to ROUTE_MAX_THREADS
#define ROUTE_MAX_THREADS 1024
template <typename TA, typename TW, int RPB>
__global__ void __launch_bounds__(ROUTE_MAX_THREADS)
moe_route_kernel(const float* __restrict__ logits, const TA* __restrict__ rows, const TW* __restrict__ router, int K,
                 const float* __restrict__ bias, int* __restrict__ chosen, float* __restrict__ weight, int T, int E,
                 int top, int mode) {
    __shared__ float z_all[RPB][32 * ROUTE_MAX_PER_LANE];
    ap_pdl_trigger();
    ap_pdl_wait();
    const int t0 = blockIdx.x * RPB, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nrows = min(RPB, T - t0);
    if (rows != nullptr) {
        const TA* a = rows + (size_t)t0 * K;
        const bool vec = sizeof(TA) == 2 && sizeof(TW) == 2 && K % 8 == 0 &&
                         ((((uintptr_t)rows) | ((uintptr_t)router)) & 15) == 0;
        for (int e = warp; e < E; e += (int)blockDim.x / 32) {
            const TW* w = router + (size_t)e * K;
            float sum[RPB];
#pragma unroll
            for (int r = 0; r < RPB; ++r) sum[r] = 0.f;
            if (vec) {
#pragma unroll 4
                for (int k = lane * 8; k < K; k += 256) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(w) + k);
                    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
                    for (int r = 0; r < RPB; ++r) {
                        if (r < nrows) {
                            const uint4 av = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(a) + (size_t)r * K + k);
                            const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const float2 x = __bfloat1622float2(a2[q]), y = __bfloat1622float2(w2[q]);
                                sum[r] = fmaf(x.y, y.y, fmaf(x.x, y.x, sum[r]));
                            }
                        }
                    }
                }
            } else {
#pragma unroll 4
                for (int k = lane; k < K; k += 32) {
                    const float wk = ap_to_float(w[k]);
#pragma unroll
                    for (int r = 0; r < RPB; ++r)
                        if (r < nrows) sum[r] = fmaf(ap_to_float(a[(size_t)r * K + k]), wk, sum[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < RPB; ++r) {
                const float v = ap_warp_sum(sum[r]);
                if (lane == 0) z_all[r][e] = v + ((bias && mode == ROUTE_TOP_SOFTMAX) ? bias[e] : 0.f);
            }
        }
    } else {
        for (int r = 0; r < nrows; ++r)
            for (int e = threadIdx.x; e < E; e += (int)blockDim.x)
                z_all[r][e] = logits[(size_t)(t0 + r) * E + e] + ((bias && mode == ROUTE_TOP_SOFTMAX) ? bias[e] : 0.f);
    }
    __syncthreads();
    if (warp >= nrows) return;
    const int t = t0 + warp;
    const float* z_s = z_all[warp];
    float z[ROUTE_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        z[i] = e < E ? z_s[e] : -FLT_MAX;
    }
    // ROUTE_SOFTMAX_ALL: scores s = softmax(z) over ALL experts; the choice goes by s + bias, the shares are
    // the chosen experts' s divided by their sum
    float sc[ROUTE_MAX_PER_LANE];
    if (mode == ROUTE_SOFTMAX_ALL) {
        float mx = -FLT_MAX;
#pragma unroll
        for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) mx = fmaxf(mx, z[i]);
        mx = ap_warp_max(mx);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
            sc[i] = lane + 32 * i < E ? expf(z[i] - mx) : 0.f;
            sum += sc[i];
        }
        sum = ap_warp_sum(sum);
#pragma unroll
        for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            sc[i] /= sum;
            z[i] = e < E ? sc[i] + (bias ? bias[e] : 0.f) : -FLT_MAX;
        }
    } else if (mode == ROUTE_SIGMOID) {
#pragma unroll
        for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            sc[i] = e < E ? 1.0f / (1.0f + expf(-z[i])) : 0.f;
            // without a bias the order of the scores is the order of the logits, which do not saturate
            z[i] = e < E ? (bias ? sc[i] + bias[e] : z[i]) : -FLT_MAX;
        }
    }
    float best[ROUTE_MAX_TOP];
    int who[ROUTE_MAX_TOP];
    for (int k = 0; k < top; ++k) {
        float v = -FLT_MAX;
        int idx = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < E && (z[i] > v || (z[i] == v && e < idx))) { v = z[i]; idx = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        if (mode != ROUTE_TOP_SOFTMAX) {
            // the chosen expert's score without the bias: its owner's lane has it
            float own = 0.f;
#pragma unroll
            for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i)
                if (lane + 32 * i == idx) own = sc[i];
            v = __shfl_sync(0xffffffffu, own, idx & 31);
        }
        best[k] = v;
        who[k] = idx;
#pragma unroll
        for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i)
            if (lane + 32 * i == idx) z[i] = -FLT_MAX;        // taken
    }
    if (lane == 0 && mode == ROUTE_SIGMOID) {
        for (int k = 0; k < top; ++k) {
            chosen[(size_t)t * top + k] = who[k];
            weight[(size_t)t * top + k] = best[k];
        }
    } else if (lane == 0 && mode == ROUTE_SOFTMAX_ALL) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) sum += best[k];
        for (int k = 0; k < top; ++k) {
            chosen[(size_t)t * top + k] = who[k];
            weight[(size_t)t * top + k] = best[k] / (sum + 1e-20f);
        }
    } else if (lane == 0) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) sum += expf(best[k] - best[0]);      // best[0] is the largest
        for (int k = 0; k < top; ++k) {
            chosen[(size_t)t * top + k] = who[k];
            weight[(size_t)t * top + k] = expf(best[k] - best[0]) / sum;
        }
    }
}

AP_EXPORT int ap_moe_route(const float* logits, const float* bias, int* chosen, float* weight, int T, int E, int top,
                           cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && E > 0 && E <= 32 * ROUTE_MAX_PER_LANE && top > 0 && top <= E && top <= ROUTE_MAX_TOP,
               "moe_route: %d experts (at most %d), %d chosen (at most %d)", E, 32 * ROUTE_MAX_PER_LANE, top, ROUTE_MAX_TOP);
    if (T == 0) return AP_OK;
    AP_CHECK_PDL_LAUNCH("moe_route", ap_launch_pdl(moe_route_kernel<float, float, 1>, dim3((unsigned)T), dim3(ROUTE_THREADS),
                                                   0, stream, logits, (const float*)nullptr, (const float*)nullptr, 0, bias,
                                                   chosen, weight, T, E, top, ROUTE_TOP_SOFTMAX));
    return AP_OK;
}

// the same from the rows themselves: rows [T, K], router [E, K]
AP_EXPORT int ap_moe_route_rows(const void* rows, int rows_dtype, const void* router, int router_dtype, int K,
                                const float* bias, int* chosen, float* weight, int T, int E, int top, int mode,
                                cudaStream_t stream) {
    AP_REQUIRE(mode == ROUTE_TOP_SOFTMAX || mode == ROUTE_SOFTMAX_ALL || mode == ROUTE_SIGMOID, "moe_route: unknown mode %d", mode);
    AP_REQUIRE(T >= 0 && K > 0 && E > 0 && E <= 32 * ROUTE_MAX_PER_LANE && top > 0 && top <= E && top <= ROUTE_MAX_TOP,
               "moe_route: %d experts (at most %d), %d chosen (at most %d)", E, 32 * ROUTE_MAX_PER_LANE, top, ROUTE_MAX_TOP);
    if (T == 0) return AP_OK;
    // four rows to a CTA in a step of many rows
    const bool four = T >= 512;
    const unsigned threads1 = (unsigned)(32 * (E < 8 ? 8 : E > 32 ? 32 : E));
#define LAUNCH_R(TA, TW, R)                                                                                        \
    AP_CHECK_PDL_LAUNCH("moe_route", ap_launch_pdl(moe_route_kernel<TA, TW, R>, dim3((unsigned)((T + R - 1) / R)),   \
                                                   dim3(R == 1 ? threads1 : ROUTE_THREADS), 0, stream, (const float*)nullptr,           \
                                                   (const TA*)rows, (const TW*)router, K, bias, chosen, weight, T, E, \
                                                   top, mode))
#define LAUNCH(TA, TW) do { if (four) LAUNCH_R(TA, TW, 4); else LAUNCH_R(TA, TW, 1); } while (0)
    if (rows_dtype == AP_F32 && router_dtype == AP_F32) LAUNCH(float, float);
    else if (rows_dtype == AP_BF16 && router_dtype == AP_BF16) LAUNCH(bf16, bf16);
    else if (rows_dtype == AP_BF16 && router_dtype == AP_F32) LAUNCH(bf16, float);
    else AP_REQUIRE(false, "moe_route: unsupported dtypes rows=%d router=%d", rows_dtype, router_dtype);
#undef LAUNCH
#undef LAUNCH_R
    return AP_OK;
}

// ---- grouping pairs by expert ------------------------------------------------------------
#define MOE_BM 64
#define MOE_BN 64
#define MOE_BK 16
#define SORT_MAX_EXPERTS 256

// One CTA.  place[pair] = position of the pair in the grouped order; perm[position] = pair;
// tiles[i] = (expert, first position, rows); tiles[max_tiles] holds their number in .x;
// offsets[e] (optional, E + 1 entries) = first position of expert e's pairs.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ chosen, int* __restrict__ perm, int* __restrict__ place, int3* __restrict__ tiles,
                int* __restrict__ offsets, int pairs, int E, int max_tiles, int real) {
    __shared__ int count[SORT_MAX_EXPERTS];
    __shared__ int first[SORT_MAX_EXPERTS + 1];
    ap_pdl_trigger();
    ap_pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&count[chosen[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            first[e] = at;
            // experts from `real` on have no weights (their result is their input): no tiles for the products
            for (int r = 0; e < real && r < count[e] && nt < max_tiles; r += MOE_BM)
                tiles[nt++] = make_int3(e, at + r, min(MOE_BM, count[e] - r));
            at += count[e];
        }
        first[E] = at;
        tiles[max_tiles] = make_int3(nt, 0, 0);
    }
    __syncthreads();
    if (offsets != nullptr)
        for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = first[e];
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = chosen[i];
        const int p = first[e] + atomicAdd(&count[e], 1);
        perm[p] = i;
        place[i] = p;
    }
}

AP_EXPORT int ap_moe_max_tiles(int pairs, int E) { return (pairs + MOE_BM - 1) / MOE_BM + E; }

AP_EXPORT int ap_moe_sort(const int* chosen, int* perm, int* place, int* tiles, int* offsets, int pairs, int E,
                          int real, cudaStream_t stream) {
    AP_REQUIRE(pairs >= 0 && E > 0 && E <= SORT_MAX_EXPERTS, "moe_sort: %d experts (at most %d)", E, SORT_MAX_EXPERTS);
    AP_REQUIRE(real >= 0 && real <= E, "moe_sort: %d of %d experts have weights", real, E);
    if (pairs == 0) return AP_OK;
    AP_CHECK_PDL_LAUNCH("moe_sort", ap_launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, chosen, perm, place,
                                                  (int3*)tiles, offsets, pairs, E, ap_moe_max_tiles(pairs, E), real));
    return AP_OK;
}

// ---- the experts' products ---------------------------------------------------------------
// GATED: the weight of expert e is [2 F, K] (gate rows, then up rows); out[p, f] = act(gate, up).
// else : the weight is [N, K]; out[p, n] 32-bit.
// A rows: GATED gathers a[perm[p] / top]; else a[p].
template <typename TA, typename TW, typename TO, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TA* __restrict__ A, long long lda, const TW* __restrict__ W, long long w_expert_stride,
                TO* __restrict__ C, long long ldc, const int* __restrict__ perm, int top, const int3* __restrict__ tiles,
                int max_tiles, int N, int K, int act, float limit, float alpha, float shift,
                const float* __restrict__ pair_scale) {
    __shared__ float As[MOE_BK][MOE_BM + 4];
    __shared__ float Ws[GATED ? 2 : 1][MOE_BK][MOE_BN + 4];
    __shared__ int src_row[MOE_BM];
    ap_pdl_trigger();
    ap_pdl_wait();
    if ((int)blockIdx.y >= tiles[max_tiles].x) return;
    const int3 tile = tiles[blockIdx.y];
    const int e = tile.x, p0 = tile.y, rows = tile.z;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int n0 = blockIdx.x * MOE_BN;
    const TW* We = W + (size_t)e * w_expert_stride;
    if (tid < MOE_BM) src_row[tid] = tid < rows ? (GATED ? perm[p0 + tid] / top : p0 + tid) : -1;
    __syncthreads();
    float acc[4][4], acc2[GATED ? 4 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.f;
            if constexpr (GATED) acc2[i][j] = 0.f;
        }
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    const int arow = src_row[lrow];
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = k0 + lk + q;
            const int wn = n0 + lrow;
            As[lk + q][lrow] = (arow >= 0 && k < K) ? ap_to_float(A[(size_t)arow * lda + k]) : 0.f;
            Ws[0][lk + q][lrow] = (wn < N && k < K) ? ap_to_float(We[(size_t)wn * K + k]) : 0.f;
            if constexpr (GATED) Ws[1][lk + q][lrow] = (wn < N && k < K) ? ap_to_float(We[(size_t)(N + wn) * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_BK; ++kk) {
            float a[4], w[4], w2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w[j] = Ws[0][kk][tx * 4 + j];
                if constexpr (GATED) w2[j] = Ws[1][kk][tx * 4 + j];
                else w2[j] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
                    if constexpr (GATED) acc2[i][j] = fmaf(a[i], w2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if constexpr (GATED) {
                // a scale of the pair's INPUT row multiplies both sums
                const float sc = pair_scale ? pair_scale[perm[p0 + r]] : 1.0f;
                v = gated_activation(acc[i][j] * sc, acc2[i][j] * sc, act, limit, alpha, shift);
            }
            C[(size_t)(p0 + r) * ldc + n] = ap_from_float<TO>(v);
        }
    }
}

// The same two products for steps of few rows in bfloat16 (decoding), where the time goes into
// reading the experts' weights once: a CTA of eight warps takes one row tile and 64 output
// columns, holds up to ROWS_MAX of the tile's rows in shared memory (more: in turns), and every
// warp walks its columns with 16-byte weight loads, the lanes across K, all rows at once; the
// lanes' sums meet by butterfly.  A row's sums do not depend on the other rows.
#define ROWS_MAX 8
#define ROWS_COLS 16             // output columns per CTA, 2 per warp (64: 0.646 ms a decode step of four layers, two of them routed, 16 experts of 1024 x 2048; 32: 0.545; 16: 0.493; 8: 0.488)

__device__ __forceinline__ float moe_rows_sum8(const float* acc, int lane) {
    float a4[4], a2[2];
    bool hi = (lane & 16) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float send = hi ? acc[i] : acc[i + 4], keep = hi ? acc[i + 4] : acc[i];
        a4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
    hi = (lane & 8) != 0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float send = hi ? a4[i] : a4[i + 2], keep = hi ? a4[i + 2] : a4[i];
        a2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    hi = (lane & 4) != 0;
    const float send = hi ? a2[0] : a2[1], keep = hi ? a2[1] : a2[0];
    float a1 = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
    a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
    return a1;
}

template <bool GATED, typename TO>
__global__ void __launch_bounds__(256)
moe_rows_kernel(const bf16* __restrict__ A, long long lda, const bf16* __restrict__ W, long long w_expert_stride,
                TO* __restrict__ C, long long ldc, const int* __restrict__ perm, int top, const int3* __restrict__ tiles,
                int max_tiles, int N, int K, int act, float limit, float alpha, float shift,
                const float* __restrict__ pair_scale) {
    extern __shared__ __align__(16) bf16 a_s[];            // [ROWS_MAX][K]
    ap_pdl_trigger();
    ap_pdl_wait();
    if ((int)blockIdx.y >= tiles[max_tiles].x) return;
    const int3 tile = tiles[blockIdx.y];
    const int e = tile.x, p0 = tile.y, rows = tile.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bf16* We = W + (size_t)e * w_expert_stride;
    const int K8 = K / 8;
    for (int r0 = 0; r0 < rows; r0 += ROWS_MAX) {
        const int R = min(ROWS_MAX, rows - r0);
        __syncthreads();
        for (int i = threadIdx.x; i < ROWS_MAX * K8; i += 256) {
            const int r = i / K8, c = i - r * K8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < R) {
                const int src = GATED ? perm[p0 + r0 + r] / top : p0 + r0 + r;
                v = *reinterpret_cast<const uint4*>(A + (size_t)src * lda + c * 8);
            }
            *reinterpret_cast<uint4*>(a_s + (size_t)r * K + c * 8) = v;
        }
        __syncthreads();
        for (int cc = 0; cc < ROWS_COLS / 8; ++cc) {
            const int n = blockIdx.x * ROWS_COLS + warp * (ROWS_COLS / 8) + cc;
            if (n >= N) break;
            float acc[ROWS_MAX], acc2[GATED ? ROWS_MAX : 1];
#pragma unroll
            for (int r = 0; r < ROWS_MAX; ++r) {
                acc[r] = 0.f;
                if constexpr (GATED) acc2[r] = 0.f;
            }
            const bf16* w1 = We + (size_t)n * K;
            const bf16* w2 = We + (size_t)(N + n) * K;
#pragma unroll 4
            for (int k = lane * 8; k < K; k += 256) {
                const uint4 wv = *reinterpret_cast<const uint4*>(w1 + k);
                uint4 wv2 = make_uint4(0, 0, 0, 0);
                if constexpr (GATED) wv2 = *reinterpret_cast<const uint4*>(w2 + k);
                const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
                const __nv_bfloat162* wp2 = reinterpret_cast<const __nv_bfloat162*>(&wv2);
                float wf[8], wf2[8];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 t = __bfloat1622float2(wp[q]);
                    wf[2 * q] = t.x; wf[2 * q + 1] = t.y;
                    if constexpr (GATED) {
                        const float2 u = __bfloat1622float2(wp2[q]);
                        wf2[2 * q] = u.x; wf2[2 * q + 1] = u.y;
                    }
                }
#pragma unroll
                for (int r = 0; r < ROWS_MAX; ++r) {
                    const uint4 av = *reinterpret_cast<const uint4*>(a_s + (size_t)r * K + k);
                    const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float2 t = __bfloat1622float2(ap[q]);
                        acc[r] = fmaf(t.y, wf[2 * q + 1], fmaf(t.x, wf[2 * q], acc[r]));
                        if constexpr (GATED) acc2[r] = fmaf(t.y, wf2[2 * q + 1], fmaf(t.x, wf2[2 * q], acc2[r]));
                    }
                }
            }
            // the eight rows' sums over the lanes in nine exchanges instead of forty: a lane hands half of its
            // values to its partner and keeps the other half, three times, then two plain steps; every row's
            // sum is formed by the same tree as a butterfly over all lanes, and ends in the lanes whose bits 4, 3, 2
            // spell the row
            const int out_row = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
            float v = moe_rows_sum8(acc, lane), v2 = 0.f;
            if constexpr (GATED) v2 = moe_rows_sum8(acc2, lane);
            if ((lane & 3) == 0 && out_row < R) {
                if constexpr (GATED) {
                    const float sc = pair_scale ? pair_scale[perm[p0 + r0 + out_row]] : 1.0f;
                    v = gated_activation(v * sc, v2 * sc, act, limit, alpha, shift);
                }
                C[(size_t)(p0 + r0 + out_row) * ldc + n] = ap_from_float<TO>(v);
            }
        }
    }
}

// whether a step of `pairs` (row, choice) pairs in bfloat16 is one for the kernel above
static bool moe_few_rows(int pairs, int E, int K, const void* a, const void* w) {
    return pairs <= 16 * E && K % 8 == 0 && (size_t)ROWS_MAX * K * 2 <= 160 * 1024 &&
           ((((uintptr_t)a) | ((uintptr_t)w)) & 15) == 0;
}

// a: [T, K]; w_gate_up: [E, 2 F, K]; y: [pairs, F] in the activation type
AP_EXPORT int ap_moe_gate_up(const void* a, int a_dtype, const void* w, int w_dtype, void* y, int y_dtype,
                             const int* perm, int top, const int* tiles, int pairs, int E, int F, int K, int act,
                             float limit, float alpha, float shift, const float* pair_scale, cudaStream_t stream) {
    AP_REQUIRE(pairs >= 0 && E > 0 && F > 0 && K > 0 && top > 0 && act >= 0 && act <= 3, "moe_gate_up: bad sizes");
    if (pairs == 0) return AP_OK;
    const int max_tiles = ap_moe_max_tiles(pairs, E);
    const dim3 grid((unsigned)((F + MOE_BN - 1) / MOE_BN), (unsigned)max_tiles);
    AP_REQUIRE(max_tiles <= 65535, "moe_gate_up: %d row tiles exceed the grid", max_tiles);
#define LAUNCH(TA, TW, TO)                                                                                           \
    AP_CHECK_PDL_LAUNCH("moe_gate_up", ap_launch_pdl(moe_gemm_kernel<TA, TW, TO, true>, grid, dim3(256), 0, stream,  \
                                                     (const TA*)a, (long long)K, (const TW*)w, (long long)2 * F * K, \
                                                     (TO*)y, (long long)F, perm, top, (const int3*)tiles, max_tiles, F, K, \
                                                     act, limit, alpha, shift, pair_scale))
    if (a_dtype == AP_BF16 && w_dtype == AP_BF16 && y_dtype == AP_BF16 && moe_few_rows(pairs, E, K, a, w)) {
        const dim3 rgrid((unsigned)((F + ROWS_COLS - 1) / ROWS_COLS), (unsigned)max_tiles);
        const size_t smem = (size_t)ROWS_MAX * K * sizeof(bf16);
        auto kern = moe_rows_kernel<true, bf16>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            AP_REQUIRE(e == cudaSuccess, "moe_gate_up: cannot reserve %zu bytes of shared memory", smem);
        }
        AP_CHECK_PDL_LAUNCH("moe_gate_up", ap_launch_pdl(kern, rgrid, dim3(256), smem, stream, (const bf16*)a, (long long)K,
                                                         (const bf16*)w, (long long)2 * F * K, (bf16*)y, (long long)F, perm,
                                                         top, (const int3*)tiles, max_tiles, F, K, act, limit, alpha, shift, pair_scale));
        return AP_OK;
    }
    if (a_dtype == AP_F32 && w_dtype == AP_F32 && y_dtype == AP_F32) LAUNCH(float, float, float);
    else if (a_dtype == AP_BF16 && w_dtype == AP_BF16 && y_dtype == AP_BF16) LAUNCH(bf16, bf16, bf16);
    else if (a_dtype == AP_BF16 && w_dtype == AP_F32 && y_dtype == AP_BF16) LAUNCH(bf16, float, bf16);
    else AP_REQUIRE(false, "moe_gate_up: unsupported dtypes a=%d w=%d y=%d", a_dtype, w_dtype, y_dtype);
#undef LAUNCH
    return AP_OK;
}

// y: [pairs, F]; w_down: [E, H, F]; o: [pairs, H] 32-bit
AP_EXPORT int ap_moe_down(const void* y, int y_dtype, const void* w, int w_dtype, float* o, const int* tiles, int pairs,
                          int E, int H, int F, cudaStream_t stream) {
    AP_REQUIRE(pairs >= 0 && E > 0 && F > 0 && H > 0, "moe_down: bad sizes");
    if (pairs == 0) return AP_OK;
    const int max_tiles = ap_moe_max_tiles(pairs, E);
    const dim3 grid((unsigned)((H + MOE_BN - 1) / MOE_BN), (unsigned)max_tiles);
    AP_REQUIRE(max_tiles <= 65535, "moe_down: %d row tiles exceed the grid", max_tiles);
#define LAUNCH(TA, TW)                                                                                               \
    AP_CHECK_PDL_LAUNCH("moe_down", ap_launch_pdl(moe_gemm_kernel<TA, TW, float, false>, grid, dim3(256), 0, stream, \
                                                  (const TA*)y, (long long)F, (const TW*)w, (long long)H * F, o,     \
                                                  (long long)H, (const int*)nullptr, 1, (const int3*)tiles, max_tiles, H, \
                                                  F, 0, 0.f, 0.f, 0.f, (const float*)nullptr))
    if (y_dtype == AP_BF16 && w_dtype == AP_BF16 && moe_few_rows(pairs, E, F, y, w)) {
        const dim3 rgrid((unsigned)((H + ROWS_COLS - 1) / ROWS_COLS), (unsigned)max_tiles);
        const size_t smem = (size_t)ROWS_MAX * F * sizeof(bf16);
        auto kern = moe_rows_kernel<false, float>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            AP_REQUIRE(e == cudaSuccess, "moe_down: cannot reserve %zu bytes of shared memory", smem);
        }
        AP_CHECK_PDL_LAUNCH("moe_down", ap_launch_pdl(kern, rgrid, dim3(256), smem, stream, (const bf16*)y, (long long)F,
                                                      (const bf16*)w, (long long)H * F, o, (long long)H,
                                                      (const int*)nullptr, 1, (const int3*)tiles, max_tiles, H, F, 0, 0.f,
                                                      0.f, 0.f, (const float*)nullptr));
        return AP_OK;
    }
    if (y_dtype == AP_F32 && w_dtype == AP_F32) LAUNCH(float, float);
    else if (y_dtype == AP_BF16 && w_dtype == AP_BF16) LAUNCH(bf16, bf16);
    else if (y_dtype == AP_BF16 && w_dtype == AP_F32) LAUNCH(bf16, float);
    else AP_REQUIRE(false, "moe_down: unsupported dtypes y=%d w=%d", y_dtype, w_dtype);
#undef LAUNCH
    return AP_OK;
}

// rows of `a` in grouped order: out[p, :] = a[perm[p] / top, :]   (16-bit elements, K a multiple of 8)
__global__ void moe_gather_kernel(const uint4* __restrict__ a, uint4* __restrict__ out, const int* __restrict__ perm,
                                  int top, int pairs, int K8) {
    ap_pdl_trigger();
    ap_pdl_wait();
    const size_t n = (size_t)pairs * K8;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t p = e / K8, c = e - p * K8;
        out[e] = a[(size_t)(perm[p] / top) * K8 + c];
    }
}

AP_EXPORT int ap_moe_gather(const void* a, void* out, const int* perm, int top, int pairs, int K, cudaStream_t stream) {
    AP_REQUIRE(pairs >= 0 && top > 0 && K > 0 && K % 8 == 0, "moe_gather: rows of %d 16-bit elements are not whole 16-byte runs", K);
    AP_REQUIRE((((uintptr_t)a | (uintptr_t)out) & 15) == 0, "moe_gather: buffers must be 16-byte aligned");
    if (pairs == 0) return AP_OK;
    long long blocks = ((long long)pairs * (K / 8) + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    AP_CHECK_PDL_LAUNCH("moe_gather", ap_launch_pdl(moe_gather_kernel, dim3((unsigned)blocks), dim3(256), 0, stream,
                                                    (const uint4*)a, (uint4*)out, perm, top, pairs, K / 8));
    return AP_OK;
}

// delta[t, :] = sum_k weight[t, k] * o[place[t * top + k], :]; a choice of an expert from `real` on (an
// identity expert: no weights) contributes the row's input itself, rows[t, :], instead
template <typename TA>
__global__ void moe_combine_kernel(const float* __restrict__ o, const int* __restrict__ place,
                                   const float* __restrict__ weight, float* __restrict__ delta, int T, int H, int top,
                                   const int* __restrict__ chosen, int real, const TA* __restrict__ rows) {
    ap_pdl_trigger();
    ap_pdl_wait();
    const size_t n = (size_t)T * H;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / H, c = e - t * H;
        float v = 0.f;
        for (int k = 0; k < top; ++k) {
            const bool identity = chosen != nullptr && chosen[t * top + k] >= real;
            v = fmaf(weight ? weight[t * top + k] : 1.0f, identity ? ap_to_float(rows[e]) : o[(size_t)place[t * top + k] * H + c], v);
        }
        delta[e] = v;
    }
}

AP_EXPORT int ap_moe_combine(const float* o, const int* place, const float* weight, float* delta, int T, int H, int top,
                             const int* chosen, int real, const void* rows, int rows_dtype, cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && H > 0 && top > 0, "moe_combine: bad sizes");
    AP_REQUIRE(chosen == nullptr || rows != nullptr, "moe_combine: identity experts need the rows' input");
    if (T == 0) return AP_OK;
    long long blocks = ((long long)T * H + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (chosen != nullptr && rows_dtype == AP_BF16)
        AP_CHECK_PDL_LAUNCH("moe_combine", ap_launch_pdl(moe_combine_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0,
                                                         stream, o, place, weight, delta, T, H, top, chosen, real,
                                                         (const bf16*)rows));
    else
        AP_CHECK_PDL_LAUNCH("moe_combine", ap_launch_pdl(moe_combine_kernel<float>, dim3((unsigned)blocks), dim3(256), 0,
                                                         stream, o, place, weight, delta, T, H, top, chosen, real,
                                                         (const float*)rows));
    return AP_OK;
}
