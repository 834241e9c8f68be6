// Prompt portions on per-head keys and values that lie one token after another:
//
//   kv : [token][head][key (DK numbers) | value (DV numbers)]     (bfloat16; what the latent mixer's product
//                                                                   forms from the gathered records)
//   where[s, j] : the row of kv that holds token j of sequence s (a sequence's rows follow one another,
//                 so a tile's first row is looked up and the others are counted from it)
//
// Plain causal attention, out = softmax(q k^T * scale) v * sigmoid(gate), for the sequences that bring
// SEVERAL rows (the others are left alone); behind a sliding window (0: none) a row sees its last `window`
// keys, and with a sink (one number per head, or none) the denominator also holds exp(sink_h).  A CTA of four warps takes 64 consecutive rows of one
// sequence and one head; every warp holds its 16 query rows as A fragments in registers.  Key and
// value tiles of 64 tokens come by cp.async into two buffers, the next one loading while this one is
// used; K is the first product's B operand as it lies (ldmatrix), V the second's through
// ldmatrix.trans; scores leave the first product as 32-bit sums, the online softmax acts on them in
// registers, and the weights are rounded to bfloat16 only as the second product's A operand (their
// sum stays 32-bit).  The 32-bit path and other sizes run on the kernels of attention_window_bias.cu.
#include "common.cuh"
#include <float.h>

#define LP_Q 64
#define LP_K 64
#define LPF_THREADS 128

__device__ __forceinline__ void lp_cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void lp_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void lp_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void lp_ldsm_x4(uint32_t (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s) : "memory");
}
__device__ __forceinline__ void lp_ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s) : "memory");
}
__device__ __forceinline__ void lp_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lp_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// DKP, DVP: key and value sizes rounded up to a multiple of 16 the kernel is built for
template <int DKP, int DVP>
__global__ void __launch_bounds__(LPF_THREADS)
latent_prefill_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ kv,
                      const int* __restrict__ where, int width, const int* __restrict__ seq_start,
                      const int* __restrict__ positions, int nseq, int nh, int DK, int DV, float scale,
                      const float* __restrict__ gate, long long gate_ld, int window, const float* __restrict__ sink) {
    extern __shared__ __align__(16) unsigned char lp_smem[];
    constexpr int KP = DKP + 8, VP = DVP + 8;                // row pitches: 16 bytes more than a row
    bf16* k_s = reinterpret_cast<bf16*>(lp_smem);            // [2][64][KP]
    bf16* v_s = k_s + 2 * LP_K * KP;                         // [2][64][VP]
    ap_pdl_trigger();
    ap_pdl_wait();
    // which sequence and which of its row tiles: the longest-running tiles (the last rows) of a sequence first
    int b = blockIdx.x, seq = -1, row0 = 0, nrows = 0;
    for (int s = 0; s < nseq; ++s) {
        const int a = seq_start[s], n = seq_start[s + 1] - a;
        const int tiles = n == 1 ? 0 : (n + LP_Q - 1) / LP_Q;
        if (b < tiles) {
            const int t = tiles - 1 - b;
            seq = s;
            row0 = a + t * LP_Q;
            nrows = min(LP_Q, n - t * LP_Q);
            break;
        }
        b -= tiles;
    }
    if (seq < 0) return;
    const int h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int RS = DK + DV;
    const int pos_first = positions[row0], pos_last = pos_first + nrows - 1;
    // Behind a window only the tokens from `lo` on were gathered (what the sequence's first row of this step
    // still sees); token j >= lo lies j - lo rows behind token lo.  This tile's rows see keys from klo on.
    const int seq_first = positions[seq_start[seq]];
    const int lo = (window > 0 && seq_first - window + 1 > 0) ? seq_first - window + 1 : 0;
    const int klo = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    const size_t base = (size_t)where[(size_t)seq * width + lo];
    const bf16* kv_h = kv + (base * nh + h) * RS;
    const size_t tok = (size_t)nh * RS;
    // this warp's 16 query rows as A fragments (rows g and g + 8)
    uint32_t qa[DKP / 16][4];
    {
        const int ra = warp * 16 + g, rb = ra + 8;
        const bf16* qra = q + ((size_t)(row0 + ra) * nh + h) * DK;
        const bf16* qrb = q + ((size_t)(row0 + rb) * nh + h) * DK;
#pragma unroll
        for (int ks = 0; ks < DKP / 16; ++ks) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int c = ks * 16 + half * 8 + 2 * t4;   // DK is a multiple of 8: a pair lies inside or outside
                qa[ks][half * 2] = (ra < nrows && c < DK) ? *reinterpret_cast<const uint32_t*>(qra + c) : 0u;
                qa[ks][half * 2 + 1] = (rb < nrows && c < DK) ? *reinterpret_cast<const uint32_t*>(qrb + c) : 0u;
            }
        }
    }
    const uint4 zero = make_uint4(0, 0, 0, 0);
    constexpr int KC = DKP / 8, VC = DVP / 8;
    auto load_tile = [&](int tile, int stage) {
        bf16* kd = k_s + (size_t)stage * LP_K * KP;
        bf16* vd = v_s + (size_t)stage * LP_K * VP;
        const int k0 = tile * LP_K;
        for (int i = threadIdx.x; i < LP_K * KC; i += LPF_THREADS) {
            const int j = i / KC, c = (i - j * KC) * 8;
            if (k0 + j <= pos_last && k0 + j >= klo && c < DK) lp_cp_async16(kd + j * KP + c, kv_h + (size_t)(k0 + j - lo) * tok + c);
            else *reinterpret_cast<uint4*>(kd + j * KP + c) = zero;
        }
        for (int i = threadIdx.x; i < LP_K * VC; i += LPF_THREADS) {
            const int j = i / VC, c = (i - j * VC) * 8;
            if (k0 + j <= pos_last && k0 + j >= klo && c < DV) lp_cp_async16(vd + j * VP + c, kv_h + (size_t)(k0 + j - lo) * tok + DK + c);
            else *reinterpret_cast<uint4*>(vd + j * VP + c) = zero;
        }
        lp_cp_async_commit();
    };
    float o[DVP / 8][4];
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-FLT_MAX, -FLT_MAX}, l[2] = {0.f, 0.f};
    const int ntiles = pos_last / LP_K + 1, tile_lo = klo / LP_K;
    const int row_a = warp * 16 + g;
    const bool has_rows = warp * 16 < nrows;
    load_tile(tile_lo, 0);
    for (int tile = tile_lo; tile < ntiles; ++tile) {
        const int stage = (tile - tile_lo) & 1;
        if (tile + 1 < ntiles) {
            load_tile(tile + 1, stage ^ 1);
            lp_cp_async_wait<1>();
        } else {
            lp_cp_async_wait<0>();
        }
        __syncthreads();
        const int k0 = tile * LP_K;
        // a warp whose rows all lie before this tile's first key has nothing to do here (it helped loading)
        if (has_rows && k0 <= pos_first + min(warp * 16 + 15, nrows - 1)) {
            const bf16* kt = k_s + (size_t)stage * LP_K * KP;
            const bf16* vt = v_s + (size_t)stage * LP_K * VP;
            float sc[LP_K / 8][4];
#pragma unroll
            for (int nb = 0; nb < LP_K / 8; ++nb) sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < DKP / 16; ++ks) {
#pragma unroll
                for (int nb = 0; nb < LP_K / 8; nb += 2) {
                    uint32_t bq[4];                          // keys nb*8 .. +15, dimensions ks*16 .. +15
                    lp_ldsm_x4(bq, kt + (nb * 8 + (lane & 7) + ((lane >> 4) & 1) * 8) * KP + ks * 16 + ((lane >> 3) & 1) * 8);
                    lp_mma(sc[nb], qa[ks], bq[0], bq[1]);
                    lp_mma(sc[nb + 1], qa[ks], bq[2], bq[3]);
                }
            }
            float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
            for (int nb = 0; nb < LP_K / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = row_a + (e >> 1) * 8;
                    const int kp = k0 + nb * 8 + 2 * t4 + (e & 1);
                    const int dist = pos_first + r - kp;
                    const float v = (r < nrows && dist >= 0 && (window <= 0 || dist < window)) ? sc[nb][e] * scale : -FLT_MAX;
                    sc[nb][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            }
            float alpha[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float m_new = fmaxf(m[i], mx[i]);
                alpha[i] = __expf(m[i] - m_new);
                m[i] = m_new;
                l[i] *= alpha[i];
            }
#pragma unroll
            for (int nb = 0; nb < LP_K / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = sc[nb][e] > -FLT_MAX ? __expf(sc[nb][e] - m[e >> 1]) : 0.f;
                    sc[nb][e] = p;
                    l[e >> 1] += p;                          // this lane's share; the quad's shares meet at the end
                }
            }
#pragma unroll
            for (int i = 0; i < DVP / 8; ++i) {
                o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
            }
#pragma unroll
            for (int kb = 0; kb < LP_K / 16; ++kb) {
                uint32_t pa[4];
                pa[0] = lp_pack(sc[2 * kb][0], sc[2 * kb][1]);
                pa[1] = lp_pack(sc[2 * kb][2], sc[2 * kb][3]);
                pa[2] = lp_pack(sc[2 * kb + 1][0], sc[2 * kb + 1][1]);
                pa[3] = lp_pack(sc[2 * kb + 1][2], sc[2 * kb + 1][3]);
#pragma unroll
                for (int nb = 0; nb < DVP / 8; nb += 2) {
                    uint32_t bv[4];                          // tokens kb*16 .. +15, value columns nb*8 .. +15
                    lp_ldsm_x4_trans(bv, vt + (kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VP + nb * 8 + ((lane >> 4) & 1) * 8);
                    lp_mma(o[nb], pa, bv[0], bv[1]);
                    lp_mma(o[nb + 1], pa, bv[2], bv[3]);
                }
            }
        }
        __syncthreads();                                     // this buffer is loaded again in the next round
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = row_a + i * 8;
        if (r >= nrows) continue;
        // the sink: an extra logit in the normalisation, to which no value belongs
        float inv = 1.0f / (sink ? l[i] + expf(sink[h] - m[i]) : l[i]);
        if (gate) inv /= 1.0f + expf(-gate[(size_t)(row0 + r) * gate_ld + h]);
        bf16* dst = out + ((size_t)(row0 + r) * nh + h) * DV;
#pragma unroll
        for (int nb = 0; nb < DVP / 8; ++nb) {
            const int c = nb * 8 + 2 * t4;
            if (c < DV) *reinterpret_cast<uint32_t*>(dst + c) = lp_pack(o[nb][2 * i] * inv, o[nb][2 * i + 1] * inv);
        }
    }
}

// Whether the kernel takes these sizes (else the caller uses the kernels of attention_window_bias.cu).
AP_EXPORT int ap_latent_prefill_takes(int DK, int DV) {
    return DK > 0 && DV > 0 && DK % 8 == 0 && DV % 8 == 0 && DK <= 192 && DV <= 128;
}

template <int DKP, int DVP>
static int launch_latent_prefill(const void* q, void* out, const void* kv, const int* where, int width,
                                 const int* seq_start, const int* positions, int nseq, int T, int nh, int DK, int DV,
                                 float scale, const float* gate, long long gate_ld, int window, const float* sink,
                                 cudaStream_t stream) {
    const size_t smem = (size_t)2 * LP_K * ((DKP + 8) + (DVP + 8)) * sizeof(bf16);
    auto kern = latent_prefill_kernel<DKP, DVP>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        AP_REQUIRE(e == cudaSuccess, "latent_prefill: cannot reserve %zu bytes of shared memory", smem);
    }
    const dim3 grid((unsigned)(T / LP_Q + nseq), (unsigned)nh);
    AP_CHECK_PDL_LAUNCH("latent_prefill",
                        ap_launch_pdl(kern, grid, dim3(LPF_THREADS), smem, stream, (const bf16*)q, (bf16*)out,
                                      (const bf16*)kv, where, width, seq_start, positions, nseq, nh, DK, DV, scale, gate,
                                      gate_ld, window, sink));
    return AP_OK;
}

AP_EXPORT int ap_latent_prefill(const void* q, void* out, const void* kv, const int* where, int width,
                                const int* seq_start, const int* positions, int nseq, int T, int nh, int DK, int DV,
                                float scale, const float* gate, long long gate_ld, int window, const float* sink,
                                cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && nseq >= 0 && nh > 0 && nh <= 65535 && width > 0, "latent_prefill: bad sizes T=%d heads=%d", T, nh);
    AP_REQUIRE(ap_latent_prefill_takes(DK, DV), "latent_prefill: head sizes %d/%d are not ones the kernel takes", DK, DV);
    AP_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)kv & 15) == 0 && ((uintptr_t)out & 3) == 0,
               "latent_prefill: operands must be 16-byte aligned");
    AP_REQUIRE(gate == nullptr || gate_ld >= nh, "latent_prefill: bad gate stride");
    if (T == 0 || nseq == 0) return AP_OK;
#define LP_ARGS q, out, kv, where, width, seq_start, positions, nseq, T, nh, DK, DV, scale, gate, gate_ld, window, sink, stream
    const int dk = DK <= 64 ? 64 : (DK <= 128 ? 128 : 192), dv = DV <= 64 ? 64 : 128;
    switch (dk * 1000 + dv) {
        case 64064: return launch_latent_prefill<64, 64>(LP_ARGS);
        case 64128: return launch_latent_prefill<64, 128>(LP_ARGS);
        case 128064: return launch_latent_prefill<128, 64>(LP_ARGS);
        case 128128: return launch_latent_prefill<128, 128>(LP_ARGS);
        case 192064: return launch_latent_prefill<192, 64>(LP_ARGS);
        default: return launch_latent_prefill<192, 128>(LP_ARGS);
    }
#undef LP_ARGS
}
