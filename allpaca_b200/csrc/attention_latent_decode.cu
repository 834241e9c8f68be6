// Decoding through a latent that all heads share: sequences that bring ONE row, bfloat16.
//
// A token's record [c | k_rot] (D numbers) is the key of every head, and its first R numbers are
// every head's value (attention_latent.cu says why).  So the H query rows of a sequence meet the
// same keys: a CTA takes 16 heads of one sequence and a slice of its keys, and every key tile that
// reaches shared memory serves all 16 rows on the tensor cores (mma.sync m16n8k16, 32-bit sums):
//
//   S [16 heads x 64 keys] = Q [16 x D] K^T      warp w of eight: keys 8w .. 8w+7 of the tile
//   online softmax over the tile                  row maxima of the eight warps meet in shared memory
//   O [16 x R] += P [16 x 64] V [64 x R]          warp w: its eighth of the R columns; V is the same
//                                                 tile, read transposed (ldmatrix.trans)
//
// Key tiles come by cp.async.  With one tile buffer (LD_STAGES 1, the default) two CTAs share an SM and
// one computes while the other loads; with two buffers a CTA loads its next tile while it uses this
// one and has the SM alone (measured: 74 against 110 us for 64 sequences of 2048 keys, 32 against 34
// for 8 of 4096, 39 against 34 for one of 8192).  The slices of a sequence's keys leave unnormalised sums with their maximum and weight sum; a second
// kernel merges them, applies the output gate and rounds.  Scores, softmax and sums are 32-bit.
// Behind a sliding window (0: none) a row sees its last `window` keys only; with a sink (one number
// per head, or none) the merged denominator also holds exp(sink_h).
#include "common.cuh"
#include <float.h>

#define LD_WARPS 8
#define LD_THREADS (LD_WARPS * 32)
#define LD_KT 64              // keys per tile: eight to a warp
#define LD_M 16               // heads per CTA
#define LD_PP 72              // row pitch of the probabilities in shared memory (64 + 8)
#ifndef LD_STAGES
#define LD_STAGES 1           // key tile buffers per CTA: with one, two CTAs share an SM and overlap each other's loads
#endif

__device__ __forceinline__ void ld_cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void ld_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void ld_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ld_ldsm_x4(uint32_t (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s) : "memory");
}
__device__ __forceinline__ void ld_ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s) : "memory");
}
__device__ __forceinline__ void ld_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ld_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// NBW: blocks of 8 value columns per warp (R <= 64 NBW)
template <int NBW>
__global__ void __launch_bounds__(LD_THREADS)
latent_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache, const int* __restrict__ block_table,
                     int max_blocks, const int* __restrict__ seq_start, const int* __restrict__ positions, int nh, int D,
                     int R, int P, size_t page_stride, float scale, int window, int nsplit, float* __restrict__ part_o,
                     float* __restrict__ part_ml) {
    extern __shared__ __align__(16) unsigned char ld_smem[];
    const int seq = blockIdx.x, h0 = blockIdx.y * LD_M, split = blockIdx.z;
    ap_pdl_trigger();
    ap_pdl_wait();
    const int row = seq_start[seq];
    if (seq_start[seq + 1] - row != 1) return;
    const int qpos = positions[row];
    const int D16 = (D + 15) & ~15;
    const int pitch = D16 + 8;                               // 16 bytes more than a row: ldmatrix meets no bank twice
    bf16* q_s = reinterpret_cast<bf16*>(ld_smem);            // [16][pitch]
    bf16* k_s = q_s + LD_M * pitch;                          // [LD_STAGES][64][pitch]
    bf16* p_s = k_s + LD_STAGES * LD_KT * pitch;             // [16][LD_PP]
    float* red = reinterpret_cast<float*>(p_s + LD_M * LD_PP);   // [LD_WARPS][16]
    const int* table = block_table + (size_t)seq * max_blocks;
    // behind a window the row sees keys klo .. qpos: tiles before the one that holds klo are never touched
    // (their pages may have gone back to the pool)
    const int klo = (window > 0 && qpos - window + 1 > 0) ? qpos - window + 1 : 0;
    const int tile_lo = klo / LD_KT, tiles = qpos / LD_KT + 1;
    const int per = (tiles - tile_lo + nsplit - 1) / nsplit;
    const int t0 = tile_lo + split * per, t1 = min(tiles, t0 + per);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int chunks = D16 / 8, dchunks = D / 8;             // 16-byte runs of a padded row, and of a record
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int r = warp; r < LD_M; r += LD_WARPS) {
        const bf16* src = q + ((size_t)row * nh + h0 + r) * D;
        for (int c = lane; c < chunks; c += 32)
            *reinterpret_cast<uint4*>(q_s + r * pitch + c * 8) =
                (h0 + r < nh && c < dchunks) ? *reinterpret_cast<const uint4*>(src + c * 8) : zero;
    }
    // a warp brings eight keys of a tile: the page and slot of a key are found once, the lanes share its record
    auto load_tile = [&](int tile, int stage) {
        bf16* dst = k_s + (size_t)stage * LD_KT * pitch;
#pragma unroll 2
        for (int jj = 0; jj < LD_KT / LD_WARPS; ++jj) {
            const int j = jj * LD_WARPS + warp;
            const int kp = tile * LD_KT + j;
            bf16* d = dst + j * pitch;
            if (kp <= qpos && kp >= klo) {
                const bf16* src = cache + (size_t)table[kp / P] * page_stride + (size_t)(kp % P) * D;
                for (int c = lane; c < chunks; c += 32) {
                    if (c < dchunks) ld_cp_async16(d + c * 8, src + c * 8);
                    else *reinterpret_cast<uint4*>(d + c * 8) = zero;
                }
            } else {
                // keys behind the row or before its window: finite, weight zero
                for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(d + c * 8) = zero;
            }
        }
        ld_cp_async_commit();
    };
    float o[NBW][4];
#pragma unroll
    for (int i = 0; i < NBW; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-FLT_MAX, -FLT_MAX}, l[2] = {0.f, 0.f};
    if (LD_STAGES == 2 && t0 < t1) load_tile(t0, 0);
    for (int tile = t0; tile < t1; ++tile) {
        const int stage = LD_STAGES == 2 ? (tile - t0) & 1 : 0;
        if (LD_STAGES == 2 && tile + 1 < t1) {
            load_tile(tile + 1, stage ^ 1);
            ld_cp_async_wait<1>();
        } else {
            if (LD_STAGES == 1) load_tile(tile, 0);
            ld_cp_async_wait<0>();
        }
        __syncthreads();                                     // the tile (and, the first time, the queries) are there
        const bf16* kt = k_s + (size_t)stage * LD_KT * pitch;
        // S for keys 8 warp .. 8 warp + 7: two sums that take the blocks of 16 dimensions in turn
        float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
        const bf16* qa = q_s + (lane & 15) * pitch + (lane >> 4) * 8;
        const bf16* kb = kt + (8 * warp + (lane & 7)) * pitch + (lane >> 3) * 8;
        int ks = 0;
        for (; ks + 1 < D16 / 16; ks += 2) {
            uint32_t a[4], a2[4], b[4];
            ld_ldsm_x4(b, kb + ks * 16);                     // this key block, dimensions 0-7, 8-15, 16-23, 24-31 of the pair
            ld_ldsm_x4(a, qa + ks * 16);
            ld_ldsm_x4(a2, qa + ks * 16 + 16);
            ld_mma(s, a, b[0], b[1]);
            ld_mma(s2, a2, b[2], b[3]);
        }
        if (ks < D16 / 16) {                                 // an odd block left: the row's padding is read and not used
            uint32_t a[4], b[4];
            ld_ldsm_x4(b, kb + ks * 16 - 16);
            ld_ldsm_x4(a, qa + ks * 16);
            ld_mma(s, a, b[2], b[3]);
        }
        float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int kp = tile * LD_KT + 8 * warp + 2 * t4 + (e & 1);
            const float v = (kp <= qpos && kp >= klo) ? (s[e] + s2[e]) * scale : -FLT_MAX;
            s[e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        }
        if (t4 == 0) {
            red[warp * LD_M + g] = mx[0];
            red[warp * LD_M + g + 8] = mx[1];
        }
        __syncthreads();
        float alpha[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = g + 8 * i;
            float mm = red[r];
#pragma unroll
            for (int w = 1; w < LD_WARPS; ++w) mm = fmaxf(mm, red[w * LD_M + r]);
            const float m_new = fmaxf(m[i], mm);
            alpha[i] = __expf(m[i] - m_new);
            m[i] = m_new;
            l[i] *= alpha[i];
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            // the weight is rounded to bfloat16 for the second product: the fast exponential's error is far below that
            const float p = s[e] > -FLT_MAX ? __expf(s[e] - m[e >> 1]) : 0.f;
            s[e] = p;
            l[e >> 1] += p;
        }
        *reinterpret_cast<uint32_t*>(p_s + g * LD_PP + 8 * warp + 2 * t4) = ld_pack(s[0], s[1]);
        *reinterpret_cast<uint32_t*>(p_s + (g + 8) * LD_PP + 8 * warp + 2 * t4) = ld_pack(s[2], s[3]);
#pragma unroll
        for (int i = 0; i < NBW; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
        __syncthreads();                                     // the probabilities of all 64 keys are written
#pragma unroll
        for (int kk = 0; kk < LD_KT / 16; ++kk) {
            uint32_t a[4];
            ld_ldsm_x4(a, p_s + (lane & 15) * LD_PP + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nb = 0; nb < NBW; nb += 2) {
                const int n0 = warp * 8 * NBW + nb * 8;
                if (n0 < R) {                                // the same for the whole warp
                    uint32_t b[4];
                    ld_ldsm_x4_trans(b, kt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * pitch + n0 + ((lane >> 4) & 1) * 8);
                    ld_mma(o[nb], a, b[0], b[1]);
                    ld_mma(o[nb + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                     // this buffer is loaded again in the next round
    }
    // the weight sums: over the quad, then over the warps (every warp has the same maxima)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    if (t4 == 0) {
        red[warp * LD_M + g] = l[0];
        red[warp * LD_M + g + 8] = l[1];
    }
    __syncthreads();
    const size_t slot = ((size_t)seq * nsplit + split) * nh;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = g + 8 * i, h = h0 + r;
        if (h >= nh) continue;
        float* dst = part_o + (slot + h) * R;
#pragma unroll
        for (int nb = 0; nb < NBW; ++nb) {
            const int c = warp * 8 * NBW + nb * 8 + 2 * t4;
            if (c < R) dst[c] = o[nb][2 * i];
            if (c + 1 < R) dst[c + 1] = o[nb][2 * i + 1];
        }
        if (warp == 0 && t4 == 0) {
            float sum = red[r];
#pragma unroll
            for (int w = 1; w < LD_WARPS; ++w) sum += red[w * LD_M + r];
            part_ml[(slot + h) * 2] = m[i];
            part_ml[(slot + h) * 2 + 1] = sum;
        }
    }
}

// one CTA per (sequence, head): the slices' sums weighed by exp(maximum - overall maximum), in slice order;
// the weights are formed once, and a thread's loads of its column are independent of one another
#define LD_MAX_SPLITS 64
__global__ void __launch_bounds__(128)
latent_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                           bf16* __restrict__ out, const int* __restrict__ seq_start, int nh, int R,
                           int nsplit, const float* __restrict__ gate, long long gate_ld,
                           const float* __restrict__ sink) {
    __shared__ float w_s[LD_MAX_SPLITS];
    __shared__ float f_s;
    const int seq = blockIdx.x, h = blockIdx.y;
    ap_pdl_trigger();
    ap_pdl_wait();
    const int row = seq_start[seq];
    if (seq_start[seq + 1] - row != 1) return;
    const size_t slot0 = (size_t)seq * nsplit * nh + h;      // slice s: slot0 + s * nh
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float m0 = -FLT_MAX, m1 = -FLT_MAX, l0 = 0.f, l1 = 0.f;
        if (lane < nsplit) {
            m0 = part_ml[(slot0 + (size_t)lane * nh) * 2];
            l0 = part_ml[(slot0 + (size_t)lane * nh) * 2 + 1];
        }
        if (lane + 32 < nsplit) {
            m1 = part_ml[(slot0 + (size_t)(lane + 32) * nh) * 2];
            l1 = part_ml[(slot0 + (size_t)(lane + 32) * nh) * 2 + 1];
        }
        const float mm = ap_warp_max(fmaxf(m0, m1));
        const float w0 = lane < nsplit ? expf(m0 - mm) : 0.f, w1 = lane + 32 < nsplit ? expf(m1 - mm) : 0.f;
        w_s[lane] = w0;
        w_s[lane + 32] = w1;
        const float den = ap_warp_sum(fmaf(l0, w0, l1 * w1));
        if (lane == 0) {
            // the sink: an extra logit in the normalisation, to which no value belongs
            float f = 1.0f / (sink ? den + expf(sink[h] - mm) : den);
            if (gate) f /= 1.0f + expf(-gate[(size_t)row * gate_ld + h]);
            f_s = f;
        }
    }
    __syncthreads();
    const float f = f_s;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        const float* src = part_o + slot0 * R + c;
        float num = 0.f;
#pragma unroll 8
        for (int s = 0; s < nsplit; ++s) num = fmaf(src[(size_t)s * nh * R], w_s[s], num);
        out[((size_t)row * nh + h) * R + c] = __float2bfloat16_rn(num * f);
    }
}

// Key slices per sequence: enough CTAs for the GPU (one CTA fills an SM's shared memory), no slice
// shorter than two tiles of the longest context the step may hold.
AP_EXPORT int ap_latent_decode_splits(int nseq, int nh, int max_context) {
    const int groups = (nh + LD_M - 1) / LD_M;
    const int tiles = (max_context > 0 ? max_context : 1) / LD_KT + 1;
    const int slots = 148 * (LD_STAGES == 1 ? 2 : 1);          // CTAs the GPU holds at once
    int want = (slots + nseq * groups - 1) / (nseq * groups > 0 ? nseq * groups : 1);
    const int most = tiles / 2 > 0 ? tiles / 2 : 1;
    if (want > most) want = most;
    if (want > 32) want = 32;                                // the merge adds them up one after another
    return want < 1 ? 1 : want;
}

// Whether the kernel takes these sizes (else the caller uses the general kernels).
AP_EXPORT int ap_latent_decode_takes(int D, int R) {
    const int D16 = (D + 15) & ~15;
    const size_t smem = (size_t)(LD_M + LD_STAGES * LD_KT) * (D16 + 8) * 2 + LD_M * LD_PP * 2 + LD_WARPS * LD_M * 4;
    return D > 0 && R > 0 && D % 8 == 0 && R % 8 == 0 && R <= D && R <= 512 && smem <= 220 * 1024;
}

AP_EXPORT int ap_latent_decode(const void* q, void* out, const void* cache, const int* block_table, int max_blocks,
                               const int* seq_start, const int* positions, int nseq, int nh, int D, int R, int P,
                               long long page_stride, float scale, const float* gate, long long gate_ld, int nsplit,
                               float* scratch, long long scratch_floats, int window, const float* sink,
                               cudaStream_t stream) {
    AP_REQUIRE(nseq >= 0 && nh > 0 && P > 0 && max_blocks > 0 && nsplit >= 1 && nsplit <= LD_MAX_SPLITS,
               "latent_decode: bad sizes (at most %d key slices)", LD_MAX_SPLITS);
    AP_REQUIRE(ap_latent_decode_takes(D, R), "latent_decode: a record of %d with a value of %d is not one the kernel takes", D, R);
    AP_REQUIRE(page_stride % 8 == 0 && ((uintptr_t)cache & 15) == 0 && ((uintptr_t)q & 15) == 0,
               "latent_decode: queries and pages must be 16-byte aligned");
    AP_REQUIRE(gate == nullptr || gate_ld >= nh, "latent_decode: bad gate stride");
    AP_REQUIRE(scratch_floats >= (long long)nseq * nsplit * nh * (R + 2), "latent_decode: the scratch is too small");
    if (nseq == 0) return AP_OK;
    const int groups = (nh + LD_M - 1) / LD_M;
    AP_REQUIRE(groups <= 65535 && nsplit <= 65535, "latent_decode: the grid is too large");
    const int D16 = (D + 15) & ~15;
    const size_t smem = (size_t)(LD_M + LD_STAGES * LD_KT) * (D16 + 8) * 2 + LD_M * LD_PP * 2 + LD_WARPS * LD_M * 4;
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)nseq * nsplit * nh * R;
    const dim3 grid((unsigned)nseq, (unsigned)groups, (unsigned)nsplit);
#define LAUNCH(NBW)                                                                                                    \
    do {                                                                                                               \
        auto kern = latent_decode_kernel<NBW>;                                                                         \
        if (smem > 48 * 1024) {                                                                                        \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
            AP_REQUIRE(e == cudaSuccess, "latent_decode: cannot reserve %zu bytes of shared memory", smem);            \
        }                                                                                                              \
        AP_CHECK_PDL_LAUNCH("latent_decode",                                                                           \
                            ap_launch_pdl(kern, grid, dim3(LD_THREADS), smem, stream, (const bf16*)q, (const bf16*)cache, \
                                          block_table, max_blocks, seq_start, positions, nh, D, R, P, (size_t)page_stride, \
                                          scale, window, nsplit, part_o, part_ml));                                    \
    } while (0)
    if (R <= 128) LAUNCH(2);
    else if (R <= 256) LAUNCH(4);
    else LAUNCH(8);
#undef LAUNCH
    AP_CHECK_PDL_LAUNCH("latent_decode_merge",
                        ap_launch_pdl(latent_decode_merge_kernel, dim3((unsigned)nseq, (unsigned)nh), dim3(128), 0, stream,
                                      (const float*)part_o, (const float*)part_ml, (bf16*)out, seq_start, nh, R, nsplit,
                                      gate, gate_ld, sink));
    return AP_OK;
}
