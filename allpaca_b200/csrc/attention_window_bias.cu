// Grouped-query attention whose scores carry a bias that depends on the distance between
// query and key, over a paged cache in which a token keeps its key and its value side by
// side (so keys and values may differ in size), behind an optional sliding window:
//
//   score(i, j) = (q_i . k_j) * scale - bias_h(i - j)       for 0 <= i - j < window, or j < keep_first
//   out_i       = softmax_j(score(i, .)) . v * sigmoid(gate[i, h])
//
// With a sink (one 32-bit number per head, or none) the softmax's denominator also holds exp(sink_h):
// an extra logit per head that enters the normalisation only (`scale` does not touch it, no value goes with it).
//
// bias_h(d) is r1[h] * ln(1 + r2[h] * d) (BIAS_LOG), r1[h] * d (BIAS_LINEAR) or nothing; the first
// keep_first tokens of a sequence stay visible behind the window, at their true distance; the gate
// (one 32-bit number per row and head, read from a strided matrix) may be absent.
//
// And the kernel that prepares its operands: every query and key head divided by its root
// mean square (with a weight per coordinate, or none), queries multiplied by
// 1 + coef * ln(floor((pos + 1) / every) + 1), keys and values written into the page and slot of
// their position.
//
//   q, out : [T, nh, D] and [T, nh, VD]
//   cache  : one run's pages, [page][nkv][P][RS]: a token's record of RS numbers holds its key at 0 and
//            its value at `voff` (side by side: RS = D + VD, voff = D; a value that is the head of the
//            key, as where queries and outputs live in a latent space all heads share: voff = 0)
//   block_table : [nseq, max_blocks] page ids; entries the window has passed are never read
//
// Scores, softmax, bias and the weighted sum are 32-bit whatever the storage type.  Head
// sizes are run-time values (any D, VD up to 256), so these kernels live in the core library.
// The step's rows are found through seq_start alone: a grid planned from the number of
// rows and sequences serves whatever lengths the sequences have.
#include "common.cuh"
#include <cooperative_groups.h>
#include <float.h>
namespace cg = cooperative_groups;

#define QKN_THREADS 128
#define MAX_HEAD 256              // head sizes the kernels take at full speed (8 value columns per lane)
#define WIDE_NC 20                // value columns per lane of the kernels built for wider values ...
#define MAX_WIDE_HEAD (32 * WIDE_NC)   // ... up to 640 (a latent of 512 with 64 rotated dimensions is 576 wide)
#define BIAS_NONE 0
#define BIAS_LOG 1
#define BIAS_LINEAR 2

__device__ __forceinline__ float awb_bias(int kind, float b1, float b2, float dist) {
    return kind == BIAS_LOG ? b1 * log1pf(b2 * dist) : (kind == BIAS_LINEAR ? b1 * dist : 0.f);
}
// the scaled score, bounded by a soft cap where there is one: cap * tanh(score / cap)
__device__ __forceinline__ float awb_cap(float score, float cap) { return cap > 0.f ? cap * tanhf(score / cap) : score; }
// Key tiles a row tile walks: the tiles that hold kept first tokens (0 .. tiles_kept-1), then the
// tiles from the window's first (tile_win) on; where the two meet or overlap, all tiles from 0.
__device__ __forceinline__ int awb_next_tile(int tile, int tiles_kept, int tile_win) {
    ++tile;
    return (tile == tiles_kept && tile < tile_win) ? tile_win : tile;
}

// one warp per (row, head) of the stacked projection [q heads | k heads | v heads]; `bias` (or null) has one
// number per column of the projection and is added as the sums are read; after the norm the first rot_dims
// coordinates of every query and key head are turned by the row's cosine/sine pairs (coordinate i with
// i + rot_dims/2); values are multiplied by value_scale on their way into the page
template <typename TI, typename TA>
__global__ void __launch_bounds__(QKN_THREADS)
qk_norm_store_kernel(const TI* __restrict__ in, long long ld_in, TA* __restrict__ q_out, TA* __restrict__ cache,
                     const int* __restrict__ positions, const int* __restrict__ token_seq,
                     const int* __restrict__ block_table, int max_blocks, int T, int nh, int nkv, int D, int VD, int P,
                     size_t page_stride, float eps, int normalise, float temp_coef, int temp_every,
                     const float* __restrict__ qw, const float* __restrict__ kw, const float* __restrict__ bias,
                     const float* __restrict__ cos_sin, int rot_dims, float value_scale) {
    __shared__ float turn_s[QKN_THREADS / 32][MAX_HEAD];
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (QKN_THREADS / 32) + (threadIdx.x >> 5);
    const int heads = nh + 2 * nkv;
    ap_pdl_trigger();
    ap_pdl_wait();
    if (unit >= (long long)T * heads) return;
    const int t = (int)(unit / heads), hh = (int)(unit % heads);
    const int pos = positions[t];
    const TI* row = in + (size_t)t * ld_in;
    if (hh < nh + nkv) {
        const bool is_q = hh < nh;
        const size_t col = is_q ? (size_t)hh * D : (size_t)nh * D + (size_t)(hh - nh) * D;
        const TI* src = row + col;
        float v[MAX_HEAD / 32];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_HEAD / 32; ++i) {
            const int d = lane + 32 * i;
            v[i] = d < D ? ap_to_float(src[d]) + (bias ? bias[col + d] : 0.f) : 0.f;
            ss = fmaf(v[i], v[i], ss);
        }
        ss = ap_warp_sum(ss);
        float f = normalise ? 1.0f / sqrtf(ss / (float)D + eps) : 1.0f;
        if (is_q && temp_every > 0) f *= 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f);
        const float* wv = is_q ? qw : kw;                    // a weight per coordinate, shared by the heads
        TA* dst;
        if (is_q) {
            dst = q_out + ((size_t)t * nh + hh) * D;
        } else {
            if (cache == nullptr) return;
            const int page = block_table[(size_t)token_seq[t] * max_blocks + pos / P];
            dst = cache + (size_t)page * page_stride + ((size_t)(hh - nh) * P + pos % P) * (D + VD);
        }
#pragma unroll
        for (int i = 0; i < MAX_HEAD / 32; ++i) {
            const int d = lane + 32 * i;
            v[i] = wv && d < D ? v[i] * f * wv[d] : v[i] * f;
        }
        if (rot_dims > 0) {
            float* mine = turn_s[threadIdx.x >> 5];
            const int half = rot_dims / 2;
#pragma unroll
            for (int i = 0; i < MAX_HEAD / 32; ++i) mine[lane + 32 * i] = v[i];
            __syncwarp();
#pragma unroll
            for (int i = 0; i < MAX_HEAD / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < rot_dims) {
                    const int j = d < half ? d : d - half;
                    const float2 cs = *reinterpret_cast<const float2*>(cos_sin + ((size_t)t * half + j) * 2);
                    v[i] = d < half ? v[i] * cs.x - mine[d + half] * cs.y : v[i] * cs.x + mine[d - half] * cs.y;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < MAX_HEAD / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < D) dst[d] = ap_from_float<TA>(v[i]);
        }
    } else {
        if (cache == nullptr) return;
        const int g = hh - nh - nkv;
        const size_t col = (size_t)(nh + nkv) * D + (size_t)g * VD;
        const TI* src = row + col;
        const int page = block_table[(size_t)token_seq[t] * max_blocks + pos / P];
        TA* dst = cache + (size_t)page * page_stride + ((size_t)g * P + pos % P) * (D + VD) + D;
        for (int d = lane; d < VD; d += 32)
            dst[d] = ap_from_float<TA>((ap_to_float(src[d]) + (bias ? bias[col + d] : 0.f)) * value_scale);
    }
}

AP_EXPORT int ap_qk_norm_store(const void* in, int in_dtype, long long ld_in, void* q_out, void* cache, int act_dtype,
                               const int* positions, const int* token_seq, const int* block_table, int max_blocks,
                               int T, int nh, int nkv, int D, int VD, int P, long long page_stride, float eps,
                               int normalise, float temp_coef, int temp_every, const float* qw, const float* kw,
                               const float* bias, const float* cos_sin, int rot_dims, float value_scale,
                               cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && nh > 0 && nkv > 0 && D > 0 && VD > 0 && D <= MAX_HEAD && VD <= MAX_HEAD,
               "qk_norm_store: bad sizes T=%d heads=%d/%d sizes %d/%d (at most %d)", T, nh, nkv, D, VD, MAX_HEAD);
    AP_REQUIRE(cache == nullptr || (token_seq && block_table && max_blocks > 0 && P > 0),
               "qk_norm_store: storing needs token_seq and a block table");
    AP_REQUIRE(temp_every >= 0, "qk_norm_store: the temperature's period must not be negative");
    AP_REQUIRE(rot_dims == 0 || (cos_sin && rot_dims > 0 && rot_dims % 2 == 0 && rot_dims <= D),
               "qk_norm_store: %d rotated coordinates of %d need an even number and a table", rot_dims, D);
    if (T == 0) return AP_OK;
    const long long units = (long long)T * (nh + 2 * nkv);
    const dim3 grid((unsigned)((units + QKN_THREADS / 32 - 1) / (QKN_THREADS / 32)));
#define LAUNCH(TI, TA)                                                                                              \
    AP_CHECK_PDL_LAUNCH("qk_norm_store",                                                                            \
                        ap_launch_pdl(qk_norm_store_kernel<TI, TA>, grid, dim3(QKN_THREADS), 0, stream, (const TI*)in, \
                                      ld_in, (TA*)q_out, (TA*)cache, positions, token_seq, block_table, max_blocks, T, \
                                      nh, nkv, D, VD, P, (size_t)page_stride, eps, normalise, temp_coef, temp_every, \
                                      qw, kw, bias, cos_sin, rot_dims, value_scale))
    if (in_dtype == AP_F32 && act_dtype == AP_F32) LAUNCH(float, float);
    else if (in_dtype == AP_F32 && act_dtype == AP_BF16) LAUNCH(float, bf16);
    else if (in_dtype == AP_BF16 && act_dtype == AP_BF16) LAUNCH(bf16, bf16);
    else AP_REQUIRE(false, "qk_norm_store: unsupported dtypes in=%d act=%d", in_dtype, act_dtype);
#undef LAUNCH
    return AP_OK;
}

// ---------------------------------------------------------------------------------------
// The attention itself.  A CTA of four warps takes up to QT consecutive rows of one
// sequence and one query head; keys come in tiles of KT (one key per lane), with their
// values, through shared memory; every warp owns up to RPW rows, runs their online softmax
// and holds their output in registers (lane c of VD / 32 columns).
// ---------------------------------------------------------------------------------------
#define AWB_THREADS 128
#define AWB_WARPS 4
#define RPW 4
#define QT (AWB_WARPS * RPW)
#define KT 32

template <typename TA, int NC>     // NC: value columns per lane the kernel is built for (VD <= 32 NC)
__global__ void __launch_bounds__(AWB_THREADS)
attention_window_bias_kernel(const TA* __restrict__ q, TA* __restrict__ out, const TA* __restrict__ cache,
                             const int* __restrict__ block_table, int max_blocks, const int* __restrict__ seq_start,
                             const int* __restrict__ positions, int nseq, int nh, int nkv, int D, int VD, int P,
                             size_t page_stride, float scale, float softcap, int window, const float* __restrict__ r1,
                             const float* __restrict__ r2, int skip_single, int RS, int voff, int bias_kind,
                             int keep_first, const float* __restrict__ gate, long long gate_ld,
                             const float* __restrict__ sink) {
    extern __shared__ __align__(16) float smem[];
    ap_pdl_trigger();
    ap_pdl_wait();
    // which sequence and which of its row tiles this CTA serves
    int b = blockIdx.x, seq = -1, row0 = 0, nrows = 0;
    for (int s = 0; s < nseq; ++s) {
        const int a = seq_start[s], n = seq_start[s + 1] - a;
        const int tiles = (skip_single && n == 1) ? 0 : (n + QT - 1) / QT;
        if (b < tiles) {
            seq = s;
            row0 = a + b * QT;
            nrows = min(QT, n - b * QT);
            break;
        }
        b -= tiles;
    }
    if (seq < 0) return;
    const int h = blockIdx.y, kvh = h / (nh / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int DP = D + 1;
    float* q_s = smem;                        // [QT][D]
    float* k_s = q_s + QT * D;                // [KT][D + 1]
    float* v_s = k_s + KT * DP;               // [KT][VD]
    float* p_s = v_s + KT * VD;               // [AWB_WARPS][RPW][KT]
    const int* table = block_table + (size_t)seq * max_blocks;
    const int pos_first = positions[row0], pos_last = pos_first + nrows - 1;
    for (int i = threadIdx.x; i < nrows * D; i += AWB_THREADS) {
        const int r = i / D, d = i - r * D;
        q_s[r * D + d] = ap_to_float(q[((size_t)(row0 + r) * nh + h) * D + d]);
    }
    const float b1 = r1 ? r1[h] : 0.f, b2 = r2 ? r2[h] : 0.f;
    const int klo = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    // keys 0 .. kfe-1 are kept first tokens that lie before the window of the tile's first row
    const int kfe = keep_first < klo ? keep_first : klo;
    const int tiles_kept = (kfe + KT - 1) / KT, tile_win = klo / KT;
    float acc[RPW][NC];
    float m[RPW], l[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        m[i] = -FLT_MAX;
        l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[i][c] = 0.f;
    }
    const int nc = (VD + 31) / 32;
    const int my_rows = min(RPW, nrows - warp * RPW);        // <= 0: this warp only helps loading
    // Key tiles start at multiples of KT whatever the rows of this CTA are: a row then meets its
    // keys in the same tiles and lanes however its prompt was cut, and gets the same bits.  Keys
    // between the kept first tokens and klo are not loaded (their pages may have gone back to the
    // pool); no row sees them.
    for (int tile = tiles_kept > 0 ? 0 : tile_win; tile * KT <= pos_last; tile = awb_next_tile(tile, tiles_kept, tile_win)) {
        const int k0 = tile * KT;
        __syncthreads();                                     // the tile before is consumed (and q_s is written)
        for (int j = warp; j < KT; j += AWB_WARPS) {
            const int kp = k0 + j;
            if ((kp >= klo || kp < kfe) && kp <= pos_last) {
                const int page = table[kp / P];
                const TA* src = cache + (size_t)page * page_stride + ((size_t)kvh * P + kp % P) * RS;
                for (int d = lane; d < D; d += 32) k_s[j * DP + d] = ap_to_float(src[d]);
                for (int d = lane; d < VD; d += 32) v_s[j * VD + d] = ap_to_float(src[voff + d]);
            } else {
                for (int d = lane; d < D; d += 32) k_s[j * DP + d] = 0.f;
                for (int d = lane; d < VD; d += 32) v_s[j * VD + d] = 0.f;
            }
        }
        __syncthreads();
        if (my_rows <= 0) continue;
        // scores of key `lane` for this warp's rows
        float s[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) s[i] = 0.f;
        const float* kr = k_s + lane * DP;
        const float* qr = q_s + (warp * RPW) * D;
        for (int d = 0; d < D; ++d) {
            const float kv = kr[d];
#pragma unroll
            for (int i = 0; i < RPW; ++i) s[i] = fmaf(qr[i * D + d], kv, s[i]);   // rows past the tile read finite junk
        }
        const int kp = k0 + lane;
        float* pw = p_s + warp * RPW * KT;
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int qpos = pos_first + warp * RPW + i;
            const int dist = qpos - kp;
            const bool seen = i < my_rows && dist >= 0 && (window <= 0 || dist < window || kp < keep_first);
            float sc = -FLT_MAX;
            if (seen) sc = awb_cap(s[i] * scale, softcap) - awb_bias(bias_kind, b1, b2, (float)dist);
            const float m_new = fmaxf(m[i], ap_warp_max(sc));
            const float p = seen ? expf(sc - m_new) : 0.f;
            const float alpha = expf(m[i] - m_new);
            l[i] = l[i] * alpha + ap_warp_sum(p);
            m[i] = m_new;
            pw[i * KT + lane] = p;
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[i][c] *= alpha;
        }
        __syncwarp();
        for (int j = 0; j < KT; ++j) {
            float pj[RPW];
#pragma unroll
            for (int i = 0; i < RPW; ++i) pj[i] = pw[i * KT + j];
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                if (c < nc) {
                    const int d = lane + 32 * c;
                    const float vv = d < VD ? v_s[j * VD + d] : 0.f;
#pragma unroll
                    for (int i = 0; i < RPW; ++i) acc[i][c] = fmaf(pj[i], vv, acc[i][c]);
                }
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        if (i < my_rows) {
            // the sink: an extra logit in the normalisation, to which no value belongs
            float inv = 1.0f / (sink ? l[i] + expf(sink[h] - m[i]) : l[i]);
            if (gate) inv /= 1.0f + expf(-gate[(size_t)(row0 + warp * RPW + i) * gate_ld + h]);
            TA* o = out + ((size_t)(row0 + warp * RPW + i) * nh + h) * VD;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int d = lane + 32 * c;
                if (d < VD) o[d] = ap_from_float<TA>(acc[i][c] * inv);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// bfloat16, sequences of several rows, head sizes up to 128: the same attention on the tensor
// cores (mma.sync m16n8k16, 32-bit accumulators).  A CTA of four warps takes 64 consecutive rows
// of one sequence and one query head, 16 rows to a warp, whose queries stay in registers as the
// first product's A operand; keys come 64 at a time through shared memory ([key][d], the B
// operand as it lies), values transposed ([d][key]) for the second product.  Scores leave the
// first product as 32-bit sums; scale, distance bias, window and the online softmax act on them
// in registers; the weights are rounded to bfloat16 only as the second product's A operand,
// their sum is kept in 32-bit.  DK, DV: the head sizes rounded up to a size the kernel is
// built for (operands are zero beyond the real sizes).
// ---------------------------------------------------------------------------------------
#define MQ 64
#define MK 64
#define MMA_BIAS_TABLE 2048      // distances the bias is tabulated for per CTA (beyond: computed in place)

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <int DK, int DV>
__global__ void __launch_bounds__(AWB_THREADS)
attention_window_bias_mma_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ cache,
                                 const int* __restrict__ block_table, int max_blocks, const int* __restrict__ seq_start,
                                 const int* __restrict__ positions, int nseq, int nh, int nkv, int D, int VD, int P,
                                 size_t page_stride, float scale, float softcap, int window, const float* __restrict__ r1,
                                 const float* __restrict__ r2, int skip_single, int RS, int voff, int bias_kind,
                                 int keep_first, const float* __restrict__ gate, long long gate_ld,
                                 const float* __restrict__ sink) {
    // the widest keys leave room for a shorter table (48 KB of static shared memory in all)
    constexpr int BIAS_TABLE = DK > 128 ? MMA_BIAS_TABLE / 2 : MMA_BIAS_TABLE;
    __shared__ __align__(16) bf16 k_s[MK][DK + 8];
    __shared__ __align__(16) bf16 vt_s[DV][MK + 8];
    __shared__ float bias_s[BIAS_TABLE];                   // r1 ln(1 + r2 d) for the distances this CTA meets
    ap_pdl_trigger();
    ap_pdl_wait();
    int b = blockIdx.x, seq = -1, row0 = 0, nrows = 0;
    for (int s = 0; s < nseq; ++s) {
        const int a = seq_start[s], n = seq_start[s + 1] - a;
        const int tiles = (skip_single && n == 1) ? 0 : (n + MQ - 1) / MQ;
        if (b < tiles) {
            seq = s;
            row0 = a + b * MQ;
            nrows = min(MQ, n - b * MQ);
            break;
        }
        b -= tiles;
    }
    if (seq < 0) return;
    const int h = blockIdx.y, kvh = h / (nh / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int* table = block_table + (size_t)seq * max_blocks;
    const int pos_first = positions[row0], pos_last = pos_first + nrows - 1;
    // this warp's queries as A fragments: rows g and g + 8 of its 16
    uint32_t qa[DK / 16][4];
    {
        const int ra = warp * 16 + g, rb = ra + 8;
        const bf16* qra = q + ((size_t)(row0 + ra) * nh + h) * D;
        const bf16* qrb = q + ((size_t)(row0 + rb) * nh + h) * D;
        const bf16 zero = __float2bfloat16_rn(0.f);
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int c = ks * 16 + half * 8 + 2 * t4;
                const bf16 a0 = (ra < nrows && c < D) ? qra[c] : zero, a1 = (ra < nrows && c + 1 < D) ? qra[c + 1] : zero;
                const bf16 b0 = (rb < nrows && c < D) ? qrb[c] : zero, b1 = (rb < nrows && c + 1 < D) ? qrb[c + 1] : zero;
                qa[ks][half * 2] = (uint32_t)__bfloat16_as_ushort(a0) | ((uint32_t)__bfloat16_as_ushort(a1) << 16);
                qa[ks][half * 2 + 1] = (uint32_t)__bfloat16_as_ushort(b0) | ((uint32_t)__bfloat16_as_ushort(b1) << 16);
            }
        }
    }
    const float b1h = r1 ? r1[h] : 0.f, b2h = r2 ? r2[h] : 0.f;
    const int klo = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    // the largest distance any row of this CTA has to a key it may see
    const int span = pos_last - klo + 1;
    const bool tabled = bias_kind == BIAS_LOG && span <= BIAS_TABLE;
    if (tabled)
        for (int d = threadIdx.x; d < span; d += AWB_THREADS) bias_s[d] = b1h * log1pf(b2h * (float)d);
    const int kfe = keep_first < klo ? keep_first : klo;       // kept first tokens before the first row's window
    const int tiles_kept = (kfe + MK - 1) / MK, tile_win = klo / MK;
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-FLT_MAX, -FLT_MAX}, l[2] = {0.f, 0.f};
    const bool vec = D % 8 == 0 && VD % 8 == 0 && RS % 8 == 0 && voff % 8 == 0 && page_stride % 8 == 0 &&
                     ((uintptr_t)cache & 15) == 0;
    const int row_a = warp * 16 + g;                        // this lane's rows: row_a and row_a + 8
    for (int tile = tiles_kept > 0 ? 0 : tile_win; tile * MK <= pos_last; tile = awb_next_tile(tile, tiles_kept, tile_win)) {
        const int k0 = tile * MK;
        __syncthreads();
        for (int idx = threadIdx.x; idx < MK * (DK / 8); idx += AWB_THREADS) {
            const int j = idx / (DK / 8), d0 = (idx - j * (DK / 8)) * 8;
            const int kp = k0 + j;
            uint4 val = make_uint4(0, 0, 0, 0);
            if ((kp >= klo || kp < kfe) && kp <= pos_last && d0 < D) {
                const bf16* src = cache + (size_t)table[kp / P] * page_stride + ((size_t)kvh * P + kp % P) * RS + d0;
                if (vec) {
                    val = *reinterpret_cast<const uint4*>(src);
                } else {
                    bf16* dst = reinterpret_cast<bf16*>(&val);
                    for (int e = 0; e < 8; ++e)
                        if (d0 + e < D) dst[e] = src[e];
                }
            }
            *reinterpret_cast<uint4*>(&k_s[j][d0]) = val;
        }
        for (int idx = threadIdx.x; idx < MK * (DV / 8); idx += AWB_THREADS) {
            const int j = idx % MK, d0 = (idx / MK) * 8;
            const int kp = k0 + j;
            uint4 val = make_uint4(0, 0, 0, 0);
            if ((kp >= klo || kp < kfe) && kp <= pos_last && d0 < VD) {
                const bf16* src = cache + (size_t)table[kp / P] * page_stride + ((size_t)kvh * P + kp % P) * RS + voff + d0;
                if (vec) {
                    val = *reinterpret_cast<const uint4*>(src);
                } else {
                    bf16* dst = reinterpret_cast<bf16*>(&val);
                    for (int e = 0; e < 8; ++e)
                        if (d0 + e < VD) dst[e] = src[e];
                }
            }
            const bf16* ve = reinterpret_cast<const bf16*>(&val);
#pragma unroll
            for (int e = 0; e < 8; ++e) vt_s[d0 + e][j] = ve[e];
        }
        __syncthreads();
        if (warp * 16 >= nrows) continue;                   // this warp has no rows (it helped loading)
        float sc[MK / 8][4];
#pragma unroll
        for (int nb = 0; nb < MK / 8; ++nb) sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
#pragma unroll
            for (int nb = 0; nb < MK / 8; ++nb) {
                const uint32_t kb0 = *reinterpret_cast<const uint32_t*>(&k_s[nb * 8 + g][ks * 16 + 2 * t4]);
                const uint32_t kb1 = *reinterpret_cast<const uint32_t*>(&k_s[nb * 8 + g][ks * 16 + 8 + 2 * t4]);
                mma_bf16_16816(sc[nb], qa[ks], kb0, kb1);
            }
        }
        // scale, bias, window; the tile's row maxima
        float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
        for (int nb = 0; nb < MK / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = row_a + (e >> 1) * 8;
                const int kp = k0 + nb * 8 + 2 * t4 + (e & 1);
                const int dist = pos_first + r - kp;
                const bool seen = r < nrows && dist >= 0 && (window <= 0 || dist < window || kp < keep_first);
                float v = -FLT_MAX;
                if (seen) v = awb_cap(sc[nb][e] * scale, softcap) - ((tabled && dist < span) ? bias_s[dist] : awb_bias(bias_kind, b1h, b2h, (float)dist));
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
        for (int nb = 0; nb < MK / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                // the weight is rounded to bfloat16 for the second product: the fast exponential's error is far below that
                const float p = sc[nb][e] > -FLT_MAX ? __expf(sc[nb][e] - m[e >> 1]) : 0.f;
                sc[nb][e] = p;
                l[e >> 1] += p;                              // this lane's share; the quad's shares meet at the end
            }
        }
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
#pragma unroll
        for (int kb = 0; kb < MK / 16; ++kb) {
            uint32_t pa[4];
            pa[0] = pack_bf16(sc[2 * kb][0], sc[2 * kb][1]);
            pa[1] = pack_bf16(sc[2 * kb][2], sc[2 * kb][3]);
            pa[2] = pack_bf16(sc[2 * kb + 1][0], sc[2 * kb + 1][1]);
            pa[3] = pack_bf16(sc[2 * kb + 1][2], sc[2 * kb + 1][3]);
#pragma unroll
            for (int nb = 0; nb < DV / 8; ++nb) {
                const uint32_t vb0 = *reinterpret_cast<const uint32_t*>(&vt_s[nb * 8 + g][kb * 16 + 2 * t4]);
                const uint32_t vb1 = *reinterpret_cast<const uint32_t*>(&vt_s[nb * 8 + g][kb * 16 + 8 + 2 * t4]);
                mma_bf16_16816(o[nb], pa, vb0, vb1);
            }
        }
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
        float inv = 1.0f / (sink ? l[i] + expf(sink[h] - m[i]) : l[i]);
        if (gate) inv /= 1.0f + expf(-gate[(size_t)(row0 + r) * gate_ld + h]);
        bf16* dst = out + ((size_t)(row0 + r) * nh + h) * VD;
#pragma unroll
        for (int nb = 0; nb < DV / 8; ++nb) {
            const int c = nb * 8 + 2 * t4;
            if (c < VD) dst[c] = __float2bfloat16_rn(o[nb][2 * i] * inv);
            if (c + 1 < VD) dst[c + 1] = __float2bfloat16_rn(o[nb][2 * i + 1] * inv);
        }
    }
}

template <int DK, int DV>
static int launch_awb_mma(const void* q, void* out, const void* cache, const int* block_table, int max_blocks,
                          const int* seq_start, const int* positions, int nseq, int T, int nh, int nkv, int D, int VD,
                          int P, long long page_stride, float scale, float softcap, int window, const float* r1, const float* r2,
                          int skip_single, int RS, int voff, int bias_kind, int keep_first, const float* gate,
                          long long gate_ld, const float* sink, cudaStream_t stream) {
    const dim3 grid((unsigned)(T / MQ + nseq), (unsigned)nh);
    AP_CHECK_PDL_LAUNCH("attention_window_bias_mma",
                        ap_launch_pdl(attention_window_bias_mma_kernel<DK, DV>, grid, dim3(AWB_THREADS), 0, stream,
                                      (const bf16*)q, (bf16*)out, (const bf16*)cache, block_table, max_blocks, seq_start,
                                      positions, nseq, nh, nkv, D, VD, P, (size_t)page_stride, scale, softcap, window, r1, r2,
                                      skip_single, RS, voff, bias_kind, keep_first, gate, gate_ld, sink));
    return AP_OK;
}

// ---------------------------------------------------------------------------------------
// Sequences that bring one row (decoding).  One CTA per (sequence, key/value head): the query
// heads that share the key/value head are served together, so every key and value is read
// once for all of them.  The eight warps take the key tiles in turn (tile i goes to warp
// i mod 8), each with an online softmax of its own; a lane reads its key's row straight from
// the page, values come row by row with the lanes across the columns; at the end the warps'
// partial results meet in shared memory and are merged in warp order.  Sequences with
// another number of rows are left to the kernel above (`skip_single` there).
// ---------------------------------------------------------------------------------------
#define DEC_REP_MAX 8             // query heads per CTA at most (more: the grid's z walks them)
#define DEC_WARPS 8               // the kernel is a chain of dependent steps per key tile: eight warps share the tiles
#define DEC_THREADS (DEC_WARPS * 32)

// DEC_REP: query heads per CTA this kernel is built for (1, 2, 4, 8); NC: value columns per lane (VD <= 32 NC)
template <typename TA, int DEC_REP, int NC>
__global__ void __launch_bounds__(DEC_THREADS)
attention_window_bias_decode_kernel(const TA* __restrict__ q, TA* __restrict__ out, const TA* __restrict__ cache,
                                    const int* __restrict__ block_table, int max_blocks,
                                    const int* __restrict__ seq_start, const int* __restrict__ positions, int nh,
                                    int nkv, int D, int VD, int P, size_t page_stride, float scale, float softcap, int window,
                                    const float* __restrict__ r1, const float* __restrict__ r2, int RS, int voff,
                                    int bias_kind, int keep_first, const float* __restrict__ gate, long long gate_ld,
                                    const float* __restrict__ sink, int nslice) {
    constexpr int rep_chunk = DEC_REP;
    extern __shared__ __align__(16) float smem[];
    ap_pdl_trigger();
    ap_pdl_wait();
    // nslice > 1: the CTAs of a thread-block cluster share a sequence's key tiles (tile n goes to warp n mod 8 of
    // CTA (n / 8) mod nslice) and the first of them merges all their warps' partial results through distributed
    // shared memory
    const int seq = blockIdx.x / nslice, slice = blockIdx.x % nslice, kvh = blockIdx.y;
    const int row = seq_start[seq];
    if (seq_start[seq + 1] - row != 1) return;
    const int rep_all = nh / nkv;
    const int h0 = kvh * rep_all + blockIdx.z * rep_chunk;      // rep_chunk <= DEC_REP query heads per CTA
    const int rep = min(rep_chunk, rep_all - (int)blockIdx.z * rep_chunk);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* q_s = smem;                                   // [DEC_REP][D]
    float* p_s = q_s + DEC_REP * D;                      // [DEC_WARPS][DEC_REP][KT]
    float* part = p_s + DEC_WARPS * DEC_REP * KT;        // [DEC_WARPS][DEC_REP][VD + 2]
    // a value row in shared memory: whole 16-byte runs, and 16 bytes more, so that the lanes' rows start in
    // different banks (rows of exactly 256 bytes would put all 32 lanes' stores on the same four banks)
    const int VDP = (VD + 7) / 8 * 8 + 8;
    TA* v_s = reinterpret_cast<TA*>(smem + ((DEC_REP * D + DEC_WARPS * DEC_REP * KT + DEC_WARPS * DEC_REP * (VD + 2) + 3) / 4) * 4) +
              (size_t)warp * KT * VDP;                       // [KT][VDP] per warp, on a 16-byte boundary
    for (int i = threadIdx.x; i < rep * D; i += DEC_THREADS)
        q_s[i] = ap_to_float(q[((size_t)row * nh + h0) * D + i]);
    __syncthreads();
    const int qpos = positions[row];
    const int* table = block_table + (size_t)seq * max_blocks;
    const int klo = (window > 0 && qpos - window + 1 > 0) ? qpos - window + 1 : 0;
    float acc[DEC_REP][NC], m[DEC_REP], l[DEC_REP], b1[DEC_REP], b2[DEC_REP];
#pragma unroll
    for (int i = 0; i < DEC_REP; ++i) {
        m[i] = -FLT_MAX;
        l[i] = 0.f;
        b1[i] = (r1 && i < rep) ? r1[h0 + i] : 0.f;
        b2[i] = (r2 && i < rep) ? r2[h0 + i] : 0.f;
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[i][c] = 0.f;
    }
    const int nc = (VD + 31) / 32;
    float* pw = p_s + warp * DEC_REP * KT;
    // the tiles of the kept first tokens (0 .. tiles_kept-1), then those from the window's first on
    const int kfe = keep_first < klo ? keep_first : klo;
    const int tile_win = klo / KT;
    const int tiles_kept = min((kfe + KT - 1) / KT, tile_win);
    const bool vec_ok = sizeof(TA) == 2 && RS % 8 == 0 && voff % 8 == 0 && (page_stride % 8) == 0 &&
                        ((uintptr_t)cache & 15) == 0;
    for (int n = warp + slice * DEC_WARPS;; n += DEC_WARPS * nslice) {
        const int tile = n < tiles_kept ? n : tile_win + (n - tiles_kept);
        if (tile * KT > qpos) break;
        const int kp = tile * KT + lane;
        const bool seen = (kp >= klo || kp < kfe) && kp <= qpos;
        float s[DEC_REP];
#pragma unroll
        for (int i = 0; i < DEC_REP; ++i) s[i] = 0.f;
        if (seen) {
            const TA* kr = cache + (size_t)table[kp / P] * page_stride + ((size_t)kvh * P + kp % P) * RS;
            if (vec_ok && D % 8 == 0) {
                // eight 16-bit elements of the key's row per load; unrolled far, so that a lane's loads of a
                // whole row are in flight together
#pragma unroll 16
                for (int d = 0; d < D; d += 8) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(kr) + d);
                    const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 kv = __bfloat1622float2(k2[e]);
#pragma unroll
                        for (int i = 0; i < DEC_REP; ++i)
                            if (i < rep) s[i] = fmaf(q_s[i * D + d + 2 * e + 1], kv.y, fmaf(q_s[i * D + d + 2 * e], kv.x, s[i]));
                    }
                }
            } else {
                for (int d = 0; d < D; ++d) {
                    const float kv = ap_to_float(kr[d]);
#pragma unroll
                    for (int i = 0; i < DEC_REP; ++i)
                        if (i < rep) s[i] = fmaf(q_s[i * D + d], kv, s[i]);
                }
            }
        }
        const float dist = (float)(qpos - kp);
#pragma unroll
        for (int i = 0; i < DEC_REP; ++i) {
            const float sc = seen ? awb_cap(s[i] * scale, softcap) - awb_bias(bias_kind, b1[i], b2[i], dist) : -FLT_MAX;
            const float m_new = fmaxf(m[i], ap_warp_max(sc));
            const float p = seen ? expf(sc - m_new) : 0.f;
            const float alpha = expf(m[i] - m_new);
            l[i] = l[i] * alpha + ap_warp_sum(p);
            m[i] = m_new;
            pw[i * KT + lane] = p;
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[i][c] *= alpha;
        }
        // every lane brings its key's value row into the warp's tile (all loads of a lane in flight at once);
        // a lane whose key no row sees clears its row: its weight is zero, and zero times what was there is not
        if (!seen) {
            TA* dst = v_s + lane * VDP;
            for (int d = 0; d < VD; ++d) dst[d] = ap_from_float<TA>(0.f);
        } else {
            const TA* vr = cache + (size_t)table[kp / P] * page_stride + ((size_t)kvh * P + kp % P) * RS + voff;
            TA* dst = v_s + lane * VDP;
            if (vec_ok && VD % 8 == 0) {
#pragma unroll 16
                for (int d = 0; d < VD; d += 8)
                    *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst) + d) =
                        *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(vr) + d);
            } else {
#pragma unroll 4
                for (int d = 0; d < VD; ++d) dst[d] = vr[d];
            }
        }
        __syncwarp();
        const int last = min(KT, qpos - tile * KT + 1);
        for (int j = 0; j < last; ++j) {
            const TA* vr = v_s + j * VDP;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                if (c < nc) {
                    const int d = lane + 32 * c;
                    const float vv = d < VD ? ap_to_float(vr[d]) : 0.f;
#pragma unroll
                    for (int i = 0; i < DEC_REP; ++i)
                        if (i < rep) acc[i][c] = fmaf(pw[i * KT + j], vv, acc[i][c]);
                }
            }
        }
        __syncwarp();
    }
    // the warps' partial results: [VD] sums, then the maximum and the sum of weights
    const int PW = VD + 2;
#pragma unroll
    for (int i = 0; i < DEC_REP; ++i) {
        if (i < rep) {
            float* dst = part + (warp * DEC_REP + i) * PW;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int d = lane + 32 * c;
                if (d < VD) dst[d] = acc[i][c];
            }
            if (lane == 0) {
                dst[VD] = m[i];
                dst[VD + 1] = l[i];
            }
        }
    }
    if (nslice > 1) {
        cg::cluster_group cl = cg::this_cluster();
        cl.sync();                                           // every CTA's partial results are in its shared memory
        if (slice == 0) {
            for (int e = threadIdx.x; e < rep * VD; e += DEC_THREADS) {
                const int i = e / VD, d = e - i * VD;
                float mm = -FLT_MAX;
                for (int c = 0; c < nslice; ++c) {
                    const float* pc = cl.map_shared_rank(part, c);
                    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, pc[(w * DEC_REP + i) * PW + VD]);
                }
                float num = 0.f, den = 0.f;
                for (int c = 0; c < nslice; ++c) {           // in the order of the slices and of their warps
                    const float* pc = cl.map_shared_rank(part, c);
                    for (int w = 0; w < DEC_WARPS; ++w) {
                        const float* src = pc + (w * DEC_REP + i) * PW;
                        const float f = expf(src[VD] - mm);
                        num = fmaf(src[d], f, num);
                        den = fmaf(src[VD + 1], f, den);
                    }
                }
                if (sink) den += expf(sink[h0 + i] - mm);
                float res = num / den;
                if (gate) res /= 1.0f + expf(-gate[(size_t)row * gate_ld + h0 + i]);
                out[((size_t)row * nh + h0 + i) * VD + d] = ap_from_float<TA>(res);
            }
        }
        cl.sync();                                           // nobody leaves while the first CTA still reads
        return;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < rep * VD; e += DEC_THREADS) {
        const int i = e / VD, d = e - i * VD;
        float mm = -FLT_MAX;
        for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, part[(w * DEC_REP + i) * PW + VD]);
        float num = 0.f, den = 0.f;
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float* src = part + (w * DEC_REP + i) * PW;
            const float f = expf(src[VD] - mm);          // 0 for a warp that saw no key (its maximum is -FLT_MAX)
            num = fmaf(src[d], f, num);
            den = fmaf(src[VD + 1], f, den);
        }
        if (sink) den += expf(sink[h0 + i] - mm);
        float res = num / den;
        if (gate) res /= 1.0f + expf(-gate[(size_t)row * gate_ld + h0 + i]);
        out[((size_t)row * nh + h0 + i) * VD + d] = ap_from_float<TA>(res);
    }
}

AP_EXPORT int ap_attention_window_bias(const void* q, void* out, const void* cache, int dtype, const int* block_table,
                                       int max_blocks, const int* seq_start, const int* positions, int nseq, int T,
                                       int nh, int nkv, int D, int VD, int P, long long page_stride, float scale,
                                       float softcap, int window, const float* r1, const float* r2, int single_rows, int other_rows,
                                       int RS, int voff, int bias_kind, int keep_first, const float* gate,
                                       long long gate_ld, const float* sink, int max_context, cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && nseq >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0 && P > 0 && max_blocks > 0,
               "attention_window_bias: bad sizes T=%d heads=%d kv_heads=%d page=%d", T, nh, nkv, P);
    AP_REQUIRE(D > 0 && VD > 0 && D <= MAX_WIDE_HEAD && VD <= MAX_WIDE_HEAD,
               "attention_window_bias: head sizes %d/%d are not in 1..%d", D, VD, MAX_WIDE_HEAD);
    AP_REQUIRE(nh <= 65535, "attention_window_bias: %d heads exceed the grid", nh);
    AP_REQUIRE(RS >= D && voff >= 0 && voff + VD <= RS, "attention_window_bias: a record of %d numbers does not hold "
               "a key of %d and a value of %d at %d", RS, D, VD, voff);
    AP_REQUIRE(bias_kind == BIAS_NONE || (bias_kind == BIAS_LOG && r1 && r2) || (bias_kind == BIAS_LINEAR && r1),
               "attention_window_bias: bias kind %d lacks its per-head numbers", bias_kind);
    AP_REQUIRE(keep_first >= 0 && (gate == nullptr || gate_ld >= nh), "attention_window_bias: bad keep_first or gate stride");
    if (window <= 0) keep_first = 0;                      // without a window every key is visible anyway
    if (bias_kind == BIAS_NONE) r1 = r2 = nullptr;
    if (T == 0 || nseq == 0) return AP_OK;
    const bool wide = VD > MAX_HEAD;                      // more value columns per lane: the kernels built for NC = 20
    // single_rows 1: sequences that bring one row go to the kernel made for them; 2: they are left out (the
    // caller serves them otherwise); other_rows: there are sequences with another number of rows (both 0:
    // everything on the general kernel)
    // the decode kernel keeps a tile of value rows per warp in shared memory: where the values are too wide
    // for that, sequences of one row run on the general kernel like the others
    if (single_rows == 1 && (size_t)DEC_WARPS * KT * ((VD + 7) / 8 * 8 + 8) * (dtype == AP_F32 ? 4 : 2) > 160 * 1024) {
        single_rows = 0;
        other_rows = 1;
    }
    if (single_rows == 1) {
        const int rep = nh / nkv;
        // all query heads of a key/value head in one CTA (every key read once) where that still fills the
        // GPU; else fewer heads per CTA and the keys read again from L2
        // key slices: where the caller knows that single rows see a thousand keys and more (max_context: the
        // longest context of the step, 0: not known), the tiles of a sequence are shared by a cluster of up to
        // eight CTAs, 256 keys and more to each
        int nslice = 1;
        const int keys = window > 0 && window < max_context ? window + keep_first : max_context;
        while (nslice < 8 && keys >= 512 * nslice && keys >= 1024) nslice *= 2;
        int rep_chunk = 1;
        while (rep_chunk < (wide ? 2 : DEC_REP_MAX) && rep_chunk < rep) rep_chunk *= 2;
        while (rep_chunk > 1 && (long long)nseq * nkv * ((rep + rep_chunk - 1) / rep_chunk) * nslice < 2 * 148) rep_chunk /= 2;
        const dim3 dgrid((unsigned)(nseq * nslice), (unsigned)nkv, (unsigned)((rep + rep_chunk - 1) / rep_chunk));
        const size_t dsmem = ((size_t)rep_chunk * D + (size_t)DEC_WARPS * rep_chunk * KT +
                              (size_t)DEC_WARPS * rep_chunk * (VD + 2)) * sizeof(float) +
                             (size_t)DEC_WARPS * KT * ((VD + 7) / 8 * 8 + 8) * (dtype == AP_F32 ? 4 : 2) + 16;
        AP_REQUIRE(nkv <= 65535, "attention_window_bias: %d key/value heads exceed the grid", nkv);
#define LAUNCH_DEC(TA)                                                                                               \
    do {                                                                                                             \
        auto kern = wide ? (rep_chunk == 1 ? attention_window_bias_decode_kernel<TA, 1, WIDE_NC>                     \
                                           : attention_window_bias_decode_kernel<TA, 2, WIDE_NC>)                    \
                  : rep_chunk == 1 ? attention_window_bias_decode_kernel<TA, 1, MAX_HEAD / 32>                       \
                  : rep_chunk == 2 ? attention_window_bias_decode_kernel<TA, 2, MAX_HEAD / 32>                       \
                  : rep_chunk == 4 ? attention_window_bias_decode_kernel<TA, 4, MAX_HEAD / 32>                       \
                                   : attention_window_bias_decode_kernel<TA, 8, MAX_HEAD / 32>;                      \
        if (dsmem > 48 * 1024) {                                                                                     \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsmem);     \
            AP_REQUIRE(e == cudaSuccess, "attention_window_bias: cannot reserve %zu bytes of shared memory", dsmem); \
        }                                                                                                            \
        if (nslice > 1) {                                                                                            \
            cudaLaunchConfig_t cfg = {};                                                                             \
            cfg.gridDim = dgrid;                                                                                     \
            cfg.blockDim = dim3(DEC_THREADS);                                                                        \
            cfg.dynamicSmemBytes = dsmem;                                                                            \
            cfg.stream = stream;                                                                                     \
            cudaLaunchAttribute attr[2];                                                                             \
            attr[0].id = cudaLaunchAttributeClusterDimension;                                                        \
            attr[0].val.clusterDim.x = (unsigned)nslice;                                                             \
            attr[0].val.clusterDim.y = 1;                                                                            \
            attr[0].val.clusterDim.z = 1;                                                                            \
            attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                         \
            attr[1].val.programmaticStreamSerializationAllowed = 1;                                                  \
            cfg.attrs = attr;                                                                                        \
            cfg.numAttrs = ap_pdl_enabled() ? 2 : 1;                                                                 \
            AP_CHECK_PDL_LAUNCH("attention_window_bias_decode",                                                      \
                                cudaLaunchKernelEx(&cfg, kern, (const TA*)q, (TA*)out, (const TA*)cache, block_table, \
                                                   max_blocks, seq_start, positions, nh, nkv, D, VD, P,              \
                                                   (size_t)page_stride, scale, softcap, window, r1, r2, RS, voff,    \
                                                   bias_kind, keep_first, gate, gate_ld, sink, nslice));             \
        } else {                                                                                                     \
            AP_CHECK_PDL_LAUNCH("attention_window_bias_decode",                                                      \
                                ap_launch_pdl(kern, dgrid, dim3(DEC_THREADS), dsmem, stream, (const TA*)q, (TA*)out, \
                                              (const TA*)cache, block_table, max_blocks, seq_start, positions, nh,   \
                                              nkv, D, VD, P, (size_t)page_stride, scale, softcap, window, r1, r2, RS, \
                                              voff, bias_kind, keep_first, gate, gate_ld, sink, 1));                 \
        }                                                                                                            \
    } while (0)
        if (dtype == AP_F32) LAUNCH_DEC(float);
        else if (dtype == AP_BF16) LAUNCH_DEC(bf16);
        else AP_REQUIRE(false, "attention_window_bias: unknown dtype %d", dtype);
#undef LAUNCH_DEC
        if (!other_rows) return AP_OK;
    }
    const int skip_single = single_rows ? 1 : 0;
    if (dtype == AP_BF16 && D <= 192 && VD <= 128) {
        // the tensor-core kernel, built for head sizes rounded up to 32, 64, 128 (keys also 192)
        const int dk = D <= 32 ? 32 : (D <= 64 ? 64 : (D <= 128 ? 128 : 192)), dv = VD <= 32 ? 32 : (VD <= 64 ? 64 : 128);
#define MMA_ARGS q, out, cache, block_table, max_blocks, seq_start, positions, nseq, T, nh, nkv, D, VD, P, page_stride, \
                 scale, softcap, window, r1, r2, skip_single, RS, voff, bias_kind, keep_first, gate, gate_ld, sink, stream
        switch (dk * 1000 + dv) {
            case 32032: return launch_awb_mma<32, 32>(MMA_ARGS);
            case 32064: return launch_awb_mma<32, 64>(MMA_ARGS);
            case 32128: return launch_awb_mma<32, 128>(MMA_ARGS);
            case 64032: return launch_awb_mma<64, 32>(MMA_ARGS);
            case 64064: return launch_awb_mma<64, 64>(MMA_ARGS);
            case 64128: return launch_awb_mma<64, 128>(MMA_ARGS);
            case 128032: return launch_awb_mma<128, 32>(MMA_ARGS);
            case 128064: return launch_awb_mma<128, 64>(MMA_ARGS);
            case 192032: return launch_awb_mma<192, 32>(MMA_ARGS);
            case 192064: return launch_awb_mma<192, 64>(MMA_ARGS);
            case 192128: return launch_awb_mma<192, 128>(MMA_ARGS);
            default: return launch_awb_mma<128, 128>(MMA_ARGS);
        }
#undef MMA_ARGS
    }
    // every sequence's rows in tiles of QT: at most T / QT whole tiles and one ragged tile per sequence
    const dim3 grid((unsigned)(T / QT + nseq), (unsigned)nh);
    const size_t smem = ((size_t)QT * D + (size_t)KT * (D + 1) + (size_t)KT * VD + AWB_WARPS * RPW * KT) * sizeof(float);
#define LAUNCH(TA)                                                                                                   \
    do {                                                                                                             \
        auto kern = wide ? attention_window_bias_kernel<TA, WIDE_NC> : attention_window_bias_kernel<TA, MAX_HEAD / 32>; \
        AP_REQUIRE(smem <= 200 * 1024, "attention_window_bias: head sizes %d/%d do not fit shared memory", D, VD);   \
        if (smem > 48 * 1024) {                                                                                      \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
            AP_REQUIRE(e == cudaSuccess, "attention_window_bias: cannot reserve %zu bytes of shared memory", smem);  \
        }                                                                                                            \
        AP_CHECK_PDL_LAUNCH("attention_window_bias",                                                                 \
                            ap_launch_pdl(kern, grid, dim3(AWB_THREADS), smem, stream, (const TA*)q, (TA*)out,       \
                                          (const TA*)cache, block_table, max_blocks, seq_start, positions, nseq, nh, \
                                          nkv, D, VD, P, (size_t)page_stride, scale, softcap, window, r1, r2, skip_single,    \
                                          RS, voff, bias_kind, keep_first, gate, gate_ld, sink));                    \
    } while (0)
    if (dtype == AP_F32) LAUNCH(float);
    else if (dtype == AP_BF16) LAUNCH(bf16);
    else AP_REQUIRE(false, "attention_window_bias: unknown dtype %d", dtype);
#undef LAUNCH
    return AP_OK;
}
