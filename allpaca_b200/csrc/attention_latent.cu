// Helpers of an attention whose keys and values are projections of one small latent vector per
// token, shared by all heads.  A token keeps in its page only that latent c (R numbers, RMS-normed)
// and one rotated key part (rot numbers) that every head uses.  With per-head matrices U_k [D, R]
// and U_v [E, R] the scores and outputs of head h are
//
//   score(i, j) = q_nope(i, h) . (U_k[h] c_j) + q_rot(i, h) . k_rot(j)  =  (U_k[h]^T q_nope(i, h)) . c_j + ...
//   out(i, h)   = sum_j p_ij U_v[h] c_j                                =  U_v[h] (sum_j p_ij c_j)
//
// so the attention itself runs in the latent space, as attention with ONE key/value head whose
// key is the token's record [c | k_rot] and whose value is the head of that record (the kernels of
// attention_window_bias.cu with voff = 0), between two small per-head products:
//
//   latent_prepare : from the stacked down-projections of a row (32-bit sums): the query latent,
//                    RMS-normed with its weight, for the up-projection; the key/value latent normed
//                    and the shared key part rotated, both written into the row's page and slot
//   head_project   : out[t, h, :N] = in[t, h, :K] W[h] for W [H, K, N]; the `tail` numbers behind
//                    in[t, h, :K] are rotated by the row's position and put behind out[t, h, :N]
//                    (queries into the latent space with their rotated part; latent outputs to values);
//                    without W the K numbers are copied (queries rotated, nothing else)
//   latent_gather  : the records of every token of the sequences that bring several rows, out of their
//                    pages into one matrix in sequence order, with a table that says where each
//                    sequence's token j went.  A long prompt is cheaper the other way round: one
//                    product turns that matrix into per-head keys and values [token][head][k | k_rot | v]
//                    (what a page of ONE token with H key/value heads looks like to the attention
//                    kernels, the table being its block table), and the attention runs on the heads'
//                    own small sizes.
//
// Norm statistics, angles and every sum are 32-bit.
#include "common.cuh"

#define LP_THREADS 128

// cos_sin: [T][half] (cos, sin) of the row's angles (any factor on them already applied); the first
// 2 * half numbers are rotated, entry i paired with entry i + half; the rest pass unchanged.
template <typename TI, typename TO>
__device__ __forceinline__ void rotate_half_row(const TI* __restrict__ src, TO* __restrict__ dst, int n, int half,
                                                const float2* __restrict__ cs, int lane) {
    for (int i = lane; i < n; i += 32) {
        float v;
        if (i < half) {
            const float2 c = cs[i];
            v = ap_to_float(src[i]) * c.x - ap_to_float(src[i + half]) * c.y;
        } else if (i < 2 * half) {
            const float2 c = cs[i - half];
            v = ap_to_float(src[i]) * c.x + ap_to_float(src[i - half]) * c.y;
        } else {
            v = ap_to_float(src[i]);
        }
        dst[i] = ap_from_float<TO>(v);
    }
}

// one warp per (row, part): part 0 the query latent (Q > 0), the other the key/value latent (cache != null)
template <typename TA>
__global__ void __launch_bounds__(LP_THREADS)
latent_prepare_kernel(const float* __restrict__ in, long long ld, int q0, int Q, const float* __restrict__ qw,
                      TA* __restrict__ cq, int kv0, int R, int rot, int half, const float* __restrict__ kvw,
                      TA* __restrict__ cache, const int* __restrict__ positions, const int* __restrict__ token_seq,
                      const int* __restrict__ block_table, int max_blocks, int P, size_t page_stride,
                      const float2* __restrict__ cos_sin, float eps, int T) {
    const int lane = threadIdx.x & 31;
    const int parts = (Q > 0 ? 1 : 0) + (cache != nullptr ? 1 : 0);
    const long long unit = (long long)blockIdx.x * (LP_THREADS / 32) + (threadIdx.x >> 5);
    ap_pdl_trigger();
    ap_pdl_wait();
    if (unit >= (long long)T * parts) return;
    const int t = (int)(unit / parts), part = (int)(unit % parts);
    const float* row = in + (size_t)t * ld;
    if (Q > 0 && part == 0) {
        const float* src = row + q0;
        float ss = 0.f;
        for (int d = lane; d < Q; d += 32) ss = fmaf(src[d], src[d], ss);
        ss = ap_warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)Q + eps);
        TA* dst = cq + (size_t)t * Q;
        for (int d = lane; d < Q; d += 32) dst[d] = ap_from_float<TA>(src[d] * inv * qw[d]);
        return;
    }
    const float* src = row + kv0;
    float ss = 0.f;
    for (int d = lane; d < R; d += 32) ss = fmaf(src[d], src[d], ss);
    ss = ap_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)R + eps);
    const int pos = positions[t];
    const int page = block_table[(size_t)token_seq[t] * max_blocks + pos / P];
    TA* dst = cache + (size_t)page * page_stride + (size_t)(pos % P) * (R + rot);
    for (int d = lane; d < R; d += 32) dst[d] = ap_from_float<TA>(src[d] * inv * kvw[d]);
    rotate_half_row(src + R, dst + R, rot, half, cos_sin + (size_t)t * half, lane);
}

AP_EXPORT int ap_latent_prepare(const float* in, long long ld, int q0, int Q, const float* qw, void* cq, int kv0, int R,
                                int rot, int rot_dims, const float* kvw, void* cache, int act_dtype,
                                const int* positions, const int* token_seq, const int* block_table, int max_blocks,
                                int P, long long page_stride, const float* cos_sin, float eps, int T,
                                cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && Q >= 0 && (Q == 0 || (qw && cq && q0 >= 0)), "latent_prepare: bad query latent Q=%d", Q);
    AP_REQUIRE(cache == nullptr || (R > 0 && rot >= 0 && kv0 >= 0 && kvw && positions && token_seq && block_table &&
                                    max_blocks > 0 && P > 0),
               "latent_prepare: storing needs the latent's sizes, its weight, token_seq and a block table");
    AP_REQUIRE(cache == nullptr || (rot_dims % 2 == 0 && rot_dims >= 0 && rot_dims <= rot && (rot_dims == 0 || cos_sin)),
               "latent_prepare: %d rotated dimensions of %d", rot_dims, rot);
    const int parts = (Q > 0 ? 1 : 0) + (cache != nullptr ? 1 : 0);
    if (T == 0 || parts == 0) return AP_OK;
    const long long units = (long long)T * parts;
    const dim3 grid((unsigned)((units + LP_THREADS / 32 - 1) / (LP_THREADS / 32)));
#define LAUNCH(TA)                                                                                                    \
    AP_CHECK_PDL_LAUNCH("latent_prepare",                                                                             \
                        ap_launch_pdl(latent_prepare_kernel<TA>, grid, dim3(LP_THREADS), 0, stream, in, ld, q0, Q, qw, \
                                      (TA*)cq, kv0, R, rot, rot_dims / 2, kvw, (TA*)cache, positions, token_seq,      \
                                      block_table, max_blocks, P, (size_t)page_stride, (const float2*)cos_sin, eps, T))
    if (act_dtype == AP_F32) LAUNCH(float);
    else if (act_dtype == AP_BF16) LAUNCH(bf16);
    else AP_REQUIRE(false, "latent_prepare: unknown dtype %d", act_dtype);
#undef LAUNCH
    return AP_OK;
}

// ---------------------------------------------------------------------------------------
// out[t, h, n] = sum_k in[t, h, k] W[h, k, n].  A CTA takes HP_ROWS rows of one head and HP_COLS
// columns; the rows' inputs wait in shared memory; thread (slice, column) walks its quarter of k
// upwards (neighbouring threads read neighbouring weights, four slices of k in flight at once:
// with few rows the walk is a chain of loads, not arithmetic), and the slices' sums are added in
// slice order.  So an output is a 32-bit sum in a fixed order whatever else the step holds.
// ---------------------------------------------------------------------------------------
#define HP_ROWS 8
#define HP_COLS 32
#define HP_SLICES 4
#define HP_THREADS (HP_COLS * HP_SLICES)

template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(HP_THREADS)
head_project_kernel(const TI* __restrict__ in, long long in_ld, int in_hs, const TW* __restrict__ w,
                    TO* __restrict__ out, long long out_ld, int out_hs, int T, int K, int N, int tail, int half,
                    const float2* __restrict__ cos_sin) {
    extern __shared__ __align__(16) float in_s[];            // [HP_ROWS][K], then [HP_SLICES][HP_ROWS][HP_COLS]
    float* part = in_s + HP_ROWS * K;
    const int row0 = blockIdx.x * HP_ROWS, h = blockIdx.y;
    const int rows = min(HP_ROWS, T - row0);
    ap_pdl_trigger();
    ap_pdl_wait();
    for (int i = threadIdx.x; i < HP_ROWS * K; i += HP_THREADS) {
        const int r = i / K, k = i - r * K;
        in_s[i] = r < rows ? ap_to_float(in[(size_t)(row0 + r) * in_ld + (size_t)h * in_hs + k]) : 0.f;
    }
    __syncthreads();
    const int col = threadIdx.x % HP_COLS, slice = threadIdx.x / HP_COLS;
    const int n = blockIdx.z * HP_COLS + col;
    float acc[HP_ROWS];
#pragma unroll
    for (int r = 0; r < HP_ROWS; ++r) acc[r] = 0.f;
    if (n < N) {
        if (w == nullptr) {                                  // no matrix: the numbers pass as they are
            if (slice == 0) {
#pragma unroll
                for (int r = 0; r < HP_ROWS; ++r) acc[r] = in_s[r * K + n];
            }
        } else {
            const int per = (K + HP_SLICES - 1) / HP_SLICES;
            const int k0 = slice * per, k1 = min(K, k0 + per);
            const TW* wc = w + (size_t)h * K * N + n;
#pragma unroll 8
            for (int k = k0; k < k1; ++k) {
                const float wv = ap_to_float(wc[(size_t)k * N]);
#pragma unroll
                for (int r = 0; r < HP_ROWS; ++r) acc[r] = fmaf(in_s[r * K + k], wv, acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < HP_ROWS; ++r) part[(slice * HP_ROWS + r) * HP_COLS + col] = acc[r];
    __syncthreads();
    for (int i = threadIdx.x; i < HP_ROWS * HP_COLS; i += HP_THREADS) {
        const int r = i / HP_COLS, c = i - r * HP_COLS;
        const int nn = blockIdx.z * HP_COLS + c;
        if (r < rows && nn < N) {
            float v = part[r * HP_COLS + c];
#pragma unroll
            for (int sl = 1; sl < HP_SLICES; ++sl) v += part[(sl * HP_ROWS + r) * HP_COLS + c];
            out[(size_t)(row0 + r) * out_ld + (size_t)h * out_hs + nn] = ap_from_float<TO>(v);
        }
    }
    if (tail > 0 && blockIdx.z == 0) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int r = warp; r < rows; r += HP_THREADS / 32)
            rotate_half_row(in + (size_t)(row0 + r) * in_ld + (size_t)h * in_hs + K,
                            out + (size_t)(row0 + r) * out_ld + (size_t)h * out_hs + N, tail, half,
                            cos_sin + (size_t)(row0 + r) * half, lane);
    }
}

AP_EXPORT int ap_head_project(const void* in, int in_dtype, long long in_ld, int in_hs, const void* w, int w_dtype,
                              void* out, int out_dtype, long long out_ld, int out_hs, int T, int H, int K, int N,
                              int tail, int tail_dims, const float* cos_sin, cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && H > 0 && K > 0 && N > 0 && tail >= 0, "head_project: bad sizes T=%d H=%d K=%d N=%d", T, H, K, N);
    AP_REQUIRE(w != nullptr || N == K, "head_project: without a matrix the numbers are copied, N must equal K");
    AP_REQUIRE(H <= 65535, "head_project: %d heads exceed the grid", H);
    AP_REQUIRE(in_hs >= K + tail && out_hs >= N + tail && in_ld >= (long long)H * in_hs && out_ld >= (long long)H * out_hs,
               "head_project: the strides do not hold the heads");
    AP_REQUIRE(tail_dims % 2 == 0 && tail_dims >= 0 && tail_dims <= tail && (tail_dims == 0 || cos_sin),
               "head_project: %d rotated dimensions of a tail of %d", tail_dims, tail);
    if (T == 0) return AP_OK;
    const size_t smem = ((size_t)HP_ROWS * K + (size_t)HP_SLICES * HP_ROWS * HP_COLS) * sizeof(float);
    AP_REQUIRE(smem <= 200 * 1024, "head_project: K=%d does not fit shared memory", K);
    const dim3 grid((unsigned)((T + HP_ROWS - 1) / HP_ROWS), (unsigned)H, (unsigned)((N + HP_COLS - 1) / HP_COLS));
#define LAUNCH(TI, TW, TO)                                                                                             \
    do {                                                                                                               \
        auto kern = head_project_kernel<TI, TW, TO>;                                                                   \
        if (smem > 48 * 1024) {                                                                                        \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
            AP_REQUIRE(e == cudaSuccess, "head_project: cannot reserve %zu bytes of shared memory", smem);             \
        }                                                                                                              \
        AP_CHECK_PDL_LAUNCH("head_project",                                                                            \
                            ap_launch_pdl(kern, grid, dim3(HP_THREADS), smem, stream, (const TI*)in, in_ld, in_hs,     \
                                          (const TW*)w, (TO*)out, out_ld, out_hs, T, K, N, tail, tail_dims / 2,        \
                                          (const float2*)cos_sin));                                                    \
    } while (0)
    if (in_dtype == AP_F32 && w_dtype == AP_F32 && out_dtype == AP_F32) LAUNCH(float, float, float);
    else if (in_dtype == AP_F32 && w_dtype == AP_BF16 && out_dtype == AP_BF16) LAUNCH(float, bf16, bf16);
    else if (in_dtype == AP_BF16 && w_dtype == AP_BF16 && out_dtype == AP_BF16) LAUNCH(bf16, bf16, bf16);
    else AP_REQUIRE(false, "head_project: unsupported dtypes in=%d w=%d out=%d", in_dtype, w_dtype, out_dtype);
#undef LAUNCH
    return AP_OK;
}

// ---------------------------------------------------------------------------------------
// One CTA per gathered token.  Sequences that bring one row are left out (their attention runs in
// the latent space); the others' tokens 0 .. context-1 follow one another in sequence order (behind a
// window: the tokens from the first one that the sequence's first row of this step still sees).
// where[s, j] is the row of `out` that holds token j of sequence s.
// ---------------------------------------------------------------------------------------
template <typename TA>
__global__ void latent_gather_kernel(const TA* __restrict__ cache, size_t page_stride, int P, int RS,
                                     const int* __restrict__ block_table, int max_blocks,
                                     const int* __restrict__ seq_start, const int* __restrict__ context_lens, int nseq,
                                     TA* __restrict__ out, int* __restrict__ where, int width, int window) {
    ap_pdl_trigger();
    ap_pdl_wait();
    int b = blockIdx.x, seq = -1;
    for (int s = 0; s < nseq; ++s) {
        const int rows = seq_start[s + 1] - seq_start[s];
        // behind a window: from the first token that the sequence's first row of this step still sees
        const int first = context_lens[s] - rows;
        const int lo = (window > 0 && first - window + 1 > 0) ? first - window + 1 : 0;
        const int n = rows > 1 ? context_lens[s] - lo : 0;
        if (b < n) {
            seq = s;
            b += lo;
            break;
        }
        b -= n;
    }
    if (seq < 0) return;
    const int page = block_table[(size_t)seq * max_blocks + b / P];
    const TA* src = cache + (size_t)page * page_stride + (size_t)(b % P) * RS;
    TA* dst = out + (size_t)blockIdx.x * RS;
    for (int d = threadIdx.x; d < RS; d += blockDim.x) dst[d] = src[d];
    if (threadIdx.x == 0) where[(size_t)seq * width + b] = blockIdx.x;
}

AP_EXPORT int ap_latent_gather(const void* cache, int dtype, long long page_stride, int P, int RS,
                               const int* block_table, int max_blocks, const int* seq_start, const int* context_lens,
                               int nseq, void* out, int* where, int width, int total, int window, cudaStream_t stream) {
    AP_REQUIRE(P > 0 && RS > 0 && max_blocks > 0 && nseq >= 0 && width > 0 && total >= 0,
               "latent_gather: bad sizes page=%d record=%d sequences=%d", P, RS, nseq);
    AP_REQUIRE(cache && block_table && seq_start && context_lens && out && where, "latent_gather: a pointer is missing");
    if (total == 0 || nseq == 0) return AP_OK;
    const int threads = RS >= 256 ? 256 : (RS >= 128 ? 128 : 64);
#define LAUNCH(TA)                                                                                                     \
    AP_CHECK_PDL_LAUNCH("latent_gather",                                                                               \
                        ap_launch_pdl(latent_gather_kernel<TA>, dim3((unsigned)total), dim3(threads), 0, stream,       \
                                      (const TA*)cache, (size_t)page_stride, P, RS, block_table, max_blocks, seq_start, \
                                      context_lens, nseq, (TA*)out, where, width, window))
    if (dtype == AP_F32) LAUNCH(float);
    else if (dtype == AP_BF16) LAUNCH(bf16);
    else AP_REQUIRE(false, "latent_gather: unknown dtype %d", dtype);
#undef LAUNCH
    return AP_OK;
}
