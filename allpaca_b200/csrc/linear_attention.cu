// Linear attention in its recurrent form: per head a state S of [D, V] 32-bit numbers that a request
// carries from step to step, written by outer products of keys and values and read by queries:
//
//   S_t = diag(a_t) S_{t-1} + k_t u_t^T        o_t = S_t^T q_t * out_scale
//
// with the variants as parameters of one kernel:
//   decay a_t   one fixed number per head (DECAY_HEAD_CONST: retention);
//               one number per head and token, exp(-exp(A_log[h]) * softplus(raw + dt_bias[h])) (DECAY_HEAD_TOKEN);
//               one number per key channel and token, sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau) (DECAY_CHANNEL)
//   write u_t   the value v_t; or, with the delta rule, beta_t (v_t - S^T k_t) with S already decayed and
//               beta_t = sigmoid(raw), so that the read-out sees the corrected state
//   q, k        as projected (QK_PLAIN); the first rot_dims coordinates of every head turned by the step's
//               cosine/sine table, coordinate i with i + rot_dims/2 (QK_ROTATE); or made unit vectors,
//               x / sqrt(sum x^2 + unit_eps) (QK_UNIT).  Several value heads may share a query/key head.
//
// and the kernel that finishes a head's read-out: RMS over the head (a weight per coordinate or none), times
// silu(gate), times a constant, rounded to the activation type for the output projection.
//
// Everything is 32-bit: inputs are 32-bit sums of the projections, decays, exponentials, the state, the
// read-out and the norm.  A sequence's rows are found through seq_start, its state row through
// state_slots; a portion whose first row has position 0 starts from zeros.  Nothing is decided on the
// host, so a step of these kernels can be replayed from a CUDA graph.
#include "common.cuh"

#define LA_PER_MAX 16            // state entries per thread at most
#define LA_CHUNK 16              // tokens staged at a time
#define DECAY_HEAD_CONST 0
#define DECAY_HEAD_TOKEN 1
#define DECAY_CHANNEL 2
#define QK_PLAIN 0
#define QK_ROTATE 1
#define QK_UNIT 2

__device__ __forceinline__ float la_softplus(float v) { return v > 20.0f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float la_silu(float v) { return v / (1.0f + expf(-v)); }

__device__ __forceinline__ void la_copy4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void la_copy16(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
struct LaScanArgs {
    float* q; long long ld_q;                  // head g of row t: q[t * ld_q + g * D + d]; made ready in place
    float* k; long long ld_k;
    const float* v; long long ld_v;            // head h of row t: v[t * ld_v + h * V + c]
    float* decay_channel; long long ld_dc;     // DECAY_CHANNEL: z[t * ld_dc + h * D + d], becomes the decay in place
    float* decay_head; long long ld_dh;        // DECAY_HEAD_TOKEN: raw[t * ld_dh + h], becomes the decay in place
    const float* decay_const;                  // DECAY_HEAD_CONST: the decay [heads]; DECAY_HEAD_TOKEN: A_log [heads]
    const float* dt_bias;                      // DECAY_HEAD_TOKEN: [heads] or null
    float* beta; long long ld_beta;            // raw[t * ld_beta + h], becomes sigmoid in place; null: no delta rule
    const float* cos_sin; int rot_dims;        // QK_ROTATE: [T, rot_dims / 2, 2]
    float* state; long long state_stride;      // [slots][heads][D][V]
    const int* seq_start; const int* positions; const int* state_slots;
    float* y; long long ld_y;                  // y[t * ld_y + h * V + c]
    int T, heads, qk_heads, D, V, NP, cols, decay_mode, qk_mode, vec;
    float inv_tau, unit_eps, out_scale;
};

// What has to happen to a step's rows before the recurrence reads them, once per row and in place (the
// recurrence's CTAs share a head's queries and keys, so none of this belongs into them): one warp per
// (row, unit) with the units of a row being its query heads, its key heads (rotation or unit vectors), its heads'
// channel decays (exp(-softplus(-z) / tau)) and one unit for the numbers per head (decay and sigmoid(beta)).
__global__ void __launch_bounds__(128) la_prepare_kernel(const LaScanArgs A) {
    ap_pdl_trigger();
    ap_pdl_wait();
    const int lane = threadIdx.x & 31;
    const int G = A.qk_heads, H = A.heads, D = A.D;
    const int qk_units = A.qk_mode == QK_PLAIN ? 0 : 2 * G;
    const int ch_units = A.decay_mode == DECAY_CHANNEL ? H : 0;
    const int sc_units = (A.decay_mode == DECAY_HEAD_TOKEN || A.beta != nullptr) ? 1 : 0;
    const int units = qk_units + ch_units + sc_units;
    const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (unit >= (long long)A.T * units) return;
    const int t = (int)(unit / units);
    int u = (int)(unit % units);
    if (u < qk_units) {
        float* p = u < G ? A.q + (size_t)t * A.ld_q + (size_t)u * D : A.k + (size_t)t * A.ld_k + (size_t)(u - G) * D;
        if (A.qk_mode == QK_ROTATE) {
            const int half = A.rot_dims / 2;
            for (int j = lane; j < half; j += 32) {
                const float2 cs = *reinterpret_cast<const float2*>(A.cos_sin + ((size_t)t * half + j) * 2);
                const float a = p[j], b = p[j + half];
                p[j] = a * cs.x - b * cs.y;
                p[j + half] = b * cs.x + a * cs.y;
            }
        } else {
            float ss = 0.f;
            for (int d = lane; d < D; d += 32) ss = fmaf(p[d], p[d], ss);
            ss = ap_warp_sum(ss);
            const float f = 1.0f / sqrtf(ss + A.unit_eps);
            for (int d = lane; d < D; d += 32) p[d] *= f;
        }
        return;
    }
    u -= qk_units;
    if (u < ch_units) {
        float* z = A.decay_channel + (size_t)t * A.ld_dc + (size_t)u * D;
        for (int d = lane; d < D; d += 32) z[d] = expf(-la_softplus(-z[d]) * A.inv_tau);
        return;
    }
    for (int h = lane; h < H; h += 32) {
        if (A.decay_mode == DECAY_HEAD_TOKEN) {
            float* a = A.decay_head + (size_t)t * A.ld_dh + h;
            *a = expf(-expf(A.decay_const[h]) * la_softplus(*a + (A.dt_bias ? A.dt_bias[h] : 0.f)));
        }
        if (A.beta) {
            float* b = A.beta + (size_t)t * A.ld_beta + h;
            *b = 1.0f / (1.0f + expf(-*b));
        }
    }
}

// One CTA per (sequence, head, block of value columns).  A thread holds PER state entries of one value
// column: the column's D entries are dealt to NP neighbouring lanes (a power of two up to 32) in runs of four
// (entry i of lane p is row (i / 4) * 4 NP + 4 p + i % 4, so that the lanes' 16-byte reads of a key lie side by
// side in shared memory), and the lanes' partial sums meet by shuffles.  Few lanes with many entries each keep the
// instructions per state entry low: a row costs a thread three operations per entry and one short reduction
// (two with the delta rule).  Tokens come LA_CHUNK at a time through two shared-memory buffers filled by
// asynchronous copies while the chunk before is computed.
template <int PER, int NP>
__global__ void __launch_bounds__(128) la_scan_kernel(const LaScanArgs A) {
    extern __shared__ __align__(16) float sm[];
    ap_pdl_trigger();
    ap_pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y;
    const int a = A.seq_start[s], n = A.seq_start[s + 1] - a;
    if (n <= 0) return;
    const int D = A.D, V = A.V, cols = A.cols;
    const int g = h / (A.heads / A.qk_heads);
    const int col0 = blockIdx.z * cols;
    const int ncols = min(cols, V - col0);
    const int vl = threadIdx.x / NP, part = threadIdx.x % NP;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int vcol = col0 + vl;
    const bool live = vl < ncols;
    const bool channel = A.decay_mode == DECAY_CHANNEL, delta = A.beta != nullptr;
    const bool token_decay = A.decay_mode == DECAY_HEAD_TOKEN;
    const int XS = (cols + 3) / 4 * 4, DS = PER * NP;        // a row of keys in shared memory is padded with zeros
    // one buffer: v [CHUNK][XS], k [CHUNK][DS], q [CHUNK][DS], channel decays [CHUNK][DS] (if any), decay [CHUNK], beta [CHUNK]
    const int buf_floats = LA_CHUNK * (XS + (channel ? 3 : 2) * DS) + 2 * LA_CHUNK;
    if (DS > D) {
        // the rows' tails beyond D stay zero for good (the copies write the first D numbers only)
        const int pad = DS - D, per_buf = (channel ? 3 : 2) * LA_CHUNK;
        for (int i = threadIdx.x; i < 2 * per_buf * pad; i += blockDim.x) {
            const int b = i / (per_buf * pad), j = i - b * per_buf * pad;
            sm[b * buf_floats + LA_CHUNK * XS + (j / pad) * DS + D + j % pad] = 0.f;
        }
    }
    float* st = A.state + (size_t)A.state_slots[s] * A.state_stride + (size_t)h * D * V;
    const bool fresh = A.positions[a] == 0;
    float S[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int nn = (i >> 2) * 4 * NP + 4 * part + (i & 3);
        S[i] = (!fresh && live && nn < D) ? st[(size_t)nn * V + vcol] : 0.f;
    }
    const float head_decay = A.decay_mode == DECAY_HEAD_CONST ? A.decay_const[h] : 1.0f;
    const bool vec = A.vec != 0;
    __syncthreads();

    auto stage = [&](int t0, float* buf) {
        const int cnt = min(LA_CHUNK, n - t0);
        float* v_b = buf;
        float* k_b = v_b + LA_CHUNK * XS;
        float* q_b = k_b + LA_CHUNK * DS;
        float* c_b = q_b + LA_CHUNK * DS;
        float* sc_b = c_b + (channel ? LA_CHUNK * DS : 0);
        const size_t row = (size_t)(a + t0);
        // values: eight threads to a row; keys, queries and channel decays: a warp to a row, the lanes across it
        for (int r = threadIdx.x >> 3; r < cnt; r += blockDim.x >> 3) {
            const float* src = A.v + (row + r) * A.ld_v + (size_t)h * V + col0;
            if (vec && ncols % 4 == 0) for (int d = (threadIdx.x & 7) * 4; d < ncols; d += 32) la_copy16(v_b + r * XS + d, src + d);
            else for (int d = threadIdx.x & 7; d < ncols; d += 8) la_copy4(v_b + r * XS + d, src + d);
        }
        for (int r = warp; r < cnt; r += nwarps) {
            const float* ks = A.k + (row + r) * A.ld_k + (size_t)g * D;
            const float* qs = A.q + (row + r) * A.ld_q + (size_t)g * D;
            const float* cs = channel ? A.decay_channel + (row + r) * A.ld_dc + (size_t)h * D : nullptr;
            if (vec) {
                for (int d = lane * 4; d < D; d += 128) {
                    la_copy16(k_b + r * DS + d, ks + d);
                    la_copy16(q_b + r * DS + d, qs + d);
                    if (channel) la_copy16(c_b + r * DS + d, cs + d);
                }
            } else {
                for (int d = lane; d < D; d += 32) {
                    la_copy4(k_b + r * DS + d, ks + d);
                    la_copy4(q_b + r * DS + d, qs + d);
                    if (channel) la_copy4(c_b + r * DS + d, cs + d);
                }
            }
        }
        if ((int)threadIdx.x < cnt) {
            if (token_decay) la_copy4(sc_b + threadIdx.x, A.decay_head + (row + threadIdx.x) * A.ld_dh + h);
            if (delta) la_copy4(sc_b + LA_CHUNK + threadIdx.x, A.beta + (row + threadIdx.x) * A.ld_beta + h);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    stage(0, sm);
    int which_buf = 0;
    for (int t0 = 0; t0 < n; t0 += LA_CHUNK, which_buf ^= 1) {
        const int cnt = min(LA_CHUNK, n - t0);
        float* buf = sm + which_buf * buf_floats;
        if (t0 + LA_CHUNK < n) {
            stage(t0 + LA_CHUNK, sm + (which_buf ^ 1) * buf_floats);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* v_s = buf;
        const float* k_s = v_s + LA_CHUNK * XS + 4 * part;
        const float* q_s = k_s + LA_CHUNK * DS;
        const float* c_s = q_s + LA_CHUNK * DS;
        const float* sc_s = buf + LA_CHUNK * (XS + (channel ? 3 : 2) * DS);
        float* yp = A.y + (size_t)(a + t0) * A.ld_y + (size_t)h * V + vcol;
#pragma unroll 2
        for (int r = 0; r < cnt; ++r, yp += A.ld_y) {
            const float vv = live ? v_s[r * XS + vl] : 0.f;
            float kk[PER], qq[PER];
#pragma unroll
            for (int j = 0; j < PER / 4; ++j) {
                *reinterpret_cast<float4*>(kk + 4 * j) = *reinterpret_cast<const float4*>(k_s + r * DS + j * 4 * NP);
                *reinterpret_cast<float4*>(qq + 4 * j) = *reinterpret_cast<const float4*>(q_s + r * DS + j * 4 * NP);
            }
            if (channel) {
#pragma unroll
                for (int j = 0; j < PER / 4; ++j) {
                    const float4 c = *reinterpret_cast<const float4*>(c_s + r * DS + j * 4 * NP);
                    S[4 * j] *= c.x; S[4 * j + 1] *= c.y; S[4 * j + 2] *= c.z; S[4 * j + 3] *= c.w;
                }
            } else {
                const float dec = token_decay ? sc_s[r] : head_decay;
#pragma unroll
                for (int i = 0; i < PER; ++i) S[i] *= dec;
            }
            float u = vv;
            if (delta) {
                float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
                for (int j = 0; j < PER / 4; ++j) {
                    d0 = fmaf(S[4 * j], kk[4 * j], d0); d1 = fmaf(S[4 * j + 1], kk[4 * j + 1], d1);
                    d2 = fmaf(S[4 * j + 2], kk[4 * j + 2], d2); d3 = fmaf(S[4 * j + 3], kk[4 * j + 3], d3);
                }
                float dot = (d0 + d1) + (d2 + d3);
#pragma unroll
                for (int o = NP >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                u = sc_s[LA_CHUNK + r] * (vv - dot);
            }
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int j = 0; j < PER / 4; ++j) {
                S[4 * j] = fmaf(kk[4 * j], u, S[4 * j]); a0 = fmaf(S[4 * j], qq[4 * j], a0);
                S[4 * j + 1] = fmaf(kk[4 * j + 1], u, S[4 * j + 1]); a1 = fmaf(S[4 * j + 1], qq[4 * j + 1], a1);
                S[4 * j + 2] = fmaf(kk[4 * j + 2], u, S[4 * j + 2]); a2 = fmaf(S[4 * j + 2], qq[4 * j + 2], a2);
                S[4 * j + 3] = fmaf(kk[4 * j + 3], u, S[4 * j + 3]); a3 = fmaf(S[4 * j + 3], qq[4 * j + 3], a3);
            }
            float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
            for (int o = NP >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && part == 0) *yp = acc * A.out_scale;
        }
        __syncthreads();                                     // this buffer is filled again two chunks on
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int nn = (i >> 2) * 4 * NP + 4 * part + (i & 3);
            if (nn < D) st[(size_t)nn * V + vcol] = S[i];
        }
    }
}

AP_EXPORT int ap_linear_scan(float* q, long long ld_q, float* k, long long ld_k, const float* v,
                             long long ld_v, float* decay_channel, long long ld_dc, float* decay_head,
                             long long ld_dh, const float* decay_const, const float* dt_bias, float* beta,
                             long long ld_beta, const float* cos_sin, int rot_dims, float* state,
                             long long state_stride, const int* seq_start, const int* positions,
                             const int* state_slots, float* y, long long ld_y, int T, int nseq, int heads,
                             int qk_heads, int D, int V, int decay_mode, int qk_mode, float tau, float unit_eps,
                             float out_scale, cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && nseq >= 0 && heads > 0 && qk_heads > 0 && heads % qk_heads == 0 && D > 0 && V > 0,
               "linear_scan: bad sizes heads=%d qk_heads=%d key=%d value=%d", heads, qk_heads, D, V);
    AP_REQUIRE(D <= LA_PER_MAX * 32, "linear_scan: keys of %d exceed %d", D, LA_PER_MAX * 32);
    AP_REQUIRE(q && k && v && y && state && state_stride >= (long long)heads * D * V,
               "linear_scan: an operand is missing or the state is too small");
    AP_REQUIRE(decay_mode == DECAY_HEAD_CONST ? decay_const != nullptr
               : decay_mode == DECAY_HEAD_TOKEN ? (decay_head != nullptr && decay_const != nullptr)
               : (decay_mode == DECAY_CHANNEL && decay_channel != nullptr && tau > 0.f),
               "linear_scan: decay mode %d lacks its numbers", decay_mode);
    AP_REQUIRE(qk_mode == QK_PLAIN || qk_mode == QK_UNIT ||
               (qk_mode == QK_ROTATE && cos_sin && rot_dims > 0 && rot_dims % 2 == 0 && rot_dims <= D),
               "linear_scan: query/key mode %d with %d rotated coordinates of %d", qk_mode, rot_dims, D);
    if (T == 0 || nseq == 0) return AP_OK;
    // as few lanes to a column as hold it (up to 16 entries a thread: the fewest instructions per state entry);
    // more of them (shorter chains per thread, more warps) only while the step's columns leave schedulers without
    // a warp (measured: with four warps to a scheduler and four entries a thread the longer reductions cost more
    // than the other warps hide, 733 -> 797 us for 2048 tokens of the delta rule on 16 heads of 128 x 128)
    int NP = 1;
    while (NP * LA_PER_MAX < D) NP *= 2;
    while (NP < 32 && NP * 4 < D && (long long)nseq * heads * V * NP / 32 < 148 * 4) NP *= 2;
    const int per = ((D + NP - 1) / NP + 3) / 4 * 4;
    int cols = 128 / NP;
    if (cols > V) cols = V;
    int threads = (cols * NP + 31) / 32 * 32;
    cols = threads / NP;
    if (cols >= 4) cols = cols / 4 * 4;                     // whole 16-byte runs of the values per CTA
    if (cols > V) cols = V;
    const dim3 grid((unsigned)nseq, (unsigned)heads, (unsigned)((V + cols - 1) / cols));
    AP_REQUIRE(heads <= 65535 && grid.z <= 65535, "linear_scan: %d heads exceed the grid", heads);
    auto aligned = [](const void* p, long long ld) { return p == nullptr || ((((uintptr_t)p) & 15) == 0 && ld % 4 == 0); };
    const int vec = (D % 4 == 0 && V % 4 == 0 && cols % 4 == 0 && aligned(q, ld_q) && aligned(k, ld_k) &&
                     aligned(v, ld_v) && aligned(decay_channel, ld_dc)) ? 1 : 0;
    const bool channel = decay_mode == DECAY_CHANNEL;
    LaScanArgs A;
    A.q = q; A.ld_q = ld_q; A.k = k; A.ld_k = ld_k; A.v = v; A.ld_v = ld_v;
    A.decay_channel = decay_channel; A.ld_dc = ld_dc; A.decay_head = decay_head; A.ld_dh = ld_dh;
    A.decay_const = decay_const; A.dt_bias = dt_bias; A.beta = beta; A.ld_beta = ld_beta;
    A.cos_sin = cos_sin; A.rot_dims = rot_dims; A.state = state; A.state_stride = state_stride;
    A.seq_start = seq_start; A.positions = positions; A.state_slots = state_slots; A.y = y; A.ld_y = ld_y;
    A.T = T; A.heads = heads; A.qk_heads = qk_heads; A.D = D; A.V = V; A.NP = NP; A.cols = cols;
    A.decay_mode = decay_mode; A.qk_mode = qk_mode; A.vec = vec;
    A.inv_tau = channel ? 1.0f / tau : 0.f; A.unit_eps = unit_eps; A.out_scale = out_scale;
    const int units = (qk_mode == QK_PLAIN ? 0 : 2 * qk_heads) + (channel ? heads : 0) +
                      ((decay_mode == DECAY_HEAD_TOKEN || beta != nullptr) ? 1 : 0);
    if (units > 0) {
        const long long blocks = ((long long)T * units + 3) / 4;
        AP_CHECK_PDL_LAUNCH("linear_scan (rows made ready)",
                            ap_launch_pdl(la_prepare_kernel, dim3((unsigned)blocks), dim3(128), 0, stream, A));
    }
    const int per_built = per <= 4 ? 4 : (per <= 8 ? 8 : LA_PER_MAX);
    const size_t smem = 2 * ((size_t)LA_CHUNK * ((cols + 3) / 4 * 4 + (channel ? 3 : 2) * (per_built * NP)) + 2 * LA_CHUNK) *
                        sizeof(float);
    void (*kern)(const LaScanArgs) = nullptr;
#define LA_PICK(P)                                                                                     \
    if (per_built == P)                                                                                \
        kern = NP == 1 ? la_scan_kernel<P, 1> : NP == 2 ? la_scan_kernel<P, 2> : NP == 4 ? la_scan_kernel<P, 4> \
             : NP == 8 ? la_scan_kernel<P, 8> : NP == 16 ? la_scan_kernel<P, 16> : la_scan_kernel<P, 32>;
    LA_PICK(4) LA_PICK(8) LA_PICK(LA_PER_MAX)
#undef LA_PICK
    if (smem > 48 * 1024) {
        AP_REQUIRE(smem <= 200 * 1024, "linear_scan: keys of %d do not fit the staging buffers", D);
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        AP_REQUIRE(e == cudaSuccess, "linear_scan: cannot reserve %zu bytes of shared memory", smem);
    }
    AP_CHECK_PDL_LAUNCH("linear_scan", ap_launch_pdl(kern, grid, dim3(threads), smem, stream, A));
    return AP_OK;
}

// ---- a head's read-out: RMS norm, gate, constant ------------------------------------------
// y: [T, ld_y] 32-bit, head h at column h * V; gate: [T, ld_g] 32-bit raw, same layout; one warp per (row, head).
template <typename TO>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ y, long long ld_y, const float* __restrict__ gate, long long ld_g,
                      const float* __restrict__ w, float eps, float out_scale, TO* __restrict__ out, int T, int heads,
                      int V) {
    ap_pdl_trigger();
    ap_pdl_wait();
    const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (unit >= (long long)T * heads) return;
    const int lane = threadIdx.x & 31;
    const int t = (int)(unit / heads), h = (int)(unit % heads);
    const float* yr = y + (size_t)t * ld_y + (size_t)h * V;
    const float* gr = gate + (size_t)t * ld_g + (size_t)h * V;
    float ss = 0.f;
    for (int i = lane; i < V; i += 32) ss = fmaf(yr[i], yr[i], ss);
    ss = ap_warp_sum(ss);
    const float inv = out_scale / sqrtf(ss / (float)V + eps);
    TO* o = out + ((size_t)t * heads + h) * V;
    for (int i = lane; i < V; i += 32)
        o[i] = ap_from_float<TO>(yr[i] * inv * (w ? w[i] : 1.0f) * la_silu(gr[i]));
}

AP_EXPORT int ap_head_norm_gate(const float* y, long long ld_y, const float* gate, long long ld_g, const float* w,
                                float eps, float out_scale, void* out, int out_dtype, int T, int heads, int V,
                                cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && heads > 0 && V > 0 && ld_y >= (long long)heads * V && ld_g >= (long long)heads * V,
               "head_norm_gate: bad sizes heads=%d value=%d", heads, V);
    if (T == 0) return AP_OK;
    const dim3 grid((unsigned)(((long long)T * heads + 3) / 4));
#define LAUNCH(TO)                                                                                                  \
    AP_CHECK_PDL_LAUNCH("head_norm_gate", ap_launch_pdl(head_norm_gate_kernel<TO>, grid, dim3(128), 0, stream, y,   \
                                                        ld_y, gate, ld_g, w, eps, out_scale, (TO*)out, T, heads, V))
    if (out_dtype == AP_F32) LAUNCH(float);
    else if (out_dtype == AP_BF16) LAUNCH(bf16);
    else AP_REQUIRE(false, "head_norm_gate: unknown dtype %d", out_dtype);
#undef LAUNCH
    return AP_OK;
}
