// Kernels that act on the residual stream element by element, for decoders whose norms need no
// statistics of a row:
//
//   add_dyt       v = x + sum_s delta[s];  out = tanh(alpha v) * w + b          (Dynamic Tanh: a norm
//                 without mean or variance; alpha is one number for the whole vector)
//   dyt_shift     the same norm, followed by a mix with the PREVIOUS token's normed row:
//                   n_t = tanh(alpha x_t) * w + b;   out_t = n_t + (n_{t-1} - n_t) * shift
//                 n_{-1} = 0; the row before a portion's first row is the request's state, which the
//                 kernel brings up to date with the portion's last row
//   stream_mix    depth-weighted average over the outputs of all layers so far:
//                   v = x + sum_s delta[s];  streams[k] = v;  x = sum_{j <= k} a[j] streams[j]
//   bias_act      out = act(in + bias) for a product that left 32-bit (or 16-bit) sums
//
// Everything is 32-bit up to the store of `out`.  The kernels are grid-stride loops over
// elements (four at a time where the width and the addresses allow); none reads a statistic of
// a row, so a row's result cannot depend on what else the step holds.
#include "common.cuh"

#define STREAM_THREADS 256
#define STREAM_MAX_BLOCKS (148 * 16)

__device__ __forceinline__ float dyt_value(float v, float alpha, float w, float b) { return fmaf(tanhf(alpha * v), w, b); }

static inline unsigned stream_blocks(size_t n) {
    size_t blocks = (n + STREAM_THREADS - 1) / STREAM_THREADS;
    if (blocks > STREAM_MAX_BLOCKS) blocks = STREAM_MAX_BLOCKS;
    return (unsigned)(blocks ? blocks : 1);
}

template <typename TO> struct Out4;
template <> struct Out4<float> {
    static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) {
        *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    }
};
template <> struct Out4<bf16> {
    static __device__ __forceinline__ void store(bf16* p, float a, float b, float c, float d) {
        uint2 v;
        *reinterpret_cast<__nv_bfloat162*>(&v.x) = __floats2bfloat162_rn(a, b);
        *reinterpret_cast<__nv_bfloat162*>(&v.y) = __floats2bfloat162_rn(c, d);
        *reinterpret_cast<uint2*>(p) = v;
    }
};

// ---- Dynamic Tanh with the pending addition ---------------------------------------------
template <typename TO, int VEC>
__global__ void __launch_bounds__(STREAM_THREADS)
add_dyt_kernel(float* __restrict__ x, const float* __restrict__ delta, int S, size_t delta_stride,
               const float* __restrict__ w, const float* __restrict__ b, float alpha, TO* __restrict__ out,
               const int* __restrict__ rows, int R, int H) {
    ap_pdl_trigger();
    ap_pdl_wait();
    const int HV = H / VEC;
    const size_t n = (size_t)R * HV;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / HV;
        const int c = (int)(e - r * HV) * VEC;
        const size_t t = rows ? (size_t)rows[r] : r;
        const size_t at = t * H + c;
        float v[VEC];
        if (VEC == 4) {
            const float4 a = *reinterpret_cast<const float4*>(x + at);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            for (int s = 0; s < S; ++s) {
                const float4 d = *reinterpret_cast<const float4*>(delta + (size_t)s * delta_stride + at);
                v[0] += d.x; v[1] += d.y; v[2] += d.z; v[3] += d.w;
            }
            if (!rows && S > 0) *reinterpret_cast<float4*>(x + at) = make_float4(v[0], v[1], v[2], v[3]);
            Out4<TO>::store(out + r * H + c, dyt_value(v[0], alpha, w[c], b[c]), dyt_value(v[1], alpha, w[c + 1], b[c + 1]),
                            dyt_value(v[2], alpha, w[c + 2], b[c + 2]), dyt_value(v[3], alpha, w[c + 3], b[c + 3]));
        } else {
            v[0] = x[at];
            for (int s = 0; s < S; ++s) v[0] += delta[(size_t)s * delta_stride + at];
            if (!rows && S > 0) x[at] = v[0];
            out[r * H + c] = ap_from_float<TO>(dyt_value(v[0], alpha, w[c], b[c]));
        }
    }
}

AP_EXPORT int ap_add_dyt(float* x, const float* delta, int S, long long delta_stride, const float* w, const float* b,
                         float alpha, void* out, int out_dtype, const int* rows, int R, int H, cudaStream_t stream) {
    AP_REQUIRE(R >= 0 && H > 0 && S >= 0 && x && w && b && out, "add_dyt: bad arguments R=%d H=%d S=%d", R, H, S);
    AP_REQUIRE(S == 0 || delta != nullptr, "add_dyt: S=%d partial sums but no buffer", S);
    if (R == 0) return AP_OK;
    const bool vec = H % 4 == 0 && ((((uintptr_t)x) | ((uintptr_t)delta) | ((uintptr_t)w) | ((uintptr_t)b)) & 15) == 0 &&
                     delta_stride % 4 == 0 && (((uintptr_t)out) & (out_dtype == AP_F32 ? 15 : 7)) == 0;
    const unsigned blocks = stream_blocks((size_t)R * (vec ? H / 4 : H));
#define LAUNCH(TO, V)                                                                                               \
    AP_CHECK_PDL_LAUNCH("add_dyt", ap_launch_pdl(add_dyt_kernel<TO, V>, dim3(blocks), dim3(STREAM_THREADS), 0, stream, x, \
                                                 delta, S, (size_t)delta_stride, w, b, alpha, (TO*)out, rows, R, H))
    if (out_dtype == AP_F32) { if (vec) LAUNCH(float, 4); else LAUNCH(float, 1); }
    else if (out_dtype == AP_BF16) { if (vec) LAUNCH(bf16, 4); else LAUNCH(bf16, 1); }
    else AP_REQUIRE(false, "add_dyt: unknown dtype %d", out_dtype);
#undef LAUNCH
    return AP_OK;
}

// ---- Dynamic Tanh, then the mix with the previous token's normed row ---------------------
// The thread of a portion's FIRST row reads the request's state and then writes the portion's
// last normed row there (computing it, where the portion has more rows than one): the same
// thread reads and writes an entry, so no other thread's read can come after the write.
// A thread takes VEC columns of ROWS consecutive rows and carries a row's normed values on to the next
// row as its `previous`, so that a step of many rows computes little more than one tanh per entry (one
// more per ROWS rows, for the row before the run); a row's result does not depend on where its run starts.
template <typename TO, int VEC, int ROWS>
__global__ void __launch_bounds__(STREAM_THREADS)
dyt_shift_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, float alpha,
                 const float* __restrict__ shift, float* __restrict__ state, size_t state_stride,
                 const int* __restrict__ seq_start, const int* __restrict__ positions, const int* __restrict__ token_seq,
                 const int* __restrict__ state_slots, TO* __restrict__ out, int T, int H) {
    ap_pdl_trigger();
    ap_pdl_wait();
    const int HV = H / VEC;
    const size_t runs = ((size_t)T + ROWS - 1) / ROWS;
    const size_t n = runs * HV;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t run = e / HV;
        const int c = (int)(e - run * HV) * VEC;
        float wc[VEC], bc[VEC], sc[VEC], cur[VEC], prev[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) { wc[i] = w[c + i]; bc[i] = b[c + i]; sc[i] = shift[c + i]; }
        const size_t t0 = run * ROWS;
        // the run's rows are fetched before any is worked on, so that their latencies overlap
        float xin[ROWS][VEC];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            if (t0 + r < (size_t)T) {
                if (VEC == 4) {
                    const float4 q = *reinterpret_cast<const float4*>(x + (t0 + r) * H + c);
                    xin[r][0] = q.x; xin[r][1] = q.y; xin[r][2] = q.z; xin[r][3] = q.w;
                } else {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) xin[r][i] = x[(t0 + r) * H + c + i];
                }
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const size_t t = t0 + r;
            if (t >= (size_t)T) break;
            const int s = token_seq[t];
            const int first = seq_start[s];
            if (r > 0) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) prev[i] = cur[i];      // row t - 1, normed: used unless t starts a portion
            }
#pragma unroll
            for (int i = 0; i < VEC; ++i) cur[i] = dyt_value(xin[r][i], alpha, wc[i], bc[i]);
            if ((int)t == first) {
                float* st = state + (size_t)state_slots[s] * state_stride + c;
                const bool fresh = positions[t] == 0;
                const size_t last = (size_t)seq_start[s + 1] - 1;
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    prev[i] = fresh ? 0.f : st[i];
                    st[i] = last == t ? cur[i] : dyt_value(x[last * H + c + i], alpha, wc[i], bc[i]);
                }
            } else if (r == 0) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) prev[i] = dyt_value(x[(t - 1) * H + c + i], alpha, wc[i], bc[i]);
            }
            float o[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) o[i] = cur[i] + (prev[i] - cur[i]) * sc[i];
            if (VEC == 4) Out4<TO>::store(out + t * H + c, o[0], o[1], o[2], o[3]);
            else out[t * H + c] = ap_from_float<TO>(o[0]);
        }
    }
}

AP_EXPORT int ap_dyt_shift(const float* x, const float* w, const float* b, float alpha, const float* shift, float* state,
                           long long state_stride, const int* seq_start, const int* positions, const int* token_seq,
                           const int* state_slots, void* out, int out_dtype, int T, int H, cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && H > 0 && x && w && b && shift && state && out, "dyt_shift: bad arguments T=%d H=%d", T, H);
    AP_REQUIRE(seq_start && positions && token_seq && state_slots && state_stride >= H,
               "dyt_shift: the step's metadata or the state rows are missing");
    if (T == 0) return AP_OK;
    const bool vec = H % 4 == 0 && state_stride % 4 == 0 && (((uintptr_t)x) & 15) == 0 &&
                     (((uintptr_t)out) & (out_dtype == AP_F32 ? 15 : 7)) == 0;
    // runs of four rows once that still leaves every SM several CTAs
    const bool runs4 = (size_t)T * (vec ? H / 4 : H) >= (size_t)4 * 4 * 148 * STREAM_THREADS;
    const size_t rows = runs4 ? ((size_t)T + 3) / 4 : (size_t)T;
    const unsigned blocks = stream_blocks(rows * (vec ? H / 4 : H));
#define LAUNCH(TO, V, R)                                                                                            \
    AP_CHECK_PDL_LAUNCH("dyt_shift", ap_launch_pdl(dyt_shift_kernel<TO, V, R>, dim3(blocks), dim3(STREAM_THREADS), 0, stream, \
                                                   x, w, b, alpha, shift, state, (size_t)state_stride, seq_start,    \
                                                   positions, token_seq, state_slots, (TO*)out, T, H))
#define LAUNCH_V(TO, V) do { if (runs4) LAUNCH(TO, V, 4); else LAUNCH(TO, V, 1); } while (0)
    if (out_dtype == AP_F32) { if (vec) LAUNCH_V(float, 4); else LAUNCH_V(float, 1); }
    else if (out_dtype == AP_BF16) { if (vec) LAUNCH_V(bf16, 4); else LAUNCH_V(bf16, 1); }
    else AP_REQUIRE(false, "dyt_shift: unknown dtype %d", out_dtype);
#undef LAUNCH_V
#undef LAUNCH
    return AP_OK;
}

// ---- depth-weighted average ----------------------------------------------------------------
// streams: [count][n] 32-bit, stream j at streams + j * stream_stride.  The sum runs over j upwards.
template <int VEC>
__global__ void __launch_bounds__(STREAM_THREADS)
stream_mix_kernel(float* __restrict__ x, const float* __restrict__ delta, int S, size_t delta_stride,
                  float* __restrict__ streams, size_t stream_stride, int k, const float* __restrict__ a, size_t n) {
    ap_pdl_trigger();
    ap_pdl_wait();
    for (size_t e = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) * VEC; e < n; e += (size_t)gridDim.x * blockDim.x * VEC) {
        float v[VEC], acc[VEC];
        if (VEC == 4) {
            const float4 q = *reinterpret_cast<const float4*>(x + e);
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
            for (int s = 0; s < S; ++s) {
                const float4 d = *reinterpret_cast<const float4*>(delta + (size_t)s * delta_stride + e);
                v[0] += d.x; v[1] += d.y; v[2] += d.z; v[3] += d.w;
            }
            *reinterpret_cast<float4*>(streams + (size_t)k * stream_stride + e) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
            v[0] = x[e];
            for (int s = 0; s < S; ++s) v[0] += delta[(size_t)s * delta_stride + e];
            streams[(size_t)k * stream_stride + e] = v[0];
        }
        if (a == nullptr) {
            if (S > 0) {
                if (VEC == 4) *reinterpret_cast<float4*>(x + e) = make_float4(v[0], v[1], v[2], v[3]);
                else x[e] = v[0];
            }
            continue;
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
        for (int j = 0; j < k; ++j) {
            const float aj = a[j];
            if (VEC == 4) {
                const float4 q = *reinterpret_cast<const float4*>(streams + (size_t)j * stream_stride + e);
                acc[0] = fmaf(aj, q.x, acc[0]); acc[1] = fmaf(aj, q.y, acc[1]);
                acc[2] = fmaf(aj, q.z, acc[2]); acc[3] = fmaf(aj, q.w, acc[3]);
            } else {
                acc[0] = fmaf(aj, streams[(size_t)j * stream_stride + e], acc[0]);
            }
        }
        const float ak = a[k];
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = fmaf(ak, v[i], acc[i]);
        if (VEC == 4) *reinterpret_cast<float4*>(x + e) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        else x[e] = acc[0];
    }
}

AP_EXPORT int ap_stream_mix(float* x, const float* delta, int S, long long delta_stride, float* streams,
                            long long stream_stride, int k, const float* a, long long n, cudaStream_t stream) {
    AP_REQUIRE(n >= 0 && S >= 0 && k >= 0 && x && streams && stream_stride >= n, "stream_mix: bad arguments k=%d S=%d", k, S);
    AP_REQUIRE(S == 0 || delta != nullptr, "stream_mix: S=%d partial sums but no buffer", S);
    if (n == 0) return AP_OK;
    const bool vec = n % 4 == 0 && stream_stride % 4 == 0 && delta_stride % 4 == 0 &&
                     ((((uintptr_t)x) | ((uintptr_t)delta) | ((uintptr_t)streams)) & 15) == 0;
    const unsigned blocks = stream_blocks(vec ? (size_t)n / 4 : (size_t)n);
    if (vec)
        AP_CHECK_PDL_LAUNCH("stream_mix", ap_launch_pdl(stream_mix_kernel<4>, dim3(blocks), dim3(STREAM_THREADS), 0, stream, x,
                                                        delta, S, (size_t)delta_stride, streams, (size_t)stream_stride, k, a,
                                                        (size_t)n));
    else
        AP_CHECK_PDL_LAUNCH("stream_mix", ap_launch_pdl(stream_mix_kernel<1>, dim3(blocks), dim3(STREAM_THREADS), 0, stream, x,
                                                        delta, S, (size_t)delta_stride, streams, (size_t)stream_stride, k, a,
                                                        (size_t)n));
    return AP_OK;
}

// ---- bias and activation behind a product ----------------------------------------------------
#define BACT_NONE 0
#define BACT_RELU 1
#define BACT_RELU2 2         // the square of relu
#define BACT_GELU_TANH 3
#define BACT_SILU 4

__device__ __forceinline__ float bias_activation(float z, int act) {
    switch (act) {
        case BACT_RELU: return fmaxf(z, 0.f);
        case BACT_RELU2: { const float r = fmaxf(z, 0.f); return r * r; }
        case BACT_GELU_TANH: return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        case BACT_SILU: return z / (1.0f + expf(-z));
        default: return z;
    }
}

// 32-bit sums, four columns at a time (N a multiple of 4, addresses aligned)
template <typename TO>
__global__ void __launch_bounds__(STREAM_THREADS)
bias_act4_kernel(const float* __restrict__ in, const float* __restrict__ bias, TO* __restrict__ out, size_t n4, int N4, int act) {
    ap_pdl_trigger();
    ap_pdl_wait();
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < n4; e += (size_t)gridDim.x * blockDim.x) {
        float4 z = reinterpret_cast<const float4*>(in)[e];
        if (bias) {
            const float4 q = reinterpret_cast<const float4*>(bias)[e % N4];
            z.x += q.x; z.y += q.y; z.z += q.z; z.w += q.w;
        }
        Out4<TO>::store(out + e * 4, bias_activation(z.x, act), bias_activation(z.y, act), bias_activation(z.z, act),
                        bias_activation(z.w, act));
    }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(STREAM_THREADS)
bias_act_kernel(const TI* __restrict__ in, const float* __restrict__ bias, TO* __restrict__ out, size_t n, int N, int act) {
    ap_pdl_trigger();
    ap_pdl_wait();
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const float z = ap_to_float(in[e]) + (bias ? bias[e % N] : 0.f);
        out[e] = ap_from_float<TO>(bias_activation(z, act));
    }
}

AP_EXPORT int ap_bias_act(const void* in, int in_dtype, const float* bias, void* out, int out_dtype, int T, int N, int act,
                          cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && N > 0 && in && out && act >= 0 && act <= 4, "bias_act: bad arguments T=%d N=%d act=%d", T, N, act);
    if (T == 0) return AP_OK;
    const size_t n = (size_t)T * N;
    if (in_dtype == AP_F32 && N % 4 == 0 && ((((uintptr_t)in) | ((uintptr_t)bias)) & 15) == 0 &&
        (((uintptr_t)out) & (out_dtype == AP_F32 ? 15 : 7)) == 0 && (out_dtype == AP_F32 || out_dtype == AP_BF16)) {
        const unsigned blocks4 = stream_blocks(n / 4);
        if (out_dtype == AP_F32)
            AP_CHECK_PDL_LAUNCH("bias_act", ap_launch_pdl(bias_act4_kernel<float>, dim3(blocks4), dim3(STREAM_THREADS), 0, stream,
                                                          (const float*)in, bias, (float*)out, n / 4, N / 4, act));
        else
            AP_CHECK_PDL_LAUNCH("bias_act", ap_launch_pdl(bias_act4_kernel<bf16>, dim3(blocks4), dim3(STREAM_THREADS), 0, stream,
                                                          (const float*)in, bias, (bf16*)out, n / 4, N / 4, act));
        return AP_OK;
    }
    const unsigned blocks = stream_blocks(n);
#define LAUNCH(TI, TO)                                                                                              \
    AP_CHECK_PDL_LAUNCH("bias_act", ap_launch_pdl(bias_act_kernel<TI, TO>, dim3(blocks), dim3(STREAM_THREADS), 0, stream, \
                                                  (const TI*)in, bias, (TO*)out, n, N, act))
    if (in_dtype == AP_F32 && out_dtype == AP_F32) LAUNCH(float, float);
    else if (in_dtype == AP_F32 && out_dtype == AP_BF16) LAUNCH(float, bf16);
    else if (in_dtype == AP_BF16 && out_dtype == AP_BF16) LAUNCH(bf16, bf16);
    else AP_REQUIRE(false, "bias_act: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
#undef LAUNCH
    return AP_OK;
}
