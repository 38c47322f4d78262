// The gated delta rule: a recurrent token mixer with a matrix state per head.
//
// Per head (state S [D, V] in FP32, carried from token to token of a request):
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// with q and k unit vectors per head (q also times D^-1/2), g = exp(-exp(A_log) softplus(a + dt_bias))
// and beta = sigmoid(b).  q, k and v first pass a short causal convolution over time per channel
// and silu; the last taps-1 inputs of every channel are part of a request's state.
//
// The step's tokens arrive as ONE fused projection `proj` (FP32 [T, ld]) with the columns
//     [ q: G D | k: G D | v: H V | gate: H V | b: H | a: H ]
// (G heads of q/k, H heads of v; head h reads q/k head h / (H / G)).  A request's state is a flat
// FP32 vector [ S: H D V | history: (taps-1) C ] with C = 2 G D + H V, found through slots[].
//
// Four kernels, all FP32 inside:
//   delta_prepare      per token: convolution + silu, unit norms, beta, decay
//   delta_history      per request: the new last taps-1 inputs (after delta_prepare has read the old)
//   delta_recurrence   per (request, head, 32 value columns): its tokens one after the other
//   delta_gated_norm   per token and head: o / rms(o) * weight * silu(gate)
// Prompt portions and single tokens are the same case; a token's result depends only on its own
// request's state and tokens, in a fixed order of operations, however the step is cut.
#include "common.cuh"

struct DeltaDims {
    int G, H, D, V, taps, ld;  // ld: row stride of proj
    __host__ __device__ int C() const { return 2 * G * D + H * V; }
    __host__ __device__ int gate_off() const { return 2 * G * D + H * V; }
    __host__ __device__ int b_off() const { return 2 * G * D + 2 * H * V; }
    __host__ __device__ int a_off() const { return 2 * G * D + 2 * H * V + H; }
    __host__ __device__ size_t hist_off() const { return (size_t)H * D * V; }
};

__device__ __forceinline__ float dr_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float dr_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float dr_softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// Convolution of channel c at token t: taps inputs ending at this token.  Inputs before the
// portion's first token come from the request's history, zeros before the sequence's start.
__device__ __forceinline__ float dr_conv(const float* __restrict__ proj, const float* __restrict__ conv_w,
                                         const float* __restrict__ hist, const DeltaDims& dm, int t, int in_portion,
                                         int c) {
    float acc = 0.f;
    const int C = dm.C();
    for (int j = 0; j < dm.taps; ++j) {
        const int back = dm.taps - 1 - j;
        float x;
        if (back <= in_portion) x = proj[(size_t)(t - back) * dm.ld + c];
        else x = hist[(size_t)(dm.taps - 1 - (back - in_portion)) * C + c];
        acc = fmaf(conv_w[(size_t)c * dm.taps + j], x, acc);
    }
    return dr_silu(acc);
}

// qkv [T, C]: q (unit, times D^-1/2), k (unit), v after convolution and silu; beta, decay [T, H].
__global__ void delta_prepare_kernel(const float* __restrict__ proj, const float* __restrict__ conv_w,
                                     const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                     const float* __restrict__ state, long long state_stride,
                                     const int* __restrict__ seq_of_token, const int* __restrict__ cu_q,
                                     const int* __restrict__ slots, DeltaDims dm, float* __restrict__ qkv,
                                     float* __restrict__ beta, float* __restrict__ decay) {
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    const int in_portion = t - cu_q[seq];
    const float* hist = state + (size_t)slots[seq] * state_stride + dm.hist_off();
    const int C = dm.C(), lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float* out = qkv + (size_t)t * C;
    // q and k heads: one warp per head, unit norm over its D channels
    for (int u = warp; u < 2 * dm.G; u += nwarps) {
        const int c0 = u * dm.D;
        float ss = 0.f;
        for (int i = lane; i < dm.D; i += 32) {
            const float y = dr_conv(proj, conv_w, hist, dm, t, in_portion, c0 + i);
            out[c0 + i] = y;
            ss += y * y;
        }
        ss = ni_warp_sum(ss);
        float r = 1.0f / sqrtf(ss + 1e-6f);
        if (u < dm.G) r *= 1.0f / sqrtf((float)dm.D);
        for (int i = lane; i < dm.D; i += 32) out[c0 + i] *= r;   // each lane rescales what it wrote itself
    }
    for (int c = 2 * dm.G * dm.D + threadIdx.x; c < C; c += blockDim.x)
        out[c] = dr_conv(proj, conv_w, hist, dm, t, in_portion, c);
    for (int h = threadIdx.x; h < dm.H; h += blockDim.x) {
        const float* row = proj + (size_t)t * dm.ld;
        beta[(size_t)t * dm.H + h] = dr_sigmoid(row[dm.b_off() + h]);
        decay[(size_t)t * dm.H + h] = expf(-expf(a_log[h]) * dr_softplus(row[dm.a_off() + h] + dt_bias[h]));
    }
}

// The request's new history: its last taps-1 inputs.  One thread per channel walks j upwards, so a
// portion shorter than the history shifts the old entries in place (it reads index j + q_len > j).
__global__ void delta_history_kernel(const float* __restrict__ proj, float* __restrict__ state, long long state_stride,
                                     const int* __restrict__ cu_q, const int* __restrict__ slots, DeltaDims dm) {
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int C = dm.C();
    if (c >= C) return;
    const int first = cu_q[seq], q_len = cu_q[seq + 1] - first;
    float* hist = state + (size_t)slots[seq] * state_stride + dm.hist_off();
    for (int j = 0; j < dm.taps - 1; ++j) {
        const int idx = q_len - (dm.taps - 1 - j);      // index into the portion; negative: before it
        hist[(size_t)j * C + c] = idx >= 0 ? proj[(size_t)(first + idx) * dm.ld + c] : hist[(size_t)(j + q_len) * C + c];
    }
}

// One warp per (request, head, 32 value columns): lane = value column, the column of S in registers.
template <int DMAX>
__global__ void __launch_bounds__(32)
delta_recurrence_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ decay,
                        float* __restrict__ state, long long state_stride, const int* __restrict__ cu_q,
                        const int* __restrict__ slots, DeltaDims dm, float* __restrict__ out) {
    __shared__ __align__(16) float ks[2][DMAX];
    __shared__ __align__(16) float qs[2][DMAX];
    const int lane = threadIdx.x, h = blockIdx.y, seq = blockIdx.z;
    const int col = blockIdx.x * 32 + lane;
    const bool live = col < dm.V;
    const int D = dm.D, C = dm.C();
    const int g = h / (dm.H / dm.G);
    const int first = cu_q[seq], last = cu_q[seq + 1];
    if (first >= last) return;
    float* S = state + (size_t)slots[seq] * state_stride + ((size_t)h * D) * dm.V + col;
    float s[DMAX];
#pragma unroll
    for (int i = 0; i < DMAX; ++i) s[i] = (live && i < D) ? S[(size_t)i * dm.V] : 0.f;
    constexpr int PER = DMAX / 32;
    float kn[PER], qn[PER];
    {
        const float* row = qkv + (size_t)first * C;
#pragma unroll
        for (int r = 0; r < PER; ++r) {
            const int i = lane + 32 * r;
            ks[0][i] = i < D ? row[(dm.G + g) * D + i] : 0.f;
            qs[0][i] = i < D ? row[g * D + i] : 0.f;
        }
    }
    __syncwarp();
    for (int t = first; t < last; ++t) {
        const int cur = (t - first) & 1;
        if (t + 1 < last) {                                  // the next token's k and q: on their way during the math
            const float* row = qkv + (size_t)(t + 1) * C;
#pragma unroll
            for (int r = 0; r < PER; ++r) {
                const int i = lane + 32 * r;
                kn[r] = i < D ? row[(dm.G + g) * D + i] : 0.f;
                qn[r] = i < D ? row[g * D + i] : 0.f;
            }
        }
        const float gd = decay[(size_t)t * dm.H + h], b = beta[(size_t)t * dm.H + h];
        const float v = live ? qkv[(size_t)t * C + 2 * dm.G * D + h * dm.V + col] : 0.f;
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
        for (int i = 0; i < DMAX; i += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(&ks[cur][i]);
            s[i] *= gd; s[i + 1] *= gd; s[i + 2] *= gd; s[i + 3] *= gd;
            d0 = fmaf(s[i], k4.x, d0); d1 = fmaf(s[i + 1], k4.y, d1);
            d2 = fmaf(s[i + 2], k4.z, d2); d3 = fmaf(s[i + 3], k4.w, d3);
        }
        const float u = b * (v - ((d0 + d1) + (d2 + d3)));
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int i = 0; i < DMAX; i += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(&ks[cur][i]);
            const float4 q4 = *reinterpret_cast<const float4*>(&qs[cur][i]);
            s[i] = fmaf(k4.x, u, s[i]); s[i + 1] = fmaf(k4.y, u, s[i + 1]);
            s[i + 2] = fmaf(k4.z, u, s[i + 2]); s[i + 3] = fmaf(k4.w, u, s[i + 3]);
            o0 = fmaf(s[i], q4.x, o0); o1 = fmaf(s[i + 1], q4.y, o1);
            o2 = fmaf(s[i + 2], q4.z, o2); o3 = fmaf(s[i + 3], q4.w, o3);
        }
        if (live) out[(size_t)t * dm.H * dm.V + h * dm.V + col] = (o0 + o1) + (o2 + o3);
        if (t + 1 < last) {
#pragma unroll
            for (int r = 0; r < PER; ++r) {
                ks[cur ^ 1][lane + 32 * r] = kn[r];
                qs[cur ^ 1][lane + 32 * r] = qn[r];
            }
        }
        __syncwarp();
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DMAX; ++i)
            if (i < D) S[(size_t)i * dm.V] = s[i];
    }
}

// y[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * silu(gate[t, h, :]); one warp per (t, h).
template <typename T>
__global__ void delta_gated_norm_kernel(const float* __restrict__ o, const float* __restrict__ proj,
                                        const float* __restrict__ weight, float eps, DeltaDims dm, int n_tokens,
                                        T* __restrict__ y) {
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * dm.H) return;
    const int lane = threadIdx.x & 31;
    const int t = (int)(item / dm.H), h = (int)(item - (long long)t * dm.H);
    const float* orow = o + ((size_t)t * dm.H + h) * dm.V;
    const float* grow = proj + (size_t)t * dm.ld + dm.gate_off() + h * dm.V;
    T* yrow = y + ((size_t)t * dm.H + h) * dm.V;
    float ss = 0.f;
    for (int i = lane; i < dm.V; i += 32) ss += orow[i] * orow[i];
    ss = ni_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dm.V + eps);
    for (int i = lane; i < dm.V; i += 32) yrow[i] = ni_from_float<T>(orow[i] * inv * weight[i] * dr_silu(grow[i]));
}

static int dr_check(const DeltaDims& dm) {
    if (dm.G <= 0 || dm.H <= 0 || dm.D <= 0 || dm.V <= 0 || dm.taps <= 0 || dm.H % dm.G) return NI_ERR_BAD_ARGUMENT;
    if (dm.ld < dm.a_off() + dm.H) return NI_ERR_BAD_ARGUMENT;
    if (dm.D > 256) return NI_ERR_UNSUPPORTED_SIZE;
    return NI_OK;
}

// Convolution, activations, unit norms, beta and decay of the step's tokens, then the new history.
NI_EXPORT int ni_delta_prepare(const float* proj, const float* conv_w, const float* a_log, const float* dt_bias,
                               float* state, long long state_stride, const int* seq_of_token, const int* cu_q,
                               const int* slots, int n_tokens, int n_seqs, int G, int H, int D, int V, int taps, int ld,
                               float* qkv, float* beta, float* decay, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    DeltaDims dm{G, H, D, V, taps, ld};
    if (int rc = dr_check(dm)) return rc;
    const int C = dm.C();
    const int threads = C >= 2048 ? 256 : 128;
    delta_prepare_kernel<<<n_tokens, threads, 0, stream>>>(proj, conv_w, a_log, dt_bias, state, state_stride,
                                                           seq_of_token, cu_q, slots, dm, qkv, beta, decay);
    if (taps > 1) {
        dim3 grid((C + 127) / 128, n_seqs);
        delta_history_kernel<<<grid, 128, 0, stream>>>(proj, state, state_stride, cu_q, slots, dm);
    }
    NI_RETURN_LAUNCH_STATUS();
}

NI_EXPORT int ni_delta_recurrence(const float* qkv, const float* beta, const float* decay, float* state,
                                  long long state_stride, const int* cu_q, const int* slots, int n_seqs, int G, int H,
                                  int D, int V, float* out, cudaStream_t stream) {
    if (n_seqs <= 0) return NI_OK;
    DeltaDims dm{G, H, D, V, 1, 2 * G * D + 2 * H * V + 2 * H};
    if (int rc = dr_check(dm)) return rc;
    if (H > 65535 || n_seqs > 65535) return NI_ERR_UNSUPPORTED_SIZE;
    dim3 grid((V + 31) / 32, H, n_seqs);
#define LAUNCH(DMAX) \
    delta_recurrence_kernel<DMAX><<<grid, 32, 0, stream>>>(qkv, beta, decay, state, state_stride, cu_q, slots, dm, out)
    if (D <= 32) LAUNCH(32);
    else if (D <= 64) LAUNCH(64);
    else if (D <= 128) LAUNCH(128);
    else LAUNCH(256);
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}

NI_EXPORT int ni_delta_gated_norm(const float* o, const float* proj, const float* weight, float eps, int n_tokens,
                                  int G, int H, int D, int V, int ld, void* y, int y_dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    DeltaDims dm{G, H, D, V, 1, ld};
    if (int rc = dr_check(dm)) return rc;
    const int warps = 4;
    const long long blocks = ((long long)n_tokens * H + warps - 1) / warps;
    if (blocks > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
    if (y_dtype == NI_DTYPE_F32)
        delta_gated_norm_kernel<float><<<(int)blocks, warps * 32, 0, stream>>>(o, proj, weight, eps, dm, n_tokens, (float*)y);
    else if (y_dtype == NI_DTYPE_BF16)
        delta_gated_norm_kernel<__nv_bfloat16><<<(int)blocks, warps * 32, 0, stream>>>(o, proj, weight, eps, dm, n_tokens,
                                                                                       (__nv_bfloat16*)y);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}
