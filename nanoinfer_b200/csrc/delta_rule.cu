// The gated delta rule: a recurrent token mixer with a matrix state per head.
//
// Per head (state S [D, V] in FP32, carried from token to token of a request):
//     S *= decay;   e = beta * (v - k S);   S += outer(k, e);   y = q S        (k, q: rows of D; v, e, y: rows of V)
// with q and k unit vectors per head (q also times D^-1/2), decay = exp(-exp(A_log) softplus(a + dt_bias))
// and beta = sigmoid(b).  q, k and v first pass a short causal convolution over time per channel
// and silu; the last taps-1 inputs of every channel are part of a request's state.
//
// The step's tokens arrive as ONE fused projection `proj` (FP32 [T, ld]) with the columns
//     [ q: G D | k: G D | v: H V | gate: H V | b: H | a: H ]
// (G heads of q/k, H heads of v; head h reads q/k head h / (H / G)).  A request's state is a flat
// FP32 vector [ S: H D V | history: (taps-1) C ] with C = 2 G D + H V, found through slots[].
//
// Three launches, all FP32 inside:
//   delta_prepare      per token: convolution + silu, unit norms, beta, decay
//   (delta_history     per request: the new last taps-1 inputs; extra blocks of the gated norm's launch, which
//                      comes after delta_prepare has read the old ones)
//   delta_recurrence   per (request, head, a few value columns): its tokens one after the other
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

// qkv [T, C]: q (unit, times D^-1/2), k (unit), v after convolution and silu; gates [T, H, 2]: decay, beta.
// One warp per unit of work of a token: a q or k head (unit norm over its D channels), or 128 channels of v;
// the first warp of a token also computes beta and decay.  grid = (tokens, units / warps per block).
#define DP_WARPS 4
#define DP_VCHUNK 128
__global__ void __launch_bounds__(DP_WARPS * 32)
delta_prepare_kernel(const float* __restrict__ proj, const float* __restrict__ conv_w,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                     const float* __restrict__ state, long long state_stride,
                     const int* __restrict__ seq_of_token, const int* __restrict__ cu_q,
                     const int* __restrict__ slots, DeltaDims dm, float* __restrict__ qkv,
                     float* __restrict__ gates) {
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.y * DP_WARPS + (threadIdx.x >> 5);
    const int C = dm.C(), HV = dm.H * dm.V;
    const int n_units = 2 * dm.G + (HV + DP_VCHUNK - 1) / DP_VCHUNK;
    if (unit >= n_units) return;
    const int seq = seq_of_token[t];
    const int in_portion = t - cu_q[seq];
    const float* hist = state + (size_t)slots[seq] * state_stride + dm.hist_off();
    float* out = qkv + (size_t)t * C;
    if (unit < 2 * dm.G) {
        const int c0 = unit * dm.D;
        float ss = 0.f;
        for (int i = lane; i < dm.D; i += 32) {
            const float y = dr_conv(proj, conv_w, hist, dm, t, in_portion, c0 + i);
            out[c0 + i] = y;
            ss += y * y;
        }
        ss = ni_warp_sum(ss);
        float r = 1.0f / sqrtf(ss + 1e-6f);
        if (unit < dm.G) r *= 1.0f / sqrtf((float)dm.D);
        for (int i = lane; i < dm.D; i += 32) out[c0 + i] *= r;   // each lane rescales what it wrote itself
    } else {
        const int c0 = 2 * dm.G * dm.D + (unit - 2 * dm.G) * DP_VCHUNK;
        for (int c = c0 + lane; c < c0 + DP_VCHUNK && c < C; c += 32)
            out[c] = dr_conv(proj, conv_w, hist, dm, t, in_portion, c);
    }
    if (unit == 0) {
        const float* row = proj + (size_t)t * dm.ld;
        for (int h = lane; h < dm.H; h += 32) {
            gates[((size_t)t * dm.H + h) * 2] = expf(-expf(a_log[h]) * dr_softplus(row[dm.a_off() + h] + dt_bias[h]));
            gates[((size_t)t * dm.H + h) * 2 + 1] = dr_sigmoid(row[dm.b_off() + h]);
        }
    }
}

// The request's new history: its last taps-1 inputs.  One thread per channel walks j upwards, so a
// portion shorter than the history shifts the old entries in place (it reads index j + q_len > j).
__device__ __forceinline__ void delta_history(const float* __restrict__ proj, float* __restrict__ state,
                                              long long state_stride, const int* __restrict__ cu_q,
                                              const int* __restrict__ slots, const DeltaDims& dm, int seq, int c) {
    const int C = dm.C();
    if (c >= C) return;
    const int first = cu_q[seq], q_len = cu_q[seq + 1] - first;
    float* hist = state + (size_t)slots[seq] * state_stride + dm.hist_off();
    for (int j = 0; j < dm.taps - 1; ++j) {
        const int idx = q_len - (dm.taps - 1 - j);      // index into the portion; negative: before it
        hist[(size_t)j * C + c] = idx >= 0 ? proj[(size_t)(first + idx) * dm.ld + c] : hist[(size_t)(j + q_len) * C + c];
    }
}

// One warp per (request, head, a few value columns).  The rows of a column of S are cut into chunks of 8;
// a lane keeps CHUNKS of them in registers and RG lanes share a column, so k S and q S are sums inside a
// lane followed by log2(RG) shuffles.  The order of every sum is fixed by the chunk numbers alone (8 rows in
// four interleaved chains, then a binary tree over the chunk index from its lowest bit up), so the two
// layouts launched below - few lanes per column for single tokens, whose cost is reading and writing S in
// whole 32-byte sectors, and more lanes per column for long portions, whose cost is the chain of dependent
// operations per token - give the same bits.  (Key size 128, 16 heads, measured: one request of 2,048 tokens
// 695 us with 4 lanes per column, 613 us with 8, 647 us with 16; a batch of 8 single tokens 8.7 / 11.2 / 27.8 us.)  Lanes of one row group sit side by side and read neighbouring
// columns.  No block barrier.  What a token brings (k, q, the warp's values, decay, beta) travels through a
// ring of tokens in shared memory, filled by asynchronous copies that run ahead of the arithmetic.
#define DR_MAX_STAGES 8

__device__ __forceinline__ void dr_copy4(float* dst_smem, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_copy8(float* dst_smem, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_copy16(float* dst_smem, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

template <int CHUNKS, int RG>
__global__ void __launch_bounds__(32)
delta_recurrence_kernel(const float* __restrict__ qkv, const float* __restrict__ gates,
                        float* __restrict__ state, long long state_stride, const int* __restrict__ cu_q,
                        const int* __restrict__ slots, DeltaDims dm, float* __restrict__ out) {
    constexpr int ROWS = 8 * CHUNKS, COLS = 32 / RG, DP = ROWS * RG;   // rows per lane; columns per warp; D rounded up
    constexpr int STAGE = 2 * DP + 12;                     // k | q | v of the warp's columns (up to 8) | decay, beta, -, -
    constexpr int STAGES = DP >= 1024 ? 4 : DR_MAX_STAGES;
    __shared__ __align__(16) float ring[STAGES][STAGE];
    const int lane = threadIdx.x, rg = lane / COLS, cl = lane % COLS;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int col = blockIdx.x * COLS + cl;
    const bool live = col < dm.V;
    const int D = dm.D, C = dm.C(), row0 = rg * ROWS;
    const int g = h / (dm.H / dm.G);
    const int first = cu_q[seq], last = cu_q[seq + 1];
    if (first >= last) return;
    const bool wide = (D % 4 == 0) && (C % 4 == 0);        // rows of k and q start on 16-byte boundaries
    const bool padded = D != DP;                           // same for the whole launch
    const bool ragged = blockIdx.x * COLS + COLS > dm.V;   // same for the whole warp: some of its columns do not exist
    if (padded || ragged) {                                // entries that no copy ever writes
        for (int st = 0; st < STAGES; ++st) {
            for (int i = lane; i < DP; i += 32)
                if (i >= D) ring[st][i] = ring[st][DP + i] = 0.f;
            if (lane < COLS && !live) ring[st][2 * DP + lane] = 0.f;
        }
    }
    // Each lane's sources of the next token to fetch, advanced by a row per token; its place in the ring likewise.
    const float* row = qkv + (size_t)first * C;
    const float* k_src = row + (dm.G + g) * D + (wide ? 4 * lane : lane);
    const float* q_src = row + g * D + (wide ? 4 * lane : lane);
    const float* v_src = row + 2 * dm.G * D + h * dm.V + col;
    const float* g_src = gates + ((size_t)first * dm.H + h) * 2;
    int fetch_t = first, fetch_stage = 0;
    auto fetch = [&]() {                                   // the next token into its stage (nothing past the portion)
        if (fetch_t < last) {
            float* sg = ring[fetch_stage];
            if (wide) {
#pragma unroll
                for (int m = 0; m < (DP + 127) / 128; ++m)
                    if (4 * lane + 128 * m < D) {
                        dr_copy16(sg + 4 * lane + 128 * m, k_src + 128 * m);
                        dr_copy16(sg + DP + 4 * lane + 128 * m, q_src + 128 * m);
                    }
            } else {
#pragma unroll
                for (int m = 0; m < DP / 32; ++m)
                    if (lane + 32 * m < D) {
                        dr_copy4(sg + lane + 32 * m, k_src + 32 * m);
                        dr_copy4(sg + DP + lane + 32 * m, q_src + 32 * m);
                    }
            }
            if (lane < COLS && live) dr_copy4(sg + 2 * DP + lane, v_src);        // rg == 0 here
            if (lane == 31) dr_copy8(sg + 2 * DP + 8, g_src);                   // decay, beta
            k_src += C; q_src += C; v_src += C; g_src += 2 * dm.H;
        }
        ++fetch_t;
        fetch_stage = fetch_stage + 1 == STAGES ? 0 : fetch_stage + 1;
        asm volatile("cp.async.commit_group;" ::: "memory");     // one group per token, empty or not
    };
    for (int p = 0; p < STAGES - 1; ++p) fetch();
    float* S = state + (size_t)slots[seq] * state_stride + ((size_t)h * D + row0) * dm.V + col;   // this lane's first row
    float s[ROWS];
    if (!padded && !ragged) {
        const float* sp = S;
#pragma unroll
        for (int j = 0; j < ROWS; ++j, sp += dm.V) s[j] = *sp;
    } else {
#pragma unroll
        for (int j = 0; j < ROWS; ++j) s[j] = (live && row0 + j < D) ? S[(size_t)j * dm.V] : 0.f;
    }
    float* orow = out + (size_t)first * dm.H * dm.V + h * dm.V + col;
    int cur_stage = 0;
    float o_pending = 0.f;
    for (int t = first; t < last; ++t) {
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");   // this lane's copies of token t
        __syncwarp();                                                            // ... and the other lanes'
        fetch();                               // token t + STAGES - 1, into the stage that token t-1 has left
        const float* sg = ring[cur_stage];
        cur_stage = cur_stage + 1 == STAGES ? 0 : cur_stage + 1;
        const float* kc = sg + row0;
        const float* qc = sg + DP + row0;
        const float gd = sg[2 * DP + 8], b = sg[2 * DP + 9];
        const float v = sg[2 * DP + cl];
        float part[CHUNKS];
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const float4 ka = *reinterpret_cast<const float4*>(kc + 8 * c);
            const float4 kb = *reinterpret_cast<const float4*>(kc + 8 * c + 4);
            float* sc = s + 8 * c;
#pragma unroll
            for (int j = 0; j < 8; ++j) sc[j] *= gd;
            const float d0 = fmaf(sc[4], kb.x, sc[0] * ka.x), d1 = fmaf(sc[5], kb.y, sc[1] * ka.y);
            const float d2 = fmaf(sc[6], kb.z, sc[2] * ka.z), d3 = fmaf(sc[7], kb.w, sc[3] * ka.w);
            part[c] = (d0 + d1) + (d2 + d3);
        }
#pragma unroll
        for (int w = 1; w < CHUNKS; w <<= 1)
#pragma unroll
            for (int c = 0; c < CHUNKS; c += 2 * w) part[c] += part[c + w];
        float dot = part[0];
        // the lanes' partial sums of this token's k S and of the token before's q S travel together: two
        // independent shuffles per level instead of two trees one after the other
#pragma unroll
        for (int off = COLS; off < 32; off <<= 1) {
            dot += __shfl_xor_sync(0xffffffffu, dot, off);
            o_pending += __shfl_xor_sync(0xffffffffu, o_pending, off);
        }
        if (t > first && rg == 0 && live) orow[0] = o_pending;
        if (t > first) orow += dm.H * dm.V;
        const float u = b * (v - dot);
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const float4 ka = *reinterpret_cast<const float4*>(kc + 8 * c);
            const float4 kb = *reinterpret_cast<const float4*>(kc + 8 * c + 4);
            const float4 qa = *reinterpret_cast<const float4*>(qc + 8 * c);
            const float4 qb = *reinterpret_cast<const float4*>(qc + 8 * c + 4);
            float* sc = s + 8 * c;
            sc[0] = fmaf(ka.x, u, sc[0]); sc[1] = fmaf(ka.y, u, sc[1]); sc[2] = fmaf(ka.z, u, sc[2]); sc[3] = fmaf(ka.w, u, sc[3]);
            sc[4] = fmaf(kb.x, u, sc[4]); sc[5] = fmaf(kb.y, u, sc[5]); sc[6] = fmaf(kb.z, u, sc[6]); sc[7] = fmaf(kb.w, u, sc[7]);
            const float o0 = fmaf(sc[4], qb.x, sc[0] * qa.x), o1 = fmaf(sc[5], qb.y, sc[1] * qa.y);
            const float o2 = fmaf(sc[6], qb.z, sc[2] * qa.z), o3 = fmaf(sc[7], qb.w, sc[3] * qa.w);
            part[c] = (o0 + o1) + (o2 + o3);
        }
#pragma unroll
        for (int w = 1; w < CHUNKS; w <<= 1)
#pragma unroll
            for (int c = 0; c < CHUNKS; c += 2 * w) part[c] += part[c + w];
        o_pending = part[0];                   // summed over the lanes while the next token's k S is
        __syncwarp();                          // every lane has left this stage before a later fetch refills it
    }
#pragma unroll
    for (int off = COLS; off < 32; off <<= 1) o_pending += __shfl_xor_sync(0xffffffffu, o_pending, off);
    if (rg == 0 && live) orow[0] = o_pending;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (!padded && !ragged) {
        float* sp = S;
#pragma unroll
        for (int j = 0; j < ROWS; ++j, sp += dm.V) *sp = s[j];
    } else if (live) {
#pragma unroll
        for (int j = 0; j < ROWS; ++j)
            if (row0 + j < D) S[(size_t)j * dm.V] = s[j];
    }
}

// y[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * silu(gate[t, h, :]); one warp per (t, h).
// The blocks behind those (from norm_blocks on) write the requests' new convolution history: by now the
// preparation, which read the old one, has ended, and one launch less stands between two steps' products.
template <typename T>
__global__ void delta_gated_norm_kernel(const float* __restrict__ o, const float* __restrict__ proj,
                                        const float* __restrict__ weight, float eps, DeltaDims dm, int n_tokens,
                                        T* __restrict__ y, int norm_blocks, int hist_blocks_per_seq,
                                        float* __restrict__ state, long long state_stride,
                                        const int* __restrict__ cu_q, const int* __restrict__ slots) {
    if ((int)blockIdx.x >= norm_blocks) {
        const int hb = blockIdx.x - norm_blocks;
        delta_history(proj, state, state_stride, cu_q, slots, dm, hb / hist_blocks_per_seq,
                      (hb % hist_blocks_per_seq) * blockDim.x + threadIdx.x);
        return;
    }
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
    if (dm.D > 1024) return NI_ERR_UNSUPPORTED_SIZE;      // a warp holds whole columns of a head's state: 32 lanes x 32 rows
    return NI_OK;
}

// Convolution, activations, unit norms, beta and decay of the step's tokens (the new history is written by
// ni_delta_gated_norm, which every step runs after this).
NI_EXPORT int ni_delta_prepare(const float* proj, const float* conv_w, const float* a_log, const float* dt_bias,
                               float* state, long long state_stride, const int* seq_of_token, const int* cu_q,
                               const int* slots, int n_tokens, int n_seqs, int G, int H, int D, int V, int taps, int ld,
                               float* qkv, float* gates, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    DeltaDims dm{G, H, D, V, taps, ld};
    if (int rc = dr_check(dm)) return rc;
    const int C = dm.C();
    const int n_units = 2 * G + (H * V + DP_VCHUNK - 1) / DP_VCHUNK;
    dim3 pgrid(n_tokens, (n_units + DP_WARPS - 1) / DP_WARPS);
    if (pgrid.y > 65535) return NI_ERR_UNSUPPORTED_SIZE;
    delta_prepare_kernel<<<pgrid, DP_WARPS * 32, 0, stream>>>(proj, conv_w, a_log, dt_bias, state, state_stride,
                                                              seq_of_token, cu_q, slots, dm, qkv, gates);
    NI_RETURN_LAUNCH_STATUS();
}

NI_EXPORT int ni_delta_recurrence(const float* qkv, const float* gates, float* state,
                                  long long state_stride, const int* cu_q, const int* slots, int n_tokens, int n_seqs,
                                  int G, int H, int D, int V, float* out, cudaStream_t stream) {
    if (n_seqs <= 0) return NI_OK;
    DeltaDims dm{G, H, D, V, 1, 2 * G * D + 2 * H * V + 2 * H};
    if (int rc = dr_check(dm)) return rc;
    if (H > 65535 || n_seqs > 65535) return NI_ERR_UNSUPPORTED_SIZE;
#define LAUNCH(CHUNKS, RG)                                                                                       \
    do {                                                                                                         \
        dim3 grid((V + 32 / (RG) - 1) / (32 / (RG)), H, n_seqs);                                                 \
        delta_recurrence_kernel<CHUNKS, RG><<<grid, 32, 0, stream>>>(qkv, gates, state, state_stride, cu_q,       \
                                                                     slots, dm, out);                            \
    } while (0)
    // Lanes per column (RG): single tokens take the fewest (whole sectors of S); long portions take the fewest that
    // still give every scheduler a warp or so (3 warps per SM and more: measured at key size 128, one request of
    // 2,048 tokens, 16 heads: 695 / 613 / 647 us with 4 / 8 / 16 lanes; 8 heads: 16 lanes ahead of 8; 8 requests
    // of 512 tokens: 483 / 488 / 734 us).  The bits are the same whichever is taken.
    const bool long_portions = n_tokens >= 8 * n_seqs;
    const int chunks_total = D <= 32 ? 4 : D <= 64 ? 8 : D <= 128 ? 16 : D <= 256 ? 32 : D <= 512 ? 64 : 128;
    int rg = chunks_total / 4 < 4 ? 4 : chunks_total / 4;             // 4 chunks per lane (1 where D <= 32)
    if (long_portions)
        while (rg < 32 && rg < chunks_total &&
               (long long)n_seqs * H * ((V + 32 / rg - 1) / (32 / rg)) < 3LL * ni_sm_count())
            rg *= 2;
    switch (chunks_total * 100 + rg) {
        case 404: LAUNCH(1, 4); break;
        case 804: LAUNCH(2, 4); break;
        case 808: LAUNCH(1, 8); break;
        case 1604: LAUNCH(4, 4); break;
        case 1608: LAUNCH(2, 8); break;
        case 1616: LAUNCH(1, 16); break;
        case 3208: LAUNCH(4, 8); break;
        case 3216: LAUNCH(2, 16); break;
        case 3232: LAUNCH(1, 32); break;
        case 6416: LAUNCH(4, 16); break;
        case 6432: LAUNCH(2, 32); break;
        case 12832: LAUNCH(4, 32); break;
        default: return NI_ERR_UNSUPPORTED_SIZE;
    }
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}

// The gated norm of the step's read-outs, and the requests' new convolution history (taps > 1).
NI_EXPORT int ni_delta_gated_norm(const float* o, const float* proj, const float* weight, float eps, int n_tokens,
                                  int n_seqs, int G, int H, int D, int V, int taps, int ld, void* y, int y_dtype,
                                  float* state, long long state_stride, const int* cu_q, const int* slots,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    DeltaDims dm{G, H, D, V, taps, ld};
    if (int rc = dr_check(dm)) return rc;
    const int warps = 4;
    const long long norm_blocks = ((long long)n_tokens * H + warps - 1) / warps;
    const int per_seq = taps > 1 ? (dm.C() + warps * 32 - 1) / (warps * 32) : 0;
    const long long blocks = norm_blocks + (long long)per_seq * n_seqs;
    if (blocks > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
    if (y_dtype == NI_DTYPE_F32)
        delta_gated_norm_kernel<float><<<(int)blocks, warps * 32, 0, stream>>>(
            o, proj, weight, eps, dm, n_tokens, (float*)y, (int)norm_blocks, per_seq, state, state_stride, cu_q, slots);
    else if (y_dtype == NI_DTYPE_BF16)
        delta_gated_norm_kernel<__nv_bfloat16><<<(int)blocks, warps * 32, 0, stream>>>(
            o, proj, weight, eps, dm, n_tokens, (__nv_bfloat16*)y, (int)norm_blocks, per_seq, state, state_stride, cu_q, slots);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}
