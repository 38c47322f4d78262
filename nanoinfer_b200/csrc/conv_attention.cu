// What stands between the projection and the attention of a mixer whose queries and keys pass a short
// causal convolution over time: convolution, per-head RMS norm, rotation of adjacent pairs, and the write
// into the paged cache, in one launch; and the request's convolution history.
//
//   u_t[c]  = the projected value of channel c at token t (q channels of all heads, then k channels)
//   y_t[c]  = sum_j w[j, c] * u_(t - taps + 1 + j)[c]          (zeros before the sequence's start; the taps are
//             handed over tap-major, [taps, C], so that neighbouring lanes read neighbouring weights)
//   value   = y of a key head, as it is                        -> value pages
//   n       = y / sqrt(mean_head(y^2) + eps) * gain[d]         (gain shared by the heads; one for q, one for k)
//   (a, b)  = (n[2i], n[2i+1]) -> (a cos - b sin, b cos + a sin), angle = position * inv_freq[i], i < rot / 2
//   query -> q_out, key -> key pages
//
// A request's history is the last taps - 1 projected rows of its sequence, FP32 [taps - 1, C] in its state
// slot (zero at admission = zeros before the start); the tokens of a portion read it for what lies before
// the portion, and conv_history_kernel, launched after, moves it on.  Convolution, norm, angles and
// rotation are FP32 whatever the tensors' type; a token's result depends on its own sequence only.
#include "common.cuh"

template <typename T, int REGS>
__global__ void conv_qk_prepare_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ conv_w,
                                       const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                                       const float* __restrict__ state, long long state_stride,
                                       const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                       const int* __restrict__ cu_q, const int* __restrict__ slots,
                                       const int* __restrict__ block_table, int bt_stride,
                                       const float* __restrict__ inv_freq, T* __restrict__ q_out,
                                       T* __restrict__ k_pages, T* __restrict__ v_pages, int n_tokens, int H, int G,
                                       int D, int rot, int taps, int page_size) {
    const int warps_per_block = blockDim.x >> 5;
    const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * (H + G)) return;
    const int lane = threadIdx.x & 31;
    const int t = (int)(item / (H + G));
    const int head = (int)(item - (long long)t * (H + G));
    const bool is_key = head >= H;
    const int C = (H + G) * D;
    const int c0 = head * D;
    const int seq = seq_of_token[t];
    const int row0 = cu_q[seq];
    const int local = t - row0;                       // index of the token inside its portion
    const float* hist = state + (size_t)slots[seq] * state_stride;
    const int pos = positions[t];

    float y[REGS];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < REGS; ++r) {
        const int d = lane + 32 * r;
        float acc = 0.f;
        if (d < D) {
            const int c = c0 + d;
            for (int j = 0; j < taps; ++j) {
                const int src = local - (taps - 1) + j;       // index inside the portion; negative: history
                const float u = src >= 0 ? ni_to_float(proj[(size_t)(row0 + src) * ld + c])
                                         : hist[(size_t)(taps - 1 + src) * C + c];
                acc = fmaf(conv_w[(size_t)j * C + c], u, acc);
            }
            ss += acc * acc;
        }
        y[r] = acc;
    }
    ss = ni_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)D + eps);
    const float* gain = is_key ? k_gain : q_gain;

    T* dst;
    T* vdst = nullptr;
    if (is_key) {
        if (k_pages == nullptr) return;               // a run that reads another run's cache writes none
        const int page = block_table[(size_t)seq * bt_stride + pos / page_size];
        const size_t off = (((size_t)page * G + (head - H)) * page_size + (pos % page_size)) * D;
        dst = k_pages + off;
        vdst = v_pages + off;
    } else {
        dst = q_out + ((size_t)t * H + head) * D;
    }
#pragma unroll
    for (int r = 0; r < REGS; ++r) {
        const int d = lane + 32 * r;
        const float n = d < D ? y[r] * inv * gain[d] : 0.f;
        const float other = __shfl_xor_sync(0xffffffffu, n, 1);      // the pair's other half sits in the neighbouring lane
        float o = n;
        if (d < rot) {
            const float ang = __fmul_rn((float)pos, inv_freq[d >> 1]);
            float sn, cs;
            sincosf(ang, &sn, &cs);
            o = (d & 1) ? fmaf(n, cs, other * sn) : fmaf(n, cs, -other * sn);
        }
        if (d < D) {
            dst[d] = ni_from_float<T>(o);
            if (vdst != nullptr) vdst[d] = ni_from_float<T>(y[r]);
        }
    }
}

// The same with four neighbouring dimensions per lane (head sizes and row strides that are multiples of 4): the
// projected values, the history and the results move in 8- or 16-byte pieces, and a rotated pair lies in one lane.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
        const uint2 x = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 x;
        x.x = *reinterpret_cast<const uint32_t*>(&a);
        x.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = x;
    }
};

// One block per token: the sines and cosines of the token's angles are computed once into shared memory and serve
// all heads; the block's warps share the heads.
template <typename T, int CHUNKS>
__global__ void __launch_bounds__(256)
conv_qk_prepare_vec_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ conv_w,
                           const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                           const float* __restrict__ state, long long state_stride,
                           const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                           const int* __restrict__ cu_q, const int* __restrict__ slots,
                           const int* __restrict__ block_table, int bt_stride,
                           const float* __restrict__ inv_freq, T* __restrict__ q_out,
                           T* __restrict__ k_pages, T* __restrict__ v_pages, int n_tokens, int H, int G,
                           int D, int rot, int taps, int page_size) {
    __shared__ float s_sin[256], s_cos[256];          // rot / 2 <= 256
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int pos = positions[t];
    const int seq = seq_of_token[t];
    for (int i = threadIdx.x; i < (rot >> 1); i += blockDim.x) sincosf(__fmul_rn((float)pos, inv_freq[i]), &s_sin[i], &s_cos[i]);
    const int C = (H + G) * D;
    const int row0 = cu_q[seq];
    const int local = t - row0;
    const float* hist = state + (size_t)slots[seq] * state_stride;
    int page = 0;
    if (k_pages != nullptr) page = block_table[(size_t)seq * bt_stride + pos / page_size];
    __syncthreads();
    for (int head = warp + blockIdx.y * n_warps; head < H + G; head += n_warps * gridDim.y) {     // few tokens: the heads are dealt over several blocks
        const bool is_key = head >= H;
        if (is_key && k_pages == nullptr) continue;
        const int c0 = head * D;
        const float* gain = is_key ? k_gain : q_gain;
        float y[CHUNKS][4];
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < CHUNKS; ++r) {
            const int d0 = 4 * lane + 128 * r;
#pragma unroll
            for (int i = 0; i < 4; ++i) y[r][i] = 0.f;
            if (d0 < D) {
                const int c = c0 + d0;
                for (int j = 0; j < taps; ++j) {
                    const int src = local - (taps - 1) + j;
                    float u[4], wj[4];
                    Vec4<float>::load(conv_w + (size_t)j * C + c, wj);       // tap j of four neighbouring channels
                    if (src >= 0) Vec4<T>::load(proj + (size_t)(row0 + src) * ld + c, u);
                    else Vec4<float>::load(hist + (size_t)(taps - 1 + src) * C + c, u);
#pragma unroll
                    for (int i = 0; i < 4; ++i) y[r][i] = fmaf(wj[i], u[i], y[r][i]);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) ss += y[r][i] * y[r][i];
            }
        }
        ss = ni_warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)D + eps);
        T* dst;
        T* vdst = nullptr;
        if (is_key) {
            const size_t off = (((size_t)page * G + (head - H)) * page_size + (pos % page_size)) * D;
            dst = k_pages + off;
            vdst = v_pages + off;
        } else {
            dst = q_out + ((size_t)t * H + head) * D;
        }
#pragma unroll
        for (int r = 0; r < CHUNKS; ++r) {
            const int d0 = 4 * lane + 128 * r;
            if (d0 >= D) continue;
            float gn[4], n[4], o[4];
            Vec4<float>::load(gain + d0, gn);
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i] = n[i] = y[r][i] * inv * gn[i];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (d0 + 2 * i < rot) {
                    const float sn = s_sin[(d0 >> 1) + i], cs = s_cos[(d0 >> 1) + i];
                    o[2 * i] = fmaf(n[2 * i], cs, -n[2 * i + 1] * sn);
                    o[2 * i + 1] = fmaf(n[2 * i + 1], cs, n[2 * i] * sn);
                }
            }
            Vec4<T>::store(dst + d0, o);
            if (vdst != nullptr) Vec4<T>::store(vdst + d0, y[r]);
        }
    }
}

// state[slot][r, c] <- the projected value of channel c at the sequence's place (end - (taps - 1) + r): from the
// portion where it reaches that far back, else from the old history, shifted (rows ascend, so a thread reads
// a row before it overwrites it).
template <typename T>
__global__ void conv_history_kernel(const T* __restrict__ proj, int ld, float* __restrict__ state,
                                    long long state_stride, const int* __restrict__ cu_q,
                                    const int* __restrict__ slots, int C, int taps) {
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int row0 = cu_q[seq], q_len = cu_q[seq + 1] - row0;
    float* hist = state + (size_t)slots[seq] * state_stride;
    for (int r = 0; r < taps - 1; ++r) {
        const int src = q_len - (taps - 1) + r;
        const float v = src >= 0 ? ni_to_float(proj[(size_t)(row0 + src) * ld + c]) : hist[(size_t)(taps - 1 + src) * C + c];
        hist[(size_t)r * C + c] = v;
    }
}

NI_EXPORT int ni_conv_qk_prepare(const void* proj, int dtype, int ld, const float* conv_w, const float* q_gain,
                                 const float* k_gain, float eps, float* state, long long state_stride,
                                 const int* positions, const int* seq_of_token, const int* cu_q, const int* slots,
                                 const int* block_table, int bt_stride, const float* inv_freq, void* q_out,
                                 void* k_pages, void* v_pages, int n_tokens, int n_seqs, int H, int G, int D, int rot,
                                 int taps, int page_size, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (H <= 0 || G <= 0 || D <= 0 || taps <= 0 || rot < 0 || rot > D || (rot & 1) || page_size <= 0 || n_seqs <= 0 ||
        ld < (H + G) * D)
        return NI_ERR_BAD_ARGUMENT;
    if (D > 512) return NI_ERR_UNSUPPORTED_SIZE;
    const int warps = 4;
    const long long items = (long long)n_tokens * (H + G);
    const long long blocks = (items + warps - 1) / warps;
    if (blocks > 2147483647LL || n_seqs > 65535) return NI_ERR_UNSUPPORTED_SIZE;
#define LAUNCH_R(T, R)                                                                                          \
    conv_qk_prepare_kernel<T, R><<<(int)blocks, warps * 32, 0, stream>>>(                                       \
        (const T*)proj, ld, conv_w, q_gain, k_gain, eps, state, state_stride, positions, seq_of_token, cu_q,    \
        slots, block_table, bt_stride, inv_freq, (T*)q_out, (T*)k_pages, (T*)v_pages, n_tokens, H, G, D, rot,   \
        taps, page_size)
#define LAUNCH_V(T, R)                                                                                          \
    conv_qk_prepare_vec_kernel<T, R><<<vec_grid, vec_threads, 0, stream>>>(                                     \
        (const T*)proj, ld, conv_w, q_gain, k_gain, eps, state, state_stride, positions, seq_of_token, cu_q,    \
        slots, block_table, bt_stride, inv_freq, (T*)q_out, (T*)k_pages, (T*)v_pages, n_tokens, H, G, D, rot,   \
        taps, page_size)
    const bool vec = (D % 4 == 0) && (ld % 4 == 0);      // whole 8- or 16-byte pieces everywhere
    const int vec_threads = 32 * (H + G < 8 ? H + G : 8);
    const dim3 vec_grid(n_tokens, n_tokens < 4 * ni_sm_count() ? (H + G + 7) / 8 : 1);     // few tokens: a warp per head
#define LAUNCH(T)                                          \
    do {                                                   \
        if (vec && D <= 128) LAUNCH_V(T, 1);               \
        else if (vec && D <= 256) LAUNCH_V(T, 2);          \
        else if (vec) LAUNCH_V(T, 4);                      \
        else if (D <= 128) LAUNCH_R(T, 4);                 \
        else if (D <= 256) LAUNCH_R(T, 8);                 \
        else LAUNCH_R(T, 16);                              \
    } while (0)
    if (dtype == NI_DTYPE_F32) LAUNCH(float);
    else if (dtype == NI_DTYPE_BF16) LAUNCH(__nv_bfloat16);
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
#undef LAUNCH_R
#undef LAUNCH_V
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (taps > 1) {
        const int C = (H + G) * D;
        dim3 grid((C + 255) / 256, n_seqs);
        if (dtype == NI_DTYPE_F32)
            conv_history_kernel<float><<<grid, 256, 0, stream>>>((const float*)proj, ld, state, state_stride, cu_q, slots, C, taps);
        else
            conv_history_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)proj, ld, state, state_stride,
                                                                        cu_q, slots, C, taps);
    }
    NI_RETURN_LAUNCH_STATUS();
}
