// Kernels around a float32 residual stream whose additions are gated: the embedding with a hashed table of token pairs,
// the gated addition + norm, the norm-and-mix of two mixers' outputs, bias + activation behind a product, and the soft cap
// of the logits.  Statistics, gates and the stream are float32; rows handed to matrix products have the run's dtype.
#include "common.cuh"

using namespace mi;

namespace {

constexpr int NT = 256;

__device__ __forceinline__ float bsum(float v, float* scratch) { return block_sum<NT>(v, scratch); }
__device__ __forceinline__ float sigm(float z) { return 1.f / (1.f + expf(-z)); }

// ------------------------------------------------------------------ x = table[id] + pairs[hash(prev, id)]
// One block per token.  prev is the token before it in the step, or for an entry's first token the one its slot remembers;
// a token at position 0 takes the pair table's last row.  The block of an entry's FIRST token also leaves the entry's last
// token in the slot (it is the only reader of the slot's old value, so nothing races).
template <typename T>
__global__ void embed_pair_stream_kernel(const int* __restrict__ ids, const T* __restrict__ table, const T* __restrict__ pairs,
                                         float* __restrict__ x, int* __restrict__ state, long long state_stride,
                                         const int* __restrict__ positions, const int* __restrict__ token_seg,
                                         const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot, int hidden, int vocab,
                                         long long buckets, long long mul_prev, long long mul_cur) {
    const int t = blockIdx.x, seg = token_seg[t], qs = seg_q_start[seg];
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;
    long long prev;
    if (t == qs) {
        int* slot = state + (long long)seg_slot[seg] * state_stride;
        prev = slot[0];
        __syncthreads();                                  // every thread has read the old value before one replaces it
        if (threadIdx.x == 0) slot[0] = ids[seg_q_start[seg + 1] - 1];
    } else {
        prev = ids[t - 1];
    }
    const long long row = positions[t] == 0 ? buckets : (prev * mul_prev + (long long)id * mul_cur) % buckets;
    const T* a = table + (size_t)id * hidden;
    const T* b = pairs + (size_t)row * hidden;
    float* dst = x + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += NT) dst[i] = to_f32(a[i]) + to_f32(b[i]);
}

// ------------------------------------------------------------------ x += sigmoid(logits + bias) * (y + y_bias); out = w * x / rms(x)
template <typename TD, typename TY>
__global__ void stream_rmsnorm_gated_kernel(float* __restrict__ x, const TD* __restrict__ y, const TD* __restrict__ logits,
                                            const float* __restrict__ bias, const float* __restrict__ y_bias, const float* __restrict__ w,
                                            TY* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
    __shared__ float scratch[32];
    const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    float* xr = x + r * hidden;
    const TD* yr = y + r * hidden;
    const TD* lr = logits + r * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        const float add = to_f32(yr[i]) + (y_bias ? y_bias[i] : 0.f);
        const float v = fmaf(sigm(to_f32(lr[i]) + bias[i]), add, xr[i]);
        if (!rows) xr[i] = v;
        ss += v * v;
    }
    const float s = rsqrtf(bsum(ss, scratch) / hidden + eps);
    TY* o = out + (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        float v = xr[i];                                  // this thread's own write of the first pass, when the stream was updated
        if (rows) {
            const float add = to_f32(yr[i]) + (y_bias ? y_bias[i] : 0.f);
            v = fmaf(sigm(to_f32(lr[i]) + bias[i]), add, v);
        }
        o[i] = from_f32<TY>(v * s * w[i]);
    }
}

// ------------------------------------------------------------------ out = sa * wa * a / rms(a) + sb * wb * b / rms(b)
template <typename T>
__global__ void dual_rmsnorm_mix_kernel(const T* __restrict__ a, const float* __restrict__ wa, float sa, const T* __restrict__ b,
                                        const float* __restrict__ wb, float sb, T* __restrict__ out, int hidden, float eps) {
    __shared__ float scratch[32];
    const T* ar = a + (size_t)blockIdx.x * hidden;
    const T* br = b + (size_t)blockIdx.x * hidden;
    float s1 = 0.f, s2 = 0.f;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        const float u = to_f32(ar[i]), v = to_f32(br[i]);
        s1 += u * u; s2 += v * v;
    }
    const float ra = sa * rsqrtf(bsum(s1, scratch) / hidden + eps);
    const float rb = sb * rsqrtf(bsum(s2, scratch) / hidden + eps);
    T* o = out + (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += NT)
        o[i] = from_f32<T>(fmaf(to_f32(ar[i]) * ra, wa[i], to_f32(br[i]) * rb * wb[i]));
}

// ------------------------------------------------------------------ z + bias, then nothing (0) or relu squared (1)
template <typename T>
__global__ void bias_act_kernel(const T* __restrict__ z, const float* __restrict__ bias, T* __restrict__ out, size_t n, int cols, int act) {
    for (size_t i = (size_t)blockIdx.x * NT + threadIdx.x; i < n; i += (size_t)gridDim.x * NT) {
        float v = to_f32(z[i]) + bias[i % cols];
        if (act == 1) { v = fmaxf(v, 0.f); v *= v; }
        out[i] = from_f32<T>(v);
    }
}

// the same, eight bfloat16 numbers (16 bytes) a thread; cols is a multiple of 8, so the eight share a row
__global__ void bias_act_vec_kernel(const uint4* __restrict__ z, const float* __restrict__ bias, uint4* __restrict__ out, size_t n8, int cols, int act) {
    for (size_t i = (size_t)blockIdx.x * NT + threadIdx.x; i < n8; i += (size_t)gridDim.x * NT) {
        const uint4 v = z[i];
        const int c = (int)((i * 8) % (size_t)cols);
        const float4 b0 = *reinterpret_cast<const float4*>(bias + c), b1 = *reinterpret_cast<const float4*>(bias + c + 4);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
        float f[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 t = __bfloat1622float2(h[e]); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
        f[0] += b0.x; f[1] += b0.y; f[2] += b0.z; f[3] += b0.w; f[4] += b1.x; f[5] += b1.y; f[6] += b1.z; f[7] += b1.w;
        if (act == 1) {
#pragma unroll
            for (int e = 0; e < 8; ++e) { f[e] = fmaxf(f[e], 0.f); f[e] *= f[e]; }
        }
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
        out[i] = o;
    }
}

__global__ void softcap_kernel(float* __restrict__ z, size_t n, float cap) {
    for (size_t i = (size_t)blockIdx.x * NT + threadIdx.x; i < n; i += (size_t)gridDim.x * NT) z[i] = cap * tanhf(z[i] / cap);
}

inline int blocks_for(long long n) {
    const long long b = (n + NT - 1) / NT, most = 8ll * device_sms();
    return (int)(b < most ? b : most);
}

}  // namespace

MI_EXPORT int mi_embed_pair_stream(const int* ids, const void* table, const void* pairs, float* x, int* state, long long state_stride,
                                   const int* positions, const int* token_seg, const int* seg_q_start, const int* seg_slot, int T_, int hidden,
                                   int vocab, long long buckets, long long mul_prev, long long mul_cur, int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    if (dtype == MI_BF16)
        embed_pair_stream_kernel<__nv_bfloat16><<<T_, NT, 0, stream>>>(ids, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs, x, state,
                                                                      state_stride, positions, token_seg, seg_q_start, seg_slot, hidden, vocab,
                                                                      buckets, mul_prev, mul_cur);
    else
        embed_pair_stream_kernel<float><<<T_, NT, 0, stream>>>(ids, (const float*)table, (const float*)pairs, x, state, state_stride, positions,
                                                              token_seg, seg_q_start, seg_slot, hidden, vocab, buckets, mul_prev, mul_cur);
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_stream_rmsnorm_gated(float* x, const void* y, const void* logits, const float* bias, const float* y_bias, const float* w,
                                      void* out, const int* rows, int n, int hidden, float eps, int delta_dtype, int out_dtype,
                                      cudaStream_t stream) {
    if (n == 0) return 0;
#define GO(TD, TY) stream_rmsnorm_gated_kernel<TD, TY><<<n, NT, 0, stream>>>(x, (const TD*)y, (const TD*)logits, bias, y_bias, w, (TY*)out, rows, hidden, eps)
    if (delta_dtype == MI_BF16 && out_dtype == MI_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else if (delta_dtype == MI_F32 && out_dtype == MI_F32) GO(float, float);
    else if (delta_dtype == MI_BF16 && out_dtype == MI_F32) GO(__nv_bfloat16, float);
    else if (delta_dtype == MI_F32 && out_dtype == MI_BF16) GO(float, __nv_bfloat16);
    else return -1;
#undef GO
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_dual_rmsnorm_mix(const void* a, const float* wa, float sa, const void* b, const float* wb, float sb, void* out, int n,
                                  int hidden, float eps, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    if (dtype == MI_BF16)
        dual_rmsnorm_mix_kernel<__nv_bfloat16><<<n, NT, 0, stream>>>((const __nv_bfloat16*)a, wa, sa, (const __nv_bfloat16*)b, wb, sb, (__nv_bfloat16*)out, hidden, eps);
    else
        dual_rmsnorm_mix_kernel<float><<<n, NT, 0, stream>>>((const float*)a, wa, sa, (const float*)b, wb, sb, (float*)out, hidden, eps);
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_bias_act(const void* z, const float* bias, void* out, long long rows, int cols, int act, int dtype, cudaStream_t stream) {
    const long long n = rows * cols;
    if (n == 0) return 0;
    if (dtype == MI_BF16 && cols % 8 == 0 && (uintptr_t)z % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)bias % 16 == 0)
        bias_act_vec_kernel<<<blocks_for(n / 8), NT, 0, stream>>>((const uint4*)z, bias, (uint4*)out, (size_t)(n / 8), cols, act);
    else if (dtype == MI_BF16) bias_act_kernel<__nv_bfloat16><<<blocks_for(n), NT, 0, stream>>>((const __nv_bfloat16*)z, bias, (__nv_bfloat16*)out, (size_t)n, cols, act);
    else bias_act_kernel<float><<<blocks_for(n), NT, 0, stream>>>((const float*)z, bias, (float*)out, (size_t)n, cols, act);
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_softcap(float* z, long long n, float cap, cudaStream_t stream) {
    if (n == 0) return 0;
    softcap_kernel<<<blocks_for(n), NT, 0, stream>>>(z, (size_t)n, cap);
    return (int)cudaGetLastError();
}
