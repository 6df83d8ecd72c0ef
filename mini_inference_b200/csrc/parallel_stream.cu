// Kernels around a float32 residual stream whose layers have ONE norm that two sublayers read:
//
//   embed_scaled_stream   x[t] = table[id_t] * scale + pos_table[p_t]   (pos_table may be absent), float32 out
//   stream_rmsnorm_pair   x += a + b + bias + pre  (each may be absent; pre is a vector for every row or a tensor row by row),
//                         y = w * x / rms(x); with `rows` only those rows are normed and the stream stays as it is
//   rows_rmsnorm          y = w * v / rms(v) over the rows of a strided view (a small latent inside a wider product)
//   bias_glu              [g | u] + bias -> act(g) * u, act one of relu, silu, gelu_tanh
//   scale_f32             z *= s
//
// Sums, statistics and the activation's arithmetic are float32; only what is handed to a matrix product is rounded to the
// run's type.  One block per row, sums over the block in a fixed order.
#include "common.cuh"
#include <math.h>

using namespace mi;

namespace {

constexpr int NT = 256;

template <typename T>
__global__ void embed_scaled_stream_kernel(const int* __restrict__ ids, const T* __restrict__ table, float scale,
                                           const T* __restrict__ pos_table, const int* __restrict__ positions, float* __restrict__ x,
                                           int hidden, int vocab, int pos_rows) {
    int id = ids[blockIdx.x];
    if (id < 0 || id >= vocab) id = 0;
    const T* src = table + (size_t)id * hidden;
    const T* pr = nullptr;
    if (pos_table) {
        int p = positions[blockIdx.x];
        p = p < 0 ? 0 : (p >= pos_rows ? pos_rows - 1 : p);
        pr = pos_table + (size_t)p * hidden;
    }
    float* dst = x + (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        float v = to_f32(src[i]) * scale;
        if (pr) v += to_f32(pr[i]);
        dst[i] = v;
    }
}

// The additions are made in one fixed order: (a + b + bias), then the pre-addition, then the stream.
template <typename TD>
__device__ __forceinline__ float pair_sum(float xv, const TD* ar, const TD* br, const float* bias, const float* pr, int i) {
    float d = 0.f;
    if (ar) d = to_f32(ar[i]);
    if (br) d += to_f32(br[i]);
    if (bias) d += bias[i];
    if (pr) xv += pr[i];
    return xv + d;
}

template <typename TD, typename TY>
__global__ void stream_rmsnorm_pair_kernel(float* __restrict__ x, const TD* __restrict__ a, const TD* __restrict__ b,
                                           const float* __restrict__ bias, const float* __restrict__ pre, long long pre_stride,
                                           const float* __restrict__ w, TY* __restrict__ y, const int* __restrict__ rows, int hidden,
                                           float eps) {
    __shared__ float scratch[32];
    const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    float* xr = x + r * hidden;
    const TD* ar = a ? a + r * hidden : nullptr;
    const TD* br = b ? b + r * hidden : nullptr;
    const float* pr = pre ? pre + r * pre_stride : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        const float v = pair_sum<TD>(xr[i], ar, br, bias, pr, i);
        ss += v * v;
    }
    const float s = rsqrtf(block_sum<NT>(ss, scratch) / hidden + eps);
    TY* yr = y + (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        const float v = pair_sum<TD>(xr[i], ar, br, bias, pr, i);
        if (!rows) xr[i] = v;
        yr[i] = from_f32<TY>(v * s * w[i]);
    }
}

template <typename T>
__global__ void rows_rmsnorm_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ w, T* __restrict__ y, int cols, float eps) {
    __shared__ float scratch[32];
    const T* xr = x + (size_t)blockIdx.x * ldx;
    float ss = 0.f;
    for (int i = threadIdx.x; i < cols; i += NT) { const float v = to_f32(xr[i]); ss += v * v; }
    const float s = rsqrtf(block_sum<NT>(ss, scratch) / cols + eps);
    T* yr = y + (size_t)blockIdx.x * cols;
    for (int i = threadIdx.x; i < cols; i += NT) yr[i] = from_f32<T>(to_f32(xr[i]) * s * w[i]);
}

template <typename T> __device__ __forceinline__ void store16v(T* p, const float* v) {
    if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        store2(p, v[0], v[1]); store2(p + 2, v[2], v[3]); store2(p + 4, v[4], v[5]); store2(p + 6, v[6], v[7]);
    }
}

__device__ __forceinline__ float glu_act(float g, int act) {
    if (act == 0) return fmaxf(g, 0.f);
    if (act == 1) return g / (1.f + expf(-g));
    return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

// grid (rows, pieces of the row)
template <typename T>
__global__ void bias_glu_kernel(const T* __restrict__ gu, const float* __restrict__ bias, T* __restrict__ out, int inter, int act) {
    const T* g = gu + (size_t)blockIdx.x * 2 * inter;
    T* o = out + (size_t)blockIdx.x * inter;
    for (int i = blockIdx.y * NT + threadIdx.x; i < inter; i += gridDim.y * NT) {
        float gv = to_f32(g[i]), uv = to_f32(g[inter + i]);
        if (bias) { gv += bias[i]; uv += bias[inter + i]; }
        o[i] = from_f32<T>(glu_act(gv, act) * uv);
    }
}

// eight bfloat16 (four float) per thread and step when the halves start on 16 bytes
template <typename T>
__global__ void bias_glu_vec_kernel(const T* __restrict__ gu, const float* __restrict__ bias, T* __restrict__ out, int inter, int act) {
    constexpr int VN = Vec16<T>::N;
    const T* g = gu + (size_t)blockIdx.x * 2 * inter;
    T* o = out + (size_t)blockIdx.x * inter;
    for (int i = (blockIdx.y * NT + threadIdx.x) * VN; i < inter; i += gridDim.y * NT * VN) {
        float gv[VN], uv[VN], r[VN];
        load16(g + i, gv);
        load16(g + inter + i, uv);
#pragma unroll
        for (int e = 0; e < VN; ++e) {
            float a = gv[e], u = uv[e];
            if (bias) { a += bias[i + e]; u += bias[inter + i + e]; }
            r[e] = glu_act(a, act) * u;
        }
        store16v(o + i, r);
    }
}

__global__ void scale_f32_kernel(float* __restrict__ z, size_t n, float s) {
    for (size_t i = (size_t)blockIdx.x * NT + threadIdx.x; i < n; i += (size_t)gridDim.x * NT) z[i] *= s;
}

}  // namespace

MI_EXPORT int mi_embed_scaled_stream(const int* ids, const void* table, float scale, const void* pos_table, const int* positions, float* x,
                                     int T_, int hidden, int vocab, int pos_rows, int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    if (pos_table && (!positions || pos_rows < 1)) return -2;
    if (dtype == MI_BF16)
        embed_scaled_stream_kernel<__nv_bfloat16><<<T_, NT, 0, stream>>>(ids, (const __nv_bfloat16*)table, scale, (const __nv_bfloat16*)pos_table,
                                                                         positions, x, hidden, vocab, pos_rows);
    else
        embed_scaled_stream_kernel<float><<<T_, NT, 0, stream>>>(ids, (const float*)table, scale, (const float*)pos_table, positions, x, hidden,
                                                                 vocab, pos_rows);
    return (int)cudaGetLastError();
}

// a, b: [T, hidden] in d_dtype (either may be null); bias float32 [hidden]; pre float32, pre_stride 0 (one vector) or hidden (row by row)
MI_EXPORT int mi_stream_rmsnorm_pair(float* x, const void* a, const void* b, const float* bias, const float* pre, long long pre_stride,
                                     const float* w, void* y, const int* rows, int n, int hidden, float eps, int d_dtype, int y_dtype,
                                     cudaStream_t stream) {
    if (n == 0) return 0;
#define GO(TD, TY) stream_rmsnorm_pair_kernel<TD, TY><<<n, NT, 0, stream>>>(x, (const TD*)a, (const TD*)b, bias, pre, pre_stride, w, (TY*)y, rows, hidden, eps)
    if (d_dtype == MI_BF16 && y_dtype == MI_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else if (d_dtype == MI_F32 && y_dtype == MI_F32) GO(float, float);
    else if (d_dtype == MI_F32 && y_dtype == MI_BF16) GO(float, __nv_bfloat16);
    else if (d_dtype == MI_BF16 && y_dtype == MI_F32) GO(__nv_bfloat16, float);
    else return -1;
#undef GO
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_rows_rmsnorm(const void* x, long long ldx, const float* w, void* y, int n, int cols, float eps, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    if (dtype == MI_BF16) rows_rmsnorm_kernel<__nv_bfloat16><<<n, NT, 0, stream>>>((const __nv_bfloat16*)x, ldx, w, (__nv_bfloat16*)y, cols, eps);
    else rows_rmsnorm_kernel<float><<<n, NT, 0, stream>>>((const float*)x, ldx, w, (float*)y, cols, eps);
    return (int)cudaGetLastError();
}

// act: 0 relu, 1 silu, 2 gelu_tanh
MI_EXPORT int mi_bias_glu(const void* gu, const float* bias, void* out, int rows, int inter, int act, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (act < 0 || act > 2) return -2;
    const int vn = dtype == MI_BF16 ? 8 : 4;
    const bool vec = inter % vn == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0;
    const int per = vec ? NT * vn : NT;
    dim3 grid(rows, rows >= 512 ? 1 : min(16, (inter + per - 1) / per));
#define GO(T) do { if (vec) bias_glu_vec_kernel<T><<<grid, NT, 0, stream>>>((const T*)gu, bias, (T*)out, inter, act); \
                   else bias_glu_kernel<T><<<grid, NT, 0, stream>>>((const T*)gu, bias, (T*)out, inter, act); } while (0)
    if (dtype == MI_BF16) GO(__nv_bfloat16); else GO(float);
#undef GO
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_scale_f32(float* z, long long n, float s, cudaStream_t stream) {
    if (n == 0) return 0;
    const long long want = (n + NT - 1) / NT;
    scale_f32_kernel<<<(int)(want < 1184 ? want : 1184), NT, 0, stream>>>(z, (size_t)n, s);
    return (int)cudaGetLastError();
}
