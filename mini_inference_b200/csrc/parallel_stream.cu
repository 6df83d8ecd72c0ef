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

// The same with the row held in registers between the statistic and the output: four neighbouring entries per thread and step
// (16-byte loads of the stream, 8- or 16-byte loads of the outputs), VPT steps per thread; hidden = 4 * k, k <= NT * VPT.
template <typename TD> __device__ __forceinline__ float4 load4(const TD* p) {
    if constexpr (sizeof(TD) == 4) {
        return *reinterpret_cast<const float4*>(p);
    } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                           __uint_as_float(raw.y & 0xffff0000u));
    }
}
template <typename TY> __device__ __forceinline__ void store4(TY* p, float4 v) {
    if constexpr (sizeof(TY) == 4) {
        *reinterpret_cast<float4*>(p) = v;
    } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&lo);
        raw.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = raw;
    }
}

template <typename TD, typename TY, int VPT>
__global__ void __launch_bounds__(NT) stream_rmsnorm_pair_vec_kernel(float* __restrict__ x, const TD* __restrict__ a, const TD* __restrict__ b,
                                                                     const float* __restrict__ bias, const float* __restrict__ pre, long long pre_stride,
                                                                     const float* __restrict__ w, TY* __restrict__ y, const int* __restrict__ rows,
                                                                     int hidden, float eps) {
    __shared__ float scratch[32];
    const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    float* xr = x + r * hidden;
    const TD* ar = a ? a + r * hidden : nullptr;
    const TD* br = b ? b + r * hidden : nullptr;
    const float* pr = pre ? pre + r * pre_stride : nullptr;
    const int quads = hidden >> 2;
    float4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (threadIdx.x + k * NT < quads) {
            float4 xv = *reinterpret_cast<const float4*>(xr + i), d = make_float4(0.f, 0.f, 0.f, 0.f);
            if (ar) d = load4<TD>(ar + i);
            if (br) { const float4 t = load4<TD>(br + i); d.x += t.x; d.y += t.y; d.z += t.z; d.w += t.w; }
            if (bias) { const float4 t = *reinterpret_cast<const float4*>(bias + i); d.x += t.x; d.y += t.y; d.z += t.z; d.w += t.w; }
            if (pr) { const float4 t = *reinterpret_cast<const float4*>(pr + i); xv.x += t.x; xv.y += t.y; xv.z += t.z; xv.w += t.w; }
            xv.x += d.x; xv.y += d.y; xv.z += d.z; xv.w += d.w;             // the order of pair_sum: (a + b + bias), the pre-addition, the stream
            v[k] = xv;
            ss += xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w;
        }
    }
    const float s = rsqrtf(block_sum<NT>(ss, scratch) / hidden + eps);
    TY* yr = y + (size_t)blockIdx.x * hidden;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (threadIdx.x + k * NT < quads) {
            if (!rows) *reinterpret_cast<float4*>(xr + i) = v[k];
            const float4 wv = *reinterpret_cast<const float4*>(w + i);
            store4<TY>(yr + i, make_float4(v[k].x * s * wv.x, v[k].y * s * wv.y, v[k].z * s * wv.z, v[k].w * s * wv.w));
        }
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
        if (bias) {                                        // the halves of the bias start on 16 bytes as the halves of the row do
#pragma unroll
            for (int e = 0; e < VN; e += 4) {
                const float4 bg = *reinterpret_cast<const float4*>(bias + i + e), bu = *reinterpret_cast<const float4*>(bias + inter + i + e);
                gv[e] += bg.x; gv[e + 1] += bg.y; gv[e + 2] += bg.z; gv[e + 3] += bg.w;
                uv[e] += bu.x; uv[e + 1] += bu.y; uv[e + 2] += bu.z; uv[e + 3] += bu.w;
            }
        }
#pragma unroll
        for (int e = 0; e < VN; ++e) r[e] = glu_act(gv[e], act) * uv[e];
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
    auto aligned = [](const void* p) { return ((uintptr_t)p % 16) == 0; };
    const int quads = hidden / 4;
    const int vpt = quads <= NT ? 1 : quads <= 2 * NT ? 2 : quads <= 4 * NT ? 4 : quads <= 8 * NT ? 8 : 0;
    const bool vec = hidden % 4 == 0 && vpt && aligned(x) && aligned(a) && aligned(b) && aligned(bias) && aligned(pre) && aligned(w) && aligned(y) &&
                     (pre_stride % 4) == 0;
#define GOV(TD, TY, V) stream_rmsnorm_pair_vec_kernel<TD, TY, V><<<n, NT, 0, stream>>>(x, (const TD*)a, (const TD*)b, bias, pre, pre_stride, w, (TY*)y, rows, hidden, eps)
#define GO(TD, TY) do { if (!vec) stream_rmsnorm_pair_kernel<TD, TY><<<n, NT, 0, stream>>>(x, (const TD*)a, (const TD*)b, bias, pre, pre_stride, w, (TY*)y, rows, hidden, eps); \
        else if (vpt == 1) GOV(TD, TY, 1); else if (vpt == 2) GOV(TD, TY, 2); else if (vpt == 4) GOV(TD, TY, 4); else GOV(TD, TY, 8); } while (0)
    if (d_dtype == MI_BF16 && y_dtype == MI_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else if (d_dtype == MI_F32 && y_dtype == MI_F32) GO(float, float);
    else if (d_dtype == MI_F32 && y_dtype == MI_BF16) GO(float, __nv_bfloat16);
    else if (d_dtype == MI_BF16 && y_dtype == MI_F32) GO(__nv_bfloat16, float);
    else return -1;
#undef GO
#undef GOV
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
    const bool vec = inter % vn == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)bias % 16) == 0;
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
