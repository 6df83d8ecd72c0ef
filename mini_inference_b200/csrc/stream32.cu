// Kernels of a model whose residual stream stays in float32 whatever the run's dtype, and whose norms have one
// learned number: embedding gather + norm, residual-add (+ pass vector) + norm, the polynomial-norm activation,
// grouped RMS norm with a sigmoid gate behind a recurrence, and the per-head sigmoid gate behind latent attention.
// All statistics, sums and the stream itself are float32; the rows handed to matrix products have the run's dtype.
#include "common.cuh"

using namespace mi;

namespace {

constexpr int NT = 256;

// Sum over the block's NT threads; every thread gets the same value, added in a fixed order.
__device__ __forceinline__ float bsum(float v, float* scratch) { return block_sum<NT>(v, scratch); }

// ------------------------------------------------------------------ embedding + scalar norm -> stream
template <typename T, typename TX>
__global__ void embed_scaled_norm_kernel(const int* __restrict__ ids, const T* __restrict__ table, const float* __restrict__ g,
                                         TX* __restrict__ x, int hidden, int vocab, float eps) {
    __shared__ float scratch[32];
    int id = ids[blockIdx.x];
    if (id < 0 || id >= vocab) id = 0;
    const T* src = table + (size_t)id * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += NT) { const float v = to_f32(src[i]); ss += v * v; }
    const float r = rsqrtf(bsum(ss, scratch) / hidden + eps) * g[0];
    TX* dst = x + (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += NT) dst[i] = from_f32<TX>(to_f32(src[i]) * r);
}

// ------------------------------------------------------------------ x += delta (+ pre); y = g * x / rms(x)
// One block per output row.  rows == nullptr: row r of the stream is updated in place; otherwise output row r
// reads stream row rows[r] and the stream is left as it is (the final norm on the rows whose logits are wanted).
template <typename TD, typename TY>
__global__ void add_scaled_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, const float* __restrict__ pre,
                                          const float* __restrict__ g, TY* __restrict__ y, const int* __restrict__ rows,
                                          int hidden, float eps) {
    __shared__ float scratch[32];
    const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    float* xr = x + r * hidden;
    const TD* dr = delta ? delta + r * hidden : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        float v = xr[i];
        if (dr) v += to_f32(dr[i]);
        if (pre) v += pre[i];
        ss += v * v;
    }
    const float s = rsqrtf(bsum(ss, scratch) / hidden + eps) * g[0];
    TY* yr = y + (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        float v = xr[i];
        if (dr) v += to_f32(dr[i]);
        if (pre) v += pre[i];
        if (!rows) xr[i] = v;
        yr[i] = from_f32<TY>(v * s);
    }
}

// ------------------------------------------------------------------ a N(z) + b N(z^2) + c N(z^3) + e
template <typename T>
__global__ void polynorm_kernel(const T* __restrict__ z, const float* __restrict__ coef, T* __restrict__ out, int n, float eps) {
    __shared__ float scratch[32];
    const T* zr = z + (size_t)blockIdx.x * n;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < n; i += NT) {
        const float v = to_f32(zr[i]), v2 = v * v;
        s2 += v2; s4 += v2 * v2; s6 += v2 * v2 * v2;
    }
    s2 = bsum(s2, scratch); s4 = bsum(s4, scratch); s6 = bsum(s6, scratch);
    const float a = coef[0] * rsqrtf(s2 / n + eps), b = coef[1] * rsqrtf(s4 / n + eps), c = coef[2] * rsqrtf(s6 / n + eps), e = coef[3];
    T* o = out + (size_t)blockIdx.x * n;
    for (int i = threadIdx.x; i < n; i += NT) {
        const float v = to_f32(zr[i]), v2 = v * v;
        o[i] = from_f32<T>(a * v + b * v2 + c * v2 * v + e);
    }
}

// ------------------------------------------------------------------ o / rms(o over a group) * w * sigmoid(gate)
// grid (tokens, groups).  o float32 [T, groups * gs]; the weight has wlen entries and column c reads w[c % wlen]
// (one vector per row: wlen = groups * gs; one vector shared by the groups: wlen = gs).
// w == nullptr: no weight.  act 0: sigmoid(gate); 1: silu(gate) = gate * sigmoid(gate).
template <typename TG, typename TY>
__global__ void group_rmsnorm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, int wlen,
                                          const TG* __restrict__ gate, int gate_stride, TY* __restrict__ y, int groups, int gs, float eps,
                                          int act) {
    __shared__ float scratch[32];
    const size_t t = blockIdx.x;
    const int c0 = blockIdx.y * gs;
    const float* orow = o + t * groups * gs + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gs; i += NT) ss += orow[i] * orow[i];
    const float r = rsqrtf(bsum(ss, scratch) / gs + eps);
    const TG* grow = gate + t * gate_stride + c0;
    TY* yrow = y + t * groups * gs + c0;
    for (int i = threadIdx.x; i < gs; i += NT) {
        const float gv = to_f32(grow[i]);
        float sg = 1.f / (1.f + expf(-gv));
        if (act == 1) sg *= gv;
        const float wv = w ? w[(c0 + i) % wlen] : 1.f;
        yrow[i] = from_f32<TY>(orow[i] * r * wv * sg);
    }
}

// ------------------------------------------------------------------ rows[t, h V + v] = o[h, t, v] * sigmoid(gate[t, h])
template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ o, const T* __restrict__ gate, int gate_stride, T* __restrict__ y, int T_, int H, int V) {
    const size_t t = blockIdx.x;
    const int h = blockIdx.y;
    const float sg = gate ? 1.f / (1.f + expf(-to_f32(gate[t * gate_stride + h]))) : 1.f;      // no gate: the heads are only laid side by side
    const T* src = o + ((size_t)h * T_ + t) * V;
    T* dst = y + (t * H + h) * V;
    for (int i = threadIdx.x; i < V; i += blockDim.x) dst[i] = from_f32<T>(to_f32(src[i]) * sg);
}

// ------------------------------------------------------------------ embedding -> float32 stream (+ its rows in the table's type)
template <typename T>
__global__ void embed_stream_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ x, T* __restrict__ rows,
                                    int hidden, int vocab) {
    int id = ids[blockIdx.x];
    if (id < 0 || id >= vocab) id = 0;
    const T* src = table + (size_t)id * hidden;
    float* dst = x + (size_t)blockIdx.x * hidden;
    T* r = rows ? rows + (size_t)blockIdx.x * hidden : nullptr;
    for (int i = threadIdx.x; i < hidden; i += NT) { const T v = src[i]; dst[i] = to_f32(v); if (r) r[i] = v; }
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ y, size_t n) {
    for (size_t i = (size_t)blockIdx.x * NT + threadIdx.x; i < n; i += (size_t)gridDim.x * NT) y[i] = from_f32<T>(x[i]);
}

// ------------------------------------------------------------------ x += mult * ls * (w * y / rms(y)); rows = cast(x)
// One block per row.  The statistic, the product and the sum are float32; the stream is written back in float32 and,
// when rows != nullptr, also in the run's type for the sublayer that reads the stream next.
template <typename TYIN, typename TR>
__global__ void out_rmsnorm_add_kernel(float* __restrict__ x, const TYIN* __restrict__ y, const float* __restrict__ w,
                                       const float* __restrict__ ls, float mult, TR* __restrict__ rows, int hidden, float eps) {
    __shared__ float scratch[32];
    const size_t r = blockIdx.x;
    const TYIN* yr = y + r * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += NT) { const float v = to_f32(yr[i]); ss += v * v; }
    const float s = rsqrtf(bsum(ss, scratch) / hidden + eps);
    float* xr = x + r * hidden;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        float n = to_f32(yr[i]) * s * w[i];
        if (ls) n *= ls[i];
        const float v = xr[i] + mult * n;
        xr[i] = v;
        if (rows) rows[r * hidden + i] = from_f32<TR>(v);
    }
}

// ------------------------------------------------------------------ (x += delta;) y = w * x / rms(x), x a float32 stream
template <typename TD, typename TY>
__global__ void stream_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, const float* __restrict__ w,
                                      TY* __restrict__ y, const int* __restrict__ rows, int hidden, float eps) {
    __shared__ float scratch[32];
    const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    float* xr = x + r * hidden;
    const TD* dr = delta ? delta + r * hidden : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        float v = xr[i];
        if (dr) v += to_f32(dr[i]);
        ss += v * v;
    }
    const float s = rsqrtf(bsum(ss, scratch) / hidden + eps);
    TY* yr = y + (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        float v = xr[i];
        if (dr) v += to_f32(dr[i]);
        if (dr && !rows) xr[i] = v;
        yr[i] = from_f32<TY>(v * s * w[i]);
    }
}

}  // namespace

MI_EXPORT int mi_embed_stream(const int* ids, const void* table, float* x, void* rows, int T_, int hidden, int vocab, int dtype,
                              cudaStream_t stream) {
    if (T_ == 0) return 0;
    if (dtype == MI_BF16) embed_stream_kernel<__nv_bfloat16><<<T_, NT, 0, stream>>>(ids, (const __nv_bfloat16*)table, x, (__nv_bfloat16*)rows, hidden, vocab);
    else embed_stream_kernel<float><<<T_, NT, 0, stream>>>(ids, (const float*)table, x, (float*)rows, hidden, vocab);
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_cast_rows(const float* x, void* y, long long n, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    if (dtype != MI_BF16) return -1;
    const int blocks = (int)((n + NT * 8 - 1) / (NT * 8) < 1184 ? (n + NT * 8 - 1) / (NT * 8) : 1184);
    cast_rows_kernel<__nv_bfloat16><<<blocks, NT, 0, stream>>>(x, (__nv_bfloat16*)y, (size_t)n);
    return (int)cudaGetLastError();
}

// y: [n, hidden] in y_dtype; rows: nullptr or [n, hidden] bfloat16
MI_EXPORT int mi_out_rmsnorm_add(float* x, const void* y, const float* w, const float* ls, float mult, void* rows, int n, int hidden,
                                 float eps, int y_dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    if (y_dtype == MI_BF16) out_rmsnorm_add_kernel<__nv_bfloat16, __nv_bfloat16><<<n, NT, 0, stream>>>(x, (const __nv_bfloat16*)y, w, ls, mult, (__nv_bfloat16*)rows, hidden, eps);
    else out_rmsnorm_add_kernel<float, __nv_bfloat16><<<n, NT, 0, stream>>>(x, (const float*)y, w, ls, mult, (__nv_bfloat16*)rows, hidden, eps);
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_stream_rmsnorm(float* x, const void* delta, const float* w, void* y, const int* rows, int n, int hidden, float eps,
                                int delta_dtype, int y_dtype, cudaStream_t stream) {
    if (n == 0) return 0;
#define GO(TD, TY) stream_rmsnorm_kernel<TD, TY><<<n, NT, 0, stream>>>(x, (const TD*)delta, w, (TY*)y, rows, hidden, eps)
    if (delta_dtype == MI_BF16 && y_dtype == MI_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else if (delta_dtype == MI_F32 && y_dtype == MI_F32) GO(float, float);
    else if (delta_dtype == MI_F32 && y_dtype == MI_BF16) GO(float, __nv_bfloat16);
    else if (delta_dtype == MI_BF16 && y_dtype == MI_F32) GO(__nv_bfloat16, float);
    else return -1;
#undef GO
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_embed_scaled_norm(const int* ids, const void* table, const float* g, void* x, int T_, int hidden, int vocab,
                                   float eps, int table_dtype, int x_dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
#define GO(T, TX) embed_scaled_norm_kernel<T, TX><<<T_, NT, 0, stream>>>(ids, (const T*)table, g, (TX*)x, hidden, vocab, eps)
    if (table_dtype == MI_BF16 && x_dtype == MI_F32) GO(__nv_bfloat16, float);
    else if (table_dtype == MI_F32 && x_dtype == MI_F32) GO(float, float);
    else if (table_dtype == MI_BF16 && x_dtype == MI_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else return -1;
#undef GO
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_add_scaled_rmsnorm(float* x, const void* delta, const float* pre, const float* g, void* y, const int* rows,
                                    int n, int hidden, float eps, int delta_dtype, int y_dtype, cudaStream_t stream) {
    if (n == 0) return 0;
#define GO(TD, TY) add_scaled_rmsnorm_kernel<TD, TY><<<n, NT, 0, stream>>>(x, (const TD*)delta, pre, g, (TY*)y, rows, hidden, eps)
    if (delta_dtype == MI_BF16 && y_dtype == MI_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else if (delta_dtype == MI_F32 && y_dtype == MI_F32) GO(float, float);
    else if (delta_dtype == MI_F32 && y_dtype == MI_BF16) GO(float, __nv_bfloat16);
    else if (delta_dtype == MI_BF16 && y_dtype == MI_F32) GO(__nv_bfloat16, float);
    else return -1;
#undef GO
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_polynorm(const void* z, const float* coef, void* out, int rows, int n, float eps, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (dtype == MI_BF16) polynorm_kernel<__nv_bfloat16><<<rows, NT, 0, stream>>>((const __nv_bfloat16*)z, coef, (__nv_bfloat16*)out, n, eps);
    else polynorm_kernel<float><<<rows, NT, 0, stream>>>((const float*)z, coef, (float*)out, n, eps);
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_group_rmsnorm_gate(const float* o, const float* w, int wlen, const void* gate, int gate_stride, void* y,
                                    int T_, int groups, int gs, float eps, int dtype, int act, cudaStream_t stream) {
    if (T_ == 0) return 0;
    if (groups > 65535) return -2;
    dim3 grid(T_, groups);
    if (dtype == MI_BF16)
        group_rmsnorm_gate_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, NT, 0, stream>>>(o, w, wlen, (const __nv_bfloat16*)gate, gate_stride,
                                                                                         (__nv_bfloat16*)y, groups, gs, eps, act);
    else
        group_rmsnorm_gate_kernel<float, float><<<grid, NT, 0, stream>>>(o, w, wlen, (const float*)gate, gate_stride, (float*)y, groups, gs, eps, act);
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_head_gate(const void* o, const void* gate, int gate_stride, void* y, int T_, int H, int V, int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    if (H > 65535) return -2;
    dim3 grid(T_, H);
    const int nt = V >= 128 ? 128 : 64;
    if (dtype == MI_BF16)
        head_gate_kernel<__nv_bfloat16><<<grid, nt, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)y, T_, H, V);
    else
        head_gate_kernel<float><<<grid, nt, 0, stream>>>((const float*)o, (const float*)gate, gate_stride, (float*)y, T_, H, V);
    return (int)cudaGetLastError();
}
