// Paged softmax attention whose mask and softmax are chosen by constants, and the kernel that prepares its inputs.
//
//   keys      j <= i; with block > 0 only those of i's own block of positions, floor(j / block) = floor(i / block)
//             (blocks counted from position 0 of the sequence); with window > 0 only the last `window`
//   sink      one more softmax term whose score is 0 and which carries no value: p_j = exp(s_j) / (1 + sum exp(s_j));
//             a running maximum that starts at 0 with a running sum that starts at 1 is exactly that
//             sink_values: the term is exp(sink_values[h]) instead (a learned score per head; it is not scaled and gets no bias)
//   bias      a float32 table [bias_last + 1, H] added to the scaled score by the distance i - j (distances beyond bias_last
//             read the last row)
//   slopes    float32 [H]: slopes[h] * (i - j) is taken off the scaled score of head h (a straight line in the distance, no table)
//   sizes     key rows of D and value rows of Dv entries (up to 256; any size, 16-byte loads where rows allow), each in a pool of its own:
//             k_cache [pages, KV, page_size, D], v_cache [pages, KV, page_size, Dv]
//
// All arithmetic is float32 on the CUDA cores (scores, softmax weights and the weighted sum), in an order that
// depends only on the request's own positions.  Prompt portions: one warp per query row; decoded tokens: the
// (visible) keys of a request cut into `splits` pieces, one warp per (head, piece), merged by a second kernel.
//
// Prepare kernel, one block per token: q and k divided by their root mean square per head (eps > 0) and, when given, multiplied by
// a weight of D entries that all heads share (one for q, one for k); q then multiplied by the temperature
// 1 + coef * ln(floor((p + 1) / every) + 1) of its position p (every > 0); v blended with another layer's values of the same
// token ((1 - lambda) v + lambda v_src), or, with v_is_k, taken from the keys AS PROJECTED (before the norm; there are no v
// columns then); k and v written to the token's slot of the pages, q written back in place.
#include "common.cuh"
#include <math.h>

using namespace mi;

namespace {

constexpr int MAX_D = 256;
constexpr int WARPS = 4;

template <typename T>
__device__ __forceinline__ void attend_keys(const float* q_s, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                            const int* __restrict__ table_row, int kvh, int KV, int D, int Dv, int ps,
                                            int lo, int hi, float& m, float& l, float (&acc)[MAX_D / 32],
                                            const float* __restrict__ bias = nullptr, int bias_last = 0, int H = 0, int h = 0, int qpos = 0,
                                            float slope = 0.f) {
    const int lane = threadIdx.x & 31;
    constexpr int VN = Vec16<T>::N;
    for (int j0 = lo; j0 < hi; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j < hi;
        long long row = 0;
        float s = -INFINITY;
        if (valid) {
            row = (long long)(table_row[j / ps] * KV + kvh) * ps + j % ps;
            const T* kr = k_cache + row * D;
            float dot = 0.f, tmp[VN];
            if (D % VN == 0) {                                     // rows start on 16 bytes: 16-byte loads
                for (int c = 0; c < D; c += VN) {
                    load16(kr + c, tmp);
#pragma unroll
                    for (int e = 0; e < VN; ++e) dot += q_s[c + e] * tmp[e];
                }
            } else {
                for (int c = 0; c < D; ++c) dot += q_s[c] * to_f32(kr[c]);
            }
            s = bias ? dot + bias[(size_t)min(qpos - j, bias_last) * H + h] : dot;
            if (slope != 0.f) s -= slope * (float)(qpos - j);
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float alpha = expf(m - m_new);              // nothing seen yet and no sink: exp(-inf) = 0
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int k = 0; k < MAX_D / 32; ++k) acc[k] *= alpha;
        const int n = min(32, hi - j0);
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long vrow = __shfl_sync(0xffffffffu, row, jj);
            const T* vr = v_cache + vrow * Dv;
#pragma unroll
            for (int k = 0; k < MAX_D / 32; ++k) {
                const int d = lane + 32 * k;
                if (d < Dv) acc[k] += pj * to_f32(vr[d]);
            }
        }
    }
}

__device__ __forceinline__ int first_key(int p, int block, int window) {
    int lo = block > 0 ? (p / block) * block : 0;
    if (window > 0) lo = max(lo, p - window + 1);
    return lo;
}

// grid (tiles, H): tile = (entry, first row); each warp takes rows of the tile in turn.
template <typename T>
__global__ void masked_prefill_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                      T* __restrict__ out, const int* __restrict__ tiles, const int* __restrict__ seg_q_start,
                                      const int* __restrict__ seg_pos0, const int* __restrict__ block_table,
                                      const int* __restrict__ table_rows, int table_stride, int H, int KV, int D, int Dv, int ps,
                                      int tile_rows, float scale, int block, int window, int sink,
                                      const float* __restrict__ sink_values, const float* __restrict__ bias, int bias_last,
                                      const float* __restrict__ slopes) {
    __shared__ float q_s[WARPS][MAX_D];
    const int seg = tiles[2 * blockIdx.x], r0 = tiles[2 * blockIdx.x + 1];
    const int h = blockIdx.y, kvh = h / (H / KV);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int qs = seg_q_start[seg], n = seg_q_start[seg + 1] - qs, pos0 = seg_pos0[seg];
    const int* table_row = block_table + (size_t)(table_rows ? table_rows[seg] : seg) * table_stride;
    const int r_end = min(r0 + tile_rows, n);
    for (int r = r0 + warp; r < r_end; r += WARPS) {
        const int tok = qs + r, p = pos0 + r;
        const T* qr = q + (size_t)tok * q_stride + (size_t)h * D;
        for (int d = lane; d < D; d += 32) q_s[warp][d] = to_f32(qr[d]) * scale;
        __syncwarp();
        float m = sink ? (sink_values ? sink_values[h] : 0.f) : -INFINITY, l = sink ? 1.f : 0.f, acc[MAX_D / 32];
#pragma unroll
        for (int k = 0; k < MAX_D / 32; ++k) acc[k] = 0.f;
        attend_keys<T>(q_s[warp], k_cache, v_cache, table_row, kvh, KV, D, Dv, ps, first_key(p, block, window), p + 1, m, l, acc,
                       bias, bias_last, H, h, p, slopes ? slopes[h] : 0.f);
        T* orow = out + ((size_t)tok * H + h) * Dv;
#pragma unroll
        for (int k = 0; k < MAX_D / 32; ++k) {
            const int d = lane + 32 * k;
            if (d < Dv) orow[d] = from_f32<T>(acc[k] / l);
        }
        __syncwarp();
    }
}

// grid (decode entries, ceil(H / 4), splits); one warp per query head.  With one split the sink is part of the
// warp's own softmax; with several the pieces are plain and the merge adds the sink's term.
template <typename T>
__global__ void masked_decode_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                     T* __restrict__ out, float* __restrict__ o_part, float* __restrict__ lse_part,
                                     const int* __restrict__ decode_segs, const int* __restrict__ seg_q_start,
                                     const int* __restrict__ seg_kv_len, const int* __restrict__ block_table,
                                     const int* __restrict__ table_rows, int table_stride, int H, int KV, int D, int Dv, int ps,
                                     float scale, int block, int window, int sink,
                                     const float* __restrict__ sink_values, const float* __restrict__ bias, int bias_last,
                                     const float* __restrict__ slopes) {
    __shared__ float q_s[WARPS][MAX_D];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y * WARPS + warp;
    if (h >= H) return;
    const int seg = decode_segs[blockIdx.x], kvh = h / (H / KV);
    const int tok = seg_q_start[seg], len = seg_kv_len[seg];
    const int S = gridDim.z, s = blockIdx.z;
    const int lo0 = first_key(len - 1, block, window);           // the query's position is len - 1
    // every request cuts ITS OWN key range into S pieces of whole 32-key chunks
    const int piece = (((len - lo0) + S - 1) / S + 31) / 32 * 32;
    const int lo = lo0 + s * piece, hi = min(lo + piece, len);
    const T* qr = q + (size_t)tok * q_stride + (size_t)h * D;
    for (int d = lane; d < D; d += 32) q_s[warp][d] = to_f32(qr[d]) * scale;
    __syncwarp();
    const bool own_sink = sink && S == 1;
    float m = own_sink ? (sink_values ? sink_values[h] : 0.f) : -INFINITY, l = own_sink ? 1.f : 0.f, acc[MAX_D / 32];
#pragma unroll
    for (int k = 0; k < MAX_D / 32; ++k) acc[k] = 0.f;
    if (lo < hi)
        attend_keys<T>(q_s[warp], k_cache, v_cache, block_table + (size_t)(table_rows ? table_rows[seg] : seg) * table_stride, kvh, KV,
                       D, Dv, ps, lo, hi, m, l, acc, bias, bias_last, H, h, len - 1, slopes ? slopes[h] : 0.f);
    const float inv = l > 0.f ? 1.f / l : 0.f;                  // empty piece: output 0, lse -inf
    if (S == 1) {
        T* orow = out + ((size_t)tok * H + h) * Dv;
#pragma unroll
        for (int k = 0; k < MAX_D / 32; ++k) { const int d = lane + 32 * k; if (d < Dv) orow[d] = from_f32<T>(acc[k] * inv); }
    } else {
        const size_t idx = ((size_t)blockIdx.x * H + h) * S + s;
        float* orow = o_part + idx * Dv;
#pragma unroll
        for (int k = 0; k < MAX_D / 32; ++k) { const int d = lane + 32 * k; if (d < Dv) orow[d] = acc[k] * inv; }
        if (lane == 0) lse_part[idx] = l > 0.f ? m + logf(l) : -INFINITY;
    }
}

// out = sum_s e^(lse_s - mx) o_s / (sum_s e^(lse_s - mx) + [sink] e^(sv - mx)),  mx = max(lse_s, [sink] sv),  sv the sink's score (0 or learned)
template <typename T>
__global__ void masked_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ lse_part, T* __restrict__ out,
                                    const int* __restrict__ decode_segs, const int* __restrict__ seg_q_start, int H, int Dv, int S, int sink,
                                    const float* __restrict__ sink_values) {
    const int i = blockIdx.x, h = blockIdx.y;
    const float sv = sink_values ? sink_values[h] : 0.f;
    const int tok = seg_q_start[decode_segs[i]];
    const size_t base = ((size_t)i * H + h) * S;
    float mx = sink ? sv : -INFINITY;
    for (int s = 0; s < S; ++s) mx = fmaxf(mx, lse_part[base + s]);
    float den = sink ? expf(sv - mx) : 0.f;
    for (int s = 0; s < S; ++s) den += expf(lse_part[base + s] - mx);
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        float num = 0.f;
        for (int s = 0; s < S; ++s) num += expf(lse_part[base + s] - mx) * o_part[(base + s) * Dv + d];
        out[((size_t)tok * H + h) * Dv + d] = from_f32<T>(num / den);
    }
}

// ------------------------------------------------------------------ unit norms, value blend, cache write
// p [T, ldp] = q [H D] | k [KV D] | v [KV Dv].  One block per token, a warp per head in turn.
template <typename T>
__global__ void unit_qk_cache_kernel(T* __restrict__ p, int ldp, const T* __restrict__ v_src, int ld_src, const float* __restrict__ lam,
                                     const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     int H, int KV, int D, int Dv, int ps, float eps, int unit, const float* __restrict__ q_w,
                                     const float* __restrict__ k_w, const int* __restrict__ positions, float temp_coef, int temp_every,
                                     int v_is_k) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    T* row = p + (size_t)t * ldp;
    const int slot = slots[t];
    const long long page = slot / ps, off = slot % ps;
    const float temp = temp_every > 0 ? 1.f + temp_coef * logf((float)((positions[t] + 1) / temp_every + 1)) : 1.f;
    for (int u = warp; u < H + KV; u += nw) {                   // q heads, then k heads
        T* x = row + (size_t)u * D;
        float r = 1.f;
        if (unit) {
            float ss = 0.f;
            for (int d = lane; d < D; d += 32) { const float v = to_f32(x[d]); ss += v * v; }
            r = rsqrtf(warp_sum(ss) / D + eps);
        }
        if (u < H) {
            if (unit || q_w || temp_every > 0)
                for (int d = lane; d < D; d += 32) x[d] = from_f32<T>(to_f32(x[d]) * r * (q_w ? q_w[d] : 1.f) * temp);
        } else if (k_cache) {
            T* dst = k_cache + ((page * KV + (u - H)) * ps + off) * D;
            for (int d = lane; d < D; d += 32) dst[d] = from_f32<T>(to_f32(x[d]) * r * (k_w ? k_w[d] : 1.f));
            if (v_is_k && v_cache) {                           // the values are these keys as projected
                T* vd = v_cache + ((page * KV + (u - H)) * ps + off) * D;
                for (int d = lane; d < D; d += 32) vd[d] = x[d];
            }
        }
    }
    if (!v_cache || v_is_k) return;
    const float l = lam ? lam[0] : 0.f;
    const T* v = row + (size_t)(H + KV) * D;
    const T* vs = v_src ? v_src + (size_t)t * ld_src : nullptr;
    for (int i = threadIdx.x; i < KV * Dv; i += blockDim.x) {
        float val = to_f32(v[i]);
        if (vs) val = (1.f - l) * val + l * to_f32(vs[i]);
        v_cache[((page * KV + i / Dv) * ps + off) * Dv + i % Dv] = from_f32<T>(val);
    }
}

}  // namespace

// q_w, k_w: float32 [D] or null; positions with temp_every > 0: the query temperature; v_is_k: p has no v columns, Dv == D
MI_EXPORT int mi_normed_qk_cache(void* p, int ldp, const void* v_src, int ld_src, const float* lam, const int* slots, void* k_cache,
                                 void* v_cache, int T_, int H, int KV, int D, int Dv, int ps, float eps, int unit, const float* q_w,
                                 const float* k_w, const int* positions, float temp_coef, int temp_every, int v_is_k, int dtype,
                                 cudaStream_t stream) {
    if (T_ == 0) return 0;
    if ((v_is_k && (Dv != D || v_src)) || (temp_every > 0 && !positions) || ((q_w == nullptr) != (k_w == nullptr))) return -2;
    // few tokens (decode steps): a warp per head, so that no warp walks several heads one after the other
    const int nt = T_ >= 256 ? 128 : min(1024, max(128, 32 * (H + KV)));
    if (dtype == MI_BF16)
        unit_qk_cache_kernel<__nv_bfloat16><<<T_, nt, 0, stream>>>((__nv_bfloat16*)p, ldp, (const __nv_bfloat16*)v_src, ld_src, lam, slots,
                                                                    (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, H, KV, D, Dv, ps, eps, unit,
                                                                    q_w, k_w, positions, temp_coef, temp_every, v_is_k);
    else
        unit_qk_cache_kernel<float><<<T_, nt, 0, stream>>>((float*)p, ldp, (const float*)v_src, ld_src, lam, slots, (float*)k_cache,
                                                           (float*)v_cache, H, KV, D, Dv, ps, eps, unit, q_w, k_w, positions, temp_coef,
                                                            temp_every, v_is_k);
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_unit_qk_cache(void* p, int ldp, const void* v_src, int ld_src, const float* lam, const int* slots, void* k_cache,
                               void* v_cache, int T_, int H, int KV, int D, int Dv, int ps, float eps, int unit, int dtype,
                               cudaStream_t stream) {
    return mi_normed_qk_cache(p, ldp, v_src, ld_src, lam, slots, k_cache, v_cache, T_, H, KV, D, Dv, ps, eps, unit, nullptr, nullptr, nullptr,
                              0.f, 0, 0, dtype, stream);
}

MI_EXPORT int mi_masked_prefill(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out, const int* tiles,
                                int num_tiles, const int* seg_q_start, const int* seg_pos0, const int* block_table,
                                const int* table_rows, int table_stride, int H, int KV, int D, int Dv, int ps, int tile_rows, float scale,
                                int block, int window, int sink, const float* sink_values, const float* bias, int bias_last,
                                const float* slopes, int dtype, cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    if (D > MAX_D || Dv > MAX_D || H > 65535) return -2;
    dim3 grid(num_tiles, H);
#define ARGS(T) (const T*)q, q_stride, (const T*)k_cache, (const T*)v_cache, (T*)out, tiles, seg_q_start, seg_pos0, block_table, table_rows, \
        table_stride, H, KV, D, Dv, ps, tile_rows, scale, block, window, sink, sink_values, bias, bias_last, slopes
    if (dtype == MI_BF16) masked_prefill_kernel<__nv_bfloat16><<<grid, WARPS * 32, 0, stream>>>(ARGS(__nv_bfloat16));
    else masked_prefill_kernel<float><<<grid, WARPS * 32, 0, stream>>>(ARGS(float));
#undef ARGS
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_masked_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out, float* o_part,
                               float* lse_part, const int* decode_segs, int num_decode, const int* seg_q_start, const int* seg_kv_len,
                               const int* block_table, const int* table_rows, int table_stride, int H, int KV, int D, int Dv, int ps,
                               int splits, float scale, int block, int window, int sink, const float* sink_values, const float* bias,
                               int bias_last, const float* slopes, int dtype, cudaStream_t stream) {
    if (num_decode == 0) return 0;
    if (D > MAX_D || Dv > MAX_D || H > 65535 * WARPS) return -2;
    dim3 grid(num_decode, (H + WARPS - 1) / WARPS, splits);
#define ARGS(T) (const T*)q, q_stride, (const T*)k_cache, (const T*)v_cache, (T*)out, o_part, lse_part, decode_segs, seg_q_start, seg_kv_len, \
        block_table, table_rows, table_stride, H, KV, D, Dv, ps, scale, block, window, sink, sink_values, bias, bias_last, slopes
    if (dtype == MI_BF16) masked_decode_kernel<__nv_bfloat16><<<grid, WARPS * 32, 0, stream>>>(ARGS(__nv_bfloat16));
    else masked_decode_kernel<float><<<grid, WARPS * 32, 0, stream>>>(ARGS(float));
#undef ARGS
    int err = (int)cudaGetLastError();
    if (err || splits == 1) return err;
    dim3 mgrid(num_decode, H);
    if (dtype == MI_BF16)
        masked_merge_kernel<__nv_bfloat16><<<mgrid, 128, 0, stream>>>(o_part, lse_part, (__nv_bfloat16*)out, decode_segs, seg_q_start, H, Dv, splits, sink, sink_values);
    else
        masked_merge_kernel<float><<<mgrid, 128, 0, stream>>>(o_part, lse_part, (float*)out, decode_segs, seg_q_start, H, Dv, splits, sink, sink_values);
    return (int)cudaGetLastError();
}
