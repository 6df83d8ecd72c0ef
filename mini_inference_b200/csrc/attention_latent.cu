// Latent attention over a one-plane paged cache: every token caches ONE row [c (C entries) | kr (R entries)]; all H
// query heads attend over these shared rows with queries of size C + R (the key up-projection absorbed into the
// query) and the weighted sum is taken over the first C entries of the same rows (the value up-projection is
// applied afterwards, per head).  Any C and R; float32 or bfloat16 storage; scores, softmax and sums in float32 on
// the CUDA cores in an order that depends only on the request's own positions.  Sizes that the tensor-core paged
// attention kernels take (C + R of 64 or 128, bfloat16) are sent there by the kernel namespace instead.
//
// Cache layout: [pages, 1, page_size, C + R]; the row of key j of a request is at (table[j / ps] * ps + j % ps) * (C + R).
// Output: element d of head h of token t goes to out[h * out_hs + t * out_ts + d] ([H, T, C]: out_hs = T C, out_ts = C, what the
// per-head value up-projection reads as a batch of matrices; or a [T, H, C + R] buffer shared with another kernel's output).
#include "common.cuh"
#include <math.h>

using namespace mi;

namespace {

constexpr int WARPS = 4;

// ------------------------------------------------------------------ per token: latent norm, rotations, cache write, query assembly
// p [T, ldp]: q heads [H, D + R] | dkv [C + R] | ...;  q_abs [H, T, C] (the absorbed unrotated queries).
// q_out [T, H, C + R] = [q_abs | rotate(q rot part)];  cache row = [rmsnorm(dkv[:C]) * w | rotate(dkv[C:])].
// Interleaved rotation: pairs (2i, 2i+1), i < nf, by the angle pos * inv_freq[i]; entries from 2 nf on pass unchanged.
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ p, int ldp, const T* __restrict__ q_rows, int ldq, int dkv_col,
                                      const T* __restrict__ q_abs, T* __restrict__ q_out,
                                      T* __restrict__ cache, const float* __restrict__ norm_w, const float* __restrict__ inv_freq,
                                      int nf, const int* __restrict__ positions, const int* __restrict__ slots, int T_, int H,
                                      int D, int R, int C, float eps) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const T* row = p + (size_t)t * ldp;
    const T* qrow = q_rows + (size_t)t * ldq;              // the query heads as projected: p itself, or a tensor of their own
    const float pos = (float)positions[t];
    T* qo = q_out + (size_t)t * H * (C + R);
    for (int idx = threadIdx.x; idx < H * C; idx += blockDim.x) {
        const int h = idx / C, i = idx - h * C;
        qo[(size_t)h * (C + R) + i] = q_abs[((size_t)h * T_ + t) * C + i];
    }
    for (int idx = threadIdx.x; idx < H * R; idx += blockDim.x) {
        const int h = idx / R, j = idx - h * R;
        const T* src = qrow + (size_t)h * (D + R) + D;
        float val = to_f32(src[j]);
        if (j < 2 * nf) {
            float sn, cs;
            sincosf(pos * inv_freq[j >> 1], &sn, &cs);
            const float other = to_f32(src[j ^ 1]);
            val = (j & 1) ? val * cs + other * sn : val * cs - other * sn;
        }
        qo[(size_t)h * (C + R) + C + j] = from_f32<T>(val);
    }
    if (cache == nullptr) return;
    const T* dkv = row + dkv_col;
    float ss = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) { const float v = to_f32(dkv[i]); ss += v * v; }
    const float r = rsqrtf(block_sum<128>(ss, scratch) / C + eps);
    T* crow = cache + (size_t)slots[t] * (C + R);
    for (int i = threadIdx.x; i < C; i += blockDim.x) crow[i] = from_f32<T>(to_f32(dkv[i]) * r * norm_w[i]);
    for (int j = threadIdx.x; j < R; j += blockDim.x) {
        float val = to_f32(dkv[C + j]);
        if (j < 2 * nf) {
            float sn, cs;
            sincosf(pos * inv_freq[j >> 1], &sn, &cs);
            const float other = to_f32(dkv[C + (j ^ 1)]);
            val = (j & 1) ? val * cs + other * sn : val * cs - other * sn;
        }
        crow[C + j] = from_f32<T>(val);
    }
}

// One warp, one query row of one head, keys lo..hi-1.  q_s: the query times scale (shared memory, Dk floats).
// Lane j of a chunk scores key j0 + j; outputs are spread over lanes as d = lane + 32 k, d < Dv.
template <typename T, int NV>
__device__ __forceinline__ void attend_rows(const float* q_s, const T* __restrict__ cache, const int* __restrict__ table_row,
                                            int Dk, int Dv, int ps, bool vec, int lo, int hi, float& m, float& l, float (&acc)[NV]) {
    const int lane = threadIdx.x & 31;
    constexpr int VN = Vec16<T>::N;
    for (int j0 = lo; j0 < hi; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j < hi;
        long long off = 0;
        float s = -INFINITY;
        if (valid) {
            off = ((long long)table_row[j / ps] * ps + j % ps) * Dk;
            const T* kr = cache + off;
            float dot = 0.f;
            if (vec) {
                float tmp[VN];
                for (int c = 0; c < Dk; c += VN) {
                    load16(kr + c, tmp);
#pragma unroll
                    for (int e = 0; e < VN; ++e) dot += q_s[c + e] * tmp[e];
                }
            } else {
                for (int c = 0; c < Dk; ++c) dot += q_s[c] * to_f32(kr[c]);
            }
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float alpha = expf(m - m_new);              // first chunk: exp(-inf) = 0
        const float pw = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(pw);
        m = m_new;
#pragma unroll
        for (int k = 0; k < NV; ++k) acc[k] *= alpha;
        const int n = min(32, hi - j0);
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, pw, jj);
            const long long voff = __shfl_sync(0xffffffffu, off, jj);
            const T* vr = cache + voff;
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                const int d = lane + 32 * k;
                if (d < Dv) acc[k] += pj * to_f32(vr[d]);
            }
        }
    }
}

// grid (tiles, H): tile = (entry, first row); each warp takes rows of the tile in turn.  Causal, no window.
template <typename T, int NV>
__global__ void latent_prefill_kernel(const T* __restrict__ q, const T* __restrict__ cache, T* __restrict__ out,
                                      const int* __restrict__ tiles, const int* __restrict__ seg_q_start,
                                      const int* __restrict__ seg_pos0, const int* __restrict__ block_table,
                                      const int* __restrict__ table_rows, int table_stride, long long out_hs, long long out_ts, int H, int Dk, int Dv, int ps,
                                      int tile_rows, float scale, int vec) {
    extern __shared__ float q_sm[];                      // [WARPS, Dk]
    const int seg = tiles[2 * blockIdx.x], r0 = tiles[2 * blockIdx.x + 1];
    const int h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* q_s = q_sm + warp * Dk;
    const int qs = seg_q_start[seg], n = seg_q_start[seg + 1] - qs, pos0 = seg_pos0[seg];
    const int* table_row = block_table + (size_t)table_rows[seg] * table_stride;
    const int r_end = min(r0 + tile_rows, n);
    for (int r = r0 + warp; r < r_end; r += WARPS) {
        const int tok = qs + r, pq = pos0 + r;
        const T* qr = q + ((size_t)tok * H + h) * Dk;
        for (int d = lane; d < Dk; d += 32) q_s[d] = to_f32(qr[d]) * scale;
        __syncwarp();
        float m = -INFINITY, l = 0.f, acc[NV];
#pragma unroll
        for (int k = 0; k < NV; ++k) acc[k] = 0.f;
        attend_rows<T, NV>(q_s, cache, table_row, Dk, Dv, ps, vec != 0, 0, pq + 1, m, l, acc);
        T* orow = out + h * out_hs + tok * out_ts;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int d = lane + 32 * k;
            if (d < Dv) orow[d] = from_f32<T>(acc[k] / l);
        }
        __syncwarp();
    }
}

// grid (decode entries, ceil(H / WARPS), splits); one warp per query head; every request cuts ITS OWN keys into
// `splits` pieces of whole 32-key chunks, so the grid depends on the batch only.
template <typename T, int NV>
__global__ void latent_decode_kernel(const T* __restrict__ q, const T* __restrict__ cache, T* __restrict__ out,
                                     float* __restrict__ o_part, float* __restrict__ lse_part, const int* __restrict__ decode_segs,
                                     const int* __restrict__ seg_q_start, const int* __restrict__ seg_kv_len,
                                     const int* __restrict__ block_table, const int* __restrict__ table_rows, int table_stride,
                                     long long out_hs, long long out_ts, int H, int Dk, int Dv, int ps, float scale, int vec) {
    extern __shared__ float q_sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y * WARPS + warp;
    if (h >= H) return;
    float* q_s = q_sm + warp * Dk;
    const int seg = decode_segs[blockIdx.x];
    const int tok = seg_q_start[seg], len = seg_kv_len[seg];
    const int S = gridDim.z, s = blockIdx.z;
    const int piece = ((len + S - 1) / S + 31) / 32 * 32;
    const int lo = s * piece, hi = min(lo + piece, len);
    const T* qr = q + ((size_t)tok * H + h) * Dk;
    for (int d = lane; d < Dk; d += 32) q_s[d] = to_f32(qr[d]) * scale;
    __syncwarp();
    float m = -INFINITY, l = 0.f, acc[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) acc[k] = 0.f;
    if (lo < hi)
        attend_rows<T, NV>(q_s, cache, block_table + (size_t)table_rows[seg] * table_stride, Dk, Dv, ps, vec != 0, lo, hi, m, l, acc);
    const float inv = l > 0.f ? 1.f / l : 0.f;                  // empty piece: output 0, lse -inf
    if (S == 1) {
        T* orow = out + h * out_hs + tok * out_ts;
#pragma unroll
        for (int k = 0; k < NV; ++k) { const int d = lane + 32 * k; if (d < Dv) orow[d] = from_f32<T>(acc[k] * inv); }
    } else {
        const size_t idx = ((size_t)blockIdx.x * H + h) * S + s;
        float* orow = o_part + idx * Dv;
#pragma unroll
        for (int k = 0; k < NV; ++k) { const int d = lane + 32 * k; if (d < Dv) orow[d] = acc[k] * inv; }
        if (lane == 0) lse_part[idx] = l > 0.f ? m + logf(l) : -INFINITY;
    }
}

// out = sum_s e^(lse_s - max) o_s / sum_s e^(lse_s - max), in split order
template <typename T>
__global__ void latent_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ lse_part, T* __restrict__ out,
                                    const int* __restrict__ decode_segs, const int* __restrict__ seg_q_start, long long out_hs, long long out_ts, int H, int Dv, int S) {
    const int i = blockIdx.x, h = blockIdx.y;
    const int tok = seg_q_start[decode_segs[i]];
    const size_t base = ((size_t)i * H + h) * S;
    float mx = -INFINITY;
    for (int s = 0; s < S; ++s) mx = fmaxf(mx, lse_part[base + s]);
    float den = 0.f;
    for (int s = 0; s < S; ++s) den += expf(lse_part[base + s] - mx);
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        float num = 0.f;
        for (int s = 0; s < S; ++s) num += expf(lse_part[base + s] - mx) * o_part[(base + s) * Dv + d];
        out[h * out_hs + tok * out_ts + d] = from_f32<T>(num / den);
    }
}

}  // namespace

// q_rows (row stride ldq): where the query heads [H, D + R] as projected lie (null: at the start of p); dkv_col: the column of p
// at which [c as projected | kr] starts (negative: behind the query heads, H (D + R)).
MI_EXPORT int mi_latent_prepare(const void* p, int ldp, const void* q_rows, int ldq, int dkv_col, const void* q_abs, void* q_out, void* cache,
                                const float* norm_w, const float* inv_freq, int nf, const int* positions, const int* slots, int T_, int H,
                                int D, int R, int C, float eps, int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    if (!q_rows) { q_rows = p; ldq = ldp; }
    if (dkv_col < 0) dkv_col = H * (D + R);
    if (dtype == MI_BF16)
        latent_prepare_kernel<__nv_bfloat16><<<T_, 128, 0, stream>>>((const __nv_bfloat16*)p, ldp, (const __nv_bfloat16*)q_rows, ldq, dkv_col,
                                                                     (const __nv_bfloat16*)q_abs, (__nv_bfloat16*)q_out,
                                                                     (__nv_bfloat16*)cache, norm_w, inv_freq, nf, positions, slots, T_, H, D, R, C, eps);
    else
        latent_prepare_kernel<float><<<T_, 128, 0, stream>>>((const float*)p, ldp, (const float*)q_rows, ldq, dkv_col, (const float*)q_abs,
                                                             (float*)q_out, (float*)cache, norm_w, inv_freq, nf, positions, slots, T_, H, D, R, C, eps);
    return (int)cudaGetLastError();
}

#define LATENT_PICK_NV(CALL) do { if (Dv <= 64) { CALL(2); } else if (Dv <= 128) { CALL(4); } else if (Dv <= 256) { CALL(8); } else { CALL(16); } } while (0)

MI_EXPORT int mi_latent_prefill(const void* q, const void* cache, void* out, const int* tiles, int num_tiles, const int* seg_q_start,
                                const int* seg_pos0, const int* block_table, const int* table_rows, int table_stride, long long out_hs,
                                long long out_ts, int H, int C, int R, int ps, int tile_rows, float scale, int dtype, cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    const int Dk = C + R, Dv = C;
    if (Dv > 512 || Dk > 2048 || H > 65535) return -2;
    const int el = dtype == MI_BF16 ? 2 : 4;
    const int vec = (Dk * el) % 16 == 0;
    const size_t smem = (size_t)WARPS * Dk * sizeof(float);
    dim3 grid(num_tiles, H);
#define CALL(NV) do { \
        if (dtype == MI_BF16) latent_prefill_kernel<__nv_bfloat16, NV><<<grid, WARPS * 32, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, \
            (__nv_bfloat16*)out, tiles, seg_q_start, seg_pos0, block_table, table_rows, table_stride, out_hs, out_ts, H, Dk, Dv, ps, tile_rows, scale, vec); \
        else latent_prefill_kernel<float, NV><<<grid, WARPS * 32, smem, stream>>>((const float*)q, (const float*)cache, (float*)out, tiles, seg_q_start, \
            seg_pos0, block_table, table_rows, table_stride, out_hs, out_ts, H, Dk, Dv, ps, tile_rows, scale, vec); } while (0)
    LATENT_PICK_NV(CALL);
#undef CALL
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_latent_decode(const void* q, const void* cache, void* out, float* o_part, float* lse_part, const int* decode_segs,
                               int num_decode, const int* seg_q_start, const int* seg_kv_len, const int* block_table,
                               const int* table_rows, int table_stride, long long out_hs, long long out_ts, int H, int C, int R, int ps, int splits,
                               float scale, int dtype, cudaStream_t stream) {
    if (num_decode == 0) return 0;
    const int Dk = C + R, Dv = C;
    if (Dv > 512 || Dk > 2048 || H > 65535 * WARPS) return -2;
    const int el = dtype == MI_BF16 ? 2 : 4;
    const int vec = (Dk * el) % 16 == 0;
    const size_t smem = (size_t)WARPS * Dk * sizeof(float);
    dim3 grid(num_decode, (H + WARPS - 1) / WARPS, splits);
#define CALL(NV) do { \
        if (dtype == MI_BF16) latent_decode_kernel<__nv_bfloat16, NV><<<grid, WARPS * 32, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, \
            (__nv_bfloat16*)out, o_part, lse_part, decode_segs, seg_q_start, seg_kv_len, block_table, table_rows, table_stride, out_hs, out_ts, H, Dk, Dv, ps, scale, vec); \
        else latent_decode_kernel<float, NV><<<grid, WARPS * 32, smem, stream>>>((const float*)q, (const float*)cache, (float*)out, o_part, lse_part, \
            decode_segs, seg_q_start, seg_kv_len, block_table, table_rows, table_stride, out_hs, out_ts, H, Dk, Dv, ps, scale, vec); } while (0)
    LATENT_PICK_NV(CALL);
#undef CALL
    int err = (int)cudaGetLastError();
    if (err || splits == 1) return err;
    dim3 mgrid(num_decode, H);
    if (dtype == MI_BF16)
        latent_merge_kernel<__nv_bfloat16><<<mgrid, 128, 0, stream>>>(o_part, lse_part, (__nv_bfloat16*)out, decode_segs, seg_q_start, out_hs, out_ts, H, Dv, splits);
    else
        latent_merge_kernel<float><<<mgrid, 128, 0, stream>>>(o_part, lse_part, (float*)out, decode_segs, seg_q_start, out_hs, out_ts, H, Dv, splits);
    return (int)cudaGetLastError();
}
