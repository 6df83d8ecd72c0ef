// Grouped products of routed experts on the tcgen05 tensor cores, for steps in which an expert gets many rows.
//
// The (token, choice) pairs have been sorted by expert, every expert's rows starting on a multiple of 128 (csrc/moe.cu,
// moe_align), so a tile of 128 sorted rows belongs to ONE expert and both operands of its product are plain 2-D boxes:
// rows [pos0, pos0 + 128) of the sorted activations and 256 rows of that expert's matrix.  One block per (row tile,
// 256 accumulator columns), two blocks to an SM (two ring stages of 48 KB and 256 of the 512 tensor-memory columns each), so that one
// block's start-up and epilogue run under the other's products: a TMA thread fills the ring (K in steps of 64, 128-byte swizzle), one thread issues
// tcgen05.mma (M = 128, N = 256, accumulator in tensor memory), and the block's eight warps read the accumulator back
// (a warp reaches the 32 lanes of its quarter; two warps share a quarter and take half of the columns each) and write the
// result.  With four warps and the exact exponential and division the epilogue of a tile took longer than its products
// (knock-out builds: the whole op 247 us; without loads 258; without loads and epilogue 125): a thread per row is a long
// chain of dependent instructions with one warp per scheduler to hide it.  Hence eight warps and the fast exponential and
// reciprocal, whose error (2^-21 relative) is far below the bfloat16 rounding of the result (212 us).  What is left is the
// operands' way through shared memory: a block that feeds M = 128 / N = 256 products from its own shared memory reads 96 bytes a
// clock while TMA writes as much, against the 128 an SM has (without loads the products run at the pipe's rate: 125 us for the op).
//   MODE 0 ("in"):  A = tokens gathered into sorted order [positions, K]; the expert's matrix is [gate rows | up rows];
//                   the 256 accumulator columns are 128 gate columns and the 128 up columns of the SAME outputs, and the
//                   epilogue writes g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(slope * g) * (u + 1).
//   MODE 1 ("out"): A = those activated rows; 256 output columns; a row is written to its pair's own row of the result.
// A block whose tile has no expert (the grid covers the most tiles there can be) leaves at once.  Every wait is bounded;
// a wait that runs out sets the error word and the block still frees its tensor memory.
#include "sm100.cuh"
#include <math.h>

using namespace mi;
using namespace mi::sm100;

namespace {

constexpr int GM = 128, GK = 64, GSTAGES = 2;
constexpr int GA_BYTES = GM * GK * 2, GB_BYTES = 256 * GK * 2, GSTAGE_BYTES = GA_BYTES + GB_BYTES;
constexpr int GTMEM_COLS = 256;

__device__ __forceinline__ float gated(float g, float u, float limit, float slope, float shift) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * __frcp_rn(1.f + __expf(-slope * g)) * (u + shift);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int MODE>
__global__ void __launch_bounds__(256, 2)
moe_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap, __nv_bfloat16* __restrict__ out,
                        int ldo, const int* __restrict__ sorted_pair, const int* __restrict__ tile_expert, int N, int K, float limit,
                        float slope, float shift, int* __restrict__ error_word) {
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    extern __shared__ unsigned char gsm_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)gsm_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + GSTAGES * GSTAGE_BYTES);        // full[], empty[], acc
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GSTAGES + 1);
    const uint32_t s0 = smem_u32(base), full = smem_u32(bars), empty = smem_u32(bars + GSTAGES), acc_bar = smem_u32(bars + 2 * GSTAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos0 = blockIdx.x * GM;
    const int n0 = blockIdx.y * (MODE == 0 ? 128 : 256);
    // rows of the stacked matrices [E * rows per expert, K]: the two boxes of 128 rows that make the 256 accumulator columns
    const int row_b0 = MODE == 0 ? e * 2 * N + n0 : e * N + n0;
    const int row_b1 = MODE == 0 ? e * 2 * N + N + n0 : e * N + n0 + 128;
    const int steps = K / GK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GSTAGES; ++s) { mbar_init(full + 8 * s, 1); mbar_init(empty + 8 * s, 1); }
        mbar_init(acc_bar, 1);
        mbar_init_fence();
        tma_prefetch_desc(&amap); tma_prefetch_desc(&bmap);
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), GTMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (threadIdx.x == 0) {
        // ---------------- loads
        for (int it = 0; it < steps; ++it) {
            const int s = it % GSTAGES;
            if (it >= GSTAGES && !mbar_wait(empty + 8 * s, ((it / GSTAGES) - 1) & 1)) { atomicExch(error_word, 61); break; }
            const uint32_t a = s0 + s * GSTAGE_BYTES, b = a + GA_BYTES;
            mbar_expect_tx(full + 8 * s, GSTAGE_BYTES);
            tma_load_2d(a, &amap, it * GK, pos0, full + 8 * s);
            tma_load_2d(b, &bmap, it * GK, row_b0, full + 8 * s);
            tma_load_2d(b + GB_BYTES / 2, &bmap, it * GK, row_b1, full + 8 * s);
        }
    } else if (threadIdx.x == 32) {
        // ---------------- MMA issue
        const uint32_t idesc = umma_idesc_bf16(GM, 256, false);
        bool ok = true;
        for (int it = 0; it < steps && ok; ++it) {
            const int s = it % GSTAGES;
            if (!mbar_wait(full + 8 * s, (it / GSTAGES) & 1)) { atomicExch(error_word, 62); ok = false; break; }
            tc_fence_after();
            const uint32_t a = s0 + s * GSTAGE_BYTES, b = a + GA_BYTES;
#pragma unroll
            for (int ks = 0; ks < GK / 16; ++ks)
                umma_ss(tmem, umma_desc_sw128(a + ks * 32, 16, 1024), umma_desc_sw128(b + ks * 32, 16, 1024), idesc, (it | ks) != 0);
            umma_commit(empty + 8 * s);                    // the stage is free once these products have run
        }
        umma_commit(acc_bar);                              // and the accumulator is whole
    }
    __syncwarp();
    // ---------------- epilogue: thread t of warp w owns row 32 (w % 4) + t (tensor-memory lane of the same number) and the
    // half w / 4 of the columns
    const bool ok = mbar_wait(acc_bar, 0);
    if (!ok && lane == 0) atomicExch(error_word, 63);
    tc_fence_after();
    if (ok) {
        const int quarter = warp & 3, part = warp >> 2;
        const int r = quarter * 32 + lane;
        const int pr = sorted_pair[pos0 + r];
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        if (MODE == 0) {
            __nv_bfloat16* orow = out + (size_t)(pos0 + r) * ldo;
#pragma unroll 1
            for (int c = 2 * part; c < 2 * part + 2; ++c) {
                uint32_t g[32], u[32];
                tmem_ld32(lane_addr + c * 32, g);
                tmem_ld32(lane_addr + 128 + c * 32, u);
                tmem_wait_ld();
#pragma unroll
                for (int v4 = 0; v4 < 4; ++v4) {
                    const int col = n0 + c * 32 + v4 * 8;
                    uint4 w;
                    uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        wp[j] = pack_bf16x2(gated(__uint_as_float(g[v4 * 8 + 2 * j]), __uint_as_float(u[v4 * 8 + 2 * j]), limit, slope, shift),
                                            gated(__uint_as_float(g[v4 * 8 + 2 * j + 1]), __uint_as_float(u[v4 * 8 + 2 * j + 1]), limit, slope, shift));
                    if (pr >= 0 && col < N) *reinterpret_cast<uint4*>(orow + col) = w;
                }
            }
        } else {
            __nv_bfloat16* orow = out + (size_t)(pr >= 0 ? pr : 0) * ldo;
#pragma unroll 1
            for (int c = 4 * part; c < 4 * part + 4; ++c) {
                uint32_t o[32];
                tmem_ld32(lane_addr + c * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int v4 = 0; v4 < 4; ++v4) {
                    const int col = n0 + c * 32 + v4 * 8;
                    uint4 w;
                    uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
                    for (int j = 0; j < 4; ++j) wp[j] = pack_bf16x2(__uint_as_float(o[v4 * 8 + 2 * j]), __uint_as_float(o[v4 * 8 + 2 * j + 1]));
                    if (pr >= 0 && col < N) *reinterpret_cast<uint4*>(orow + col) = w;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, GTMEM_COLS);
}

// sorted[pos] = h[sorted_pair[pos] / top] (zeros where the position is padding): the rows of the first grouped product
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ h, int ldh, const int* __restrict__ sorted_pair, int top,
                                       __nv_bfloat16* __restrict__ sorted, int K, const float* __restrict__ weights) {
    const int pr = sorted_pair[blockIdx.x];
    uint4* dst = reinterpret_cast<uint4*>(sorted + (size_t)blockIdx.x * K);
    if (pr < 0) {
        for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(pr / top) * ldh);
    if (!weights) {
        for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = src[i];
        return;
    }
    const float w = weights[pr];                                    // the pair's score multiplies the expert's input
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
        uint4 raw = src[i];
        __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(v[j]); v[j] = __floats2bfloat162_rn(w * f.x, w * f.y); }
        dst[i] = raw;
    }
}

}  // namespace

MI_EXPORT int mi_moe_gather_rows(const void* h, int ldh, const int* sorted_pair, int top, void* sorted, int cap_pos, int K, const float* weights,
                                 cudaStream_t stream) {
    if (cap_pos == 0) return 0;
    if (K % 8 || ldh % 8 || ((uintptr_t)h % 16) || ((uintptr_t)sorted % 16)) return -2;
    moe_gather_rows_kernel<<<cap_pos, 128, 0, stream>>>((const __nv_bfloat16*)h, ldh, sorted_pair, top, (__nv_bfloat16*)sorted, K, weights);
    return (int)cudaGetLastError();
}

// A [cap_tiles * 128, K] contiguous bfloat16 (sorted rows); W [E, mode 0 ? 2 N : N, K] contiguous; out: mode 0 [cap_tiles * 128, N]
// (ldo = N), mode 1 [pairs, N].  K % 64 == 0, N % 8 == 0.
MI_EXPORT int mi_moe_gemm_tcgen05(const void* A, const void* W, int E, void* out, int ldo, const int* sorted_pair, const int* tile_expert,
                                  int cap_tiles, int N, int K, float limit, float slope, float shift, int mode, int* error_word, cudaStream_t stream) {
    if (cap_tiles == 0) return 0;
    if (K % GK || K < GK || N % 8 || ldo % 8 || ((uintptr_t)A % 16) || ((uintptr_t)W % 16) || ((uintptr_t)out % 16)) return -2;
    CUtensorMap amap, bmap;
    if (!sm100_host::make_map_bf16(&amap, A, (uint64_t)cap_tiles * GM, K, K, GM, GK)) return -5;
    if (!sm100_host::make_map_bf16(&bmap, W, (uint64_t)E * (mode == 0 ? 2 : 1) * N, K, K, 128, GK)) return -5;
    const size_t smem = (size_t)GSTAGES * GSTAGE_BYTES + 1024 + 256;
    dim3 grid(cap_tiles, (N + (mode == 0 ? 128 : 256) - 1) / (mode == 0 ? 128 : 256));
    if (grid.y > 65535) return -2;
    static bool configured[2] = {false, false};
#define GO(MODE) do { \
        if (!configured[MODE]) { \
            cudaError_t err = cudaFuncSetAttribute(moe_gemm_tcgen05_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (err != cudaSuccess) return (int)err; \
            configured[MODE] = true; \
        } \
        moe_gemm_tcgen05_kernel<MODE><<<grid, 256, smem, stream>>>(amap, bmap, (__nv_bfloat16*)out, ldo, sorted_pair, tile_expert, N, K, limit, \
                                                                  slope, shift, error_word); } while (0)
    if (mode == 0) GO(0); else GO(1);
#undef GO
    return (int)cudaGetLastError();
}
