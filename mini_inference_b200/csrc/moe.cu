// Routed feed-forward: a float32 router with group-limited top-k choice, a device-side sort of the (token, choice)
// pairs by expert, two grouped products over the sorted rows, and the weighted sum per token.
//
//   route_topk   one block per token: logits = W_r h as float32 sums in a fixed order, s = softmax over all experts,
//                choice scores c = s + correction; with groups, only experts of the `keep` groups (equal groups of
//                neighbouring experts) whose largest c (or, as an option, the sum of whose two largest c) is largest stay eligible (the others count as -inf); the `top`
//                largest c are chosen (ties: the lower index); the weights are the chosen experts' s, as they are.
//                Options: s = sigmoid(logit) per expert instead of the softmax; no correction; `extra` further rows behind the
//                experts' rows of the router matrix whose float32 logits are handed out as they are (a gate that reads the
//                same input rides along in the router's pass).
//   scale rows   a design whose scores multiply the experts' INPUTS: row p = weight[p] * h[p / top] per pair, rounded to the
//                run's dtype; the products then run with one choice per row and the sum adds the rows unweighted.
//   align        pairs p = token * top + j counted per expert; every expert's rows start on a multiple of the row tile
//                (padding rows are marked -1), so a tile of rows belongs to ONE expert: tile_expert[tile] (-1 past the end).
//                Nothing returns to the host: the grids of the products cover the most tiles there can be, and a block
//                whose tile has no expert leaves at once.
//   grouped in   rows gathered by token; per expert [gate rows | up rows]; the epilogue applies
//                g = min(gate, limit), u = clamp(up, -limit, limit), y = g * sigmoid(slope * g) * (u + shift)  (shift 1 with finite limits; shift 0, slope 1 and no limit: silu(gate) * up).
//   grouped out  y rows times the expert's down matrix, written to the pair's own row (so the order of pairs inside an
//                expert's segment, which comes from atomics, does not reach the result).
//   combine      out[t] = sum_j weight[t, j] * row[t * top + j] (+ the shared expert's row), float32, in the order of choice.
//
// The products exist in two forms: bfloat16 operands on mma.sync tensor-core tiles (float32 accumulation), and a plain
// float32 form on the CUDA cores (true 32-bit, sums in a fixed order along K) that also takes bfloat16 shapes the first
// does not.
#include "common.cuh"
#include <limits.h>
#include <math.h>

using namespace mi;

namespace {

// ------------------------------------------------------------------ router
// (value, index) of the best candidate over a warp: the larger value, on a tie the lower index; index INT_MAX: none
__device__ __forceinline__ void warp_best(float& bv, int& bi) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != INT_MAX && (bi == INT_MAX || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
}

// One warp makes one token's choice from its logits s[E] (left as softmax scores); c and gb are scratch of E floats each.
__device__ __forceinline__ void warp_choose(float* s, float* c, float* gb, const float* __restrict__ corr, int E, int top, int g_count,
                                            int g_keep, int* __restrict__ chosen, float* __restrict__ weights, int lane, int sigmoid_scores,
                                            int group_top2, int renorm, float weight_eps, float route_scale) {
    if (sigmoid_scores) {
        for (int e = lane; e < E; e += 32) { s[e] = 1.f / (1.f + expf(-s[e])); c[e] = corr ? s[e] + corr[e] : s[e]; }
    } else {
        float mx = -INFINITY, den = 0.f;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
        mx = warp_max(mx);
        for (int e = lane; e < E; e += 32) { const float v = expf(s[e] - mx); s[e] = v; den += v; }
        den = warp_sum(den);
        for (int e = lane; e < E; e += 32) { s[e] = s[e] / den; c[e] = corr ? s[e] + corr[e] : s[e]; }
    }
    __syncwarp();
    if (g_count > 0) {
        const int per = E / g_count;
        for (int g = lane; g < g_count; g += 32) {
            float b = -INFINITY, b2 = -INFINITY;               // the largest and the second largest choice score of the group
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = c[e];
                if (v > b) { b2 = b; b = v; } else if (v > b2) b2 = v;
            }
            gb[g] = group_top2 && per > 1 ? b + b2 : b;
        }
        __syncwarp();
        for (int k = 0; k < g_keep; ++k) {                 // a kept group's entry becomes +inf
            float bv = -INFINITY;
            int bi = INT_MAX;
            for (int g = lane; g < g_count; g += 32)
                if (gb[g] != INFINITY && (bi == INT_MAX || gb[g] > bv)) { bv = gb[g]; bi = g; }
            warp_best(bv, bi);
            __syncwarp();
            if (lane == 0 && bi != INT_MAX) gb[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gb[e / per] != INFINITY) c[e] = -INFINITY;
        __syncwarp();
    }
    for (int j = 0; j < top; ++j) {
        float bv = -INFINITY;
        int bi = INT_MAX;
        for (int e = lane; e < E; e += 32)
            if (!isnan(c[e]) && c[e] > -INFINITY && (bi == INT_MAX || c[e] > bv)) { bv = c[e]; bi = e; }
        warp_best(bv, bi);
        if (bi == INT_MAX) bi = 0;         // fewer eligible experts than `top`: the configuration reader refuses that
        __syncwarp();
        if (lane == 0) { chosen[j] = bi; weights[j] = s[bi]; c[bi] = NAN; }       // NaN: taken
        __syncwarp();
    }
    if (renorm || route_scale != 1.f) {                     // weights <- weights / (their sum + eps) * route_scale, summed in the order of choice
        if (lane == 0) {
            float sum = 0.f;
            for (int j = 0; j < top; ++j) sum += weights[j];
            for (int j = 0; j < top; ++j) weights[j] = renorm ? weights[j] / (sum + weight_eps) * route_scale : weights[j] * route_scale;
        }
        __syncwarp();
    }
}

// One block per TOK tokens: 8 warps for 8 tokens (prompt steps), up to a warp per expert for one token (decode steps, where the
// time is the chain of loads of one warp).  The tokens' rows wait in shared memory as float32; a warp takes experts in turn and
// reads an expert's router row ONCE for all TOK tokens (with one token per block every token would fetch the whole matrix
// again).  Sums are float32, per lane in steps of the row, then across the lanes in a fixed order, so a token's logits do
// not depend on its neighbours.  Warp i of the block then makes token i's choice.
template <typename T, int TOK>
__global__ void __launch_bounds__(TOK == 1 ? 1024 : 256) route_topk_kernel(const T* __restrict__ h, int ldh, const T* __restrict__ router, const float* __restrict__ corr,
                                                         int* __restrict__ chosen, float* __restrict__ weights, int T_, int hidden, int E, int top,
                                                         int g_count, int g_keep, int sigmoid_scores, int extra, float* __restrict__ extra_out,
                                                         int group_top2, int renorm, float weight_eps, float route_scale) {
    extern __shared__ __align__(16) float rsm[];
    const int EA = E + extra;                          // rows of the router matrix: the experts', then the extra ones
    float* hs = rsm;                                   // [TOK][hidden]
    float* sc = hs + (size_t)TOK * hidden;             // [TOK][3][EA]: logits -> scores, choice scores, group scratch
    const int t0 = blockIdx.x * TOK, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int nt = min(TOK, T_ - t0);
    for (int i = threadIdx.x; i < TOK * hidden; i += blockDim.x) {
        const int tk = i / hidden, c = i % hidden;
        hs[i] = tk < nt ? to_f32(h[(size_t)(t0 + tk) * ldh + c]) : 0.f;
    }
    __syncthreads();
    const bool vec = hidden % 4 == 0 && ((uintptr_t)router % 16) == 0;
    for (int e = warp; e < EA; e += nw) {
        const T* w = router + (size_t)e * hidden;
        float dot[TOK];
#pragma unroll
        for (int k = 0; k < TOK; ++k) dot[k] = 0.f;
        if (vec) {                                     // four neighbouring entries per lane and step: the lanes of a warp read one
#pragma unroll 4
            for (int i = lane * 4; i < hidden; i += 128) {         // contiguous piece of the row and of every token (no bank conflicts)
                float w0, w1, w2, w3;
                load2(w + i, w0, w1);
                load2(w + i + 2, w2, w3);
#pragma unroll
                for (int k = 0; k < TOK; ++k) {
                    const float4 hv = *reinterpret_cast<const float4*>(hs + (size_t)k * hidden + i);
                    dot[k] = fmaf(hv.x, w0, dot[k]); dot[k] = fmaf(hv.y, w1, dot[k]);
                    dot[k] = fmaf(hv.z, w2, dot[k]); dot[k] = fmaf(hv.w, w3, dot[k]);
                }
            }
        } else {
            for (int i = lane; i < hidden; i += 32) {
                const float wv = to_f32(w[i]);
#pragma unroll
                for (int k = 0; k < TOK; ++k) dot[k] = fmaf(hs[(size_t)k * hidden + i], wv, dot[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < TOK; ++k) {
            const float d = warp_sum(dot[k]);
            if (lane == 0) sc[(size_t)k * 3 * EA + e] = d;
        }
    }
    __syncthreads();
    for (int tk = warp; tk < nt; tk += nw) {
        float* s = sc + (size_t)tk * 3 * EA;
        const size_t t = t0 + tk;
        for (int r = lane; r < extra; r += 32) extra_out[t * extra + r] = s[E + r];
        warp_choose(s, s + EA, s + 2 * EA, corr, E, top, g_count, g_keep, chosen + t * top, weights + t * top, lane, sigmoid_scores,
                    group_top2, renorm, weight_eps, route_scale);
    }
}

// ------------------------------------------------------------------ g = min(gate, limit); u = clamp(up); g sigmoid(slope g) (u + 1)
__device__ __forceinline__ float clamped_glu(float g, float u, float limit, float slope, float shift) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + expf(-slope * g)) * (u + shift);
}

template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, float limit, float slope, float shift, int vec) {
    const T* row = gu + (size_t)blockIdx.x * 2 * inter;
    T* o = out + (size_t)blockIdx.x * inter;
    constexpr int VN = Vec16<T>::N;
    if (vec) {                                                      // 16 bytes of gate and of up per thread and step
        for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * VN; i < inter; i += gridDim.y * blockDim.x * VN) {
            float g[VN], u[VN];
            load16(row + i, g);
            load16(row + inter + i, u);
            T y[VN];
#pragma unroll
            for (int j = 0; j < VN; ++j) y[j] = from_f32<T>(clamped_glu(g[j], u[j], limit, slope, shift));
            *reinterpret_cast<uint4*>(o + i) = *reinterpret_cast<const uint4*>(y);
        }
        return;
    }
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter; i += gridDim.y * blockDim.x)
        o[i] = from_f32<T>(clamped_glu(to_f32(row[i]), to_f32(row[inter + i]), limit, slope, shift));
}

// ------------------------------------------------------------------ sort the pairs by expert
__global__ void moe_align_kernel(const int* __restrict__ chosen, int P, int E, int BM, int* __restrict__ sorted_pair, int cap_pos,
                                 int* __restrict__ tile_expert, int cap_tiles) {
    extern __shared__ int asm_[];
    int* cnt = asm_;            // [E]
    int* cur = cnt + E;         // [E]
    int* off = cur + E;         // [E + 1]
    for (int e = threadIdx.x; e < E; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&cnt[chosen[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        off[0] = 0;
        for (int e = 0; e < E; ++e) off[e + 1] = off[e] + (cnt[e] + BM - 1) / BM * BM;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < cap_pos; i += blockDim.x) sorted_pair[i] = -1;
    for (int t = threadIdx.x; t < cap_tiles; t += blockDim.x) {
        const int pos = t * BM;
        int e = -1;
        if (pos < off[E]) { e = 0; while (off[e + 1] <= pos) ++e; }
        tile_expert[t] = e;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = chosen[p];
        sorted_pair[off[e] + atomicAdd(&cur[e], 1)] = p;
    }
}

// ------------------------------------------------------------------ grouped product, CUDA cores, float32 sums in k order
// MODE 0 ("in"):  row pos reads A[sorted_pair[pos] / top], W = [E, 2 N, K] (gate rows, then up rows), out[pos, n] = act(gate, up)
// MODE 1 ("out"): row pos reads A[pos], W = [E, N, K], out[sorted_pair[pos], n]
constexpr int SM_ = 32, SN_ = 64, SK_ = 32;

template <typename T, int MODE>
__global__ void __launch_bounds__(256) moe_gemm_simt_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, T* __restrict__ out, int ldo,
                                                            const int* __restrict__ sorted_pair, const int* __restrict__ tile_expert,
                                                            int top, int N, int K, float limit, float slope, float shift) {
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    __shared__ float As[SM_][SK_ + 1], Bs[SN_][SK_ + 1], Bu[MODE == 0 ? SN_ : 1][SK_ + 1];
    __shared__ int pair_s[SM_];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int pos0 = blockIdx.x * SM_, n0 = blockIdx.y * SN_;
    if (tid < SM_) pair_s[tid] = sorted_pair[pos0 + tid];
    __syncthreads();
    const T* We = W + (size_t)e * (MODE == 0 ? 2 : 1) * N * K;
    float acc[2][4] = {}, accu[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += SK_) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256, r = idx >> 5, c = idx & 31, pr = pair_s[r];
            const long long src = MODE == 0 ? pr / top : pos0 + r;
            As[r][c] = (pr >= 0 && k0 + c < K) ? to_f32(A[src * lda + k0 + c]) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int idx = tid + i * 256, r = idx >> 5, c = idx & 31, n = n0 + r;
            const bool ok = n < N && k0 + c < K;
            Bs[r][c] = ok ? to_f32(We[(size_t)n * K + k0 + c]) : 0.f;
            if constexpr (MODE == 0) Bu[r][c] = ok ? to_f32(We[(size_t)(N + n) * K + k0 + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < SK_; ++kk) {
            const float a0 = As[ty][kk], a1 = As[ty + 16][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = Bs[tx + 16 * j][kk];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
                if constexpr (MODE == 0) {
                    const float u = Bu[tx + 16 * j][kk];
                    accu[0][j] = fmaf(a0, u, accu[0][j]);
                    accu[1][j] = fmaf(a1, u, accu[1][j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty + 16 * i, pr = pair_s[r];
        if (pr < 0) continue;
        const long long dst = MODE == 0 ? pos0 + r : pr;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n < N) out[dst * ldo + n] = from_f32<T>(MODE == 0 ? clamped_glu(acc[i][j], accu[i][j], limit, slope, shift) : acc[i][j]);
        }
    }
}

// ------------------------------------------------------------------ grouped product, bfloat16 on mma.sync tiles
// A block of 8 warps (WM x WN) owns BM = 16 MT WM sorted rows of ONE expert and 128 rows of the expert's matrix
// (MODE 1: 128 output columns; MODE 0: 64 gate rows and the 64 up rows of the same columns, interleaved per warp so that
// a thread holds gate and up of the same output in its accumulators).  K runs in steps of 64 through a three-stage
// cp.async ring; rows of shared memory are padded to 144 bytes, which keeps ldmatrix free of bank conflicts.
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                                   // 0 bytes read: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_commit_group() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait_group() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N) : "memory"); }

constexpr int TK = 64, TROW = 72, TSTAGES = 3;                      // k per stage, padded row (elements), ring depth

template <int MODE, int MT, int WM, int WN>
__global__ void __launch_bounds__(256, 2) moe_gemm_tc_kernel(const __nv_bfloat16* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W,
                                                          __nv_bfloat16* __restrict__ out, int ldo, const int* __restrict__ sorted_pair,
                                                          const int* __restrict__ tile_expert, int top, int N, int K, float limit, float slope, float shift) {
    constexpr int BM = 16 * MT * WM, WNE = 128 / WN, NT = WNE / 8, BN_OUT = MODE == 0 ? 64 : 128;
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    extern __shared__ __align__(16) unsigned char tsm[];
    __nv_bfloat16* sA = reinterpret_cast<__nv_bfloat16*>(tsm);                  // [TSTAGES][BM][TROW]
    __nv_bfloat16* sB = sA + TSTAGES * BM * TROW;                               // [TSTAGES][128][TROW]
    int* pair_s = reinterpret_cast<int*>(sB + TSTAGES * 128 * TROW);            // [BM]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, wm = warp / WN, wn = warp % WN;
    const int pos0 = blockIdx.x * BM, n0 = blockIdx.y * BN_OUT;
    for (int i = tid; i < BM; i += 256) pair_s[i] = sorted_pair[pos0 + i];
    __syncthreads();
    const __nv_bfloat16* We = W + (size_t)e * (MODE == 0 ? 2 : 1) * N * K;
    // what this thread copies per stage: chunks of 16 bytes, (row, k chunk)
    constexpr int CPR = TK / 8;                                     // 16-byte chunks per row and stage
    constexpr int A_CH = BM * CPR, B_CH = 128 * CPR;
    auto load_stage = [&](int stage, int k0) {
        for (int c = tid; c < A_CH; c += 256) {
            const int r = c / CPR, kc = c % CPR, pr = pair_s[r];
            const long long src = MODE == 0 ? pr / top : pos0 + r;
            cp16((uint32_t)__cvta_generic_to_shared(sA + (stage * BM + r) * TROW + kc * 8), A + (pr >= 0 ? src * lda + k0 + kc * 8 : 0), pr >= 0);
        }
        for (int c = tid; c < B_CH; c += 256) {
            const int r = c / CPR, kc = c % CPR;
            int col, grow;
            if (MODE == 0) {                                        // warp w's rows: its gate columns, then the up rows of the same columns
                const int w = r / WNE, rr = r % WNE;
                col = n0 + w * (WNE / 2) + rr % (WNE / 2);
                grow = rr < WNE / 2 ? col : N + col;
            } else {
                col = n0 + r;
                grow = col;
            }
            const bool ok = col < N;
            cp16((uint32_t)__cvta_generic_to_shared(sB + (stage * 128 + r) * TROW + kc * 8), We + (ok ? (size_t)grow * K + k0 + kc * 8 : 0), ok);
        }
    };
    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int x = 0; x < 4; ++x) acc[i][j][x] = 0.f;
    const int steps = K / TK;
    for (int s = 0; s < TSTAGES - 1; ++s) {
        if (s < steps) load_stage(s, s * TK);
        cp_commit_group();
    }
    for (int it = 0; it < steps; ++it) {
        cp_wait_group<TSTAGES - 2>();
        __syncthreads();                                            // stage `it` has landed; everybody is done with stage it - 1
        if (it + TSTAGES - 1 < steps) load_stage((it + TSTAGES - 1) % TSTAGES, (it + TSTAGES - 1) * TK);
        cp_commit_group();
        const __nv_bfloat16* a_s = sA + (it % TSTAGES) * BM * TROW;
        const __nv_bfloat16* b_s = sB + (it % TSTAGES) * 128 * TROW;
#pragma unroll
        for (int k16 = 0; k16 < TK / 16; ++k16) {
            uint32_t af[MT][4], bfr[NT / 2][4];
#pragma unroll
            for (int i = 0; i < MT; ++i)
                ldsm4(af[i], (uint32_t)__cvta_generic_to_shared(a_s + ((wm * MT + i) * 16 + (lane & 15)) * TROW + k16 * 16 + (lane >> 4) * 8));
#pragma unroll
            for (int j = 0; j < NT / 2; ++j)
                ldsm4(bfr[j], (uint32_t)__cvta_generic_to_shared(b_s + (wn * WNE + j * 16 + (lane & 7) + (lane >> 4) * 8) * TROW + k16 * 16 + ((lane >> 3) & 1) * 8));
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma16816(acc[i][j], af[i], bfr[j / 2][(j & 1) * 2], bfr[j / 2][(j & 1) * 2 + 1]);
        }
    }
    cp_wait_group<0>();
    const int g = lane >> 2, c2 = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = (wm * MT + i) * 16 + g + half * 8, pr = pair_s[r];
            if (pr < 0) continue;
            __nv_bfloat16* orow = out + (MODE == 0 ? (long long)(pos0 + r) : (long long)pr) * ldo;
            if (MODE == 0) {
#pragma unroll
                for (int j = 0; j < NT / 2; ++j) {
                    const int col = n0 + wn * (WNE / 2) + j * 8 + c2;
                    if (col < N) {                                   // N is even: col + 1 < N as well
                        const float y0 = clamped_glu(acc[i][j][half * 2], acc[i][j + NT / 2][half * 2], limit, slope, shift);
                        const float y1 = clamped_glu(acc[i][j][half * 2 + 1], acc[i][j + NT / 2][half * 2 + 1], limit, slope, shift);
                        *reinterpret_cast<__nv_bfloat162*>(orow + col) = __floats2bfloat162_rn(y0, y1);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const int col = n0 + wn * WNE + j * 8 + c2;
                    if (col + 1 < N) *reinterpret_cast<__nv_bfloat162*>(orow + col) = __floats2bfloat162_rn(acc[i][j][half * 2], acc[i][j][half * 2 + 1]);
                    else if (col < N) orow[col] = __float2bfloat16_rn(acc[i][j][half * 2]);
                }
            }
        }
}

// ------------------------------------------------------------------ weighted sum per token
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ rows, const float* __restrict__ weights, const T* __restrict__ shared,
                                   const float* __restrict__ shared_gate, T* __restrict__ out, int hidden, int top) {
    const size_t t = blockIdx.x;
    const float sg = shared_gate ? 1.f / (1.f + expf(-shared_gate[t])) : 1.f;      // the shared expert's row times sigmoid(its gate's logit)
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < hidden; c += gridDim.y * blockDim.x) {
        float acc = 0.f;
        if (weights) for (int j = 0; j < top; ++j) acc = fmaf(weights[t * top + j], to_f32(rows[(t * top + j) * hidden + c]), acc);
        else for (int j = 0; j < top; ++j) acc += to_f32(rows[(t * top + j) * hidden + c]);
        if (shared) acc = fmaf(sg, to_f32(shared[t * hidden + c]), acc);
        out[t * hidden + c] = from_f32<T>(acc);
    }
}

// ------------------------------------------------------------------ row p = weight[p] * h[p / top]
template <typename T>
__global__ void moe_scale_rows_kernel(const T* __restrict__ h, int ldh, const float* __restrict__ weights, int top, T* __restrict__ out, int K) {
    const size_t p = blockIdx.x;
    const float w = weights[p];
    const T* src = h + (p / top) * ldh;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < K; c += gridDim.y * blockDim.x) out[p * K + c] = from_f32<T>(w * to_f32(src[c]));
}

}  // namespace

MI_EXPORT int mi_moe_scale_rows(const void* h, int ldh, const float* weights, int top, void* out, int P, int K, int dtype, cudaStream_t stream) {
    if (P == 0) return 0;
    dim3 grid(P, P >= 512 ? 1 : min(8, (K + 255) / 256));
    if (dtype == MI_BF16) moe_scale_rows_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)h, ldh, weights, top, (__nv_bfloat16*)out, K);
    else moe_scale_rows_kernel<float><<<grid, 256, 0, stream>>>((const float*)h, ldh, weights, top, (float*)out, K);
    return (int)cudaGetLastError();
}

// router [E + extra, hidden] in the dtype of h (its values are read as they are stored and multiplied and added in float32)
// group_top2: a group is ranked by the sum of its two largest choice scores (0: by its largest); renorm: the chosen scores are divided
// by their sum + weight_eps; route_scale multiplies the weights last
MI_EXPORT int mi_route_topk(const void* h, int ldh, const void* router, const float* corr, int* chosen, float* weights, int T_, int hidden,
                            int E, int top, int g_count, int g_keep, int sigmoid_scores, int extra, float* extra_out, int group_top2,
                            int renorm, float weight_eps, float route_scale, int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    if (top > E || (g_count > 0 && E % g_count) || extra < 0 || (extra > 0 && !extra_out)) return -2;
    const int tok = T_ >= 1024 ? 8 : 1;
    const size_t smem = ((size_t)tok * hidden + 3 * (size_t)tok * (E + extra)) * sizeof(float);
    if (smem > 200 * 1024) return -2;
    const int grid = (T_ + tok - 1) / tok;
#define GO(T, TOK) do { \
        if (smem > 48 * 1024) cudaFuncSetAttribute(route_topk_kernel<T, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        route_topk_kernel<T, TOK><<<grid, TOK == 1 ? min(1024, max(128, 32 * (E + extra))) : 256, smem, stream>>>((const T*)h, ldh, (const T*)router, corr, chosen, weights, T_, hidden, E, top, \
                                                               g_count, g_keep, sigmoid_scores, extra, extra_out, group_top2, renorm, weight_eps, route_scale); } while (0)
    if (dtype == MI_BF16) { if (tok == 8) GO(__nv_bfloat16, 8); else GO(__nv_bfloat16, 1); }
    else { if (tok == 8) GO(float, 8); else GO(float, 1); }
#undef GO
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_clamped_glu(const void* gu, void* out, int rows, int inter, float limit, float slope, float shift, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    const int vn = dtype == MI_BF16 ? 8 : 4;
    const int vec = inter % vn == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0;
    const int per = vec ? 256 * vn : 256;
    dim3 grid(rows, rows >= 512 ? 1 : min(16, (inter + per - 1) / per));
    if (dtype == MI_BF16) clamped_glu_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, limit, slope, shift, vec);
    else clamped_glu_kernel<float><<<grid, 256, 0, stream>>>((const float*)gu, (float*)out, inter, limit, slope, shift, vec);
    return (int)cudaGetLastError();
}

// sorted_pair: cap_pos ints, tile_expert: cap_tiles ints; cap_pos = cap_tiles * BM >= P + E * (BM - 1)
MI_EXPORT int mi_moe_align(const int* chosen, int P, int E, int BM, int* sorted_pair, int cap_pos, int* tile_expert, int cap_tiles,
                           cudaStream_t stream) {
    if (P == 0) return 0;
    if (E > 4096 || cap_pos < cap_tiles * BM) return -2;
    moe_align_kernel<<<1, 1024, (3 * E + 1) * sizeof(int), stream>>>(chosen, P, E, BM, sorted_pair, cap_pos, tile_expert, cap_tiles);
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_moe_tile_rows_simt() { return SM_; }

// mode 0: A = tokens [T, K], W [E, 2 N, K], out [cap_pos, N] activated; mode 1: A = [cap_pos, K], W [E, N, K], out [P, N]
MI_EXPORT int mi_moe_gemm_simt(const void* A, int lda, const void* W, void* out, int ldo, const int* sorted_pair, const int* tile_expert,
                               int cap_tiles, int top, int N, int K, float limit, float slope, float shift, int mode, int dtype, cudaStream_t stream) {
    if (cap_tiles == 0) return 0;
    dim3 grid(cap_tiles, (N + SN_ - 1) / SN_);
    if (grid.y > 65535) return -2;
#define GO(T, MODE) moe_gemm_simt_kernel<T, MODE><<<grid, 256, 0, stream>>>((const T*)A, lda, (const T*)W, (T*)out, ldo, sorted_pair, tile_expert, \
                                                                           top, N, K, limit, slope, shift)
    if (dtype == MI_BF16) { if (mode == 0) GO(__nv_bfloat16, 0); else GO(__nv_bfloat16, 1); }
    else { if (mode == 0) GO(float, 0); else GO(float, 1); }
#undef GO
    return (int)cudaGetLastError();
}

// rows per tile of the tensor-core form for P pairs over E experts: tall tiles when an expert gets many rows
MI_EXPORT int mi_moe_tile_rows_tc(int P, int E) {
    const int avg = (P + E - 1) / E;
    return avg > 48 ? 128 : avg > 12 ? 64 : 16;
}

// bfloat16 only; K % 64 == 0, N even, lda % 8 == 0; BM as mi_moe_tile_rows_tc said (and as mi_moe_align sorted)
MI_EXPORT int mi_moe_gemm_tc(const void* A, int lda, const void* W, void* out, int ldo, const int* sorted_pair, const int* tile_expert,
                             int cap_tiles, int top, int N, int K, float limit, float slope, float shift, int mode, int BM, int dtype, cudaStream_t stream) {
    if (cap_tiles == 0) return 0;
    if (dtype != MI_BF16) return -1;
    if (K % TK || N % 2 || lda % 8 || ldo % 2) return -2;
    dim3 grid(cap_tiles, (N + (mode == 0 ? 64 : 128) - 1) / (mode == 0 ? 64 : 128));
    if (grid.y > 65535) return -2;
    const size_t smem = (size_t)TSTAGES * (BM + 128) * TROW * sizeof(__nv_bfloat16) + BM * sizeof(int);
#define GO(MODE, MT, WM, WN) do { \
        auto kern = moe_gemm_tc_kernel<MODE, MT, WM, WN>; \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        kern<<<grid, 256, smem, stream>>>((const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, (__nv_bfloat16*)out, ldo, sorted_pair, \
                                          tile_expert, top, N, K, limit, slope, shift); } while (0)
    if (BM == 128) { if (mode == 0) GO(0, 4, 2, 4); else GO(1, 4, 2, 4); }
    else if (BM == 64) { if (mode == 0) GO(0, 2, 2, 4); else GO(1, 2, 2, 4); }
    else if (BM == 16) { if (mode == 0) GO(0, 1, 1, 8); else GO(1, 1, 1, 8); }
    else return -2;
#undef GO
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_moe_combine(const void* rows, const float* weights, const void* shared, const float* shared_gate, void* out, int T_, int hidden,
                             int top, int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    dim3 grid(T_, T_ >= 512 ? 1 : min(8, (hidden + 255) / 256));
    if (dtype == MI_BF16)
        moe_combine_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)rows, weights, (const __nv_bfloat16*)shared, shared_gate, (__nv_bfloat16*)out, hidden, top);
    else
        moe_combine_kernel<float><<<grid, 256, 0, stream>>>((const float*)rows, weights, (const float*)shared, shared_gate, (float*)out, hidden, top);
    return (int)cudaGetLastError();
}
