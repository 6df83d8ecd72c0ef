// Matrix-state recurrences: a decayed outer-product accumulation ("lightning") and a gated delta rule with one decay
// per key channel, both over a float32 state S [heads, key_dim, value_dim] that lives in a request's state slot.
//
// The columns of S never mix: every update is "row factors times S, plus key times a row vector", and the read-out
// is S^T q.  So a PAIR of neighbouring columns is given to LN lanes of a warp that hold its rows in registers for the
// whole entry (lane l owns the rows 4 (l + LN g) + e, g = 0 .. NG-1, e = 0 .. 3: groups of four neighbouring rows, so
// that the lanes fetch a token's q, k and g from shared memory as full wavefronts of 16-byte loads, and each fetched
// number serves two columns).  With LN = 8 a warp holds 4 pairs = 8 neighbouring columns (a 32-byte piece of every
// row: loading and storing the state moves whole sectors) and a block 32: the form for decode steps.  For prompt
// portions what counts is the chain of dependent instructions per token, so LN grows to 16 or 32 (one group of four
// rows per lane) and eight times as many warps share a head.  A block
// walks the tokens of ONE entry (a prompt portion or a single decoded token) of ONE head in order.  What a token
// brings (q, k, g, its 32 values, beta: float32, written by a prologue kernel) is staged a few tokens at a time in
// one of two shared-memory buffers with cp.async, the next chunk travelling while the current one is worked on.  The
// delta rule's S^T k of a token's two columns is finished together with log2(LN) + 1 shuffles, since the update needs it;
// the partial sums of the read-out S^T q wait in shared memory and are added up (in lane order) and stored, coalesced,
// once per chunk.  Everything is float32.
//
// Prologue kernels, one small block per (token, unit): lightning: silu of q, k, v.  Delta rule: the short causal
// convolutions (the inputs before an entry's first token come from the state slot), silu, the unit norms of q and k,
// sigmoid(beta logits), and the decay exp(-exp(A_log) softplus(a + dt_bias)); a last kernel then moves the
// convolutions' newest inputs into the slot.
#include "common.cuh"
#include <math.h>

using namespace mi;

namespace {

constexpr int SCAN_THREADS = 128;
// LN lanes share a pair of columns (8: a warp holds 4 pairs, the state moves in 32-byte pieces, few blocks: decode steps,
// where the state's bytes are the cost; 16 or 32: fewer rows per lane, so a token's chain of dependent instructions is
// shorter and more warps share the work: prompt portions, where the tokens' latency is the cost).  Columns per block:
__host__ __device__ constexpr int cols_of(int LN) { return 4 * (32 / LN) * 2; }

__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + expf(-x)); }

__device__ __forceinline__ void cp16(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N) : "memory"); }

// Forms of the recurrence (MODE):
//   0  S <- decay[h] S + k v^T                                   (one constant per head)
//   1  S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T       (rows q, k, g; one number beta per token and head)
//   2  S <- diag(g) S - c (u^T S) + k v^T, both terms reading the old S   (rows q, k, g, u, c = removal rate times u)
//   3  S <- f S + k v^T with one number f per token and head      (rows q, k; k arrives already multiplied by its input gate)
// always followed by o = S^T q.
__host__ __device__ constexpr int rows_of(int MODE) { return MODE == 1 ? 3 : MODE == 2 ? 5 : 2; }
__host__ __device__ constexpr bool scalar_of(int MODE) { return MODE == 1 || MODE == 3; }

// Where the scan finds a token's numbers in its float32 row (ld floats per token).
struct ScanLayout {
    int ld, q_off, k_off, v_off, g_off, b_off;      // q/k: + kv_head * D; v: + head * V; g: + head * D; the per-token number (beta or f): + head
    int u_off, c_off;                               // MODE 2: + head * D
};

// One chunk of nt tokens into a buffer: rows of Dp floats (D copied, the rest stays zero), v [COLS], the per-token number.
template <int MODE, int COLS>
__device__ __forceinline__ void stage_chunk(float* buf, int Dp, int TC, const float* __restrict__ prep, const ScanLayout L,
                                            int tok0, int nt, int h, int kvh, int D, int V, int col0, bool vec) {
    constexpr int NR = rows_of(MODE);
    float* qsm = buf;
    float* ksm = qsm + TC * Dp;
    float* gsm = ksm + TC * Dp;                               // MODE 1, 2
    float* usm = gsm + TC * Dp;                               // MODE 2
    float* csm = usm + TC * Dp;                               // MODE 2
    float* vsm = buf + NR * TC * Dp;                          // [TC, COLS]
    float* bsm = vsm + TC * COLS;                             // [TC] (MODE 1, 3)
    const int ncol = min(COLS, V - col0);
    if (vec) {
        const int dq = D >> 2, vq = ncol >> 2;
        for (int idx = threadIdx.x; idx < nt * dq; idx += SCAN_THREADS) {
            const int tt = idx / dq, c = (idx - tt * dq) << 2;
            const float* row = prep + (size_t)(tok0 + tt) * L.ld;
            cp16(qsm + tt * Dp + c, row + L.q_off + kvh * D + c);
            cp16(ksm + tt * Dp + c, row + L.k_off + kvh * D + c);
            if (MODE == 1 || MODE == 2) cp16(gsm + tt * Dp + c, row + L.g_off + h * D + c);
            if (MODE == 2) { cp16(usm + tt * Dp + c, row + L.u_off + h * D + c); cp16(csm + tt * Dp + c, row + L.c_off + h * D + c); }
        }
        for (int idx = threadIdx.x; idx < nt * vq; idx += SCAN_THREADS) {
            const int tt = idx / vq, c = (idx - tt * vq) << 2;
            cp16(vsm + tt * COLS + c, prep + (size_t)(tok0 + tt) * L.ld + L.v_off + h * V + col0 + c);
        }
    } else {
        for (int idx = threadIdx.x; idx < nt * D; idx += SCAN_THREADS) {
            const int tt = idx / D, c = idx - tt * D;
            const float* row = prep + (size_t)(tok0 + tt) * L.ld;
            qsm[tt * Dp + c] = row[L.q_off + kvh * D + c];
            ksm[tt * Dp + c] = row[L.k_off + kvh * D + c];
            if (MODE == 1 || MODE == 2) gsm[tt * Dp + c] = row[L.g_off + h * D + c];
            if (MODE == 2) { usm[tt * Dp + c] = row[L.u_off + h * D + c]; csm[tt * Dp + c] = row[L.c_off + h * D + c]; }
        }
        for (int idx = threadIdx.x; idx < nt * ncol; idx += SCAN_THREADS) {
            const int tt = idx / ncol, c = idx - tt * ncol;
            vsm[tt * COLS + c] = prep[(size_t)(tok0 + tt) * L.ld + L.v_off + h * V + col0 + c];
        }
    }
    if (scalar_of(MODE))
        for (int tt = threadIdx.x; tt < nt; tt += SCAN_THREADS) bsm[tt] = prep[(size_t)(tok0 + tt) * L.ld + L.b_off + h];
}

// Sums a0 and a1 over the LN row lanes of a column pair (the low lane bits) with log2(LN) + 1 shuffles; every lane gets both.
template <int LN>
__device__ __forceinline__ float2 reduce_pair(float a0, float a1, int l) {
    const bool odd = l & 1;
    float keep = odd ? a1 : a0;
    keep += __shfl_xor_sync(0xffffffffu, odd ? a0 : a1, 1);
#pragma unroll
    for (int o = 2; o < LN; o <<= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
    const float other = __shfl_xor_sync(0xffffffffu, keep, 1);
    return odd ? make_float2(other, keep) : make_float2(keep, other);
}

// grid (entries, heads, ceil(V / cols_of(LN))).  NG: groups of four rows per lane (key_dim <= 4 LN NG).
template <int MODE, int LN, int NG>
__global__ void __launch_bounds__(SCAN_THREADS) state_scan_kernel(
        const float* __restrict__ prep, const ScanLayout L, const float* __restrict__ decay, float* __restrict__ state,
        long long state_stride, float* __restrict__ out, const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot,
        int H, int KV, int D, int V, int TC, int vec) {
    extern __shared__ __align__(16) float sm[];
    constexpr int LANES = LN, COLS = cols_of(LN), Dp = 4 * LN * NG, NR = rows_of(MODE);
    constexpr bool DELTA = MODE == 1;
    const int buf_floats = TC * (NR * Dp + COLS + (scalar_of(MODE) ? 1 : 0));
    const int buf_stride = (buf_floats + 3) & ~3;
    float* part = sm + 2 * buf_stride;                         // [TC, COLS, LN + 1] partial sums of the read-out
    const int seg = blockIdx.x, h = blockIdx.y, kvh = h / (H / KV);
    const int qs = seg_q_start[seg], n = seg_q_start[seg + 1] - qs, slot = seg_slot[seg];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane & (LANES - 1), wcol = (warp * (32 / LANES) + lane / LANES) * 2, col0 = blockIdx.z * COLS, col = col0 + wcol;
    const bool v0 = col < V, v1 = col + 1 < V;
    for (int i = threadIdx.x; i < 2 * buf_stride; i += SCAN_THREADS) sm[i] = 0.f;       // the pads beyond D (and V) stay zero
    float* S = state + (long long)slot * state_stride + (long long)h * D * V;
    __syncthreads();
    // the first chunk's copies start before the state is fetched, so that the two waits for global memory overlap
    const int chunks = (n + TC - 1) / TC;
    stage_chunk<MODE, COLS>(sm, Dp, TC, prep, L, qs, min(TC, n), h, kvh, D, V, col0, (vec & 1) != 0);
    cp_commit();
    float s0[4 * NG], s1[4 * NG];
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = 4 * (l + LANES * g) + e;
            if (vec & 2) {                                     // even V and slot size: a pair of columns is one 8-byte access
                const float2 t = (r < D && v0) ? *reinterpret_cast<const float2*>(S + (size_t)r * V + col) : make_float2(0.f, 0.f);
                s0[4 * g + e] = t.x; s1[4 * g + e] = t.y;
            } else {
                s0[4 * g + e] = (r < D && v0) ? S[(size_t)r * V + col] : 0.f;
                s1[4 * g + e] = (r < D && v1) ? S[(size_t)r * V + col + 1] : 0.f;
            }
        }
    float dec = MODE == 0 ? decay[h] : 0.f;
    for (int c = 0; c < chunks; ++c) {
        const int t0 = c * TC, nt = min(TC, n - t0);
        if (c + 1 < chunks) {
            stage_chunk<MODE, COLS>(sm + ((c + 1) & 1) * buf_stride, Dp, TC, prep, L, qs + t0 + TC, min(TC, n - t0 - TC), h, kvh, D, V, col0, (vec & 1) != 0);
            cp_commit();
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        const float* buf = sm + (c & 1) * buf_stride;
        const float* qsm = buf;
        const float* ksm = qsm + TC * Dp;
        const float* gsm = ksm + TC * Dp;
        const float* usm = gsm + TC * Dp;
        const float* csm = usm + TC * Dp;
        const float* vsm = buf + NR * TC * Dp;
        const float* bsm = vsm + TC * COLS;
        // two partial sums per dot product and column keep the chains of dependent additions short
        for (int tt = 0; tt < nt; ++tt) {
            const float2 vv = *reinterpret_cast<const float2*>(vsm + tt * COLS + wcol);
            const float4* kk = reinterpret_cast<const float4*>(ksm + tt * Dp) + l;
            const float4* qq = reinterpret_cast<const float4*>(qsm + tt * Dp) + l;
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;                 // a: first column, b: second column
            if (DELTA) {
                const float4* gg = reinterpret_cast<const float4*>(gsm + tt * Dp) + l;
                float d0 = 0.f, d1 = 0.f, e0 = 0.f, e1 = 0.f;
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    const float4 gv = gg[LANES * g], kv = kk[LANES * g];
                    s0[4 * g] *= gv.x; s0[4 * g + 1] *= gv.y; s0[4 * g + 2] *= gv.z; s0[4 * g + 3] *= gv.w;
                    s1[4 * g] *= gv.x; s1[4 * g + 1] *= gv.y; s1[4 * g + 2] *= gv.z; s1[4 * g + 3] *= gv.w;
                    d0 = fmaf(s0[4 * g], kv.x, d0); d1 = fmaf(s0[4 * g + 1], kv.y, d1);
                    d0 = fmaf(s0[4 * g + 2], kv.z, d0); d1 = fmaf(s0[4 * g + 3], kv.w, d1);
                    e0 = fmaf(s1[4 * g], kv.x, e0); e1 = fmaf(s1[4 * g + 1], kv.y, e1);
                    e0 = fmaf(s1[4 * g + 2], kv.z, e0); e1 = fmaf(s1[4 * g + 3], kv.w, e1);
                }
                const float2 dot = reduce_pair<LN>(d0 + d1, e0 + e1, l);
                const float beta = bsm[tt];
                const float u0 = beta * (vv.x - dot.x), u1 = beta * (vv.y - dot.y);
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    const float4 kv = kk[LANES * g], qv = qq[LANES * g];
                    s0[4 * g] = fmaf(kv.x, u0, s0[4 * g]); s0[4 * g + 1] = fmaf(kv.y, u0, s0[4 * g + 1]);
                    s0[4 * g + 2] = fmaf(kv.z, u0, s0[4 * g + 2]); s0[4 * g + 3] = fmaf(kv.w, u0, s0[4 * g + 3]);
                    s1[4 * g] = fmaf(kv.x, u1, s1[4 * g]); s1[4 * g + 1] = fmaf(kv.y, u1, s1[4 * g + 1]);
                    s1[4 * g + 2] = fmaf(kv.z, u1, s1[4 * g + 2]); s1[4 * g + 3] = fmaf(kv.w, u1, s1[4 * g + 3]);
                    a0 = fmaf(s0[4 * g], qv.x, a0); a1 = fmaf(s0[4 * g + 1], qv.y, a1);
                    a0 = fmaf(s0[4 * g + 2], qv.z, a0); a1 = fmaf(s0[4 * g + 3], qv.w, a1);
                    b0 = fmaf(s1[4 * g], qv.x, b0); b1 = fmaf(s1[4 * g + 1], qv.y, b1);
                    b0 = fmaf(s1[4 * g + 2], qv.z, b0); b1 = fmaf(s1[4 * g + 3], qv.w, b1);
                }
            } else if (MODE == 2) {
                const float4* gg = reinterpret_cast<const float4*>(gsm + tt * Dp) + l;
                const float4* uu = reinterpret_cast<const float4*>(usm + tt * Dp) + l;
                const float4* cc = reinterpret_cast<const float4*>(csm + tt * Dp) + l;
                float d0 = 0.f, d1 = 0.f, e0 = 0.f, e1 = 0.f;
#pragma unroll
                for (int g = 0; g < NG; ++g) {                            // what the unit key sees of the old state
                    const float4 uv = uu[LANES * g];
                    d0 = fmaf(s0[4 * g], uv.x, d0); d1 = fmaf(s0[4 * g + 1], uv.y, d1);
                    d0 = fmaf(s0[4 * g + 2], uv.z, d0); d1 = fmaf(s0[4 * g + 3], uv.w, d1);
                    e0 = fmaf(s1[4 * g], uv.x, e0); e1 = fmaf(s1[4 * g + 1], uv.y, e1);
                    e0 = fmaf(s1[4 * g + 2], uv.z, e0); e1 = fmaf(s1[4 * g + 3], uv.w, e1);
                }
                const float2 dot = reduce_pair<LN>(d0 + d1, e0 + e1, l);
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    const float4 gv = gg[LANES * g], cv = cc[LANES * g], kv = kk[LANES * g], qv = qq[LANES * g];
                    s0[4 * g] = fmaf(gv.x, s0[4 * g], fmaf(-cv.x, dot.x, kv.x * vv.x)); s0[4 * g + 1] = fmaf(gv.y, s0[4 * g + 1], fmaf(-cv.y, dot.x, kv.y * vv.x));
                    s0[4 * g + 2] = fmaf(gv.z, s0[4 * g + 2], fmaf(-cv.z, dot.x, kv.z * vv.x)); s0[4 * g + 3] = fmaf(gv.w, s0[4 * g + 3], fmaf(-cv.w, dot.x, kv.w * vv.x));
                    s1[4 * g] = fmaf(gv.x, s1[4 * g], fmaf(-cv.x, dot.y, kv.x * vv.y)); s1[4 * g + 1] = fmaf(gv.y, s1[4 * g + 1], fmaf(-cv.y, dot.y, kv.y * vv.y));
                    s1[4 * g + 2] = fmaf(gv.z, s1[4 * g + 2], fmaf(-cv.z, dot.y, kv.z * vv.y)); s1[4 * g + 3] = fmaf(gv.w, s1[4 * g + 3], fmaf(-cv.w, dot.y, kv.w * vv.y));
                    a0 = fmaf(s0[4 * g], qv.x, a0); a1 = fmaf(s0[4 * g + 1], qv.y, a1);
                    a0 = fmaf(s0[4 * g + 2], qv.z, a0); a1 = fmaf(s0[4 * g + 3], qv.w, a1);
                    b0 = fmaf(s1[4 * g], qv.x, b0); b1 = fmaf(s1[4 * g + 1], qv.y, b1);
                    b0 = fmaf(s1[4 * g + 2], qv.z, b0); b1 = fmaf(s1[4 * g + 3], qv.w, b1);
                }
            } else {
                if (MODE == 3) dec = bsm[tt];
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    const float4 kv = kk[LANES * g], qv = qq[LANES * g];
                    s0[4 * g] = fmaf(dec, s0[4 * g], kv.x * vv.x); s0[4 * g + 1] = fmaf(dec, s0[4 * g + 1], kv.y * vv.x);
                    s0[4 * g + 2] = fmaf(dec, s0[4 * g + 2], kv.z * vv.x); s0[4 * g + 3] = fmaf(dec, s0[4 * g + 3], kv.w * vv.x);
                    s1[4 * g] = fmaf(dec, s1[4 * g], kv.x * vv.y); s1[4 * g + 1] = fmaf(dec, s1[4 * g + 1], kv.y * vv.y);
                    s1[4 * g + 2] = fmaf(dec, s1[4 * g + 2], kv.z * vv.y); s1[4 * g + 3] = fmaf(dec, s1[4 * g + 3], kv.w * vv.y);
                    a0 = fmaf(s0[4 * g], qv.x, a0); a1 = fmaf(s0[4 * g + 1], qv.y, a1);
                    a0 = fmaf(s0[4 * g + 2], qv.z, a0); a1 = fmaf(s0[4 * g + 3], qv.w, a1);
                    b0 = fmaf(s1[4 * g], qv.x, b0); b1 = fmaf(s1[4 * g + 1], qv.y, b1);
                    b0 = fmaf(s1[4 * g + 2], qv.z, b0); b1 = fmaf(s1[4 * g + 3], qv.w, b1);
                }
            }
            // the read-out feeds nothing back: its partial sums wait in shared memory until the chunk's tokens are done
            part[(tt * COLS + wcol) * (LANES + 1) + l] = a0 + a1;
            part[(tt * COLS + wcol + 1) * (LANES + 1) + l] = b0 + b1;
        }
        __syncthreads();                                       // partial sums complete; the staging buffer is free for the chunk after the next
        for (int o = threadIdx.x; o < nt * COLS; o += SCAN_THREADS) {
            const int tt = o / COLS, ci = o - tt * COLS;
            const float* pp = part + o * (LANES + 1);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < LANES; ++i) acc += pp[i];
            if (col0 + ci < V) out[(size_t)(qs + t0 + tt) * H * V + (size_t)h * V + col0 + ci] = acc;
        }
    }
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = 4 * (l + LANES * g) + e;
            if (vec & 2) {
                if (r < D && v0) *reinterpret_cast<float2*>(S + (size_t)r * V + col) = make_float2(s0[4 * g + e], s1[4 * g + e]);
            } else {
                if (r < D && v0) S[(size_t)r * V + col] = s0[4 * g + e];
                if (r < D && v1) S[(size_t)r * V + col + 1] = s1[4 * g + e];
            }
        }
}

template <int MODE>
int launch_scan(const float* prep, ScanLayout L, const float* decay, float* state, long long state_stride, float* out,
                const int* seg_q_start, const int* seg_slot, int T_, int num_segs, int H, int KV, int D, int V, cudaStream_t stream) {
    if (num_segs == 0) return 0;
    if (D > 256 || H > 65535) return -2;
    constexpr int NR = rows_of(MODE);
    // entries of many tokens: as many lanes per column pair as leave a lane one group of four rows (up to a warp);
    // decode steps: 8 lanes, so that a warp moves the state in whole sectors
    int LN = 8;
    if (T_ > 4 * num_segs) LN = D > 64 ? 32 : D > 32 ? 16 : 8;
    int NG = (D + 4 * LN - 1) / (4 * LN);
    if (LN == 8) NG = NG <= 2 ? NG : NG <= 4 ? 4 : 8;                      // the forms that exist: the kernel's rows have 4 LN NG floats
    const int COLS = cols_of(LN);
    const int per_token = NR * 4 * LN * NG + COLS + 1;
    const int per_chunk_token = 2 * per_token + COLS * (LN + 1);          // two staging buffers and the partial sums
    const int TC = T_ <= 4 * num_segs ? 4 : per_chunk_token * 16 * 4 <= 96 * 1024 ? 16 : per_chunk_token * 8 * 4 <= 96 * 1024 ? 8 : 4;   // decode steps: small buffers, more blocks per SM
    const size_t smem = (2 * (size_t)((TC * per_token + 3) & ~3) + (size_t)TC * COLS * (LN + 1)) * sizeof(float);
    // 16-byte copies need every piece on a 16-byte boundary: sizes and offsets in multiples of four floats
    const int vec = (((uintptr_t)prep % 16 == 0 && D % 4 == 0 && V % 4 == 0 && L.ld % 4 == 0 && L.q_off % 4 == 0 && L.k_off % 4 == 0 &&
                     L.v_off % 4 == 0 && (!(MODE == 1 || MODE == 2) || L.g_off % 4 == 0) && (MODE != 2 || (L.u_off % 4 == 0 && L.c_off % 4 == 0))) ? 1 : 0)
                  | ((V % 2 == 0 && state_stride % 2 == 0 && (uintptr_t)state % 8 == 0) ? 2 : 0);      // bit 1: the state in 8-byte pairs
    dim3 grid(num_segs, H, (V + COLS - 1) / COLS);
#define GO(LN_, N) do { \
        auto kern = state_scan_kernel<MODE, LN_, N>; \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
        kern<<<grid, SCAN_THREADS, smem, stream>>>(prep, L, decay, state, state_stride, out, seg_q_start, seg_slot, H, KV, D, V, TC, vec); } while (0)
    if (LN == 32) { if (NG == 1) GO(32, 1); else GO(32, 2); }
    else if (LN == 16) GO(16, 1);
    else { if (NG == 1) GO(8, 1); else if (NG == 2) GO(8, 2); else if (NG == 4) GO(8, 4); else GO(8, 8); }
#undef GO
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ lightning prologue: out = silu(p[:, :n]) in float32
template <typename T>
__global__ void silu_f32_kernel(const T* __restrict__ p, int ldp, float* __restrict__ out, int n) {
    const T* row = p + (size_t)blockIdx.x * ldp;
    float* o = out + (size_t)blockIdx.x * n;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) o[i] = silu(to_f32(row[i]));
}

// ------------------------------------------------------------------ retention prologue: rotate q and k, scale k, all to float32
// p [T, ldp] = q [H D] | k [H D] | v [H V].  The first 2 * half coordinates of every q and k head are turned in the
// rotate-half layout (coordinate i pairs with i + half; angle = position * inv_freq[i], float32), the rest pass;
// k is then multiplied by k_scale.  out [T, 2 H D + H V] float32.
template <typename T>
__global__ void rotate_f32_kernel(const T* __restrict__ p, int ldp, float* __restrict__ out, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int half, float k_scale, int H, int D, int V) {
    const T* row = p + (size_t)blockIdx.x * ldp;
    const int HD = H * D, n = 2 * HD + H * V;
    float* o = out + (size_t)blockIdx.x * n;
    const float pos = (float)positions[blockIdx.x];
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
        float v = to_f32(row[i]);
        if (i < 2 * HD) {
            const int d = i % D;
            if (d < 2 * half) {
                const bool low = d < half;
                const float other = to_f32(row[low ? i + half : i - half]);
                float sn, cs;
                sincosf(pos * inv_freq[low ? d : d - half], &sn, &cs);
                v = low ? v * cs - other * sn : v * cs + other * sn;
            }
            if (i >= HD) v *= k_scale;
        }
        o[i] = v;
    }
}

// ------------------------------------------------------------------ delta-rule prologue, one block per (token, unit)
// p [T, ldp]: q | k | v (C = 2 KV D + H V channels that pass the convolution) | beta logits [H] | ...
// a [T, lda]: decay logits [H D].  conv [C, taps], the last tap multiplies the current token.  The inputs of the
// taps - 1 positions before an entry's first token are rows of hist = state[slot] + hist_off, [taps - 1, C]
// (zeros for a request's first entry: the slot is zeroed when it is claimed).
// Units: 0 .. 2 KV - 1 a q or k head (convolution, silu, unit norm; q also * D^-1/2); then H value heads
// (convolution, silu); then H decay heads; then one unit for all beta.  out [T, ldo]: q | k | v | g | beta (ldo may pad).
template <typename T>
__device__ __forceinline__ float conv_silu(const T* __restrict__ p, int ldp, const float* __restrict__ conv, const float* __restrict__ hist,
                                           int C, int taps, int qs, int r, int c) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int off = r - (taps - 1 - j);
        const float x = off >= 0 ? to_f32(p[(size_t)(qs + off) * ldp + c]) : hist[(size_t)(taps - 1 + off) * C + c];
        acc = fmaf(conv[(size_t)c * taps + j], x, acc);
    }
    return silu(acc);
}

template <typename T>
__global__ void delta_prepare_kernel(const T* __restrict__ p, int ldp, const T* __restrict__ a, int lda,
                                     const float* __restrict__ conv, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                     const float* __restrict__ state, long long state_stride, long long hist_off,
                                     float* __restrict__ out, int ldo, const int* __restrict__ token_seg,
                                     const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot,
                                     int H, int KV, int D, int V, int taps, float unit_eps, int T_, int toks) {
    __shared__ float scratch[32];
    const int unit = blockIdx.y;
    const int C = 2 * KV * D + H * V;
    for (int t = blockIdx.x * toks; t < min(T_, (int)(blockIdx.x + 1) * toks); ++t) {      // a block takes a unit of a few neighbouring tokens
    const int seg = token_seg[t], qs = seg_q_start[seg], r = t - qs;
    const float* hist = state + (long long)seg_slot[seg] * state_stride + hist_off;
    float* o = out + (size_t)t * ldo;
    if (unit < 2 * KV) {
        const int c0 = unit * D;
        float ss = 0.f;
        for (int d = threadIdx.x; d < D; d += 128) { const float y = conv_silu(p, ldp, conv, hist, C, taps, qs, r, c0 + d); ss += y * y; }
        float inv = 1.f / sqrtf(block_sum<128>(ss, scratch) + unit_eps);
        if (unit < KV) inv *= rsqrtf((float)D);
        for (int d = threadIdx.x; d < D; d += 128) o[c0 + d] = conv_silu(p, ldp, conv, hist, C, taps, qs, r, c0 + d) * inv;
    } else if (unit < 2 * KV + H) {
        const int c0 = 2 * KV * D + (unit - 2 * KV) * V;
        for (int i = threadIdx.x; i < V; i += 128) o[c0 + i] = conv_silu(p, ldp, conv, hist, C, taps, qs, r, c0 + i);
    } else if (unit < 2 * KV + 2 * H) {
        const int hh = unit - 2 * KV - H;
        const float rate = expf(A_log[hh]);
        for (int d = threadIdx.x; d < D; d += 128) {
            const float x = to_f32(a[(size_t)t * lda + hh * D + d]) + dt_bias[hh * D + d];
            const float sp = x > 20.f ? x : log1pf(expf(x));
            o[C + hh * D + d] = expf(-rate * sp);
        }
    } else {
        for (int h = threadIdx.x; h < H; h += 128) o[C + H * D + h] = sigmoidf(to_f32(p[(size_t)t * ldp + C + h]));
    }
    }
}

// hist[j] <- input at (entry's end - (taps - 1) + j), j = 0 .. taps - 2; a thread owns a channel and goes up in j, so an
// entry shorter than taps - 1 shifts its own rows safely.
template <typename T>
__global__ void conv_tail_kernel(const T* __restrict__ p, int ldp, float* __restrict__ state, long long state_stride, long long hist_off,
                                 const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot, int C, int taps) {
    const int seg = blockIdx.x, qs = seg_q_start[seg], n = seg_q_start[seg + 1] - qs;
    float* hist = state + (long long)seg_slot[seg] * state_stride + hist_off;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    for (int j = 0; j < taps - 1; ++j) {
        const int src = n - (taps - 1) + j;
        hist[(size_t)j * C + c] = src >= 0 ? to_f32(p[(size_t)(qs + src) * ldp + c]) : hist[(size_t)(taps - 1 + src) * C + c];
    }
}


// ------------------------------------------------------------------ short causal convolution over time, per channel
// out[t, c] = act(sum_j w[c, j] x(t - taps + 1 + j, c) + bias[c]) (+ x(t, c) when residual), x before an entry's first token
// read from hist = state[slot] + hist_off, [taps - 1, C] (zeros for a request's first entry).  conv_tail_kernel then
// moves the entry's newest inputs into the slot.
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ h, int ldh, const float* __restrict__ w, const float* __restrict__ bias,
                                  const float* __restrict__ state, long long state_stride, long long hist_off, T* __restrict__ out,
                                  const int* __restrict__ token_seg, const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot,
                                  int C, int taps, int residual, int act, int shift) {
    // shift != 0 (every entry of the step brings ONE token, so a channel of a slot has one reader): the thread also moves the
    // slot's inputs up by one and appends the token's own, which conv_tail_kernel does for steps of any other shape
    const int t = blockIdx.x, seg = token_seg[t], qs = seg_q_start[seg], r = t - qs;
    const float* hist = taps > 1 ? state + (long long)seg_slot[seg] * state_stride + hist_off : nullptr;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float acc = 0.f;
        const float own = to_f32(h[(size_t)t * ldh + c]);
        for (int j = 0; j < taps; ++j) {
            const int off = r - (taps - 1 - j);
            const float x = j == taps - 1 ? own : off >= 0 ? to_f32(h[(size_t)(qs + off) * ldh + c]) : hist[(size_t)(taps - 1 + off) * C + c];
            acc = fmaf(w[(size_t)c * taps + j], x, acc);
        }
        if (bias) acc += bias[c];
        if (act == 1) acc = silu(acc);
        if (residual) acc += own;
        out[(size_t)t * C + c] = from_f32<T>(acc);
        if (shift && taps > 1) {
            float* hw = const_cast<float*>(hist);
            for (int j = 0; j + 2 < taps; ++j) hw[(size_t)j * C + c] = hw[(size_t)(j + 1) * C + c];
            hw[(size_t)(taps - 2) * C + c] = own;
        }
    }
}

// The same for bfloat16 rows whose channels come in multiples of eight: a thread owns eight channels (16-byte loads and stores), keeps
// their TAPS weights in registers and walks TOK neighbouring tokens (each looks its own entry up: an entry may end between them).
template <int TAPS, int TOK>
__global__ void short_conv_vec_kernel(const __nv_bfloat16* __restrict__ h, int ldh, const float* __restrict__ w, const float* __restrict__ bias,
                                      const float* __restrict__ state, long long state_stride, long long hist_off, __nv_bfloat16* __restrict__ out,
                                      const int* __restrict__ token_seg, const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot,
                                      int T_, int C, int residual, int act) {
    // where each of the block's tokens stands in its entry: looked up first, all at once, so that the chains of dependent reads
    // (token -> entry -> start and slot) run side by side and under the staging of the weights
    const int t0 = blockIdx.x * TOK;
    int qs_[TOK], slot_[TOK];
#pragma unroll
    for (int k = 0; k < TOK; ++k) {
        const int seg = token_seg[min(t0 + k, T_ - 1)];
        qs_[k] = seg_q_start[seg];
        slot_[k] = seg_slot[seg];
    }
    // the block's weights pass through shared memory: read from w in order, then each thread takes its own 8 TAPS numbers
    // (rows of 8 TAPS + 1 floats keep the threads on different banks)
    constexpr int ROW = 8 * TAPS + 1;
    __shared__ float wsm[256 * ROW];
    const int cb = blockIdx.y * blockDim.x * 8;                                   // the block's first channel
    const int mine = min((int)blockDim.x * 8, C - cb) * TAPS;
    for (int i = threadIdx.x; i < mine; i += blockDim.x) wsm[(i / (8 * TAPS)) * ROW + i % (8 * TAPS)] = w[(size_t)cb * TAPS + i];
    __syncthreads();
    const int c = cb + threadIdx.x * 8;
    if (c >= C) return;
    float wreg[8][TAPS], breg[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wreg[e][j] = wsm[threadIdx.x * ROW + e * TAPS + j];
    }
    if (bias) {
        const float4 a = *reinterpret_cast<const float4*>(bias + c), b = *reinterpret_cast<const float4*>(bias + c + 4);
        breg[0] = a.x; breg[1] = a.y; breg[2] = a.z; breg[3] = a.w; breg[4] = b.x; breg[5] = b.y; breg[6] = b.z; breg[7] = b.w;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) breg[e] = 0.f;
    }
#pragma unroll
    for (int k = 0; k < TOK; ++k) {
        const int t = t0 + k;
        if (t >= T_) break;
        const int qs = qs_[k], r = t - qs;
        const float* hist = TAPS > 1 ? state + (long long)slot_[k] * state_stride + hist_off : nullptr;
        float acc[8], x[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = breg[e];
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
            const int off = r - (TAPS - 1 - j);
            if (off >= 0) {
                const uint4 v = *reinterpret_cast<const uint4*>(h + (size_t)(qs + off) * ldh + c);
                const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(hp[e]); x[2 * e] = f.x; x[2 * e + 1] = f.y; }
            } else {
                const float* hr = hist + (size_t)(TAPS - 1 + off) * C + c;
                const float4 a = *reinterpret_cast<const float4*>(hr), b = *reinterpret_cast<const float4*>(hr + 4);
                x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = fmaf(wreg[e][j], x[e], acc[e]);
        }
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            if (act == 1) acc[e] = silu(acc[e]);
            if (residual) acc[e] += x[e];                    // x holds the last tap's input: the token's own
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
        *reinterpret_cast<uint4*>(out + (size_t)t * C + c) = o;
    }
}

// ------------------------------------------------------------------ general delta rule, prologue
// p [T, ldp] = r | k | v | a | g | low (H D, H D, H V, H D, H V, rank columns).  A block takes TOK neighbouring tokens and a
// range of channels: low = tanh(.), decay = exp(-decay_scale sigmoid(w2 low + w0)) with w2 [H D, rank] read once for the
// TOK tokens, removal a = sigmoid(. + a_b), unit key u = k / sqrt(sum k^2 + unit_eps) per head.
// out [T, ldo] float32 = r | k | u | a u | decay | v.
template <typename T, int TOK>
__global__ void __launch_bounds__(256) general_delta_prepare_kernel(const T* __restrict__ p, int ldp, const T* __restrict__ w2,
                                                                    const float* __restrict__ w0, const float* __restrict__ a_b,
                                                                    float* __restrict__ out, int ldo, int T_, int H, int D, int V, int rank,
                                                                    float decay_scale, float unit_eps) {
    extern __shared__ __align__(16) float gsm[];
    float* low_s = gsm;                              // [TOK][rank]
    float* inv_s = low_s + TOK * rank;               // [TOK][H]
    const int HD = H * D, HV = H * V, t0 = blockIdx.x * TOK, nt = min(TOK, T_ - t0);
    const int a_off = 2 * HD + HV, low_off = 3 * HD + 2 * HV;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < TOK * rank; i += 256) {
        const int k = i / rank, j = i - k * rank;
        low_s[i] = k < nt ? tanhf(to_f32(p[(size_t)(t0 + k) * ldp + low_off + j])) : 0.f;
    }
    for (int u = warp; u < nt * H; u += 8) {
        const int k = u / H, hh = u - k * H;
        const T* kr = p + (size_t)(t0 + k) * ldp + HD + hh * D;
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) { const float v = to_f32(kr[d]); ss += v * v; }
        ss = warp_sum(ss);
        if (lane == 0) inv_s[k * H + hh] = 1.f / sqrtf(ss + unit_eps);
    }
    __syncthreads();
    for (int i = blockIdx.y * 256 + threadIdx.x; i < HD; i += gridDim.y * 256) {
        float acc[TOK];
#pragma unroll
        for (int k = 0; k < TOK; ++k) acc[k] = 0.f;
        const T* wr = w2 + (size_t)i * rank;
        if (sizeof(T) == 2 && rank % 8 == 0 && (uintptr_t)w2 % 16 == 0) {
            // a row of w2 is read sixteen bytes at a time: a warp's 32 rows are 32 cache lines, each used whole
            for (int j = 0; j < rank; j += 8) {
                const uint4 v = *reinterpret_cast<const uint4*>(wr + j);
                const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&v);
                const float2 w01 = __bfloat1622float2(hp[0]), w23 = __bfloat1622float2(hp[1]), w45 = __bfloat1622float2(hp[2]), w67 = __bfloat1622float2(hp[3]);
#pragma unroll
                for (int k = 0; k < TOK; ++k) {                  // the token's eight inputs in two 16-byte reads (every thread the same address)
                    const float4 la = *reinterpret_cast<const float4*>(low_s + k * rank + j), lb = *reinterpret_cast<const float4*>(low_s + k * rank + j + 4);
                    float a = acc[k];
                    a = fmaf(la.x, w01.x, a); a = fmaf(la.y, w01.y, a); a = fmaf(la.z, w23.x, a); a = fmaf(la.w, w23.y, a);
                    a = fmaf(lb.x, w45.x, a); a = fmaf(lb.y, w45.y, a); a = fmaf(lb.z, w67.x, a); a = fmaf(lb.w, w67.y, a);
                    acc[k] = a;
                }
            }
        } else {
            for (int j = 0; j < rank; ++j) {
                const float wv = to_f32(wr[j]);
#pragma unroll
                for (int k = 0; k < TOK; ++k) acc[k] = fmaf(low_s[k * rank + j], wv, acc[k]);
            }
        }
        const float b0 = w0[i], ab = a_b[i];
        const int hh = i / D;
#pragma unroll
        for (int k = 0; k < TOK; ++k) {
            if (k >= nt) break;
            const T* row = p + (size_t)(t0 + k) * ldp;
            float* o = out + (size_t)(t0 + k) * ldo;
            const float kv = to_f32(row[HD + i]), u = kv * inv_s[k * H + hh];
            o[i] = to_f32(row[i]);
            o[HD + i] = kv;
            o[2 * HD + i] = u;
            o[3 * HD + i] = sigmoidf(to_f32(row[a_off + i]) + ab) * u;
            o[4 * HD + i] = expf(-decay_scale * sigmoidf(acc[k] + b0));
        }
    }
    for (int i = blockIdx.y * 256 + threadIdx.x; i < nt * HV; i += gridDim.y * 256) {
        const int k = i / HV, c = i - k * HV;
        out[(size_t)(t0 + k) * ldo + 5 * HD + c] = to_f32(p[(size_t)(t0 + k) * ldp + 2 * HD + c]);
    }
}

// ------------------------------------------------------------------ matrix memory with exponential gates
// (1) per token and head, in parallel: the capped gate logits -> log input gate i and log forget gate f = logsigmoid(.)
__global__ void memory_gates_kernel(const float* __restrict__ gl, const float* __restrict__ bias, float* __restrict__ lg, int n, int H,
                                    float cap, int capped) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int c = idx % (2 * H);
    float z = gl[idx] + bias[c];
    if (capped) z = cap * tanhf(z / cap);
    if (c >= H) z = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));          // logsigmoid
    lg[idx] = z;
}

// (2) per (entry, head), in order: m' = max(f + m, i) from the slot's m; lg becomes [f + m - m' | i - m'] and mneg = -m'.
// m -> max(m + f, i) composes: first (F1, I1), then (F2, I2) is (F1 + F2, max(I1 + F2, I2)).  A warp takes a head and scans 32 tokens at a
// time with shuffles, carrying m from one group of 32 to the next.
__global__ void memory_max_kernel(float* __restrict__ lg, float* __restrict__ mneg, float* __restrict__ state, long long state_stride,
                                  long long m_off, const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot, int H) {
    const int seg = blockIdx.x, qs = seg_q_start[seg], n = seg_q_start[seg + 1] - qs;
    const int lane = threadIdx.x & 31, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (h >= H) return;
    float* ms = state + (long long)seg_slot[seg] * state_stride + m_off;
    float m = ms[h];
    for (int base = 0; base < n; base += 32) {
        const bool ok = base + lane < n;
        const size_t t = (size_t)qs + base + lane;
        const float i = ok ? lg[t * 2 * H + h] : -INFINITY, f = ok ? lg[t * 2 * H + H + h] : 0.f;
        float F = f, I = i;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const float Fp = __shfl_up_sync(0xffffffffu, F, d), Ip = __shfl_up_sync(0xffffffffu, I, d);
            if (lane >= d) { I = fmaxf(Ip + F, I); F += Fp; }
        }
        const float mn = fmaxf(m + F, I);                       // the maximum after this lane's token
        float before = __shfl_up_sync(0xffffffffu, mn, 1);
        if (lane == 0) before = m;
        if (ok) {
            lg[t * 2 * H + h] = i - mn;
            lg[t * 2 * H + H + h] = f + before - mn;
            mneg[t * H + h] = -mn;
        }
        m = __shfl_sync(0xffffffffu, mn, min(31, n - base - 1));
    }
    if (lane == 0) ms[h] = m;
}

// (3) per token: what the scan stages, float32: q * q_scale | e^(i - m') k | per head [v, 1, 0, 0, 0] | e^(f + m - m') per head
template <typename T>
__device__ __forceinline__ void memory_prepare_row(const T* __restrict__ row, const float* __restrict__ g, float* __restrict__ o, int H, int D, int V, float q_scale) {
    const int HD = H * D, W = V + 4;
    for (int i = threadIdx.x; i < HD; i += blockDim.x) {
        o[i] = to_f32(row[i]) * q_scale;
        o[HD + i] = to_f32(row[HD + i]) * expf(g[i / D]);
    }
    for (int i = threadIdx.x; i < H * W; i += blockDim.x) {
        const int hh = i / W, c = i - hh * W;
        o[2 * HD + i] = c < V ? to_f32(row[2 * HD + hh * V + c]) : c == V ? 1.f : 0.f;
    }
    for (int hh = threadIdx.x; hh < H; hh += blockDim.x) o[2 * HD + H * W + hh] = expf(g[H + hh]);
}

template <typename T>
__global__ void memory_prepare_kernel(const T* __restrict__ p, int ldp, const float* __restrict__ lg, float* __restrict__ out, int ldo,
                                      int H, int D, int V, float q_scale) {
    const size_t t = blockIdx.x;
    memory_prepare_row(p + t * ldp, lg + t * 2 * H, out + t * ldo, H, D, V, q_scale);
}

// (1) - (3) in one kernel for a step in which every entry brings ONE token (decode steps): a block per entry
template <typename T>
__global__ void memory_step_kernel(const T* __restrict__ p, int ldp, const float* __restrict__ gl, const float* __restrict__ bias, float cap, int capped,
                                   float* __restrict__ mneg, float* __restrict__ out, int ldo, float* __restrict__ state, long long state_stride,
                                   long long m_off, const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot, int H, int D, int V, float q_scale) {
    extern __shared__ float gsh[];                          // [2 H]: i - m' | f + m - m'
    const int seg = blockIdx.x;
    const size_t t = seg_q_start[seg];
    float* ms = state + (long long)seg_slot[seg] * state_stride + m_off;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float zi = gl[t * 2 * H + h] + bias[h], zf = gl[t * 2 * H + H + h] + bias[H + h];
        if (capped) { zi = cap * tanhf(zi / cap); zf = cap * tanhf(zf / cap); }
        const float f = fminf(zf, 0.f) - log1pf(expf(-fabsf(zf)));          // logsigmoid
        const float m = ms[h], mn = fmaxf(f + m, zi);
        gsh[h] = zi - mn;
        gsh[H + h] = f + m - mn;
        mneg[t * H + h] = -mn;
        ms[h] = mn;
    }
    __syncthreads();
    memory_prepare_row(p + t * ldp, gsh, out + t * ldo, H, D, V, q_scale);
}

// (4) per (token, head): o = full[:V] / (max(|full[V]|, e^(-m)) + den_eps); rows = o / rms(o) * weight * sigmoid(gate)
template <typename T>
__global__ void memory_output_kernel(const float* __restrict__ full, const float* __restrict__ mneg, const float* __restrict__ w,
                                     const T* __restrict__ gate, int gate_stride, T* __restrict__ y, int H, int V, float den_eps, float eps) {
    const size_t t = blockIdx.x;
    const int hh = blockIdx.y, lane = threadIdx.x;
    const float* f = full + (t * H + hh) * (V + 4);
    const float den = fmaxf(fabsf(f[V]), expf(mneg[t * H + hh])) + den_eps;
    float ss = 0.f;
    for (int v = lane; v < V; v += 32) { const float o = f[v] / den; ss += o * o; }
    const float r = rsqrtf(warp_sum(ss) / V + eps);
    for (int v = lane; v < V; v += 32) {
        const float sg = sigmoidf(to_f32(gate[t * gate_stride + hh * V + v]));
        y[t * H * V + hh * V + v] = from_f32<T>(f[v] / den * r * w[hh * V + v] * sg);
    }
}

// ------------------------------------------------------------------ selective state-space scan
// grid (entries, ceil(I / 32)), 256 threads: 8 lanes share a channel, lane l holding the states n = l + 8 g in registers.
// Per chunk of SS_TC tokens the block stages B and C [N] of each token, and for its 32 channels the step softplus(dt + dt_b),
// x and z, all float32.  S <- exp(step A) S + step x B;  y = sum_n S C + D x;  out = y * silu(z).
constexpr int SS_TC = 16;
template <typename T, int NG>
__global__ void __launch_bounds__(256) selective_scan_kernel(const T* __restrict__ x, const float* __restrict__ dt, const float* __restrict__ dt_b,
                                                             const float* __restrict__ A, const T* __restrict__ B, int ldb,
                                                             const T* __restrict__ Cm, int ldc, const float* __restrict__ Dv,
                                                             const T* __restrict__ z, int ldz, float* __restrict__ state, long long state_stride,
                                                             T* __restrict__ out, const int* __restrict__ seg_q_start,
                                                             const int* __restrict__ seg_slot, int I, int N) {
    extern __shared__ __align__(16) float ssm[];
    float* Bs = ssm;                        // [SS_TC][N]
    float* Cs = Bs + SS_TC * N;             // [SS_TC][N]
    float* st = Cs + SS_TC * N;             // [SS_TC][32] step
    float* xs = st + SS_TC * 32;            // [SS_TC][32]
    float* zs = xs + SS_TC * 32;            // [SS_TC][32]
    float* ys = zs + SS_TC * 32;            // [SS_TC][32] the read-outs of a chunk, finished after the chunk's tokens
    const int seg = blockIdx.x, qs = seg_q_start[seg], n = seg_q_start[seg + 1] - qs;
    const int c0 = blockIdx.y * 32, cl = threadIdx.x >> 3, l = threadIdx.x & 7, c = c0 + cl;
    const bool live = c < I;
    float* S = state + (long long)seg_slot[seg] * state_stride + (size_t)(live ? c : 0) * N;
    float s[NG], a[NG];
#pragma unroll
    for (int g = 0; g < NG; ++g) {
        const int nn = l + 8 * g;
        const bool ok = live && nn < N;
        s[g] = ok ? S[nn] : 0.f;
        a[g] = ok ? A[(size_t)c * N + nn] : 0.f;
    }
    // a chunk's inputs are fetched into registers while the chunk before it is computed, and stored to shared memory after it
    constexpr int RB = (SS_TC * 8 * NG + 255) / 256;
    T rB[RB], rC[RB], rx[2], rz[2];             // as loaded: converting here would wait for the load
    float rs[2], rb[2];
    auto fetch = [&](int t0) {
        const int nt = min(SS_TC, n - t0);
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            const int i = threadIdx.x + 256 * r;
            if (i < nt * N) {
                const int tt = i / N, nn = i - tt * N;
                rB[r] = B[(size_t)(qs + t0 + tt) * ldb + nn];
                rC[r] = Cm[(size_t)(qs + t0 + tt) * ldc + nn];
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int i = threadIdx.x + 256 * r, tt = i >> 5, cc = c0 + (i & 31);
            if (tt < nt && cc < I) {
                const size_t tok = qs + t0 + tt;
                rs[r] = dt[tok * I + cc];
                rb[r] = dt_b[cc];
                rx[r] = x[tok * I + cc];
                rz[r] = z[tok * ldz + cc];
            }
        }
    };
    static_assert(SS_TC * 32 <= 2 * 256, "two step / input / gate values a thread");
    if (n > 0) fetch(0);
    for (int t0 = 0; t0 < n; t0 += SS_TC) {
        const int nt = min(SS_TC, n - t0);
        __syncthreads();
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            const int i = threadIdx.x + 256 * r;
            if (i < nt * N) { Bs[i] = to_f32(rB[r]); Cs[i] = to_f32(rC[r]); }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int i = threadIdx.x + 256 * r, tt = i >> 5, cc = c0 + (i & 31);
            if (tt < nt && cc < I) {
                const float v = rs[r] + rb[r];
                st[i] = v > 20.f ? v : log1pf(expf(v));
                xs[i] = to_f32(rx[r]);
                zs[i] = to_f32(rz[r]);
            }
        }
        __syncthreads();
        if (t0 + SS_TC < n) fetch(t0 + SS_TC);
        // only the state's own update is a chain from token to token: the exponentials, the read-out's sum over the states and
        // its reduction over the eight lanes of a channel overlap between neighbouring tokens once the loop is unrolled
#pragma unroll 4
        for (int tt = 0; tt < nt; ++tt) {
            const float step = st[tt * 32 + cl], sx = step * xs[tt * 32 + cl];
            float y = 0.f;
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                const int nn = l + 8 * g;
                if (nn < N) {
                    s[g] = fmaf(expf(step * a[g]), s[g], sx * Bs[tt * N + nn]);
                    y = fmaf(s[g], Cs[tt * N + nn], y);
                }
            }
            y += __shfl_xor_sync(0xffffffffu, y, 1);
            y += __shfl_xor_sync(0xffffffffu, y, 2);
            y += __shfl_xor_sync(0xffffffffu, y, 4);
            if (l == 0) ys[tt * 32 + cl] = y;
        }
        __syncthreads();
        // skip term, gate and store for the whole chunk: a warp writes 32 neighbouring channels of one token
        for (int i = threadIdx.x; i < nt * 32; i += 256) {
            const int tt = i >> 5, cc = c0 + (i & 31);
            if (cc < I) out[(size_t)(qs + t0 + tt) * I + cc] = from_f32<T>((ys[i] + Dv[cc] * xs[i]) * silu(zs[i]));
        }
    }
#pragma unroll
    for (int g = 0; g < NG; ++g) {
        const int nn = l + 8 * g;
        if (live && nn < N) S[nn] = s[g];
    }
}

}  // namespace

// p [T, ldp] = q | k | v before silu (2 H D + H V columns); prep: float32 scratch [T, 2 H D + H V]; out float32 [T, H V].
MI_EXPORT int mi_lightning_scan(const void* p, int ldp, float* prep, const float* decay, float* state, long long state_stride, float* out,
                                const int* seg_q_start, const int* seg_slot, int T_, int num_segs, int H, int D, int V, int dtype,
                                cudaStream_t stream) {
    if (num_segs == 0 || T_ == 0) return 0;
    const int n = 2 * H * D + H * V;
    dim3 pgrid(T_, T_ >= 256 ? 1 : min(8, (n + 255) / 256));
    if (dtype == MI_BF16) silu_f32_kernel<__nv_bfloat16><<<pgrid, 256, 0, stream>>>((const __nv_bfloat16*)p, ldp, prep, n);
    else silu_f32_kernel<float><<<pgrid, 256, 0, stream>>>((const float*)p, ldp, prep, n);
    int err = (int)cudaGetLastError();
    if (err) return err;
    ScanLayout L{n, 0, H * D, 2 * H * D, 0, 0, 0, 0};
    return launch_scan<0>(prep, L, decay, state, state_stride, out, seg_q_start, seg_slot, T_, num_segs, H, H, D, V, stream);
}

// p [T, ldp] = q | k | v as projected; inv_freq: half frequencies (nullptr or half = 0: no rotation).  Otherwise as mi_lightning_scan.
MI_EXPORT int mi_retention_scan(const void* p, int ldp, float* prep, const int* positions, const float* inv_freq, int half, float k_scale,
                                const float* decay, float* state, long long state_stride, float* out, const int* seg_q_start,
                                const int* seg_slot, int T_, int num_segs, int H, int D, int V, int dtype, cudaStream_t stream) {
    if (num_segs == 0 || T_ == 0) return 0;
    if (2 * half > D) return -2;
    const int n = 2 * H * D + H * V;
    dim3 pgrid(T_, T_ >= 256 ? 1 : min(8, (n + 255) / 256));
    if (dtype == MI_BF16) rotate_f32_kernel<__nv_bfloat16><<<pgrid, 256, 0, stream>>>((const __nv_bfloat16*)p, ldp, prep, positions, inv_freq, inv_freq ? half : 0, k_scale, H, D, V);
    else rotate_f32_kernel<float><<<pgrid, 256, 0, stream>>>((const float*)p, ldp, prep, positions, inv_freq, inv_freq ? half : 0, k_scale, H, D, V);
    int err = (int)cudaGetLastError();
    if (err) return err;
    ScanLayout L{n, 0, H * D, 2 * H * D, 0, 0, 0, 0};
    return launch_scan<0>(prep, L, decay, state, state_stride, out, seg_q_start, seg_slot, T_, num_segs, H, H, D, V, stream);
}

MI_EXPORT int mi_delta_scan(const float* prep, int ld, float* state, long long state_stride, float* out, const int* seg_q_start,
                            const int* seg_slot, int T_, int num_segs, int H, int KV, int D, int V, cudaStream_t stream) {
    const int C = 2 * KV * D + H * V;
    ScanLayout L{ld, 0, KV * D, 2 * KV * D, C, C + H * D, 0, 0};
    return launch_scan<1>(prep, L, nullptr, state, state_stride, out, seg_q_start, seg_slot, T_, num_segs, H, KV, D, V, stream);
}

MI_EXPORT int mi_delta_prepare(const void* p, int ldp, const void* a, int lda, const float* conv, const float* A_log, const float* dt_bias,
                               float* state, long long state_stride, long long hist_off, float* out, int ldo, const int* token_seg,
                               const int* seg_q_start, const int* seg_slot, int T_, int num_segs, int H, int KV, int D, int V, int taps,
                               float unit_eps, int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    const int C = 2 * KV * D + H * V;
    const int units = 2 * KV + 2 * H + 1;
    if (units > 65535) return -2;
    const int toks = T_ >= 1024 ? 8 : 1;
    dim3 pgrid((T_ + toks - 1) / toks, units);
    if (dtype == MI_BF16)
        delta_prepare_kernel<__nv_bfloat16><<<pgrid, 128, 0, stream>>>((const __nv_bfloat16*)p, ldp, (const __nv_bfloat16*)a, lda, conv, A_log, dt_bias,
                                                                       state, state_stride, hist_off, out, ldo, token_seg, seg_q_start, seg_slot,
                                                                       H, KV, D, V, taps, unit_eps, T_, toks);
    else
        delta_prepare_kernel<float><<<pgrid, 128, 0, stream>>>((const float*)p, ldp, (const float*)a, lda, conv, A_log, dt_bias, state, state_stride,
                                                               hist_off, out, ldo, token_seg, seg_q_start, seg_slot, H, KV, D, V, taps, unit_eps, T_, toks);
    int err = (int)cudaGetLastError();
    if (err || taps <= 1) return err;
    dim3 grid(num_segs, (C + 255) / 256);
    if (dtype == MI_BF16)
        conv_tail_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)p, ldp, state, state_stride, hist_off, seg_q_start, seg_slot, C, taps);
    else
        conv_tail_kernel<float><<<grid, 256, 0, stream>>>((const float*)p, ldp, state, state_stride, hist_off, seg_q_start, seg_slot, C, taps);
    return (int)cudaGetLastError();
}


// h [T, ldh] (C channels read), out [T, C] contiguous in the same type; the history lies at state[slot] + hist_off
MI_EXPORT int mi_short_conv(const void* h, int ldh, const float* w, const float* bias, float* state, long long state_stride, long long hist_off,
                            void* out, const int* token_seg, const int* seg_q_start, const int* seg_slot, int T_, int num_segs, int C, int taps,
                            int residual, int act, int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    dim3 grid(T_, T_ >= 256 ? 1 : min(8, (C + 255) / 256));
    const int shift = (T_ == num_segs && T_ < 256) ? 1 : 0;      // a step of single tokens: one kernel filters and moves the slot's inputs
    // prompt portions only: a decode step's few tokens are done sooner by the kernel that needs no staging of weights
    const bool vec = dtype == MI_BF16 && T_ >= 256 && taps >= 1 && taps <= 4 && C % 8 == 0 && ldh % 8 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                     (taps == 1 || (state_stride % 4 == 0 && hist_off % 4 == 0 && (uintptr_t)state % 16 == 0)) && (!bias || (uintptr_t)bias % 16 == 0);
    if (vec) {
        const int tok = T_ >= 1024 ? 8 : 2, threads = min(256, (C / 8 + 31) / 32 * 32);
        dim3 vgrid((T_ + tok - 1) / tok, (C / 8 + threads - 1) / threads);
#define GO(TAPS, TOK) short_conv_vec_kernel<TAPS, TOK><<<vgrid, threads, 0, stream>>>((const __nv_bfloat16*)h, ldh, w, bias, state, state_stride, hist_off, \
                          (__nv_bfloat16*)out, token_seg, seg_q_start, seg_slot, T_, C, residual, act)
#define PICK(TAPS) do { if (tok == 8) GO(TAPS, 8); else GO(TAPS, 2); } while (0)
        if (taps == 1) PICK(1); else if (taps == 2) PICK(2); else if (taps == 3) PICK(3); else PICK(4);
#undef PICK
#undef GO
    } else if (dtype == MI_BF16)
        short_conv_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)h, ldh, w, bias, state, state_stride, hist_off, (__nv_bfloat16*)out,
                                                                    token_seg, seg_q_start, seg_slot, C, taps, residual, act, shift);
    else
        short_conv_kernel<float><<<grid, 256, 0, stream>>>((const float*)h, ldh, w, bias, state, state_stride, hist_off, (float*)out, token_seg,
                                                            seg_q_start, seg_slot, C, taps, residual, act, shift);
    int err = (int)cudaGetLastError();
    if (err || taps <= 1 || shift) return err;
    dim3 tgrid(num_segs, (C + 255) / 256);
    if (dtype == MI_BF16)
        conv_tail_kernel<__nv_bfloat16><<<tgrid, 256, 0, stream>>>((const __nv_bfloat16*)h, ldh, state, state_stride, hist_off, seg_q_start, seg_slot, C, taps);
    else
        conv_tail_kernel<float><<<tgrid, 256, 0, stream>>>((const float*)h, ldh, state, state_stride, hist_off, seg_q_start, seg_slot, C, taps);
    return (int)cudaGetLastError();
}

// out [T, ldo] float32 = r | k | u | a u | decay | v (ldo >= 5 H D + H V)
MI_EXPORT int mi_general_delta_prepare(const void* p, int ldp, const void* w2, const float* w0, const float* a_b, float* out, int ldo, int T_,
                                       int H, int D, int V, int rank, float decay_scale, float unit_eps, int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    const int tok = T_ >= 512 ? 8 : 1;
    const size_t smem = (size_t)tok * (rank + H) * sizeof(float);
    if (smem > 48 * 1024) return -2;
    const int HD = H * D;
    dim3 grid((T_ + tok - 1) / tok, tok == 8 ? 1 : min(16, (HD + 255) / 256));
#define GO(T, TOK) general_delta_prepare_kernel<T, TOK><<<grid, 256, smem, stream>>>((const T*)p, ldp, (const T*)w2, w0, a_b, out, ldo, T_, H, D, V, rank, \
                                                                                     decay_scale, unit_eps)
    if (dtype == MI_BF16) { if (tok == 8) GO(__nv_bfloat16, 8); else GO(__nv_bfloat16, 1); }
    else { if (tok == 8) GO(float, 8); else GO(float, 1); }
#undef GO
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_general_delta_scan(const float* prep, int ld, float* state, long long state_stride, float* out, const int* seg_q_start,
                                    const int* seg_slot, int T_, int num_segs, int H, int D, int V, cudaStream_t stream) {
    const int HD = H * D;
    ScanLayout L{ld, 0, HD, 5 * HD, 4 * HD, 0, 2 * HD, 3 * HD};
    return launch_scan<2>(prep, L, nullptr, state, state_stride, out, seg_q_start, seg_slot, T_, num_segs, H, H, D, V, stream);
}

// p [T, ldp] = q | k | v (| gate, at `gate`); gl float32 [T, 2 H] gate logits; lg [T, 2 H], mneg [T, H], prep [T, ldprep], full [T, H (V + 4)]:
// float32 scratch.  The slot holds H D (V + 4) state floats, then the H running maxima.  y [T, H V] in the type of p.
MI_EXPORT int mi_matrix_memory(const void* p, int ldp, const float* gl, const float* gate_bias, float cap, int capped, float den_eps,
                               const float* norm, const void* gate, int gate_stride, float eps, float* lg, float* mneg, float* prep, int ldprep,
                               float* full, void* y, float* state, long long state_stride, const int* seg_q_start, const int* seg_slot,
                               int T_, int num_segs, int H, int D, int V, int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    const int W = V + 4, HD = H * D, n = T_ * 2 * H;
    if (H > 65535) return -2;
    const float q_scale = 1.f / sqrtf((float)D);
    if (T_ == num_segs && (size_t)2 * H * sizeof(float) <= 48 * 1024) {          // every entry brings one token: gates, maximum and prologue in one kernel
        if (dtype == MI_BF16)
            memory_step_kernel<__nv_bfloat16><<<num_segs, 256, 2 * H * sizeof(float), stream>>>((const __nv_bfloat16*)p, ldp, gl, gate_bias, cap, capped, mneg, prep, ldprep,
                                                                                                 state, state_stride, (long long)HD * W, seg_q_start, seg_slot, H, D, V, q_scale);
        else
            memory_step_kernel<float><<<num_segs, 256, 2 * H * sizeof(float), stream>>>((const float*)p, ldp, gl, gate_bias, cap, capped, mneg, prep, ldprep, state, state_stride,
                                                                                         (long long)HD * W, seg_q_start, seg_slot, H, D, V, q_scale);
    } else {
        memory_gates_kernel<<<(n + 255) / 256, 256, 0, stream>>>(gl, gate_bias, lg, n, H, cap, capped);
        memory_max_kernel<<<dim3(num_segs, (H + 7) / 8), 256, 0, stream>>>(lg, mneg, state, state_stride, (long long)HD * W, seg_q_start, seg_slot, H);
        if (dtype == MI_BF16) memory_prepare_kernel<__nv_bfloat16><<<T_, 256, 0, stream>>>((const __nv_bfloat16*)p, ldp, lg, prep, ldprep, H, D, V, q_scale);
        else memory_prepare_kernel<float><<<T_, 256, 0, stream>>>((const float*)p, ldp, lg, prep, ldprep, H, D, V, q_scale);
    }
    int err = (int)cudaGetLastError();
    if (err) return err;
    ScanLayout L{ldprep, 0, HD, 2 * HD, 0, 2 * HD + H * W, 0, 0};
    err = launch_scan<3>(prep, L, nullptr, state, state_stride, full, seg_q_start, seg_slot, T_, num_segs, H, H, D, W, stream);
    if (err) return err;
    dim3 grid(T_, H);
    if (dtype == MI_BF16)
        memory_output_kernel<__nv_bfloat16><<<grid, 32, 0, stream>>>(full, mneg, norm, (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)y, H, V, den_eps, eps);
    else
        memory_output_kernel<float><<<grid, 32, 0, stream>>>(full, mneg, norm, (const float*)gate, gate_stride, (float*)y, H, V, den_eps, eps);
    return (int)cudaGetLastError();
}

// x [T, I] and out [T, I] contiguous in the run's type; dt float32 [T, I] (before bias and softplus); B, C, z: strided views; A float32 [I, N]
MI_EXPORT int mi_selective_scan(const void* x, const float* dt, const float* dt_b, const float* A, const void* B, int ldb, const void* C, int ldc,
                                const float* Dv, const void* z, int ldz, float* state, long long state_stride, void* out,
                                const int* seg_q_start, const int* seg_slot, int T_, int num_segs, int I, int N, int dtype, cudaStream_t stream) {
    if (T_ == 0 || num_segs == 0) return 0;
    if (N > 128) return -2;
    const int NG = (N + 7) / 8;
    const size_t smem = (size_t)SS_TC * (2 * N + 128) * sizeof(float);
    dim3 grid(num_segs, (I + 31) / 32);
    if (grid.y > 65535) return -2;
#define GO(T, G) selective_scan_kernel<T, G><<<grid, 256, smem, stream>>>((const T*)x, dt, dt_b, A, (const T*)B, ldb, (const T*)C, ldc, Dv, (const T*)z, ldz, \
                                                                          state, state_stride, (T*)out, seg_q_start, seg_slot, I, N)
#define PICK(T) do { if (NG <= 1) GO(T, 1); else if (NG == 2) GO(T, 2); else if (NG == 3) GO(T, 3); else if (NG == 4) GO(T, 4); \
                     else if (NG <= 8) GO(T, 8); else GO(T, 16); } while (0)
    if (dtype == MI_BF16) PICK(__nv_bfloat16); else PICK(float);
#undef PICK
#undef GO
    return (int)cudaGetLastError();
}
