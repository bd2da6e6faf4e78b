// Retention: linear attention with one fixed decay per head and neither softmax nor denominator.  Per head, with a
// state S [dk, dv] that starts at zero and is carried from token to token in the request's state slot:
//
//     S <- decay S + k v^T;      o = S^T q
//
//  * retention_prep_kernel turns the first `rd` dimensions of every head of q and k by position * inv_freq[pair] (pairs by
//    halves, or of neighbours) and multiplies k by a scale, in place on the FP32 result of the projection; a block per token.
//    Before that it may pass the row's first `act_cols` columns (q, k and v of a mixer that activates them) through silu.
//  * retention_kernel walks a request's tokens in order.  A block owns 16 columns of one head of one request; a thread holds
//    a stretch of consecutive rows of ONE column in registers (lane = column and one of two stretches, eight warps = sixteen
//    stretches), so k and q of its rows come as 16-byte reads every lane of a half-warp shares and a token costs three
//    floating-point instructions per element of the state and little else.  A token's sum over the rows is the thread's own
//    (in row order), then the two stretches of a warp (one shuffle), then the eight warps' through shared memory, in the
//    warps' order: the same tree for every token wherever a prompt was cut.  q, k and v of eight tokens at a time are
//    copied to shared memory asynchronously, three tiles ahead of the one that is walked (a tile's first read is a miss in
//    L2 for one block of a head, and its latency is several times a tile's work).
//
// Everything is FP32: angles, the rotation, decays and their powers, the state and every sum.
#include "common.cuh"

namespace {

constexpr int RET_WARPS = 8, RET_THREADS = RET_WARPS * 32, RET_COLS = 16, RET_CHUNKS = 2 * RET_WARPS, RET_TILE = 8, RET_STAGES = 4, RET_MAX_DK = 256;

// One block per token: the sines and cosines of its rd / 2 angles are made once (they are the same for every head, for q
// and for k), then every pair of q and of k is turned in place and the rest of k scaled; what neither turns nor scales
// is not touched.
__global__ void __launch_bounds__(256) retention_prep_kernel(float* p, int ld, int H, int dk, int q_col, int k_col,
                                                             const float* inv_freq, int rd, int neighbours, float k_scale,
                                                             const int* positions, int act_cols) {
    pdl_enter();
    extern __shared__ float xs[];            // cos [rd / 2] | sin [rd / 2]
    const int t = blockIdx.x, half = rd / 2;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &xs[half + i], &xs[i]);
    float* row = p + (size_t)t * ld;
    for (int c = threadIdx.x; c < act_cols; c += blockDim.x) {             // silu on the projections, before anything else
        const float z = row[c];
        row[c] = z / (1.0f + expf(-z));
    }
    __syncthreads();
    for (int w = threadIdx.x; w < 2 * H * half; w += blockDim.x) {          // (q or k, head, pair)
        const int i = w % half, h = (w / half) % H, is_k = w / (half * H);
        float* x = row + (is_k ? k_col : q_col) + (size_t)h * dk;
        const int a = neighbours ? 2 * i : i, b = neighbours ? 2 * i + 1 : i + half;
        const float u = x[a], v = x[b], cs = xs[i], sn = xs[half + i], mul = is_k ? k_scale : 1.0f;
        x[a] = (u * cs - v * sn) * mul;
        x[b] = (v * cs + u * sn) * mul;
    }
    if (k_scale != 1.0f) {
        const int rest = dk - rd;
        for (int w = threadIdx.x; w < H * rest; w += blockDim.x) {
            float* x = row + k_col + (size_t)(w / rest) * dk + rd + w % rest;
            *x *= k_scale;
        }
    }
}

// Four bytes from global to shared memory without passing registers; `in` false writes a zero and reads nothing.
__device__ __forceinline__ void ret_copy(float* dst, const float* src, bool in) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = in ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void ret_copy16(float* dst, const float* src, bool in) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = in ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

// grid (R, H, ceil(dv / 16)), 256 threads.  p: FP32 [T, ld] with q, k (prepared) and v at their columns; state: FP32
// [slots, H, dk, dv]; o: FP32 [T, H dv].  RPT: rows per thread (dk <= 16 RPT).  STAGES tiles are in flight or in use.
// WIDE: every head's q and k start on 16 bytes in every row of p and dk is a multiple of 4 (copies of 16 bytes).
template <int RPT, int STAGES, bool WIDE>
__global__ void __launch_bounds__(RET_THREADS) retention_kernel(const float* p, int ld, int q_col, int k_col, int v_col, const float* decay,
                                                                float* state, const int* q_start, const int* slot_ids, float* o, int H,
                                                                int dk, int dv) {
    pdl_enter();
    constexpr int DKP = RET_CHUNKS * RPT;                                // rows, padded
    constexpr int PER_THREAD = RET_TILE * DKP / RET_THREADS;             // elements of q (and of k) a thread stages per tile
    static_assert(RPT % 4 == 0 && RET_TILE * DKP % RET_THREADS == 0 && RET_TILE * RET_COLS <= RET_THREADS, "16-byte reads; a tile divides among the threads");
    extern __shared__ __align__(16) float sm[];   // q [STAGES][TILE][DKP] | k likewise | v [STAGES][TILE][COLS] | sums [2][TILE][WARPS][COLS]
    float* qs = sm;
    float* ks = qs + STAGES * RET_TILE * DKP;
    float* vs = ks + STAGES * RET_TILE * DKP;
    float* red = vs + STAGES * RET_TILE * RET_COLS;
    const int r = blockIdx.x, head = blockIdx.y, c0 = blockIdx.z * RET_COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, cl = lane % RET_COLS, col = c0 + cl;
    const int row0 = (warp * 2 + lane / RET_COLS) * RPT;                 // this thread's first row
    const int t0 = q_start[r], t1 = q_start[r + 1];
    if (t0 >= t1) return;
    const float d = decay[head];
    float* mine = state + ((size_t)slot_ids[r] * H + head) * dk * dv + (col < dv ? col : 0);
    float s[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) s[i] = (col < dv && row0 + i < dk) ? mine[(size_t)(row0 + i) * dv] : 0.0f;
    auto fetch = [&](int ta, int b) {         // this thread's share of the tile that starts at token ta, on its way to buffer b
        const int n = min(RET_TILE, t1 - ta);
        if (n > 0) {
            if (WIDE) {
#pragma unroll
                for (int e = 0; e < (PER_THREAD + 3) / 4; ++e) {
                    const int i = (threadIdx.x + e * RET_THREADS) * 4, tt = i / DKP, row = i % DKP;
                    if (PER_THREAD >= 4 || i < RET_TILE * DKP) {
                        const bool in = tt < n && row < dk;
                        const float* src = in ? p + (size_t)(ta + tt) * ld + (size_t)head * dk + row : p;
                        ret_copy16(qs + b * RET_TILE * DKP + i, src + (in ? q_col : 0), in);
                        ret_copy16(ks + b * RET_TILE * DKP + i, src + (in ? k_col : 0), in);
                    }
                }
            } else {
#pragma unroll
                for (int e = 0; e < PER_THREAD; ++e) {
                    const int i = threadIdx.x + e * RET_THREADS, tt = i / DKP, row = i % DKP;
                    const bool in = tt < n && row < dk;
                    const float* src = in ? p + (size_t)(ta + tt) * ld + (size_t)head * dk + row : p;
                    ret_copy(qs + b * RET_TILE * DKP + i, src + (in ? q_col : 0), in);
                    ret_copy(ks + b * RET_TILE * DKP + i, src + (in ? k_col : 0), in);
                }
            }
            if (threadIdx.x < RET_TILE * RET_COLS) {
                const int tt = threadIdx.x / RET_COLS, cc = c0 + threadIdx.x % RET_COLS;
                const bool in = tt < n && cc < dv;
                ret_copy(vs + b * RET_TILE * RET_COLS + threadIdx.x, in ? p + (size_t)(ta + tt) * ld + v_col + (size_t)head * dv + cc : p, in);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto finish = [&](int ta, int b2) {       // the warps' sums of one (token, column), in the warps' order
        if (threadIdx.x < RET_TILE * RET_COLS) {
            const int tt = threadIdx.x / RET_COLS, cc = threadIdx.x % RET_COLS;
            if (ta + tt < t1 && c0 + cc < dv) {
                const float* src = red + (b2 * RET_TILE + tt) * RET_WARPS * RET_COLS + cc;
                float sum = src[0];
#pragma unroll
                for (int w = 1; w < RET_WARPS; ++w) sum += src[w * RET_COLS];
                o[((size_t)(ta + tt) * H + head) * dv + c0 + cc] = sum;
            }
        }
    };
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) fetch(t0 + st * RET_TILE, st);
    int b = 0, b2 = 0;
    for (int ta = t0; ta < t1; ta += RET_TILE, b = b + 1 == STAGES ? 0 : b + 1, b2 ^= 1) {
        const int n = min(RET_TILE, t1 - ta);
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
        __syncthreads();                      // this tile has landed for everyone; the tile before it is done with
        if (ta > t0) finish(ta - RET_TILE, b2 ^ 1);
        fetch(ta + (STAGES - 1) * RET_TILE, b == 0 ? STAGES - 1 : b - 1);
        const float* qb = qs + b * RET_TILE * DKP + row0;
        const float* kb = ks + b * RET_TILE * DKP + row0;
        const float* vb = vs + b * RET_TILE * RET_COLS + cl;
        float* rb = red + (b2 * RET_TILE * RET_WARPS + warp) * RET_COLS + cl;
        auto token = [&](int tt) {
            const float v = vb[tt * RET_COLS];
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < RPT; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kb + tt * DKP + i);
                const float4 q4 = *reinterpret_cast<const float4*>(qb + tt * DKP + i);
                s[i] = fmaf(d, s[i], k4.x * v);
                acc = fmaf(s[i], q4.x, acc);
                s[i + 1] = fmaf(d, s[i + 1], k4.y * v);
                acc = fmaf(s[i + 1], q4.y, acc);
                s[i + 2] = fmaf(d, s[i + 2], k4.z * v);
                acc = fmaf(s[i + 2], q4.z, acc);
                s[i + 3] = fmaf(d, s[i + 3], k4.w * v);
                acc = fmaf(s[i + 3], q4.w, acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, RET_COLS);       // the lane with the same column and the warp's other rows
            if (lane < RET_COLS) rb[tt * RET_WARPS * RET_COLS] = acc;
        };
        if (n == RET_TILE) {                  // a full tile: the next token's rows are read while this one's are summed
            float4 kk[2][RPT / 4], qq[2][RPT / 4];
            float vv[RET_TILE];
#pragma unroll
            for (int tt = 0; tt < RET_TILE; ++tt) vv[tt] = vb[tt * RET_COLS];
#pragma unroll
            for (int i = 0; i < RPT / 4; ++i) {
                kk[0][i] = *reinterpret_cast<const float4*>(kb + 4 * i);
                qq[0][i] = *reinterpret_cast<const float4*>(qb + 4 * i);
            }
#pragma unroll
            for (int tt = 0; tt < RET_TILE; ++tt) {
                if (tt + 1 < RET_TILE) {
#pragma unroll
                    for (int i = 0; i < RPT / 4; ++i) {
                        kk[(tt + 1) & 1][i] = *reinterpret_cast<const float4*>(kb + (tt + 1) * DKP + 4 * i);
                        qq[(tt + 1) & 1][i] = *reinterpret_cast<const float4*>(qb + (tt + 1) * DKP + 4 * i);
                    }
                }
                const float v = vv[tt];
                float acc = 0.0f;
#pragma unroll
                for (int i = 0; i < RPT / 4; ++i) {
                    const float4 k4 = kk[tt & 1][i], q4 = qq[tt & 1][i];
                    s[4 * i] = fmaf(d, s[4 * i], k4.x * v);
                    acc = fmaf(s[4 * i], q4.x, acc);
                    s[4 * i + 1] = fmaf(d, s[4 * i + 1], k4.y * v);
                    acc = fmaf(s[4 * i + 1], q4.y, acc);
                    s[4 * i + 2] = fmaf(d, s[4 * i + 2], k4.z * v);
                    acc = fmaf(s[4 * i + 2], q4.z, acc);
                    s[4 * i + 3] = fmaf(d, s[4 * i + 3], k4.w * v);
                    acc = fmaf(s[4 * i + 3], q4.w, acc);
                }
                acc += __shfl_xor_sync(0xffffffffu, acc, RET_COLS);
                if (lane < RET_COLS) rb[tt * RET_WARPS * RET_COLS] = acc;
            }
        } else {
#pragma unroll
            for (int tt = 0; tt < RET_TILE; ++tt)
                if (tt < n) token(tt);
        }
    }
    __syncthreads();
    finish(t0 + (t1 - t0 - 1) / RET_TILE * RET_TILE, b2 ^ 1);
    if (col < dv) {
#pragma unroll
        for (int i = 0; i < RPT; ++i)
            if (row0 + i < dk) mine[(size_t)(row0 + i) * dv] = s[i];
    }
}

template <int RPT, int STAGES, bool WIDE>
int launch_retention(dim3 grid, cudaStream_t st, const float* p, int ld, int q_col, int k_col, int v_col, const float* decay, float* state,
                     const int* q_start, const int* slot_ids, float* o, int H, int dk, int dv) {
    const size_t smem = (size_t)(STAGES * RET_TILE * (2 * RET_CHUNKS * RPT + RET_COLS) + 2 * RET_TILE * RET_WARPS * RET_COLS) * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(retention_kernel<RPT, STAGES, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    q6k_launch(retention_kernel<RPT, STAGES, WIDE>, grid, RET_THREADS, smem, st, p, ld, q_col, k_col, v_col, decay, state, q_start, slot_ids, o, H, dk, dv);
    return 0;
}

}  // namespace

Q6K_API int q6k_retention_max_dim() { return RET_MAX_DK; }

// Rotates q and k of every head in place and scales k.
Q6K_API int q6k_retention_prep(float* p, int ld, int T_, int H, int dk, int q_col, int k_col,
                               const float* inv_freq, int rd, int neighbours, float k_scale, const int* positions, int act_cols,
                               cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && H > 0 && dk > 0 && 2 * H <= 65535, "retention_prep: bad sizes T=%d H=%d dk=%d", T_, H, dk);
    Q6K_REQUIRE(rd >= 0 && rd % 2 == 0 && rd <= dk && (rd == 0 || inv_freq), "retention_prep: %d turning dimensions of %d", rd, dk);
    Q6K_REQUIRE(act_cols >= 0 && act_cols <= ld, "retention_prep: %d activated columns of %d", act_cols, ld);
    if (rd == 0 && k_scale == 1.0f && act_cols == 0) return 0;
    q6k_launch(retention_prep_kernel, dim3(T_), 256, (size_t)rd * sizeof(float), st, p, ld, H, dk, q_col, k_col,
               inv_freq, rd, neighbours, k_scale, positions, act_cols);
    return q6k_check_launch("retention_prep");
}

Q6K_API int q6k_retention(const float* p, int ld, int q_col, int k_col, int v_col, const float* decay, float* state, const int* q_start,
                          const int* slot_ids, int R, float* o, int H, int dk, int dv, cudaStream_t st) {
    if (R == 0) return 0;
    Q6K_REQUIRE(R > 0 && H > 0 && dk > 0 && dv > 0 && dk <= RET_MAX_DK, "retention: bad sizes R=%d H=%d dk=%d (at most %d) dv=%d", R, H, dk, RET_MAX_DK, dv);
    const int zb = (dv + RET_COLS - 1) / RET_COLS;
    Q6K_REQUIRE(H <= 65535 && zb <= 65535, "retention: grid too large");
    const dim3 grid(R, H, zb);
    const bool wide = dk % 4 == 0 && ld % 4 == 0 && q_col % 4 == 0 && k_col % 4 == 0 && (reinterpret_cast<uintptr_t>(p) & 15) == 0;
#define RET_LAUNCH(RPT)                                                                                                               \
    do {                                                                                                                              \
        if (wide) launch_retention<RPT, RET_STAGES, true>(grid, st, p, ld, q_col, k_col, v_col, decay, state, q_start, slot_ids, o, H, dk, dv);       \
        else launch_retention<RPT, RET_STAGES, false>(grid, st, p, ld, q_col, k_col, v_col, decay, state, q_start, slot_ids, o, H, dk, dv);           \
    } while (0)
    if (dk <= 64) RET_LAUNCH(4);
    else if (dk <= 128) RET_LAUNCH(8);
    else RET_LAUNCH(16);
#undef RET_LAUNCH
    return q6k_check_launch("retention");
}
