// Retention: linear attention with one fixed decay per head and neither softmax nor denominator.  Per head, with a
// state S [dk, dv] that starts at zero and is carried from token to token in the request's state slot:
//
//     S <- decay S + k v^T;      o = S^T q
//
//  * retention_prep_kernel turns the first `rd` dimensions of every head of q and k by position * inv_freq[pair] (pairs by
//    halves, or of neighbours) and multiplies k by a scale, in place on the FP32 result of the projection; a block per token.
//  * retention_kernel walks a request's tokens in order.  A block owns 16 columns of one head of one request, a warp four of
//    them (wide keys: two warps, half of the rows each): lane l holds rows l, l + 32, ... of its four columns in registers, so
//    a token costs two shared-memory reads (k and q of a row) per twelve floating-point instructions.  The sums over the rows are left until eight tokens are done:
//    the 32 partial sums a lane then holds (8 tokens x 4 columns) are summed over the lanes by one butterfly that halves
//    the values with every stage (31 shuffles for all of them, and every value takes the same tree of additions, so a token's
//    result does not depend on where in a tile it stands or where a prompt was cut).  q, k and v of eight tokens at a time
//    are staged in shared memory, the next tile fetched into registers while this one is walked.
//
// Everything is FP32: angles, the rotation, decays and their powers, the state and every sum.
#include "common.cuh"

namespace {

constexpr int RET_WARPS = 4, RET_C = 4, RET_TILE = 8, RET_MAX_DK = 256;

// One block per token: the sines and cosines of its rd / 2 angles are made once (they are the same for every head, for q
// and for k), then every pair of q and of k is turned in place and the rest of k scaled; what neither turns nor scales
// is not touched.
__global__ void __launch_bounds__(256) retention_prep_kernel(float* p, int ld, int H, int dk, int q_col, int k_col,
                                                             const float* inv_freq, int rd, int neighbours, float k_scale,
                                                             const int* positions) {
    pdl_enter();
    extern __shared__ float xs[];            // cos [rd / 2] | sin [rd / 2]
    const int t = blockIdx.x, half = rd / 2;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &xs[half + i], &xs[i]);
    __syncthreads();
    float* row = p + (size_t)t * ld;
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

// grid (R, H, ceil(dv / 16)), 128 RS threads.  p: FP32 [T, ld] with q, k (prepared) and v at their columns; state: FP32
// [slots, H, dv, dk] (a column's rows lie together); o: FP32 [T, H dv].  JN: rows per lane over the whole key (dk <= 32 JN);
// RS: warps that share a column group, each with JN / RS of those rows (their sums meet in shared memory, in a fixed order).
template <int JN, int RS>
__global__ void __launch_bounds__(RET_WARPS * 32 * RS) retention_kernel(const float* p, int ld, int q_col, int k_col, int v_col, const float* decay,
                                                                        float* state, const int* q_start, const int* slot_ids, float* o, int H,
                                                                        int dk, int dv) {
    pdl_enter();
    constexpr int DKP = 32 * JN, JW = JN / RS, THREADS = RET_WARPS * 32 * RS, COLS = RET_WARPS * RET_C;
    constexpr int PER_THREAD = RET_TILE * DKP / THREADS;                 // elements of q (and of k) a thread stages per tile
    static_assert(JN % RS == 0 && RET_TILE * DKP % THREADS == 0, "rows divide among the warps, a tile among the threads");
    static_assert(RET_TILE * RET_C == 32 && RET_TILE * COLS == RET_WARPS * 32, "one value per lane after the butterfly; one v per thread");
    extern __shared__ __align__(16) float sm[];   // q [2][TILE][DKP] | k [2][TILE][DKP] | v [2][TILE][COLS] | sums [2][WARPS][32]
    float* qs = sm;
    float* ks = qs + 2 * RET_TILE * DKP;
    float* vs = ks + 2 * RET_TILE * DKP;
    float* red = vs + 2 * RET_TILE * COLS;
    const int r = blockIdx.x, head = blockIdx.y, c0 = blockIdx.z * COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, cg = warp % RET_WARPS, rs = warp / RET_WARPS;
    const int cw = c0 + cg * RET_C, row0 = rs * 32 * JW + lane;
    const int t0 = q_start[r], t1 = q_start[r + 1];
    const float d = decay[head];
    float* cols = state + ((size_t)slot_ids[r] * H + head) * dv * dk;
    float s[JW][RET_C];
#pragma unroll
    for (int j = 0; j < JW; ++j)
#pragma unroll
        for (int c = 0; c < RET_C; ++c) {
            const int row = row0 + 32 * j;
            s[j][c] = (cw + c < dv && row < dk) ? cols[(size_t)(cw + c) * dk + row] : 0.0f;
        }
    float fq[PER_THREAD], fk[PER_THREAD], fv = 0.0f;
    auto fetch = [&](int ta) {                // this thread's share of the tile that starts at token ta, into registers
        const int n = min(RET_TILE, t1 - ta);
#pragma unroll
        for (int e = 0; e < PER_THREAD; ++e) {
            const int i = threadIdx.x + e * THREADS, tt = i / DKP, row = i % DKP;
            const bool in = tt < n && row < dk;
            const float* src = p + (size_t)(ta + tt) * ld + (size_t)head * dk + row;
            fq[e] = in ? src[q_col] : 0.0f;
            fk[e] = in ? src[k_col] : 0.0f;
        }
        if (threadIdx.x < RET_TILE * COLS) {
            const int tt = threadIdx.x / COLS, cc = c0 + threadIdx.x % COLS;
            fv = (tt < n && cc < dv) ? p[(size_t)(ta + tt) * ld + v_col + (size_t)head * dv + cc] : 0.0f;
        }
    };
    auto put = [&](int b) {
#pragma unroll
        for (int e = 0; e < PER_THREAD; ++e) {
            const int i = threadIdx.x + e * THREADS;
            qs[b * RET_TILE * DKP + i] = fq[e];
            ks[b * RET_TILE * DKP + i] = fk[e];
        }
        if (threadIdx.x < RET_TILE * COLS) vs[b * RET_TILE * COLS + threadIdx.x] = fv;
    };
    if (t0 < t1) {
        fetch(t0);
        put(0);
    }
    __syncthreads();
    int b = 0;
    for (int ta = t0; ta < t1; ta += RET_TILE, b ^= 1) {
        const int n = min(RET_TILE, t1 - ta);
        const bool more = ta + RET_TILE < t1;
        if (more) fetch(ta + RET_TILE);
        float a[RET_TILE * RET_C];
        if (cw < dv) {
            const float* qb = qs + b * RET_TILE * DKP + row0;
            const float* kb = ks + b * RET_TILE * DKP + row0;
            const float* vb = vs + b * RET_TILE * COLS + cg * RET_C;
#pragma unroll
            for (int i = 0; i < RET_TILE * RET_C; ++i) a[i] = 0.0f;
            auto token = [&](int tt) {
                const float4 v = *reinterpret_cast<const float4*>(vb + tt * COLS);
                const float vv[RET_C] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < JW; ++j) {
                    const float kk = kb[tt * DKP + 32 * j], qq = qb[tt * DKP + 32 * j];
#pragma unroll
                    for (int c = 0; c < RET_C; ++c) {
                        s[j][c] = fmaf(d, s[j][c], kk * vv[c]);
                        a[tt * RET_C + c] = fmaf(s[j][c], qq, a[tt * RET_C + c]);
                    }
                }
            };
            if (n == RET_TILE) {              // a full tile: nothing stands between the tokens' loads and sums
#pragma unroll
                for (int tt = 0; tt < RET_TILE; ++tt) token(tt);
            } else {
#pragma unroll
                for (int tt = 0; tt < RET_TILE; ++tt)
                    if (tt < n) token(tt);
            }
            // lane l ends with the sum over all lanes of value l (token l / 4 of the tile, column l % 4)
#pragma unroll
            for (int half = 16; half >= 1; half >>= 1) {
                const bool up = (lane & half) != 0;
#pragma unroll
                for (int i = 0; i < half; ++i) {
                    const float send = up ? a[i] : a[i + half];
                    const float keep = up ? a[i + half] : a[i];
                    a[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
                }
            }
            if (rs > 0) red[(b * RET_WARPS + cg) * 32 + lane] = a[0];
        }
        if (more) put(b ^ 1);
        __syncthreads();
        if (rs == 0 && cw < dv) {
            const int tt = lane / RET_C, c = cw + lane % RET_C;
            const float sum = RS > 1 ? a[0] + red[(b * RET_WARPS + cg) * 32 + lane] : a[0];
            if (tt < n && c < dv) o[((size_t)(ta + tt) * H + head) * dv + c] = sum;
        }
    }
    if (t0 < t1) {
#pragma unroll
        for (int j = 0; j < JW; ++j)
#pragma unroll
            for (int c = 0; c < RET_C; ++c) {
                const int row = row0 + 32 * j;
                if (cw + c < dv && row < dk) cols[(size_t)(cw + c) * dk + row] = s[j][c];
            }
    }
}

template <int JN, int RS>
void launch_retention(dim3 grid, cudaStream_t st, const float* p, int ld, int q_col, int k_col, int v_col, const float* decay, float* state,
                      const int* q_start, const int* slot_ids, float* o, int H, int dk, int dv) {
    const size_t smem = (size_t)(4 * RET_TILE * 32 * JN + 2 * RET_TILE * RET_WARPS * RET_C + 2 * RET_WARPS * 32) * sizeof(float);
    q6k_launch(retention_kernel<JN, RS>, grid, RET_WARPS * 32 * RS, smem, st, p, ld, q_col, k_col, v_col, decay, state, q_start, slot_ids, o, H, dk, dv);
}

}  // namespace

Q6K_API int q6k_retention_max_dim() { return RET_MAX_DK; }

// Rotates q and k of every head in place and scales k.
Q6K_API int q6k_retention_prep(float* p, int ld, int T_, int H, int dk, int q_col, int k_col,
                               const float* inv_freq, int rd, int neighbours, float k_scale, const int* positions, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && H > 0 && dk > 0 && 2 * H <= 65535, "retention_prep: bad sizes T=%d H=%d dk=%d", T_, H, dk);
    Q6K_REQUIRE(rd >= 0 && rd % 2 == 0 && rd <= dk && (rd == 0 || inv_freq), "retention_prep: %d turning dimensions of %d", rd, dk);
    if (rd == 0 && k_scale == 1.0f) return 0;
    q6k_launch(retention_prep_kernel, dim3(T_), 256, (size_t)rd * sizeof(float), st, p, ld, H, dk, q_col, k_col,
               inv_freq, rd, neighbours, k_scale, positions);
    return q6k_check_launch("retention_prep");
}

Q6K_API int q6k_retention(const float* p, int ld, int q_col, int k_col, int v_col, const float* decay, float* state, const int* q_start,
                          const int* slot_ids, int R, float* o, int H, int dk, int dv, cudaStream_t st) {
    if (R == 0) return 0;
    Q6K_REQUIRE(R > 0 && H > 0 && dk > 0 && dv > 0 && dk <= RET_MAX_DK, "retention: bad sizes R=%d H=%d dk=%d (at most %d) dv=%d", R, H, dk, RET_MAX_DK, dv);
    const int zb = (dv + RET_WARPS * RET_C - 1) / (RET_WARPS * RET_C);
    Q6K_REQUIRE(H <= 65535 && zb <= 65535, "retention: grid too large");
    const dim3 grid(R, H, zb);
    if (dk <= 32) launch_retention<1, 1>(grid, st, p, ld, q_col, k_col, v_col, decay, state, q_start, slot_ids, o, H, dk, dv);
    else if (dk <= 64) launch_retention<2, 2>(grid, st, p, ld, q_col, k_col, v_col, decay, state, q_start, slot_ids, o, H, dk, dv);
    else if (dk <= 128) launch_retention<4, 2>(grid, st, p, ld, q_col, k_col, v_col, decay, state, q_start, slot_ids, o, H, dk, dv);
    else launch_retention<8, 2>(grid, st, p, ld, q_col, k_col, v_col, decay, state, q_start, slot_ids, o, H, dk, dv);
    return q6k_check_launch("retention");
}
