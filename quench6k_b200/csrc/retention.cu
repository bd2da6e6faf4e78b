// Retention: linear attention with one fixed decay per head and neither softmax nor denominator.  Per head, with a
// state S [dk, dv] that starts at zero and is carried from token to token in the request's state slot:
//
//     S <- decay S + k v^T;      o = S^T q
//
//  * retention_prep_kernel turns the first `rd` dimensions of every head of q and k by position * inv_freq[pair] (pairs by
//    halves, or of neighbours) and multiplies k by a scale, in place on the FP32 result of the projection.
//  * retention_kernel walks a request's tokens in order.  A block owns 8 columns of one head of one request, a warp one
//    column: lane l holds rows l, l + 32, ... of it in registers.  A token costs one fused multiply-add per element and
//    one sum over the rows (lane-strided partial sums, then a butterfly: the same order for every token wherever a prompt
//    was cut).  q, k and v of 16 tokens at a time are staged in shared memory.
//
// Everything is FP32: angles, the rotation, decays and their powers, the state and every sum.
#include "common.cuh"

namespace {

constexpr int RET_COLS = 8, RET_TILE = 16, RET_MAX_DK = 256;

__global__ void __launch_bounds__(128) retention_prep_kernel(float* p, int ld, int H, int dk, int q_col, int k_col,
                                                             const float* inv_freq, int rd, int neighbours, float k_scale,
                                                             const int* positions) {
    pdl_enter();
    extern __shared__ float xs[];            // dk floats
    const int t = blockIdx.x, h = blockIdx.y % H, is_k = blockIdx.y / H;
    float* row = p + (size_t)t * ld + (is_k ? k_col : q_col) + (size_t)h * dk;
    for (int d = threadIdx.x; d < dk; d += blockDim.x) {
        xs[d] = row[d];
    }
    __syncthreads();
    const int pos = positions[t], half = rd / 2;
    const float mul = is_k ? k_scale : 1.0f;
    for (int d = threadIdx.x; d < dk; d += blockDim.x) {
        float v = xs[d];
        if (d < rd) {
            const int i = neighbours ? d >> 1 : (d < half ? d : d - half);
            const bool first = neighbours ? !(d & 1) : d < half;
            const int partner = neighbours ? d ^ 1 : (first ? d + half : d - half);
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            v = first ? xs[d] * cs - xs[partner] * sn : xs[d] * cs + xs[partner] * sn;
        }
        row[d] = v * mul;
    }
}

// grid (R, H, ceil(dv / 8)), 256 threads.  p: FP32 [T, ld] with q, k (prepared) and v at their columns; state: FP32
// [slots, H, dv, dk] (a column's rows lie together); o: FP32 [T, H dv].
__global__ void __launch_bounds__(RET_COLS * 32) retention_kernel(const float* p, int ld, int q_col, int k_col, int v_col, const float* decay,
                                                                  float* state, const int* q_start, const int* slot_ids, float* o, int H,
                                                                  int dk, int dv) {
    pdl_enter();
    extern __shared__ float sm[];            // q [TILE][dk] | k [TILE][dk] | v [TILE][8]
    float* qs = sm;
    float* ks = qs + RET_TILE * dk;
    float* vs = ks + RET_TILE * dk;
    const int r = blockIdx.x, head = blockIdx.y, c0 = blockIdx.z * RET_COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, c = c0 + warp;
    const int t0 = q_start[r], t1 = q_start[r + 1];
    const float d = decay[head];
    float* col = state + (((size_t)slot_ids[r] * H + head) * dv + (c < dv ? c : 0)) * dk;
    float s[RET_MAX_DK / 32];
#pragma unroll
    for (int j = 0; j < RET_MAX_DK / 32; ++j) {
        const int row = lane + 32 * j;
        s[j] = (c < dv && row < dk) ? col[row] : 0.0f;
    }
    for (int ta = t0; ta < t1; ta += RET_TILE) {
        const int n = min(RET_TILE, t1 - ta);
        __syncthreads();
        for (int i = threadIdx.x; i < n * dk; i += blockDim.x) {
            const int tt = i / dk, e = i % dk;
            const float* src = p + (size_t)(ta + tt) * ld + (size_t)head * dk + e;
            qs[tt * dk + e] = src[q_col];
            ks[tt * dk + e] = src[k_col];
        }
        for (int i = threadIdx.x; i < n * RET_COLS; i += blockDim.x) {
            const int tt = i / RET_COLS, cc = c0 + i % RET_COLS;
            vs[i] = cc < dv ? p[(size_t)(ta + tt) * ld + v_col + (size_t)head * dv + cc] : 0.0f;
        }
        __syncthreads();
        if (c >= dv) continue;
        for (int tt = 0; tt < n; ++tt) {
            const float v = vs[tt * RET_COLS + warp];
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < RET_MAX_DK / 32; ++j) {
                const int row = lane + 32 * j;
                if (row < dk) {
                    s[j] = fmaf(d, s[j], ks[tt * dk + row] * v);
                    acc = fmaf(s[j], qs[tt * dk + row], acc);
                }
            }
            acc = warp_sum(acc);
            if (lane == 0) o[((size_t)(ta + tt) * H + head) * dv + c] = acc;
        }
    }
    if (c < dv) {
#pragma unroll
        for (int j = 0; j < RET_MAX_DK / 32; ++j) {
            const int row = lane + 32 * j;
            if (row < dk) col[row] = s[j];
        }
    }
}

}  // namespace

Q6K_API int q6k_retention_max_dim() { return RET_MAX_DK; }

// Rotates q and k of every head in place and scales k.
Q6K_API int q6k_retention_prep(float* p, int ld, int T_, int H, int dk, int q_col, int k_col,
                               const float* inv_freq, int rd, int neighbours, float k_scale, const int* positions, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && H > 0 && dk > 0 && 2 * H <= 65535, "retention_prep: bad sizes T=%d H=%d dk=%d", T_, H, dk);
    Q6K_REQUIRE(rd >= 0 && rd % 2 == 0 && rd <= dk && (rd == 0 || inv_freq), "retention_prep: %d turning dimensions of %d", rd, dk);
    Q6K_REQUIRE((size_t)dk * sizeof(float) <= 48 * 1024, "retention_prep: heads of %d do not fit shared memory", dk);
    q6k_launch(retention_prep_kernel, dim3(T_, 2 * H), 128, (size_t)dk * sizeof(float), st, p, ld, H, dk, q_col, k_col,
               inv_freq, rd, neighbours, k_scale, positions);
    return q6k_check_launch("retention_prep");
}

Q6K_API int q6k_retention(const float* p, int ld, int q_col, int k_col, int v_col, const float* decay, float* state, const int* q_start,
                          const int* slot_ids, int R, float* o, int H, int dk, int dv, cudaStream_t st) {
    if (R == 0) return 0;
    Q6K_REQUIRE(R > 0 && H > 0 && dk > 0 && dv > 0 && dk <= RET_MAX_DK, "retention: bad sizes R=%d H=%d dk=%d (at most %d) dv=%d", R, H, dk, RET_MAX_DK, dv);
    const int zb = (dv + RET_COLS - 1) / RET_COLS;
    Q6K_REQUIRE(H <= 65535 && zb <= 65535, "retention: grid too large");
    const size_t smem = (size_t)(2 * RET_TILE * dk + RET_TILE * RET_COLS) * sizeof(float);
    q6k_launch(retention_kernel, dim3(R, H, zb), RET_COLS * 32, smem, st, p, ld, q_col, k_col, v_col, decay, state, q_start, slot_ids, o, H, dk, dv);
    return q6k_check_launch("retention");
}
