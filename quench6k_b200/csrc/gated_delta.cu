// Two things a mixer with per-request state needs, for any mix of prompt portions and single tokens:
//
// 1. A short causal convolution over time on every channel of a projection, with the last taps - 1 projected
//    values of each request kept in its state slot:
//
//      y[t, c] = act(sum_j w[c, j] * p[t - taps + 1 + j, c]),   p = projection (+ bias), zeros before the sequence's start
//
//    short_conv_kernel computes y from the step's rows and the slot's tail, short_conv_tail_kernel then moves the
//    tail on.  The projection may come as split-K partial sums, which are added in order.
//
// 2. The gated delta rule.  Per head, with a state S [dk, dv] in FP32:
//
//      S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
//
//    with q and k made unit vectors per head first (q also times dk^-1/2), beta = sigmoid(b) and the decay
//    g = exp(-exp(A_log) softplus(a + dt_bias)), all in FP32.  The columns of S do not meet: column j of S, v, u and o
//    is a recurrence of its own given q, k, g and beta.  A block owns DELTA_COLS columns of one head of one request;
//    DELTA_LANES lanes share a column, each holding a stretch of consecutive rows; the sums over the rows are a running
//    sum per lane and a butterfly over the lanes, so their order depends on dk alone.
//    prompt cut anywhere leaves the same state as the whole prompt (up to rounding: tokens are taken a few at a time,
//    counted from the start of a portion, see gated_delta_kernel).
//    The state is kept column-major, [slots, heads, dv, dk]: a column's rows lie together.
//
//    delta_out_kernel closes the mixer: every head's o is divided by its root mean square over dv, multiplied by a
//    weight shared by the heads and by silu (or the sigmoid) of a gate projection, and leaves in the operand dtype for the
//    output product.  Called with ONE head of all heads' values it norms them together.
#include "common.cuh"

namespace {

constexpr int CONV_MAX_TAPS = 16;
constexpr int DELTA_LANES = 8;       // lanes that share a column of the state
constexpr int DELTA_COLS = 16;      // columns of the state per block
constexpr int DELTA_PER = 1;        // of them per thread (what a thread reads of k and q serves all of its columns)
constexpr int DELTA_THREADS = DELTA_COLS / DELTA_PER * DELTA_LANES;
constexpr int DELTA_TILE = 16;       // tokens whose inputs are staged in shared memory at a time

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }
// what the output gate passes through: 0 silu, 1 sigmoid
__device__ __forceinline__ float gate_f(float v, int gate) { return gate == 1 ? 1.0f / (1.0f + expf(-v)) : silu_f(v); }

// the projected value of row `row`, channel c: the slices in order, then the bias
__device__ __forceinline__ float projected(const float* x, int slices, size_t slice_stride, int ldx, const float* bias, size_t row, int c) {
    float v = x[row * ldx + c];
    for (int s = 1; s < slices; ++s) v += x[s * slice_stride + row * ldx + c];
    return bias ? v + bias[c] : v;
}

// grid (T, ceil(C / 256)).  x: FP32 [slices, T, ldx], the convolved channels in its first C columns; the columns from C
// to `copy_to` pass through (summed, no bias); tail: FP32 [slots, taps-1, C]; out: FP32 [T, ldo].
__global__ void __launch_bounds__(256) short_conv_kernel(const float* x, int slices, size_t slice_stride, int ldx, const float* bias,
                                                         const float* w, const float* tail, const int* req_of_token, const int* q_start,
                                                         const int* slot_ids, float* out, int ldo, int C, int copy_to, int taps, int act) {
    pdl_enter();
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= copy_to) return;
    if (c >= C) {
        out[(size_t)t * ldo + c] = projected(x, slices, slice_stride, ldx, nullptr, t, c);
        return;
    }
    const int r = req_of_token[t], first = q_start[r], i = t - first;
    const float* old = tail + (size_t)slot_ids[r] * (taps - 1) * C;
    float acc = 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int src = i - (taps - 1 - j);                      // index within the portion; negative: before it
        const float v = src >= 0 ? projected(x, slices, slice_stride, ldx, bias, first + src, c) : old[(size_t)(taps - 1 + src) * C + c];
        acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    out[(size_t)t * ldo + c] = act ? silu_f(acc) : acc;
}

// grid (R, ceil(C / 256)): the slot's tail becomes the last taps - 1 projected values of the request, this step's rows included.
__global__ void __launch_bounds__(256) short_conv_tail_kernel(const float* x, int slices, size_t slice_stride, int ldx, const float* bias,
                                                              float* tail, const int* q_start, const int* slot_ids, int C, int taps) {
    pdl_enter();
    const int r = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int first = q_start[r], n = q_start[r + 1] - first;
    float* mine = tail + (size_t)slot_ids[r] * (taps - 1) * C;
    float keep[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
        if (j < taps - 1) {
            const int src = n - (taps - 1) + j;                  // index within the portion; negative: what the tail held
            keep[j] = src >= 0 ? projected(x, slices, slice_stride, ldx, bias, first + src, c) : mine[(size_t)(taps - 1 + src) * C + c];
        }
    }
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
        if (j < taps - 1) mine[(size_t)j * C + c] = keep[j];
}

// What the recurrence needs of a token besides v, made once per token by delta_prepare_kernel for steps with long
// portions (the recurrence kernel makes it itself for a few tokens): the unit vectors (in place over q and k in u),
// and per token [beta (H) | decay (H)] in `bg`.  The same arithmetic in the same order as in the kernel below.
__device__ __forceinline__ void delta_unit_vectors(float* ur, int q_at, int k_at, int dk, float q_mult, int lane, float* k_out, float* q_out,
                                                   int seg, int pad) {
    float kk = 0.0f, qq = 0.0f;
    for (int i = lane; i < dk; i += 32) {
        const float kv = ur[k_at + i], qv = ur[q_at + i];
        kk = fmaf(kv, kv, kk), qq = fmaf(qv, qv, qq);
    }
    kk = warp_sum(kk), qq = warp_sum(qq);
    const float k_inv = rsqrtf(kk + 1e-6f), q_inv = rsqrtf(qq + 1e-6f) * q_mult;
    for (int i = lane; i < dk; i += 32) {
        const float kv = ur[k_at + i] * k_inv, qv = ur[q_at + i] * q_inv;
        const int at = seg ? (i / seg) * (seg + pad) + i % seg : i;        // seg: rows per lane of the recurrence's shared layout
        k_out[at] = kv, q_out[at] = qv;
    }
}

// grid (T), 128 threads.
__global__ void __launch_bounds__(128) delta_prepare_kernel(float* u, int ldu, const float* p, int ldp, int b_col, int a_col, const float* A_log,
                                                            const float* dt_bias, float* bg, int H, int G, int dk) {
    pdl_enter();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* ur = u + (size_t)t * ldu;
    float* out = bg + (size_t)t * 2 * H;
    const float q_mult = rsqrtf((float)dk);
    for (int g = warp; g < G; g += 4) delta_unit_vectors(ur, g * dk, G * dk + g * dk, dk, q_mult, lane, ur + G * dk + g * dk, ur + g * dk, 0, 0);
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float* pr = p + (size_t)t * ldp;
        out[h] = 1.0f / (1.0f + expf(-pr[b_col + h]));
        out[H + h] = expf(-expf(A_log[h]) * softplus_f(pr[a_col + h] + dt_bias[h]));
    }
}

// grid (heads * ceil(dv / DELTA_COLS), R), DELTA_THREADS threads.  RPL: rows of the state per lane, a multiple of 4
// (dk <= RPL * DELTA_LANES); lane l of a column holds rows l RPL .. l RPL + RPL - 1, and in shared memory a lane's stretch
// of k and q is RPL + 4 floats long, so that the 16-byte reads of a quarter warp's lanes fall into different banks.
//
// Tokens are taken DELTA_CHUNK at a time, counted from the start of the request's portion.  With S the state before the
// chunk, P_i the product of the decays up to token i, and w_m = u_m times the decays after token m up to the one at hand,
//   S_(i-1)^T k_i = P_(i-1) (S^T k_i) + sum_(m<i) w_m (k_m . k_i),      likewise with q_i,
// so one pass over S gives the sums with every k_i and q_i of the chunk (one butterfly over the lanes for all of them),
// a few scalar steps per column give u_i and o_i in order, and one more pass writes S <- P S + sum_m w_m k_m.  The
// products k_m . k_i and k_m . q_i of a chunk do not depend on the column; a warp makes them when the tile is staged.
// Against the walk token by token this only regroups sums: results differ by rounding, also between two ways to cut a prompt.
//
// u: FP32 [T, ldu] with q at column 0 (G heads of dk), k after it, v after that (H heads of dv); p: FP32 [T, ldp] with
// the H beta logits at b_col and the H decay inputs at a_col.  PREPARED: q and k in u are unit vectors already and bg
// holds [beta | decay] per token (delta_prepare_kernel); the next tile's inputs are then fetched into registers while
// this tile is walked.
constexpr int DELTA_CHUNK = 4;

template <int RPL, bool PREPARED>
__global__ void __launch_bounds__(DELTA_THREADS) gated_delta_kernel(const float* u, int ldu, const float* p, int ldp, int b_col, int a_col,
                                                                              const float* A_log, const float* dt_bias, const float* bg,
                                                                              float* state, const int* q_start, const int* slot_ids, float* o,
                                                                              int H, int G, int dk, int dv) {
    pdl_enter();
    constexpr int SEG = RPL + 4, KS = DELTA_LANES * SEG, NT = DELTA_THREADS, CH = DELTA_CHUNK, PER = DELTA_PER, CT = DELTA_COLS / DELTA_PER;
    constexpr int PRE = PREPARED ? DELTA_TILE * DELTA_LANES * RPL / NT : 1;      // k (and q) entries of a tile per thread
    static_assert(DELTA_TILE % CH == 0 && NT % 32 == 0 && 2 * DELTA_TILE <= NT, "whole chunks, whole warps, a thread per staged scalar");
    extern __shared__ __align__(16) float sm[];
    float* s_k = sm;                                  // [TILE][KS] unit keys
    float* s_q = s_k + DELTA_TILE * KS;               // [TILE][KS] unit queries times dk^-1/2
    float* s_v = s_q + DELTA_TILE * KS;               // [TILE][COLS]
    float* s_beta = s_v + DELTA_TILE * DELTA_COLS;    // [TILE]
    float* s_g = s_beta + DELTA_TILE;                 // [TILE]
    float* s_kk = s_g + DELTA_TILE;                   // [TILE][CH]: k_m . k_i for token m and place i of its chunk (m's place < i)
    float* s_kq = s_kk + DELTA_TILE * CH;             // [TILE][CH]: k_m . q_i (m's place <= i)
    const int col_blocks = (dv + DELTA_COLS - 1) / DELTA_COLS;
    const int head = blockIdx.x / col_blocks, col0 = (blockIdx.x % col_blocks) * DELTA_COLS, r = blockIdx.y;
    const int kvh = head / (H / G);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int sub = threadIdx.x % DELTA_LANES, cl = threadIdx.x / DELTA_LANES;       // the thread's columns: col0 + cl + CT j
    const int first = q_start[r], n = q_start[r + 1] - first;
    const int q_at = kvh * dk, k_at = G * dk + kvh * dk, v_at = 2 * G * dk + head * dv;
    const float decay_rate = PREPARED ? 0.0f : -expf(A_log[head]), bias = PREPARED ? 0.0f : dt_bias[head], q_mult = rsqrtf((float)dk);
    float* mine = state + ((size_t)slot_ids[r] * H + head) * dv * dk;
    float S[PER][RPL];
    const bool by4 = dk % 4 == 0;                     // a column's rows start on 16 bytes: the state moves 16 bytes at a time
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int col = col0 + cl + CT * j;
        if (by4) {
#pragma unroll
            for (int i = 0; i < RPL; i += 4) {
                const int row = sub * RPL + i;
                const float4 v = col < dv && row < dk ? *reinterpret_cast<const float4*>(mine + (size_t)col * dk + row) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                S[j][i] = v.x, S[j][i + 1] = v.y, S[j][i + 2] = v.z, S[j][i + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                const int row = sub * RPL + i;
                S[j][i] = col < dv && row < dk ? mine[(size_t)col * dk + row] : 0.0f;
            }
        }
    }
    // the padding of the stretches, the rows beyond dk and the tokens beyond a portion read as zero (the products within a
    // chunk are summed over whole stretches)
    for (int i = threadIdx.x; i < 2 * DELTA_TILE * KS; i += NT) sm[i] = 0.0f;
    float pre_k[PRE], pre_q[PRE], pre_v[DELTA_TILE * DELTA_COLS / NT], pre_s = 0.0f;
    auto fetch = [&](int t0) {                        // PREPARED: a tile's inputs into registers
        const int nt = min(DELTA_TILE, n - t0);
#pragma unroll
        for (int j = 0; j < PRE; ++j) {
            const int idx = threadIdx.x + j * NT, t = idx / (DELTA_LANES * RPL), row = idx % (DELTA_LANES * RPL);
            const bool ok = t < nt && row < dk;
            const float* ur = u + (size_t)(first + t0 + t) * ldu;
            pre_k[j] = ok ? ur[k_at + row] : 0.0f;
            pre_q[j] = ok ? ur[q_at + row] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < DELTA_TILE * DELTA_COLS / NT; ++j) {
            const int idx = threadIdx.x + j * NT, t = idx / DELTA_COLS, c = col0 + idx % DELTA_COLS;
            pre_v[j] = t < nt && c < dv ? u[(size_t)(first + t0 + t) * ldu + v_at + c] : 0.0f;
        }
        if (threadIdx.x < 2 * DELTA_TILE) {
            const int what = threadIdx.x / DELTA_TILE, t = threadIdx.x % DELTA_TILE;
            pre_s = t < nt ? bg[(size_t)(first + t0 + t) * 2 * H + what * H + head] : 0.0f;
        }
    };
    if (PREPARED && n > 0) fetch(0);
    for (int t0 = 0; t0 < n; t0 += DELTA_TILE) {
        const int nt = min(DELTA_TILE, n - t0);
        __syncthreads();
        if (PREPARED) {
#pragma unroll
            for (int j = 0; j < PRE; ++j) {
                const int idx = threadIdx.x + j * NT, t = idx / (DELTA_LANES * RPL), row = idx % (DELTA_LANES * RPL);
                const int at = t * KS + (row / RPL) * SEG + row % RPL;
                s_k[at] = pre_k[j], s_q[at] = pre_q[j];
            }
#pragma unroll
            for (int j = 0; j < DELTA_TILE * DELTA_COLS / NT; ++j) s_v[threadIdx.x + j * NT] = pre_v[j];
            if (threadIdx.x < 2 * DELTA_TILE) s_beta[threadIdx.x] = pre_s;       // s_beta and s_g lie one after the other
            __syncthreads();
            if (t0 + DELTA_TILE < n) fetch(t0 + DELTA_TILE);                   // in flight while this tile is walked
        } else {
            // the tile's inputs: a warp per token makes the unit vectors, beta and the decay
            for (int t = warp; t < nt; t += nwarps) {
                delta_unit_vectors(const_cast<float*>(u) + (size_t)(first + t0 + t) * ldu, q_at, k_at, dk, q_mult, lane, s_k + t * KS, s_q + t * KS,
                                   RPL, 4);
                if (lane == 0) {
                    const float* pr = p + (size_t)(first + t0 + t) * ldp;
                    s_beta[t] = 1.0f / (1.0f + expf(-pr[b_col + head]));
                    s_g[t] = expf(decay_rate * softplus_f(pr[a_col + head] + bias));
                }
            }
            for (int i = threadIdx.x; i < nt * DELTA_COLS; i += NT) {
                const int t = i / DELTA_COLS, c = col0 + i % DELTA_COLS;
                s_v[i] = c < dv ? u[(size_t)(first + t0 + t) * ldu + v_at + c] : 0.0f;
            }
            __syncthreads();
        }
        // the products within each chunk, a warp per chunk (sums over the padded stretches, whose padding is zero)
        for (int cw = warp; cw * CH < nt; cw += nwarps) {
            float kk[CH][CH], kq[CH][CH];
#pragma unroll
            for (int m = 0; m < CH; ++m)
#pragma unroll
                for (int i = 0; i < CH; ++i) kk[m][i] = 0.0f, kq[m][i] = 0.0f;
            const float* kb = s_k + cw * CH * KS;
            const float* qb = s_q + cw * CH * KS;
            for (int x = lane; x < KS; x += 32) {
                float kx[CH], qx[CH];
#pragma unroll
                for (int m = 0; m < CH; ++m) kx[m] = kb[m * KS + x], qx[m] = qb[m * KS + x];
#pragma unroll
                for (int m = 0; m < CH; ++m)
#pragma unroll
                    for (int i = m; i < CH; ++i) {
                        kq[m][i] = fmaf(kx[m], qx[i], kq[m][i]);
                        if (i > m) kk[m][i] = fmaf(kx[m], kx[i], kk[m][i]);
                    }
            }
#pragma unroll
            for (int m = 0; m < CH; ++m)
#pragma unroll
                for (int i = m; i < CH; ++i) {
                    const float a = warp_sum(kq[m][i]);
                    const float b = i > m ? warp_sum(kk[m][i]) : 0.0f;
                    if (lane == 0) s_kq[(cw * CH + m) * CH + i] = a, s_kk[(cw * CH + m) * CH + i] = b;
                }
        }
        __syncthreads();
        for (int c0 = 0; c0 < nt; c0 += CH) {
            const int cnt = min(CH, nt - c0);
            float kreg[CH][RPL], sk[PER][CH], sq[PER][CH];
#pragma unroll
            for (int j = 0; j < PER; ++j)
#pragma unroll
                for (int c = 0; c < CH; ++c) sk[j][c] = 0.0f, sq[j][c] = 0.0f;
#pragma unroll
            for (int i = 0; i < RPL / 4; ++i) {
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    const float4 k4 = reinterpret_cast<const float4*>(s_k + (c0 + c) * KS + sub * SEG)[i];
                    const float4 q4 = reinterpret_cast<const float4*>(s_q + (c0 + c) * KS + sub * SEG)[i];
                    kreg[c][4 * i] = k4.x, kreg[c][4 * i + 1] = k4.y, kreg[c][4 * i + 2] = k4.z, kreg[c][4 * i + 3] = k4.w;
#pragma unroll
                    for (int j = 0; j < PER; ++j) {
                        sk[j][c] = fmaf(S[j][4 * i], k4.x, sk[j][c]), sk[j][c] = fmaf(S[j][4 * i + 1], k4.y, sk[j][c]);
                        sk[j][c] = fmaf(S[j][4 * i + 2], k4.z, sk[j][c]), sk[j][c] = fmaf(S[j][4 * i + 3], k4.w, sk[j][c]);
                        sq[j][c] = fmaf(S[j][4 * i], q4.x, sq[j][c]), sq[j][c] = fmaf(S[j][4 * i + 1], q4.y, sq[j][c]);
                        sq[j][c] = fmaf(S[j][4 * i + 2], q4.z, sq[j][c]), sq[j][c] = fmaf(S[j][4 * i + 3], q4.w, sq[j][c]);
                    }
                }
            }
#pragma unroll
            for (int off = DELTA_LANES / 2; off > 0; off >>= 1) {
#pragma unroll
                for (int j = 0; j < PER; ++j)
#pragma unroll
                    for (int c = 0; c < CH; ++c) {
                        sk[j][c] += __shfl_xor_sync(0xffffffffu, sk[j][c], off);
                        sq[j][c] += __shfl_xor_sync(0xffffffffu, sq[j][c], off);
                    }
            }
            float P = 1.0f, w[PER][CH];
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                const bool live = i < cnt;
                const float g = live ? s_g[c0 + i] : 1.0f;
#pragma unroll
                for (int j = 0; j < PER; ++j) {
                    const int col = col0 + cl + CT * j;
                    float a = P * sk[j][i], b = P * sq[j][i];
#pragma unroll
                    for (int m = 0; m < i; ++m) {
                        a = fmaf(w[j][m], s_kk[(c0 + m) * CH + i], a);
                        b = fmaf(w[j][m], s_kq[(c0 + m) * CH + i], b);
                    }
                    const float uu = live ? s_beta[c0 + i] * (s_v[(c0 + i) * DELTA_COLS + cl + CT * j] - g * a) : 0.0f;
                    if (live && sub == 0 && col < dv) o[(size_t)(first + t0 + c0 + i) * H * dv + head * dv + col] = fmaf(s_kq[(c0 + i) * CH + i], uu, g * b);
#pragma unroll
                    for (int m = 0; m < i; ++m) w[j][m] *= g;
                    w[j][i] = uu;
                }
                P *= g;
            }
#pragma unroll
            for (int j = 0; j < PER; ++j)
#pragma unroll
                for (int i = 0; i < RPL; ++i) {
                    float acc = P * S[j][i];
#pragma unroll
                    for (int c = 0; c < CH; ++c) acc = fmaf(w[j][c], kreg[c][i], acc);
                    S[j][i] = acc;
                }
        }
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int col = col0 + cl + CT * j;
        if (col < dv && by4) {
#pragma unroll
            for (int i = 0; i < RPL; i += 4) {
                const int row = sub * RPL + i;
                if (row < dk) *reinterpret_cast<float4*>(mine + (size_t)col * dk + row) = make_float4(S[j][i], S[j][i + 1], S[j][i + 2], S[j][i + 3]);
            }
        } else if (col < dv) {
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                const int row = sub * RPL + i;
                if (row < dk) mine[(size_t)col * dk + row] = S[j][i];
            }
        }
    }
}

// grid (T, ceil(H / 4)), a warp per (token, head): out = T(o / rms(o) * w * silu(gate)).  Heads up to 256 wide keep their
// values and gates in registers, all loads asked for before the sum; wider ones read the row twice.
template <typename T>
__global__ void __launch_bounds__(128) delta_out_kernel(const float* o, const float* p, int ldp, int g_col, const float* w, float eps, T* out,
                                                        int H, int dv, int gate) {
    pdl_enter();
    const int t = blockIdx.x, head = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (head >= H) return;
    const float* orow = o + ((size_t)t * H + head) * dv;
    const float* grow = p + (size_t)t * ldp + g_col + head * dv;
    T* dst = out + ((size_t)t * H + head) * dv;
    if (dv <= 256) {
        float v[8], g[8], ww[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = lane + 32 * j;
            v[j] = i < dv ? orow[i] : 0.0f, g[j] = i < dv ? grow[i] : 0.0f, ww[j] = i < dv ? w[i] : 0.0f;
        }
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)dv + eps);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = lane + 32 * j;
            if (i < dv) dst[i] = from_f32<T>(v[j] * inv * ww[j] * gate_f(g[j], gate));
        }
        return;
    }
    float ss = 0.0f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(orow[i], orow[i], ss);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)dv + eps);
    for (int i = lane; i < dv; i += 32) dst[i] = from_f32<T>(orow[i] * inv * w[i] * gate_f(grow[i], gate));
}

// The same for ONE wide head (all heads' values normed together): a block per token, the row's values kept in registers
// between the sum of squares and the products (up to 16 a thread), read again beyond that.
template <typename T>
__global__ void __launch_bounds__(256) delta_out_row_kernel(const float* o, const float* p, int ldp, int g_col, const float* w, float eps, T* out,
                                                            int N, int gate) {
    pdl_enter();
    __shared__ float red[32];
    const int t = blockIdx.x;
    const float* orow = o + (size_t)t * N;
    const float* grow = p + (size_t)t * ldp + g_col;
    T* dst = out + (size_t)t * N;
    constexpr int PER = 16;
    float v[PER];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int i = threadIdx.x + 256 * j;
        v[j] = i < N ? orow[i] : 0.0f;
        ss = fmaf(v[j], v[j], ss);
    }
    for (int i = threadIdx.x + 256 * PER; i < N; i += 256) ss = fmaf(orow[i], orow[i], ss);
    const float inv = rsqrtf(block_sum(ss, red) / (float)N + eps);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int i = threadIdx.x + 256 * j;
        if (i < N) dst[i] = from_f32<T>(v[j] * inv * w[i] * gate_f(grow[i], gate));
    }
    for (int i = threadIdx.x + 256 * PER; i < N; i += 256) dst[i] = from_f32<T>(orow[i] * inv * w[i] * gate_f(grow[i], gate));
}

}  // namespace

// out[t, c] = act(short convolution of the projected channel c up to row t) for c < C; columns C..copy_to of x are
// copied (their slices summed).  act: 0 none, 1 silu.  Then call q6k_short_conv_tail with the same x.
Q6K_API int q6k_short_conv(const float* x, int slices, long long slice_stride, int ldx, const float* bias, const float* w, const float* tail,
                           const int* req_of_token, const int* q_start, const int* slot_ids, float* out, int ldo, int T_, int C, int copy_to,
                           int taps, int act, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && C > 0 && copy_to >= C && taps >= 1 && taps <= CONV_MAX_TAPS && slices >= 1,
                "short_conv: bad sizes T=%d C=%d taps=%d (at most %d taps) slices=%d", T_, C, taps, CONV_MAX_TAPS, slices);
    Q6K_REQUIRE(ldx >= copy_to && ldo >= copy_to && (act == 0 || act == 1), "short_conv: rows of %d and %d for %d columns, act %d", ldx, ldo, copy_to, act);
    dim3 grid(T_, (copy_to + 255) / 256);
    Q6K_REQUIRE(grid.y <= 65535, "short_conv: %d channels exceed the grid limit", copy_to);
    q6k_launch(short_conv_kernel, grid, 256, 0, st, x, slices, (size_t)slice_stride, ldx, bias, w, tail, req_of_token, q_start, slot_ids, out,
               ldo, C, copy_to, taps, act);
    return q6k_check_launch("short_conv");
}

Q6K_API int q6k_short_conv_tail(const float* x, int slices, long long slice_stride, int ldx, const float* bias, float* tail, const int* q_start,
                                const int* slot_ids, int R, int C, int taps, cudaStream_t st) {
    if (R == 0 || taps <= 1) return 0;
    Q6K_REQUIRE(R > 0 && C > 0 && taps <= CONV_MAX_TAPS && slices >= 1, "short_conv_tail: bad sizes R=%d C=%d taps=%d", R, C, taps);
    q6k_launch(short_conv_tail_kernel, dim3(R, (C + 255) / 256), 256, 0, st, x, slices, (size_t)slice_stride, ldx, bias, tail, q_start, slot_ids,
               C, taps);
    return q6k_check_launch("short_conv_tail");
}

Q6K_API int q6k_gated_delta_max_dim() { return 32 * DELTA_LANES; }

// state: FP32 [slots, H, dv, dk]; o: FP32 [T, H * dv].  bg: null, or FP32 scratch [T, 2 H]: the per-token values are then made
// by a kernel of their own first, which also turns q and k in u into unit vectors (for steps with long portions).
Q6K_API int q6k_gated_delta(float* u, int ldu, const float* p, int ldp, int b_col, int a_col, const float* A_log, const float* dt_bias,
                            float* bg, float* state, const int* q_start, const int* slot_ids, float* o, int T_, int R, int H, int G, int dk,
                            int dv, cudaStream_t st) {
    if (R == 0 || T_ == 0) return 0;
    Q6K_REQUIRE(R > 0 && T_ > 0 && H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0, "gated_delta: bad sizes R=%d H=%d G=%d dk=%d dv=%d", R, H, G, dk, dv);
    Q6K_REQUIRE(dk <= 32 * DELTA_LANES, "gated_delta: keys of %d entries exceed the supported %d", dk, 32 * DELTA_LANES);
    Q6K_REQUIRE(R <= 65535, "gated_delta: %d requests exceed the grid limit", R);
    if (bg) {
        q6k_launch(delta_prepare_kernel, T_, 128, 0, st, u, ldu, p, ldp, b_col, a_col, A_log, dt_bias, bg, H, G, dk);
        if (int rc = q6k_check_launch("delta_prepare")) return rc;
    }
    const dim3 grid(H * ((dv + DELTA_COLS - 1) / DELTA_COLS), R);
    const int rpl = ((dk + DELTA_LANES - 1) / DELTA_LANES + 3) / 4 * 4;
    const int RPL_ = rpl <= 4 ? 4 : rpl <= 8 ? 8 : rpl <= 16 ? 16 : 32;
    const size_t smem = (size_t)(2 * DELTA_TILE * DELTA_LANES * (RPL_ + 4) + DELTA_TILE * DELTA_COLS + 2 * DELTA_TILE + 2 * DELTA_TILE * DELTA_CHUNK) * sizeof(float);
#define Q6K_DELTA_GO(R_, P_) q6k_launch(gated_delta_kernel<R_, P_>, grid, DELTA_THREADS, smem, st, u, ldu, p, ldp, b_col, a_col, A_log, dt_bias, bg, state, q_start, slot_ids, o, H, G, dk, dv)
    if (bg) {
        if (RPL_ == 4) Q6K_DELTA_GO(4, true);
        else if (RPL_ == 8) Q6K_DELTA_GO(8, true);
        else if (RPL_ == 16) Q6K_DELTA_GO(16, true);
        else Q6K_DELTA_GO(32, true);
    } else {
        if (RPL_ == 4) Q6K_DELTA_GO(4, false);
        else if (RPL_ == 8) Q6K_DELTA_GO(8, false);
        else if (RPL_ == 16) Q6K_DELTA_GO(16, false);
        else Q6K_DELTA_GO(32, false);
    }
#undef Q6K_DELTA_GO
    return q6k_check_launch("gated_delta");
}

Q6K_API int q6k_delta_out(const float* o, const float* p, int ldp, int g_col, const float* w, float eps, void* out, int T_, int H, int dv, int dtype,
                          int gate, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && H > 0 && dv > 0 && (gate == 0 || gate == 1), "delta_out: bad sizes T=%d H=%d dv=%d gate=%d", T_, H, dv, gate);
    Q6K_REQUIRE((H + 3) / 4 <= 65535, "delta_out: %d heads exceed the grid limit", H);
    if (H == 1 && dv > 256) {                 // one wide head: a block per token
        Q6K_DISPATCH(dtype, q6k_launch(delta_out_row_kernel<T>, dim3(T_), 256, 0, st, o, p, ldp, g_col, w, eps, (T*)out, dv, gate););
        return q6k_check_launch("delta_out");
    }
    Q6K_DISPATCH(dtype, q6k_launch(delta_out_kernel<T>, dim3(T_, (H + 3) / 4), 128, 0, st, o, p, ldp, g_col, w, eps, (T*)out, H, dv, gate););
    return q6k_check_launch("delta_out");
}
