// The flexible attention of attention_flex.cu on tensor cores, for bfloat16 storage: any key width that is a multiple
// of 16 and any value width that is a multiple of 8 up to 512, values optionally a leading slice of the key rows, a
// query given as an FP32 part and a bfloat16 part, causal mask narrowed by a window and/or chunks, and the heads'
// softmax weights mixed by a matrix (see the end of this comment).
//
// A CTA of 8 warps takes 32 query rows that share their keys: the G query heads of one KV head for 32 / G consecutive
// tokens of one request.  Keys come in tiles of 64 (aligned to multiples of 64 of the key index).  For each tile every
// warp computes the scores of all 32 rows against 8 of the keys (QK^T over the key width with mma.sync m16n8k16,
// operands through ldmatrix from shared memory), the row maxima and sums are exchanged through shared memory, the
// weights go to shared memory as two bfloat16 terms (the rounded weight and what the rounding left, so that together
// they carry 16 bits of the FP32 weight), and every warp adds weights x values into its own eighth of the value width
// with one product per term (FP32 accumulators in registers: 32 rows x dv / 8 columns).  Scores, maxima, exponentials
// and sums are FP32.
//
// With few row tiles (decode steps) the keys are also split over blockIdx.z in fixed ranges of `split_keys` keys;
// each range leaves an unnormalised partial result with its maximum and sum, and a second kernel merges the ranges in
// order.  The ranges depend on the key index only, so a position's sums do not depend on the batch around it.
//
// Mixed heads: out_h = sum_g talk[h, g] * (softmax_g x V of h's KV head), so every head's weights are needed against the
// values of every KV head.  blockIdx.z then names the value head: the CTA of (row tile, key head, value head) leaves
// softmax_g x V_value-head for its G query heads as FP32, and a second kernel takes the sum over g with the FP32 mixing
// matrix.  The scores are computed once per value head; with chunks the keys a row sees are few.
#include "common.cuh"

namespace {

constexpr int ROWS = 32, KEYS = 64, WARPS = 8, PAD = 8;

struct MmaArgs {
    const float* qa; int da;
    const __nv_bfloat16* qb; int db;
    int q_head_major;
    const __nv_bfloat16* k_pages; long long k_head_stride; int k_ld;
    const __nv_bfloat16* v_pages; long long v_head_stride; int v_ld; int dv;
    const int* block_table; int max_blocks; int page_size;
    const int* req_of_token; const int* positions;
    const int* tile_tok0; const int* tile_ntok;
    int window, chunk; float scale;
    __nv_bfloat16* out; int out_head_major;
    float* part_o; float* part_ml;      // [splits][rows][dv], [splits][rows][2] when the keys are split
    int split_keys, nsplit;
    int T_, H, Hkv;
    int nbuf;                           // 2: the next key tile is fetched (cp.async) while this one is used; 1: one buffer
    int v_heads;                        // > 0 (mixed heads): blockIdx.z is the value head and part_o is [T, H, v_heads, dv]
    const float* sinks;                 // [H] or null: exp(sinks[h]) joins head h's softmax denominator (with split keys, in the merge)
    float softcap;                      // > 0: a scaled score s becomes softcap * tanh(s / softcap)
    int maps;                           // > 1: every head attends `maps` times with keys of its own over the same values (see
                                        // attention_flex.cu): q rows heads x maps, key heads groups x maps, value heads groups
    float* out_f32;                     // not null: the result leaves as FP32 here instead of through `out`
};

// exp and tanh on the hardware's exponential (ex2.approx): the scores here come from bfloat16 operands and the weights leave
// as two bfloat16 terms, so 2^-21 of relative error is far below what the operands carry.  (The FP32 path has its own kernel.)
__device__ __forceinline__ float fast_exp(float x) { return __expf(x); }
__device__ __forceinline__ float fast_tanh(float x) { return 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * x)); }

__device__ __forceinline__ int mma_query_head(int kh, int g, int G, int maps) { return maps > 1 ? ((kh / maps) * G + g) * maps + kh % maps : kh * G + g; }

__device__ __forceinline__ int first_visible_mma(int pos, int window, int chunk) {
    int lo = 0;
    if (window > 0) lo = max(lo, pos - window + 1);
    if (chunk > 0) lo = max(lo, pos / chunk * chunk);
    return lo;
}

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned& r0, unsigned& r1, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x2_trans(unsigned& r0, unsigned& r1, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16 bytes global -> shared without passing registers; !valid: zeros (nothing is read).
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// NB: value n-blocks (of 8 columns) per warp: ceil(ceil(dv / 8) / 8), 1..8.
template <int NB>
__global__ void __launch_bounds__(WARPS * 32) attention_flex_mma_kernel(const MmaArgs a) {
    pdl_enter();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int dk = a.da + a.db, G = a.H / a.Hkv;
    const int ldq = dk + PAD, ldv = a.dv + PAD;
    const bool shared_v = a.v_pages == a.k_pages && a.v_ld == a.k_ld && a.v_head_stride == a.k_head_stride;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);             // [ROWS][ldq]
    __nv_bfloat16* Kbase = Qs + ROWS * ldq;                                     // [nbuf][KEYS][ldq]
    __nv_bfloat16* Vbase = shared_v ? Kbase : Kbase + a.nbuf * KEYS * ldq;      // [nbuf][KEYS][ldv] (or the key tiles themselves)
    const int ldvs = shared_v ? ldq : ldv;
    const int k_tile = KEYS * ldq, v_tile = shared_v ? k_tile : KEYS * ldv;
    __nv_bfloat16* Ps = (shared_v ? Kbase + a.nbuf * k_tile : Vbase + a.nbuf * v_tile);   // [ROWS][KEYS + PAD]
    __nv_bfloat16* Pl = Ps + ROWS * (KEYS + PAD);                               // the same shape: what rounding the weights left
    float* wmax = reinterpret_cast<float*>(Pl + ROWS * (KEYS + PAD));           // [WARPS][ROWS]
    float* wsum = wmax + WARPS * ROWS;                                          // [WARPS][ROWS]
    int* row_pos = reinterpret_cast<int*>(wsum + WARPS * ROWS);                 // [ROWS]
    int* row_lo = row_pos + ROWS;                                               // [ROWS]
    int* key_rows = row_lo + ROWS;                                              // [2][KEYS]

    const int tile = blockIdx.x, kh = blockIdx.y, split = a.v_heads > 0 ? 0 : blockIdx.z, vh = a.v_heads > 0 ? blockIdx.z : a.maps > 1 ? kh / a.maps : kh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tok0 = a.tile_tok0[tile], ntok = a.tile_ntok[tile];
    const int* bt = a.block_table + (size_t)a.req_of_token[tok0] * a.max_blocks;
    const int tokens = ROWS / G;                                                 // tokens a tile can hold

    // rows: r = token * G + head-in-group
    if (tid < ROWS) {
        const int tk = tid / G;
        const bool valid = tk < ntok && tk < tokens;
        const int pos = valid ? a.positions[tok0 + tk] : -1;
        row_pos[tid] = pos;
        row_lo[tid] = valid ? first_visible_mma(pos, a.window, a.chunk) : 0x7fffffff;
    }
    for (int i = tid; i < ROWS * (dk / 8); i += blockDim.x) {
        const int r = i / (dk / 8), c8 = (i % (dk / 8)) * 8;
        const int tk = r / G, g = r % G;
        __align__(16) __nv_bfloat16 v[8];
        if (tk < ntok && tk < tokens) {
            const int t = tok0 + tk, h = mma_query_head(kh, g, G, a.maps);
            const size_t row = a.q_head_major ? (size_t)h * a.T_ + t : (size_t)t * a.H + h;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int d = c8 + e;
                v[e] = d < a.da ? __float2bfloat16_rn(a.qa[row * a.da + d]) : a.qb[row * a.db + (d - a.da)];
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __float2bfloat16_rn(0.0f);
        }
        *reinterpret_cast<uint4*>(Qs + r * ldq + c8) = *reinterpret_cast<const uint4*>(v);
    }
    __syncthreads();
    int pos_max = -1, lo_min = 0x7fffffff;
    for (int r = 0; r < ROWS; ++r) {
        pos_max = max(pos_max, row_pos[r]);
        lo_min = min(lo_min, row_lo[r]);
    }
    int k_begin = lo_min, k_end = pos_max + 1;                                   // keys [k_begin, k_end) matter to some row
    if (a.nsplit > 1) {
        k_begin = max(k_begin, split * a.split_keys);
        k_end = min(k_end, (split + 1) * a.split_keys);
    }
    // this thread's accumulator rows: m-block mb, rows mb*16 + lane/4 and + 8
    const int qr = lane >> 2, qc = (lane & 3) * 2;
    float m_run[2][2], l_run[2][2], o[2][NB][4];
#pragma unroll
    for (int mb = 0; mb < 2; ++mb) {
        m_run[mb][0] = m_run[mb][1] = -INFINITY;
        l_run[mb][0] = l_run[mb][1] = 0.0f;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[mb][nb][e] = 0.0f;
    }
    const int total_nb = (a.dv + 7) / 8;
    const float inv_cap = a.softcap > 0.0f ? 1.0f / a.softcap : 0.0f;
    // a thread's places in a key tile and a value tile (16-byte pieces, 256 apart): where 256 is a multiple of the pieces a
    // row has, the piece's column stays and the row moves on by 256 / pieces, and no division is left in the loop
    const int kper = dk / 8, vper = a.dv / 8;
    const bool kfast = 256 % kper == 0, vfast = 256 % vper == 0;
    const int k_kk0 = tid / kper, k_c8 = (tid % kper) * 8, k_step = 256 / kper;
    const int v_kk0 = tid / vper, v_c8 = (tid % vper) * 8, v_step = 256 / vper;
    const __nv_bfloat16* kp = a.k_pages + (size_t)kh * a.k_head_stride;
    const __nv_bfloat16* vp = a.v_pages + (size_t)vh * a.v_head_stride;

    // the page rows of a tile's keys (-1: not a key of this block), then the tile itself on its way into a buffer
    auto find_rows = [&](int j0, int buf) {
        if (tid < KEYS) {
            const int j = j0 + tid;
            int row = -1;
            if (j >= k_begin && j < k_end) {
                const int page = bt[j / a.page_size];
                row = page < 0 ? -1 : page * a.page_size + j % a.page_size;
            }
            key_rows[buf * KEYS + tid] = row;
        }
    };
    auto fetch = [&](int buf) {
        const int* rows_of = key_rows + buf * KEYS;
        __nv_bfloat16* Kd = Kbase + buf * k_tile;
        if (kfast) {
            for (int kk = k_kk0; kk < KEYS; kk += k_step) {
                const int row = rows_of[kk];
                cp_async16(Kd + kk * ldq + k_c8, kp + (size_t)(row < 0 ? 0 : row) * a.k_ld + k_c8, row >= 0);
            }
        } else {
            for (int i = tid; i < KEYS * kper; i += blockDim.x) {
                const int kk = i / kper, c8 = (i % kper) * 8, row = rows_of[kk];
                cp_async16(Kd + kk * ldq + c8, kp + (size_t)(row < 0 ? 0 : row) * a.k_ld + c8, row >= 0);
            }
        }
        if (!shared_v) {
            __nv_bfloat16* Vd = Vbase + buf * v_tile;
            if (vfast) {
                for (int kk = v_kk0; kk < KEYS; kk += v_step) {
                    const int row = rows_of[kk];
                    cp_async16(Vd + kk * ldv + v_c8, vp + (size_t)(row < 0 ? 0 : row) * a.v_ld + v_c8, row >= 0);
                }
            } else {
                for (int i = tid; i < KEYS * vper; i += blockDim.x) {
                    const int kk = i / vper, c8 = (i % vper) * 8, row = rows_of[kk];
                    cp_async16(Vd + kk * ldv + c8, vp + (size_t)(row < 0 ? 0 : row) * a.v_ld + c8, row >= 0);
                }
            }
        }
        cp_async_commit();
    };
    const int j_first = k_begin & ~(KEYS - 1);
    if (j_first < k_end) {
        find_rows(j_first, 0);
        __syncthreads();
        fetch(0);
    }
    int it = 0;
    for (int j0 = j_first; j0 < k_end; j0 += KEYS, ++it) {
        const int buf = a.nbuf == 2 ? (it & 1) : 0;
        const bool more = j0 + KEYS < k_end;
        if (a.nbuf == 2) {
            if (more) find_rows(j0 + KEYS, buf ^ 1);
            __syncthreads();                                                     // rows known; the other buffer is no longer read
            if (more) {
                fetch(buf ^ 1);
                cp_async_wait<1>();                                              // this tile has landed, the next is on its way
            } else {
                cp_async_wait<0>();
            }
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16* Ks = Kbase + buf * k_tile;
        const __nv_bfloat16* Vs = Vbase + buf * v_tile;
        const int* key_row = key_rows + buf * KEYS;
        // scores of the 32 rows against this warp's 8 keys
        float s[2][4];
#pragma unroll
        for (int mb = 0; mb < 2; ++mb)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[mb][e] = 0.0f;
        const __nv_bfloat16* kb = Ks + (warp * 8 + (lane & 7)) * ldq + ((lane >> 3) & 1) * 8;
        const __nv_bfloat16* qa0 = Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * ldq + (lane >> 4) * 8;
#pragma unroll 4
        for (int k0 = 0; k0 < dk; k0 += 16) {
            unsigned b0, b1, a0, a1, a2, a3;
            ldmatrix_x2(b0, b1, kb + k0);
            ldmatrix_x4(a0, a1, a2, a3, qa0 + k0);
            mma_bf16(s[0], a0, a1, a2, a3, b0, b1);
            ldmatrix_x4(a0, a1, a2, a3, qa0 + 16 * ldq + k0);
            mma_bf16(s[1], a0, a1, a2, a3, b0, b1);
        }
        // mask, scale, row maxima of this warp's 8 keys
        float tmax[2][2];
#pragma unroll
        for (int mb = 0; mb < 2; ++mb) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int r = mb * 16 + qr + hf * 8;
                const int pos = row_pos[r], lo = row_lo[r];
                float mx = -INFINITY;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int kk = warp * 8 + qc + e, j = j0 + kk;
                    const bool ok = j >= lo && j <= pos && key_row[kk] >= 0;
                    float v = ok ? s[mb][hf * 2 + e] * a.scale : -INFINITY;
                    if (ok && a.softcap > 0.0f) v = a.softcap * fast_tanh(v * inv_cap);
                    s[mb][hf * 2 + e] = v;
                    mx = fmaxf(mx, v);
                }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                tmax[mb][hf] = mx;
                if ((lane & 3) == 0) wmax[warp * ROWS + r] = mx;
            }
        }
        __syncthreads();
        float corr[2][2];
#pragma unroll
        for (int mb = 0; mb < 2; ++mb) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int r = mb * 16 + qr + hf * 8;
                float mx = wmax[r];
#pragma unroll
                for (int w = 1; w < WARPS; ++w) mx = fmaxf(mx, wmax[w * ROWS + r]);
                const float mn = fmaxf(m_run[mb][hf], mx);
                corr[mb][hf] = (m_run[mb][hf] == -INFINITY) ? 0.0f : fast_exp(m_run[mb][hf] - mn);
                m_run[mb][hf] = mn;
                float sum = 0.0f;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float v = s[mb][hf * 2 + e];
                    const float p = (v == -INFINITY) ? 0.0f : fast_exp(v - mn);
                    sum += p;
                    s[mb][hf * 2 + e] = p;
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                if ((lane & 3) == 0) wsum[warp * ROWS + r] = sum;
                const __nv_bfloat162 pp = __floats2bfloat162_rn(s[mb][hf * 2], s[mb][hf * 2 + 1]);
                *reinterpret_cast<__nv_bfloat162*>(Ps + r * (KEYS + PAD) + warp * 8 + qc) = pp;
                *reinterpret_cast<__nv_bfloat162*>(Pl + r * (KEYS + PAD) + warp * 8 + qc) =
                    __floats2bfloat162_rn(s[mb][hf * 2] - __low2float(pp), s[mb][hf * 2 + 1] - __high2float(pp));
            }
        }
        __syncthreads();
#pragma unroll
        for (int mb = 0; mb < 2; ++mb) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int r = mb * 16 + qr + hf * 8;
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) sum += wsum[w * ROWS + r];
                l_run[mb][hf] = l_run[mb][hf] * corr[mb][hf] + sum;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    o[mb][nb][hf * 2] *= corr[mb][hf];
                    o[mb][nb][hf * 2 + 1] *= corr[mb][hf];
                }
            }
        }
        // weights x values into this warp's value columns
        const __nv_bfloat16* pa0 = Ps + ((lane & 7) + ((lane >> 3) & 1) * 8) * (KEYS + PAD) + (lane >> 4) * 8;
#pragma unroll
        for (int k0 = 0; k0 < KEYS; k0 += 16) {
            unsigned p0[4], p1[4], r0[4], r1[4];
            ldmatrix_x4(p0[0], p0[1], p0[2], p0[3], pa0 + k0);
            ldmatrix_x4(p1[0], p1[1], p1[2], p1[3], pa0 + 16 * (KEYS + PAD) + k0);
            ldmatrix_x4(r0[0], r0[1], r0[2], r0[3], pa0 + ROWS * (KEYS + PAD) + k0);
            ldmatrix_x4(r1[0], r1[1], r1[2], r1[3], pa0 + (ROWS + 16) * (KEYS + PAD) + k0);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                const int blk = warp * NB + nb;
                if (blk < total_nb) {
                    unsigned b0, b1;
                    ldmatrix_x2_trans(b0, b1, Vs + (k0 + (lane & 15)) * ldvs + blk * 8);
                    mma_bf16(o[0][nb], p0[0], p0[1], p0[2], p0[3], b0, b1);
                    mma_bf16(o[1][nb], p1[0], p1[1], p1[2], p1[3], b0, b1);
                    mma_bf16(o[0][nb], r0[0], r0[1], r0[2], r0[3], b0, b1);
                    mma_bf16(o[1][nb], r1[0], r1[1], r1[2], r1[3], b0, b1);
                }
            }
        }
        if (a.nbuf == 1 && more) {
            __syncthreads();                                                     // the one buffer is no longer read
            find_rows(j0 + KEYS, 0);
            __syncthreads();
            fetch(0);
        }
    }
    // results
#pragma unroll
    for (int mb = 0; mb < 2; ++mb) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int r = mb * 16 + qr + hf * 8;
            const int tk = r / G, g = r % G;
            if (tk >= ntok || tk >= tokens) continue;
            const int t = tok0 + tk, h = mma_query_head(kh, g, G, a.maps);
            if (a.v_heads > 0) {
                const float inv = l_run[mb][hf] > 0.0f ? 1.0f / l_run[mb][hf] : 0.0f;
                float* dst = a.part_o + (((size_t)t * a.H + h) * a.v_heads + vh) * a.dv;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const int d = (warp * NB + nb) * 8 + qc;
                    if (d < a.dv) *reinterpret_cast<float2*>(dst + d) = make_float2(o[mb][nb][hf * 2] * inv, o[mb][nb][hf * 2 + 1] * inv);
                }
            } else if (a.nsplit > 1) {
                const size_t prow = ((size_t)split * a.T_ + t) * a.H + h;
                if (warp == 0 && (lane & 3) == 0) {
                    a.part_ml[prow * 2] = m_run[mb][hf];
                    a.part_ml[prow * 2 + 1] = l_run[mb][hf];
                }
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const int d = (warp * NB + nb) * 8 + qc;
                    if (d < a.dv) *reinterpret_cast<float2*>(a.part_o + prow * a.dv + d) = make_float2(o[mb][nb][hf * 2], o[mb][nb][hf * 2 + 1]);
                }
            } else {
                float l = l_run[mb][hf], corr = 1.0f;
                if (a.sinks) {                                                   // the sink counts once in the denominator
                    const float sk = a.sinks[h], mn = fmaxf(m_run[mb][hf], sk);
                    corr = m_run[mb][hf] == -INFINITY ? 0.0f : expf(m_run[mb][hf] - mn);
                    l = l * corr + expf(sk - mn);
                }
                const float inv = l > 0.0f ? corr / l : 0.0f;
                const size_t orow = a.out_head_major ? (size_t)h * a.T_ + t : (size_t)t * a.H + h;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const int d = (warp * NB + nb) * 8 + qc;
                    if (d < a.dv) {
                        if (a.out_f32) *reinterpret_cast<float2*>(a.out_f32 + orow * a.dv + d) = make_float2(o[mb][nb][hf * 2] * inv, o[mb][nb][hf * 2 + 1] * inv);
                        else *reinterpret_cast<__nv_bfloat162*>(a.out + orow * a.dv + d) = __floats2bfloat162_rn(o[mb][nb][hf * 2] * inv, o[mb][nb][hf * 2 + 1] * inv);
                    }
                }
            }
        }
    }
}

// Merges the key ranges of one (token, head) in order: out = sum_s e^(m_s - M) O_s / sum_s e^(m_s - M) l_s.
__global__ void __launch_bounds__(128) attention_flex_merge_kernel(const float* part_o, const float* part_ml, int nsplit, int T_, int H, int dv,
                                                                   __nv_bfloat16* out, int out_head_major, const float* sinks, float* out_f32) {
    pdl_enter();
    const int t = blockIdx.x, h = blockIdx.y;
    const size_t row = (size_t)t * H + h, stride = (size_t)T_ * H;
    float M = sinks ? sinks[h] : -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(s * stride + row) * 2]);
    float L = sinks ? expf(sinks[h] - M) : 0.0f;
    for (int s = 0; s < nsplit; ++s) {
        const float m = part_ml[(s * stride + row) * 2];
        if (m != -INFINITY) L += expf(m - M) * part_ml[(s * stride + row) * 2 + 1];
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    const size_t orow = out_head_major ? (size_t)h * T_ + t : row;
    for (int d = threadIdx.x; d < dv; d += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < nsplit; ++s) {
            const float m = part_ml[(s * stride + row) * 2];
            if (m != -INFINITY) acc = fmaf(expf(m - M), part_o[(s * stride + row) * dv + d], acc);
        }
        if (out_f32) out_f32[orow * dv + d] = acc * inv;
        else out[orow * dv + d] = __float2bfloat16_rn(acc * inv);
    }
}

// out[t, h] = sum_g talk[h, g] * part[t, g, KV head of h], FP32 sums in the order of g.
__global__ void __launch_bounds__(128) attention_talk_mix_kernel(const float* part, const float* talk, int H, int Hkv, int dv,
                                                                 __nv_bfloat16* out) {
    pdl_enter();
    const int t = blockIdx.x, h = blockIdx.y, kv = h / (H / Hkv);
    for (int d = threadIdx.x; d < dv; d += blockDim.x) {
        float acc = 0.0f;
        for (int g = 0; g < H; ++g) acc = fmaf(talk[h * H + g], part[(((size_t)t * H + g) * Hkv + kv) * dv + d], acc);
        out[((size_t)t * H + h) * dv + d] = __float2bfloat16_rn(acc);
    }
}

size_t flex_mma_smem(int dk, int dv, bool shared_v, int nbuf) {
    size_t b = (size_t)(ROWS + nbuf * KEYS) * (dk + PAD) * 2;
    if (!shared_v) b += (size_t)nbuf * KEYS * (dv + PAD) * 2;
    b += (size_t)2 * ROWS * (KEYS + PAD) * 2 + (size_t)2 * WARPS * ROWS * 4 + (size_t)(2 * ROWS + 2 * KEYS) * 4;
    return b;
}

}  // namespace

// Whether the tensor-core kernel takes these shapes (bfloat16 only): group size, key and value widths, alignment of the rows.
Q6K_API int q6k_attention_flex_mma_supported(int H, int Hkv, int dk, int dv, int k_ld, int v_ld, int db, int shared_v) {
    if (Hkv <= 0 || H % Hkv || H / Hkv > ROWS) return 0;
    if (dk % 16 || dv % 8 || dv > 512 || k_ld % 8 || v_ld % 8 || db % 8) return 0;
    return flex_mma_smem(dk, dv, shared_v != 0, 1) <= 220 * 1024;
}

// Tokens of one request a row tile holds for this group size.
Q6K_API int q6k_attention_flex_mma_tile_tokens(int H, int Hkv) { return ROWS / (H / Hkv) > 0 ? ROWS / (H / Hkv) : 1; }

// Bytes of scratch for `nsplit` key ranges: partial results and their (maximum, sum).
Q6K_API long long q6k_attention_flex_mma_workspace(int T_, int H, int dv, int nsplit) {
    return nsplit > 1 ? (long long)nsplit * T_ * H * (dv + 2) * 4 : 0;
}

// The same with mixed heads: every head's result against every KV head's values.
Q6K_API long long q6k_attention_flex_mma_talk_workspace(int T_, int H, int Hkv, int dv) { return (long long)T_ * H * Hkv * dv * 4; }

Q6K_API int q6k_attention_flex_mma(const float* qa, int da, const void* qb, int db, int q_head_major, const void* k_pages,
                                   long long k_head_stride, int k_ld, const void* v_pages, long long v_head_stride, int v_ld, int dv,
                                   const int* block_table, int max_blocks, int page_size, const int* req_of_token, const int* positions,
                                   const int* tile_tok0, const int* tile_ntok, int n_tiles, int window, int chunk, float scale, void* out,
                                   int out_head_major, int T_, int H, int Hkv, int nsplit, int split_keys, float* workspace,
                                   const float* talk, const float* sinks, float softcap, int maps, float* out_f32, cudaStream_t st) {
    if (T_ == 0 || n_tiles == 0) return 0;
    Q6K_REQUIRE(maps >= 1 && Hkv % maps == 0 && softcap >= 0.0f, "attention_flex_mma: %d maps over %d key heads, softcap %f", maps, Hkv, softcap);
    Q6K_REQUIRE(!talk || (maps == 1 && softcap == 0.0f && !out_f32), "attention_flex_mma: mixed heads take neither maps, a cap nor FP32 results");
    const int dk = da + db;
    const bool shared_v = v_pages == k_pages && v_ld == k_ld && v_head_stride == k_head_stride;
    Q6K_REQUIRE(q6k_attention_flex_mma_supported(H, Hkv, dk, dv, k_ld, v_ld, db, shared_v), "attention_flex_mma: shapes H=%d Hkv=%d dk=%d dv=%d not taken", H, Hkv, dk, dv);
    Q6K_REQUIRE((da == 0 || qa) && (db == 0 || qb) && nsplit >= 1 && (nsplit == 1 || (workspace && split_keys > 0 && split_keys % KEYS == 0)),
                "attention_flex_mma: bad query parts or key split");
    Q6K_REQUIRE(Hkv <= 65535 && nsplit <= 65535, "attention_flex_mma: grid too large");
    Q6K_REQUIRE(!talk || (nsplit == 1 && workspace && !out_head_major && !sinks), "attention_flex_mma: mixed heads take one key range, scratch, token-major output and no sinks");
    MmaArgs a{qa, da, (const __nv_bfloat16*)qb, db, q_head_major, (const __nv_bfloat16*)k_pages, k_head_stride, k_ld,
              (const __nv_bfloat16*)v_pages, v_head_stride, v_ld, dv, block_table, max_blocks, page_size, req_of_token, positions,
              tile_tok0, tile_ntok, window, chunk, scale, (__nv_bfloat16*)out, out_head_major,
              workspace, workspace ? workspace + (size_t)nsplit * T_ * H * dv : nullptr, split_keys, nsplit, T_, H, Hkv,
              flex_mma_smem(dk, dv, shared_v, 2) <= 220 * 1024 ? 2 : 1, talk ? Hkv : 0, sinks, softcap, maps, out_f32};
    const size_t smem = flex_mma_smem(dk, dv, shared_v, a.nbuf);
    const int nb = ((dv + 7) / 8 + WARPS - 1) / WARPS;
    dim3 grid(n_tiles, Hkv, talk ? Hkv : nsplit);
#define FLEX_LAUNCH(NB)                                                                                                   \
    do {                                                                                                                  \
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_flex_mma_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        q6k_launch(attention_flex_mma_kernel<NB>, grid, WARPS * 32, smem, st, a);                                         \
    } while (0)
    if (nb <= 1) FLEX_LAUNCH(1);
    else if (nb <= 2) FLEX_LAUNCH(2);
    else if (nb <= 4) FLEX_LAUNCH(4);
    else FLEX_LAUNCH(8);
#undef FLEX_LAUNCH
    if (int rc = q6k_check_launch("attention_flex_mma")) return rc;
    if (talk) {
        q6k_launch(attention_talk_mix_kernel, dim3(T_, H), 128, 0, st, (const float*)workspace, talk, H, Hkv, dv, (__nv_bfloat16*)out);
        return q6k_check_launch("attention_talk_mix");
    }
    if (nsplit > 1) {
        q6k_launch(attention_flex_merge_kernel, dim3(T_, H), 128, 0, st, (const float*)a.part_o, (const float*)a.part_ml, nsplit, T_, H, dv,
                   (__nv_bfloat16*)out, out_head_major, sinks, out_f32);
        return q6k_check_launch("attention_flex_merge");
    }
    return 0;
}
