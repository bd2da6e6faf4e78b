// Attention over the paged cache with the shapes and masks the fixed-shape kernels do not take:
// keys and values of different widths (any width), values that are a leading slice of the key rows
// (a cached latent shared by all heads), a query given as an FP32 part followed by a part in the
// storage type, a causal mask narrowed by a sliding window and/or by chunks of positions, and,
// optionally, the heads' softmax weights mixed by a matrix before they meet the values.
// FP32 arithmetic on FP32 or bfloat16 storage: the kernels of the true 32-bit path for these
// shapes, and of the bfloat16 path where no tensor-core kernel covers the shape.
//
// Also here: the kernels that prepare q, k and v for them.
//
// Keys are walked in tiles of 32 aligned to multiples of 32 of the key index, so the order of
// every sum for a (position, head) depends neither on how the tokens were cut into steps nor on
// what else is in the batch.  Scores, softmax weights and their sums are FP32.
#include "common.cuh"

namespace {

constexpr int MAX_DV = 512, DPL = MAX_DV / 32;

// First visible key of position pos: causal, then the window (last `window` keys), then the chunk (keys of pos's own
// block of `chunk` positions, blocks counted from position 0).
__device__ __forceinline__ int first_visible(int pos, int window, int chunk) {
    int lo = 0;
    if (window > 0) lo = max(lo, pos - window + 1);
    if (chunk > 0) lo = max(lo, pos / chunk * chunk);
    return lo;
}

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int n = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int n = 8; };

// q (FP32, shared memory) . row (storage type, global), dk elements; vec: the row starts on 16 bytes and dk is a multiple of the vector.
template <typename T>
__device__ __forceinline__ float dot_row(const float* q, const T* row, int dk, bool vec) {
    float acc = 0.0f;
    if (vec) {
        constexpr int V = Vec<T>::n;
        for (int d = 0; d < dk; d += V) {
            const uint4 raw = *reinterpret_cast<const uint4*>(row + d);
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int i = 0; i < V; ++i) acc = fmaf(q[d + i], to_f32(e[i]), acc);
        }
    } else {
        for (int d = 0; d < dk; ++d) acc = fmaf(q[d], to_f32(row[d]), acc);
    }
    return acc;
}

struct FlexArgs {
    const float* qa; int da;            // FP32 leading part of a query row (or null)
    const void* qb; int db;             // the rest, in the storage type (or null)
    int q_head_major;                   // row of (t, h): h * T + t, else t * H + h
    const void* k_pages; long long k_head_stride; int k_ld;
    const void* v_pages; long long v_head_stride; int v_ld; int dv;
    const int* block_table; int max_blocks; int page_size;
    const int* req_of_token; const int* positions;
    int window, chunk; float scale;
    const float* talk;                  // [H, H] or null
    void* out; int out_head_major;
    int T_, H, Hkv;
    const float* sinks;                 // [H] or null: exp(sinks[h]) joins head h's softmax denominator (no key, no value, not scaled)
    float softcap;                      // > 0: a scaled score s becomes softcap * tanh(s / softcap)
    int maps;                           // > 1: every head attends `maps` times with keys of its own over the same values: q holds
                                        // heads x maps rows per token (a head's maps side by side), the key pages Hkv = groups x maps
                                        // heads (a group's maps side by side), the value pages one head per group
    float* out_f32;                     // not null: the result leaves as FP32 here instead of through `out`
};

// The query row (of H per token) that key head kh serves as the g-th of its G, and the value head that goes with kh.
__device__ __forceinline__ int flex_query_head(int kh, int g, int G, int maps) { return maps > 1 ? ((kh / maps) * G + g) * maps + kh % maps : kh * G + g; }

template <typename T>
__device__ __forceinline__ void load_query(const FlexArgs& a, int t, int h, float* q) {
    const size_t row = a.q_head_major ? (size_t)h * a.T_ + t : (size_t)t * a.H + h;
    const int lane = threadIdx.x & 31;
    for (int d = lane; d < a.da; d += 32) q[d] = a.qa[row * a.da + d];
    const T* qb = (const T*)a.qb;
    for (int d = lane; d < a.db; d += 32) q[a.da + d] = to_f32(qb[row * a.db + d]);
}

// A block takes one (token, KV head); its warps take the G query heads of the group in turn.
template <typename T>
__global__ void __launch_bounds__(128) attention_flex_kernel(const FlexArgs a) {
    pdl_enter();
    extern __shared__ float qs[];             // [warps][dk]
    const int t = blockIdx.x, kh = blockIdx.y, G = a.H / a.Hkv, dk = a.da + a.db;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int pos = a.positions[t];
    const int* bt = a.block_table + (size_t)a.req_of_token[t] * a.max_blocks;
    const int lo = first_visible(pos, a.window, a.chunk);
    float* qw = qs + warp * dk;
    const T* kp = (const T*)a.k_pages + (size_t)kh * a.k_head_stride;
    const T* vp = (const T*)a.v_pages + (size_t)(a.maps > 1 ? kh / a.maps : kh) * a.v_head_stride;
    const bool vec = dk % Vec<T>::n == 0 && ((size_t)a.k_ld * sizeof(T)) % 16 == 0 && ((size_t)kp % 16) == 0;
    T* out = (T*)a.out;

    for (int g = warp; g < G; g += nwarps) {
        const int h = flex_query_head(kh, g, G, a.maps);
        load_query<T>(a, t, h, qw);
        __syncwarp();
        float m = -INFINITY, l = 0.0f, o[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[i] = 0.0f;
        for (int j0 = lo & ~31; j0 <= pos; j0 += 32) {
            const int j = j0 + lane;
            const bool ok = j >= lo && j <= pos;
            float s = -INFINITY;
            int rowi = 0;
            if (ok) {
                rowi = bt[j / a.page_size] * a.page_size + j % a.page_size;
                s = dot_row<T>(qw, kp + (size_t)rowi * a.k_ld, dk, vec) * a.scale;
                if (a.softcap > 0.0f) s = a.softcap * tanhf(s / a.softcap);
            }
            const float mn = fmaxf(m, warp_max(s));     // finite: the tile holds at least one visible key
            const float corr = m == -INFINITY ? 0.0f : expf(m - mn);
            const float p = ok ? expf(s - mn) : 0.0f;
            l = l * corr + warp_sum(p);
#pragma unroll
            for (int i = 0; i < DPL; ++i) o[i] *= corr;
            const int nk = min(32, pos - j0 + 1);
            for (int jj = max(0, lo - j0); jj < nk; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                const int rj = __shfl_sync(0xffffffffu, rowi, jj);
                if (pj == 0.0f) continue;               // uniform across the warp
                const T* vr = vp + (size_t)rj * a.v_ld;
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const int d = lane + 32 * i;
                    if (d < a.dv) o[i] = fmaf(pj, to_f32(vr[d]), o[i]);
                }
            }
            m = mn;
        }
        if (a.sinks) {                                  // the sink counts once in the denominator
            const float sk = a.sinks[h], mn = fmaxf(m, sk), corr = expf(m - mn);
            l = l * corr + expf(sk - mn);
#pragma unroll
            for (int i = 0; i < DPL; ++i) o[i] *= corr;
        }
        const float inv = 1.0f / l;
        const size_t orow = a.out_head_major ? (size_t)h * a.T_ + t : (size_t)t * a.H + h;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            if (d < a.dv) {
                if (a.out_f32) a.out_f32[orow * a.dv + d] = o[i] * inv;
                else out[orow * a.dv + d] = from_f32<T>(o[i] * inv);
            }
        }
        __syncwarp();
    }
}

// The heads' weights mixed before the values: w'_h(j) = sum_g talk[h, g] * softmax_g(j); head h applies w'_h to the values
// of its own KV head.  A block takes one token and all heads.  First every head's maximum and denominator over the
// visible keys, then, tile by tile, the normalised weights of all heads into shared memory, their mixture, and the
// weighted sum of the values.
template <typename T>
__global__ void __launch_bounds__(256) attention_talk_kernel(const FlexArgs a) {
    pdl_enter();
    extern __shared__ float sm[];             // q [H][dk] | max [H] | 1/den [H] | weights [H][32] | talk [H][H]
    const int t = blockIdx.x, H = a.H, G = H / a.Hkv, dk = a.da + a.db;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float* q = sm;
    float* mx = q + (size_t)H * dk;
    float* rden = mx + H;
    float* pw = rden + H;
    float* tk = pw + H * 32;
    const int pos = a.positions[t];
    const int* bt = a.block_table + (size_t)a.req_of_token[t] * a.max_blocks;
    const int lo = first_visible(pos, a.window, a.chunk);
    const bool vec = dk % Vec<T>::n == 0 && ((size_t)a.k_ld * sizeof(T)) % 16 == 0 && ((size_t)a.k_pages % 16) == 0 &&
                     ((size_t)a.k_head_stride * sizeof(T)) % 16 == 0;
    T* out = (T*)a.out;
    for (int i = threadIdx.x; i < H * H; i += blockDim.x) tk[i] = a.talk[i];
    for (int g = warp; g < H; g += nwarps) {
        load_query<T>(a, t, g, q + (size_t)g * dk);
        __syncwarp();
        const T* kp = (const T*)a.k_pages + (size_t)(g / G) * a.k_head_stride;
        float m = -INFINITY, l = 0.0f;
        for (int j0 = lo & ~31; j0 <= pos; j0 += 32) {
            const int j = j0 + lane;
            const bool ok = j >= lo && j <= pos;
            float s = -INFINITY;
            if (ok) {
                const int rowi = bt[j / a.page_size] * a.page_size + j % a.page_size;
                s = dot_row<T>(q + (size_t)g * dk, kp + (size_t)rowi * a.k_ld, dk, vec) * a.scale;
            }
            const float mn = fmaxf(m, warp_max(s));
            const float corr = m == -INFINITY ? 0.0f : expf(m - mn);
            l = l * corr + warp_sum(ok ? expf(s - mn) : 0.0f);
            m = mn;
        }
        if (lane == 0) {
            mx[g] = m;
            rden[g] = 1.0f / l;
        }
    }
    __syncthreads();
    // each warp keeps the running sums of the heads it owns: heads warp, warp + nwarps, ... (at most MAX_OWN of them)
    constexpr int MAX_OWN = 8, DPLT = 8;       // at most 64 heads, value widths up to 256 here
    float o[MAX_OWN][DPLT];
#pragma unroll
    for (int u = 0; u < MAX_OWN; ++u)
#pragma unroll
        for (int i = 0; i < DPLT; ++i) o[u][i] = 0.0f;
    for (int j0 = lo & ~31; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const bool ok = j >= lo && j <= pos;
        const int rowi = ok ? bt[j / a.page_size] * a.page_size + j % a.page_size : 0;
        for (int g = warp; g < H; g += nwarps) {
            const T* kp = (const T*)a.k_pages + (size_t)(g / G) * a.k_head_stride;
            float p = 0.0f;
            if (ok) p = expf(dot_row<T>(q + (size_t)g * dk, kp + (size_t)rowi * a.k_ld, dk, vec) * a.scale - mx[g]) * rden[g];
            pw[g * 32 + lane] = p;
        }
        __syncthreads();
        const int nk = min(32, pos - j0 + 1);
#pragma unroll
        for (int u = 0; u < MAX_OWN; ++u) {
            const int h = warp + u * nwarps;
            if (h < H) {
                float mixed = 0.0f;
                for (int g = 0; g < H; ++g) mixed = fmaf(tk[h * H + g], pw[g * 32 + lane], mixed);
                const T* vp = (const T*)a.v_pages + (size_t)(h / G) * a.v_head_stride;
                for (int jj = max(0, lo - j0); jj < nk; ++jj) {
                    const float pj = __shfl_sync(0xffffffffu, mixed, jj);
                    const int rj = __shfl_sync(0xffffffffu, rowi, jj);
                    const T* vr = vp + (size_t)rj * a.v_ld;
#pragma unroll
                    for (int i = 0; i < DPLT; ++i) {
                        const int d = lane + 32 * i;
                        if (d < a.dv) o[u][i] = fmaf(pj, to_f32(vr[d]), o[u][i]);
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int u = 0; u < MAX_OWN; ++u) {
        const int h = warp + u * nwarps;
        if (h < H) {
            const size_t orow = a.out_head_major ? (size_t)h * a.T_ + t : (size_t)t * H + h;
#pragma unroll
            for (int i = 0; i < DPLT; ++i) {
                const int d = lane + 32 * i;
                if (d < a.dv) out[orow * a.dv + d] = from_f32<T>(o[u][i]);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ preparation
// The first `rd` of n values in shared memory x turn by pos * inv_freq[pair]; returns element d's new value.
__device__ __forceinline__ float rotated(const float* x, int d, int rd, int neighbours, int pos, const float* inv_freq) {
    if (d >= rd) return x[d];
    const int half = rd / 2;
    const int i = neighbours ? d >> 1 : (d < half ? d : d - half);
    const bool first = neighbours ? !(d & 1) : d < half;
    const int partner = neighbours ? d ^ 1 : (first ? d + half : d - half);
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    return first ? x[d] * cs - x[partner] * sn : x[d] * cs + x[partner] * sn;
}

// qkv: FP32 [T, ld] = [Hq heads of hd | Hkv heads of hd | Hv heads of vd].  Per-head RMS norm of q and k (weights or
// null), rotation of their first rd dimensions (inv_freq or null), q -> q_out [T, Hq, hd]; k, v -> pages
// [Hkv, num_pages, page_size, hd] and [Hv, .., vd].  Grid (T, Hq + Hkv + Hv) (or (T, Hq) when nothing is written).
// bias: one entry per column of a row, added to the summed slices, or null.  v_is_k: the rows hold no v heads; a value is its
// key as projected (bias included, before norm and rotation).
template <typename T>
__global__ void __launch_bounds__(128) qkv_pages_kernel(const float* qkv, int ld, int splits, size_t split_stride, int Hq, int Hkv, int hd, int vd,
                                                        const float* q_norm, const float* k_norm, float eps, const float* inv_freq, int rd,
                                                        int neighbours, const int* positions, const int* req_of_token,
                                                        const int* block_table, int max_blocks, int page_size, int num_pages, T* q_out,
                                                        T* k_pages, T* v_pages, int Hv, const float* bias, int v_is_k) {
    pdl_enter();
    extern __shared__ float xs[];            // max(hd, vd) floats
    __shared__ float red[32];
    const int t = blockIdx.x, h = blockIdx.y;
    const int kind = h < Hq ? 0 : h < Hq + Hkv ? 1 : 2;
    const int pos = positions[t];
    const int n = kind == 2 ? vd : hd;
    // a value head of a layer whose values are its keys reads the key head of its number (as projected)
    const size_t col = kind == 0 ? (size_t)h * hd : kind == 1 ? (size_t)Hq * hd + (size_t)(h - Hq) * hd
                     : v_is_k    ? (size_t)Hq * hd + (size_t)(h - Hq - Hkv) * hd
                                 : (size_t)(Hq + Hkv) * hd + (size_t)(h - Hq - Hkv) * vd;
    const float* src = qkv + (size_t)t * ld + col;
    float ss = 0.0f;
    for (int d = threadIdx.x; d < n; d += blockDim.x) {
        float v = src[d];
        for (int s = 1; s < splits; ++s) v += src[s * split_stride + d];
        if (bias) v += bias[col + d];
        xs[d] = v;
        ss = fmaf(v, v, ss);
    }
    const float* nw = kind == 0 ? q_norm : kind == 1 ? k_norm : nullptr;
    if (nw) {
        const float inv = rsqrtf(block_sum(ss, red) / (float)n + eps);
        for (int d = threadIdx.x; d < n; d += blockDim.x) xs[d] = xs[d] * inv * nw[d];
    }
    __syncthreads();
    T* dst;
    if (kind == 0) {
        dst = q_out + ((size_t)t * Hq + h) * hd;
    } else {
        const int page = block_table[(size_t)req_of_token[t] * max_blocks + pos / page_size];
        if (page < 0) return;
        const int kh = kind == 1 ? h - Hq : h - Hq - Hkv;
        dst = (kind == 1 ? k_pages : v_pages) + (((size_t)kh * num_pages + page) * page_size + pos % page_size) * n;
    }
    const bool turns = inv_freq && kind != 2;
    for (int d = threadIdx.x; d < n; d += blockDim.x) dst[d] = from_f32<T>(turns ? rotated(xs, d, rd, neighbours, pos, inv_freq) : xs[d]);
}

// The same with a warp per (token, head), eight heads a block, for heads of at most 256 entries: a lane keeps its entries
// (lane, lane + 32, ...) in registers, the head passes through the warp's stretch of shared memory once for the rotation's
// partners, and the sums of squares are a warp's shuffles.  Same arithmetic and order of sums per head as the block kernel
// has for one warp's share; which of the two runs depends on the head widths alone.
template <typename T>
__global__ void __launch_bounds__(256) qkv_pages_warp_kernel(const float* qkv, int ld, int splits, size_t split_stride, int Hq, int Hkv, int hd, int vd,
                                                             const float* q_norm, const float* k_norm, float eps, const float* inv_freq, int rd,
                                                             int neighbours, const int* positions, const int* req_of_token,
                                                             const int* block_table, int max_blocks, int page_size, int num_pages, T* q_out,
                                                             T* k_pages, T* v_pages, int heads, const float* bias, int v_is_k) {
    pdl_enter();
    __shared__ float stage[8][256];
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * 8 + warp;
    if (h >= heads) return;
    const int kind = h < Hq ? 0 : h < Hq + Hkv ? 1 : 2;
    const int pos = positions[t];
    const int n = kind == 2 ? vd : hd;
    // a value head of a layer whose values are its keys reads the key head of its number (as projected)
    const size_t col = kind == 0 ? (size_t)h * hd : kind == 1 ? (size_t)Hq * hd + (size_t)(h - Hq) * hd
                     : v_is_k    ? (size_t)Hq * hd + (size_t)(h - Hq - Hkv) * hd
                                 : (size_t)(Hq + Hkv) * hd + (size_t)(h - Hq - Hkv) * vd;
    const float* src = qkv + (size_t)t * ld + col;
    float x[8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int d = lane + 32 * j;
        float v = 0.0f;
        if (d < n) {
            v = src[d];
            for (int s = 1; s < splits; ++s) v += src[s * split_stride + d];
            if (bias) v += bias[col + d];
        }
        x[j] = v;
        ss = fmaf(v, v, ss);
    }
    const float* nw = kind == 0 ? q_norm : kind == 1 ? k_norm : nullptr;
    if (nw) {
        const float inv = rsqrtf(warp_sum(ss) / (float)n + eps);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int d = lane + 32 * j;
            if (d < n) x[j] = x[j] * inv * nw[d];
        }
    }
    T* dst;
    if (kind == 0) {
        dst = q_out + ((size_t)t * Hq + h) * hd;
    } else {
        const int page = block_table[(size_t)req_of_token[t] * max_blocks + pos / page_size];
        if (page < 0) return;
        const int kh = kind == 1 ? h - Hq : h - Hq - Hkv;
        dst = (kind == 1 ? k_pages : v_pages) + (((size_t)kh * num_pages + page) * page_size + pos % page_size) * n;
    }
    const bool turns = inv_freq && kind != 2 && rd > 0;
    if (turns) {
        float* xs = stage[warp];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int d = lane + 32 * j;
            if (d < n) xs[d] = x[j];
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int d = lane + 32 * j;
            if (d < n) dst[d] = from_f32<T>(rotated(xs, d, rd, neighbours, pos, inv_freq));
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int d = lane + 32 * j;
        if (d < n) dst[d] = from_f32<T>(x[j]);
    }
}

// The inputs of attention over a cached latent.  x: FP32 [T, ld] = [H query heads of (dim + rd) | latent of `rank` | rd].
// Block (t, h < H): the head's first `dim` values -> qn[(h T + t) dim] (they go through the key up-projection next), its
// last rd values, the first `turn` of them rotated -> qr[(h T + t) rd].  Block (t, H): the latent, RMS-normed with weight
// cw -> the page row's first `rank` values; the shared rotated key part -> the row's last rd.  neighbours: the rotation
// pairs 2i with 2i+1 instead of i with i + turn/2.  A layer that reads another layer's pages has no block (t, H) (and x no
// latent columns).
template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(const float* x, int ld, int H, int dim, int rd, int rank, const float* cw, float eps,
                                                          const float* inv_freq, int turn, int neighbours, const int* positions,
                                                          const int* req_of_token, const int* block_table, int max_blocks, int page_size,
                                                          T* qn, T* qr, T* pages, int T_) {
    pdl_enter();
    extern __shared__ float xs[];            // rd floats (the part that turns)
    __shared__ float red[32];
    const int t = blockIdx.x, h = blockIdx.y, pos = positions[t];
    if (h < H) {
        const float* src = x + (size_t)t * ld + (size_t)h * (dim + rd);
        const size_t row = (size_t)h * T_ + t;
        for (int d = threadIdx.x; d < dim; d += blockDim.x) qn[row * dim + d] = from_f32<T>(src[d]);
        for (int d = threadIdx.x; d < rd; d += blockDim.x) xs[d] = src[dim + d];
        __syncthreads();
        for (int d = threadIdx.x; d < rd; d += blockDim.x) qr[row * rd + d] = from_f32<T>(rotated(xs, d, turn, neighbours, pos, inv_freq));
        return;
    }
    const float* src = x + (size_t)t * ld + (size_t)H * (dim + rd);
    float ss = 0.0f;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) ss = fmaf(src[d], src[d], ss);
    const float inv = rsqrtf(block_sum(ss, red) / (float)rank + eps);
    for (int d = threadIdx.x; d < rd; d += blockDim.x) xs[d] = src[rank + d];
    __syncthreads();
    const int page = block_table[(size_t)req_of_token[t] * max_blocks + pos / page_size];
    if (page < 0) return;
    T* dst = pages + ((size_t)page * page_size + pos % page_size) * (rank + rd);
    for (int d = threadIdx.x; d < rank; d += blockDim.x) dst[d] = from_f32<T>(src[d] * inv * cw[d]);
    for (int d = threadIdx.x; d < rd; d += blockDim.x) dst[rank + d] = from_f32<T>(rotated(xs, d, turn, neighbours, pos, inv_freq));
}

// src: FP32 [H, T, n] -> out: [T, H n] in the storage type.
template <typename T>
__global__ void heads_to_rows_kernel(const float* src, T* out, int H, int T_, int n) {
    pdl_enter();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)H * T_ * n) return;
    const int d = i % n;
    const size_t th = i / n;
    const int h = th % H;
    const size_t t = th / H;
    out[i] = from_f32<T>(src[((size_t)h * T_ + t) * n + d]);
}

// The two maps of a head combined: a FP32 [T, H, 2, dv] (a head's maps side by side) -> out [T, H dv] in the storage type,
// o = a1 - lambda a2, then o / sqrt(mean(o^2) + eps) * mult over the head's dv values.  A warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128) map_difference_kernel(const float* a, T* out, int rows, int dv, float lambda, float eps, float mult) {
    pdl_enter();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* a1 = a + (size_t)row * 2 * dv;
    const float* a2 = a1 + dv;
    float ss = 0.0f;
    for (int d = lane; d < dv; d += 32) {
        const float o = a1[d] - lambda * a2[d];
        ss = fmaf(o, o, ss);
    }
    const float inv = rsqrtf(warp_sum(ss) / (float)dv + eps) * mult;
    for (int d = lane; d < dv; d += 32) out[(size_t)row * dv + d] = from_f32<T>((a1[d] - lambda * a2[d]) * inv);
}

}  // namespace

Q6K_API int q6k_map_difference(const float* a, void* out, int T_, int H, int dv, float lambda, float eps, float mult, int dtype, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && H > 0 && dv > 0, "map_difference: bad sizes T=%d H=%d dv=%d", T_, H, dv);
    const long long rows = (long long)T_ * H;
    Q6K_REQUIRE(rows <= 0x7fffffffLL, "map_difference: too many rows");
    Q6K_DISPATCH(dtype, q6k_launch(map_difference_kernel<T>, dim3((unsigned)((rows + 3) / 4)), 128, 0, st, a, (T*)out, (int)rows, dv, lambda, eps, mult););
    return q6k_check_launch("map_difference");
}

Q6K_API int q6k_attention_flex(const float* qa, int da, const void* qb, int db, int q_head_major, const void* k_pages,
                               long long k_head_stride, int k_ld, const void* v_pages, long long v_head_stride, int v_ld, int dv,
                               const int* block_table, int max_blocks, int page_size, const int* req_of_token, const int* positions,
                               int window, int chunk, float scale, const float* talk, const float* sinks, void* out, int out_head_major,
                               int T_, int H, int Hkv, int dtype, float softcap, int maps, float* out_f32, cudaStream_t st) {
    if (T_ == 0) return 0;
    const int dk = da + db;
    Q6K_REQUIRE(maps >= 1 && Hkv % maps == 0 && softcap >= 0.0f, "attention: %d maps over %d key heads, softcap %f", maps, Hkv, softcap);
    Q6K_REQUIRE(!talk || (maps == 1 && softcap == 0.0f && !out_f32), "attention with mixed heads takes neither maps, a cap nor FP32 results");
    Q6K_REQUIRE(T_ > 0 && H > 0 && Hkv > 0 && H % Hkv == 0, "attention: bad head counts H=%d Hkv=%d", H, Hkv);
    Q6K_REQUIRE(da >= 0 && db >= 0 && dk > 0 && (da == 0 || qa) && (db == 0 || qb), "attention: bad query parts %d + %d", da, db);
    Q6K_REQUIRE(dv > 0 && dv <= MAX_DV, "attention: value width %d outside 1..%d", dv, MAX_DV);
    Q6K_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0 && chunk >= 0, "attention: bad page_size %d / max_blocks %d / window %d / chunk %d",
                page_size, max_blocks, window, chunk);
    FlexArgs a{qa, da, qb, db, q_head_major, k_pages, k_head_stride, k_ld, v_pages, v_head_stride, v_ld, dv, block_table, max_blocks,
               page_size, req_of_token, positions, window, chunk, scale, talk, out, out_head_major, T_, H, Hkv, sinks, softcap, maps, out_f32};
    if (talk) {
        Q6K_REQUIRE(!sinks, "attention with mixed heads takes no sinks");
        Q6K_REQUIRE(dv <= 256 && H <= 64, "attention with mixed heads: value width %d (at most 256), %d heads (at most 64)", dv, H);
        const int warps = H < 8 ? H : 8;
        const size_t smem = ((size_t)H * dk + 2 * H + (size_t)H * 32 + (size_t)H * H) * sizeof(float);
        Q6K_REQUIRE(smem <= 200 * 1024, "attention with mixed heads: %d heads of %d do not fit shared memory", H, dk);
        Q6K_DISPATCH(dtype, {
            if (smem > 48 * 1024) cudaFuncSetAttribute(attention_talk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            q6k_launch(attention_talk_kernel<T>, dim3(T_), warps * 32, smem, st, a);
        });
        return q6k_check_launch("attention_talk");
    }
    Q6K_REQUIRE(Hkv <= 65535, "attention: %d KV heads exceed the grid limit", Hkv);
    const int G = H / Hkv;
    const int warps = G < 4 ? G : 4;
    const size_t smem = (size_t)warps * dk * sizeof(float);
    Q6K_REQUIRE(smem <= 48 * 1024, "attention: keys of %d do not fit shared memory", dk);
    Q6K_DISPATCH(dtype, q6k_launch(attention_flex_kernel<T>, dim3(T_, Hkv), warps * 32, smem, st, a););
    return q6k_check_launch("attention_flex");
}

Q6K_API int q6k_qkv_pages(const float* qkv, int ld, int splits, long long split_stride, int T_, int Hq, int Hkv, int hd, int vd,
                          const float* q_norm, const float* k_norm, float eps, const float* inv_freq, int rotary_dim, int neighbours,
                          const int* positions, const int* req_of_token, const int* block_table, int max_blocks, int page_size,
                          int num_pages, void* q_out, void* k_pages, void* v_pages, int write_kv, int dtype, int Hv, const float* bias, int v_is_k,
                          cudaStream_t st) {
    if (T_ == 0) return 0;
    if (Hv <= 0) Hv = Hkv;
    Q6K_REQUIRE(!v_is_k || (Hv == Hkv && vd == hd), "qkv_pages: values that are the keys have the keys' heads and width");
    Q6K_REQUIRE(T_ > 0 && Hq > 0 && Hkv > 0 && hd > 0 && vd > 0 && splits >= 1, "qkv_pages: bad sizes T=%d Hq=%d Hkv=%d hd=%d vd=%d", T_, Hq, Hkv, hd, vd);
    Q6K_REQUIRE(!inv_freq || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= hd), "qkv_pages: %d rotating dimensions of a head of %d", rotary_dim, hd);
    Q6K_REQUIRE(!write_kv || (page_size > 0 && max_blocks > 0), "qkv_pages: bad page_size %d / max_blocks %d", page_size, max_blocks);
    const int heads = write_kv ? Hq + Hkv + Hv : Hq;
    Q6K_REQUIRE(heads <= 65535, "qkv_pages: %d heads exceed the grid limit", heads);
    const size_t smem = (size_t)(hd > vd ? hd : vd) * sizeof(float);
    Q6K_REQUIRE(smem <= 48 * 1024, "qkv_pages: heads of %d do not fit shared memory", hd > vd ? hd : vd);
    if (hd <= 256 && vd <= 256 && (heads + 7) / 8 <= 65535) {                 // narrow heads: a warp per head
        Q6K_DISPATCH(dtype, q6k_launch(qkv_pages_warp_kernel<T>, dim3(T_, (heads + 7) / 8), 256, 0, st, qkv, ld, splits, (size_t)split_stride, Hq, Hkv,
                                       hd, vd, q_norm, k_norm, eps, inv_freq, inv_freq ? rotary_dim : 0, neighbours, positions, req_of_token,
                                       block_table, max_blocks, page_size, num_pages, (T*)q_out, (T*)k_pages, (T*)v_pages, heads, bias, v_is_k););
        return q6k_check_launch("qkv_pages");
    }
    Q6K_DISPATCH(dtype, q6k_launch(qkv_pages_kernel<T>, dim3(T_, heads), 128, smem, st, qkv, ld, splits, (size_t)split_stride, Hq, Hkv, hd, vd,
                                   q_norm, k_norm, eps, inv_freq, inv_freq ? rotary_dim : 0, neighbours, positions, req_of_token, block_table,
                                   max_blocks, page_size, num_pages, (T*)q_out, (T*)k_pages, (T*)v_pages, Hv, bias, v_is_k););
    return q6k_check_launch("qkv_pages");
}

Q6K_API int q6k_latent_prep(const float* x, int ld, int T_, int H, int dim, int rd, int rank, const float* cw, float eps,
                            const float* inv_freq, int turn, int neighbours, const int* positions, const int* req_of_token,
                            const int* block_table, int max_blocks, int page_size, void* qn, void* qr, void* pages, int dtype, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && H > 0 && dim > 0 && rd >= 0 && (rank > 0 || !pages), "latent_prep: bad sizes T=%d H=%d dim=%d rd=%d rank=%d", T_, H, dim, rd, rank);
    Q6K_REQUIRE(turn >= 0 && turn % 2 == 0 && turn <= rd && (turn == 0 || inv_freq), "latent_prep: %d turning dimensions of %d", turn, rd);
    Q6K_REQUIRE(H + 1 <= 65535 && (!pages || (page_size > 0 && max_blocks > 0 && cw)), "latent_prep: bad grid or pages");
    const size_t smem = (size_t)(rd > 0 ? rd : 1) * sizeof(float);
    Q6K_DISPATCH(dtype, q6k_launch(latent_prep_kernel<T>, dim3(T_, pages ? H + 1 : H), 128, smem, st, x, ld, H, dim, rd, rank, cw, eps, inv_freq, turn,
                                   neighbours, positions, req_of_token, block_table, max_blocks, page_size, (T*)qn, (T*)qr, (T*)pages, T_););
    return q6k_check_launch("latent_prep");
}

Q6K_API int q6k_heads_to_rows(const float* src, void* out, int H, int T_, int n, int dtype, cudaStream_t st) {
    if (T_ == 0) return 0;
    const size_t total = (size_t)H * T_ * n;
    Q6K_DISPATCH(dtype, q6k_launch(heads_to_rows_kernel<T>, dim3((unsigned)((total + 255) / 256)), 256, 0, st, src, (T*)out, H, T_, n););
    return q6k_check_launch("heads_to_rows");
}
