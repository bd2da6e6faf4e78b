// The closing add of a block whose sublayers run side by side, and the norms that open the next block, in one pass over
// the row:
//
//   h[t] += m * (a[t] + bias + b[t] + sum_s pw[t, s] * py[row(t, s)])   (each of the four optional; bias: one vector for all rows)
//   out1[r] = T(h[t] * rsqrt(mean(h[t]^2) + eps) * w1),  out2[r] likewise with w2    (each optional; t = rows[r] or r)
//
// a and b may be split-K partial sums [slices, T, D], added in order.  Everything is FP32; the outputs are in the
// operand dtype.  One block per row; a thread re-reads only what it wrote itself.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256) scaled_add_norm_kernel(float* h, const float* a, int a_slices, const float* b, int b_slices, size_t slice_stride,
                                                              const float* py, const int* pair_row, const float* pw, int S, float m,
                                                              const int* rows, const float* w1, T* out1, const float* w2, T* out2, float eps,
                                                              int D, const float* bias) {
    pdl_enter();
    __shared__ float red[32];
    const int r = blockIdx.x, t = rows ? rows[r] : r;
    float* hr = h + (size_t)t * D;
    const bool adds = a || b || py || bias;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = hr[i];
        if (adds) {
            float sum = 0.0f;
            if (a) {
                sum = a[(size_t)t * D + i];
                for (int s = 1; s < a_slices; ++s) sum += a[s * slice_stride + (size_t)t * D + i];
            }
            if (bias) sum += bias[i];
            if (b) {
                float sb = b[(size_t)t * D + i];
                for (int s = 1; s < b_slices; ++s) sb += b[s * slice_stride + (size_t)t * D + i];
                sum += sb;
            }
            if (py) {
                float sp = 0.0f;
                for (int s = 0; s < S; ++s) sp = fmaf(pw[t * S + s], py[(size_t)(pair_row ? pair_row[t * S + s] : t * S + s) * D + i], sp);
                sum += sp;
            }
            v = fmaf(m, sum, v);
            hr[i] = v;
        }
        ss = fmaf(v, v, ss);
    }
    if (!out1 && !out2) return;
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = hr[i] * inv;
        if (out1) out1[(size_t)r * D + i] = from_f32<T>(v * w1[i]);
        if (out2) out2[(size_t)r * D + i] = from_f32<T>(v * w2[i]);
    }
}

// The same, four columns per thread step with 16-byte loads (D a multiple of 4, every pointer on 16 bytes); up to four
// steps of a thread stay in registers between the two passes (rows up to 4,096 wide), wider rows are read again.
__device__ __forceinline__ void add4(float4& a, const float4 b) { a.x += b.x, a.y += b.y, a.z += b.z, a.w += b.w; }

template <typename T>
__global__ void __launch_bounds__(256) scaled_add_norm4_kernel(float* h, const float* a, int a_slices, const float* b, int b_slices, size_t slice_stride,
                                                               const float* py, const int* pair_row, const float* pw, int S, float m,
                                                               const int* rows, const float* w1, T* out1, const float* w2, T* out2, float eps,
                                                               int D, const float* bias) {
    pdl_enter();
    __shared__ float red[32];
    const int r = blockIdx.x, t = rows ? rows[r] : r, D4 = D >> 2;
    float4* hr = reinterpret_cast<float4*>(h + (size_t)t * D);
    const bool adds = a || b || py || bias;
    float4 keep[4];
    float ss = 0.0f;
#pragma unroll
    for (int step = 0; step < 4; ++step) {
        const int i = threadIdx.x + 256 * step;
        if (i >= D4) break;
        float4 v = hr[i];
        if (adds) {
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (a) {
                sum = reinterpret_cast<const float4*>(a + (size_t)t * D)[i];
                for (int s = 1; s < a_slices; ++s) add4(sum, reinterpret_cast<const float4*>(a + s * slice_stride + (size_t)t * D)[i]);
            }
            if (bias) add4(sum, reinterpret_cast<const float4*>(bias)[i]);
            if (b) {
                float4 sb = reinterpret_cast<const float4*>(b + (size_t)t * D)[i];
                for (int s = 1; s < b_slices; ++s) add4(sb, reinterpret_cast<const float4*>(b + s * slice_stride + (size_t)t * D)[i]);
                add4(sum, sb);
            }
            if (py) {
                float4 sp = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int s = 0; s < S; ++s) {
                    const float ws = pw[t * S + s];
                    const float4 y = reinterpret_cast<const float4*>(py + (size_t)(pair_row ? pair_row[t * S + s] : t * S + s) * D)[i];
                    sp.x = fmaf(ws, y.x, sp.x), sp.y = fmaf(ws, y.y, sp.y), sp.z = fmaf(ws, y.z, sp.z), sp.w = fmaf(ws, y.w, sp.w);
                }
                add4(sum, sp);
            }
            v.x = fmaf(m, sum.x, v.x), v.y = fmaf(m, sum.y, v.y), v.z = fmaf(m, sum.z, v.z), v.w = fmaf(m, sum.w, v.w);
            hr[i] = v;
        }
        keep[step] = v;
        ss = fmaf(v.x, v.x, ss), ss = fmaf(v.y, v.y, ss), ss = fmaf(v.z, v.z, ss), ss = fmaf(v.w, v.w, ss);
    }
    if (!out1 && !out2) return;
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
    for (int step = 0; step < 4; ++step) {
        const int i = threadIdx.x + 256 * step;
        if (i >= D4) break;
        const float4 v = keep[step];
        if (out1) {
            const float4 g = reinterpret_cast<const float4*>(w1)[i];
            T* o = out1 + (size_t)r * D + 4 * i;
            o[0] = from_f32<T>(v.x * inv * g.x), o[1] = from_f32<T>(v.y * inv * g.y), o[2] = from_f32<T>(v.z * inv * g.z), o[3] = from_f32<T>(v.w * inv * g.w);
        }
        if (out2) {
            const float4 g = reinterpret_cast<const float4*>(w2)[i];
            T* o = out2 + (size_t)r * D + 4 * i;
            o[0] = from_f32<T>(v.x * inv * g.x), o[1] = from_f32<T>(v.y * inv * g.y), o[2] = from_f32<T>(v.z * inv * g.z), o[3] = from_f32<T>(v.w * inv * g.w);
        }
    }
}

// act: 0 silu, 1 the tanh form of gelu, 2 the square of relu
__device__ __forceinline__ float activation(float z, int act) {
    if (act == 0) return z / (1.0f + expf(-z));
    if (act == 1) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    const float p = fmaxf(z, 0.0f);
    return p * p;
}

// out[r, i] = T(act(x[r, i]) * x[r, I + i]) (gated: x has 2 I columns) or T(act(x[r, i])).
template <typename T>
__global__ void activate_kernel(const float* x, int ldx, T* out, int I, size_t count, int gated, int act) {
    pdl_enter();
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= count) return;
    const size_t r = idx / I;
    const int i = (int)(idx % I);
    const float z = activation(x[r * ldx + i], act);
    out[idx] = from_f32<T>(gated ? z * x[r * ldx + I + i] : z);
}

// One warp per token: scores s = sigmoid(logits), the k largest of s + bias (ties to the lower index), weights
// s / (sum of the chosen s + 1e-20) * scale, or s * scale when renorm is 0.  logits: [slices, T, E], summed in order.
// groups > 1: the experts form `groups` equal groups of neighbours; a group's worth is the sum of its two largest choice
// values (its one value, if it has one expert), and only experts of the `keep` groups of most worth (ties to the lower
// index) can be chosen.  Shared memory: E floats a warp (the choice values), E more (the scores) and `groups` more.
__global__ void route_biased_kernel(const float* logits, int slices, size_t slice_stride, const float* bias, float scale, int T_, int E, int k,
                                    int* sel_e, float* sel_w, int renorm, int groups, int keep) {
    pdl_enter();
    extern __shared__ float sc[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int t = blockIdx.x * warps + warp;
    if (t >= T_) return;
    float* choice = sc + (size_t)warp * (2 * E + groups);
    float* score = choice + E;
    float* worth = score + E;
    for (int e = lane; e < E; e += 32) {
        float z = logits[(size_t)t * E + e];
        for (int s = 1; s < slices; ++s) z += logits[s * slice_stride + (size_t)t * E + e];
        const float sg = 1.0f / (1.0f + expf(-z));
        score[e] = sg;
        choice[e] = bias ? sg + bias[e] : sg;
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {                              // a lane per group: its two largest choice values
            float a = -INFINITY, b = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float c = choice[e];
                if (c > a) b = a, a = c;
                else if (c > b) b = c;
            }
            worth[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        for (int j = 0; j < keep; ++j) {                                       // the kept groups are marked by +inf
            float best = -INFINITY;
            int best_g = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float c = worth[g];
                if (c != INFINITY && (c > best || (c == best && g < best_g) || best_g == 0x7fffffff)) best = c, best_g = g;
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, off);
                const int og = __shfl_xor_sync(0xffffffffu, best_g, off);
                if (og != 0x7fffffff && (best_g == 0x7fffffff || ob > best || (ob == best && og < best_g))) best = ob, best_g = og;
            }
            __syncwarp();
            if (lane == 0 && best_g < groups) worth[best_g] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (worth[e / per] != INFINITY) choice[e] = -INFINITY;
        __syncwarp();
    }
    float sum = 0.0f, mine = 0.0f;
    int mine_e = 0;
    for (int j = 0; j < k; ++j) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float c = choice[e];
            if (c > best || (c == best && e < best_e)) best = c, best_e = e;       // NaN never wins; taken experts are -inf
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, off);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
            if (ob > best || (ob == best && oe < best_e)) best = ob, best_e = oe;
        }
        if (best_e >= E) best_e = 0;                                               // every value NaN: a defined answer
        const float sg = score[best_e];
        sum += sg;
        if ((j & 31) == lane) {
            if (j >= 32) sel_w[(size_t)t * k + j - 32] = mine, sel_e[(size_t)t * k + j - 32] = mine_e;
            mine = sg, mine_e = best_e;
        }
        __syncwarp();
        if (lane == 0) choice[best_e] = -INFINITY;
        __syncwarp();
    }
    const float den = renorm ? sum + 1e-20f : 1.0f;
    // every lane's last result, then the earlier ones it parked in memory
    const int last = lane < k ? ((k - 1 - lane) >> 5) * 32 + lane : -1;
    if (last >= 0) sel_w[(size_t)t * k + last] = mine, sel_e[(size_t)t * k + last] = mine_e;
    __syncwarp();
    for (int j = lane; j < k; j += 32) sel_w[(size_t)t * k + j] = sel_w[(size_t)t * k + j] / den * scale;
}

}  // namespace

Q6K_API int q6k_scaled_add_norm(float* h, const float* a, int a_slices, const float* b, int b_slices, long long slice_stride, const float* py,
                                const int* pair_row, const float* pw, int S, float m, const int* rows, const float* w1, void* out1,
                                const float* w2, void* out2, float eps, int R, int D, int dtype, const float* bias, cudaStream_t st) {
    if (R == 0) return 0;
    Q6K_REQUIRE(R > 0 && D > 0 && a_slices >= 1 && b_slices >= 1, "scaled_add_norm: bad sizes R=%d D=%d", R, D);
    Q6K_REQUIRE(!(rows && (a || b || py || bias)), "scaled_add_norm: the add takes no row selection");
    Q6K_REQUIRE(!py || (pw && S > 0), "scaled_add_norm: weighted rows need their weights");
    Q6K_REQUIRE((out1 == nullptr || w1) && (out2 == nullptr || w2), "scaled_add_norm: an output needs its weight");
    auto on16 = [](const void* ptr) { return ((uintptr_t)ptr & 15) == 0; };
    const bool vec = D % 4 == 0 && D <= 4096 && slice_stride % 4 == 0 && on16(h) && on16(a) && on16(b) && on16(py) && on16(w1) && on16(w2) && on16(bias);
    // which of the two kernels runs depends on the row width and the buffers' alignment alone, never on the step
    if (vec) {
        Q6K_DISPATCH(dtype, q6k_launch(scaled_add_norm4_kernel<T>, R, 256, 0, st, h, a, a_slices, b, b_slices, (size_t)slice_stride, py, pair_row, pw, S, m,
                                       rows, w1, (T*)out1, w2, (T*)out2, eps, D, bias););
        return q6k_check_launch("scaled_add_norm");
    }
    Q6K_DISPATCH(dtype, q6k_launch(scaled_add_norm_kernel<T>, R, 256, 0, st, h, a, a_slices, b, b_slices, (size_t)slice_stride, py, pair_row, pw, S, m,
                                   rows, w1, (T*)out1, w2, (T*)out2, eps, D, bias););
    return q6k_check_launch("scaled_add_norm");
}

Q6K_API int q6k_activate(const float* x, int ldx, void* out, int rows, int I, int gated, int act, int dtype, cudaStream_t st) {
    if (rows == 0) return 0;
    Q6K_REQUIRE(rows > 0 && I > 0 && ldx >= (gated ? 2 * I : I) && act >= 0 && act <= 2, "activate: bad sizes rows=%d I=%d ldx=%d act=%d", rows, I, ldx, act);
    const size_t count = (size_t)rows * I;
    Q6K_DISPATCH(dtype, q6k_launch(activate_kernel<T>, (unsigned)((count + 255) / 256), 256, 0, st, x, ldx, (T*)out, I, count, gated, act););
    return q6k_check_launch("activate");
}

Q6K_API int q6k_route_biased(const float* logits, int slices, const float* bias, float scale, int T_, int E, int k, int* sel_e, float* sel_w,
                             int renorm, int groups, int keep, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && E > 0 && k > 0 && k <= E && slices >= 1, "route_biased: bad sizes T=%d E=%d k=%d slices=%d", T_, E, k, slices);
    Q6K_REQUIRE(E <= 4096, "route_biased: %d experts exceed the supported 4096", E);
    Q6K_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups && k <= keep * (E / groups),
                "route_biased: %d experts in %d groups, %d kept, %d chosen", E, groups, keep, k);
    const int warps = E <= 1024 ? 4 : 1;
    q6k_launch(route_biased_kernel, (T_ + warps - 1) / warps, warps * 32, (size_t)warps * (2 * E + groups) * sizeof(float), st, logits, slices,
               (size_t)T_ * E, bias, scale, T_, E, k, sel_e, sel_w, renorm, groups, keep);
    return q6k_check_launch("route_biased");
}
