// The closing add of a sublayer whose result passes an RMS norm of its own before it joins the stream, and the stream in
// the operand dtype for the sublayer that reads it next, in one pass over the row:
//
//   y[t] = a[t] (+ sum_s pw[t, s] * py[row(t, s)])            a: FP32 [T, D] or split-K partial sums [slices, T, D], added in order
//   h[t] += y[t] * rsqrt(mean(y[t]^2) + eps) * w              (skipped when there is neither a nor py)
//   out[t] = T(h[t])                                           (optional)
//
// One block per row; the row of y waits in shared memory between the two passes.  Everything is FP32.  Rows whose length
// is a multiple of four move 16 bytes at a time.
//
// Also here: the gate of a per-token side input, out[t, j] = T(gelu_tanh(p[t, j]) * e[t, col0 + j]).
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256) add_normed_kernel(float* h, const float* a, int slices, size_t slice_stride, const float* py,
                                                         const int* pair_row, const float* pw, int S, const float* w, float eps, T* out, int D) {
    pdl_enter();
    extern __shared__ float ys[];            // D floats
    __shared__ float red[32];
    const int t = blockIdx.x;
    float* hr = h + (size_t)t * D;
    if (!a && !py) {
        for (int i = threadIdx.x; i < D; i += blockDim.x) out[(size_t)t * D + i] = from_f32<T>(hr[i]);
        return;
    }
    float ss = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = 0.0f;
        if (a) {
            v = a[(size_t)t * D + i];
            for (int s = 1; s < slices; ++s) v += a[s * slice_stride + (size_t)t * D + i];
        }
        if (py) {
            float sp = 0.0f;
            for (int s = 0; s < S; ++s) sp = fmaf(pw[t * S + s], py[(size_t)(pair_row ? pair_row[t * S + s] : t * S + s) * D + i], sp);
            v += sp;
        }
        ys[i] = v;
        ss = fmaf(v, v, ss);
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = hr[i] + ys[i] * inv * w[i];
        hr[i] = v;
        if (out) out[(size_t)t * D + i] = from_f32<T>(v);
    }
}

// Four elements of a row as T: 16 bytes of FP32 or 8 of bfloat16.
__device__ __forceinline__ void store4(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const unsigned*>(&lo);
    u.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(dst) = u;
}

// The same for rows whose length is a multiple of four and whose operands start on 16 bytes: every read and write moves
// 16 bytes (8 for a bfloat16 result).  An element's sums are made in the same order as above.
template <typename T>
__global__ void __launch_bounds__(256) add_normed_vec_kernel(float* h, const float* a, int slices, size_t slice_stride, const float* py,
                                                             const int* pair_row, const float* pw, int S, const float* w, float eps, T* out, int D) {
    pdl_enter();
    extern __shared__ __align__(16) float ys[];            // D floats
    __shared__ float red[32];
    const int t = blockIdx.x, D4 = D / 4;
    float4* hr = reinterpret_cast<float4*>(h + (size_t)t * D);
    if (!a && !py) {
        for (int i = threadIdx.x; i < D4; i += blockDim.x) store4(out + (size_t)t * D + 4 * i, hr[i]);
        return;
    }
    float4* ys4 = reinterpret_cast<float4*>(ys);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < D4; i += blockDim.x) {
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (a) {
            v = *reinterpret_cast<const float4*>(a + (size_t)t * D + 4 * i);
            for (int s = 1; s < slices; ++s) {
                const float4 x = *reinterpret_cast<const float4*>(a + s * slice_stride + (size_t)t * D + 4 * i);
                v.x += x.x, v.y += x.y, v.z += x.z, v.w += x.w;
            }
        }
        if (py) {
            float4 sp = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int s = 0; s < S; ++s) {
                const float g = pw[t * S + s];
                const float4 x = *reinterpret_cast<const float4*>(py + (size_t)(pair_row ? pair_row[t * S + s] : t * S + s) * D + 4 * i);
                sp.x = fmaf(g, x.x, sp.x), sp.y = fmaf(g, x.y, sp.y), sp.z = fmaf(g, x.z, sp.z), sp.w = fmaf(g, x.w, sp.w);
            }
            v.x += sp.x, v.y += sp.y, v.z += sp.z, v.w += sp.w;
        }
        ys4[i] = v;
        ss = fmaf(v.x, v.x, ss), ss = fmaf(v.y, v.y, ss), ss = fmaf(v.z, v.z, ss), ss = fmaf(v.w, v.w, ss);
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)D + eps);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    for (int i = threadIdx.x; i < D4; i += blockDim.x) {
        const float4 y = ys4[i], g = w4[i];
        float4 v = hr[i];
        v.x = v.x + y.x * inv * g.x, v.y = v.y + y.y * inv * g.y, v.z = v.z + y.z * inv * g.z, v.w = v.w + y.w * inv * g.w;
        hr[i] = v;
        if (out) store4(out + (size_t)t * D + 4 * i, v);
    }
}

template <typename T>
__global__ void side_gate_kernel(const float* p, int slices, size_t slice_stride, const float* e, int lde, int col0, T* out, int n, size_t count) {
    pdl_enter();
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= count) return;
    const size_t t = idx / n;
    const int j = (int)(idx % n);
    float z = p[idx];
    for (int s = 1; s < slices; ++s) z += p[s * slice_stride + idx];
    out[idx] = from_f32<T>(q6k_activation(z, 1) * e[t * lde + col0 + j]);
}

}  // namespace

Q6K_API int q6k_add_normed(float* h, const float* a, int slices, long long slice_stride, const float* py, const int* pair_row, const float* pw,
                           int S, const float* w, float eps, void* out, int T_, int D, int dtype, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && D > 0 && slices >= 1, "add_normed: bad sizes T=%d D=%d", T_, D);
    Q6K_REQUIRE(!py || (pw && S > 0), "add_normed: weighted rows need their weights");
    Q6K_REQUIRE((!a && !py) ? out != nullptr : w != nullptr, "add_normed: nothing to do, or a norm without its weight");
    const size_t smem = (size_t)D * sizeof(float);
    Q6K_REQUIRE(smem <= 200 * 1024, "add_normed: rows of %d do not fit shared memory", D);
    auto on16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = D % 4 == 0 && slice_stride % 4 == 0 && on16(h) && on16(a) && on16(py) && on16(w) && on16(out);
    Q6K_DISPATCH(dtype, {
        auto kernel = vec ? add_normed_vec_kernel<T> : add_normed_kernel<T>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        q6k_launch(kernel, T_, 256, smem, st, h, a, slices, (size_t)slice_stride, py, pair_row, pw, S, w, eps, (T*)out, D);
    });
    return q6k_check_launch("add_normed");
}

Q6K_API int q6k_side_gate(const float* p, int slices, long long slice_stride, const float* e, int lde, int col0, void* out, int T_, int n,
                          int dtype, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && n > 0 && col0 >= 0 && col0 + n <= lde && slices >= 1, "side_gate: bad sizes T=%d n=%d col0=%d lde=%d", T_, n, col0, lde);
    const size_t count = (size_t)T_ * n;
    Q6K_DISPATCH(dtype, q6k_launch(side_gate_kernel<T>, (unsigned)((count + 255) / 256), 256, 0, st, p, slices, (size_t)slice_stride, e, lde, col0,
                                   (T*)out, n, count););
    return q6k_check_launch("side_gate");
}
