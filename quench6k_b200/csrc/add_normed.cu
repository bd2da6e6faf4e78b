// The closing add of a sublayer whose result passes an RMS norm of its own before it joins the stream, and the stream in
// the operand dtype for the sublayer that reads it next, in one pass over the row:
//
//   y[t] = a[t] (+ sum_s pw[t, s] * py[row(t, s)])            a: FP32 [T, D] or split-K partial sums [slices, T, D], added in order
//   h[t] += y[t] * rsqrt(mean(y[t]^2) + eps) * w              (skipped when there is neither a nor py)
//   out[t] = T(h[t])                                           (optional)
//
// One block per row; the row of y waits in shared memory between the two passes.  Everything is FP32.
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
    Q6K_DISPATCH(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_normed_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        q6k_launch(add_normed_kernel<T>, T_, 256, smem, st, h, a, slices, (size_t)slice_stride, py, pair_row, pw, S, w, eps, (T*)out, D);
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
