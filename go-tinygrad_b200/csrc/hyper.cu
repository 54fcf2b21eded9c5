// Hyper-connections: the hidden state in S copies x_1..x_S per token, float32,
// stored [token][copy][channel].
//
// A sublayer reads u = sum_s in[s] x_s through an RMS norm, and its output y goes
// back as  x_t <- sum_s mix[s,t] x_s + out[t] y  (mix is indexed [from, to]; all
// copies at once, from the old ones).  One kernel does what stands between two
// sublayers: it applies the update the sublayer before has left pending, writes
// the new copies, reads them with the next sublayer's `in` and norms:
//
//   x_t <- sum_s mix[s,t] x_s + out[t] y        (when y is given)
//   u    = sum_t in[t] x_t                      (in null: the plain sum)
//   r    = u / sqrt(mean(u^2) + eps) * w
//
// With `seed` the copies do not exist yet: every copy is the seed's row (the
// embedding output) and is written as such.  With `rows` only those tokens are
// read, nothing is written back, and r has one row per entry (the final norm on
// the wanted rows).  S = 1 with mix = in = 1 is the ordinary residual sum with a
// multiplier on the update.  Everything is float32 but y (float or the compute
// type) and r (the compute type).
#include "common.cuh"
#include <math.h>

namespace {
constexpr int kMaxCopies = 8;

struct Coefficients {
    float mix[kMaxCopies * kMaxCopies];   // [from][to]
    float out[kMaxCopies];
    float in[kMaxCopies];
};

template <typename TY, typename TR>
__global__ void __launch_bounds__(256)
hyper_norm_kernel(float* __restrict__ copies, const float* __restrict__ seed, const TY* __restrict__ y,
                  const float* __restrict__ mix, const float* __restrict__ out_w, const float* __restrict__ in_w,
                  const float* __restrict__ norm_w, float eps, TR* __restrict__ normed,
                  const int* __restrict__ rows, int S, int H) {
    chain_release();
    chain_wait();
    extern __shared__ float smem[];
    float* us = smem;                       // [H] the row read through `in`
    float* scratch = smem + H;              // 33
    __shared__ Coefficients c;
    if (threadIdx.x < S * S) c.mix[threadIdx.x] = (y && mix) ? mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) {
        c.out[threadIdx.x] = (y && out_w) ? out_w[threadIdx.x] : 0.f;
        c.in[threadIdx.x] = in_w ? in_w[threadIdx.x] : 1.f;
    }
    __syncthreads();
    const int r = blockIdx.x;
    const int n = rows ? rows[r] : r;
    float* xrow = copies + (size_t)n * S * H;
    const bool update = y != nullptr;
    const bool write = !rows && (update || seed);
    float sq = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x[kMaxCopies];
        if (seed) {
            const float v = seed[(size_t)n * H + i];
#pragma unroll
            for (int s = 0; s < kMaxCopies; ++s) x[s] = v;
        } else {
#pragma unroll
            for (int s = 0; s < kMaxCopies; ++s) x[s] = s < S ? xrow[(size_t)s * H + i] : 0.f;
        }
        float u = 0.f;
        if (update) {
            const float yv = to_f32<TY>(y[(size_t)n * H + i]);
#pragma unroll
            for (int t = 0; t < kMaxCopies; ++t) {
                if (t >= S) break;
                float v = 0.f;
#pragma unroll
                for (int s = 0; s < kMaxCopies; ++s)
                    if (s < S) v = fmaf(c.mix[s * S + t], x[s], v);
                v = fmaf(c.out[t], yv, v);
                if (write) xrow[(size_t)t * H + i] = v;
                u = fmaf(c.in[t], v, u);
            }
        } else {
#pragma unroll
            for (int t = 0; t < kMaxCopies; ++t) {
                if (t >= S) break;
                if (write) xrow[(size_t)t * H + i] = x[t];
                u = fmaf(c.in[t], x[t], u);
            }
        }
        us[i] = u;
        sq = fmaf(u, u, sq);
    }
    const float total = block_sum(sq, scratch);
    const float inv = 1.0f / sqrtf(total / (float)H + eps);
    TR* dst = normed + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = from_f32<TR>(us[i] * inv * norm_w[i]);
}

template <typename TY, typename TR>
int launch(float* copies, const float* seed, const void* y, const float* mix, const float* out_w, const float* in_w,
           const float* norm_w, float eps, void* normed, const int* rows, int R, int S, int H, cudaStream_t stream) {
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    auto kernel = hyper_norm_kernel<TY, TR>;
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) return kErrUnsupported;
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_chained(kernel, dim3(R), dim3(H >= 1024 ? 256 : 128), smem, stream, copies, seed, (const TY*)y, mix, out_w,
                          in_w, norm_w, eps, (TR*)normed, rows, S, H);
}
}  // namespace

// dtype: the type of `normed` (0 float, 1 bfloat16); y_f32: y is float whatever dtype says.
GTG_API int gtg_hyper_norm(int dtype, int y_f32, float* copies, const float* seed, const void* y, const float* mix,
                           const float* out_w, const float* in_w, const float* norm_w, float eps, void* normed,
                           const int* rows, int R, int S, int H, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (S <= 0 || H <= 0 || !copies || !norm_w || !normed) return kErrBadArgument;
    if (S > kMaxCopies) return kErrUnsupported;
    if (dtype == 0) return launch<float, float>(copies, seed, y, mix, out_w, in_w, norm_w, eps, normed, rows, R, S, H, stream);
    if (dtype == 1 && y_f32) return launch<float, bf16>(copies, seed, y, mix, out_w, in_w, norm_w, eps, normed, rows, R, S, H, stream);
    if (dtype == 1) return launch<bf16, bf16>(copies, seed, y, mix, out_w, in_w, norm_w, eps, normed, rows, R, S, H, stream);
    return kErrBadArgument;
}
