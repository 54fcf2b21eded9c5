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

// V channels of a row at once (V = 4 where H and the pointers allow 16-byte accesses, else 1)
template <int V> struct Chan { float v[V]; };
template <int V> __device__ __forceinline__ Chan<V> load_f32(const float* p) {
    Chan<V> c;
    if constexpr (V == 4) { const float4 t = *reinterpret_cast<const float4*>(p); c.v[0] = t.x; c.v[1] = t.y; c.v[2] = t.z; c.v[3] = t.w; }
    else c.v[0] = *p;
    return c;
}
template <int V> __device__ __forceinline__ Chan<V> load_any(const float* p) { return load_f32<V>(p); }
template <int V> __device__ __forceinline__ Chan<V> load_any(const bf16* p) {
    Chan<V> c;
    if constexpr (V == 4) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
        c.v[0] = a.x; c.v[1] = a.y; c.v[2] = b.x; c.v[3] = b.y;
    } else c.v[0] = __bfloat162float(*p);
    return c;
}
template <int V> __device__ __forceinline__ void store_any(float* p, const Chan<V>& c) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(c.v[0], c.v[1], c.v[2], c.v[3]);
    else *p = c.v[0];
}
template <int V> __device__ __forceinline__ void store_any(bf16* p, const Chan<V>& c) {
    if constexpr (V == 4) {
        uint2 t;
        *reinterpret_cast<__nv_bfloat162*>(&t.x) = __floats2bfloat162_rn(c.v[0], c.v[1]);
        *reinterpret_cast<__nv_bfloat162*>(&t.y) = __floats2bfloat162_rn(c.v[2], c.v[3]);
        *reinterpret_cast<uint2*>(p) = t;
    } else *p = __float2bfloat16_rn(c.v[0]);
}

// SC: the number of copies when it is 1, 2, 3 or 4 (the loops then unroll to straight code), else 0.
template <typename TY, typename TR, int V, int SC>
__global__ void __launch_bounds__(256)
hyper_norm_kernel(float* __restrict__ copies, const float* __restrict__ seed, const TY* __restrict__ y,
                  const float* __restrict__ mix, const float* __restrict__ out_w, const float* __restrict__ in_w,
                  const float* __restrict__ norm_w, float eps, TR* __restrict__ normed,
                  const int* __restrict__ rows, int S_any, int H) {
    chain_release();
    chain_wait();
    constexpr int kCopies = SC > 0 ? SC : kMaxCopies;
    const int S = SC > 0 ? SC : S_any;
    extern __shared__ __align__(16) float smem[];
    float* us = smem;                       // [H] the row read through `in`
    float* scratch = smem + ((H + 3) & ~3); // 33
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
    for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
        Chan<V> x[kCopies];
        if (seed) {
            const Chan<V> v = load_f32<V>(seed + (size_t)n * H + i);
#pragma unroll
            for (int s = 0; s < kCopies; ++s) x[s] = v;
        } else {
#pragma unroll
            for (int s = 0; s < kCopies; ++s) {
                if (s < S) x[s] = load_f32<V>(xrow + (size_t)s * H + i);
                else {
#pragma unroll
                    for (int e = 0; e < V; ++e) x[s].v[e] = 0.f;
                }
            }
        }
        Chan<V> u;
#pragma unroll
        for (int e = 0; e < V; ++e) u.v[e] = 0.f;
        if (update) {
            const Chan<V> yv = load_any<V>(y + (size_t)n * H + i);
#pragma unroll
            for (int t = 0; t < kCopies; ++t) {
                if (t >= S) break;
                Chan<V> v;
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    float a = 0.f;
#pragma unroll
                    for (int s = 0; s < kCopies; ++s)
                        if (s < S) a = fmaf(c.mix[s * S + t], x[s].v[e], a);
                    a = fmaf(c.out[t], yv.v[e], a);
                    v.v[e] = a;
                    u.v[e] = fmaf(c.in[t], a, u.v[e]);
                }
                if (write) store_any<V>(xrow + (size_t)t * H + i, v);
            }
        } else {
#pragma unroll
            for (int t = 0; t < kCopies; ++t) {
                if (t >= S) break;
                if (write) store_any<V>(xrow + (size_t)t * H + i, x[t]);
#pragma unroll
                for (int e = 0; e < V; ++e) u.v[e] = fmaf(c.in[t], x[t].v[e], u.v[e]);
            }
        }
        store_any<V>(us + i, u);
#pragma unroll
        for (int e = 0; e < V; ++e) sq = fmaf(u.v[e], u.v[e], sq);
    }
    const float total = block_sum(sq, scratch);
    const float inv = 1.0f / sqrtf(total / (float)H + eps);
    TR* dst = normed + (size_t)r * H;
    for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
        const Chan<V> a = load_f32<V>(us + i), w = load_f32<V>(norm_w + i);
        Chan<V> o;
#pragma unroll
        for (int e = 0; e < V; ++e) o.v[e] = a.v[e] * inv * w.v[e];
        store_any<V>(dst + i, o);
    }
}

template <typename TY, typename TR, int V, int SC>
int launch_as(float* copies, const float* seed, const void* y, const float* mix, const float* out_w, const float* in_w,
              const float* norm_w, float eps, void* normed, const int* rows, int R, int S, int H, cudaStream_t stream) {
    const size_t smem = (size_t)(((H + 3) & ~3) + 33) * sizeof(float);
    auto kernel = hyper_norm_kernel<TY, TR, V, SC>;
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) return kErrUnsupported;
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int per = H / V;                    // accesses a row
    const int threads = per >= 1024 ? 256 : per >= 256 ? 128 : 64;
    return launch_chained(kernel, dim3(R), dim3(threads), smem, stream, copies, seed, (const TY*)y, mix, out_w,
                          in_w, norm_w, eps, (TR*)normed, rows, S, H);
}

template <typename TY, typename TR>
int launch(float* copies, const float* seed, const void* y, const float* mix, const float* out_w, const float* in_w,
           const float* norm_w, float eps, void* normed, const int* rows, int R, int S, int H, cudaStream_t stream) {
    auto aligned = [](const void* p, size_t a) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) % a) == 0; };
    const bool wide = H % 4 == 0 && aligned(copies, 16) && aligned(seed, 16) && aligned(y, 4 * sizeof(TY)) &&
                      aligned(norm_w, 16) && aligned(normed, 4 * sizeof(TR));
#define GTG_HYPER(V, SC) return launch_as<TY, TR, V, SC>(copies, seed, y, mix, out_w, in_w, norm_w, eps, normed, rows, R, S, H, stream)
    if (wide) {                               // more than four copies at four channels each would not fit the registers
        switch (S) { case 1: GTG_HYPER(4, 1); case 2: GTG_HYPER(4, 2); case 3: GTG_HYPER(4, 3); case 4: GTG_HYPER(4, 4); default: break; }
    }
    GTG_HYPER(1, 0);
#undef GTG_HYPER
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
