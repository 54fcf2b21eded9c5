// A mixture of experts: routing, the ordering of a step's (token, expert) pairs
// by expert, products over the ordered rows, and the weighted sum that brings a
// token's experts together again.  Nothing here talks to the host: a step with
// experts can be recorded as a graph.
//
//   route    z = R x + b in float; the `top` largest z (ties: the lower index)
//            are the token's experts, their weights softmax over those z alone
//            (scoring 0) or each chosen expert's own sigmoid(z), not renormalised
//            (scoring 1; the largest sigmoid is the largest z).
//   arrange  item i = (token i / top, its (i % top)-th expert).  Items of one
//            expert get consecutive rows, every expert's stretch padded to whole
//            tiles of `tile` rows, so that a tile of rows has one expert:
//            row_item[row] = item or -1, item_row[item] = row, tile_expert[tile]
//            = expert or -1 past the last tile.  Which of an expert's rows an
//            item gets is arbitrary; no result depends on it, since every row is
//            computed by itself.
//   product  C[row,:] = A[source(row),:] . W[expert(row)]^T, tiles of 64 rows,
//            one accumulator per output walking k in order.
//   gather   G[row,:] = x[token of row_item[row],:] (zeros for padding): the arranged
//            copy of the inputs that a product fed by tensor copies reads.  With
//            weights, G[row,:] = weight[item] * x[token,:], the product in float and
//            rounded once: a mixture whose weights scale an expert's input.
//   combine  out[t,:] = sum_k weight[t,k] * Y[item_row[t*top+k],:], k in order
//            (weights null: the plain sum).
#include "common.cuh"
#include <math.h>

namespace {
// ---- route ----------------------------------------------------------------------
// One block of eight warps per TB tokens: the tokens' rows are staged in shared memory as
// they are, every warp takes every eighth expert (lanes striding over the channels, the
// router's rows read coalesced, each value read once for all TB tokens; products and sums
// in float), and one thread a token picks from the logits.  A token's sums are added in the
// same order whatever TB is.
__device__ __forceinline__ float4 four_channels(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 four_channels(const bf16* p) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T, int TB>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ router, const float* __restrict__ bias,
                 int* __restrict__ chosen, float* __restrict__ weights, int N, int H, int E, int top, int scoring) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) unsigned char route_smem[];
    constexpr int kPer16 = 16 / (int)sizeof(T);          // channels in 16 bytes
    const int Hp = (H + kPer16 - 1) / kPer16 * kPer16;   // a staged row, whole 16 bytes
    T* xs = reinterpret_cast<T*>(route_smem);            // [TB][Hp]
    float* zs = reinterpret_cast<float*>(route_smem + (size_t)TB * Hp * sizeof(T));   // [TB][2 E]: logits, then the chosen scores
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TB;
    const int nt = min(TB, N - n0);
    const bool wide_rows = H % kPer16 == 0 && ldx % kPer16 == 0 && (reinterpret_cast<uintptr_t>(x) % 16) == 0;
#pragma unroll
    for (int t = 0; t < TB; ++t) {
        const T* xr = x + (size_t)(n0 + t) * ldx;
        T* dst = xs + (size_t)t * Hp;
        if (t >= nt) {
            for (int i = threadIdx.x; i < Hp; i += blockDim.x) dst[i] = from_f32<T>(0.f);
        } else if (wide_rows) {
            for (int i = threadIdx.x; i < H / kPer16; i += blockDim.x)
                reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(xr)[i];
        } else {
            for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = xr[i];
        }
    }
    __syncthreads();
    const int n_warps = blockDim.x >> 5;
    for (int e = warp; e < E; e += n_warps) {
        // a warp an expert: two chains over alternate steps, four channels a lane and step where the row allows it,
        // the loads of several steps in flight together
        const float* r = router + (size_t)e * H;
        float s0[TB], s1[TB];
#pragma unroll
        for (int t = 0; t < TB; ++t) s0[t] = s1[t] = 0.f;
        if (H % 256 == 0 && (reinterpret_cast<uintptr_t>(router) % 16) == 0) {
#pragma unroll 4
            for (int i = lane * 4; i < H; i += 256) {
                const float4 a = *reinterpret_cast<const float4*>(r + i), b = *reinterpret_cast<const float4*>(r + i + 128);
#pragma unroll
                for (int t = 0; t < TB; ++t) {
                    const float4 v0 = four_channels(xs + (size_t)t * Hp + i), v1 = four_channels(xs + (size_t)t * Hp + i + 128);
                    s0[t] = fmaf(v0.x, a.x, s0[t]); s0[t] = fmaf(v0.y, a.y, s0[t]); s0[t] = fmaf(v0.z, a.z, s0[t]); s0[t] = fmaf(v0.w, a.w, s0[t]);
                    s1[t] = fmaf(v1.x, b.x, s1[t]); s1[t] = fmaf(v1.y, b.y, s1[t]); s1[t] = fmaf(v1.z, b.z, s1[t]); s1[t] = fmaf(v1.w, b.w, s1[t]);
                }
            }
        } else {
            for (int i = lane; i < H; i += 32) {
                const float rv = r[i];
#pragma unroll
                for (int t = 0; t < TB; ++t) s0[t] = fmaf(to_f32<T>(xs[(size_t)t * Hp + i]), rv, s0[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < TB; ++t) {
            const float sum = warp_sum(s0[t] + s1[t]);
            if (lane == 0) zs[t * 2 * E + e] = sum + (bias ? bias[e] : 0.f);
        }
    }
    __syncthreads();
    if (threadIdx.x < nt) {
        const int n = n0 + threadIdx.x;
        float* z = zs + threadIdx.x * 2 * E;
        float* kept = z + E;
        // top <= E rounds of a first-maximum search; a chosen logit becomes NaN, which no comparison picks again
        float best0 = 0.f, total = 0.f;
        for (int k = 0; k < top; ++k) {
            int arg = -1;
            float best = -INFINITY;
            for (int e = 0; e < E; ++e) {
                const float v = z[e];
                if (v != v) continue;                       // chosen in an earlier round
                if (arg < 0 || v > best) { best = v; arg = e; }
            }
            z[arg] = __int_as_float(0x7fc00000);
            if (k == 0) best0 = best;
            chosen[(size_t)n * top + k] = arg;
            const float p = scoring == 1 ? 1.0f / (1.0f + expf(-best)) : expf(best - best0);
            kept[k] = p;
            total += p;
        }
        const float inv = scoring == 1 ? 1.0f : 1.0f / total;
        for (int k = 0; k < top; ++k) weights[(size_t)n * top + k] = kept[k] * inv;
    }
}

// ---- arrange --------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_arrange_kernel(const int* __restrict__ chosen, int n_items, int E, int tile, int n_tiles_cap,
                   int* __restrict__ row_item, int* __restrict__ item_row, int* __restrict__ tile_expert) {
    chain_release();
    chain_wait();
    extern __shared__ int ism[];
    int* count = ism;            // [E]
    int* first = ism + E;        // [E] first row of the expert's stretch
    int* cursor = ism + 2 * E;   // [E]
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = cursor[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_items; i += blockDim.x) atomicAdd(&count[chosen[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int e = 0; e < E; ++e) {
            first[e] = t * tile;
            const int tiles = (count[e] + tile - 1) / tile;
            for (int j = 0; j < tiles; ++j) tile_expert[t + j] = e;
            t += tiles;
        }
        for (; t < n_tiles_cap; ++t) tile_expert[t] = -1;
    }
    for (int r = threadIdx.x; r < n_tiles_cap * tile; r += blockDim.x) row_item[r] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
        const int e = chosen[i];
        const int row = first[e] + atomicAdd(&cursor[e], 1);
        row_item[row] = i;
        item_row[i] = row;
    }
}

// ---- product over arranged rows ---------------------------------------------------
constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
grouped_simt_kernel(const TA* __restrict__ A, int lda, const int* __restrict__ row_item, int item_div,
                    const TW* __restrict__ W, int ldw, long long expert_stride, const int* __restrict__ tile_expert,
                    TC* __restrict__ C, int ldc, int N, int K) {
    chain_release();
    chain_wait();
    const int expert = tile_expert[blockIdx.y];
    if (expert < 0) return;
    W += (size_t)expert * expert_stride;
    __shared__ float As[BK][BM + PAD];
    __shared__ float Ws[BK][BN + PAD];
    __shared__ int src[BM];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    if (tid < BM) {
        const int item = row_item[m0 + tid];
        // item_div > 0: the row's source is its item's token (item / item_div); 0: the row itself
        src[tid] = item < 0 ? -1 : item_div > 0 ? item / item_div : m0 + tid;
    }
    __syncthreads();
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    const int arow = src[lrow];
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int wn = n0 + lrow;
            As[lk + j][lrow] = (arow >= 0 && k < K) ? to_f32<TA>(A[(size_t)arow * lda + k]) : 0.f;
            Ws[lk + j][lrow] = (wn < N && k < K) ? to_f32<TW>(W[(size_t)wn * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (src[ty * 4 + i] < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
        }
    }
}

// ---- gather -------------------------------------------------------------------------
__global__ void moe_gather_kernel(const bf16* __restrict__ x, int ldx, const int* __restrict__ row_item, int item_div,
                                  bf16* __restrict__ out, int H8) {
    chain_release();
    chain_wait();
    const int item = row_item[blockIdx.x];
    const uint4* src = item < 0 ? nullptr : reinterpret_cast<const uint4*>(x + (size_t)(item / item_div) * ldx);
    uint4* dst = reinterpret_cast<uint4*>(out) + (size_t)blockIdx.x * H8;
    for (int i = threadIdx.x; i < H8; i += blockDim.x) dst[i] = src ? src[i] : make_uint4(0u, 0u, 0u, 0u);
}

// The same with a weight per item, any type and width: G[row,:] = weights[item] * x[token,:].
template <typename T>
__global__ void moe_gather_scaled_kernel(const T* __restrict__ x, int ldx, const int* __restrict__ row_item, int item_div,
                                         const float* __restrict__ weights, T* __restrict__ out, int H) {
    chain_release();
    chain_wait();
    const int item = row_item[blockIdx.x];
    T* dst = out + (size_t)blockIdx.x * H;
    if (item < 0) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = from_f32<T>(0.f);
        return;
    }
    const float w = weights ? weights[item] : 1.0f;
    const T* src = x + (size_t)(item / item_div) * ldx;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = from_f32<T>(w * to_f32<T>(src[i]));
}

// bfloat16 rows of a multiple of 8 channels, 16 bytes an access: each channel is widened, multiplied
// in float and rounded once, as in the kernel above.
__global__ void moe_gather_scaled_wide_kernel(const bf16* __restrict__ x, int ldx, const int* __restrict__ row_item, int item_div,
                                              const float* __restrict__ weights, bf16* __restrict__ out, int H8) {
    chain_release();
    chain_wait();
    const int item = row_item[blockIdx.x];
    uint4* dst = reinterpret_cast<uint4*>(out) + (size_t)blockIdx.x * H8;
    if (item < 0) {
        for (int i = threadIdx.x; i < H8; i += blockDim.x) dst[i] = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const float w = weights ? weights[item] : 1.0f;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(item / item_div) * ldx);
    for (int i = threadIdx.x; i < H8; i += blockDim.x) {
        uint4 t = src[i];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            h[e] = __floats2bfloat162_rn(w * f.x, w * f.y);
        }
        dst[i] = t;
    }
}

// ---- combine ----------------------------------------------------------------------
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, int ldy, const int* __restrict__ item_row,
                                   const float* __restrict__ weights, T* __restrict__ out, int H, int top) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k)
            s = fmaf(weights ? weights[(size_t)t * top + k] : 1.0f, y[(size_t)item_row[(size_t)t * top + k] * ldy + i], s);
        out[(size_t)t * H + i] = from_f32<T>(s);
    }
}
}  // namespace

GTG_API int gtg_moe_route(int dtype, const void* x, int ldx, const float* router, const float* bias, int* chosen,
                          float* weights, int N, int H, int E, int top, int scoring, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || H <= 0 || scoring < 0 || scoring > 1) return kErrBadArgument;
    // many tokens: four share a block, so that the router is read a quarter as often
    const size_t elem = dtype == 0 ? 4 : 2;
    const size_t row = ((size_t)H * elem + 15) / 16 * 16;
    const int tb = (N >= 1024 && 4 * (row + 2 * (size_t)E * sizeof(float)) <= 64 * 1024) ? 4 : 1;
    const size_t smem = tb * (row + 2 * (size_t)E * sizeof(float));
    if (smem > 160 * 1024) return kErrUnsupported;
    const dim3 grid((N + tb - 1) / tb);
#define GTG_ROUTE(T, TB)                                                                                           \
    do {                                                                                                           \
        auto kernel = moe_route_kernel<T, TB>;                                                                     \
        if (smem > 48 * 1024) {                                                                                    \
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                   \
        }                                                                                                          \
        return launch_chained(kernel, grid, dim3(256), smem, stream, (const T*)x, ldx, router, bias, chosen, weights, \
                              N, H, E, top, scoring);                                                              \
    } while (0)
    if (dtype == 0) { if (tb == 4) GTG_ROUTE(float, 4); else GTG_ROUTE(float, 1); }
    if (dtype == 1) { if (tb == 4) GTG_ROUTE(bf16, 4); else GTG_ROUTE(bf16, 1); }
#undef GTG_ROUTE
    return kErrBadArgument;
}

// Rows the arranged order may need at most: every expert's stretch rounded up to whole tiles.
GTG_API int gtg_moe_tiles_cap(int n_items, int E, int tile) {
    return (n_items + tile - 1) / tile + E;
}

GTG_API int gtg_moe_arrange(const int* chosen, int n_items, int E, int tile, int n_tiles_cap, int* row_item,
                            int* item_row, int* tile_expert, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (E <= 0 || tile <= 0 || n_tiles_cap < gtg_moe_tiles_cap(n_items, E, tile)) return kErrBadArgument;
    const size_t smem = (size_t)3 * E * sizeof(int);
    if (smem > 48 * 1024) return kErrUnsupported;
    return launch_chained(moe_arrange_kernel, dim3(1), dim3(1024), smem, stream, chosen, n_items, E, tile, n_tiles_cap,
                          row_item, item_row, tile_expert);
}

// C[row,:] = A[source(row),:] . W[expert of the row's tile]^T over tiles of 64 arranged rows.
// item_div > 0: source(row) = row_item[row] / item_div (the item's token); 0: the row itself.
// dtype 0: float operands; 1: bfloat16 operands.  c_f32: float result, else the operands' type.
GTG_API int gtg_moe_product_simt(int dtype, int c_f32, const void* A, int lda, const int* row_item, int item_div,
                                 const void* W, int ldw, long long expert_stride, const int* tile_expert,
                                 int n_tiles_cap, void* C, int ldc, int N, int K, cudaStream_t stream) {
    if (n_tiles_cap <= 0 || N <= 0) return 0;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return kErrBadArgument;
    const dim3 grid((N + BN - 1) / BN, n_tiles_cap);
    if (grid.y > 65535) return kErrUnsupported;
    if (dtype == 0 && c_f32)
        return launch_chained(grouped_simt_kernel<float, float, float>, grid, dim3(256), 0, stream, (const float*)A, lda, row_item,
                              item_div, (const float*)W, ldw, expert_stride, tile_expert, (float*)C, ldc, N, K);
    if (dtype == 1 && c_f32)
        return launch_chained(grouped_simt_kernel<bf16, bf16, float>, grid, dim3(256), 0, stream, (const bf16*)A, lda, row_item,
                              item_div, (const bf16*)W, ldw, expert_stride, tile_expert, (float*)C, ldc, N, K);
    if (dtype == 1)
        return launch_chained(grouped_simt_kernel<bf16, bf16, bf16>, grid, dim3(256), 0, stream, (const bf16*)A, lda, row_item,
                              item_div, (const bf16*)W, ldw, expert_stride, tile_expert, (bf16*)C, ldc, N, K);
    return kErrBadArgument;
}

// out[row, :] = x[row_item[row] / item_div, :], zeros where row_item[row] < 0 (bfloat16 rows of a multiple of 8 channels).
GTG_API int gtg_moe_gather(const void* x, int ldx, const int* row_item, int item_div, void* out, int rows, int H,
                           cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H <= 0 || item_div <= 0) return kErrBadArgument;
    if (H % 8 || ldx % 8 || ((uintptr_t)x % 16) || ((uintptr_t)out % 16)) return kErrUnsupported;
    return launch_chained(moe_gather_kernel, dim3(rows), dim3(128), 0, stream, (const bf16*)x, ldx, row_item, item_div, (bf16*)out, H / 8);
}

// out[row, :] = weights[item] * x[item / item_div, :] (weights null: 1), zeros in padding rows; any width.
GTG_API int gtg_moe_gather_scaled(int dtype, const void* x, int ldx, const int* row_item, int item_div, const float* weights,
                                  void* out, int rows, int H, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H <= 0 || item_div <= 0) return kErrBadArgument;
    if (dtype == 0) return launch_chained(moe_gather_scaled_kernel<float>, dim3(rows), dim3(128), 0, stream, (const float*)x, ldx, row_item, item_div, weights, (float*)out, H);
    if (dtype == 1 && H % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)out % 16) == 0)
        return launch_chained(moe_gather_scaled_wide_kernel, dim3(rows), dim3(128), 0, stream, (const bf16*)x, ldx, row_item, item_div, weights, (bf16*)out, H / 8);
    if (dtype == 1) return launch_chained(moe_gather_scaled_kernel<bf16>, dim3(rows), dim3(128), 0, stream, (const bf16*)x, ldx, row_item, item_div, weights, (bf16*)out, H);
    return kErrBadArgument;
}

GTG_API int gtg_moe_combine(int dtype, const float* y, int ldy, const int* item_row, const float* weights, void* out,
                            int N, int H, int top, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || top <= 0) return kErrBadArgument;
    if (dtype == 0) return launch_chained(moe_combine_kernel<float>, dim3(N), dim3(256), 0, stream, y, ldy, item_row, weights, (float*)out, H, top);
    if (dtype == 1) return launch_chained(moe_combine_kernel<bf16>, dim3(N), dim3(256), 0, stream, y, ldy, item_row, weights, (bf16*)out, H, top);
    return kErrBadArgument;
}
