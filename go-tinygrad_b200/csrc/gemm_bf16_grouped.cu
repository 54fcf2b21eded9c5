// Many bfloat16 products of one shape in one launch, on the warp-level tensor-core
// path (cp.async stages, ldmatrix, mma.sync.m16n8k16, float accumulation):
//
//   batched   C_b[M,N] = A_b[M,K] . W_b[N,K]^T for b < batch (blockIdx.z), operand b
//             starting batch_* elements after operand b-1: the per-head products of a
//             mixer, whose heads lie side by side in wider rows;
//   arranged  C[row,:] = A[source(row),:] . W_e[N,K]^T where tiles of BM rows share
//             one weight matrix e = tile_expert[tile] (-1: no such tile): routed
//             experts.  source(row) = row_item[row] / item_div (the token of a
//             (token, expert) pair) or the row itself; rows whose item is -1 are
//             padding: they read zeros and write nothing.
//
// Epilogues, applied to the float sums: 0 none; 1 gated silu, W's rows alternating
// in blocks of 8 gate and 8 up features, C[:, N/2] = silu(gate) * up; 2 C = sum *
// sigmoid(G) with G laid out like C (a gate on a mixer's heads).
// K, the row strides and the batch strides of A and W are multiples of 8 elements
// and A, W are 16-byte aligned.
#include "mma_helpers.cuh"

namespace {
constexpr int BN = 128;
// BK, the channels of k a stage holds, is 32 or 64: arranged rows of few tokens an expert (decode steps) are all
// weight streaming, and stages of 64 channels ask for a weight row's bytes a whole 128-byte line at a time.
constexpr int kThreads = 256;

template <typename OutT>
__device__ __forceinline__ void put(OutT* p, float v);
template <> __device__ __forceinline__ void put<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void put<float>(float* p, float v) { *p = v; }
// two neighbouring columns at once (the address is a multiple of two elements)
template <typename OutT>
__device__ __forceinline__ void put2(OutT* p, float v0, float v1);
template <> __device__ __forceinline__ void put2<bf16>(bf16* p, float v0, float v1) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v0, v1);
}
template <> __device__ __forceinline__ void put2<float>(float* p, float v0, float v1) {
    *reinterpret_cast<float2*>(p) = make_float2(v0, v1);
}

template <int BM, int BK, int STAGES, typename OutT>
__global__ void __launch_bounds__(kThreads)
grouped_mma_kernel(const bf16* __restrict__ A, int lda, long long batch_a, const int* __restrict__ row_item, int item_div,
                   const bf16* __restrict__ W, int ldw, long long batch_w, const int* __restrict__ tile_expert,
                   OutT* __restrict__ C, int ldc, long long batch_c, int M, int N, int K, int epilogue,
                   const bf16* __restrict__ G, int ldg, long long batch_g) {
    chain_release();
    chain_wait();
    constexpr int MI = BM / 32;                        // 16-row fragments per warp (2 x 4 warps)
    constexpr int kStageBytes = (BM + BN) * BK * 2;
    constexpr int CPR = BK / 8;                        // 16-byte chunks per staged row
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int src[BM];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp >> 2, wn = warp & 3;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    if (tile_expert) {
        const int expert = tile_expert[blockIdx.y];
        if (expert < 0) return;
        W += (size_t)expert * batch_w;
    } else {
        A += (size_t)blockIdx.z * batch_a;
        W += (size_t)blockIdx.z * batch_w;
        C += (size_t)blockIdx.z * batch_c;
        if (G) G += (size_t)blockIdx.z * batch_g;
    }
    if (tid < BM) {
        const int m = m0 + tid;
        int s = m < M ? m : -1;
        if (row_item && s >= 0) {
            const int item = row_item[m];
            s = item < 0 ? -1 : item_div > 0 ? item / item_div : m;
        }
        src[tid] = s;
    }
    __syncthreads();
    const uint32_t smem_base = smem_u32(smem);
    const int nk = (K + BK - 1) / BK;

    auto load_stage = [&](int stage, int kt) {
        const uint32_t a_base = smem_base + stage * kStageBytes;
        const uint32_t w_base = a_base + BM * BK * 2;
        const int k0 = kt * BK;
#pragma unroll
        for (int i = 0; i < BM * CPR / kThreads; ++i) {
            const int id = tid + i * kThreads;
            const int r = id / CPR, c = id % CPR;
            const int k = k0 + c * 8;
            const int s = src[r];
            const bool ok = s >= 0 && k < K;
            cp_async16(a_base + swz_offset<BK>(r, c), ok ? A + (size_t)s * lda + k : A, ok ? 16 : 0);
        }
#pragma unroll
        for (int i = 0; i < BN * CPR / kThreads; ++i) {
            const int id = tid + i * kThreads;
            const int r = id / CPR, c = id % CPR;
            const int k = k0 + c * 8;
            const int n = n0 + r;
            const bool ok = n < N && k < K;
            cp_async16(w_base + swz_offset<BK>(r, c), ok ? W + (size_t)n * ldw + k : W, ok ? 16 : 0);
        }
    };

    // A 16-row fragment none of whose rows exists (the padding of an expert's last tile; nearly all of a tile in a
    // decode step) is neither read nor multiplied: its sums would not be written.  Warp-uniform.
    bool live[MI];
    bool any_live = false;
#pragma unroll
    for (int i = 0; i < MI; ++i) {
        live[i] = false;
        const int r0 = wm * (BM / 2) + i * 16;
        for (int r = 0; r < 16; ++r) live[i] = live[i] || src[r0 + r] >= 0;
        any_live = any_live || live[i];
    }

    float acc[MI][4][4];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < nk) load_stage(s, s);
        cp_async_commit();
    }
    for (int kt = 0; kt < nk; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            const int nxt = kt + STAGES - 1;
            if (nxt < nk) load_stage(nxt % STAGES, nxt);
            cp_async_commit();
        }
        const uint32_t a_base = smem_base + (kt % STAGES) * kStageBytes;
        const uint32_t w_base = a_base + BM * BK * 2;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            if (!any_live) break;
            uint32_t af[MI][4];
#pragma unroll
            for (int i = 0; i < MI; ++i) {
                if (!live[i]) continue;
                const int r = wm * (BM / 2) + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int c = kk * 2 + (lane >> 4);
                ldmatrix_x4(af[i][0], af[i][1], af[i][2], af[i][3], a_base + swz_offset<BK>(r, c));
            }
            uint32_t bfr[4][2];
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int r = wn * 32 + jj * 16 + (lane & 7) + (lane >> 4) * 8;
                const int c = kk * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(bfr[jj * 2][0], bfr[jj * 2][1], bfr[jj * 2 + 1][0], bfr[jj * 2 + 1][1],
                            w_base + swz_offset<BK>(r, c));
            }
#pragma unroll
            for (int i = 0; i < MI; ++i) {
                if (!live[i]) continue;
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], af[i], bfr[j][0], bfr[j][1]);
            }
        }
    }
    cp_async_wait<0>();

    const int g = lane >> 2, t = lane & 3;
    // pairs of columns go out in one access where every pair's address is aligned
    const bool pairs = (ldc % 2 == 0) && (batch_c % 2 == 0) && ((reinterpret_cast<uintptr_t>(C) % (2 * sizeof(OutT))) == 0) &&
                       (epilogue != 2 || ((ldg % 2 == 0) && (batch_g % 2 == 0) && (reinterpret_cast<uintptr_t>(G) % 4) == 0));
#pragma unroll
    for (int i = 0; i < MI; ++i) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm * (BM / 2) + i * 16 + g + half * 8;
            if (src[r] < 0) continue;
            const size_t m = (size_t)(m0 + r);
            if (epilogue == 1) {
#pragma unroll
                for (int j = 0; j < 4; j += 2) {
                    const int n = n0 + wn * 32 + j * 8;              // a block of 8 gate rows, then their 8 up rows
                    if (pairs && n + 16 <= N) {
                        const float g0 = acc[i][j][half * 2], g1 = acc[i][j][half * 2 + 1];
                        put2<OutT>(C + m * ldc + n / 2 + t * 2, g0 / (1.0f + expf(-g0)) * acc[i][j + 1][half * 2],
                                   g1 / (1.0f + expf(-g1)) * acc[i][j + 1][half * 2 + 1]);
                        continue;
                    }
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int col = n / 2 + t * 2 + e;
                        if (n + 8 + t * 2 + e < N) {
                            const float gate = acc[i][j][half * 2 + e], up = acc[i][j + 1][half * 2 + e];
                            put<OutT>(C + m * ldc + col, gate / (1.0f + expf(-gate)) * up);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int n2 = n0 + wn * 32 + j * 8 + t * 2;
                    if (pairs && n2 + 1 < N) {
                        float v0 = acc[i][j][half * 2], v1 = acc[i][j][half * 2 + 1];
                        if (epilogue >= kEpiActivation) { v0 = activate(v0, epilogue - kEpiActivation); v1 = activate(v1, epilogue - kEpiActivation); }
                        if (epilogue == 2) {
                            const float2 gg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(G + m * ldg + n2));
                            v0 *= 1.0f / (1.0f + expf(-gg.x));
                            v1 *= 1.0f / (1.0f + expf(-gg.y));
                        }
                        put2<OutT>(C + m * ldc + n2, v0, v1);
                        continue;
                    }
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int n = n0 + wn * 32 + j * 8 + t * 2 + e;
                        if (n >= N) continue;
                        float v = acc[i][j][half * 2 + e];
                        if (epilogue >= kEpiActivation) v = activate(v, epilogue - kEpiActivation);
                        if (epilogue == 2) v *= 1.0f / (1.0f + expf(-__bfloat162float(G[m * ldg + n])));
                        put<OutT>(C + m * ldc + n, v);
                    }
                }
            }
        }
    }
}

template <int BM, int BK, int STAGES, typename OutT>
int launch(const bf16* A, int lda, long long batch_a, const int* row_item, int item_div, const bf16* W, int ldw,
           long long batch_w, const int* tile_expert, OutT* C, int ldc, long long batch_c, int batch, int M, int N, int K,
           int epilogue, const bf16* G, int ldg, long long batch_g, cudaStream_t stream) {
    const int smem = STAGES * (BM + BN) * BK * 2;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(grouped_mma_kernel<BM, BK, STAGES, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batch);
    if (grid.y > 65535 || grid.z > 65535) return kErrUnsupported;
    return launch_chained(grouped_mma_kernel<BM, BK, STAGES, OutT>, grid, dim3(kThreads), (size_t)smem, stream, A, lda, batch_a, row_item,
                          item_div, W, ldw, batch_w, tile_expert, C, ldc, batch_c, M, N, K, epilogue, G, ldg, batch_g);
}
}  // namespace

// tile_rows: 64 or 128 rows of C per thread block (arranged rows: the arrangement's tile).
// tile_expert non-null: arranged rows (batch is then 1 and M the rows of the arrangement);
// null: `batch` products side by side.  out_f32: C is float, else bfloat16.
GTG_API int gtg_gemm_bf16_grouped(const void* A, int lda, long long batch_a, const int* row_item, int item_div,
                                  const void* W, int ldw, long long batch_w, const int* tile_expert, void* C, int ldc,
                                  long long batch_c, int out_f32, int batch, int M, int N, int K, int tile_rows,
                                  int epilogue, const void* G, int ldg, long long batch_g, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    if (K <= 0 || lda < K || ldw < K || epilogue < 0 || (epilogue > 2 && !(epilogue >= kEpiActivation && epilogue < kEpiActivation + kActivations)) ||
        (epilogue == 2 && !G)) return kErrBadArgument;
    if (K % 8 || lda % 8 || ldw % 8 || batch_a % 8 || batch_w % 8 || ((uintptr_t)A % 16) || ((uintptr_t)W % 16)) return kErrUnsupported;
    if (epilogue == 1 && N % 16) return kErrUnsupported;
    if (tile_expert && batch != 1) return kErrBadArgument;
#define GTG_GROUPED(BM, BK, ST, T)                                                                                  \
    return launch<BM, BK, ST, T>((const bf16*)A, lda, batch_a, row_item, item_div, (const bf16*)W, ldw, batch_w, tile_expert, \
                         (T*)C, ldc, batch_c, batch, M, N, K, epilogue, (const bf16*)G, ldg, batch_g, stream)
    if (tile_rows == 64 && tile_expert && K >= 256) {
        // Four stages (two blocks a multiprocessor, which leaves room for the first blocks of the kernel behind it)
        // up to three blocks a multiprocessor, counting the arrangement's spare tiles, which do not exist and end at
        // once; beyond that three stages (three blocks a multiprocessor).  Measured both ways at either size.
        static int n_sm = 0;
        if (n_sm == 0) {
            int dev = 0;
            if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n_sm = 1;
        }
        const long long blocks = (long long)((N + BN - 1) / BN) * ((M + 63) / 64);
        if (blocks <= 3LL * n_sm) { if (out_f32) GTG_GROUPED(64, 64, 4, float); else GTG_GROUPED(64, 64, 4, bf16); }
        if (out_f32) GTG_GROUPED(64, 64, 3, float); else GTG_GROUPED(64, 64, 3, bf16);
    }
    if (tile_rows == 64) { if (out_f32) GTG_GROUPED(64, 32, 4, float); else GTG_GROUPED(64, 32, 4, bf16); }
    if (tile_rows == 128) { if (out_f32) GTG_GROUPED(128, 32, 4, float); else GTG_GROUPED(128, 32, 4, bf16); }
#undef GTG_GROUPED
    return kErrBadArgument;
}
