// Kernels of the gated delta rule: a recurrent mixer whose per-sequence state is,
// per head, a matrix S of d x dv floats (key channels by value channels) that is
// decayed row by row and corrected towards the new value along the new key:
//
//     S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// with one decay g_t[i] in (0, 1) per head and key channel, a step beta_t in (0, 1)
// per head, and q_t, k_t of a key/value group (several heads may share them).
//
// All of them serve a step of packed rows: sequence b owns rows
// cu_seqlens[b]..cu_seqlens[b+1], continues from the state kept for its cache slot
// and leaves the state for its next step; a prompt, a portion of one and a single
// token are the same case.  Everything here is float whatever the activation type:
// unit norms, decays with their softplus and exponentials, steps, the state and the
// sums of the recurrence, and the norm of the read-out.
#include "common.cuh"
#include <math.h>

namespace {
// log(1 + exp(x)) without overflow and without a cut-off
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// ------------------------------------------------------------- per-token preparation
// One block per token.  In place, on float rows:
//   * every query and key head (n_groups of each, d channels, side by side from qk):
//     x / sqrt(sum(x^2) + unit_eps); queries also times q_scale;
//   * decay[n, h, i] <- exp(-exp(a_log[h]) * softplus(decay[n, h, i] + dt_bias[h, i]));
//   * beta[n, h] <- sigmoid(beta_in[n, h]).
__global__ void __launch_bounds__(256)
delta_prepare_kernel(float* __restrict__ qk, int ld_qk, float* __restrict__ decay, int ld_decay,
                     const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                     const float* __restrict__ beta_in, int ld_beta_in, float* __restrict__ beta,
                     int n_heads, int n_groups, int d, float unit_eps, float q_scale) {
    chain_release();
    chain_wait();
    const size_t n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    for (int item = warp; item < 2 * n_groups; item += n_warps) {
        float* x = qk + n * ld_qk + (size_t)item * d;
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) ss = fmaf(x[i], x[i], ss);
        const float inv = (item < n_groups ? q_scale : 1.0f) / sqrtf(warp_sum(ss) + unit_eps);
        for (int i = lane; i < d; i += 32) x[i] *= inv;
    }
    float* g = decay + n * ld_decay;
    for (int c = threadIdx.x; c < n_heads * d; c += blockDim.x) {
        const float rate = expf(a_log[c / d]);
        g[c] = expf(-rate * softplus_f(g[c] + dt_bias[c]));
    }
    for (int h = threadIdx.x; h < n_heads; h += blockDim.x)
        beta[n * n_heads + h] = 1.0f / (1.0f + expf(-beta_in[n * ld_beta_in + h]));
}

// ------------------------------------------------------------ the recurrence
// The columns of S never meet: column j is a recurrence of its own over d numbers,
//     r1 = sum_i g_i S_ij k_i,  r2 = sum_i g_i S_ij q_i,  u_j = beta (v_j - r1),
//     S_ij <- g_i S_ij + k_i u_j,  o_j = r2 + u_j (k . q)
// (o = S^T q over the new S, written out so that both sums run over the old one and
// meet in one exchange).  One block serves (head, a slice of kColsPerBlock columns,
// sequence).  R threads share a column: thread (r, j) owns rows r, r + R, ... (up to
// kRows of them); their partial sums meet by shuffles.  q, k, g, v and beta of a tile
// of tokens at a time are staged in shared memory.  Tokens are walked strictly in
// order: the result does not depend on the cut of the sequence into steps, on the
// batch or on the slices.
constexpr int kRows = 16;          // rows of S a thread owns at most
constexpr int kScanThreads = 128;
constexpr int kTile = 16;          // tokens staged at a time

__device__ __forceinline__ void copy_async_4(void* smem_dst, const void* gmem_src) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void copy_async_16(void* smem_dst, const void* gmem_src) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// The tiles arrive one ahead of the arithmetic by asynchronous copies into two buffers that take
// turns (`wide`: rows and addresses allow 16-byte copies of q, k and g; else 4-byte ones).
__global__ void __launch_bounds__(kScanThreads)
delta_scan_kernel(const float* __restrict__ qk, int ld_qk, const float* __restrict__ v, int ld_v,
                  const float* __restrict__ decay, int ld_decay, const float* __restrict__ beta,
                  float* __restrict__ state, float* __restrict__ out, int ld_out,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                  int n_heads, int n_groups, int d, int dv, int R, int slices, int wide) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float smem[];
    const int cols = kScanThreads / R;                       // columns a block serves
    const int per_buffer = 3 * kTile * d + kTile * cols + 2 * kTile;
    const int h = blockIdx.x / slices, slice = blockIdx.x % slices;
    const int b = blockIdx.y;
    const int grp = h / (n_heads / n_groups);
    const int row0 = cu_seqlens[b], n_rows = cu_seqlens[b + 1] - row0;
    const int tid = threadIdx.x;
    const int cw = 32 / R;                                   // columns a warp serves: the R lanes of a column lie cw apart
    const int jj = (tid >> 5) * cw + (tid & 31) % cw, r = (tid & 31) / cw;
    const int j = slice * cols + jj;
    const bool col_ok = j < dv;
    float* S = state + ((size_t)slots[b] * n_heads + h) * (size_t)d * dv;
    float s[kRows];
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
        const int row = r + i * R;
        s[i] = (col_ok && row < d) ? S[(size_t)row * dv + j] : 0.f;
    }
    // a buffer: q, k, g [kTile][d] each, v [kTile][cols], beta [kTile], k . q [kTile]
    auto stage = [&](int buffer, int t0) {
        float* sq = smem + buffer * per_buffer;
        float* sk = sq + kTile * d;
        float* sg = sk + kTile * d;
        float* sv = sg + kTile * d;
        float* sb = sv + kTile * cols;
        const int nt = min(kTile, n_rows - t0);
        if (wide) {
            const int d4 = d >> 2;
            for (int idx = tid; idx < nt * d4; idx += kScanThreads) {
                const int t = idx / d4, i = (idx - t * d4) * 4;
                const size_t row = (size_t)(row0 + t0 + t);
                copy_async_16(sq + t * d + i, qk + row * ld_qk + (size_t)grp * d + i);
                copy_async_16(sk + t * d + i, qk + row * ld_qk + (size_t)(n_groups + grp) * d + i);
                copy_async_16(sg + t * d + i, decay + row * ld_decay + (size_t)h * d + i);
            }
        } else {
            for (int idx = tid; idx < nt * d; idx += kScanThreads) {
                const int t = idx / d, i = idx - t * d;
                const size_t row = (size_t)(row0 + t0 + t);
                copy_async_4(sq + t * d + i, qk + row * ld_qk + (size_t)grp * d + i);
                copy_async_4(sk + t * d + i, qk + row * ld_qk + (size_t)(n_groups + grp) * d + i);
                copy_async_4(sg + t * d + i, decay + row * ld_decay + (size_t)h * d + i);
            }
        }
        for (int idx = tid; idx < nt * cols; idx += kScanThreads) {
            const int t = idx / cols, c = idx - t * cols;
            const int col = min(slice * cols + c, dv - 1);   // a column beyond the head's last: any value, never used
            copy_async_4(sv + t * cols + c, v + (size_t)(row0 + t0 + t) * ld_v + (size_t)h * dv + col);
        }
        if (tid < nt) copy_async_4(sb + tid, beta + (size_t)(row0 + t0 + tid) * n_heads + h);
        copy_async_commit();
    };
    if (n_rows > 0) stage(0, 0);
    int buffer = 0;
    for (int t0 = 0; t0 < n_rows; t0 += kTile, buffer ^= 1) {
        const int nt = min(kTile, n_rows - t0);
        if (t0 + kTile < n_rows) {
            stage(buffer ^ 1, t0 + kTile);                   // the other buffer: its tile was used up before the barrier that ended the last pass of this loop
            copy_async_wait<1>();
        } else {
            copy_async_wait<0>();
        }
        __syncthreads();
        const float* sq = smem + buffer * per_buffer;
        const float* sk = sq + kTile * d;
        const float* sg = sk + kTile * d;
        const float* sv = sg + kTile * d;
        float* sb = const_cast<float*>(sv) + kTile * cols;
        // k . q of every token of the tile: a warp a token at a time, in a fixed order
        for (int t = tid >> 5; t < nt; t += kScanThreads / 32) {
            float kq = 0.f;
            for (int i = tid & 31; i < d; i += 32) kq = fmaf(sk[t * d + i], sq[t * d + i], kq);
            kq = warp_sum(kq);
            if ((tid & 31) == 0) sb[kTile + t] = kq;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float* kt = sk + t * d;
            const float* qt = sq + t * d;
            const float* gt = sg + t * d;
            float r1 = 0.f, r2 = 0.f;
#pragma unroll
            for (int i = 0; i < kRows; ++i) {
                const int row = r + i * R;
                if (row < d) {
                    s[i] *= gt[row];
                    r1 = fmaf(s[i], kt[row], r1);
                    r2 = fmaf(s[i], qt[row], r2);
                }
            }
            for (int o = cw; o < 32; o <<= 1) {
                r1 += __shfl_xor_sync(0xffffffffu, r1, o);
                r2 += __shfl_xor_sync(0xffffffffu, r2, o);
            }
            const float u = sb[t] * (sv[t * cols + jj] - r1);
#pragma unroll
            for (int i = 0; i < kRows; ++i) {
                const int row = r + i * R;
                if (row < d) s[i] = fmaf(kt[row], u, s[i]);
            }
            if (r == 0 && col_ok)
                out[(size_t)(row0 + t0 + t) * ld_out + (size_t)h * dv + j] = fmaf(u, sb[kTile + t], r2);
        }
        __syncthreads();                                     // this buffer is free for the tile after next
    }
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
        const int row = r + i * R;
        if (col_ok && row < d) S[(size_t)row * dv + j] = s[i];
    }
}

// The same recurrence for the usual head sizes, with the split known when compiling: d = KR * RT
// rows, RT lanes a column, a lane owns KR rows in a run (its q, k and g arrive by 16-byte reads from
// shared memory, every offset is a constant and no row needs a test).  The launcher picks RT by how
// many warps the step's columns make: few columns (one prompt) take many lanes a column, so that a
// scheduler has several warps to turn to while one waits for its own last result.
constexpr int kFixedThreads = 256;

template <int KR, int RT>
__global__ void __launch_bounds__(kFixedThreads)
delta_scan_fixed_kernel(const float* __restrict__ qk, int ld_qk, const float* __restrict__ v, int ld_v,
                        const float* __restrict__ decay, int ld_decay, const float* __restrict__ beta,
                        float* __restrict__ state, float* __restrict__ out, int ld_out,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                        int n_heads, int n_groups, int dv, int slices) {
    chain_release();
    chain_wait();
    constexpr int d = KR * RT, cw = 32 / RT, cols = kFixedThreads / RT;
    constexpr int per_buffer = 3 * kTile * d + kTile * cols + 2 * kTile;
    extern __shared__ __align__(16) float smem[];
    const int h = blockIdx.x / slices, slice = blockIdx.x % slices;
    const int b = blockIdx.y;
    const int grp = h / (n_heads / n_groups);
    const int row0 = cu_seqlens[b], n_rows = cu_seqlens[b + 1] - row0;
    const int tid = threadIdx.x;
    const int jj = (tid >> 5) * cw + (tid & 31) % cw, r = (tid & 31) / cw;
    const int j = slice * cols + jj;
    const bool col_ok = j < dv;
    float* S = state + ((size_t)slots[b] * n_heads + h) * (size_t)d * dv + (size_t)r * KR * dv;
    float s[KR];
#pragma unroll
    for (int i = 0; i < KR; ++i) s[i] = col_ok ? S[(size_t)i * dv + j] : 0.f;
    auto stage = [&](int buffer, int t0) {
        float* sq = smem + buffer * per_buffer;
        float* sk = sq + kTile * d;
        float* sg = sk + kTile * d;
        float* sv = sg + kTile * d;
        float* sb = sv + kTile * cols;
        const int nt = min(kTile, n_rows - t0);
        constexpr int d4 = d / 4;
        for (int idx = tid; idx < nt * d4; idx += kFixedThreads) {
            const int t = idx / d4, i = (idx - t * d4) * 4;
            const size_t row = (size_t)(row0 + t0 + t);
            copy_async_16(sq + t * d + i, qk + row * ld_qk + (size_t)grp * d + i);
            copy_async_16(sk + t * d + i, qk + row * ld_qk + (size_t)(n_groups + grp) * d + i);
            copy_async_16(sg + t * d + i, decay + row * ld_decay + (size_t)h * d + i);
        }
        for (int idx = tid; idx < nt * cols; idx += kFixedThreads) {
            const int t = idx / cols, c = idx - t * cols;
            const int col = min(slice * cols + c, dv - 1);
            copy_async_4(sv + t * cols + c, v + (size_t)(row0 + t0 + t) * ld_v + (size_t)h * dv + col);
        }
        if (tid < nt) copy_async_4(sb + tid, beta + (size_t)(row0 + t0 + tid) * n_heads + h);
        copy_async_commit();
    };
    if (n_rows > 0) stage(0, 0);
    int buffer = 0;
    for (int t0 = 0; t0 < n_rows; t0 += kTile, buffer ^= 1) {
        const int nt = min(kTile, n_rows - t0);
        if (t0 + kTile < n_rows) {
            stage(buffer ^ 1, t0 + kTile);
            copy_async_wait<1>();
        } else {
            copy_async_wait<0>();
        }
        __syncthreads();
        const float* sq = smem + buffer * per_buffer;
        const float* sk = sq + kTile * d;
        const float* sg = sk + kTile * d;
        const float* sv = sg + kTile * d;
        float* sb = const_cast<float*>(sv) + kTile * cols;
        for (int t = tid >> 5; t < nt; t += kFixedThreads / 32) {
            float kq = 0.f;
            for (int i = tid & 31; i < d; i += 32) kq = fmaf(sk[t * d + i], sq[t * d + i], kq);
            kq = warp_sum(kq);
            if ((tid & 31) == 0) sb[kTile + t] = kq;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            float kk[KR], qq[KR], gg[KR];
            if constexpr (KR % 4 == 0) {
#pragma unroll
                for (int i = 0; i < KR; i += 4) {
                    *reinterpret_cast<float4*>(gg + i) = *reinterpret_cast<const float4*>(sg + t * d + r * KR + i);
                    *reinterpret_cast<float4*>(kk + i) = *reinterpret_cast<const float4*>(sk + t * d + r * KR + i);
                    *reinterpret_cast<float4*>(qq + i) = *reinterpret_cast<const float4*>(sq + t * d + r * KR + i);
                }
            } else {
#pragma unroll
                for (int i = 0; i < KR; ++i) {
                    gg[i] = sg[t * d + r * KR + i];
                    kk[i] = sk[t * d + r * KR + i];
                    qq[i] = sq[t * d + r * KR + i];
                }
            }
            float r1[2] = {0.f, 0.f}, r2[2] = {0.f, 0.f};      // two sums each, so that a sum does not wait for its own last term
#pragma unroll
            for (int i = 0; i < KR; ++i) {
                s[i] *= gg[i];
                r1[i & 1] = fmaf(s[i], kk[i], r1[i & 1]);
                r2[i & 1] = fmaf(s[i], qq[i], r2[i & 1]);
            }
            float a1 = r1[0] + r1[1], a2 = r2[0] + r2[1];
#pragma unroll
            for (int o = cw; o < 32; o <<= 1) {
                a1 += __shfl_xor_sync(0xffffffffu, a1, o);
                a2 += __shfl_xor_sync(0xffffffffu, a2, o);
            }
            const float u = sb[t] * (sv[t * cols + jj] - a1);
#pragma unroll
            for (int i = 0; i < KR; ++i) s[i] = fmaf(kk[i], u, s[i]);
            if (r == 0 && col_ok)
                out[(size_t)(row0 + t0 + t) * ld_out + (size_t)h * dv + j] = fmaf(u, sb[kTile + t], a2);
        }
        __syncthreads();
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < KR; ++i) S[(size_t)i * dv + j] = s[i];
    }
}

template <int KR, int RT>
static int launch_fixed(const float* qk, int ld_qk, const float* v, int ld_v, const float* decay, int ld_decay, const float* beta,
                        float* state, float* out, int ld_out, const int* cu_seqlens, const int* slots, int n_seqs, int n_heads,
                        int n_groups, int dv, cudaStream_t stream) {
    constexpr int d = KR * RT, cols = kFixedThreads / RT;
    const int slices = (dv + cols - 1) / cols;
    const size_t smem = (size_t)2 * (3 * kTile * d + kTile * cols + 2 * kTile) * sizeof(float);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(delta_scan_fixed_kernel<KR, RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return launch_chained(delta_scan_fixed_kernel<KR, RT>, dim3(n_heads * slices, n_seqs), dim3(kFixedThreads), smem, stream, qk, ld_qk,
                          v, ld_v, decay, ld_decay, beta, state, out, ld_out, cu_seqlens, slots, n_heads, n_groups, dv, slices);
}

// A step in which every sequence brings one token: what costs is the state, read and written
// once, so a thread owns four neighbouring columns (16-byte accesses; a row of S is one
// contiguous run of the block's threads) for the rows rs, rs + RS, ...; the RS partial sums
// of a column meet through shared memory in a fixed order.  One block per (head, sequence).
constexpr int kStepThreads = 256;
constexpr int kStepRows = 16;      // rows of S a thread owns at most

__global__ void __launch_bounds__(kStepThreads, 2)
delta_step_kernel(const float* __restrict__ qk, int ld_qk, const float* __restrict__ v, int ld_v,
                  const float* __restrict__ decay, int ld_decay, const float* __restrict__ beta,
                  float* __restrict__ state, float* __restrict__ out, int ld_out, const int* __restrict__ slots,
                  int n_heads, int n_groups, int d, int dv, int CG, int RS) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float smem[];
    const int dpad = (d + 3) & ~3;                           // so that what follows q, k and g starts on a 16-byte boundary
    float* sq = smem;                                        // [dpad] each
    float* sk = sq + dpad;
    float* sg = sk + dpad;
    float* red = sg + dpad;                                  // [2][RS][dv]: the partial sums of r1, then of r2
    float* kq_s = red + 2 * RS * dv;
    const int h = blockIdx.x, b = blockIdx.y;
    const int grp = h / (n_heads / n_groups);
    const int tid = threadIdx.x;
    const size_t n = (size_t)b;
    for (int i = tid; i < d; i += kStepThreads) {
        sq[i] = qk[n * ld_qk + (size_t)grp * d + i];
        sk[i] = qk[n * ld_qk + (size_t)(n_groups + grp) * d + i];
        sg[i] = decay[n * ld_decay + (size_t)h * d + i];
    }
    __syncthreads();
    if (tid < 32) {
        float kq = 0.f;
        for (int i = tid; i < d; i += 32) kq = fmaf(sk[i], sq[i], kq);
        kq = warp_sum(kq);
        if (tid == 0) *kq_s = kq;
    }
    const int cg = tid % CG, rs = tid / CG;
    const bool live = rs < RS;
    float4* S4 = reinterpret_cast<float4*>(state + ((size_t)slots[b] * n_heads + h) * (size_t)d * dv);
    float4 s[kStepRows];
    float4 r1 = make_float4(0.f, 0.f, 0.f, 0.f), r2 = r1;
    if (live) {
#pragma unroll
        for (int i = 0; i < kStepRows; ++i) {
            const int row = rs + i * RS;
            if (row < d) s[i] = S4[(size_t)row * CG + cg];
        }
#pragma unroll
        for (int i = 0; i < kStepRows; ++i) {
            const int row = rs + i * RS;
            if (row < d) {
                const float g = sg[row], kk = sk[row], qq = sq[row];
                s[i].x *= g; s[i].y *= g; s[i].z *= g; s[i].w *= g;
                r1.x = fmaf(s[i].x, kk, r1.x); r1.y = fmaf(s[i].y, kk, r1.y); r1.z = fmaf(s[i].z, kk, r1.z); r1.w = fmaf(s[i].w, kk, r1.w);
                r2.x = fmaf(s[i].x, qq, r2.x); r2.y = fmaf(s[i].y, qq, r2.y); r2.z = fmaf(s[i].z, qq, r2.z); r2.w = fmaf(s[i].w, qq, r2.w);
            }
        }
        *reinterpret_cast<float4*>(red + (size_t)rs * dv + 4 * cg) = r1;
        *reinterpret_cast<float4*>(red + (size_t)(RS + rs) * dv + 4 * cg) = r2;
    }
    __syncthreads();
    if (live) {
        float4 t1 = make_float4(0.f, 0.f, 0.f, 0.f), t2 = t1;
        for (int k = 0; k < RS; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(red + (size_t)k * dv + 4 * cg);
            const float4 c = *reinterpret_cast<const float4*>(red + (size_t)(RS + k) * dv + 4 * cg);
            t1.x += a.x; t1.y += a.y; t1.z += a.z; t1.w += a.w;
            t2.x += c.x; t2.y += c.y; t2.z += c.z; t2.w += c.w;
        }
        const float bt = beta[n * n_heads + h], kq = *kq_s;
        const float4 vv = *reinterpret_cast<const float4*>(v + n * ld_v + (size_t)h * dv + 4 * cg);
        const float4 u = make_float4(bt * (vv.x - t1.x), bt * (vv.y - t1.y), bt * (vv.z - t1.z), bt * (vv.w - t1.w));
        if (rs == 0)
            *reinterpret_cast<float4*>(out + n * ld_out + (size_t)h * dv + 4 * cg) =
                make_float4(fmaf(u.x, kq, t2.x), fmaf(u.y, kq, t2.y), fmaf(u.z, kq, t2.z), fmaf(u.w, kq, t2.w));
#pragma unroll
        for (int i = 0; i < kStepRows; ++i) {
            const int row = rs + i * RS;
            if (row < d) {
                const float kk = sk[row];
                S4[(size_t)row * CG + cg] = make_float4(fmaf(kk, u.x, s[i].x), fmaf(kk, u.y, s[i].y), fmaf(kk, u.z, s[i].z), fmaf(kk, u.w, s[i].w));
            }
        }
    }
}

// ---------------------------------------------- norm per head, weight, sigmoid gate
// out[n, h, c] = y[n, h, c] / sqrt(mean_c(y[n, h, :]^2) + eps) * weight[c] * sigmoid(gate[n, h, c]):
// every head of the read-out by its own root mean square, a weight of dv channels that
// the heads share, and a gate from float logits.  A warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ y, int ld_y, const float* __restrict__ gate, int ld_gate,
                      const float* __restrict__ weight, float eps, T* __restrict__ out, int ld_out,
                      long long n_items, int n_heads, int dv) {
    chain_release();
    chain_wait();
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= n_items) return;
    const int lane = threadIdx.x & 31;
    const size_t n = (size_t)(item / n_heads);
    const int h = (int)(item % n_heads);
    const float* src = y + n * ld_y + (size_t)h * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(src[c], src[c], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
    const float* gt = gate + n * ld_gate + (size_t)h * dv;
    T* dst = out + n * ld_out + (size_t)h * dv;
    for (int c = lane; c < dv; c += 32)
        dst[c] = from_f32<T>(src[c] * inv * weight[c] * (1.0f / (1.0f + expf(-gt[c]))));
}
}  // namespace

GTG_API int gtg_delta_prepare(float* qk, int ld_qk, float* decay, int ld_decay, const float* dt_bias, const float* a_log,
                              const float* beta_in, int ld_beta_in, float* beta, int N, int n_heads, int n_groups, int d,
                              float unit_eps, float q_scale, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_heads <= 0 || n_groups <= 0 || n_heads % n_groups || d <= 0) return kErrBadArgument;
    if (ld_qk < 2 * n_groups * d || ld_decay < n_heads * d || ld_beta_in < n_heads) return kErrBadArgument;
    return launch_chained(delta_prepare_kernel, dim3(N), dim3(256), 0, stream, qk, ld_qk, decay, ld_decay, dt_bias, a_log,
                          beta_in, ld_beta_in, beta, n_heads, n_groups, d, unit_eps, q_scale);
}

// How many threads share a column of the state: the least power of two that leaves a
// thread at most kRows rows.
static int delta_split(int d) {
    int R = 1;
    while (R < 32 && (d + R - 1) / R > kRows) R *= 2;
    return R;
}

// Measurements may fix the lanes that share a column (8, 16 or 32; 0: the launcher chooses).
static int g_delta_lanes = 0;
GTG_API void gtg_delta_scan_lanes(int lanes) { g_delta_lanes = lanes; }

GTG_API int gtg_delta_scan_supports(int d, int dv) {
    return d > 0 && dv > 0 && d <= 32 * kRows && (size_t)2 * (3 * kTile * d + kTile * kFixedThreads + 2 * kTile) * 4 <= 200 * 1024;
}

// `one_token_each`: row b is sequence b's only token (a decode step); a kernel of its own serves it
// where the sizes allow (value channels a multiple of 4, at most 16 rows of the state a thread).
GTG_API int gtg_delta_scan(const float* qk, int ld_qk, const float* v, int ld_v, const float* decay, int ld_decay,
                           const float* beta, float* state, float* out, int ld_out, const int* cu_seqlens,
                           const int* slots, int n_seqs, int n_heads, int n_groups, int d, int dv, int one_token_each,
                           cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (n_heads <= 0 || n_groups <= 0 || n_heads % n_groups) return kErrBadArgument;
    if (!gtg_delta_scan_supports(d, dv)) return kErrUnsupported;
    if (ld_qk < 2 * n_groups * d || ld_v < n_heads * dv || ld_decay < n_heads * d || ld_out < n_heads * dv) return kErrBadArgument;
    if (n_seqs > 65535) return kErrUnsupported;
    if (one_token_each && dv % 4 == 0 && dv / 4 <= kStepThreads && ld_v % 4 == 0 && ld_out % 4 == 0 &&
        ((uintptr_t)v % 16) == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)state % 16) == 0) {
        const int CG = dv / 4;
        int RS = kStepThreads / CG;
        if (RS > d) RS = d;
        if ((d + RS - 1) / RS <= kStepRows) {
            const size_t smem = (size_t)(3 * ((d + 3) & ~3) + 2 * RS * dv + 4) * sizeof(float);
            if (smem <= 48 * 1024)
                return launch_chained(delta_step_kernel, dim3(n_heads, n_seqs), dim3(kStepThreads), smem, stream, qk, ld_qk, v, ld_v,
                                      decay, ld_decay, beta, state, out, ld_out, slots, n_heads, n_groups, d, dv, CG, RS);
        }
    }
    const int wide16 = ld_qk % 4 == 0 && ld_decay % 4 == 0 && ((uintptr_t)qk % 16) == 0 && ((uintptr_t)decay % 16) == 0;
    if (wide16 && (d == 64 || d == 128 || d == 256)) {
        // lanes a column: the fewest (fewest exchanges, fewest reads of shared memory a column) that still give the
        // device about seven warps a multiprocessor, not quite two a scheduler.  Measured at d = 128 with 2,048-token
        // prompts: 2,048 columns 0.86 / 0.58 / 0.65 ms at 8 / 16 / 32 lanes, 4,096 columns 0.86 / 0.80 / 1.10,
        // 8,192 columns 1.21 / 1.42 / 1.91: more warps hide a token's chain of dependent steps, but every warp
        // reads the whole of q, k and g, and beyond some thousand warps shared memory is the limit.
        int device = 0, sms = 148;
        if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        const long long columns = (long long)n_seqs * n_heads * dv;
        int RT = d / kRows;
        while (RT < 32 && columns * RT / 32 < 27LL * sms / 4) RT *= 2;
        if (g_delta_lanes >= d / kRows && g_delta_lanes <= 32 && (g_delta_lanes & (g_delta_lanes - 1)) == 0) RT = g_delta_lanes;
#define GTG_FIXED(KR, R) launch_fixed<KR, R>(qk, ld_qk, v, ld_v, decay, ld_decay, beta, state, out, ld_out, cu_seqlens, slots, n_seqs, \
                                             n_heads, n_groups, dv, stream)
        if (d == 64) return RT == 4 ? GTG_FIXED(16, 4) : RT == 8 ? GTG_FIXED(8, 8) : RT == 16 ? GTG_FIXED(4, 16) : GTG_FIXED(2, 32);
        if (d == 128) return RT == 8 ? GTG_FIXED(16, 8) : RT == 16 ? GTG_FIXED(8, 16) : GTG_FIXED(4, 32);
        return RT == 16 ? GTG_FIXED(16, 16) : GTG_FIXED(8, 32);
#undef GTG_FIXED
    }
    const int R = delta_split(d);
    const int cols = kScanThreads / R;
    const int slices = (dv + cols - 1) / cols;
    const size_t smem = (size_t)2 * (3 * kTile * d + kTile * cols + 2 * kTile) * sizeof(float);
    const int wide = d % 4 == 0 && ld_qk % 4 == 0 && ld_decay % 4 == 0 && ((uintptr_t)qk % 16) == 0 && ((uintptr_t)decay % 16) == 0 &&
                     cols % 4 == 0;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_chained(delta_scan_kernel, dim3(n_heads * slices, n_seqs), dim3(kScanThreads), smem, stream, qk, ld_qk, v, ld_v,
                          decay, ld_decay, beta, state, out, ld_out, cu_seqlens, slots, n_heads, n_groups, d, dv, R, slices, wide);
}

GTG_API int gtg_head_norm_gate(int dtype, const float* y, int ld_y, const float* gate, int ld_gate, const float* weight,
                               float eps, void* out, int ld_out, int N, int n_heads, int dv, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_heads <= 0 || dv <= 0 || ld_y < n_heads * dv || ld_gate < n_heads * dv || ld_out < n_heads * dv) return kErrBadArgument;
    const long long items = (long long)N * n_heads;
    const long long blocks = (items + 7) / 8;
    if (blocks > 0x7fffffffLL) return kErrUnsupported;
    if (dtype == 0) return launch_chained(head_norm_gate_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, y, ld_y, gate,
                                          ld_gate, weight, eps, (float*)out, ld_out, items, n_heads, dv);
    if (dtype == 1) return launch_chained(head_norm_gate_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, stream, y, ld_y, gate,
                                          ld_gate, weight, eps, (bf16*)out, ld_out, items, n_heads, dv);
    return kErrBadArgument;
}
