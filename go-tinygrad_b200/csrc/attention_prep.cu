// What stands between the fused projection of an attention mixer and the
// attention itself, for mixers whose projections have more to them than a
// rotation: of a token's float sums out of the projection,
//   [ q: n_heads x hd | k: n_kv x hd | v: n_kv x vd | g: n_heads ],
// a warp takes one head (or the gates) and, all in float,
//   * adds the biases of q, k and v;
//   * rotates the first `rot` channels of every query and key head, channel i with
//     i + rot/2, by the token's (cos, sin) table; the rest of a head passes;
//   * with `unit_norm`, divides every rotated query and key head by its root mean
//     square, x / sqrt(mean(x^2) + eps);
//   * blends the values with those an earlier layer left for the step,
//     v <- (1 - lambda) v + lambda v_first, or leaves its own for later layers;
//   * turns the gate columns into sigmoid factors, one per query head;
// then rounds once: queries to `q_out`, keys and values into the token's place in
// the paged cache (key rows of hd, value rows of vd channels).
#include "common.cuh"
#include <math.h>

namespace {
// two neighbouring channels in one access (the address is a multiple of two elements)
__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(bf16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }

// A block a token: the token's sums are staged in shared memory (all loads in flight at once), then a warp
// takes a head at a time.  For the many tokens of a prompt.
template <typename T>
__global__ void __launch_bounds__(256)
qkv_finish_rows_kernel(const float* __restrict__ sums, int ld, const float* __restrict__ bias,
                  const float2* __restrict__ cos_sin, int rot, int unit_norm, float eps,
                  const float* __restrict__ v_first, float* __restrict__ v_keep, float lambda,
                  T* __restrict__ q_out, int ldq, float* __restrict__ gate_out,
                  T* __restrict__ kc, T* __restrict__ vc, long long page_stride,
                  const int* __restrict__ block_table, int table_stride,
                  const int* __restrict__ token_seq, const int* __restrict__ slots,
                  const int* __restrict__ positions,
                  int n_heads, int n_kv, int hd, int vd, int has_gate) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float row[];
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const int q_w = n_heads * hd, k_w = n_kv * hd, v_w = n_kv * vd;
    const int biased = q_w + k_w + v_w;
    const int width = biased + (has_gate ? n_heads : 0);
    const float* src = sums + (size_t)n * ld;
    if (ld % 4 == 0 && (reinterpret_cast<uintptr_t>(sums) % 16) == 0) {
        // four sums an access; the biases are the same for every token and come from the caches
        const int whole = width & ~3;
        for (int i = threadIdx.x * 4; i < whole; i += blockDim.x * 4) {
            float4 t = *reinterpret_cast<const float4*>(src + i);
            if (bias) {
                if (i + 0 < biased) t.x += __ldg(bias + i + 0);
                if (i + 1 < biased) t.y += __ldg(bias + i + 1);
                if (i + 2 < biased) t.z += __ldg(bias + i + 2);
                if (i + 3 < biased) t.w += __ldg(bias + i + 3);
            }
            *reinterpret_cast<float4*>(row + i) = t;
        }
        for (int i = whole + threadIdx.x; i < width; i += blockDim.x) row[i] = src[i] + ((bias && i < biased) ? bias[i] : 0.f);
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = src[i] + ((bias && i < biased) ? bias[i] : 0.f);
    }
    __syncthreads();

    const int pos = positions[n];
    size_t page_off = 0;
    if (kc) {
        const int slot = slots[token_seq[n]];
        page_off = (size_t)block_table[(size_t)slot * table_stride + pos / kPageTokens] * page_stride;
    }
    const int rhalf = rot >> 1;
    // queries and keys: a warp a head
    for (int head = warp; head < n_heads + n_kv; head += n_warps) {
        float* x = row + (size_t)head * hd;
        if (cos_sin) {
            for (int i = lane; i < rhalf; i += 32) {
                const float2 cs = cos_sin[(size_t)n * rhalf + i];
                const float a = x[i], b = x[i + rhalf];
                x[i] = a * cs.x - b * cs.y;
                x[i + rhalf] = b * cs.x + a * cs.y;
            }
            __syncwarp();
        }
        float inv = 1.f;
        if (unit_norm) {
            float sq = 0.f;
            for (int i = lane; i < hd; i += 32) sq = fmaf(x[i], x[i], sq);
            inv = 1.0f / sqrtf(warp_sum(sq) / (float)hd + eps);
        }
        T* dst;
        if (head < n_heads) dst = q_out + (size_t)n * ldq + (size_t)head * hd;
        else if (kc) dst = kc + page_off + ((size_t)(head - n_heads) * kPageTokens + (pos % kPageTokens)) * hd;
        else continue;
        if (hd % 2 == 0 && (reinterpret_cast<uintptr_t>(dst) % (2 * sizeof(T))) == 0) {
            for (int i = lane * 2; i < hd; i += 64) store_pair(dst + i, x[i] * inv, x[i + 1] * inv);
        } else {
            for (int i = lane; i < hd; i += 32) dst[i] = from_f32<T>(x[i] * inv);
        }
    }
    // values
    const float* v = row + q_w + k_w;
    const bool v_pairs = vd % 2 == 0 && (q_w + k_w) % 2 == 0 && (!vc || (page_stride % 2 == 0 && (reinterpret_cast<uintptr_t>(vc) % (2 * sizeof(T))) == 0)) &&
                         (!v_keep || (reinterpret_cast<uintptr_t>(v_keep) % 8) == 0) && (!v_first || (reinterpret_cast<uintptr_t>(v_first) % 8) == 0);
    if (v_pairs) {
        for (int i = threadIdx.x * 2; i < v_w; i += blockDim.x * 2) {
            float2 val = *reinterpret_cast<const float2*>(v + i);
            if (v_keep) *reinterpret_cast<float2*>(v_keep + (size_t)n * v_w + i) = val;
            if (v_first) {
                const float2 f = *reinterpret_cast<const float2*>(v_first + (size_t)n * v_w + i);
                val.x = (1.0f - lambda) * val.x + lambda * f.x;
                val.y = (1.0f - lambda) * val.y + lambda * f.y;
            }
            if (vc) {
                const int head = i / vd, c = i - head * vd;
                store_pair(vc + page_off + ((size_t)head * kPageTokens + (pos % kPageTokens)) * vd + c, val.x, val.y);
            }
        }
    } else
    for (int i = threadIdx.x; i < v_w; i += blockDim.x) {
        float val = v[i];
        if (v_keep) v_keep[(size_t)n * v_w + i] = val;
        if (v_first) val = (1.0f - lambda) * val + lambda * v_first[(size_t)n * v_w + i];
        if (vc) {
            const int head = i / vd, c = i - head * vd;
            vc[page_off + ((size_t)head * kPageTokens + (pos % kPageTokens)) * vd + c] = from_f32<T>(val);
        }
    }
    if (has_gate)
        for (int h = threadIdx.x; h < n_heads; h += blockDim.x)
            gate_out[(size_t)n * n_heads + h] = 1.0f / (1.0f + expf(-row[biased + h]));
}

constexpr int kFinishWarps = 8;

// A warp an item: a query head, a key head, a value head, or the token's gates; a token's items
// are dealt to gridDim.y blocks of kFinishWarps warps and nothing meets across warps.  For the few
// tokens of a decode step or a short portion, which a block a token leaves most of the device idle
// for.  Both kernels do the same arithmetic in the same order: their results are the same bits.
template <typename T>
__global__ void __launch_bounds__(kFinishWarps * 32)
qkv_finish_heads_kernel(const float* __restrict__ sums, int ld, const float* __restrict__ bias,
                  const float2* __restrict__ cos_sin, int rot, int unit_norm, float eps,
                  const float* __restrict__ v_first, float* __restrict__ v_keep, float lambda,
                  T* __restrict__ q_out, int ldq, float* __restrict__ gate_out,
                  T* __restrict__ kc, T* __restrict__ vc, long long page_stride,
                  const int* __restrict__ block_table, int table_stride,
                  const int* __restrict__ token_seq, const int* __restrict__ slots,
                  const int* __restrict__ positions,
                  int n_heads, int n_kv, int hd, int vd, int has_gate) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float staged[];          // [warp][hd]: the head a warp is turning
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_w = n_heads * hd, k_w = n_kv * hd, v_w = n_kv * vd;
    const int n_turning = n_heads + n_kv;
    const int n_items = n_turning + n_kv + (has_gate ? 1 : 0);
    const float* src = sums + (size_t)n * ld;
    const int pos = positions[n];
    size_t page_off = 0;
    bool page_known = false;
    for (int item = blockIdx.y * kFinishWarps + warp; item < n_items; item += gridDim.y * kFinishWarps) {
        if (kc && !page_known && item >= n_heads && item < n_turning + n_kv) {
            const int slot = slots[token_seq[n]];
            page_off = (size_t)block_table[(size_t)slot * table_stride + pos / kPageTokens] * page_stride;
            page_known = true;
        }
        if (item < n_turning) {
            // a query or key head: bias, rotation, unit norm, store
            float* x = staged + (size_t)warp * hd;
            const int at = item * hd;
            for (int i = lane; i < hd; i += 32) x[i] = src[at + i] + (bias ? __ldg(bias + at + i) : 0.f);
            __syncwarp();
            const int rhalf = rot >> 1;
            if (cos_sin) {
                for (int i = lane; i < rhalf; i += 32) {
                    const float2 cs = cos_sin[(size_t)n * rhalf + i];
                    const float a = x[i], b = x[i + rhalf];
                    x[i] = a * cs.x - b * cs.y;
                    x[i + rhalf] = b * cs.x + a * cs.y;
                }
                __syncwarp();
            }
            float inv = 1.f;
            if (unit_norm) {
                float sq = 0.f;
                for (int i = lane; i < hd; i += 32) sq = fmaf(x[i], x[i], sq);
                inv = 1.0f / sqrtf(warp_sum(sq) / (float)hd + eps);
            }
            T* dst;
            if (item < n_heads) dst = q_out + (size_t)n * ldq + (size_t)item * hd;
            else if (kc) dst = kc + page_off + ((size_t)(item - n_heads) * kPageTokens + (pos % kPageTokens)) * hd;
            else { __syncwarp(); continue; }
            if (hd % 2 == 0 && (reinterpret_cast<uintptr_t>(dst) % (2 * sizeof(T))) == 0) {
                for (int i = lane * 2; i < hd; i += 64) store_pair(dst + i, x[i] * inv, x[i + 1] * inv);
            } else {
                for (int i = lane; i < hd; i += 32) dst[i] = from_f32<T>(x[i] * inv);
            }
            __syncwarp();                                        // before the warp's next head overwrites x
            continue;
        }
        if (item < n_turning + n_kv) {
            // a value head: bias, kept for later layers, blended, store
            const int head = item - n_turning;
            const int at = q_w + k_w + head * vd;
            const size_t step_at = (size_t)n * v_w + (size_t)head * vd;
            T* dst = vc ? vc + page_off + ((size_t)head * kPageTokens + (pos % kPageTokens)) * vd : nullptr;
            for (int c = lane; c < vd; c += 32) {
                float val = src[at + c] + (bias ? __ldg(bias + at + c) : 0.f);
                if (v_keep) v_keep[step_at + c] = val;
                if (v_first) val = (1.0f - lambda) * val + lambda * v_first[step_at + c];
                if (dst) dst[c] = from_f32<T>(val);
            }
            continue;
        }
        // the gates: one sigmoid a query head, no bias
        for (int h = lane; h < n_heads; h += 32)
            gate_out[(size_t)n * n_heads + h] = 1.0f / (1.0f + expf(-src[q_w + k_w + v_w + h]));
    }
}
// ---- projections that pass a short convolution over time -------------------------------
// For mixers whose q, k and v pass, channel by channel, a causal convolution over
// the last `taps` tokens before anything else happens to them.  Of a token's float
// sums out of the projection,  [ q: n_heads x hd | k: n_kv x hd | v: n_kv x vd ]
// (n_kv = 0: the layer has queries only and reads another layer's keys and values),
// a warp takes one head and, all in float,
//   * adds the bias and convolves: y_t[c] = sum_j w[j, c] u_(t - taps + 1 + j)[c], u the
//     biased sums; tokens of this step are read from the sums, earlier ones from
//     conv_state[slot] ([taps-1, C], the sequence's last raw sums, oldest first), and
//     what lies before the sequence's first token is zero.  The taps are added oldest
//     first, whatever the cut of the sequence into steps;
//   * norms every query and key head, x / sqrt(mean(x^2) + eps) * w (weights of hd
//     channels, shared by the heads; null: no norm);
//   * rotates the first `rot` channels of every query and key head by the token's
//     (cos, sin) table: channel 2i with 2i+1 (`interleaved`) or i with i + rot/2;
// then rounds once: queries to q_out, keys and values into the token's cache place.
// The state is left as it was: `conv_state_update` over the same sums follows.
template <typename T>
__global__ void __launch_bounds__(kFinishWarps * 32)
qkv_conv_finish_kernel(const float* __restrict__ sums, int ld, const float* __restrict__ bias,
                       const float* __restrict__ conv_w, int taps, const float* __restrict__ conv_state,
                       const int* __restrict__ cu_seqlens,
                       const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                       const float2* __restrict__ cos_sin, int rot, int interleaved,
                       T* __restrict__ q_out, int ldq, T* __restrict__ kc, T* __restrict__ vc, long long page_stride,
                       const int* __restrict__ block_table, int table_stride,
                       const int* __restrict__ token_seq, const int* __restrict__ slots,
                       const int* __restrict__ positions, int n_heads, int n_kv, int hd, int vd) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float staged[];          // [warp][hd]: the head a warp is working on
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_w = n_heads * hd, k_w = n_kv * hd;
    const int C = q_w + k_w + n_kv * vd;
    const int n_turning = n_heads + n_kv, n_items = n_turning + n_kv;
    const int b = token_seq[n];
    const int before = n - cu_seqlens[b];                    // rows of this sequence before n in the step
    const int pos = positions[n];
    const int keep = taps - 1;
    const float* st = keep > 0 ? conv_state + (size_t)slots[b] * keep * C : nullptr;
    auto convolved = [&](int c) -> float {
        const float bc = bias ? __ldg(bias + c) : 0.f;
        if (keep <= 0) return sums[(size_t)n * ld + c] + bc;
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = keep - j;
            if (pos - back < 0) continue;                    // before the sequence's first token: nothing
            const float u = before - back >= 0 ? sums[(size_t)(n - back) * ld + c] : st[(size_t)(keep + before - back) * C + c];
            acc = fmaf(__ldg(conv_w + (size_t)j * C + c), u + bc, acc);
        }
        return acc;
    };
    size_t page_off = 0;
    if (kc) page_off = (size_t)block_table[(size_t)slots[b] * table_stride + pos / kPageTokens] * page_stride;
    const int rhalf = rot >> 1;
    for (int item = blockIdx.y * kFinishWarps + warp; item < n_items; item += gridDim.y * kFinishWarps) {
        if (item >= n_turning) {
            // a value head: convolved and stored
            const int head = item - n_turning;
            if (!vc) continue;
            T* dst = vc + page_off + ((size_t)head * kPageTokens + (pos % kPageTokens)) * vd;
            for (int c = lane; c < vd; c += 32) dst[c] = from_f32<T>(convolved(q_w + k_w + head * vd + c));
            continue;
        }
        const bool is_q = item < n_heads;
        if (!is_q && !kc) continue;
        float* x = staged + (size_t)warp * hd;
        float sq = 0.f;
        for (int i = lane; i < hd; i += 32) {
            const float v = convolved(item * hd + i);
            x[i] = v;
            sq = fmaf(v, v, sq);
        }
        const float* w = is_q ? q_norm : k_norm;
        if (w) {
            const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)hd + eps);
            for (int i = lane; i < hd; i += 32) x[i] = x[i] * inv * __ldg(w + i);
        }
        __syncwarp();
        if (cos_sin) {
            for (int i = lane; i < rhalf; i += 32) {
                const float2 cs = cos_sin[(size_t)n * rhalf + i];
                const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + rhalf;
                const float a = x[ia], bb = x[ib];
                x[ia] = a * cs.x - bb * cs.y;
                x[ib] = bb * cs.x + a * cs.y;
            }
            __syncwarp();
        }
        T* dst = is_q ? q_out + (size_t)n * ldq + (size_t)item * hd
                      : kc + page_off + ((size_t)(item - n_heads) * kPageTokens + (pos % kPageTokens)) * hd;
        if (hd % 2 == 0 && (reinterpret_cast<uintptr_t>(dst) % (2 * sizeof(T))) == 0) {
            for (int i = lane * 2; i < hd; i += 64) store_pair(dst + i, x[i], x[i + 1]);
        } else {
            for (int i = lane; i < hd; i += 32) dst[i] = from_f32<T>(x[i]);
        }
        __syncwarp();                                        // before the warp's next head overwrites x
    }
}
// The same for the many tokens of a prompt: a warp takes one head of kRunTokens consecutive rows.  The
// rows a channel's taps reach, this step's kRunTokens + TAPS - 1 of them, are read once into registers and
// serve all of the run's tokens, as do the channel's taps and bias; a row that belongs to another sequence
// (or lies before the step) is never used: such a tap reads the state, or nothing, exactly as above.
// The arithmetic and its order are those of the kernel above: their results are the same bits.
constexpr int kRunTokens = 4;

template <typename T, int TAPS>
__global__ void __launch_bounds__(kFinishWarps * 32)
qkv_conv_finish_run_kernel(const float* __restrict__ sums, int ld, const float* __restrict__ bias,
                           const float* __restrict__ conv_w, const float* __restrict__ conv_state,
                           const int* __restrict__ cu_seqlens,
                           const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                           const float2* __restrict__ cos_sin, int rot, int interleaved,
                           T* __restrict__ q_out, int ldq, T* __restrict__ kc, T* __restrict__ vc, long long page_stride,
                           const int* __restrict__ block_table, int table_stride,
                           const int* __restrict__ token_seq, const int* __restrict__ slots,
                           const int* __restrict__ positions, int N, int n_heads, int n_kv, int hd, int vd) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float staged[];          // [warp][kRunTokens][hd]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kRunTokens;
    const int q_w = n_heads * hd, k_w = n_kv * hd;
    const int C = q_w + k_w + n_kv * vd;
    const int n_turning = n_heads + n_kv, n_items = n_turning + n_kv;
    constexpr int keep = TAPS - 1;
    int before[kRunTokens], pos[kRunTokens], slot[kRunTokens];
#pragma unroll
    for (int tk = 0; tk < kRunTokens; ++tk) {
        const int n = min(n0 + tk, N - 1);
        const int b = token_seq[n];
        before[tk] = n - cu_seqlens[b];
        pos[tk] = positions[n];
        slot[tk] = slots[b];
    }
    const int rhalf = rot >> 1;
    for (int item = blockIdx.y * kFinishWarps + warp; item < n_items; item += gridDim.y * kFinishWarps) {
        const bool is_v = item >= n_turning, is_q = item < n_heads;
        if (!is_q && !kc) continue;
        const int width = is_v ? vd : hd;
        const int c0 = is_v ? q_w + k_w + (item - n_turning) * vd : item * hd;
        float* x = staged + (size_t)warp * kRunTokens * hd;
        for (int i = lane; i < width; i += 32) {
            const int c = c0 + i;
            float win[kRunTokens + keep], w[TAPS];
#pragma unroll
            for (int k = 0; k < kRunTokens + keep; ++k) {
                const int row = n0 - keep + k;
                win[k] = (row >= 0 && row < N) ? sums[(size_t)row * ld + c] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < TAPS; ++j) w[j] = __ldg(conv_w + (size_t)j * C + c);
            const float bc = bias ? __ldg(bias + c) : 0.f;
#pragma unroll
            for (int tk = 0; tk < kRunTokens; ++tk) {
                float acc = 0.f;
#pragma unroll
                for (int j = 0; j < TAPS; ++j) {
                    const int back = keep - j;
                    if (pos[tk] - back < 0) continue;
                    const float u = before[tk] - back >= 0 ? win[tk + j]
                                                           : conv_state[((size_t)slot[tk] * keep + (keep + before[tk] - back)) * C + c];
                    acc = fmaf(w[j], u + bc, acc);
                }
                x[tk * hd + i] = acc;
            }
        }
        __syncwarp();
        for (int tk = 0; tk < kRunTokens; ++tk) {
            const int n = n0 + tk;
            if (n >= N) break;
            float* xt = x + tk * hd;
            size_t page_off = 0;
            if (kc) page_off = (size_t)block_table[(size_t)slot[tk] * table_stride + pos[tk] / kPageTokens] * page_stride;
            if (is_v) {
                T* dst = vc + page_off + ((size_t)(item - n_turning) * kPageTokens + (pos[tk] % kPageTokens)) * vd;
                for (int i = lane; i < vd; i += 32) dst[i] = from_f32<T>(xt[i]);
                continue;
            }
            const float* nw = is_q ? q_norm : k_norm;
            if (nw) {
                float sq = 0.f;
                for (int i = lane; i < hd; i += 32) sq = fmaf(xt[i], xt[i], sq);
                const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)hd + eps);
                for (int i = lane; i < hd; i += 32) xt[i] = xt[i] * inv * __ldg(nw + i);
                __syncwarp();
            }
            if (cos_sin) {
                for (int i = lane; i < rhalf; i += 32) {
                    const float2 cs = cos_sin[(size_t)n * rhalf + i];
                    const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + rhalf;
                    const float a = xt[ia], bb = xt[ib];
                    xt[ia] = a * cs.x - bb * cs.y;
                    xt[ib] = bb * cs.x + a * cs.y;
                }
                __syncwarp();
            }
            T* dst = is_q ? q_out + (size_t)n * ldq + (size_t)item * hd
                          : kc + page_off + ((size_t)(item - n_heads) * kPageTokens + (pos[tk] % kPageTokens)) * hd;
            if (hd % 2 == 0 && (reinterpret_cast<uintptr_t>(dst) % (2 * sizeof(T))) == 0) {
                for (int i = lane * 2; i < hd; i += 64) store_pair(dst + i, xt[i], xt[i + 1]);
            } else {
                for (int i = lane; i < hd; i += 32) dst[i] = from_f32<T>(xt[i]);
            }
        }
        __syncwarp();                                        // before the warp's next head overwrites x
    }
}
}  // namespace

GTG_API int gtg_qkv_finish(int dtype, const float* sums, int ld, const float* bias, const float* cos_sin, int rot,
                           int unit_norm, float eps, const float* v_first, float* v_keep, float lambda,
                           void* q_out, int ldq, float* gate_out, void* kc, void* vc, long long page_stride,
                           const int* block_table, int table_stride, const int* token_seq, const int* slots,
                           const int* positions, int N, int n_heads, int n_kv, int hd, int vd, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || hd <= 0 || vd <= 0 || rot < 0 || (rot & 1) || rot > hd) return kErrBadArgument;
    if ((cos_sin != nullptr) != (rot > 0) || (kc == nullptr) != (vc == nullptr)) return kErrBadArgument;
    const int has_gate = gate_out != nullptr;
    const int width = n_heads * hd + n_kv * (hd + vd) + (has_gate ? n_heads : 0);
    if (ld < width) return kErrBadArgument;
    // up to kFewTokens tokens a warp per head over several blocks a token, beyond a block per token
    constexpr int kFewTokens = 512;
    const bool few = N <= kFewTokens;
    const size_t smem = few ? (size_t)kFinishWarps * hd * sizeof(float) : (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return kErrUnsupported;
    const int n_items = n_heads + 2 * n_kv + has_gate;
    const dim3 grid(N, few ? (n_items + kFinishWarps - 1) / kFinishWarps : 1);
    if (grid.y > 65535) return kErrUnsupported;
#define GTG_FINISH(T)                                                                                              \
    do {                                                                                                           \
        auto kernel = few ? qkv_finish_heads_kernel<T> : qkv_finish_rows_kernel<T>;                                \
        if (smem > 48 * 1024) {                                                                                    \
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                   \
        }                                                                                                          \
        return launch_chained(kernel, grid, dim3(kFinishWarps * 32), smem, stream, sums, ld, bias, (const float2*)cos_sin, rot, \
                              unit_norm, eps, v_first, v_keep, lambda, (T*)q_out, ldq, gate_out, (T*)kc, (T*)vc,    \
                              page_stride, block_table, table_stride, token_seq, slots, positions, n_heads, n_kv,  \
                              hd, vd, has_gate);                                                                   \
    } while (0)
    if (dtype == 0) GTG_FINISH(float);
    if (dtype == 1) GTG_FINISH(bf16);
#undef GTG_FINISH
    return kErrBadArgument;
}

GTG_API int gtg_qkv_conv_finish(int dtype, const float* sums, int ld, const float* bias, const float* conv_w, int taps,
                                const float* conv_state, const int* cu_seqlens, const float* q_norm, const float* k_norm,
                                float eps, const float* cos_sin, int rot, int interleaved, void* q_out, int ldq,
                                void* kc, void* vc, long long page_stride, const int* block_table, int table_stride,
                                const int* token_seq, const int* slots, const int* positions, int N, int n_heads,
                                int n_kv, int hd, int vd, int one_token_each, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_heads <= 0 || n_kv < 0 || hd <= 0 || vd <= 0 || rot < 0 || (rot & 1) || rot > hd || taps < 1) return kErrBadArgument;
    if ((cos_sin != nullptr) != (rot > 0) || (kc == nullptr) != (vc == nullptr)) return kErrBadArgument;
    if (taps > 1 && (!conv_w || !conv_state)) return kErrBadArgument;
    if (n_kv == 0 && kc) return kErrBadArgument;
    if (ld < n_heads * hd + n_kv * (hd + vd)) return kErrBadArgument;
    const size_t smem = (size_t)kFinishWarps * hd * sizeof(float);
    if (smem > 200 * 1024) return kErrUnsupported;
    const int n_items = n_heads + 2 * n_kv;
    const dim3 grid(N, (n_items + kFinishWarps - 1) / kFinishWarps);
    if (grid.y > 65535) return kErrUnsupported;
    // many tokens and two to four taps: a warp takes a head of four consecutive rows at a time
    constexpr int kManyTokens = 64;
    const size_t smem_run = smem * kRunTokens;
    // (not a step of one token a sequence: there neighbouring rows share nothing)
    if (!one_token_each && N >= kManyTokens && taps >= 2 && taps <= 4 && vd <= hd && smem_run <= 200 * 1024) {
        const dim3 grid_run((N + kRunTokens - 1) / kRunTokens, grid.y);
#define GTG_CONV_RUN(T, TAPS)                                                                                      \
        do {                                                                                                       \
            auto kernel = qkv_conv_finish_run_kernel<T, TAPS>;                                                     \
            if (smem_run > 48 * 1024) {                                                                            \
                const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_run); \
                if (e != cudaSuccess) return (int)e;                                                               \
            }                                                                                                      \
            return launch_chained(kernel, grid_run, dim3(kFinishWarps * 32), smem_run, stream, sums, ld, bias, conv_w, \
                                  conv_state, cu_seqlens, q_norm, k_norm, eps, (const float2*)cos_sin, rot, interleaved, \
                                  (T*)q_out, ldq, (T*)kc, (T*)vc, page_stride, block_table, table_stride, token_seq,   \
                                  slots, positions, N, n_heads, n_kv, hd, vd);                                      \
        } while (0)
        if (dtype == 0) { if (taps == 2) GTG_CONV_RUN(float, 2); if (taps == 3) GTG_CONV_RUN(float, 3); GTG_CONV_RUN(float, 4); }
        if (dtype == 1) { if (taps == 2) GTG_CONV_RUN(bf16, 2); if (taps == 3) GTG_CONV_RUN(bf16, 3); GTG_CONV_RUN(bf16, 4); }
#undef GTG_CONV_RUN
        return kErrBadArgument;
    }
#define GTG_CONV_FINISH(T)                                                                                         \
    do {                                                                                                           \
        auto kernel = qkv_conv_finish_kernel<T>;                                                                   \
        if (smem > 48 * 1024) {                                                                                    \
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                   \
        }                                                                                                          \
        return launch_chained(kernel, grid, dim3(kFinishWarps * 32), smem, stream, sums, ld, bias, conv_w, taps,   \
                              conv_state, cu_seqlens, q_norm, k_norm, eps, (const float2*)cos_sin, rot, interleaved, \
                              (T*)q_out, ldq, (T*)kc, (T*)vc, page_stride, block_table, table_stride, token_seq,   \
                              slots, positions, n_heads, n_kv, hd, vd);                                            \
    } while (0)
    if (dtype == 0) GTG_CONV_FINISH(float);
    if (dtype == 1) GTG_CONV_FINISH(bf16);
#undef GTG_CONV_FINISH
    return kErrBadArgument;
}
