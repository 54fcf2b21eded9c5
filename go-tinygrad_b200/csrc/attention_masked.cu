// bfloat16 attention over the paged cache for mixers whose keys and values differ
// in width, whose keys are seen through a window or within stretches (chunks) of
// positions, and whose heads may carry a gate.  Warp-level tensor-core path
// (mma.sync.m16n8k16, operands through ldmatrix, pages staged by cp.async).
//
// Rows of the score matrix are (token, query head of the group) pairs: all query
// heads that share a key/value head meet the same keys, so a block of 64 such
// rows reads every page once for the whole group.  One block per (64-row tile,
// key/value head, sequence) and, for steps that bring few rows (decode), per
// share of the pages the tile sees (`n_splits`): a share leaves its unnormalised
// output with its running maximum and sum, and `attention_masked_merge` adds the
// shares up in a fixed order.  A prompt, a portion of one and a decode step are
// the same kernel: the token at position p sees the keys lo(p)..p of its own
// sequence,
//     lo(p) = max(0, p - window + 1, p - p % chunk)       (window, chunk 0: none),
// the chunks counted from the sequence's first token, whatever the step brings.
//
// Scores are scaled after the dot product and exponentiated with exp2 on
// log2(e)-scaled values; maximum, sum and the output accumulator are float.  Key
// rows of hd and value rows of vd channels (multiples of 8) are zero-padded in
// shared memory to DKP and DVP (64 or 128).  `gate` (or null) is a float factor per
// (token, query head) on the output; with `gate_ld` > 0 it holds one logit per output
// channel instead (rows of gate_ld floats, heads side by side vd apart) and the factor is
// the logit's sigmoid.  `softcap` c > 0: a scaled score s becomes c tanh(s / c) (the
// hyperbolic tangent as 1 - 2 / (1 + e^(2x)): its error, times c, is far below a score's own).
#include "mma_helpers.cuh"
#include <math.h>

namespace {
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kTileRows = 64;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// tanh(x) = 1 - 2 / (1 + e^(2x)); exact at both ends (e^(2x) = inf or 0), absolute error about 1e-7
__device__ __forceinline__ float tanh_by_exp(float x) {
    return 1.0f - __fdividef(2.0f, 1.0f + fast_exp2(x * (2.0f * kLog2e)));
}

__device__ __forceinline__ int first_seen(int pos, int window, int chunk) {
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, pos - pos % chunk);
    return lo;
}

template <int DKP, int DVP>
constexpr int masked_smem_bytes() { return 3 * kTileRows * DKP * 2 + 2 * kTileRows * DVP * 2; }

template <int DKP, int DVP>
__global__ void __launch_bounds__(128)
attention_masked_kernel(const bf16* __restrict__ q, int ldq, bf16* __restrict__ out, int ldo,
                        const bf16* __restrict__ kc, const bf16* __restrict__ vc, long long page_stride,
                        const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                        const int* __restrict__ start_pos,
                        int n_heads, int n_kv, int hd, int vd, float scale, int window, int chunk,
                        const float* __restrict__ gate, int n_splits,
                        float* __restrict__ part_o, float* __restrict__ part_ml, float softcap, int gate_ld) {
    chain_release();
    chain_wait();
    constexpr int KCPR = DKP / 8, VCPR = DVP / 8;          // 16-byte chunks per staged row
    constexpr int KTILE = kTileRows * DKP * 2, VTILE = kTileRows * DVP * 2;
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t sQ = smem_u32(smem);
    const uint32_t sK = sQ + KTILE;                        // two stages
    const uint32_t sV = sK + 2 * KTILE;                    // two stages

    const int b = blockIdx.z, kvh = blockIdx.y;
    const int tile = blockIdx.x / n_splits, split = blockIdx.x % n_splits;
    const int group = n_heads / n_kv;
    const int q_begin = cu_seqlens[b];
    const int q_len = cu_seqlens[b + 1] - q_begin;
    const int n_rows = q_len * group;                      // (token, head of the group) pairs of this sequence
    if (tile * kTileRows >= n_rows) return;
    const int start = start_pos[b];
    const int* table = block_table + (size_t)slots[b] * table_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;

    const int rows_here = min(kTileRows, n_rows - tile * kTileRows);
    const int tok_first = (tile * kTileRows) / group, tok_last = (tile * kTileRows + rows_here - 1) / group;
    const int kv_total = start + q_len;                    // keys that exist after this step
    const int k_max = start + tok_last;
    const int k_min = first_seen(start + tok_first, window, chunk);
    const int p_first = k_min / kPageTokens, p_last = k_max / kPageTokens;
    const int n_pages = p_last - p_first + 1;
    const int per_split = (n_pages + n_splits - 1) / n_splits;
    const int j_lo = p_first + split * per_split;
    const int j_hi = min(p_last, j_lo + per_split - 1);

    // this thread's two rows of the warp's sixteen: where they go and what they see
    int row_tok[2], row_head[2], row_pos[2];
    bool row_ok[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + g + r * 8;
        row_ok[r] = row < rows_here;
        const int rr = tile * kTileRows + (row_ok[r] ? row : rows_here - 1);
        row_tok[r] = rr / group;
        row_head[r] = kvh * group + rr % group;
        row_pos[r] = start + row_tok[r];
    }
    if (j_lo > j_hi) {
        // nothing of this tile falls to this share: say so (the merge passes over it)
        if (t4 == 0) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                if (!row_ok[r]) continue;
                const size_t pidx = ((size_t)(q_begin + row_tok[r]) * n_heads + row_head[r]) * n_splits + split;
                part_ml[pidx * 2] = -INFINITY;
                part_ml[pidx * 2 + 1] = 0.f;
            }
        }
        return;
    }

    // ---- stage the query rows
    for (int id = tid; id < kTileRows * KCPR; id += 128) {
        const int r = id / KCPR, c = id % KCPR;
        const bool ok = r < rows_here && c * 8 < hd;
        const int rr = tile * kTileRows + r;
        const bf16* src = ok ? q + (size_t)(q_begin + rr / group) * ldq + (size_t)(kvh * group + rr % group) * hd + c * 8 : q;
        cp_async16(sQ + swz_offset<DKP>(r, c), src, ok ? 16 : 0);
    }
    auto load_kv = [&](int stage, int j) {
        const size_t page = (size_t)table[j] * page_stride;
        const size_t kbase = page + (size_t)kvh * kPageTokens * hd, vbase = page + (size_t)kvh * kPageTokens * vd;
        for (int id = tid; id < kTileRows * KCPR; id += 128) {
            const int r = id / KCPR, c = id % KCPR;
            const bool ok = (j * kPageTokens + r) < kv_total && c * 8 < hd;
            cp_async16(sK + stage * KTILE + swz_offset<DKP>(r, c), kc + (ok ? kbase + (size_t)r * hd + c * 8 : 0), ok ? 16 : 0);
        }
        for (int id = tid; id < kTileRows * VCPR; id += 128) {
            const int r = id / VCPR, c = id % VCPR;
            const bool ok = (j * kPageTokens + r) < kv_total && c * 8 < vd;
            cp_async16(sV + stage * VTILE + swz_offset<DVP>(r, c), vc + (ok ? vbase + (size_t)r * vd + c * 8 : 0), ok ? 16 : 0);
        }
    };
    load_kv(0, j_lo);
    cp_async_commit();

    uint32_t qf[DKP / 16][4];
    float o[DVP / 8][4];
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_row[2] = {-INFINITY, -INFINITY};   // running max of scaled scores (log2 domain)
    float l_row[2] = {0.f, 0.f};               // this thread's share of the running sum
    // with a cap the scores are scaled and capped as they leave the product, and only log2(e) is left to multiply
    const float sl2 = softcap > 0.f ? kLog2e : scale * kLog2e;
    const float cap_in = softcap > 0.f ? scale / softcap : 0.f;
    // what every row of this warp sees of a page without looking closer: the first row's position
    // bounds the keys from above, the last row's first seen key from below
    const int w_first = tile * kTileRows + warp * 16, w_last = min(w_first + 15, tile * kTileRows + rows_here - 1);
    const int warp_pos_lo = start + w_first / group;
    const int warp_seen_hi = w_last >= w_first ? first_seen(start + w_last / group, window, chunk) : 0;
    int row_lo[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) row_lo[r] = first_seen(row_pos[r], window, chunk);

    // a warp none of whose sixteen rows exists (three of four in a decode step of four heads a group) stages
    // pages with the others and computes nothing
    const bool warp_live = warp * 16 < rows_here;
    for (int j = j_lo, it = 0; j <= j_hi; ++j, ++it) {
        const int stage = it & 1;
        if (j + 1 <= j_hi) {
            load_kv(stage ^ 1, j + 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (warp_live) {
            if (it == 0) {
#pragma unroll
                for (int kk = 0; kk < DKP / 16; ++kk) {
                    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int c = kk * 2 + (lane >> 4);
                    ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], sQ + swz_offset<DKP>(r, c));
                }
            }
            // ---- S = Q K^T for this warp's 16 rows and the page's 64 keys
            float s[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
            const uint32_t kbase = sK + stage * KTILE, vbase = sV + stage * VTILE;
#pragma unroll
            for (int kk = 0; kk < DKP / 16; ++kk) {
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    uint32_t b0, b1, b2, b3;
                    const int r = jj * 16 + (lane & 7) + (lane >> 4) * 8;
                    const int c = kk * 2 + ((lane >> 3) & 1);
                    ldmatrix_x4(b0, b1, b2, b3, kbase + swz_offset<DKP>(r, c));
                    mma_bf16_16816(s[jj * 2], qf[kk], b0, b1);
                    mma_bf16_16816(s[jj * 2 + 1], qf[kk], b2, b3);
                }
            }
            if (softcap > 0.f) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[i][e] = softcap * tanh_by_exp(s[i][e] * cap_in);
                }
            }
            // ---- mask by position (only pages that cross an edge for some row of this warp)
            const bool all_visible = (j * kPageTokens + kPageTokens - 1 <= warp_pos_lo) && (j * kPageTokens >= warp_seen_hi);
            if (!all_visible) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = j * kPageTokens + i * 8 + t4 * 2 + (e & 1);
                        const int r = e >> 1;
                        if (key > row_pos[r] || key < row_lo[r]) s[i][e] = -INFINITY;
                    }
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[i][e]);
            }
            float corr[2], m_use[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_row[r], mx[r] * sl2);          // scale > 0: max commutes with it
                m_use[r] = m_new == -INFINITY ? 0.f : m_new;
                corr[r] = fast_exp2(m_row[r] - m_use[r]);
                m_row[r] = m_new;
                l_row[r] *= corr[r];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = fast_exp2(fmaf(s[i][e], sl2, -m_use[e >> 1]));
                    s[i][e] = p;
                    l_row[e >> 1] += p;
                }
            }
#pragma unroll
            for (int i = 0; i < DVP / 8; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
            // ---- O += P V
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t pa[4];
                pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dd = 0; dd < DVP / 16; ++dd) {
                    uint32_t b0, b1, b2, b3;
                    const int r = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                    const int c = dd * 2 + (lane >> 4);
                    ldmatrix_x4_trans(b0, b1, b2, b3, vbase + swz_offset<DVP>(r, c));
                    mma_bf16_16816(o[dd * 2], pa, b0, b1);
                    mma_bf16_16816(o[dd * 2 + 1], pa, b2, b3);
                }
            }
        }
        __syncthreads();
    }

    // ---- the rows' sums; then the output, or this share of it
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 1);
        l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (!row_ok[r]) continue;
        const size_t th = (size_t)(q_begin + row_tok[r]) * n_heads + row_head[r];
        if (n_splits > 1) {
            const size_t pidx = th * n_splits + split;
            float* po = part_o + pidx * DVP;
#pragma unroll
            for (int i = 0; i < DVP / 8; ++i)
                *reinterpret_cast<float2*>(po + i * 8 + t4 * 2) = make_float2(o[i][r * 2], o[i][r * 2 + 1]);
            if (t4 == 0) { part_ml[pidx * 2] = m_row[r]; part_ml[pidx * 2 + 1] = l_row[r]; }
            continue;
        }
        const float inv = l_row[r] > 0.f ? ((gate && gate_ld <= 0) ? gate[th] : 1.0f) / l_row[r] : 0.f;
        bf16* dst = out + (size_t)(q_begin + row_tok[r]) * ldo + (size_t)row_head[r] * vd;
        const float* logits = (gate && gate_ld > 0) ? gate + (size_t)(q_begin + row_tok[r]) * gate_ld + (size_t)row_head[r] * vd : nullptr;
#pragma unroll
        for (int i = 0; i < DVP / 8; ++i) {
            const int d = i * 8 + t4 * 2;
            if (d < vd) {
                float a = o[i][r * 2] * inv, b = o[i][r * 2 + 1] * inv;
                if (logits) {
                    a *= 1.0f / (1.0f + expf(-logits[d]));
                    b *= 1.0f / (1.0f + expf(-logits[d + 1]));
                }
                *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(a, b);
            }
        }
    }
}

// One block per (token, query head): the shares in order, each scaled to the common maximum.
__global__ void attention_masked_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              bf16* __restrict__ out, int ldo, const float* __restrict__ gate,
                                              int n_heads, int vd, int dvp, int n_splits, int gate_ld) {
    chain_release();
    chain_wait();
    const size_t th = blockIdx.x;
    const int n = (int)(th / n_heads), h = (int)(th % n_heads);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(th * n_splits + s) * 2]);
    const float Mu = M == -INFINITY ? 0.f : M;
    for (int d = threadIdx.x; d < vd; d += blockDim.x) {
        float acc = 0.f, L = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const size_t pidx = th * n_splits + s;
            const float m = part_ml[pidx * 2];
            if (m == -INFINITY) continue;            // a share without keys wrote no output
            const float f = exp2f(m - Mu);
            acc += f * part_o[pidx * dvp + d];
            L += f * part_ml[pidx * 2 + 1];
        }
        const float gt = !gate ? 1.0f : gate_ld <= 0 ? gate[th] : 1.0f / (1.0f + expf(-gate[(size_t)n * gate_ld + (size_t)h * vd + d]));
        out[(size_t)n * ldo + (size_t)h * vd + d] = __float2bfloat16_rn(L > 0.f ? acc * gt / L : 0.f);
    }
}

inline int padded(int d) { return d <= 64 ? 64 : 128; }

template <int DKP, int DVP>
int launch_masked(const bf16* q, int ldq, bf16* out, int ldo, const bf16* kc, const bf16* vc, long long page_stride,
                  const int* block_table, int table_stride, const int* cu_seqlens, const int* slots, const int* start_pos,
                  int n_seqs, int tiles, int n_heads, int n_kv, int hd, int vd, float scale, int window, int chunk,
                  const float* gate, int n_splits, float* part_o, float* part_ml, float softcap, int gate_ld, cudaStream_t stream) {
    auto kernel = attention_masked_kernel<DKP, DVP>;
    constexpr int smem = masked_smem_bytes<DKP, DVP>();
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return launch_chained(kernel, dim3(tiles * n_splits, n_kv, n_seqs), dim3(128), smem, stream, q, ldq, out, ldo, kc, vc,
                          page_stride, block_table, table_stride, cu_seqlens, slots, start_pos, n_heads, n_kv, hd, vd, scale,
                          window, chunk, gate, n_splits, part_o, part_ml, softcap, gate_ld);
}
}  // namespace

// Whether the tensor-core kernel takes heads of these widths (else: the plain kernel).
GTG_API int gtg_attention_masked_supports(int hd, int vd) {
    return hd > 0 && vd > 0 && hd % 8 == 0 && vd % 8 == 0 && hd <= 128 && vd <= 128;
}

// Floats of scratch that `n_splits` shares need: per (token, head, share) the padded output, maximum and sum.
GTG_API long long gtg_attention_masked_scratch_floats(int n_tokens, int n_heads, int vd, int n_splits) {
    if (n_splits <= 1) return 0;
    return (long long)n_tokens * n_heads * n_splits * (padded(vd) + 2);
}

// Into how many shares the pages of a step's tiles are cut: 1 while the tiles alone fill the device;
// else as many as bring about two blocks per multiprocessor, each share two pages at least.
GTG_API int gtg_attention_masked_splits(int n_seqs, int max_q_len, int n_heads, int n_kv, int max_kv_len, int window, int chunk) {
    if (n_seqs <= 0 || n_kv <= 0) return 1;
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int group = n_heads / n_kv;
    const long long tiles = ((long long)max_q_len * group + kTileRows - 1) / kTileRows;
    const long long blocks = tiles * n_kv * n_seqs;
    int keys = max_kv_len;
    if (window > 0) keys = min(keys, window + max_q_len);
    if (chunk > 0) keys = min(keys, chunk);
    const int pages = (keys + kPageTokens - 1) / kPageTokens + 1;
    if (blocks >= 2LL * sms || pages < 4) return 1;
    long long want = (2LL * sms + blocks - 1) / blocks;
    want = min(want, (long long)pages / 2);
    return (int)max(1LL, min(want, 32LL));
}

GTG_API int gtg_attention_masked_bf16(const void* q, int ldq, void* out, int ldo, const void* kc, const void* vc,
                                      long long page_stride, const int* block_table, int table_stride,
                                      const int* cu_seqlens, const int* slots, const int* start_pos, int n_seqs, int max_q_len,
                                      int n_tokens, int n_heads, int n_kv, int hd, int vd, float scale, int window, int chunk,
                                      const float* gate, int n_splits, float* scratch, float softcap, int gate_ld,
                                      cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || window < 0 || chunk < 0 || n_splits < 1) return kErrBadArgument;
    if (softcap < 0.f || (gate && gate_ld > 0 && gate_ld < n_heads * vd)) return kErrBadArgument;
    if (!gtg_attention_masked_supports(hd, vd)) return kErrUnsupported;
    if (n_splits > 1 && !scratch) return kErrBadArgument;
    if (ldq % 8 || page_stride % 8 || ((uintptr_t)q % 16) || ((uintptr_t)kc % 16) || ((uintptr_t)vc % 16) || ldo % 2 ||
        ((uintptr_t)out % 4)) return kErrUnsupported;
    const int group = n_heads / n_kv;
    const long long tiles = ((long long)max_q_len * group + kTileRows - 1) / kTileRows;
    if (tiles * n_splits > 0x7fffffffLL || n_seqs > 65535 || n_kv > 65535) return kErrUnsupported;
    const int dvp = padded(vd);
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)n_tokens * n_heads * n_splits * dvp : nullptr;
#define GTG_MASKED(DKP, DVP)                                                                                          \
    launch_masked<DKP, DVP>((const bf16*)q, ldq, (bf16*)out, ldo, (const bf16*)kc, (const bf16*)vc, page_stride,       \
                            block_table, table_stride, cu_seqlens, slots, start_pos, n_seqs, (int)tiles, n_heads, n_kv, \
                            hd, vd, scale, window, chunk, gate, n_splits, part_o, part_ml, softcap, gate_ld, stream)
    int st;
    if (padded(hd) == 64) st = dvp == 64 ? GTG_MASKED(64, 64) : GTG_MASKED(64, 128);
    else st = dvp == 64 ? GTG_MASKED(128, 64) : GTG_MASKED(128, 128);
#undef GTG_MASKED
    if (st != 0 || n_splits == 1) return st;
    return launch_chained(attention_masked_merge_kernel, dim3((unsigned)((long long)n_tokens * n_heads)), dim3(dvp >= 128 ? 128 : 64),
                          0, stream, (const float*)part_o, (const float*)part_ml, (bf16*)out, ldo, gate, n_heads, vd, dvp, n_splits, gate_ld);
}
