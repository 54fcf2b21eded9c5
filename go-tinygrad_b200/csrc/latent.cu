// Attention through a latent: what stands between the projections and the
// attention kernel.
//
// A token leaves two things in the cache instead of keys and values per head: a
// latent vector c of `rank` channels, normed (c = x / sqrt(mean(x^2) + eps) * w
// over the rank channels of the down projection), and one rotated key part of
// `rot` channels that all heads share.  A cache row is [c | rotated part]:
// rank + rot channels of a single key/value head.  Head h's unrotated key would
// be U_h c; its score against a query q_h = [a_h | b_h] is
//     a_h . (U_h c) + b_h' . k'  =  (U_h^T a_h) . c + b_h' . k'        (' = rotated)
// so the query that meets the cache row is [U_h^T a_h | b_h'], also rank + rot
// channels, and the value of a row is its first rank channels.
//
// latent_prepare, one block per token, does the per-token work in float:
//   * with a down projection: the norm of the latent, the rotation of the shared
//     key part, and the store of both into the token's cache row;
//   * the rotation of every head's b_h into the tail of the head's query row
//     (the head of the row is written by the product with U_h^T), or, without
//     such rows (q_full null), in place.
// rows_out, if given, receives the token's cache row once more, token by token.
// Rotation: of the part's first `rdims` channels, (2i, 2i+1) (`interleaved`) or (i, i + rdims/2) turn by the
// angle of pair i, whose cosine and sine (amplitude included) come from the step's table [token, rdims/2].
#include "mma_helpers.cuh"
#include <math.h>

namespace {
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(T* __restrict__ q, int ldq, const T* __restrict__ dkv, int ldd,
                      const float2* __restrict__ cos_sin, const float* __restrict__ norm_w, float eps,
                      T* __restrict__ kc, long long page_stride, const int* __restrict__ block_table,
                      int table_stride, const int* __restrict__ token_seq, const int* __restrict__ slots,
                      const int* __restrict__ positions, T* __restrict__ q_full, int ldf,
                      int n_heads, int dim, int rot, int rdims, int rank, T* __restrict__ rows_out, int ldo,
                      int interleaved) {
    chain_release();
    chain_wait();
    __shared__ float scratch[33];
    const int n = blockIdx.x;
    const int half = rdims / 2;   // pairs that turn; channels rdims..rot-1 of the part pass unchanged
    const int pa = interleaved ? 2 : 1, pb = interleaved ? 1 : half;     // pair i is channels (pa * i, pa * i + pb)
    const float2* cs = cos_sin + (size_t)n * half;
    if (dkv) {
        const T* d = dkv + (size_t)n * ldd;
        float ss = 0.f;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) {
            const float x = to_f32<T>(d[i]);
            ss += x * x;
        }
        const float total = block_sum(ss, scratch);
        const float s = 1.0f / sqrtf(total / (float)rank + eps);
        const int pos = positions[n];
        const int slot = slots[token_seq[n]];
        const int page = block_table[(size_t)slot * table_stride + pos / kPageTokens];
        T* row = kc + (size_t)page * page_stride + (size_t)(pos % kPageTokens) * (rank + rot);
        T* copy = rows_out ? rows_out + (size_t)n * ldo : nullptr;      // the same row, token by token, for the step's own use
        for (int i = threadIdx.x; i < rank; i += blockDim.x) {
            row[i] = from_f32<T>((norm_w[i] * to_f32<T>(d[i])) * s);
            if (copy) copy[i] = row[i];
        }
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const int ia = pa * i, ib = ia + pb;
            const float u = to_f32<T>(d[rank + ia]), v = to_f32<T>(d[rank + ib]);
            const float2 a = cs[i];
            row[rank + ia] = from_f32<T>(u * a.x - v * a.y);
            row[rank + ib] = from_f32<T>(v * a.x + u * a.y);
            if (copy) { copy[rank + ia] = row[rank + ia]; copy[rank + ib] = row[rank + ib]; }
        }
        for (int i = rdims + threadIdx.x; i < rot; i += blockDim.x) {
            row[rank + i] = d[rank + i];
            if (copy) copy[rank + i] = d[rank + i];
        }
    }
    if (!q_full) {
        // the rotated parts go back where they came from: the query rows stay [a_h | b_h'] per head
        for (int idx = threadIdx.x; idx < n_heads * half; idx += blockDim.x) {
            const int h = idx / half, i = idx % half;
            T* p = q + (size_t)n * ldq + (size_t)h * (dim + rot) + dim;
            const int ia = pa * i, ib = ia + pb;
            const float u = to_f32<T>(p[ia]), v = to_f32<T>(p[ib]);
            const float2 a = cs[i];
            p[ia] = from_f32<T>(u * a.x - v * a.y);
            p[ib] = from_f32<T>(v * a.x + u * a.y);
        }
        return;
    }
    const int D = rank + rot;
    for (int idx = threadIdx.x; idx < n_heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx % half;
        const T* src = q + (size_t)n * ldq + (size_t)h * (dim + rot) + dim;
        const int ia = pa * i, ib = ia + pb;
        const float u = to_f32<T>(src[ia]), v = to_f32<T>(src[ib]);
        const float2 a = cs[i];
        T* dst = q_full + (size_t)n * ldf + (size_t)h * D + rank;
        dst[ia] = from_f32<T>(u * a.x - v * a.y);
        dst[ib] = from_f32<T>(v * a.x + u * a.y);
    }
    for (int idx = threadIdx.x; idx < n_heads * (rot - rdims); idx += blockDim.x) {
        const int h = idx / (rot - rdims), i = rdims + idx % (rot - rdims);
        q_full[(size_t)n * ldf + (size_t)h * D + rank + i] = q[(size_t)n * ldq + (size_t)h * (dim + rot) + dim + i];
    }
}
}  // namespace

GTG_API int gtg_latent_prepare(int dtype, void* q, int ldq, const void* dkv, int ldd, const float* cos_sin,
                               const float* norm_w, float eps, void* kc, long long page_stride,
                               const int* block_table, int table_stride, const int* token_seq, const int* slots,
                               const int* positions, void* q_full, int ldf, int N, int n_heads, int dim, int rot,
                               int rdims, int rank, void* rows_out, int ldo, int interleaved, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_heads <= 0 || dim <= 0 || rot <= 0 || rdims < 0 || rdims > rot || rdims % 2 || rank <= 0) return kErrBadArgument;
    if (dkv && (!kc || !norm_w || !block_table)) return kErrBadArgument;
    if (dtype == 0)
        return launch_chained(latent_prepare_kernel<float>, dim3(N), dim3(128), 0, stream, (float*)q, ldq,
                              (const float*)dkv, ldd, (const float2*)cos_sin, norm_w, eps, (float*)kc, page_stride,
                              block_table, table_stride, token_seq, slots, positions, (float*)q_full, ldf, n_heads,
                              dim, rot, rdims, rank, (float*)rows_out, ldo, interleaved);
    if (dtype == 1)
        return launch_chained(latent_prepare_kernel<bf16>, dim3(N), dim3(128), 0, stream, (bf16*)q, ldq,
                              (const bf16*)dkv, ldd, (const float2*)cos_sin, norm_w, eps, (bf16*)kc, page_stride,
                              block_table, table_stride, token_seq, slots, positions, (bf16*)q_full, ldf, n_heads,
                              dim, rot, rdims, rank, (bf16*)rows_out, ldo, interleaved);
    return kErrBadArgument;
}

// ---- attention over the latent rows, on the warp-level tensor cores ------------------
// All heads of a token meet the same cache rows, so the (token, head) pairs of a
// sequence's new tokens are one list of query rows; a thread block takes 32
// consecutive ones (two tokens of 16 heads, a quarter of a token of 128, eleven
// of 3) and walks the pages their windows span, each page staged once in shared
// memory by the copy engine (a bulk copy a row, counted on the page's barrier; waits
// are bounded), two pages in flight.  Per page, sixteen warps as 2 row
// groups x 8: first every warp multiplies its 16 query rows with an eighth of
// the page's 64 keys over all rank + rot channels (S, float), the row maxima and
// sums meet through shared memory (streaming softmax in float, powers of two), the
// weights go to shared memory as bfloat16; then every warp adds, for its 16
// rows, an eighth of the value channels: O[16, rank/8] += P[16, 64] . page[64,
// eighth], the page's first rank columns read transposed (ldmatrix.trans).  O
// stays in registers (up to 32 floats a thread at rank 512).  Sixteen warps, not
// eight, because a block has a multiprocessor to itself (its staged pages fill the
// shared memory) and two warps a scheduler hid too little latency.  Prompts, portions
// and single tokens are one code path; a row sees keys lo..pos of its sequence,
// lo = 0 or pos - window + 1.  Needs rank + rot a multiple of 16 and rank of 8.

// 0, or 1 if a block ever gave up waiting for a page it had asked for (it then went on with
// whatever the buffer held: the result of that launch is not to be used).
__device__ int g_latent_status = 0;
static bool g_latent_test_waits = false;       // set by the test hook

namespace {
constexpr unsigned kPageWaitLimit = 1u << 22;      // polls of a page's barrier before a block gives up

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// Polls until the phase with `parity` completes or the limit is hit (then the status word is set).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned limit) {
    for (unsigned i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                     "selp.u32 %0, 1, 0, p;\n}\n" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    atomicExch(&g_latent_status, 1);
    return false;
}
// One row of `bytes` (a multiple of 16, both addresses 16-byte aligned) global -> shared by the copy
// engine; its arrival is counted on the barrier.
__device__ __forceinline__ void bulk_row(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// 2^x by the special-function unit (the bfloat16 attention kernels of this library all do: scores are
// scaled by log2(e) so that exponentials are powers of two).  ex2(-inf) = 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
constexpr float kLog2e = 1.4426950408889634f;

constexpr int kTileRows = 32;
constexpr int kLatThreads = 512;
constexpr int kParts = 8;            // warps that share a row group: each takes 8 of a page's 64 keys, then an eighth of the value channels
constexpr int kPad = 8;              // bfloat16 of padding per staged row: rows fall into different banks

template <int NT>                    // value n-tiles (8 channels) per warp at most: rank <= 64 * NT
__global__ void __launch_bounds__(kLatThreads)
latent_attention_mma_kernel(const bf16* __restrict__ q, int ldq, bf16* __restrict__ out, int ldo,
                            const bf16* __restrict__ kc, long long page_stride, const int* __restrict__ block_table,
                            int table_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                            const int* __restrict__ start_pos, int n_heads, int D, int rank, float scale, int window,
                            int n_splits, float* __restrict__ scratch, int total_rows, int test_waits,
                            const float* __restrict__ sinks) {
    // sinks (or null): float [n_heads]; exp(sinks[h]) joins head h's softmax denominator without a key or a value
    // (with several runs of keys the merge kernel adds it).
    // test_waits (the test hook's form of the launch): no page is ever copied and a wait polls a thousand
    // times, so that every wait runs out, the status word is set and the block still returns
    chain_release();
    chain_wait();
    extern __shared__ __align__(128) unsigned char smem[];
    const int b = blockIdx.y;
    const int tok0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - tok0;
    const int r0 = blockIdx.x * kTileRows;
    if (r0 >= n_new * n_heads) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rg = warp & 1, part_i = warp >> 1;
    const int g = lane >> 2, t = lane & 3;
    const int ldr = D + kPad;                                   // staged row, in elements
    bf16* q_s = reinterpret_cast<bf16*>(smem);                  // [32][ldr]
    bf16* page_s = q_s + kTileRows * ldr;                       // [2][64][ldr]
    bf16* p_s = page_s + 2 * kPageTokens * ldr;                 // [32][64 + kPad]
    float* part = reinterpret_cast<float*>(p_s + kTileRows * (kPageTokens + kPad));   // [2][8][32]: maxima, sums
    int* row_pos = reinterpret_cast<int*>(part + 2 * kParts * kTileRows);                  // [32] position or -1
    const uint32_t bars = smem_u32(row_pos + kTileRows);        // two barriers of 8 bytes: a staged page has arrived
    volatile int* gave_up = row_pos + kTileRows + 4;            // set by a thread whose wait ran out
    const int start = start_pos[b];
    const int* table = block_table + (size_t)slots[b] * table_stride;
    const int last_row = min(r0 + kTileRows, n_new * n_heads) - 1;
    const int pos_min = start + r0 / n_heads, pos_max = start + last_row / n_heads;
    const int lo_min = (window > 0 && pos_min - window + 1 > 0) ? pos_min - window + 1 : 0;
    int page_lo = lo_min / kPageTokens, page_hi = pos_max / kPageTokens;
    if (n_splits > 1) {
        // the pages of the tile in n_splits equal runs; this block takes run blockIdx.z and leaves
        // (maximum, sum, unnormalised values) of its rows in `scratch` for the merge kernel
        const int chunk = (page_hi - page_lo + n_splits) / n_splits;
        page_lo += blockIdx.z * chunk;
        page_hi = min(page_hi, page_lo + chunk - 1);
        if (page_lo > page_hi) {
            if (tid < kTileRows && r0 + tid <= last_row) {
                float* dst = scratch + ((size_t)blockIdx.z * total_rows + (size_t)tok0 * n_heads + r0 + tid) * (rank + 2);
                dst[0] = -INFINITY;
                dst[1] = 0.f;
            }
            return;
        }
    }
    if (tid < kTileRows) {
        const int r = r0 + tid;
        row_pos[tid] = r < n_new * n_heads ? start + r / n_heads : -1;
    }
    const int chunks = D / 8;
    for (int r = warp; r < kTileRows; r += kLatThreads / 32) {
        const int row = r0 + r;
        const bool ok = row < n_new * n_heads;
        const bf16* src = ok ? q + (size_t)(tok0 + row / n_heads) * ldq + (size_t)(row % n_heads) * D : q;
        for (int c = lane; c < chunks; c += 32)
            cp_async16(smem_u32(q_s + r * ldr + c * 8), ok ? src + c * 8 : q, ok ? 16 : 0);
    }

    // A page is staged by the copy engine, a row a copy (64 copies, two a lane of warp 0), so that no
    // warp that multiplies waits in a queue of copies; the page's barrier counts the bytes.
    if (tid == 0) {
        *gave_up = 0;
        mbar_init(bars, 1);
        mbar_init(bars + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::);
    }
    __syncthreads();                                            // barriers and row_pos
    auto load_page = [&](int buf, int p) {
        // every warp asks for its own share of the rows (a few lanes of one instruction): copies asked for by
        // one warp alone hold that warp, and with it the block, for as long as the copy engine takes them in
        const bf16* src = kc + (size_t)table[p] * page_stride;
        const uint32_t dst = smem_u32(page_s + (size_t)buf * kPageTokens * ldr);
        if (tid == 0) mbar_expect_tx(bars + 8 * buf, (uint32_t)(kPageTokens * D * 2));
        if (test_waits) return;
        constexpr int kShare = kPageTokens / (kLatThreads / 32);
        if (lane < kShare) {
            const int r = warp * kShare + lane;
            bulk_row(dst + (uint32_t)(r * ldr * 2), src + (size_t)r * D, (uint32_t)(D * 2), bars + 8 * buf);
        }
    };
    const int n_pages = page_hi - page_lo + 1;
    load_page(0, page_lo);
    cp_async_commit();                                          // the query rows

    const int tiles_total = rank / 8;
    const int per = (tiles_total + kParts - 1) / kParts;
    const int tile_lo = part_i * per;
    const int my_tiles = max(0, min(per, tiles_total - tile_lo));
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    cp_async_wait<0>();                                         // this thread's share of the query rows
    // a row group without a live row (a decode step of at most 16 heads fills one group of two)
    // multiplies nothing; it still stages pages and meets the barriers
    const bool rg_live = r0 + rg * 16 <= last_row;
    int pos_r[2], lo_r[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        pos_r[hh] = row_pos[rg * 16 + g + hh * 8];
        lo_r[hh] = (window > 0 && pos_r[hh] - window + 1 > 0) ? pos_r[hh] - window + 1 : 0;
    }

    for (int i = 0; i < n_pages; ++i) {
        const int p = page_lo + i;
        const int buf = i & 1;
        if (i > 0) __syncthreads();                             // everyone is done with the page before and its weights
        // A wait ran out: the block stops asking and waiting (a barrier whose phase never completed must
        // not be armed again) and goes on to its end with what it has; everyone sees the flag alike here.
        if (*gave_up) break;
        if (i + 1 < n_pages) load_page(buf ^ 1, p + 1);
        if (!mbar_wait(bars + 8 * buf, ((uint32_t)i >> 1) & 1u, test_waits ? 1024u : kPageWaitLimit)) *gave_up = 1;   // else page p has arrived
        if (i == 0) __syncthreads();                            // and everyone's share of the query rows
        const bf16* pg = page_s + (size_t)buf * kPageTokens * ldr;
        // S: rows rg*16.., keys part_i*8.. of the page
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        if (rg_live) {
            // fragments of channel step k+1 are asked for before the product of step k is issued, and
            // even and odd steps add into accumulators of their own: two chains instead of one
            const uint32_t a_addr = smem_u32(q_s + (rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldr + (lane >> 4) * 8);
            const uint32_t b_addr = smem_u32(pg + (part_i * 8 + (lane & 7)) * ldr + ((lane >> 3) & 1) * 8);
            const int n_ks = D / 16;
            float s2[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t a0[4], b0[2], a1[4], b1[2];
            ldmatrix_x4(a0[0], a0[1], a0[2], a0[3], a_addr);
            ldmatrix_x2(b0[0], b0[1], b_addr);
            int ks = 0;
            for (; ks + 2 <= n_ks; ks += 2) {
                ldmatrix_x4(a1[0], a1[1], a1[2], a1[3], a_addr + (ks + 1) * 32);
                ldmatrix_x2(b1[0], b1[1], b_addr + (ks + 1) * 32);
                mma_bf16_16816(s, a0, b0[0], b0[1]);
                if (ks + 2 < n_ks) {
                    ldmatrix_x4(a0[0], a0[1], a0[2], a0[3], a_addr + (ks + 2) * 32);
                    ldmatrix_x2(b0[0], b0[1], b_addr + (ks + 2) * 32);
                }
                mma_bf16_16816(s2, a1, b1[0], b1[1]);
            }
            if (ks < n_ks) mma_bf16_16816(s, a0, b0[0], b0[1]);
#pragma unroll
            for (int e = 0; e < 4; ++e) s[e] += s2[e];
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int hh = e >> 1;
            const int key = p * kPageTokens + part_i * 8 + t * 2 + (e & 1);
            const bool seen = pos_r[hh] >= 0 && key <= pos_r[hh] && key >= lo_r[hh];
            s[e] = seen ? s[e] * (scale * kLog2e) : -INFINITY;
            mx[hh] = fmaxf(mx[hh], s[e]);
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
            if (t == 0) part[part_i * kTileRows + rg * 16 + g + hh * 8] = mx[hh];
        }
        __syncthreads();
        float corr[2], sum[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int r = rg * 16 + g + hh * 8;
            float m_new = m_run[hh];
#pragma unroll
            for (int qq = 0; qq < kParts; ++qq) m_new = fmaxf(m_new, part[qq * kTileRows + r]);
            corr[hh] = m_new == -INFINITY ? 1.f : fast_exp2(m_run[hh] - m_new);
            m_run[hh] = m_new;
            const float p0 = m_new == -INFINITY ? 0.f : fast_exp2(s[hh * 2] - m_new);
            const float p1 = m_new == -INFINITY ? 0.f : fast_exp2(s[hh * 2 + 1] - m_new);
            const __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
            // the sum runs over the rounded weights, the ones the values are multiplied with
            sum[hh] = __bfloat162float(pr.x) + __bfloat162float(pr.y);
            *reinterpret_cast<__nv_bfloat162*>(p_s + r * (kPageTokens + kPad) + part_i * 8 + t * 2) = pr;
            sum[hh] += __shfl_xor_sync(0xffffffffu, sum[hh], 1);
            sum[hh] += __shfl_xor_sync(0xffffffffu, sum[hh], 2);
            if (t == 0) part[kParts * kTileRows + part_i * kTileRows + r] = sum[hh];
        }
        __syncthreads();
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int r = rg * 16 + g + hh * 8;
            float total = 0.f;
#pragma unroll
            for (int qq = 0; qq < kParts; ++qq) total += part[kParts * kTileRows + qq * kTileRows + r];
            l_run[hh] = l_run[hh] * corr[hh] + total;
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
        }
        // O += P . page[:, my value channels]
        if (rg_live) {
            // per 16 keys: the value fragments of up to eight channel tiles are asked for together, then multiplied
            const uint32_t a_addr = smem_u32(p_s + (rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * (kPageTokens + kPad) + (lane >> 4) * 8);
            const uint32_t v_addr = smem_u32(pg + ((lane & 7) + ((lane >> 3) & 1) * 8) * ldr + tile_lo * 8 + (lane >> 4) * 8);
            constexpr int CH = NT < 8 ? NT : 8;
#pragma unroll
            for (int ks = 0; ks < kPageTokens / 16; ++ks) {
                uint32_t a[4];
                ldmatrix_x4(a[0], a[1], a[2], a[3], a_addr + ks * 32);
#pragma unroll
                for (int c = 0; c < NT; c += CH) {
                    uint32_t v[CH / 2][4];
#pragma unroll
                    for (int j = 0; j < CH; j += 2)
                        if (c + j < my_tiles)
                            ldmatrix_x4_trans(v[j / 2][0], v[j / 2][1], v[j / 2][2], v[j / 2][3], v_addr + (ks * 16 * ldr + (c + j) * 8) * 2);
#pragma unroll
                    for (int j = 0; j < CH; j += 2)
                        if (c + j < my_tiles) {
                            mma_bf16_16816(o[c + j], a, v[j / 2][0], v[j / 2][1]);
                            mma_bf16_16816(o[c + j + 1], a, v[j / 2][2], v[j / 2][3]);
                        }
                }
            }
        }
    }
    if (n_splits > 1) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            if (pos_r[hh] < 0) continue;
            float* dst = scratch + ((size_t)blockIdx.z * total_rows + (size_t)tok0 * n_heads + r0 + rg * 16 + g + hh * 8) * (rank + 2);
            if (part_i == 0 && t == 0) { dst[0] = m_run[hh]; dst[1] = l_run[hh]; }
#pragma unroll
            for (int j = 0; j < NT; ++j)
                if (j < my_tiles)
                    *reinterpret_cast<float2*>(dst + 2 + (tile_lo + j) * 8 + t * 2) = make_float2(o[j][hh * 2], o[j][hh * 2 + 1]);
        }
        return;
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int row = r0 + rg * 16 + g + hh * 8;
        if (pos_r[hh] < 0 || l_run[hh] <= 0.f) continue;
        const float inv = 1.0f / (l_run[hh] + (sinks ? exp2f(sinks[row % n_heads] * kLog2e - m_run[hh]) : 0.f));
        bf16* dst = out + (size_t)(tok0 + row / n_heads) * ldo + (size_t)(row % n_heads) * rank + tile_lo * 8 + t * 2;
#pragma unroll
        for (int j = 0; j < NT; ++j)
            if (j < my_tiles)
                *reinterpret_cast<__nv_bfloat162*>(dst + j * 8) = __floats2bfloat162_rn(o[j][hh * 2] * inv, o[j][hh * 2 + 1] * inv);
    }
}

// out[row, :] = sum_z exp(m_z - M) O_z / sum_z exp(m_z - M) l_z, M = max_z m_z: the runs of a row's
// keys brought together, z in order.
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* __restrict__ scratch, bf16* __restrict__ out, int ldo, int n_heads, int rank,
                              int n_splits, int total_rows, const float* __restrict__ sinks) {
    chain_release();
    chain_wait();
    __shared__ float ms[64], ls[64], ws[64];
    const int row = blockIdx.x;
    const size_t stride = (size_t)total_rows * (rank + 2);
    const float* base = scratch + (size_t)row * (rank + 2);
    if (threadIdx.x < n_splits) {
        ms[threadIdx.x] = base[threadIdx.x * stride];
        ls[threadIdx.x] = base[threadIdx.x * stride + 1];
    }
    __syncthreads();
    float M = -INFINITY;
    for (int z = 0; z < n_splits; ++z) M = fmaxf(M, ms[z]);
    if (M == -INFINITY) return;
    if (threadIdx.x < n_splits) ws[threadIdx.x] = ms[threadIdx.x] == -INFINITY ? 0.f : exp2f(ms[threadIdx.x] - M);   // maxima are in powers of two
    __syncthreads();
    float L = 0.f;
    for (int z = 0; z < n_splits; ++z) L = fmaf(ws[z], ls[z], L);
    if (sinks) L += exp2f(sinks[row % n_heads] * kLog2e - M);
    const float inv = 1.0f / L;
    bf16* dst = out + (size_t)(row / n_heads) * ldo + (size_t)(row % n_heads) * rank;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float acc = 0.f;
#pragma unroll 4
        for (int z = 0; z < n_splits; ++z)
            if (ws[z] != 0.f) acc = fmaf(ws[z], base[z * stride + 2 + c], acc);
        dst[c] = __float2bfloat16_rn(acc * inv);
    }
}

size_t latent_attention_smem(int D) {
    const size_t ldr = D + kPad;
    return (kTileRows + 2 * kPageTokens) * ldr * 2 + kTileRows * (kPageTokens + kPad) * 2 + 2 * kParts * kTileRows * 4 + kTileRows * 4 + 32;
}
}  // namespace

// 0, or 1 if a block of the attention kernel ever gave up a bounded wait for a staged page
// (reading it synchronises the device).
GTG_API int gtg_latent_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_latent_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// For tests of the give-up path only: while set, the attention kernel is launched in its test form
// (see the kernel).  The call synchronises the device and clears the status word.
GTG_API int gtg_latent_test_hooks(int test_waits) {
    const int zero = 0;
    cudaError_t e = cudaDeviceSynchronize();
    g_latent_test_waits = test_waits != 0;
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_latent_status, &zero, sizeof(zero));
    return (int)e;
}

// Whether the tensor-core kernel takes rows of D = rank + rot channels with `rank` value channels.
GTG_API int gtg_latent_attention_supports(int D, int rank) {
    return D > 0 && D % 16 == 0 && rank > 0 && rank % 8 == 0 && rank <= 512 && rank <= D && latent_attention_smem(D) <= 220 * 1024;
}

// Into how many runs the keys of a tile are best cut, for a step of n_seqs sequences that bring
// max_q_len tokens at most and reach max_kv_len keys at most: enough thread blocks for every
// place on the device twice over, runs of two pages at least.  1 for prompts.
GTG_API int gtg_latent_attention_splits(int n_seqs, int max_q_len, int n_heads, int D, int max_kv_len, int window) {
    static int sms = 0;
    if (!sms) {
        int dev = 0, n = 0;
        sms = (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
    }
    const long long tiles = (((long long)max_q_len * n_heads + kTileRows - 1) / kTileRows) * n_seqs;
    int keys = max_kv_len;
    if (window > 0 && window + max_q_len < keys) keys = window + max_q_len;
    const int pages = keys / kPageTokens + 1;
    const size_t per_sm = (size_t)220 * 1024 / latent_attention_smem(D);
    const long long places = 2LL * sms * (per_sm > 0 ? (long long)per_sm : 1);
    long long splits = (places + tiles - 1) / tiles;
    if (splits > pages / 2) splits = pages / 2;
    if (splits > 32) splits = 32;
    return splits < 1 ? 1 : (int)splits;
}

GTG_API long long gtg_latent_attention_scratch_floats(int total_rows, int rank, int n_splits) {
    return n_splits > 1 ? (long long)n_splits * total_rows * (rank + 2) : 0;
}

GTG_API int gtg_latent_attention_bf16(const void* q, int ldq, void* out, int ldo, const void* kc, long long page_stride,
                                      const int* block_table, int table_stride, const int* cu_seqlens, const int* slots,
                                      const int* start_pos, int n_seqs, int max_q_len, int n_heads, int D, int rank,
                                      float scale, int window, int n_splits, float* scratch, int n_tokens,
                                      const float* sinks, cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (n_heads <= 0) return kErrBadArgument;
    if (!gtg_latent_attention_supports(D, rank)) return kErrUnsupported;
    if (ldq % 8 || ((uintptr_t)q % 16) || ((uintptr_t)kc % 16) || page_stride % 8 || ldo % 2 || ((uintptr_t)out % 4)) return kErrUnsupported;
    const size_t smem = latent_attention_smem(D);
    const long long tiles = ((long long)max_q_len * n_heads + kTileRows - 1) / kTileRows;
    if (tiles > 0x7fffffffLL || n_seqs > 65535) return kErrUnsupported;
    if (n_splits < 1 || n_splits > 64 || (n_splits > 1 && (!scratch || rank % 2))) return kErrBadArgument;
    const dim3 grid((unsigned)tiles, n_seqs, n_splits);
    const int total_rows = n_tokens * n_heads;
#define GTG_LATENT(NT)                                                                                              \
    do {                                                                                                            \
        static bool configured = false;                                                                             \
        if (!configured) {                                                                                          \
            const cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel<NT>,                             \
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);    \
            if (e != cudaSuccess) return (int)e;                                                                    \
            configured = true;                                                                                      \
        }                                                                                                           \
        st = launch_chained(latent_attention_mma_kernel<NT>, grid, dim3(kLatThreads), smem, stream, (const bf16*)q, ldq, \
                            (bf16*)out, ldo, (const bf16*)kc, page_stride, block_table, table_stride, cu_seqlens, slots, \
                            start_pos, n_heads, D, rank, scale, window, n_splits, scratch, total_rows,              \
                            g_latent_test_waits ? 1 : 0, sinks);                                                   \
    } while (0)
    const int per = ((rank / 8) + kParts - 1) / kParts;
    int st = 0;
    if (per <= 2) GTG_LATENT(2); else if (per <= 4) GTG_LATENT(4); else GTG_LATENT(8);
#undef GTG_LATENT
    if (st != 0 || n_splits == 1) return st;
    return launch_chained(latent_attention_merge_kernel, dim3(total_rows), dim3(128), 0, stream, (const float*)scratch,
                          (bf16*)out, ldo, n_heads, rank, n_splits, total_rows, sinks);
}

// ---- prompts that start their sequences: keys and values expanded per head ---------------
// When every sequence of a step starts at its first token, the step's own rows are all the keys
// there are, and expanding them per head (K_h = U_h c, V_h = V_h c: two products over the step's
// latents) costs less than attending in the folded form: dim + rot channels per score and vdim
// per value instead of rank + rot and rank.  This kernel is the attention over those expanded
// rows: q [N, heads, dim + rot] (rotated part last, already rotated), and per token and head one
// run kv [N, heads, dim + vdim + rot] = [U_h c | V_h c | k'] (the product leaves the rotated key
// part's place empty and `latent_spread` copies it in for every head, so that a key is one bulk
// copy: what costs in staging is the number of copies, not their bytes) -> out [N, heads, vdim].  One block of eight warps per (128 queries, head, sequence); a warp owns 16 query rows
// with their fragments in registers, walks tiles of 64 keys staged by bulk copies (three in flight;
// bounded waits as in the kernel above),
// S and the streaming softmax (float, powers of two) stay in its registers, the weights become the
// left operand of the value product without leaving them, O stays in registers.  Causal, window
// as everywhere.  KS = (dim + rot) / 16 and NV = vdim / 8 at most (template), dim and rot
// multiples of 16, vdim of 8.
namespace {
constexpr int kQTile = 128, kKTile = 64, kExpThreads = 256;
constexpr int kStages = 4;           // tiles of keys and values in flight: a tile's copies take several tiles' worth of arithmetic to land

template <int KS, int NV>
__global__ void __launch_bounds__(kExpThreads)
expanded_attention_kernel(const bf16* __restrict__ q, int ldq, const bf16* __restrict__ kv, int ldkv,
                          bf16* __restrict__ out, int ldo, const int* __restrict__ cu_seqlens,
                          int dim, int rot, int vdim, float scale, int window, int test_waits,
                          const float* __restrict__ sinks) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(128) unsigned char smem[];
    const int b = blockIdx.z, h = blockIdx.y;
    const int tok0 = cu_seqlens[b], len = cu_seqlens[b + 1] - tok0;
    // the last queries of a sequence see the most keys: their blocks are started first
    const int q0 = (int)(gridDim.x - 1 - blockIdx.x) * kQTile;
    if (q0 >= len) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int dk = dim + rot;
    const int per = dim + vdim + rot;                           // a key's run: [unrotated key | value | rotated key part]
    const int ldks = dk + kPad, ldt = per + kPad;               // staged rows, in elements
    bf16* k_s = reinterpret_cast<bf16*>(smem);                  // the queries at the start [128][ldks], then
    bf16* t_s = k_s;                                            // [stages][64][ldt]: the tiles of keys and values
    const uint32_t bars = smem_u32(t_s + kStages * kKTile * ldt);     // a barrier of 8 bytes per stage: a staged tile has arrived
    volatile int* gave_up = reinterpret_cast<int*>(t_s + kStages * kKTile * ldt) + 2 * kStages;       // set by a thread whose wait ran out
    const int n_ks = dk / 16, n_nv = vdim / 8;
    if (tid == 0) {
        *gave_up = 0;
        for (int st = 0; st < kStages; ++st) mbar_init(bars + 8 * st, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::);
    }

    // the queries: staged, then each warp's 16 rows into registers
    for (int r = warp; r < kQTile; r += kExpThreads / 32) {
        const bool ok = q0 + r < len;
        const bf16* src = q + (size_t)(tok0 + (ok ? q0 + r : 0)) * ldq + (size_t)h * dk;
        for (int c = lane; c < dk / 8; c += 32) cp_async16(smem_u32(k_s + r * ldks + c * 8), src + c * 8, ok ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    uint32_t qf[KS][4];
    {
        const uint32_t a_addr = smem_u32(k_s + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldks + (lane >> 4) * 8);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
            if (ks < n_ks) ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], a_addr + ks * 32);
    }
    __syncthreads();                                            // the queries' place is free for keys

    const int q_hi = min(q0 + kQTile, len) - 1;
    const int lo_min = (window > 0 && q0 - window + 1 > 0) ? q0 - window + 1 : 0;
    const int t_lo = lo_min / kKTile, t_hi = q_hi / kKTile;
    // A tile of keys and values is staged by the copy engine, one bulk copy a key, issued by warp 0 and
    // counted on the tile's barrier: the warps that multiply issue no copy.  Value rows past the
    // sequence's end are zeroed by hand (their weights are zero, but zero times a stale NaN is not).
    auto load_tile = [&](int buf, int kt) {
        bf16* td = t_s + (size_t)buf * kKTile * ldt;
        const int valid = min(kKTile, len - kt * kKTile);
        for (int idx = valid * (vdim / 2) + tid; idx < kKTile * (vdim / 2); idx += kExpThreads)
            reinterpret_cast<uint32_t*>(td + (idx / (vdim / 2)) * ldt + dim)[idx % (vdim / 2)] = 0u;
        if (tid == 0) mbar_expect_tx(bars + 8 * buf, (uint32_t)(valid * per * 2));
        if (test_waits) return;
        constexpr int kShare = kKTile / (kExpThreads / 32);     // every warp asks for its own share of the keys
        const int r = warp * kShare + lane;
        if (lane < kShare && r < valid)
            bulk_row(smem_u32(td + r * ldt), kv + (size_t)(tok0 + kt * kKTile + r) * ldkv + (size_t)h * per, (uint32_t)(per * 2), bars + 8 * buf);
    };
    for (int st = 0; st < kStages - 1; ++st)
        if (t_lo + st <= t_hi) load_tile(st, t_lo + st);

    float o[NV][4];
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    int pos_r[2], lo_r[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = q0 + warp * 16 + g + hh * 8;
        pos_r[hh] = r < len ? r : -1;
        lo_r[hh] = (window > 0 && r - window + 1 > 0) ? r - window + 1 : 0;
    }

    for (int kt = t_lo; kt <= t_hi; ++kt) {
        const int buf = (kt - t_lo) % kStages;
        __syncthreads();                                        // everyone is done with the tile before (and sees the zeroed rows)
        if (*gave_up) break;                                    // a wait ran out: no barrier is armed again (see the kernel above)
        if (kt + kStages - 1 <= t_hi) load_tile((kt + kStages - 1 - t_lo) % kStages, kt + kStages - 1);   // into the buffer of the tile before
        if (!mbar_wait(bars + 8 * buf, ((uint32_t)(kt - t_lo) / kStages) & 1u, test_waits ? 1024u : kPageWaitLimit)) *gave_up = 1;
        const bf16* td = t_s + (size_t)buf * kKTile * ldt;
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
        {
            const uint32_t b_addr = smem_u32(td + ((lane & 7) + (lane >> 4) * 8) * ldt + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                if (ks < n_ks) {
                    uint32_t bfr[4][4];
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj)
                        // channel step ks: the unrotated key's channels first, the rotated part's behind the value
                        ldmatrix_x4(bfr[jj][0], bfr[jj][1], bfr[jj][2], bfr[jj][3], b_addr + (jj * 16 * ldt + (ks * 16 < dim ? ks * 16 : vdim + ks * 16)) * 2);
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        mma_bf16_16816(s[2 * jj], qf[ks], bfr[jj][0], bfr[jj][1]);
                        mma_bf16_16816(s[2 * jj + 1], qf[ks], bfr[jj][2], bfr[jj][3]);
                    }
                }
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int hh = e >> 1;
                const int key = kt * kKTile + j * 8 + t * 2 + (e & 1);
                const bool seen = pos_r[hh] >= 0 && key <= pos_r[hh] && key >= lo_r[hh];
                s[j][e] = seen ? s[j][e] * (scale * kLog2e) : -INFINITY;
                mx[hh] = fmaxf(mx[hh], s[j][e]);
            }
        float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
            const float m_new = fmaxf(m_run[hh], mx[hh]);
            corr[hh] = m_new == -INFINITY ? 1.f : fast_exp2(m_run[hh] - m_new);
            m_run[hh] = m_new;
        }
        uint32_t pf[4][4];                                      // the weights as left operand: 4 steps of 16 keys
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) p[e] = m_run[e >> 1] == -INFINITY ? 0.f : fast_exp2(s[j][e] - m_run[e >> 1]);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(p[0], p[1]), hi = __floats2bfloat162_rn(p[2], p[3]);
            // the sums run over the rounded weights, the ones the values are multiplied with
            sum[0] += __bfloat162float(lo.x) + __bfloat162float(lo.y);
            sum[1] += __bfloat162float(hi.x) + __bfloat162float(hi.y);
            pf[j >> 1][(j & 1) * 2] = *reinterpret_cast<const uint32_t*>(&lo);
            pf[j >> 1][(j & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&hi);
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            sum[hh] += __shfl_xor_sync(0xffffffffu, sum[hh], 1);
            sum[hh] += __shfl_xor_sync(0xffffffffu, sum[hh], 2);
            l_run[hh] = l_run[hh] * corr[hh] + sum[hh];
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
        }
        {
            const uint32_t v_addr = smem_u32(td + ((lane & 7) + ((lane >> 3) & 1) * 8) * ldt + dim + (lane >> 4) * 8);
#pragma unroll
            for (int ks = 0; ks < kKTile / 16; ++ks) {
#pragma unroll
                for (int c = 0; c < NV; c += 8) {
                    uint32_t vf[4][4];
#pragma unroll
                    for (int j = 0; j < 8; j += 2)
                        if (c + j < n_nv)
                            ldmatrix_x4_trans(vf[j / 2][0], vf[j / 2][1], vf[j / 2][2], vf[j / 2][3], v_addr + (ks * 16 * ldt + (c + j) * 8) * 2);
#pragma unroll
                    for (int j = 0; j < 8; j += 2)
                        if (c + j < n_nv) {
                            mma_bf16_16816(o[c + j], pf[ks], vf[j / 2][0], vf[j / 2][1]);
                            if (c + j + 1 < NV) mma_bf16_16816(o[c + j + 1], pf[ks], vf[j / 2][2], vf[j / 2][3]);
                        }
                }
            }
        }
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        if (pos_r[hh] < 0 || l_run[hh] <= 0.f) continue;
        const float inv = 1.0f / (l_run[hh] + (sinks ? exp2f(sinks[h] * kLog2e - m_run[hh]) : 0.f));
        bf16* dst = out + (size_t)(tok0 + pos_r[hh]) * ldo + (size_t)h * vdim + t * 2;
#pragma unroll
        for (int j = 0; j < NV; ++j)
            if (j < n_nv)
                *reinterpret_cast<__nv_bfloat162*>(dst + j * 8) = __floats2bfloat162_rn(o[j][hh * 2] * inv, o[j][hh * 2 + 1] * inv);
    }
}

size_t expanded_attention_smem(int dk, int vdim) {
    const size_t tiles = (size_t)kStages * kKTile * (dk + vdim + kPad) * 2, queries = (size_t)kQTile * (dk + kPad) * 2;
    return (tiles > queries ? tiles : queries) + 8 * kStages + 16;
}

// kv[n, h, dim + vdim : dim + vdim + rot] = kr[n, :] for every head: the shared rotated key part into its place in every head's run.
__global__ void latent_spread_kernel(const bf16* __restrict__ kr, int ldr, bf16* __restrict__ kv, int ldkv, int n_heads, int per,
                                     int offset, int rot8) {
    chain_release();
    chain_wait();
    const int n = blockIdx.x;
    for (int idx = threadIdx.x; idx < n_heads * rot8; idx += blockDim.x) {
        const int h = idx / rot8, c = idx % rot8;
        *reinterpret_cast<uint4*>(kv + (size_t)n * ldkv + (size_t)h * per + offset + c * 8) =
            *reinterpret_cast<const uint4*>(kr + (size_t)n * ldr + c * 8);
    }
}
}  // namespace

GTG_API int gtg_expanded_attention_supports(int dim, int rot, int vdim) {
    return dim > 0 && rot > 0 && vdim > 0 && dim % 16 == 0 && rot % 16 == 0 && vdim % 8 == 0 && dim + rot <= 256 && vdim <= 128;
}

// Attention of a step whose sequences all start at their first token, over the step's own rows expanded per head.
// kv[n, h, offset : offset + rot] = kr[n, 0 : rot] for every head h (runs of `per` channels a head; all multiples of 8).
GTG_API int gtg_latent_spread(const void* kr, int ldr, void* kv, int ldkv, int N, int n_heads, int per, int offset, int rot,
                              cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_heads <= 0 || rot <= 0 || offset < 0 || offset + rot > per) return kErrBadArgument;
    if (rot % 8 || per % 8 || offset % 8 || ldr % 8 || ldkv % 8 || ((uintptr_t)kr % 16) || ((uintptr_t)kv % 16)) return kErrUnsupported;
    return launch_chained(latent_spread_kernel, dim3(N), dim3(128), 0, stream, (const bf16*)kr, ldr, (bf16*)kv, ldkv, n_heads, per,
                          offset, rot / 8);
}

GTG_API int gtg_expanded_attention_bf16(const void* q, int ldq, const void* kv, int ldkv,
                                        void* out, int ldo, const int* cu_seqlens, int n_seqs,
                                        int max_q_len, int n_heads, int dim, int rot, int vdim, float scale, int window,
                                        const float* sinks, cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (n_heads <= 0) return kErrBadArgument;
    if (!gtg_expanded_attention_supports(dim, rot, vdim)) return kErrUnsupported;
    if (ldq % 8 || ldkv % 8 || ldo % 2 || ((uintptr_t)q % 16) || ((uintptr_t)kv % 16) || ((uintptr_t)out % 4)) return kErrUnsupported;
    if (n_heads > 65535 || n_seqs > 65535) return kErrUnsupported;
    const size_t smem = expanded_attention_smem(dim + rot, vdim);
    const dim3 grid((max_q_len + kQTile - 1) / kQTile, n_heads, n_seqs);
#define GTG_EXPANDED(KS, NV)                                                                                        \
    do {                                                                                                            \
        static bool configured = false;                                                                             \
        if (!configured) {                                                                                          \
            const cudaError_t e = cudaFuncSetAttribute(expanded_attention_kernel<KS, NV>,                           \
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);    \
            if (e != cudaSuccess) return (int)e;                                                                    \
            configured = true;                                                                                      \
        }                                                                                                           \
        return launch_chained(expanded_attention_kernel<KS, NV>, grid, dim3(kExpThreads), smem, stream, (const bf16*)q, ldq, \
                              (const bf16*)kv, ldkv, (bf16*)out, ldo, cu_seqlens,                                  \
                              dim, rot, vdim, scale, window, g_latent_test_waits ? 1 : 0, sinks);                  \
    } while (0)
    const int ks = (dim + rot) / 16;
    if (vdim <= 64) {
        if (ks <= 4) GTG_EXPANDED(4, 8); else if (ks <= 8) GTG_EXPANDED(8, 8); else if (ks <= 12) GTG_EXPANDED(12, 8); else GTG_EXPANDED(16, 8);
    }
    if (ks <= 4) GTG_EXPANDED(4, 16); else if (ks <= 8) GTG_EXPANDED(8, 16); else if (ks <= 12) GTG_EXPANDED(12, 16); else GTG_EXPANDED(16, 16);
#undef GTG_EXPANDED
}
