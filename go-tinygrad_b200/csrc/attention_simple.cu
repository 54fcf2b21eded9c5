// Causal grouped-query attention over the paged cache, one warp per
// (token, query head).  This is the attention of the float32 path (and the
// bfloat16 path's route for head sizes its tiled kernels refuse).  It serves a
// prompt and a decode step alike: token n at position p sees keys lo..p of its
// own sequence, lo = 0, or p-window+1 (a sliding window), or the first position
// of p's chunk, p - p % chunk (chunked attention: positions are cut into
// stretches of `chunk`, counted from the sequence's start, and a token sees the
// keys of its own stretch only).
//
// Scores are (q.k)*scale with the scale applied after the dot; softmax is the
// streaming form of max / exp / sum / normalise (model/llama.go:1626-1660), with
// expf, never a fast approximation.  Keys are walked 32 at a time from lo, so
// the value for a (token, head) depends on nothing but its own keys: not on the
// batch, not on how the tokens were cut into steps.
//
// `vd` is how many channels a value has: the first vd channels of a row of the
// value plane (vd = hd for ordinary heads).  A mixer whose values are a leading
// part of what it stores as keys passes the key plane for both and a smaller vd;
// the output then has vd channels per head.  `vrow` is the width of a row of the
// value plane (hd when keys and values share a page layout; a cache whose values
// have a size of their own stores rows of vd channels).  `gate` (or null):
// float [N, n_heads], a factor on each head's output; with `gate_ld` > 0 it holds
// instead one logit per output channel, rows of gate_ld floats, heads side by side
// vd apart, and the factor is the logit's sigmoid.  `softcap` c > 0: a score
// becomes c tanh(score / c) after the scale.  `sinks` (or null): float [n_heads];
// exp(sinks[h]) joins head h's softmax denominator, without a key or a value.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int kWarps = 4;
constexpr int kMaxHeadDim = 2048;

// kMaxPerLane: value channels per lane (vd <= 32 * kMaxPerLane)
template <typename T, int kMaxPerLane>
__global__ void __launch_bounds__(kWarps * 32)
attention_simple_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo,
                        const T* __restrict__ kc, const T* __restrict__ vc, long long page_stride,
                        const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ token_seq, const int* __restrict__ slots,
                        const int* __restrict__ positions,
                        int N, int n_heads, int n_kv, int hd, int vd, int vrow, float scale, int window, int chunk,
                        const float* __restrict__ gate, int gate_ld, float softcap, const float* __restrict__ sinks) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * kWarps + warp;
    if (wid >= (long long)N * n_heads) return;
    const int n = (int)(wid / n_heads), h = (int)(wid % n_heads);
    const int kvh = h / (n_heads / n_kv);
    const int pos = positions[n];
    const int slot = slots[token_seq[n]];
    const int* table = block_table + (size_t)slot * table_stride;
    int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (chunk > 0) lo = max(lo, pos - pos % chunk);

    float* qs = smem + warp * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = to_f32<T>(q[(size_t)n * ldq + h * hd + d]);
    __syncwarp();

    float acc[kMaxPerLane];
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) acc[j] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int t0 = lo; t0 <= pos; t0 += 32) {
        const int t = t0 + lane;
        const bool valid = t <= pos;
        int page = 0;
        float score = -INFINITY;
        if (valid) {
            page = table[t / kPageTokens];
            const T* kp = kc + (size_t)page * page_stride + ((size_t)kvh * kPageTokens + (t % kPageTokens)) * hd;
            float s = 0.f;
            for (int d = 0; d < hd; ++d) s = fmaf(qs[d], to_f32<T>(kp[d]), s);
            score = s * scale;
            if (softcap > 0.f) score = softcap * tanhf(score / softcap);
        }
        const float m_new = fmaxf(m, warp_max(score));
        const float p = valid ? expf(score - m_new) : 0.f;
        const float corr = expf(m - m_new);      // 0 on the first chunk (m = -inf)
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) acc[j] *= corr;
        const int count = min(32, pos - t0 + 1);
        for (int src = 0; src < count; ++src) {
            const float pj = __shfl_sync(0xffffffffu, p, src);
            const int pg = __shfl_sync(0xffffffffu, page, src);
            const int tj = t0 + src;
            const T* vp = vc + (size_t)pg * page_stride + ((size_t)kvh * kPageTokens + (tj % kPageTokens)) * vrow;
#pragma unroll
            for (int j = 0; j < kMaxPerLane; ++j) {
                const int d = lane + 32 * j;
                if (d < vd) acc[j] = fmaf(pj, to_f32<T>(vp[d]), acc[j]);
            }
        }
        m = m_new;
    }
    if (sinks) {
        // the sink joins the sum as one more weight that carries no value
        const float sink = sinks[h];
        const float m_new = fmaxf(m, sink);
        const float corr = expf(m - m_new);
        l = l * corr + expf(sink - m_new);
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) acc[j] *= corr;
    }
    const float inv = ((gate && gate_ld <= 0) ? gate[(size_t)n * n_heads + h] : 1.0f) / l;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
        const int d = lane + 32 * j;
        if (d < vd) {
            float val = acc[j] * inv;
            if (gate && gate_ld > 0) val *= 1.0f / (1.0f + expf(-gate[(size_t)n * gate_ld + h * vd + d]));
            out[(size_t)n * ldo + h * vd + d] = from_f32<T>(val);
        }
    }
}
}  // namespace

GTG_API int gtg_attention_simple(int dtype, const void* q, int ldq, void* out, int ldo,
                                 const void* kc, const void* vc, long long page_stride,
                                 const int* block_table, int table_stride,
                                 const int* token_seq, const int* slots, const int* positions,
                                 int N, int n_heads, int n_kv, int hd, int vd, int vrow, float scale, int window, int chunk,
                                 const float* gate, int gate_ld, float softcap, const float* sinks, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || hd <= 0) return kErrBadArgument;
    if (vd <= 0 || vd > vrow || window < 0 || chunk < 0 || softcap < 0.f) return kErrBadArgument;
    if (gate && gate_ld > 0 && gate_ld < n_heads * vd) return kErrBadArgument;
    if (hd > kMaxHeadDim || vd > 32 * 32) return kErrUnsupported;
    const long long warps = (long long)N * n_heads;
    const long long blocks = (warps + kWarps - 1) / kWarps;
    if (blocks > 0x7fffffffLL) return kErrUnsupported;
    const size_t smem = (size_t)kWarps * hd * sizeof(float);
#define GTG_SIMPLE(T, PER)                                                                                   \
    attention_simple_kernel<T, PER><<<(unsigned)blocks, kWarps * 32, smem, stream>>>(                            \
        (const T*)q, ldq, (T*)out, ldo, (const T*)kc, (const T*)vc, page_stride, block_table, table_stride,      \
        token_seq, slots, positions, N, n_heads, n_kv, hd, vd, vrow, scale, window, chunk, gate, gate_ld, softcap, sinks)
    if (dtype == 0) {
        if (vd <= 256) GTG_SIMPLE(float, 8); else if (vd <= 512) GTG_SIMPLE(float, 16); else GTG_SIMPLE(float, 32);
    } else if (dtype == 1) {
        if (vd <= 256) GTG_SIMPLE(bf16, 8); else if (vd <= 512) GTG_SIMPLE(bf16, 16); else GTG_SIMPLE(bf16, 32);
    }
#undef GTG_SIMPLE
    else return kErrBadArgument;
    return launch_status();
}
