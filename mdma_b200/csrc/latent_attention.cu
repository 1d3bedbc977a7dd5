// Attention over a cached latent: every token keeps ONE vector c of `rank` numbers per layer
// (a down-projection of its input, divided by its root mean square and weighted); keys and
// values of all heads are linear maps of c.  With the keys' map moved onto the query
// (q' = W_uk,h^T q_h, `rank` numbers per head) the score is q' . c, and with the values' map
// applied after the weighted sum (o_h = W_uv,h sum_j p_j c_j) the cache is read as one shared
// key-and-value head of size `rank`.  The softmax has a sink: exp(sink_h) is added to the
// denominator once, with no key, no value and no scale (no sink pointer: the ordinary softmax).
//
// Plain kernels: one warp per (token, head), keys visited in position order, 32 at a time
// (their scores first, then their maximum, then their weighted sum from zero, which is
// folded into the running sum: short chains of roundings), everything in float; the result
// of a token does not depend on the step's cut or on the batch.
#include "common.cuh"

namespace mdma {

constexpr int kMaxRank = 1024;

// c = x / sqrt(mean(x^2) + eps) * w for x = columns [col0, col0 + rank) of the token's projection
// row; written to the token's row of the paged cache ([pages, page_size, rank]).
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
latent_norm_store_kernel(const T* __restrict__ proj, int proj_stride, int col0, const TW* __restrict__ w, float eps,
                         int rank, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                         const int* __restrict__ seq_slot, const int* __restrict__ page_table, int max_pages,
                         int page_size, T* __restrict__ cache) {
    chain_release();
    chain_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * proj_stride + col0;
    float ss = 0.f;
    for (int e = threadIdx.x; e < rank; e += blockDim.x) {
        const float v = to_float(row[e]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)rank + eps);
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    const size_t page = (size_t)page_table[(size_t)slot * max_pages + pos / page_size];
    T* dst = cache + (page * page_size + (size_t)(pos % page_size)) * rank;
    for (int e = threadIdx.x; e < rank; e += blockDim.x)
        dst[e] = from_float<T>(to_float(row[e]) * scale * to_float(w[e]));
}

// out[t,h,:] = sum_{j<=pos} p_j c_j,  p_j = exp(s_j - m) / (sum_i exp(s_i - m) + exp(sink_h - m)),
// s_j = (q'[t,h,:] . c_j) * scale.  `window` > 0 keeps the last `window` keys only.
template <typename T, typename TS>
__global__ void __launch_bounds__(128)
latent_attention_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ cache,
                        const TS* __restrict__ sink, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                        const int* __restrict__ seq_slot, const int* __restrict__ page_table, int max_pages,
                        int page_size, T* __restrict__ out, int n_heads, int rank, int window, float scale) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int h = blockIdx.y * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (h >= n_heads) return;
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    const int first = window > 0 ? max(0, pos + 1 - window) : 0;
    float qv[kMaxRank / 32], acc[kMaxRank / 32];
    const T* qp = q + (size_t)t * q_row_stride + (size_t)h * rank;
#pragma unroll
    for (int j = 0; j < kMaxRank / 32; ++j) {
        const int d = lane + 32 * j;
        qv[j] = d < rank ? to_float(qp[d]) : 0.f;
        acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int* pages = page_table + (size_t)slot * max_pages;
    for (int p0 = first; p0 <= pos; p0 += 32) {
        const int nk = min(32, pos + 1 - p0);
        // the scores of up to 32 keys: lane j keeps the score of key p0 + j
        float mine = -INFINITY;
        for (int k = 0; k < nk; ++k) {
            const int p = p0 + k;
            const T* cp = cache + ((size_t)pages[p / page_size] * page_size + (size_t)(p % page_size)) * rank;
            float part = 0.f;
#pragma unroll
            for (int j = 0; j < kMaxRank / 32; ++j) {
                const int d = lane + 32 * j;
                if (d < rank) part = fmaf(qv[j], to_float(cp[d]), part);
            }
            const float s = warp_sum(part) * scale;
            if (lane == k) mine = s;
        }
        const float m_new = fmaxf(m, warp_max(mine));
        const float corr = expf(m - m_new);          // exp(-inf) = 0 at the first keys
        const float pe_mine = lane < nk ? expf(mine - m_new) : 0.f;
        float sum[kMaxRank / 32];
#pragma unroll
        for (int j = 0; j < kMaxRank / 32; ++j) sum[j] = 0.f;
        float l_new = 0.f;
        for (int k = 0; k < nk; ++k) {
            const int p = p0 + k;
            const T* cp = cache + ((size_t)pages[p / page_size] * page_size + (size_t)(p % page_size)) * rank;
            const float pe = __shfl_sync(0xffffffffu, pe_mine, k);
            l_new += pe;
#pragma unroll
            for (int j = 0; j < kMaxRank / 32; ++j) {
                const int d = lane + 32 * j;
                if (d < rank) sum[j] = fmaf(pe, to_float(cp[d]), sum[j]);
            }
        }
        l = l * corr + l_new;
#pragma unroll
        for (int j = 0; j < kMaxRank / 32; ++j) acc[j] = acc[j] * corr + sum[j];
        m = m_new;
    }
    float inv = 1.0f / l;                       // no sink: the ordinary softmax
    if (sink != nullptr) {
        const float sk = to_float(sink[h]);
        const float m_all = fmaxf(m, sk);
        const float corr = expf(m - m_all);
        l = l * corr + expf(sk - m_all);
        inv = corr / l;
    }
    T* op = out + ((size_t)t * n_heads + h) * rank;
#pragma unroll
    for (int j = 0; j < kMaxRank / 32; ++j) {
        const int d = lane + 32 * j;
        if (d < rank) op[d] = from_float<T>(acc[j] * inv);
    }
}

}  // namespace mdma

using namespace mdma;

extern "C" {

int mdma_latent_norm_store(const void* proj, int dtype, int proj_stride, int col0, const void* w, int w_dtype,
                           float eps, int rank, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                           const int* page_table, int max_pages, int page_size, void* cache, int n_tokens,
                           cudaStream_t stream) {
    MDMA_REQUIRE(rank > 0 && proj_stride >= col0 + rank && page_table && page_size > 0 && max_pages > 0,
                 "latent_norm_store: bad sizes");
    if (n_tokens == 0) return 0;
    MDMA_DISPATCH_DTYPE(dtype, T, MDMA_DISPATCH_DTYPE(w_dtype, TW,
        launch_chained(latent_norm_store_kernel<T, TW>, dim3(n_tokens), dim3(128), 0, stream, (const T*)proj,
                       proj_stride, col0, (const TW*)w, eps, rank, tok_seq, tok_pos, seq_slot, page_table, max_pages,
                       page_size, (T*)cache)));
    MDMA_LAUNCH_OK("latent_norm_store");
    return 0;
}

int mdma_latent_attention(const void* q, int dtype, int q_row_stride, const void* cache, const void* sink,
                          int sink_dtype, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                          const int* page_table, int max_pages, int page_size, void* out, int n_tokens, int n_heads,
                          int rank, int window, float scale, cudaStream_t stream) {
    MDMA_REQUIRE(n_heads > 0 && rank > 0 && rank <= kMaxRank, "latent_attention: rank %d is beyond the limit %d", rank, kMaxRank);
    MDMA_REQUIRE(page_table && page_size > 0 && max_pages > 0 && window >= 0, "latent_attention: bad cache geometry");
    MDMA_REQUIRE((n_heads + 3) / 4 <= 65535, "latent_attention: too many heads");
    if (n_tokens == 0) return 0;
    dim3 grid(n_tokens, (n_heads + 3) / 4);
    MDMA_DISPATCH_DTYPE(dtype, T, MDMA_DISPATCH_DTYPE(sink_dtype, TS,
        launch_chained(latent_attention_kernel<T, TS>, grid, dim3(128), 0, stream, (const T*)q, q_row_stride,
                       (const T*)cache, (const TS*)sink, tok_seq, tok_pos, seq_slot, page_table, max_pages, page_size,
                       (T*)out, n_heads, rank, window, scale)));
    MDMA_LAUNCH_OK("latent_attention");
    return 0;
}

}  // extern "C"
