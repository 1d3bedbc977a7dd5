// Small kernels of attention over a cached latent that also keeps one turned key part per token.
//
// latent_prepare: a token's fused projection row holds [query latent (q_rank) | kv latent (kv_rank) | key part
// (rot_dim) | ...].  The query latent is divided by its root mean square, weighted and written to `cq`; the kv latent
// likewise, and the key part is turned by the token's position (its first `rotary_dim` numbers, pairs (2i, 2i+1) or
// (i, i + rotary_dim/2), angle = float(position) * inv_freq[i], cos and sin times `magnitude`); both go to the
// token's row of the paged cache as one vector [latent | key part].  A site that reads another site's cache writes
// only `cq`.
//
// rotate_heads: columns [offset, offset + rotary_dim) of every head of q [tokens, heads, head_pitch] are turned in
// place the same way.
//
// All arithmetic is float; a number is rounded once, when it is stored.
#include "common.cuh"

namespace mdma {

constexpr int kMaxRotary = 512;

__device__ __forceinline__ float vec_weight(const void* w, int dtype, int e) {
    return dtype == kF32 ? reinterpret_cast<const float*>(w)[e] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[e]);
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ proj, int proj_stride, int q_col, int q_rank, const void* __restrict__ q_w,
                      int kv_col, int kv_rank, const void* __restrict__ kv_w, int w_dtype, float eps, int rot_dim,
                      int rotary_dim, int interleaved, const float* __restrict__ inv_freq, float magnitude,
                      const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                      const int* __restrict__ page_table, int max_pages, int page_size, T* __restrict__ cq,
                      T* __restrict__ cache, int write_cache) {
    chain_release();
    chain_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * proj_stride;
    float ss = 0.f;
    for (int e = threadIdx.x; e < q_rank; e += blockDim.x) {
        const float v = to_float(row[q_col + e]);
        ss = fmaf(v, v, ss);
    }
    const float q_inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
    for (int e = threadIdx.x; e < q_rank; e += blockDim.x)
        cq[(size_t)t * q_rank + e] = from_float<T>(to_float(row[q_col + e]) * q_inv * vec_weight(q_w, w_dtype, e));
    if (!write_cache) return;
    ss = 0.f;
    for (int e = threadIdx.x; e < kv_rank; e += blockDim.x) {
        const float v = to_float(row[kv_col + e]);
        ss = fmaf(v, v, ss);
    }
    const float kv_inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)kv_rank + eps);
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    const size_t page = (size_t)page_table[(size_t)slot * max_pages + pos / page_size];
    T* dst = cache + (page * page_size + (size_t)(pos % page_size)) * (kv_rank + rot_dim);
    for (int e = threadIdx.x; e < kv_rank; e += blockDim.x)
        dst[e] = from_float<T>(to_float(row[kv_col + e]) * kv_inv * vec_weight(kv_w, w_dtype, e));
    const T* kr = row + kv_col + kv_rank;
    const int half = rotary_dim / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        s *= magnitude;
        c *= magnitude;
        const int d0 = interleaved ? 2 * i : i, d1 = interleaved ? 2 * i + 1 : i + half;
        const float a = to_float(kr[d0]), b = to_float(kr[d1]);
        dst[kv_rank + d0] = from_float<T>(a * c - b * s);
        dst[kv_rank + d1] = from_float<T>(b * c + a * s);
    }
    for (int e = rotary_dim + threadIdx.x; e < rot_dim; e += blockDim.x) dst[kv_rank + e] = kr[e];
}

template <typename T>
__global__ void __launch_bounds__(128)
rotate_heads_kernel(T* __restrict__ q, int row_stride, int n_heads, int head_pitch, int offset, int rotary_dim,
                    int interleaved, const float* __restrict__ inv_freq, float magnitude, const int* __restrict__ tok_pos) {
    chain_release();
    chain_wait();
    __shared__ float sines[kMaxRotary / 2], cosines[kMaxRotary / 2];
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int half = rotary_dim / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        sines[i] = s * magnitude;
        cosines[i] = c * magnitude;
    }
    __syncthreads();
    T* row = q + (size_t)t * row_stride;
    for (int j = threadIdx.x; j < n_heads * half; j += blockDim.x) {
        const int h = j / half, i = j % half;
        T* v = row + (size_t)h * head_pitch + offset;
        const int d0 = interleaved ? 2 * i : i, d1 = interleaved ? 2 * i + 1 : i + half;
        const float a = to_float(v[d0]), b = to_float(v[d1]);
        v[d0] = from_float<T>(a * cosines[i] - b * sines[i]);
        v[d1] = from_float<T>(b * cosines[i] + a * sines[i]);
    }
}

}  // namespace mdma

using namespace mdma;

extern "C" {

int mdma_latent_prepare(const void* proj, int dtype, int proj_stride, int q_col, int q_rank, const void* q_w, int kv_col,
                        int kv_rank, const void* kv_w, int w_dtype, float eps, int rot_dim, int rotary_dim, int interleaved,
                        const float* inv_freq, float magnitude, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                        const int* page_table, int max_pages, int page_size, void* cq, void* cache, int write_cache,
                        int n_tokens, cudaStream_t stream) {
    MDMA_REQUIRE(q_rank > 0 && q_w && cq && proj_stride >= q_col + q_rank, "latent_prepare: bad query latent");
    MDMA_REQUIRE(w_dtype == kF32 || w_dtype == kBF16, "latent_prepare: unknown weight dtype %d", w_dtype);
    if (write_cache) {
        MDMA_REQUIRE(kv_rank > 0 && rot_dim >= 0 && kv_w && proj_stride >= kv_col + kv_rank + rot_dim, "latent_prepare: bad kv latent");
        MDMA_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= rot_dim && (rotary_dim == 0 || inv_freq),
                     "latent_prepare: %d turned numbers do not fit a key part of %d", rotary_dim, rot_dim);
        MDMA_REQUIRE(cache && page_table && page_size > 0 && max_pages > 0, "latent_prepare: no cache pages");
    }
    if (n_tokens == 0) return 0;
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(latent_prepare_kernel<T>, dim3(n_tokens), dim3(128), 0, stream, (const T*)proj, proj_stride, q_col,
                       q_rank, q_w, kv_col, kv_rank, kv_w, w_dtype, eps, rot_dim, rotary_dim, interleaved, inv_freq,
                       magnitude, tok_seq, tok_pos, seq_slot, page_table, max_pages, page_size, (T*)cq, (T*)cache,
                       write_cache));
    MDMA_LAUNCH_OK("latent_prepare");
    return 0;
}

int mdma_rotate_heads(void* q, int dtype, int row_stride, int n_heads, int head_pitch, int offset, int rotary_dim,
                      int interleaved, const float* inv_freq, float magnitude, const int* tok_pos, int n_tokens,
                      cudaStream_t stream) {
    MDMA_REQUIRE(n_heads > 0 && head_pitch > 0 && offset >= 0 && rotary_dim >= 0 && rotary_dim % 2 == 0 &&
                 offset + rotary_dim <= head_pitch && rotary_dim <= kMaxRotary,
                 "rotate_heads: %d turned numbers at %d do not fit a head of %d (limit %d)", rotary_dim, offset, head_pitch, kMaxRotary);
    MDMA_REQUIRE(rotary_dim == 0 || inv_freq, "rotate_heads: a rotation needs its frequencies");
    if (n_tokens == 0 || rotary_dim == 0) return 0;
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(rotate_heads_kernel<T>, dim3(n_tokens), dim3(128), 0, stream, (T*)q, row_stride, n_heads, head_pitch,
                       offset, rotary_dim, interleaved, inv_freq, magnitude, tok_pos));
    MDMA_LAUNCH_OK("rotate_heads");
    return 0;
}

}  // extern "C"
