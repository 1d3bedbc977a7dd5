// Small kernels around attention and around a sublayer whose result is normed before it joins the residual stream.
//
// qk_prepare: a token's fused projection row [q heads | k heads | v heads | ...] is made ready for attention in one
// pass.  Every q and k head is rotated by the token's position (the first `rotary_dim` numbers of a head, pairs
// (2i, 2i+1) or (i, i + rotary_dim/2), angle = float(position) * inv_freq[i]) and then, if asked, divided by its own
// root mean square, x / sqrt(mean(x^2) + eps), without a weight.  q is written back in place; k and v go to the
// token's row of the paged cache (v heads may have a size of their own).  All arithmetic is float; a number is
// rounded once, when it is stored.
//
// head_gate: out[t, h, :] *= sigmoid(g[t, h]) * scale, one gate number per head (no gate: the scale alone).
//
// rmsnorm_add: x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w, the norm that follows a sublayer, in float.
#include "common.cuh"

namespace mdma {

constexpr int kPrepMaxDim = 256, kPrepWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
qk_prepare_kernel(T* __restrict__ proj, int row_stride, int k_col, int v_col, const int* __restrict__ tok_seq,
                  const int* __restrict__ tok_pos, const int* __restrict__ seq_slot, const float* __restrict__ inv_freq,
                  T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ page_table, int max_pages,
                  int page_size, int n_heads, int n_kv_heads, int dim, int v_dim, int rotary_dim, int interleaved,
                  int unit_norm, float eps, int write_kv) {
    chain_release();
    chain_wait();
    __shared__ float sines[kPrepMaxDim / 2], cosines[kPrepMaxDim / 2];
    __shared__ float rows[kPrepWarps][kPrepMaxDim];
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int half = rotary_dim / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sines[i], &cosines[i]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    const int head = blockIdx.y * kPrepWarps + warp;
    if (head >= total) return;
    T* row = proj + (size_t)t * row_stride;
    size_t cache_row = 0;
    if (write_kv) {
        const int slot = seq_slot[tok_seq[t]];
        cache_row = ((size_t)page_table[(size_t)slot * max_pages + pos / page_size] * page_size + (size_t)(pos % page_size)) * n_kv_heads;
    }
    if (head >= n_heads + n_kv_heads) {                 // a value head: copied as it is
        const int g = head - n_heads - n_kv_heads;
        const T* src = row + v_col + (size_t)g * v_dim;
        T* dst = v_cache + (cache_row + g) * v_dim;
        for (int d = lane; d < v_dim; d += 32) dst[d] = src[d];
        return;
    }
    const bool is_q = head < n_heads;
    T* src = is_q ? row + (size_t)head * dim : row + k_col + (size_t)(head - n_heads) * dim;
    T* dst = is_q ? src : k_cache + (cache_row + (head - n_heads)) * dim;
    float* v = rows[warp];
    for (int d = lane; d < dim; d += 32) v[d] = to_float(src[d]);
    __syncwarp();
    for (int i = lane; i < half; i += 32) {
        const int d0 = interleaved ? 2 * i : i, d1 = interleaved ? 2 * i + 1 : i + half;
        const float a = v[d0], b = v[d1], s = sines[i], c = cosines[i];
        v[d0] = a * c - b * s;
        v[d1] = b * c + a * s;
    }
    __syncwarp();
    float inv = 1.0f;
    if (unit_norm) {
        float sq = 0.f;
        for (int d = lane; d < dim; d += 32) sq = fmaf(v[d], v[d], sq);
        inv = 1.0f / sqrtf(warp_sum(sq) / (float)dim + eps);
    }
    for (int d = lane; d < dim; d += 32) dst[d] = from_float<T>(v[d] * inv);
}

template <typename T>
__global__ void __launch_bounds__(256)
head_gate_kernel(T* __restrict__ out, const T* __restrict__ gate, int gate_stride, int n_heads, int v_dim, float scale) {
    chain_release();
    chain_wait();
    const size_t t = blockIdx.x;
    const int width = n_heads * v_dim;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        const float f = gate ? scale / (1.0f + expf(-to_float(gate[t * gate_stride + e / v_dim]))) : scale;
        out[t * width + e] = from_float<T>(to_float(out[t * width + e]) * f);
    }
}

// `partial` [splits][rows][width]: y is first completed by the partial sums a K-split product left (in split order).
template <typename TW>
__global__ void __launch_bounds__(256)
rmsnorm_add_kernel(float* __restrict__ x, float* __restrict__ y, const float* __restrict__ partial, int splits,
                   size_t split_stride, const TW* __restrict__ w, int width, float eps) {
    chain_release();
    chain_wait();
    __shared__ float scratch[32];
    const size_t t = blockIdx.x;
    float* yr = y + t * width;
    float sq = 0.f;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        float v = yr[e];
        for (int s = 0; s < splits; ++s) v += partial[(size_t)s * split_stride + t * width + e];
        if (splits > 0) yr[e] = v;
        sq = fmaf(v, v, sq);
    }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    float* xr = x + t * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x) xr[e] += yr[e] * inv * to_float(w[e]);
}

// y[t] += a * z[t]
__global__ void __launch_bounds__(256)
add_scaled_kernel(float* __restrict__ y, const float* __restrict__ z, float a, long n) {
    chain_release();
    chain_wait();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) y[i] = fmaf(a, z[i], y[i]);
}

}  // namespace mdma

using namespace mdma;

extern "C" {

int mdma_qk_prepare(void* proj, int dtype, int row_stride, int k_col, int v_col, const int* tok_seq, const int* tok_pos,
                    const int* seq_slot, const float* inv_freq, void* k_cache, void* v_cache, const int* page_table,
                    int max_pages, int page_size, int n_tokens, int n_heads, int n_kv_heads, int dim, int v_dim,
                    int rotary_dim, int interleaved, int unit_norm, float eps, int write_kv, cudaStream_t stream) {
    MDMA_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads >= 0, "qk_prepare: bad sizes");
    MDMA_REQUIRE(dim > 0 && dim <= kPrepMaxDim && v_dim > 0, "qk_prepare: head size %d is beyond the limit %d", dim, kPrepMaxDim);
    MDMA_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= dim, "qk_prepare: rotary_dim %d does not fit head size %d", rotary_dim, dim);
    MDMA_REQUIRE(rotary_dim == 0 || inv_freq, "qk_prepare: a rotation needs its frequencies");
    MDMA_REQUIRE(!write_kv || (page_table && k_cache && v_cache && page_size > 0 && max_pages > 0), "qk_prepare: no cache pages");
    if (n_tokens == 0) return 0;
    const int total = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(qk_prepare_kernel<T>, dim3(n_tokens, (total + kPrepWarps - 1) / kPrepWarps), dim3(kPrepWarps * 32), 0,
                       stream, (T*)proj, row_stride, k_col, v_col, tok_seq, tok_pos, seq_slot, inv_freq, (T*)k_cache,
                       (T*)v_cache, page_table, max_pages, page_size, n_heads, n_kv_heads, dim, v_dim, rotary_dim,
                       interleaved, unit_norm, eps, write_kv));
    MDMA_LAUNCH_OK("qk_prepare");
    return 0;
}

int mdma_head_gate(void* out, const void* gate, int dtype, int gate_stride, int n_rows, int n_heads, int v_dim, float scale,
                   cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && n_heads > 0 && v_dim > 0, "head_gate: bad sizes");
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(head_gate_kernel<T>, dim3(n_rows), dim3(256), 0, stream, (T*)out, (const T*)gate, gate_stride, n_heads,
                       v_dim, scale));
    MDMA_LAUNCH_OK("head_gate");
    return 0;
}

int mdma_rmsnorm_add(float* x, float* y, const float* partial, int splits, long split_stride, const void* w, int w_dtype,
                     int n_rows, int width, float eps, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0, "rmsnorm_add: bad sizes");
    MDMA_REQUIRE(splits >= 0 && (splits == 0 || partial), "rmsnorm_add: partial sums need a pointer");
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_DTYPE(w_dtype, TW,
        launch_chained(rmsnorm_add_kernel<TW>, dim3(n_rows), dim3(256), 0, stream, x, y, partial, splits, (size_t)split_stride,
                       (const TW*)w, width, eps));
    MDMA_LAUNCH_OK("rmsnorm_add");
    return 0;
}

int mdma_add_scaled(float* y, const float* z, float a, long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    long blocks = (n + 255) / 256;
    if (blocks > 1184) blocks = 1184;
    launch_chained(add_scaled_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, y, z, a, n);
    MDMA_LAUNCH_OK("add_scaled");
    return 0;
}

}  // extern "C"
