// Attention whose heads talk to one another before the softmax.
//
// qk_norm_rotate: a token's fused projection row [q heads | k heads | v heads] is made ready in one pass.  Every q and
// k head is (if asked) divided by its root mean square, x / sqrt(mean(x^2) + eps), and multiplied by a weight vector
// shared by all heads, THEN its first `rotary_dim` numbers are turned by the token's position (pairs (2i, 2i+1) or
// (i, i + rotary_dim/2), cos and sin times `magnitude`).  q is written back in place; k and v go to the token's row
// of the paged cache (value heads may have a size of their own).
//
// talking_attention: raw scores s_g = (q_g . k_kv(g)) * scale of ALL query heads g for a key are mixed by a matrix,
// s'_h = sum_g T[h, g] s_g, before the softmax of head h; a query at position p sees the keys up to p; the
// denominator of head h also holds exp(sink_h) when sinks are given (a sink of 0 adds one); the result of head h is
// sum_j p'_hj v_kv(h),j.  Without T the heads are independent.
//
// Plain kernel: a block per token, a warp per head, keys in position order 32 at a time (every warp its head's raw
// scores into shared memory; then every warp mixes its own row, folds the 32 into its running maximum, sum and
// weighted value sum).  Everything in float in one fixed order: the result of a token does not depend on the
// step's cut or on the batch.
//
// Tiled kernel: a block takes up to eight consecutive rows of one sequence and ALL heads (the mixing needs every
// head's score of a key).  Keys are walked 32 at a time.  For every kv head in turn the chunk's keys are staged in
// shared memory as float and the raw scores of its query heads are computed, a lane per key, up to four heads on
// one read of a key; then a warp per (row, head) mixes the raw scores of all heads, applies the mask, and folds the
// chunk into the running maximum and normaliser, leaving the chunk's weights in shared memory; then, for every kv
// head in turn, the chunk's values are staged and the weighted sums are folded into the running sums, lanes over the
// value columns.  The serving engine's kernel: sums in another order than the plain one, rounding only.
#include "common.cuh"

namespace mdma {

constexpr int kTalkMaxDim = 256, kTalkMaxHeads = 32, kPrepWarpsT = 4;

__device__ __forceinline__ float talk_weight(const void* w, int dtype, int e) {
    if (w == nullptr) return 1.0f;
    return dtype == kF32 ? reinterpret_cast<const float*>(w)[e] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[e]);
}

template <typename T>
__global__ void __launch_bounds__(kPrepWarpsT * 32)
qk_norm_rotate_kernel(T* __restrict__ proj, int row_stride, int k_col, int v_col, const int* __restrict__ tok_seq,
                      const int* __restrict__ tok_pos, const int* __restrict__ seq_slot, const float* __restrict__ inv_freq,
                      float magnitude, const void* __restrict__ q_w, const void* __restrict__ k_w, int w_dtype, int norm,
                      float eps, T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ page_table,
                      int max_pages, int page_size, int n_heads, int n_kv_heads, int dim, int v_dim, int rotary_dim,
                      int interleaved, int write_kv) {
    chain_release();
    chain_wait();
    __shared__ float sines[kTalkMaxDim / 2], cosines[kTalkMaxDim / 2];
    __shared__ float rows[kPrepWarpsT][kTalkMaxDim];
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
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    const int head = blockIdx.y * kPrepWarpsT + warp;
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
    float sq = 0.f;
    for (int d = lane; d < dim; d += 32) {
        v[d] = to_float(src[d]);
        sq = fmaf(v[d], v[d], sq);
    }
    if (norm) {
        const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)dim + eps);
        const void* w = is_q ? q_w : k_w;
        for (int d = lane; d < dim; d += 32) v[d] = v[d] * inv * talk_weight(w, w_dtype, d);
    }
    __syncwarp();
    for (int i = lane; i < half; i += 32) {
        const int d0 = interleaved ? 2 * i : i, d1 = interleaved ? 2 * i + 1 : i + half;
        const float a = v[d0], b = v[d1], s = sines[i], c = cosines[i];
        v[d0] = a * c - b * s;
        v[d1] = b * c + a * s;
    }
    __syncwarp();
    for (int d = lane; d < dim; d += 32) dst[d] = from_float<T>(v[d]);
}

// Plain: block = token, warp = head.
template <typename T>
__global__ void __launch_bounds__(kTalkMaxHeads * 32)
talking_attention_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ k_cache,
                         const T* __restrict__ v_cache, const float* __restrict__ talk, const float* __restrict__ sinks,
                         const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                         const int* __restrict__ page_table, int max_pages, int page_size, T* __restrict__ out, int n_heads,
                         int n_kv_heads, int dim, int v_dim, int window, float scale) {
    chain_release();
    chain_wait();
    __shared__ float raw[kTalkMaxHeads][33];
    const int t = blockIdx.x;
    const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = h / (n_heads / n_kv_heads);
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    const int first = window > 0 ? max(0, pos + 1 - window) : 0;
    float qv[kTalkMaxDim / 32], acc[kTalkMaxDim / 32];
    const T* qp = q + (size_t)t * q_row_stride + (size_t)h * dim;
#pragma unroll
    for (int j = 0; j < kTalkMaxDim / 32; ++j) {
        const int d = lane + 32 * j;
        qv[j] = d < dim ? to_float(qp[d]) : 0.f;
        acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int* pages = page_table + (size_t)slot * max_pages;
    for (int p0 = first; p0 <= pos; p0 += 32) {
        const int nk = min(32, pos + 1 - p0);
        float mine = 0.f;
        for (int k = 0; k < nk; ++k) {
            const int p = p0 + k;
            const T* kp = k_cache + (((size_t)pages[p / page_size] * page_size + (size_t)(p % page_size)) * n_kv_heads + kvh) * dim;
            float part = 0.f;
#pragma unroll
            for (int j = 0; j < kTalkMaxDim / 32; ++j) {
                const int d = lane + 32 * j;
                if (d < dim) part = fmaf(qv[j], to_float(kp[d]), part);
            }
            const float s = warp_sum(part) * scale;
            if (lane == k) mine = s;
        }
        if (talk != nullptr) {
            __syncthreads();                    // the mixing of the chunk before has read `raw`
            raw[h][lane] = mine;
            __syncthreads();
            float mixed = 0.f;
            for (int g = 0; g < n_heads; ++g) mixed = fmaf(talk[h * n_heads + g], raw[g][lane], mixed);
            mine = mixed;
        }
        if (lane >= nk) mine = -INFINITY;
        const float m_new = fmaxf(m, warp_max(mine));
        const float corr = expf(m - m_new);          // exp(-inf) = 0 at the first keys
        const float pe_mine = lane < nk ? expf(mine - m_new) : 0.f;
        float sum[kTalkMaxDim / 32];
#pragma unroll
        for (int j = 0; j < kTalkMaxDim / 32; ++j) sum[j] = 0.f;
        float l_new = 0.f;
        for (int k = 0; k < nk; ++k) {
            const int p = p0 + k;
            const T* vp = v_cache + (((size_t)pages[p / page_size] * page_size + (size_t)(p % page_size)) * n_kv_heads + kvh) * v_dim;
            const float pe = __shfl_sync(0xffffffffu, pe_mine, k);
            l_new += pe;
#pragma unroll
            for (int j = 0; j < kTalkMaxDim / 32; ++j) {
                const int d = lane + 32 * j;
                if (d < v_dim) sum[j] = fmaf(pe, to_float(vp[d]), sum[j]);
            }
        }
        l = l * corr + l_new;
#pragma unroll
        for (int j = 0; j < kTalkMaxDim / 32; ++j) acc[j] = acc[j] * corr + sum[j];
        m = m_new;
    }
    float inv = 1.0f / l;
    if (sinks != nullptr) {
        const float sk = sinks[h];
        const float m_all = fmaxf(m, sk);
        const float corr = expf(m - m_all);
        l = l * corr + expf(sk - m_all);
        inv = corr / l;
    }
    T* op = out + ((size_t)t * n_heads + h) * v_dim;
#pragma unroll
    for (int j = 0; j < kTalkMaxDim / 32; ++j) {
        const int d = lane + 32 * j;
        if (d < v_dim) op[d] = from_float<T>(acc[j] * inv);
    }
}

// ---------------------------------------------------------------- tiled kernel
constexpr int kTalkChunk = 32, kTalkWarps = 8, kTalkTogether = 4, kTalkMaxRows = 8;

__device__ __forceinline__ void talk_stage8(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void talk_stage8(const __nv_bfloat16* p, float* v) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
}

// rows [chunk keys][width] of kv head `kvh` into shared memory as float, row pitch `pitch`
template <typename T>
__device__ __forceinline__ void talk_stage(const T* __restrict__ cache, const int* __restrict__ pages, int page_size,
                                           int n_kv_heads, int kvh, int width, int c0, int n_keys, float* dst, int pitch) {
    constexpr int kPerKey = kTalkWarps * 32 / kTalkChunk;
    const int j = threadIdx.x / kPerKey, part = threadIdx.x % kPerKey;
    if (j >= n_keys) return;
    const int p = c0 + j;
    const T* src = cache + (((size_t)pages[p / page_size] * page_size + (size_t)(p % page_size)) * n_kv_heads + kvh) * width;
    float* row = dst + (size_t)j * pitch;
    if (width % 8 == 0 && ((uintptr_t)cache & 15) == 0) {
        for (int d = part * 8; d < width; d += kPerKey * 8) {
            float t8[8];
            talk_stage8(src + d, t8);
#pragma unroll
            for (int i = 0; i < 8; ++i) row[d + i] = t8[i];
        }
    } else {
        for (int d = part; d < width; d += kPerKey) row[d] = to_float(src[d]);
    }
}

static size_t talk_tiled_smem(int rows, int n_heads, int dim, int v_dim) {
    const size_t pairs = (size_t)rows * n_heads;
    const size_t stage = (size_t)kTalkChunk * (size_t)((dim + 1) > v_dim ? (dim + 1) : v_dim);
    return (pairs * dim + pairs * v_dim + stage + 2 * pairs * kTalkChunk + 3 * pairs) * sizeof(float);
}

template <typename T>
__global__ void __launch_bounds__(kTalkWarps * 32)
talking_attention_tiled_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ k_cache,
                               const T* __restrict__ v_cache, const float* __restrict__ talk, const float* __restrict__ sinks,
                               const int* __restrict__ seq_start, const int* __restrict__ seq_pos0,
                               const int* __restrict__ seq_slot, const int* __restrict__ page_table, int max_pages,
                               int page_size, T* __restrict__ out, int n_heads, int n_kv_heads, int dim, int v_dim,
                               int window, float scale, int tile_rows) {
    chain_release();
    chain_wait();
    extern __shared__ float smem[];
    const int s = blockIdx.y;
    const int t0 = seq_start[s], n_new = seq_start[s + 1] - t0;
    const int r0 = blockIdx.x * tile_rows;
    if (r0 >= n_new) return;
    const int rows = min(tile_rows, n_new - r0);
    const int group = n_heads / n_kv_heads;
    const int pos0 = seq_pos0[s] + r0;                     // position of the tile's first row
    const int last = pos0 + rows - 1;
    const int first = window > 0 ? max(0, pos0 + 1 - window) : 0;
    const int* pages = page_table + (size_t)seq_slot[s] * max_pages;
    const int kd = dim + 1;                                // padded key rows: lanes read different keys
    const int pairs = tile_rows * n_heads;                 // (head, row) pairs, head-major: pair = h * tile_rows + r
    float* sq = smem;                                      // [pairs][dim]
    float* so = sq + (size_t)pairs * dim;                  // [pairs][v_dim] running sums
    float* st = so + (size_t)pairs * v_dim;                // [chunk][dim + 1] keys or [chunk][v_dim] values
    float* raw = st + (size_t)kTalkChunk * max(kd, v_dim); // [pairs][chunk] raw scores
    float* sp = raw + (size_t)pairs * kTalkChunk;          // [pairs][chunk] weights of the chunk
    float* sm = sp + (size_t)pairs * kTalkChunk;           // [pairs] running maximum
    float* sl = sm + pairs;                                // [pairs] normaliser
    float* sc = sl + pairs;                                // [pairs] this chunk's correction of the running sums
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (int e = threadIdx.x; e < n_heads * rows * dim; e += blockDim.x) {
        const int h = e / (rows * dim), r = (e / dim) % rows, d = e % dim;
        sq[(size_t)(h * tile_rows + r) * dim + d] = to_float(q[(size_t)(t0 + r0 + r) * q_row_stride + (size_t)h * dim + d]);
    }
    for (int e = threadIdx.x; e < pairs * v_dim; e += blockDim.x) so[e] = 0.f;
    for (int e = threadIdx.x; e < pairs; e += blockDim.x) { sm[e] = -INFINITY; sl[e] = 0.f; }

    for (int c0 = first; c0 <= last; c0 += kTalkChunk) {
        const int n_keys = min(kTalkChunk, last + 1 - c0);
        // raw scores, kv head by kv head
        for (int kvh = 0; kvh < n_kv_heads; ++kvh) {
            __syncthreads();                               // the staging buffer is free (and q is in place)
            talk_stage(k_cache, pages, page_size, n_kv_heads, kvh, dim, c0, n_keys, st, kd);
            __syncthreads();
            const int head_chunks = (group + kTalkTogether - 1) / kTalkTogether;
            for (int unit = warp; unit < rows * head_chunks; unit += kTalkWarps) {
                const int r = unit / head_chunks, g0 = (unit % head_chunks) * kTalkTogether;
                const int ng = min(kTalkTogether, group - g0);
                const int h0 = kvh * group + g0;
                float a[kTalkTogether];
#pragma unroll
                for (int g = 0; g < kTalkTogether; ++g) a[g] = 0.f;
                if (lane < n_keys) {
                    const float* kp = st + lane * kd;
                    const float* qp = sq + (size_t)(h0 * tile_rows + r) * dim;
                    for (int d = 0; d < dim; ++d) {
                        const float kv = kp[d];
#pragma unroll
                        for (int g = 0; g < kTalkTogether; ++g)
                            if (g < ng) a[g] = fmaf(qp[(size_t)g * tile_rows * dim + d], kv, a[g]);
                    }
                }
#pragma unroll
                for (int g = 0; g < kTalkTogether; ++g)
                    if (g < ng) raw[(size_t)((h0 + g) * tile_rows + r) * kTalkChunk + lane] = a[g] * scale;
            }
        }
        __syncthreads();
        // mix, mask, fold into the running maximum and normaliser; the chunk's weights stay in `sp`
        for (int unit = warp; unit < rows * n_heads; unit += kTalkWarps) {
            const int h = unit / rows, r = unit % rows;
            const int pr = h * tile_rows + r;
            const int pos = pos0 + r, p = c0 + lane;
            const int lo = window > 0 ? max(0, pos + 1 - window) : 0;
            float mixed;
            if (talk != nullptr) {
                mixed = 0.f;
                for (int g = 0; g < n_heads; ++g)
                    mixed = fmaf(talk[h * n_heads + g], raw[(size_t)(g * tile_rows + r) * kTalkChunk + lane], mixed);
            } else {
                mixed = raw[(size_t)pr * kTalkChunk + lane];
            }
            const bool seen = lane < n_keys && p <= pos && p >= lo;
            const float score = seen ? mixed : -INFINITY;
            const float cmax = warp_max(score);
            const bool live = cmax != -INFINITY;           // else none of the chunk's keys is visible to this row
            const float m_old = sm[pr];
            const float m_new = live ? fmaxf(m_old, cmax) : m_old;
            const float corr = live ? expf(m_old - m_new) : 1.f;
            const float pe = seen ? expf(score - m_new) : 0.f;
            sp[(size_t)pr * kTalkChunk + lane] = pe;
            const float lsum = warp_sum(pe);
            if (lane == 0) { sm[pr] = m_new; sl[pr] = sl[pr] * corr + lsum; sc[pr] = corr; }
        }
        // weighted sums over the chunk's values, kv head by kv head
        for (int kvh = 0; kvh < n_kv_heads; ++kvh) {
            __syncthreads();                               // weights are written; the staging buffer is free
            talk_stage(v_cache, pages, page_size, n_kv_heads, kvh, v_dim, c0, n_keys, st, v_dim);
            __syncthreads();
            const int head_chunks = (group + kTalkTogether - 1) / kTalkTogether;
            for (int unit = warp; unit < rows * head_chunks; unit += kTalkWarps) {
                const int r = unit / head_chunks, g0 = (unit % head_chunks) * kTalkTogether;
                const int ng = min(kTalkTogether, group - g0);
                const int pr0 = (kvh * group + g0) * tile_rows + r;
                for (int d = lane; d < v_dim; d += 32) {
                    float a[kTalkTogether];
#pragma unroll
                    for (int g = 0; g < kTalkTogether; ++g)
                        a[g] = (g < ng) ? so[(size_t)(pr0 + g * tile_rows) * v_dim + d] * sc[pr0 + g * tile_rows] : 0.f;
                    for (int j = 0; j < n_keys; ++j) {
                        const float v = st[j * v_dim + d];
#pragma unroll
                        for (int g = 0; g < kTalkTogether; ++g)
                            if (g < ng) a[g] = fmaf(sp[(size_t)(pr0 + g * tile_rows) * kTalkChunk + j], v, a[g]);
                    }
#pragma unroll
                    for (int g = 0; g < kTalkTogether; ++g)
                        if (g < ng) so[(size_t)(pr0 + g * tile_rows) * v_dim + d] = a[g];
                }
            }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_heads * rows * v_dim; e += blockDim.x) {
        const int h = e / (rows * v_dim), r = (e / v_dim) % rows, d = e % v_dim;
        const int pr = h * tile_rows + r;
        float o = so[(size_t)pr * v_dim + d], l = sl[pr];
        if (sinks) {
            const float sink = sinks[h], m = sm[pr];
            if (sink > m) { const float c = expf(m - sink); o *= c; l = l * c + 1.0f; }
            else l += expf(sink - m);
        }
        out[((size_t)(t0 + r0 + r) * n_heads + h) * v_dim + d] = from_float<T>(o / l);
    }
}

}  // namespace mdma

using namespace mdma;

extern "C" {

int mdma_qk_norm_rotate(void* proj, int dtype, int row_stride, int k_col, int v_col, const int* tok_seq, const int* tok_pos,
                        const int* seq_slot, const float* inv_freq, float magnitude, const void* q_w, const void* k_w,
                        int w_dtype, int norm, float eps, void* k_cache, void* v_cache, const int* page_table,
                        int max_pages, int page_size, int n_tokens, int n_heads, int n_kv_heads, int dim, int v_dim,
                        int rotary_dim, int interleaved, int write_kv, cudaStream_t stream) {
    MDMA_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads >= 0, "qk_norm_rotate: bad sizes");
    MDMA_REQUIRE(dim > 0 && dim <= kTalkMaxDim && v_dim > 0, "qk_norm_rotate: head size %d is beyond the limit %d", dim, kTalkMaxDim);
    MDMA_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= dim, "qk_norm_rotate: rotary_dim %d does not fit head size %d", rotary_dim, dim);
    MDMA_REQUIRE(rotary_dim == 0 || inv_freq, "qk_norm_rotate: a rotation needs its frequencies");
    MDMA_REQUIRE(w_dtype == kF32 || w_dtype == kBF16, "qk_norm_rotate: unknown weight dtype %d", w_dtype);
    MDMA_REQUIRE(!write_kv || (page_table && k_cache && v_cache && page_size > 0 && max_pages > 0), "qk_norm_rotate: no cache pages");
    if (n_tokens == 0) return 0;
    const int total = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(qk_norm_rotate_kernel<T>, dim3(n_tokens, (total + kPrepWarpsT - 1) / kPrepWarpsT), dim3(kPrepWarpsT * 32),
                       0, stream, (T*)proj, row_stride, k_col, v_col, tok_seq, tok_pos, seq_slot, inv_freq, magnitude, q_w, k_w,
                       w_dtype, norm, eps, (T*)k_cache, (T*)v_cache, page_table, max_pages, page_size, n_heads, n_kv_heads,
                       dim, v_dim, rotary_dim, interleaved, write_kv));
    MDMA_LAUNCH_OK("qk_norm_rotate");
    return 0;
}

// Rows a tile of the tiled kernel can take for this geometry within its shared memory (8, 4, 2, 1), or 0.
int mdma_talking_attention_tile_rows(int n_heads, int n_kv_heads, int dim, int v_dim, int most_rows) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || dim <= 0 || v_dim <= 0) return 0;
    for (int rows = kTalkMaxRows; rows >= 1; rows >>= 1) {
        if (rows > 1 && rows / 2 >= most_rows) continue;          // a smaller tile holds every row a sequence brings
        if (talk_tiled_smem(rows, n_heads, dim, v_dim) <= 200 * 1024) return rows;
    }
    return 0;
}

int mdma_talking_attention_tiled(const void* q, int dtype, int q_row_stride, const void* k_cache, const void* v_cache,
                                 const float* talk, const float* sinks, const int* seq_start, const int* seq_pos0,
                                 const int* seq_slot, const int* page_table, int max_pages, int page_size, void* out,
                                 int n_tokens, int n_seqs, int max_new, int n_heads, int n_kv_heads, int dim, int v_dim,
                                 int window, float scale, cudaStream_t stream) {
    MDMA_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && dim > 0 && v_dim > 0, "talking_attention: bad sizes");
    MDMA_REQUIRE(page_table && page_size > 0 && max_pages > 0 && window >= 0 && seq_start && seq_pos0, "talking_attention: bad cache geometry");
    if (n_tokens == 0 || n_seqs == 0) return 0;
    const int rows = mdma_talking_attention_tile_rows(n_heads, n_kv_heads, dim, v_dim, max_new);
    MDMA_REQUIRE(rows > 0, "talking_attention: the tiled kernel's shared memory does not fit %d heads of %d/%d", n_heads, dim, v_dim);
    MDMA_REQUIRE(n_seqs <= 65535, "talking_attention: too many sequences");
    const size_t smem = talk_tiled_smem(rows, n_heads, dim, v_dim);
    dim3 grid((max_new + rows - 1) / rows, n_seqs);
    MDMA_DISPATCH_DTYPE(dtype, T, {
        static bool raised = false;
        if (!raised) {
            cudaFuncSetAttribute(talking_attention_tiled_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            raised = true;
        }
        launch_chained(talking_attention_tiled_kernel<T>, grid, dim3(kTalkWarps * 32), smem, stream, (const T*)q, q_row_stride,
                       (const T*)k_cache, (const T*)v_cache, talk, sinks, seq_start, seq_pos0, seq_slot, page_table, max_pages,
                       page_size, (T*)out, n_heads, n_kv_heads, dim, v_dim, window, scale, rows);
    });
    MDMA_LAUNCH_OK("talking_attention_tiled");
    return 0;
}

int mdma_talking_attention(const void* q, int dtype, int q_row_stride, const void* k_cache, const void* v_cache,
                           const float* talk, const float* sinks, const int* tok_seq, const int* tok_pos,
                           const int* seq_slot, const int* page_table, int max_pages, int page_size, void* out,
                           int n_tokens, int n_heads, int n_kv_heads, int dim, int v_dim, int window, float scale,
                           cudaStream_t stream) {
    MDMA_REQUIRE(n_heads > 0 && n_heads <= kTalkMaxHeads && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
                 "talking_attention: %d heads over %d kv heads (at most %d heads)", n_heads, n_kv_heads, kTalkMaxHeads);
    MDMA_REQUIRE(dim > 0 && dim <= kTalkMaxDim && v_dim > 0 && v_dim <= kTalkMaxDim,
                 "talking_attention: head sizes %d/%d are beyond the limit %d", dim, v_dim, kTalkMaxDim);
    MDMA_REQUIRE(page_table && page_size > 0 && max_pages > 0 && window >= 0, "talking_attention: bad cache geometry");
    if (n_tokens == 0) return 0;
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(talking_attention_kernel<T>, dim3(n_tokens), dim3(n_heads * 32), 0, stream, (const T*)q, q_row_stride,
                       (const T*)k_cache, (const T*)v_cache, talk, sinks, tok_seq, tok_pos, seq_slot, page_table, max_pages,
                       page_size, (T*)out, n_heads, n_kv_heads, dim, v_dim, window, scale));
    MDMA_LAUNCH_OK("talking_attention");
    return 0;
}

}  // extern "C"
