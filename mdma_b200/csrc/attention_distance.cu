// Attention whose positions enter as a penalty on distance, over the paged cache.
//
//   score(i, j) = (q_i . k_j) * scale - slope[h] * (i - j),  0 <= i - j < window (or every j <= i),
// an ordinary softmax over the visible keys, values of a size of their own (`v_dim` may differ from
// the key size), and optionally an output gate: the weighted sum is multiplied element by element
// with sigmoid(gate[t, h * v_dim + d]) (or, with `gate_heads`, by sigmoid(gate[t, h]), one number per head).
// `sinks` [heads]: a softmax with a sink: exp(sink_h) joins head h's normaliser once, with no key and no value.
// `out_scale` multiplies the result.  No rotation is applied here.  Scores, the running maximum, the
// normaliser and the sums are float.
//
// Keys and values live in pages: row (page_table[slot][p / page_size] * page_size + p % page_size) of
// a pool [rows, kv_heads, dim] for keys and [rows, kv_heads, v_dim] for values.
//
// Two kernels compute it.  The plain one keeps one warp per (token, head) and visits the keys in
// position order, so its result does not depend on how the tokens were cut into steps or on the rest
// of the batch: the 32-bit engine's, and the reference of the other.  The tiled one gives a block
// one (sequence, kv head, tile of query rows): keys and values of a range are staged in shared
// memory once for all its rows and query heads; each warp owns a few (row, head) pairs.
#include "common.cuh"

namespace mdma {

constexpr int kMaxDim = 256;

// ---------------------------------------------------------------- cache write
// k rows [kv_heads * dim] and v rows [kv_heads * v_dim] of the projection (columns k_col.., v_col..) go
// to the token's cache row.
template <typename T>
__global__ void __launch_bounds__(256)
kv_store_kernel(const T* __restrict__ proj, int proj_stride, int k_col, int v_col, int k_width, int v_width,
                const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                const int* __restrict__ page_table, int max_pages, int page_size,
                T* __restrict__ k_cache, T* __restrict__ v_cache) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    const size_t row = (size_t)page_table[(size_t)slot * max_pages + pos / page_size] * page_size + (size_t)(pos % page_size);
    const T* src = proj + (size_t)t * proj_stride;
    for (int e = threadIdx.x; e < k_width; e += blockDim.x) k_cache[row * k_width + e] = src[k_col + e];
    for (int e = threadIdx.x; e < v_width; e += blockDim.x) v_cache[row * v_width + e] = src[v_col + e];
}

// ---------------------------------------------------------------- plain kernel
template <typename T>
__global__ void __launch_bounds__(128)
attention_distance_plain_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ k_cache,
                                const T* __restrict__ v_cache, const int* __restrict__ tok_seq,
                                const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                                const int* __restrict__ page_table, int max_pages, int page_size,
                                const float* __restrict__ slopes, const T* __restrict__ gate, int gate_stride,
                                T* __restrict__ out, int n_heads, int n_kv_heads, int dim, int v_dim, int window,
                                float scale, const float* __restrict__ sinks, int gate_heads, float out_scale) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int h = blockIdx.y * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (h >= n_heads) return;
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    const int kvh = h / (n_heads / n_kv_heads);
    const int first = window > 0 ? max(0, pos + 1 - window) : 0;
    const float slope = slopes ? slopes[h] : 0.f;

    float qv[kMaxDim / 32], acc[kMaxDim / 32];
    const T* qp = q + (size_t)t * q_row_stride + (size_t)h * dim;
#pragma unroll
    for (int j = 0; j < kMaxDim / 32; ++j) {
        const int d = lane + 32 * j;
        qv[j] = d < dim ? to_float(qp[d]) : 0.f;
        acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int* pages = page_table + (size_t)slot * max_pages;
    for (int p = first; p <= pos; ++p) {
        const size_t row = ((size_t)pages[p / page_size] * page_size + (size_t)(p % page_size)) * n_kv_heads + kvh;
        const T* kp = k_cache + row * dim;
        const T* vp = v_cache + row * v_dim;
        float part = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxDim / 32; ++j) {
            const int d = lane + 32 * j;
            if (d < dim) part = fmaf(qv[j], to_float(kp[d]), part);
        }
        const float s = warp_sum(part) * scale - slope * (float)(pos - p);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);     // exp(-inf) = 0 on the first key
        const float pe = expf(s - m_new);
        l = l * corr + pe;
#pragma unroll
        for (int j = 0; j < kMaxDim / 32; ++j) {
            const int d = lane + 32 * j;
            if (d < v_dim) acc[j] = acc[j] * corr + pe * to_float(vp[d]);
        }
        m = m_new;
    }
    if (sinks) {
        const float sink = sinks[h];
        const float m_new = fmaxf(m, sink);
        const float corr = expf(m - m_new);
        l = l * corr + expf(sink - m_new);
#pragma unroll
        for (int j = 0; j < kMaxDim / 32; ++j) acc[j] *= corr;
    }
    T* op = out + ((size_t)t * n_heads + h) * v_dim;
    const T* gp = gate ? gate + (size_t)t * gate_stride + (gate_heads ? (size_t)h : (size_t)h * v_dim) : nullptr;
    const float inv = out_scale / l;
#pragma unroll
    for (int j = 0; j < kMaxDim / 32; ++j) {
        const int d = lane + 32 * j;
        if (d < v_dim) {
            float o = acc[j] * inv;
            if (gp) o *= 1.0f / (1.0f + expf(-to_float(gp[gate_heads ? 0 : d])));
            op[d] = from_float<T>(o);
        }
    }
}

// ---------------------------------------------------------------- tiled kernel
// Block = (tile of kTileRows query rows of one sequence, kv head).  The keys a tile can see are
// [first key of its first row, position of its last row]; they are walked in chunks of kChunkKeys keys
// that are staged in shared memory as float (keys [chunk][dim + 1], values [chunk][v_dim]).  Each warp
// owns rows of the tile in turn, with up to four of the group's heads at once; a lane takes the keys lane,
// lane + 32, ... of the chunk: it computes whole scores from shared memory (no shuffles per key; a key's
// numbers are read once for the heads together), the warp agrees on each head's maximum of the chunk, and
// the weighted sums over the chunk's values are taken with lanes over the value columns.  The running
// maximum, normaliser and sums of a (row, head) pair live in shared memory between chunks.
constexpr int kTileRows = 16, kChunkKeys = 64, kTileWarps = 8, kHeadsTogether = 4;

// eight consecutive elements as floats by 16-byte loads (the address is 16-byte aligned)
__device__ __forceinline__ void stage8(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void stage8(const __nv_bfloat16* p, float* v) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
}

// GH: how many of a group's heads a warp takes together (4, or 1 for steps whose tiles have a row or two: there the
// warps would be left without work).
template <typename T, int GH>
__global__ void __launch_bounds__(kTileWarps * 32)
attention_distance_tiled_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ k_cache,
                                const T* __restrict__ v_cache, const int* __restrict__ seq_start,
                                const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot,
                                const int* __restrict__ page_table, int max_pages, int page_size,
                                const float* __restrict__ slopes, const T* __restrict__ gate, int gate_stride,
                                T* __restrict__ out, int n_heads, int n_kv_heads, int dim, int v_dim, int window,
                                float scale, const float* __restrict__ sinks, int gate_heads, float out_scale) {
    chain_release();
    chain_wait();
    extern __shared__ float smem[];
    const int s = blockIdx.z, kvh = blockIdx.y;
    const int t0 = seq_start[s], n_new = seq_start[s + 1] - t0;
    const int r0 = blockIdx.x * kTileRows;
    if (r0 >= n_new) return;
    const int rows = min(kTileRows, n_new - r0);
    const int group = n_heads / n_kv_heads;
    const int pairs = rows * group;
    const int pos0 = seq_pos0[s] + r0;                     // position of the tile's first row
    const int last = pos0 + rows - 1;
    const int first = window > 0 ? max(0, pos0 + 1 - window) : 0;
    const int* pages = page_table + (size_t)seq_slot[s] * max_pages;
    const int kd = dim + 1;                                // padded key rows: lanes read different keys
    float* sq = smem;                                      // [kTileRows * group][dim]
    float* sk = sq + (size_t)kTileRows * group * dim;      // [kChunkKeys][dim + 1]
    float* sv = sk + (size_t)kChunkKeys * kd;              // [kChunkKeys][v_dim]
    float* so = sv + (size_t)kChunkKeys * v_dim;           // [kTileRows * group][v_dim]
    float* sm = so + (size_t)kTileRows * group * v_dim;    // [kTileRows * group] running maximum
    float* sl = sm + kTileRows * group;                    // [kTileRows * group] normaliser
    float* sp = sl + kTileRows * group;                    // [kTileWarps][kHeadsTogether][kChunkKeys] weights of the chunk
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec_k = dim % 8 == 0 && ((uintptr_t)k_cache & 15) == 0, vec_v = v_dim % 8 == 0 && ((uintptr_t)v_cache & 15) == 0;

    for (int e = threadIdx.x; e < pairs * dim; e += blockDim.x) {
        const int pr = e / dim, d = e % dim;
        const int r = pr / group, g = pr % group;
        sq[e] = to_float(q[(size_t)(t0 + r0 + r) * q_row_stride + (size_t)(kvh * group + g) * dim + d]);
    }
    for (int e = threadIdx.x; e < pairs * v_dim; e += blockDim.x) so[e] = 0.f;
    for (int e = threadIdx.x; e < pairs; e += blockDim.x) { sm[e] = -INFINITY; sl[e] = 0.f; }

    for (int c0 = first; c0 <= last; c0 += kChunkKeys) {
        const int n_keys = min(kChunkKeys, last + 1 - c0);
        __syncthreads();                                   // the chunk before is done with (and q is in place)
        {   // four threads a key: one look at the page table, then 16-byte loads where the rows allow them
            constexpr int kPerKey = kTileWarps * 32 / kChunkKeys;
            const int j = threadIdx.x / kPerKey, part = threadIdx.x % kPerKey;
            if (j < n_keys) {
                const int p = c0 + j;
                const size_t row = ((size_t)pages[p / page_size] * page_size + (size_t)(p % page_size)) * n_kv_heads + kvh;
                const T* kp = k_cache + row * dim;
                const T* vp = v_cache + row * v_dim;
                float* kd_row = sk + j * kd;
                float* vd_row = sv + j * v_dim;
                if (vec_k) {
                    for (int d = part * 8; d < dim; d += kPerKey * 8) {
                        float t8[8];
                        stage8(kp + d, t8);
#pragma unroll
                        for (int i = 0; i < 8; ++i) kd_row[d + i] = t8[i];
                    }
                } else {
                    for (int d = part; d < dim; d += kPerKey) kd_row[d] = to_float(kp[d]);
                }
                if (vec_v) {
                    for (int d = part * 8; d < v_dim; d += kPerKey * 8) {
                        float t8[8];
                        stage8(vp + d, t8);
#pragma unroll
                        for (int i = 0; i < 8; ++i) vd_row[d + i] = t8[i];
                    }
                } else {
                    for (int d = part; d < v_dim; d += kPerKey) vd_row[d] = to_float(vp[d]);
                }
            }
        }
        __syncthreads();
        // a warp takes a row and up to kHeadsTogether of the group's heads at once: a key's numbers (and later a
        // value's) are read from shared memory once for all of them
        float* wp = sp + warp * kHeadsTogether * kChunkKeys;
        const int head_chunks = (group + GH - 1) / GH;
        for (int unit = warp; unit < rows * head_chunks; unit += kTileWarps) {
            const int r = unit / head_chunks, g0 = (unit % head_chunks) * GH;
            const int ng = min(GH, group - g0);
            const int pr0 = r * group + g0;
            const int pos = pos0 + r;
            const int lo = window > 0 ? max(0, pos + 1 - window) : 0;
            const float* qp = sq + (size_t)pr0 * dim;
            float sc[kChunkKeys / 32][GH];
            float cmax[GH];
#pragma unroll
            for (int g = 0; g < GH; ++g) cmax[g] = -INFINITY;
#pragma unroll
            for (int u = 0; u < kChunkKeys / 32; ++u) {
                const int j = lane + 32 * u, p = c0 + j;
                const bool seen = j < n_keys && p <= pos && p >= lo;
                float a[GH];
#pragma unroll
                for (int g = 0; g < GH; ++g) a[g] = 0.f;
                if (seen) {
                    const float* kp = sk + j * kd;
                    for (int d = 0; d < dim; ++d) {
                        const float kv = kp[d];
#pragma unroll
                        for (int g = 0; g < GH; ++g)
                            if (g < ng) a[g] = fmaf(qp[(size_t)g * dim + d], kv, a[g]);
                    }
                }
#pragma unroll
                for (int g = 0; g < GH; ++g) {
                    const float slope = (slopes && g < ng) ? slopes[kvh * group + g0 + g] : 0.f;
                    sc[u][g] = (seen && g < ng) ? a[g] * scale - slope * (float)(pos - p) : -INFINITY;
                    cmax[g] = fmaxf(cmax[g], sc[u][g]);
                }
            }
            float corr[GH], lsum[GH], m_new[GH];
            bool any = false;
#pragma unroll
            for (int g = 0; g < GH; ++g) {
                cmax[g] = warp_max(cmax[g]);
                const bool live = cmax[g] != -INFINITY;        // else none of the chunk's keys is visible to this row and head
                any = any || live;
                const float m_old = (g < ng) ? sm[pr0 + g] : -INFINITY;
                m_new[g] = live ? fmaxf(m_old, cmax[g]) : m_old;
                corr[g] = live ? expf(m_old - m_new[g]) : 1.f;
                float part = 0.f;
#pragma unroll
                for (int u = 0; u < kChunkKeys / 32; ++u) {
                    const float pe = (!live || sc[u][g] == -INFINITY) ? 0.f : expf(sc[u][g] - m_new[g]);
                    wp[g * kChunkKeys + lane + 32 * u] = pe;
                    part += pe;
                }
                lsum[g] = warp_sum(part);
            }
            if (!any) continue;
            __syncwarp();
            float* op = so + (size_t)pr0 * v_dim;
            for (int d = lane; d < v_dim; d += 32) {
                float a[GH];
#pragma unroll
                for (int g = 0; g < GH; ++g) a[g] = (g < ng) ? op[(size_t)g * v_dim + d] * corr[g] : 0.f;
                for (int j = 0; j < n_keys; ++j) {
                    const float v = sv[j * v_dim + d];
#pragma unroll
                    for (int g = 0; g < GH; ++g) a[g] = fmaf(wp[g * kChunkKeys + j], v, a[g]);
                }
#pragma unroll
                for (int g = 0; g < GH; ++g)
                    if (g < ng) op[(size_t)g * v_dim + d] = a[g];
            }
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int g = 0; g < GH; ++g)
                    if (g < ng) { sm[pr0 + g] = m_new[g]; sl[pr0 + g] = sl[pr0 + g] * corr[g] + lsum[g]; }
            }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < pairs * v_dim; e += blockDim.x) {
        const int pr = e / v_dim, d = e % v_dim;
        const int r = pr / group, g = pr % group;
        const int h = kvh * group + g;
        const size_t t = (size_t)(t0 + r0 + r);
        float o = so[e], l = sl[pr];
        if (sinks) {
            const float sink = sinks[h], m = sm[pr];
            if (sink > m) { const float c = expf(m - sink); o *= c; l = l * c + 1.0f; }
            else l += expf(sink - m);
        }
        o = o / l * out_scale;
        if (gate) o *= 1.0f / (1.0f + expf(-to_float(gate[t * gate_stride + (gate_heads ? (size_t)h : (size_t)h * v_dim + d)])));
        out[(t * n_heads + h) * v_dim + d] = from_float<T>(o);
    }
}

static size_t tiled_smem_bytes(int group, int dim, int v_dim) {
    const size_t pairs = (size_t)kTileRows * group;
    return sizeof(float) * (pairs * dim + (size_t)kChunkKeys * (dim + 1) + (size_t)kChunkKeys * v_dim + pairs * v_dim +
                            2 * pairs + (size_t)kTileWarps * kHeadsTogether * kChunkKeys);
}

}  // namespace mdma

using namespace mdma;

extern "C" {

int mdma_kv_store(const void* proj, int dtype, int proj_stride, int k_col, int v_col, int k_width, int v_width,
                  const int* tok_seq, const int* tok_pos, const int* seq_slot, const int* page_table, int max_pages,
                  int page_size, void* k_cache, void* v_cache, int n_tokens, cudaStream_t stream) {
    MDMA_REQUIRE(n_tokens >= 0 && k_width > 0 && v_width > 0 && page_size > 0 && max_pages > 0, "kv_store: bad sizes");
    if (n_tokens == 0) return 0;
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(kv_store_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (const T*)proj, proj_stride, k_col, v_col,
                       k_width, v_width, tok_seq, tok_pos, seq_slot, page_table, max_pages, page_size, (T*)k_cache,
                       (T*)v_cache));
    MDMA_LAUNCH_OK("kv_store");
    return 0;
}

// Whether the tiled kernel takes this geometry (its shared memory must fit one block).
int mdma_attention_distance_tiled_fits(int n_heads, int n_kv_heads, int dim, int v_dim) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
    return tiled_smem_bytes(n_heads / n_kv_heads, dim, v_dim) <= 200 * 1024 ? 1 : 0;
}

// tiled != 0: the tiled kernel (needs seq_start / seq_pos0 and max_new, the most rows a sequence brings).
int mdma_attention_distance(const void* q, int dtype, int q_row_stride, const void* k_cache, const void* v_cache,
                            const int* tok_seq, const int* tok_pos, const int* seq_slot, const int* seq_start,
                            const int* seq_pos0, const int* page_table, int max_pages, int page_size,
                            const float* slopes, const void* gate, int gate_stride, void* out, int n_tokens, int n_seqs,
                            int max_new, int n_heads, int n_kv_heads, int dim, int v_dim, int window, float scale,
                            int tiled, const float* sinks, int gate_heads, float out_scale, cudaStream_t stream) {
    MDMA_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention: %d heads over %d kv heads", n_heads, n_kv_heads);
    MDMA_REQUIRE(dim > 0 && dim <= kMaxDim && v_dim > 0 && v_dim <= kMaxDim, "attention: head sizes %d / %d are beyond the limit %d", dim, v_dim, kMaxDim);
    MDMA_REQUIRE(page_table && page_size > 0 && max_pages > 0 && window >= 0, "attention: bad cache geometry");
    if (n_tokens == 0) return 0;
    if (tiled) {
        const int group = n_heads / n_kv_heads;
        const size_t smem = tiled_smem_bytes(group, dim, v_dim);
        MDMA_REQUIRE(smem <= 200 * 1024, "attention: the tiled kernel's shared memory (%zu bytes) does not fit", smem);
        MDMA_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && n_kv_heads <= 65535 && max_new > 0, "attention: bad batch");
        dim3 grid((max_new + kTileRows - 1) / kTileRows, n_kv_heads, n_seqs);
        const int tile_rows = max_new < kTileRows ? max_new : kTileRows;
        const bool together = tile_rows * ((group + kHeadsTogether - 1) / kHeadsTogether) >= kTileWarps;
#define MDMA_TILED_LAUNCH(GH)                                                                                              \
        do {                                                                                                                \
            static bool raised = false;                                                                                     \
            if (!raised) {                                                                                                  \
                cudaFuncSetAttribute(attention_distance_tiled_kernel<T, GH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
                raised = true;                                                                                              \
            }                                                                                                               \
            launch_chained(attention_distance_tiled_kernel<T, GH>, grid, dim3(kTileWarps * 32), smem, stream, (const T*)q,  \
                           q_row_stride, (const T*)k_cache, (const T*)v_cache, seq_start, seq_pos0, seq_slot, page_table,   \
                           max_pages, page_size, slopes, (const T*)gate, gate_stride, (T*)out, n_heads, n_kv_heads, dim,    \
                           v_dim, window, scale, sinks, gate_heads, out_scale);                                             \
        } while (0)
        MDMA_DISPATCH_DTYPE(dtype, T, {
            if (together) MDMA_TILED_LAUNCH(kHeadsTogether);
            else MDMA_TILED_LAUNCH(1);
        });
#undef MDMA_TILED_LAUNCH
        MDMA_LAUNCH_OK("attention_distance_tiled");
        return 0;
    }
    dim3 grid(n_tokens, (n_heads + 3) / 4);
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(attention_distance_plain_kernel<T>, grid, dim3(128), 0, stream, (const T*)q, q_row_stride,
                       (const T*)k_cache, (const T*)v_cache, tok_seq, tok_pos, seq_slot, page_table, max_pages, page_size,
                       slopes, (const T*)gate, gate_stride, (T*)out, n_heads, n_kv_heads, dim, v_dim, window, scale,
                       sinks, gate_heads, out_scale));
    MDMA_LAUNCH_OK("attention_distance");
    return 0;
}

}  // extern "C"
