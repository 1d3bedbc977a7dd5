// Attention whose heads' scores are mixed before the softmax, on the tensor cores (bfloat16, mma.sync m16n8k16).
//
// The mixed score of head h for a key is  s'_h = sum_g T[h, g] (q_g . k_kv(g)) scale.  Query heads of one group c share
// their key head, so the sum over that group is one dot product with k_c:  s'_h = sum_c (sum_{g in c} T[h, g] q_g) . k_c.
// With the mixed queries of all groups side by side, x_h = [x_h,0 | x_h,1 | ...] (kv_heads * dim numbers, x_h,c =
// scale * sum_{g in c} T[h, g] q_g), and a token's key heads side by side as they lie in the cache row,
// kk = [k_0 | k_1 | ...], the mixed score is ONE dot product  s'_h = x_h . kk:  ordinary attention whose query and key
// are kv_heads * dim wide, with one key row for all heads, and whose values are still those of the head's own group.
//
// talking_mix:        x[t, h, :] from q[t, :, :] and T, times scale * log2(e), rounded once to bfloat16.
// talking_attention_mma: block = 16 query rows of one sequence x up to four heads (a warp each).  Keys are walked 32
//   at a time: the key rows of the chunk (all kv heads, one contiguous vector per key) are copied into shared memory
//   once for the block's heads (cp.async; with 108 KB a block two blocks share an SM, so one multiplies while the
//   other waits for its copies); the value rows once for the block when its heads are of one group, else per warp.  S = X K^T by mma.sync with X and K
//   fragments by ldmatrix; mask; online softmax in float with base-2 exponentials; P rounded to bfloat16 in registers
//   is the A operand of O += P V, V fragments by transposed ldmatrix.  Rows of the chunk that no key owns are
//   zero-filled, never loaded.  The denominator takes 2^sink_h at the end when sinks are given.  Single tokens of
//   a few sequences: the keys are divided over `splits` blocks that leave unnormalised sums, merged in split order.
#include "common.cuh"

namespace mdma {

constexpr int kTmChunk = 32, kTmRows = 16, kTmMaxWarps = 4, kTmMaxV = 128;

__device__ __forceinline__ void tm_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void tm_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void tm_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void tm_copy16(void* dst_shared, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src) : "memory");
}
__device__ __forceinline__ void tm_copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tm_copies_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ uint32_t tm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// x[t, h, c * dim + d] = factor * sum_{g in group c} T[h, c * group + g] * q[t, c * group + g, d]
__global__ void __launch_bounds__(256)
talking_mix_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, const float* __restrict__ talk,
                   __nv_bfloat16* __restrict__ x, int n_heads, int n_kv_heads, int dim, float factor) {
    chain_release();
    chain_wait();
    const size_t t = blockIdx.x;
    const int h = blockIdx.y;                              // a block per (token, head)
    const int group = n_heads / n_kv_heads, kd = n_kv_heads * dim;
    const __nv_bfloat16* qr = q + t * q_row_stride;
    for (int e = threadIdx.x; e < kd; e += blockDim.x) {
        const int c = e / dim, d = e - c * dim;
        const float* tw = talk + h * n_heads + c * group;
        const __nv_bfloat16* qc = qr + (size_t)c * group * dim + d;
        float acc = 0.f;
#pragma unroll 4
        for (int g = 0; g < group; ++g) acc = fmaf(tw[g], __bfloat162float(qc[(size_t)g * dim]), acc);
        x[(t * n_heads + h) * (size_t)kd + e] = __float2bfloat16_rn(acc * factor);
    }
}

// the block's mixed queries, a chunk's key rows, and its value rows: once when the block's heads are of one group
// (`v_regions` 1), else once per warp
static size_t tm_smem_bytes(int warps, int v_regions, int kd, int v_dim) {
    return ((size_t)warps * kTmRows * (kd + 8) + (size_t)kTmChunk * (kd + 8) + (size_t)v_regions * kTmChunk * (v_dim + 8)) * 2;
}
constexpr size_t kTmSmemLimit = 220 * 1024;

// VT: value n-tiles of eight columns (v_dim / 8) the accumulators are sized for.
template <int VT>
__global__ void __launch_bounds__(kTmMaxWarps * 32)
talking_attention_mma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ k_cache,
                             const __nv_bfloat16* __restrict__ v_cache, const float* __restrict__ sinks_log2,
                             const int* __restrict__ seq_start, const int* __restrict__ seq_pos0,
                             const int* __restrict__ seq_slot, const int* __restrict__ page_table, int max_pages,
                             int page_size, __nv_bfloat16* __restrict__ out, int n_heads, int n_kv_heads, int dim, int v_dim,
                             int window, int splits, float* __restrict__ partial) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) unsigned char tm_smem[];
    const int s = blockIdx.z;
    const int t0 = seq_start[s], n_new = seq_start[s + 1] - t0;
    const int split = blockIdx.x % splits;
    const int r0 = (blockIdx.x / splits) * kTmRows;
    if (r0 >= n_new) return;
    const int rows = min(kTmRows, n_new - r0);
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * warps + warp;
    const bool active = h < n_heads;
    const int group = n_heads / n_kv_heads;
    const int kvh = active ? h / group : 0;
    const int kd = n_kv_heads * dim, qp = kd + 8, vp = v_dim + 8;         // row pitches in elements (16 bytes of padding)
    __nv_bfloat16* sx = reinterpret_cast<__nv_bfloat16*>(tm_smem);         // [warps][16][kd + 8]
    __nv_bfloat16* sk = sx + (size_t)warps * kTmRows * qp;                 // [32][kd + 8]
    const bool shared_v = group % warps == 0;                              // the block's heads read one kv head
    __nv_bfloat16* sv = sk + (size_t)kTmChunk * qp + (shared_v ? 0 : (size_t)warp * kTmChunk * vp);   // [32][v_dim + 8]
    __nv_bfloat16* sxw = sx + (size_t)warp * kTmRows * qp;
    const int pos0 = seq_pos0[s] + r0, last = pos0 + rows - 1;
    const int first = window > 0 ? max(0, pos0 + 1 - window) : 0;
    const int* pages = page_table + (size_t)seq_slot[s] * max_pages;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);

    // the warp's mixed queries, rows beyond the tile zero
    for (int e = lane; e < kTmRows * (kd / 8); e += 32) {
        const int r = e / (kd / 8), d8 = e % (kd / 8);
        uint4 v = zero4;
        if (active && r < rows) v = *reinterpret_cast<const uint4*>(x + ((size_t)(t0 + r0 + r) * n_heads + h) * kd + d8 * 8);
        *reinterpret_cast<uint4*>(sxw + (size_t)r * qp + d8 * 8) = v;
    }
    float o[VT][4];
#pragma unroll
    for (int n = 0; n < VT; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;       // rows lane/4 and lane/4 + 8
    const int row_lo = lane >> 2, row_hi = row_lo + 8;
    const uint32_t sx_addr = (uint32_t)__cvta_generic_to_shared(sxw);

    // a chunk's key rows and value rows, asked for 16 bytes at a time (a warp takes whole rows: one look at the page
    // table per row); rows no key owns: zero.  Two blocks share an SM: while one waits for its copies the other multiplies.
    const int k_cols = kd / 8, v_cols = v_dim / 8;
    // with `splits` > 1 this block takes a run of the tile's chunks and leaves unnormalised sums for the merge kernel
    const int n_chunks = (last + 1 - first + kTmChunk - 1) / kTmChunk, per_split = (n_chunks + splits - 1) / splits;
    const int c_begin = first + split * per_split * kTmChunk;
    const int c_end = min(last, first + (split + 1) * per_split * kTmChunk - 1);
    for (int c0 = c_begin; c0 <= c_end; c0 += kTmChunk) {
        const int n_keys = min(kTmChunk, last + 1 - c0);
        __syncthreads();                                   // every warp is done with the chunk before
        for (int j = warp; j < kTmChunk; j += warps) {
            __nv_bfloat16* dst = sk + (size_t)j * qp;
            if (j < n_keys) {
                const int p = c0 + j;
                const __nv_bfloat16* src = k_cache + ((size_t)pages[p / page_size] * page_size + (size_t)(p % page_size)) * kd;
                for (int d8 = lane; d8 < k_cols; d8 += 32) tm_copy16(dst + d8 * 8, src + d8 * 8);
            } else {
                for (int d8 = lane; d8 < k_cols; d8 += 32) *reinterpret_cast<uint4*>(dst + d8 * 8) = zero4;
            }
        }
        if (active) {
            // value rows: the block's warps share the work when they share the kv head, else every warp its own
            for (int j = shared_v ? warp : 0; j < kTmChunk; j += shared_v ? warps : 1) {
                __nv_bfloat16* dst = sv + (size_t)j * vp;
                if (j < n_keys) {
                    const int p = c0 + j;
                    const __nv_bfloat16* src = v_cache + (((size_t)pages[p / page_size] * page_size + (size_t)(p % page_size)) * n_kv_heads + kvh) * v_dim;
                    for (int d8 = lane; d8 < v_cols; d8 += 32) tm_copy16(dst + d8 * 8, src + d8 * 8);
                } else {
                    for (int d8 = lane; d8 < v_cols; d8 += 32) *reinterpret_cast<uint4*>(dst + d8 * 8) = zero4;
                }
            }
        }
        tm_copies_commit();
        tm_copies_wait();
        __syncthreads();
        if (!active) continue;
        const uint32_t sk_addr = (uint32_t)__cvta_generic_to_shared(sk), sv_addr = (uint32_t)__cvta_generic_to_shared(sv);
        // S [16 x 32] = X [16 x kd] K^T
        float sc[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n) { sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f; }
#pragma unroll 4
        for (int k0 = 0; k0 < kd; k0 += 16) {
            uint32_t a0, a1, a2, a3;
            tm_ldmatrix_x4(sx_addr + (uint32_t)(((lane & 15) * qp + k0 + (lane >> 4) * 8) * 2), a0, a1, a2, a3);
#pragma unroll
            for (int n2 = 0; n2 < 2; ++n2) {               // two key tiles of eight at a time
                uint32_t b0, b1, b2, b3;
                const int krow = n2 * 16 + (lane & 7) + (lane >> 4) * 8;
                tm_ldmatrix_x4(sk_addr + (uint32_t)((krow * qp + k0 + ((lane >> 3) & 1) * 8) * 2), b0, b1, b2, b3);
                tm_mma(sc[n2 * 2], a0, a1, a2, a3, b0, b1);
                tm_mma(sc[n2 * 2 + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // mask, running maximum and sum (scores are in powers of two already)
        const int p_lo = pos0 + row_lo, p_hi = pos0 + row_hi;
        const int lo_lo = window > 0 ? max(0, p_lo + 1 - window) : 0, lo_hi = window > 0 ? max(0, p_hi + 1 - window) : 0;
        float c_lo = -INFINITY, c_hi = -INFINITY;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int p = c0 + n * 8 + (lane & 3) * 2 + i;
                if (!(p <= p_lo && p >= lo_lo && p <= last)) sc[n][i] = -INFINITY;
                if (!(p <= p_hi && p >= lo_hi && p <= last)) sc[n][2 + i] = -INFINITY;
                c_lo = fmaxf(c_lo, sc[n][i]);
                c_hi = fmaxf(c_hi, sc[n][2 + i]);
            }
        }
        c_lo = fmaxf(c_lo, __shfl_xor_sync(0xffffffffu, c_lo, 1));
        c_lo = fmaxf(c_lo, __shfl_xor_sync(0xffffffffu, c_lo, 2));
        c_hi = fmaxf(c_hi, __shfl_xor_sync(0xffffffffu, c_hi, 1));
        c_hi = fmaxf(c_hi, __shfl_xor_sync(0xffffffffu, c_hi, 2));
        const float n_lo = fmaxf(m_lo, c_lo), n_hi = fmaxf(m_hi, c_hi);
        // a row that has seen no key yet keeps its zero sums (exp2(-inf - -inf) is avoided)
        const float f_lo = n_lo == -INFINITY ? 1.f : exp2f(m_lo - n_lo), f_hi = n_hi == -INFINITY ? 1.f : exp2f(m_hi - n_hi);
        float s_lo = 0.f, s_hi = 0.f;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                sc[n][i] = sc[n][i] == -INFINITY ? 0.f : exp2f(sc[n][i] - n_lo);
                sc[n][2 + i] = sc[n][2 + i] == -INFINITY ? 0.f : exp2f(sc[n][2 + i] - n_hi);
                s_lo += sc[n][i];
                s_hi += sc[n][2 + i];
            }
        }
        s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 1);
        s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 2);
        s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 1);
        s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 2);
        l_lo = l_lo * f_lo + s_lo;
        l_hi = l_hi * f_hi + s_hi;
        m_lo = n_lo;
        m_hi = n_hi;
#pragma unroll
        for (int n = 0; n < VT; ++n) { o[n][0] *= f_lo; o[n][1] *= f_lo; o[n][2] *= f_hi; o[n][3] *= f_hi; }
        // O += P V, P from the score registers
#pragma unroll
        for (int j = 0; j < 2; ++j) {                      // sixteen keys at a time
            const uint32_t a0 = tm_pack(sc[2 * j][0], sc[2 * j][1]), a1 = tm_pack(sc[2 * j][2], sc[2 * j][3]);
            const uint32_t a2 = tm_pack(sc[2 * j + 1][0], sc[2 * j + 1][1]), a3 = tm_pack(sc[2 * j + 1][2], sc[2 * j + 1][3]);
#pragma unroll
            for (int n2 = 0; n2 < VT / 2; ++n2) {
                if (n2 * 16 >= v_dim) continue;            // value tiles beyond the head's width do not exist in shared memory
                uint32_t b0, b1, b2, b3;
                const int vrow = j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                tm_ldmatrix_x4_trans(sv_addr + (uint32_t)((vrow * vp + n2 * 16 + (lane >> 4) * 8) * 2), b0, b1, b2, b3);
                tm_mma(o[n2 * 2], a0, a1, a2, a3, b0, b1);
                tm_mma(o[n2 * 2 + 1], a0, a1, a2, a3, b2, b3);
            }
        }
    }
    if (!active) return;
    if (splits > 1) {
        // [(token, head), split][v_dim + 2]: sums, running maximum, normaliser
#pragma unroll
        for (int n = 0; n < VT; ++n) {
            const int d = n * 8 + (lane & 3) * 2;
            if (d < v_dim) {
                if (row_lo < rows) {
                    float* dst = partial + (((size_t)(t0 + r0 + row_lo) * n_heads + h) * splits + split) * (v_dim + 2);
                    dst[d] = o[n][0]; dst[d + 1] = o[n][1];
                }
                if (row_hi < rows) {
                    float* dst = partial + (((size_t)(t0 + r0 + row_hi) * n_heads + h) * splits + split) * (v_dim + 2);
                    dst[d] = o[n][2]; dst[d + 1] = o[n][3];
                }
            }
        }
        if ((lane & 3) == 0) {
            if (row_lo < rows) {
                float* dst = partial + (((size_t)(t0 + r0 + row_lo) * n_heads + h) * splits + split) * (v_dim + 2);
                dst[v_dim] = m_lo; dst[v_dim + 1] = l_lo;
            }
            if (row_hi < rows) {
                float* dst = partial + (((size_t)(t0 + r0 + row_hi) * n_heads + h) * splits + split) * (v_dim + 2);
                dst[v_dim] = m_hi; dst[v_dim + 1] = l_hi;
            }
        }
        return;
    }
    if (sinks_log2 != nullptr) {
        const float sk2 = sinks_log2[h];
        const float a_lo = fmaxf(m_lo, sk2), a_hi = fmaxf(m_hi, sk2);
        const float f_lo = exp2f(m_lo - a_lo), f_hi = exp2f(m_hi - a_hi);
        l_lo = l_lo * f_lo + exp2f(sk2 - a_lo);
        l_hi = l_hi * f_hi + exp2f(sk2 - a_hi);
#pragma unroll
        for (int n = 0; n < VT; ++n) { o[n][0] *= f_lo; o[n][1] *= f_lo; o[n][2] *= f_hi; o[n][3] *= f_hi; }
    }
    const float i_lo = 1.0f / l_lo, i_hi = 1.0f / l_hi;
#pragma unroll
    for (int n = 0; n < VT; ++n) {
        const int d = n * 8 + (lane & 3) * 2;
        if (d < v_dim) {
            if (row_lo < rows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + r0 + row_lo) * n_heads + h) * v_dim + d) = tm_pack(o[n][0] * i_lo, o[n][1] * i_lo);
            if (row_hi < rows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + r0 + row_hi) * n_heads + h) * v_dim + d) = tm_pack(o[n][2] * i_hi, o[n][3] * i_hi);
        }
    }
}

// out[t, h] = sum_s o_s 2^(m_s - M) / (sum_s l_s 2^(m_s - M) + 2^(sink_h - M)), splits in their order; a warp per (t, h)
__global__ void __launch_bounds__(128)
talking_merge_kernel(const float* __restrict__ partial, const float* __restrict__ sinks_log2, __nv_bfloat16* __restrict__ out,
                     int n_pairs, int n_heads, int v_dim, int splits) {
    chain_release();
    chain_wait();
    const int pair = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= n_pairs) return;
    const float* src = partial + (size_t)pair * splits * (v_dim + 2);
    float M = sinks_log2 ? sinks_log2[pair % n_heads] : -INFINITY;
    for (int k = 0; k < splits; ++k) M = fmaxf(M, src[(size_t)k * (v_dim + 2) + v_dim]);
    float L = sinks_log2 ? exp2f(sinks_log2[pair % n_heads] - M) : 0.f;
    for (int k = 0; k < splits; ++k) {
        const float m = src[(size_t)k * (v_dim + 2) + v_dim];
        if (m != -INFINITY) L += src[(size_t)k * (v_dim + 2) + v_dim + 1] * exp2f(m - M);
    }
    const float inv = 1.0f / L;
    for (int d = lane; d < v_dim; d += 32) {
        float acc = 0.f;
        for (int k = 0; k < splits; ++k) {
            const float m = src[(size_t)k * (v_dim + 2) + v_dim];
            if (m != -INFINITY) acc = fmaf(src[(size_t)k * (v_dim + 2) + d], exp2f(m - M), acc);
        }
        out[(size_t)pair * v_dim + d] = __float2bfloat16_rn(acc * inv);
    }
}

static int tm_warps_for(int n_heads, int n_kv_heads, int dim, int v_dim) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
    const int kd = n_kv_heads * dim;
    if (dim % 8 || kd % 16 || v_dim % 16 || v_dim > kTmMaxV || v_dim <= 0) return 0;
    const int group = n_heads / n_kv_heads;
    for (int w = kTmMaxWarps; w >= 2; w >>= 1)          // one head a block would leave the tensor cores waiting
        if (tm_smem_bytes(w, group % w == 0 ? 1 : w, kd, v_dim) <= kTmSmemLimit) return w;
    return 0;
}

}  // namespace mdma

using namespace mdma;

extern "C" {

// Whether the tensor-core kernel takes this geometry (heads a block takes at a time, or 0).
int mdma_talking_attention_mma_fits(int n_heads, int n_kv_heads, int dim, int v_dim) {
    return tm_warps_for(n_heads, n_kv_heads, dim, v_dim);
}

// x [tokens, heads, kv_heads * dim] bfloat16 is scratch of the caller.  `sinks_log2`: the sinks times log2(e), or null.
int mdma_talking_attention_mma(const void* q, int q_row_stride, const float* talk, void* x, const void* k_cache,
                               const void* v_cache, const float* sinks_log2, const int* seq_start, const int* seq_pos0,
                               const int* seq_slot, const int* page_table, int max_pages, int page_size, void* out,
                               int n_tokens, int n_seqs, int max_new, int n_heads, int n_kv_heads, int dim, int v_dim,
                               int window, float scale, int splits, float* partial, cudaStream_t stream) {
    const int warps = tm_warps_for(n_heads, n_kv_heads, dim, v_dim);
    MDMA_REQUIRE(warps > 0, "talking_attention_mma: %d/%d heads of %d/%d are not a geometry this kernel takes", n_heads, n_kv_heads, dim, v_dim);
    MDMA_REQUIRE(talk && x && page_table && page_size > 0 && max_pages > 0 && window >= 0 && seq_start && seq_pos0, "talking_attention_mma: bad arguments");
    MDMA_REQUIRE(n_seqs <= 65535 && (n_heads + warps - 1) / warps <= 65535, "talking_attention_mma: too many sequences or heads");
    MDMA_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 && ((uintptr_t)out & 3) == 0,
                 "talking_attention_mma: pointers must be 16-byte aligned");
    MDMA_REQUIRE(splits >= 1 && (splits == 1 || partial), "talking_attention_mma: split keys need scratch");
    if (n_tokens == 0 || n_seqs == 0) return 0;
    launch_chained(talking_mix_kernel, dim3(n_tokens, n_heads), dim3(256), 0, stream, (const __nv_bfloat16*)q, q_row_stride, talk,
                   (__nv_bfloat16*)x, n_heads, n_kv_heads, dim, scale * 1.4426950408889634f);
    MDMA_LAUNCH_OK("talking_mix");
    const size_t smem = tm_smem_bytes(warps, (n_heads / n_kv_heads) % warps == 0 ? 1 : warps, n_kv_heads * dim, v_dim);
    dim3 grid(((max_new + kTmRows - 1) / kTmRows) * splits, (n_heads + warps - 1) / warps, n_seqs);
#define MDMA_TM_LAUNCH(VT)                                                                                                  \
    do {                                                                                                                    \
        static bool raised = false;                                                                                         \
        if (!raised) {                                                                                                      \
            cudaFuncSetAttribute(talking_attention_mma_kernel<VT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTmSmemLimit); \
            raised = true;                                                                                                  \
        }                                                                                                                   \
        launch_chained(talking_attention_mma_kernel<VT>, grid, dim3(warps * 32), smem, stream, (const __nv_bfloat16*)x,    \
                       (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, sinks_log2, seq_start, seq_pos0,      \
                       seq_slot, page_table, max_pages, page_size, (__nv_bfloat16*)out, n_heads, n_kv_heads, dim, v_dim,   \
                       window, splits, partial);                                                                            \
    } while (0)
    if (v_dim <= 32) MDMA_TM_LAUNCH(4);
    else if (v_dim <= 64) MDMA_TM_LAUNCH(8);
    else MDMA_TM_LAUNCH(16);
#undef MDMA_TM_LAUNCH
    MDMA_LAUNCH_OK("talking_attention_mma");
    if (splits > 1) {
        launch_chained(talking_merge_kernel, dim3((n_tokens * n_heads + 3) / 4), dim3(128), 0, stream, (const float*)partial,
                       sinks_log2, (__nv_bfloat16*)out, n_tokens * n_heads, n_heads, v_dim, splits);
        MDMA_LAUNCH_OK("talking_merge");
    }
    return 0;
}

}  // extern "C"
