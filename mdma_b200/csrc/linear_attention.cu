// Linear attention with a fixed decay per head, and the gated norm that follows it.
//
// Per head, with q, k [dim] and v [vdim] of a token (each the SiLU of its projection, taken in float):
//     S_t = decay * S_(t-1) + k_t v_t^T          S [dim][vdim], floats, carried from token to token per sequence
//     o_t = S_t^T q_t
// The columns of S do not touch one another, so a block owns one (sequence, head, part of the columns).
//
// Row by row (`linear_attention_scan_kernel`): the block keeps its part of S in shared memory, walks the sequence's
// rows in order and writes S back at the end.  Every sum has one fixed order, so the result does not depend on how
// the rows were cut into steps: the 32-bit engine's walk, single tokens, and the reference of the other.
//
// A chunk of rows at a time (`linear_attention_chunk_kernel`, steps of many rows): kChunk rows are staged, and
// within a chunk  o_i = decay^(i+1) S^T q_i + sum_(j <= i) decay^(i-j) (q_i . k_j) v_j,  and afterwards
// S <- decay^n S + sum_j decay^(n-1-j) k_j v_j^T.  Equal to the walk row by row up to rounding.  Long sequences are
// cut into runs of `run_rows` rows that are walked side by side, since the recurrence is linear in S: pass kLinLocal
// walks every run but the last from S = 0 and leaves the run's last S in scratch; pass kLinFrom sums up each run's
// starting S from those in order (start[r+1] = decay^run_rows start[r] + local[r]), walks the run from there and
// writes o, the last run also the sequence's state.
//
// gated_rmsnorm: out = o / sqrt(mean(o^2) + eps) * w * sigmoid(g) * scale over the heads side by side.
#include "common.cuh"

namespace mdma {

__device__ __forceinline__ float silu_float(float z) { return z / (1.0f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(256)
linear_attention_scan_kernel(const T* __restrict__ proj, int row_stride, int q_col, int k_col, int v_col,
                             const float* __restrict__ decay, const int* __restrict__ seq_start,
                             const int* __restrict__ seq_slot, float* __restrict__ state, size_t state_stride,
                             float* __restrict__ out, int heads, int dim, int vdim, int cols) {
    chain_release();
    chain_wait();
    extern __shared__ float sm[];
    const int s = blockIdx.x, h = blockIdx.y;
    const int c0 = blockIdx.z * cols, cw = min(cols, vdim - c0);
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    if (t1 <= t0) return;
    float* S = sm;                     // [dim][cols]
    float* sq = S + (size_t)dim * cols;
    float* sk = sq + dim;
    float* sv = sk + dim;              // [cols]
    float* red = sv + cols;            // [row groups][columns of this block]: at most 256
    float* st = state + (size_t)seq_slot[s] * state_stride + (size_t)h * dim * vdim;
    for (int e = threadIdx.x; e < dim * cw; e += blockDim.x) S[(e / cw) * cols + e % cw] = st[(size_t)(e / cw) * vdim + c0 + e % cw];
    const int groups = blockDim.x / cw > 0 ? blockDim.x / cw : 1;      // cw <= blockDim.x
    const int r = threadIdx.x / cw, j = threadIdx.x % cw;
    const bool active = r < groups;
    const float dk = decay[h];
    for (int t = t0; t < t1; ++t) {
        const T* row = proj + (size_t)t * row_stride;
        for (int e = threadIdx.x; e < dim; e += blockDim.x) {
            sq[e] = silu_float(to_float(row[q_col + h * dim + e]));
            sk[e] = silu_float(to_float(row[k_col + h * dim + e]));
        }
        for (int e = threadIdx.x; e < cw; e += blockDim.x) sv[e] = silu_float(to_float(row[v_col + h * vdim + c0 + e]));
        __syncthreads();
        if (active) {
            const float vj = sv[j];
            float acc = 0.f;
            for (int i = r; i < dim; i += groups) {
                const float v = fmaf(dk, S[i * cols + j], sk[i] * vj);
                S[i * cols + j] = v;
                acc = fmaf(v, sq[i], acc);
            }
            red[r * cw + j] = acc;
        }
        __syncthreads();
        if (threadIdx.x < cw) {
            float o = 0.f;
            for (int g = 0; g < groups; ++g) o += red[g * cw + threadIdx.x];
            out[(size_t)t * heads * vdim + (size_t)h * vdim + c0 + threadIdx.x] = o;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < dim * cw; e += blockDim.x) st[(size_t)(e / cw) * vdim + c0 + e % cw] = S[(e / cw) * cols + e % cw];
}

// ---------------------------------------------------------------- single rows
// Steps that bring one row a sequence: S never enters shared memory.  Block = (sequence, head, kStepCols columns), 256
// threads; a thread owns four neighbouring columns of every 64th row of S, reads them from the state row, brings them up
// to date, writes them back and sums its part of o; the 64 parts of a column are added in one fixed order.  A sequence
// of several rows is walked row by row from the state row itself (right, but slow: the serving engine takes this kernel
// only where no sequence brings more than one row).
constexpr int kStepCols = 16, kStepQuads = kStepCols / 4, kStepGroups = 256 / kStepQuads;

template <typename T>
__global__ void __launch_bounds__(256)
linear_attention_step_kernel(const T* __restrict__ proj, int row_stride, int q_col, int k_col, int v_col,
                             const float* __restrict__ decay, const int* __restrict__ seq_start,
                             const int* __restrict__ seq_slot, float* __restrict__ state, size_t state_stride,
                             float* __restrict__ out, int heads, int dim, int vdim) {
    chain_release();
    chain_wait();
    extern __shared__ float sm[];
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * kStepCols;
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    if (t1 <= t0) return;
    float* sq = sm;                    // [dim]
    float* sk = sq + dim;              // [dim]
    float* sv = sk + dim;              // [kStepCols]
    float* red = sv + kStepCols;       // [kStepGroups][kStepCols]
    const int quad = threadIdx.x % kStepQuads, rg = threadIdx.x / kStepQuads;
    const int c = c0 + 4 * quad;
    const bool active = c < vdim;      // vdim is a multiple of four
    float* st = state + (size_t)seq_slot[s] * state_stride + (size_t)h * dim * vdim + c;
    const float dk = decay[h];
    for (int t = t0; t < t1; ++t) {
        const T* row = proj + (size_t)t * row_stride;
        for (int e = threadIdx.x; e < dim; e += blockDim.x) {
            sq[e] = silu_float(to_float(row[q_col + h * dim + e]));
            sk[e] = silu_float(to_float(row[k_col + h * dim + e]));
        }
        if (threadIdx.x < kStepCols) sv[threadIdx.x] = c0 + threadIdx.x < vdim ? silu_float(to_float(row[v_col + h * vdim + c0 + threadIdx.x])) : 0.f;
        __syncthreads();
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (active) {
            const float4 v4 = *reinterpret_cast<const float4*>(sv + 4 * quad);
            for (int i = rg; i < dim; i += kStepGroups) {
                float4 e = *reinterpret_cast<const float4*>(st + (size_t)i * vdim);
                const float ki = sk[i], qi = sq[i];
                e.x = fmaf(dk, e.x, ki * v4.x); e.y = fmaf(dk, e.y, ki * v4.y);
                e.z = fmaf(dk, e.z, ki * v4.z); e.w = fmaf(dk, e.w, ki * v4.w);
                *reinterpret_cast<float4*>(st + (size_t)i * vdim) = e;
                acc.x = fmaf(e.x, qi, acc.x); acc.y = fmaf(e.y, qi, acc.y);
                acc.z = fmaf(e.z, qi, acc.z); acc.w = fmaf(e.w, qi, acc.w);
            }
        }
        *reinterpret_cast<float4*>(red + rg * kStepCols + 4 * quad) = acc;
        __syncthreads();
        if (threadIdx.x < kStepCols && c0 + threadIdx.x < vdim) {
            float o = 0.f;
            for (int g = 0; g < kStepGroups; ++g) o += red[g * kStepCols + threadIdx.x];
            out[(size_t)t * heads * vdim + (size_t)h * vdim + c0 + threadIdx.x] = o;
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------- a chunk of rows at a time
// Block = (sequence or run, head, part of the columns), 256 threads.  Shared memory, floats, every row a multiple
// of four long so that threads read four neighbours at once: S [dimP][colsP] (dimP a multiple of 8); q, k
// [kChunk][dimP + 4]; v [kChunk][colsP]; A [kChunk][kChunk + 4]; decay^0 .. decay^kChunk; one factor per row.  Rows
// and columns beyond the data are zero.
//   A[i][j] = decay^(i-j) (q_i . k_j), j <= i: a thread owns two rows and two columns.
//   o_i[c]  = decay^(i+1) sum_d q_i[d] S[d][c] + sum_j A[i][j] v_j[c]: a thread owns two rows of four columns.
//   S[d][c] = decay^n S[d][c] + sum_j decay^(n-1-j) k_j[d] v_j[c]: a thread owns eight by four entries.
// Where every row part starts on a 16-byte boundary (`staged`: bfloat16 rows, sizes and offsets multiples of 8) the
// next chunk's rows are on their way into a raw buffer (cp.async) while this chunk is computed.
// Passes over runs: kLinLocal leaves in `run_state[run]` the run's last S from zero (v_j carries the whole factor
// decay^(rows after j in the run), so S is never rescaled), and the block of a sequence's last run leaves a copy of
// the sequence's state there instead; kLinFrom starts run r from
// decay^(r run_rows) state + sum_(p < r) decay^((r-1-p) run_rows) local[p], summed in order.
constexpr int kChunk = 32;
constexpr int kAPitch = kChunk + 4;
enum LinPass : int { kLinWhole = 0, kLinLocal = 1, kLinFrom = 2 };
constexpr int kLinSingleRows = 2;      // value of the launcher's `chunked` that asks for the single-row kernel

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void fma4(float4& acc, float a, const float4& b) {
    acc.x = fmaf(a, b.x, acc.x); acc.y = fmaf(a, b.y, acc.y); acc.z = fmaf(a, b.z, acc.z); acc.w = fmaf(a, b.w, acc.w);
}
__device__ __forceinline__ void scale4(float4& v, float a) { v.x *= a; v.y *= a; v.z *= a; v.w *= a; }
__device__ __forceinline__ float dot4(const float4& a, const float4& b, float acc) {
    return fmaf(a.w, b.w, fmaf(a.z, b.z, fmaf(a.y, b.y, fmaf(a.x, b.x, acc))));
}
__device__ __forceinline__ void copy16_async(void* dst_shared, const void* src_global) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst_shared);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(d), "l"(src_global) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
// eight bfloat16 -> the SiLU of each, times `f`, as two float4
__device__ __forceinline__ void silu8(const uint4& raw, float f, float4& lo, float4& hi) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]), c = __bfloat1622float2(p[2]), d = __bfloat1622float2(p[3]);
    lo = make_float4(silu_float(a.x) * f, silu_float(a.y) * f, silu_float(b.x) * f, silu_float(b.y) * f);
    hi = make_float4(silu_float(c.x) * f, silu_float(c.y) * f, silu_float(d.x) * f, silu_float(d.y) * f);
}

template <typename T, int PASS>
__global__ void __launch_bounds__(256)
linear_attention_chunk_kernel(const T* __restrict__ proj, int row_stride, int q_col, int k_col, int v_col,
                              const float* __restrict__ decay, const int* __restrict__ seq_start,
                              const int* __restrict__ seq_slot, float* __restrict__ state, size_t state_stride,
                              float* __restrict__ out, int heads, int dim, int vdim, int cols, int run_rows, int max_runs,
                              float* __restrict__ run_state, int staged) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float sm[];
    const int s = PASS == kLinWhole ? blockIdx.x : blockIdx.x / max_runs;
    const int run = PASS == kLinWhole ? 0 : blockIdx.x % max_runs;
    const int h = blockIdx.y;
    const int c0 = blockIdx.z * cols, cw = min(cols, vdim - c0);
    int t0 = seq_start[s], t1 = seq_start[s + 1];
    const size_t head_floats = (size_t)dim * vdim;
    float* st = state + (size_t)seq_slot[s] * state_stride + (size_t)h * head_floats;
    float* rs = PASS == kLinWhole ? nullptr : run_state + ((size_t)blockIdx.x * heads + h) * head_floats;
    bool last_run = true;
    if (PASS != kLinWhole) {
        const int runs = (t1 - t0 + run_rows - 1) / run_rows;
        last_run = run == runs - 1;
        if (run >= runs) return;                                           // the whole block leaves together
        if (PASS == kLinLocal && last_run) {                               // the second pass reads the state from here
            for (int e = threadIdx.x; e < dim * cw; e += blockDim.x) {
                const size_t at = (size_t)(e / cw) * vdim + c0 + e % cw;
                rs[at] = st[at];
            }
            return;
        }
        t0 += run * run_rows;
        t1 = min(t1, t0 + run_rows);
    }
    if (t1 <= t0) return;
    const int dimP = (dim + 7) & ~7, colsP = (cols + 3) & ~3, kd = dimP + 4;
    const int cg = colsP >> 2;
    float* S = sm;                                   // [dimP][colsP]
    float* sq = S + (size_t)dimP * colsP;            // [kChunk][kd]
    float* sk = sq + (size_t)kChunk * kd;            // [kChunk][kd]
    float* sv = sk + (size_t)kChunk * kd;            // [kChunk][colsP]
    float* sa = sv + (size_t)kChunk * colsP;         // [kChunk][kAPitch]
    float* pw = sa + (size_t)kChunk * kAPitch;       // decay^0 .. decay^kChunk, then room up to kChunk + 4
    float* rowf = pw + kChunk + 4;                   // [kChunk] the local pass's factor of each row of the chunk
    __nv_bfloat16* raw = reinterpret_cast<__nv_bfloat16*>(rowf + kChunk);   // staged: q, k [kChunk][dim], v [kChunk][cols]
    const float dk = decay[h];
    if (threadIdx.x <= kChunk) pw[threadIdx.x] = powf(dk, (float)threadIdx.x);
    if (PASS == kLinFrom) {
        // the run's start: the sequence's state and the runs before this one, in order
        const float dr = powf(dk, (float)run_rows);
        const float* s0 = run_state + (((size_t)s * max_runs + (size_t)((seq_start[s + 1] - seq_start[s] + run_rows - 1) / run_rows - 1)) * heads + h) * head_floats;
        const float* first = run_state + ((size_t)s * max_runs * heads + h) * head_floats;
        const size_t pitch = (size_t)heads * head_floats;
        if (((vdim | cw | c0) & 3) == 0 && ((uintptr_t)run_state & 15) == 0) {
            // four neighbouring columns a thread: every earlier run's part is read 16 bytes at a time, four runs in flight
            for (int e = threadIdx.x; e < dimP * cg; e += blockDim.x) {
                const int d = e / cg, c = (e % cg) << 2;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                if (d < dim && c < cw) {
                    const size_t at = (size_t)d * vdim + c0 + c;
                    acc = ld4(s0 + at);
#pragma unroll 4
                    for (int p = 0; p < run; ++p) {
                        const float4 l = ld4(first + (size_t)p * pitch + at);
                        acc.x = fmaf(dr, acc.x, l.x); acc.y = fmaf(dr, acc.y, l.y);
                        acc.z = fmaf(dr, acc.z, l.z); acc.w = fmaf(dr, acc.w, l.w);
                    }
                }
                st4(S + (size_t)d * colsP + c, acc);
            }
        } else {
            for (int e = threadIdx.x; e < dimP * colsP; e += blockDim.x) {
                const int d = e / colsP, c = e % colsP;
                float acc = 0.f;
                if (d < dim && c < cw) {
                    const size_t at = (size_t)d * vdim + c0 + c;
                    acc = s0[at];
#pragma unroll 4
                    for (int p = 0; p < run; ++p) acc = fmaf(dr, acc, first[(size_t)p * pitch + at]);
                }
                S[e] = acc;
            }
        }
    } else {
        for (int e = threadIdx.x; e < dimP * colsP; e += blockDim.x) {
            const int d = e / colsP, c = e % colsP;
            S[e] = (PASS == kLinWhole && d < dim && c < cw) ? st[(size_t)d * vdim + c0 + c] : 0.f;
        }
    }
    const T* qbase = proj + q_col + h * dim;
    const T* kbase = proj + k_col + h * dim;
    const T* vbase = proj + v_col + h * vdim + c0;
    const int d8 = dim >> 3, c8 = cw >> 3;          // staged: 16-byte pieces of a row's q or k part, of its v part
    __nv_bfloat16* rq = raw;
    __nv_bfloat16* rk = raw + (size_t)kChunk * dim;
    __nv_bfloat16* rv = rk + (size_t)kChunk * dim;
    auto issue = [&](int r0, int n) {
        for (int e = threadIdx.x; e < n * d8; e += blockDim.x) {
            const int i = e / d8, p = (e % d8) << 3;
            const size_t at = (size_t)(r0 + i) * row_stride + p;
            if (PASS != kLinLocal) copy16_async(rq + i * dim + p, qbase + at);
            copy16_async(rk + i * dim + p, kbase + at);
        }
        for (int e = threadIdx.x; e < n * c8; e += blockDim.x) {
            const int i = e / c8, p = (e % c8) << 3;
            copy16_async(rv + i * cols + p, vbase + (size_t)(r0 + i) * row_stride + p);
        }
        copies_commit();
    };
    if (staged) issue(t0, min(kChunk, t1 - t0));
    for (int r0 = t0; r0 < t1; r0 += kChunk) {
        const int n = min(kChunk, t1 - r0);
        if (staged) copies_wait();
        __syncthreads();       // the chunk before is done with q, k, v; this chunk's raw rows have landed for everyone
        if (PASS == kLinLocal && threadIdx.x < kChunk) rowf[threadIdx.x] = powf(dk, (float)max(0, t1 - 1 - r0 - (int)threadIdx.x));
        if (PASS == kLinLocal) __syncthreads();
        if (staged) {
            for (int e = threadIdx.x; e < kChunk * d8; e += blockDim.x) {
                const int i = e / d8, p = (e % d8) << 3;
                float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
                if (PASS != kLinLocal) {
                    if (i < n) silu8(*reinterpret_cast<const uint4*>(rq + i * dim + p), 1.0f, lo, hi);
                    st4(sq + i * kd + p, lo); st4(sq + i * kd + p + 4, hi);
                    lo = make_float4(0.f, 0.f, 0.f, 0.f); hi = lo;
                }
                if (i < n) silu8(*reinterpret_cast<const uint4*>(rk + i * dim + p), 1.0f, lo, hi);
                st4(sk + i * kd + p, lo); st4(sk + i * kd + p + 4, hi);
            }
            for (int e = threadIdx.x; e < kChunk * (colsP >> 3); e += blockDim.x) {
                const int i = e / (colsP >> 3), p = (e % (colsP >> 3)) << 3;
                float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
                if (i < n && p < cw) silu8(*reinterpret_cast<const uint4*>(rv + i * cols + p), PASS == kLinLocal ? rowf[i] : 1.0f, lo, hi);
                st4(sv + i * colsP + p, lo); st4(sv + i * colsP + p + 4, hi);
            }
            __syncthreads();
            if (r0 + kChunk < t1) issue(r0 + kChunk, min(kChunk, t1 - r0 - kChunk));
        } else {
            for (int e = threadIdx.x; e < kChunk * dimP; e += blockDim.x) {
                const int i = e / dimP, d = e % dimP;
                const bool have = i < n && d < dim;
                const size_t at = (size_t)(r0 + i) * row_stride + d;
                if (PASS != kLinLocal) sq[i * kd + d] = have ? silu_float(to_float(qbase[at])) : 0.f;
                sk[i * kd + d] = have ? silu_float(to_float(kbase[at])) : 0.f;
            }
            for (int e = threadIdx.x; e < kChunk * colsP; e += blockDim.x) {
                const int i = e / colsP, c = e % colsP;
                const float f = PASS == kLinLocal ? rowf[i] : 1.0f;
                sv[e] = (i < n && c < cw) ? silu_float(to_float(vbase[(size_t)(r0 + i) * row_stride + c])) * f : 0.f;
            }
            __syncthreads();
        }
        if (PASS != kLinLocal) {
            {   // A: rows 2 ti, 2 ti + 1; columns tj, tj + 16
                const int ti = threadIdx.x >> 4, tj = threadIdx.x & 15;
                const int i0 = 2 * ti, i1 = i0 + 1, j0 = tj, j1 = tj + 16;
                float a00 = 0.f, a01 = 0.f, a10 = 0.f, a11 = 0.f;
                if (j0 <= i1) {
                    const float* q0 = sq + i0 * kd; const float* q1 = sq + i1 * kd;
                    const float* k0 = sk + j0 * kd; const float* k1 = sk + j1 * kd;
                    if (j1 <= i1) {
#pragma unroll 2
                        for (int d = 0; d < dimP; d += 4) {
                            const float4 x0 = ld4(q0 + d), x1 = ld4(q1 + d), y0 = ld4(k0 + d), y1 = ld4(k1 + d);
                            a00 = dot4(x0, y0, a00); a10 = dot4(x1, y0, a10);
                            a01 = dot4(x0, y1, a01); a11 = dot4(x1, y1, a11);
                        }
                    } else {
#pragma unroll 2
                        for (int d = 0; d < dimP; d += 4) {
                            const float4 x0 = ld4(q0 + d), x1 = ld4(q1 + d), y0 = ld4(k0 + d);
                            a00 = dot4(x0, y0, a00); a10 = dot4(x1, y0, a10);
                        }
                    }
                }
                sa[i0 * kAPitch + j0] = j0 <= i0 ? a00 * pw[i0 - j0] : 0.f;
                sa[i1 * kAPitch + j0] = j0 <= i1 ? a10 * pw[i1 - j0] : 0.f;
                sa[i0 * kAPitch + j1] = j1 <= i0 ? a01 * pw[i0 - j1] : 0.f;
                sa[i1 * kAPitch + j1] = j1 <= i1 ? a11 * pw[i1 - j1] : 0.f;
            }
            __syncthreads();
            // o: two rows of four columns a thread
            for (int tile = threadIdx.x; tile < (kChunk / 2) * cg; tile += blockDim.x) {
                const int c = (tile % cg) << 2, i0 = (tile / cg) << 1, i1 = i0 + 1;
                if (i0 >= n) continue;
                const float* q0 = sq + i0 * kd; const float* q1 = sq + i1 * kd;
                float4 o0 = make_float4(0.f, 0.f, 0.f, 0.f), o1 = o0;
#pragma unroll 2
                for (int d = 0; d < dimP; d += 4) {
                    const float4 x0 = ld4(q0 + d), x1 = ld4(q1 + d);
                    const float4 s0 = ld4(S + (size_t)d * colsP + c), s1 = ld4(S + (size_t)(d + 1) * colsP + c);
                    const float4 s2 = ld4(S + (size_t)(d + 2) * colsP + c), s3 = ld4(S + (size_t)(d + 3) * colsP + c);
                    fma4(o0, x0.x, s0); fma4(o0, x0.y, s1); fma4(o0, x0.z, s2); fma4(o0, x0.w, s3);
                    fma4(o1, x1.x, s0); fma4(o1, x1.y, s1); fma4(o1, x1.z, s2); fma4(o1, x1.w, s3);
                }
                scale4(o0, pw[i0 + 1]);
                scale4(o1, pw[i1 + 1]);
                for (int j = 0; j <= i1; j += 4) {   // A is zero beyond the diagonal, v beyond the chunk's rows
                    const float4 a0 = ld4(sa + i0 * kAPitch + j), a1 = ld4(sa + i1 * kAPitch + j);
                    const float4 v0 = ld4(sv + j * colsP + c), v1 = ld4(sv + (j + 1) * colsP + c);
                    const float4 v2 = ld4(sv + (j + 2) * colsP + c), v3 = ld4(sv + (j + 3) * colsP + c);
                    fma4(o0, a0.x, v0); fma4(o0, a0.y, v1); fma4(o0, a0.z, v2); fma4(o0, a0.w, v3);
                    fma4(o1, a1.x, v0); fma4(o1, a1.y, v1); fma4(o1, a1.z, v2); fma4(o1, a1.w, v3);
                }
                float* w0 = out + (size_t)(r0 + i0) * heads * vdim + (size_t)h * vdim + c0 + c;
                const float r0v[4] = {o0.x, o0.y, o0.z, o0.w}, r1v[4] = {o1.x, o1.y, o1.z, o1.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (c + e < cw) {
                        w0[e] = r0v[e];
                        if (i1 < n) w0[(size_t)heads * vdim + e] = r1v[e];
                    }
                }
            }
            if (PASS == kLinFrom && !last_run && r0 + kChunk >= t1) break;     // nobody reads this run's last S
            __syncthreads();                         // every o has read S before it changes
        }
        // S: eight by four entries a thread
        const float pn = PASS == kLinLocal ? 1.0f : pw[n];
        for (int tile = threadIdx.x; tile < (dimP >> 3) * cg; tile += blockDim.x) {
            const int c = (tile % cg) << 2, d = (tile / cg) << 3;
            float* Sd = S + (size_t)d * colsP + c;
            float4 acc[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) { acc[r] = ld4(Sd + r * colsP); if (PASS != kLinLocal) scale4(acc[r], pn); }
#pragma unroll 2
            for (int j = 0; j < n; ++j) {
                const float4 vv = ld4(sv + j * colsP + c);
                float4 ka = ld4(sk + j * kd + d), kb = ld4(sk + j * kd + d + 4);
                if (PASS != kLinLocal) { const float w = pw[n - 1 - j]; scale4(ka, w); scale4(kb, w); }
                fma4(acc[0], ka.x, vv); fma4(acc[1], ka.y, vv); fma4(acc[2], ka.z, vv); fma4(acc[3], ka.w, vv);
                fma4(acc[4], kb.x, vv); fma4(acc[5], kb.y, vv); fma4(acc[6], kb.z, vv); fma4(acc[7], kb.w, vv);
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) st4(Sd + r * colsP, acc[r]);
        }
    }
    __syncthreads();
    float* to = PASS == kLinLocal ? rs : (last_run ? st : nullptr);
    if (to != nullptr)
        for (int e = threadIdx.x; e < dim * cw; e += blockDim.x) to[(size_t)(e / cw) * vdim + c0 + e % cw] = S[(e / cw) * colsP + e % cw];
}

template <typename TG, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* __restrict__ o, const TG* __restrict__ gate, int gate_stride, const TW* __restrict__ w,
                     TO* __restrict__ out, int width, float eps, float scale) {
    chain_release();
    chain_wait();
    __shared__ float scratch[32];
    const size_t t = blockIdx.x;
    const float* row = o + t * width;
    float sq = 0.f;
    for (int e = threadIdx.x; e < width; e += blockDim.x) sq = fmaf(row[e], row[e], sq);
    const float inv = scale / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        const float g = to_float(gate[t * gate_stride + e]);
        out[t * width + e] = from_float<TO>(row[e] * inv * to_float(w[e]) / (1.0f + expf(-g)));
    }
}

static size_t scan_smem(int dim, int cols) { return sizeof(float) * ((size_t)dim * cols + 2 * dim + cols + 256); }
static size_t chunk_smem(int dim, int cols) {
    const size_t dimP = (dim + 7) & ~7, colsP = (cols + 3) & ~3;
    return sizeof(float) * (dimP * colsP + 2 * (size_t)kChunk * (dimP + 4) + (size_t)kChunk * colsP +
                            (size_t)kChunk * kAPitch + kChunk + 4 + kChunk) +
           sizeof(__nv_bfloat16) * (size_t)kChunk * (2 * (size_t)dim + cols);       // the raw rows on their way
}
constexpr size_t kLinSmemMost = 200 * 1024;

}  // namespace mdma

using namespace mdma;

extern "C" {

// How many of a head's columns a block takes: as many as keep its part of S within 48 KB, at most 64.
int mdma_linear_attention_cols(int dim, int vdim) {
    int cols = vdim < 64 ? vdim : 64;
    while (cols > 1 && (size_t)dim * cols > 12288) cols = (cols + 1) / 2;
    return cols;
}

// Whether heads of dim x vdim fit a block's shared memory: row by row (chunked == 0) or a chunk of rows at a time.
int mdma_linear_attention_fits(int dim, int vdim, int chunked) {
    const int cols = mdma_linear_attention_cols(dim, vdim);
    return (chunked ? chunk_smem(dim, cols) : scan_smem(dim, cols)) <= kLinSmemMost ? 1 : 0;
}

// proj rows hold q at q_col + head * dim, k at k_col + head * dim, v at v_col + head * vdim (before their SiLU);
// state [slots][heads * dim * vdim] floats; out [n_tokens][heads * vdim] floats.  chunked == 0: row by row.
// chunked == 2 (kLinSingleRows): the kernel for steps of one row a sequence (row by row where the state's layout does
// not allow its 16-byte accesses).  chunked == 1: a chunk of rows at a time, and with run_rows > 0 in runs of that many rows side by side
// (`max_runs`: the most runs of a sequence; `scratch`: n_seqs * max_runs * heads * dim * vdim floats).
int mdma_linear_attention(const void* proj, int dtype, int row_stride, int q_col, int k_col, int v_col, const float* decay,
                          const int* seq_start, const int* seq_slot, float* state, long state_stride, float* out,
                          int n_seqs, int heads, int dim, int vdim, int chunked, int run_rows, int max_runs,
                          float* scratch, long scratch_floats, cudaStream_t stream) {
    MDMA_REQUIRE(n_seqs >= 0 && heads > 0 && dim > 0 && vdim > 0, "linear_attention: bad sizes");
    MDMA_REQUIRE(n_seqs <= 65535 * 32 && heads <= 65535, "linear_attention: too many sequences or heads");
    if (n_seqs == 0) return 0;
    if (chunked == kLinSingleRows) {
        // four neighbouring floats of a state row at a time: every head's part and every slot's row start on 16 bytes
        const bool fits = vdim % 4 == 0 && state_stride % 4 == 0 && ((uintptr_t)state & 15) == 0 && dim <= 4096;
        if (fits) {
            const size_t step_smem = (size_t)(2 * dim + kStepCols + kStepGroups * kStepCols) * sizeof(float);
            dim3 step_grid(n_seqs, heads, (vdim + kStepCols - 1) / kStepCols);
            MDMA_DISPATCH_DTYPE(dtype, T, {
                launch_chained(linear_attention_step_kernel<T>, step_grid, dim3(256), step_smem, stream, (const T*)proj, row_stride,
                               q_col, k_col, v_col, decay, seq_start, seq_slot, state, (size_t)state_stride, out, heads, dim, vdim);
            });
            MDMA_LAUNCH_OK("linear_attention (single rows)");
            return 0;
        }
        chunked = 0;
    }
    const int cols = mdma_linear_attention_cols(dim, vdim);
    const size_t smem = chunked ? chunk_smem(dim, cols) : scan_smem(dim, cols);
    MDMA_REQUIRE(smem <= kLinSmemMost, "linear_attention: heads of %d x %d do not fit a block's shared memory", dim, vdim);
    dim3 grid(n_seqs, heads, (vdim + cols - 1) / cols);
    if (!chunked) {
        MDMA_DISPATCH_DTYPE(dtype, T, {
            static bool raised = false;
            if (!raised) { cudaFuncSetAttribute(linear_attention_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLinSmemMost); raised = true; }
            launch_chained(linear_attention_scan_kernel<T>, grid, dim3(256), smem, stream, (const T*)proj, row_stride, q_col,
                           k_col, v_col, decay, seq_start, seq_slot, state, (size_t)state_stride, out, heads, dim, vdim, cols);
        });
        MDMA_LAUNCH_OK("linear_attention (row by row)");
        return 0;
    }
    const size_t head_floats = (size_t)dim * vdim;
    if (run_rows > 0) {
        const long slots = (long)n_seqs * max_runs;
        MDMA_REQUIRE(max_runs >= 1 && n_seqs <= 65535 && slots <= 65535l * 32 && scratch != nullptr && scratch_floats >= slots * (long)(heads * head_floats),
                     "linear_attention: %ld runs need %ld floats of scratch, %ld given", slots, slots * (long)(heads * head_floats), scratch_floats);
        grid.x = (unsigned)slots;
    } else {
        run_rows = 0; max_runs = 1;
    }
    const int staged = dtype == ::mdma::kBF16 && dim % 8 == 0 && vdim % 8 == 0 && cols % 8 == 0 && q_col % 8 == 0 &&
                       k_col % 8 == 0 && v_col % 8 == 0 && row_stride % 8 == 0 && ((uintptr_t)proj & 15) == 0;
#define MDMA_LA_CHUNK(PASS_, what)                                                                                        \
    MDMA_DISPATCH_DTYPE(dtype, T, {                                                                                       \
        static bool raised = false;                                                                                       \
        if (!raised) { cudaFuncSetAttribute(linear_attention_chunk_kernel<T, PASS_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLinSmemMost); raised = true; } \
        launch_chained(linear_attention_chunk_kernel<T, PASS_>, grid, dim3(256), smem, stream, (const T*)proj, row_stride, \
                       q_col, k_col, v_col, decay, seq_start, seq_slot, state, (size_t)state_stride, out, heads, dim, vdim, \
                       cols, run_rows, max_runs, scratch, staged);                                                        \
    });                                                                                                                   \
    MDMA_LAUNCH_OK(what)
    if (run_rows > 0) {
        MDMA_LA_CHUNK(kLinLocal, "linear_attention (runs from zero)");
        MDMA_LA_CHUNK(kLinFrom, "linear_attention (runs from their starts)");
        return 0;
    }
    MDMA_LA_CHUNK(kLinWhole, "linear_attention (chunks)");
#undef MDMA_LA_CHUNK
    return 0;
}

int mdma_gated_rmsnorm(const float* o, const void* gate, int g_dtype, int gate_stride, const void* w, int w_dtype, void* out,
                       int out_dtype, int n_rows, int width, float eps, float scale, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0, "gated_rmsnorm: bad sizes");
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_DTYPE(g_dtype, TG, MDMA_DISPATCH_DTYPE(w_dtype, TW, MDMA_DISPATCH_DTYPE(out_dtype, TO,
        launch_chained(gated_rmsnorm_kernel<TG, TW, TO>, dim3(n_rows), dim3(256), 0, stream, o, (const TG*)gate, gate_stride,
                       (const TW*)w, (TO*)out, width, eps, scale))));
    MDMA_LAUNCH_OK("gated_rmsnorm");
    return 0;
}

}  // extern "C"
