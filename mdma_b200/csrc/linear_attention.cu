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
// walks every run but the last from S = 0 and leaves the run's last S in scratch; linear_attention_starts_kernel
// turns those, in order, into every run's starting S (start[r+1] = decay^run_rows start[r] + local[r]); pass
// kLinFrom walks every run from its start and writes o, the last run also the sequence's state.
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

// ---------------------------------------------------------------- a chunk of rows at a time
// Block = (sequence or run, head, part of the columns), 256 threads.  Shared memory, all floats, every row a
// multiple of four long so that threads read four neighbours at once: S [dimP][colsP]; q, k [kChunk][dimP + 4];
// v [kChunk][colsP]; A [kChunk][kChunk + 4]; decay^0 .. decay^kChunk.  Rows and columns beyond the data are zero.
//   A[i][j] = decay^(i-j) (q_i . k_j), j <= i: a thread owns two rows and two columns.
//   o_i[c]  = decay^(i+1) sum_d q_i[d] S[d][c] + sum_j A[i][j] v_j[c]: a thread owns two rows of four columns.
//   S[d][c] = decay^n S[d][c] + sum_j decay^(n-1-j) k_j[d] v_j[c]: a thread owns four by four entries.
constexpr int kChunk = 32;
constexpr int kAPitch = kChunk + 4;
enum LinPass : int { kLinWhole = 0, kLinLocal = 1, kLinFrom = 2 };

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void fma4(float4& acc, float a, const float4& b) {
    acc.x = fmaf(a, b.x, acc.x); acc.y = fmaf(a, b.y, acc.y); acc.z = fmaf(a, b.z, acc.z); acc.w = fmaf(a, b.w, acc.w);
}
__device__ __forceinline__ float dot4(const float4& a, const float4& b, float acc) {
    return fmaf(a.w, b.w, fmaf(a.z, b.z, fmaf(a.y, b.y, fmaf(a.x, b.x, acc))));
}

template <typename T, int PASS>
__global__ void __launch_bounds__(256)
linear_attention_chunk_kernel(const T* __restrict__ proj, int row_stride, int q_col, int k_col, int v_col,
                              const float* __restrict__ decay, const int* __restrict__ seq_start,
                              const int* __restrict__ seq_slot, float* __restrict__ state, size_t state_stride,
                              float* __restrict__ out, int heads, int dim, int vdim, int cols, int run_rows, int max_runs,
                              float* __restrict__ run_state) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float sm[];
    const int s = PASS == kLinWhole ? blockIdx.x : blockIdx.x / max_runs;
    const int run = PASS == kLinWhole ? 0 : blockIdx.x % max_runs;
    const int h = blockIdx.y;
    const int c0 = blockIdx.z * cols, cw = min(cols, vdim - c0);
    int t0 = seq_start[s], t1 = seq_start[s + 1];
    bool last_run = true;
    if (PASS != kLinWhole) {
        const int runs = (t1 - t0 + run_rows - 1) / run_rows;
        last_run = run == runs - 1;
        if (run >= runs || (PASS == kLinLocal && last_run)) return;        // the whole block leaves together
        t0 += run * run_rows;
        t1 = min(t1, t0 + run_rows);
    }
    if (t1 <= t0) return;
    const int dimP = (dim + 3) & ~3, colsP = (cols + 3) & ~3, kd = dimP + 4;
    const int cg = colsP >> 2, dg = dimP >> 2;
    float* S = sm;                                   // [dimP][colsP]
    float* sq = S + (size_t)dimP * colsP;            // [kChunk][kd]
    float* sk = sq + (size_t)kChunk * kd;            // [kChunk][kd]
    float* sv = sk + (size_t)kChunk * kd;            // [kChunk][colsP]
    float* sa = sv + (size_t)kChunk * colsP;         // [kChunk][kAPitch]
    float* pw = sa + (size_t)kChunk * kAPitch;       // decay^0 .. decay^kChunk
    const size_t head_floats = (size_t)dim * vdim;
    float* st = state + (size_t)seq_slot[s] * state_stride + (size_t)h * head_floats;
    float* rs = PASS == kLinWhole ? nullptr : run_state + ((size_t)blockIdx.x * heads + h) * head_floats;
    const float* from = PASS == kLinWhole ? st : rs;
    for (int e = threadIdx.x; e < dimP * colsP; e += blockDim.x) {
        const int d = e / colsP, c = e % colsP;
        S[e] = (PASS != kLinLocal && d < dim && c < cw) ? from[(size_t)d * vdim + c0 + c] : 0.f;
    }
    const float dk = decay[h];
    if (threadIdx.x <= kChunk) pw[threadIdx.x] = powf(dk, (float)threadIdx.x);
    const T* qbase = proj + q_col + h * dim;
    const T* kbase = proj + k_col + h * dim;
    const T* vbase = proj + v_col + h * vdim + c0;
    for (int r0 = t0; r0 < t1; r0 += kChunk) {
        const int n = min(kChunk, t1 - r0);
        __syncthreads();                             // the chunk before is done with q, k, v (and S, pw are written)
        for (int e = threadIdx.x; e < kChunk * dimP; e += blockDim.x) {
            const int i = e / dimP, d = e % dimP;
            const bool have = i < n && d < dim;
            const size_t at = (size_t)(r0 + i) * row_stride + d;
            if (PASS != kLinLocal) sq[i * kd + d] = have ? silu_float(to_float(qbase[at])) : 0.f;
            sk[i * kd + d] = have ? silu_float(to_float(kbase[at])) : 0.f;
        }
        for (int e = threadIdx.x; e < kChunk * colsP; e += blockDim.x) {
            const int i = e / colsP, c = e % colsP;
            sv[e] = (i < n && c < cw) ? silu_float(to_float(vbase[(size_t)(r0 + i) * row_stride + c])) : 0.f;
        }
        __syncthreads();
        if (PASS != kLinLocal) {
            {   // A: rows 2 ti, 2 ti + 1; columns tj, tj + 16
                const int ti = threadIdx.x >> 4, tj = threadIdx.x & 15;
                const int i0 = 2 * ti, i1 = i0 + 1, j0 = tj, j1 = tj + 16;
                float a00 = 0.f, a01 = 0.f, a10 = 0.f, a11 = 0.f;
                if (j0 <= i1) {
                    const float* q0 = sq + i0 * kd; const float* q1 = sq + i1 * kd;
                    const float* k0 = sk + j0 * kd; const float* k1 = sk + j1 * kd;
                    const bool second = j1 <= i1;
                    for (int d = 0; d < dimP; d += 4) {
                        const float4 x0 = ld4(q0 + d), x1 = ld4(q1 + d), y0 = ld4(k0 + d);
                        a00 = dot4(x0, y0, a00); a10 = dot4(x1, y0, a10);
                        if (second) {
                            const float4 y1 = ld4(k1 + d);
                            a01 = dot4(x0, y1, a01); a11 = dot4(x1, y1, a11);
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
                for (int d = 0; d < dimP; d += 4) {
                    const float4 x0 = ld4(q0 + d), x1 = ld4(q1 + d);
                    const float4 s0 = ld4(S + (size_t)d * colsP + c), s1 = ld4(S + (size_t)(d + 1) * colsP + c);
                    const float4 s2 = ld4(S + (size_t)(d + 2) * colsP + c), s3 = ld4(S + (size_t)(d + 3) * colsP + c);
                    fma4(o0, x0.x, s0); fma4(o0, x0.y, s1); fma4(o0, x0.z, s2); fma4(o0, x0.w, s3);
                    fma4(o1, x1.x, s0); fma4(o1, x1.y, s1); fma4(o1, x1.z, s2); fma4(o1, x1.w, s3);
                }
                const float p0 = pw[i0 + 1], p1 = pw[i1 + 1];
                o0.x *= p0; o0.y *= p0; o0.z *= p0; o0.w *= p0;
                o1.x *= p1; o1.y *= p1; o1.z *= p1; o1.w *= p1;
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
            __syncthreads();                         // every o has read S before it changes
        }
        // S: four by four entries a thread
        const float pn = pw[n];
        for (int tile = threadIdx.x; tile < dg * cg; tile += blockDim.x) {
            const int c = (tile % cg) << 2, d = (tile / cg) << 2;
            float* Sd = S + (size_t)d * colsP + c;
            float4 s0 = ld4(Sd), s1 = ld4(Sd + colsP), s2 = ld4(Sd + 2 * colsP), s3 = ld4(Sd + 3 * colsP);
            s0.x *= pn; s0.y *= pn; s0.z *= pn; s0.w *= pn;  s1.x *= pn; s1.y *= pn; s1.z *= pn; s1.w *= pn;
            s2.x *= pn; s2.y *= pn; s2.z *= pn; s2.w *= pn;  s3.x *= pn; s3.y *= pn; s3.z *= pn; s3.w *= pn;
            for (int j = 0; j < n; ++j) {
                const float w = pw[n - 1 - j];
                const float4 kk = ld4(sk + j * kd + d), vv = ld4(sv + j * colsP + c);
                fma4(s0, w * kk.x, vv); fma4(s1, w * kk.y, vv); fma4(s2, w * kk.z, vv); fma4(s3, w * kk.w, vv);
            }
            *reinterpret_cast<float4*>(Sd) = s0;
            *reinterpret_cast<float4*>(Sd + colsP) = s1;
            *reinterpret_cast<float4*>(Sd + 2 * colsP) = s2;
            *reinterpret_cast<float4*>(Sd + 3 * colsP) = s3;
        }
    }
    __syncthreads();
    float* to = PASS == kLinLocal ? rs : (last_run ? st : nullptr);
    if (to != nullptr)
        for (int e = threadIdx.x; e < dim * cw; e += blockDim.x) to[(size_t)(e / cw) * vdim + c0 + e % cw] = S[(e / cw) * colsP + e % cw];
}

// The runs' starting states, in order: start[0] = the sequence's state, start[r+1] = decay^run_rows start[r] + local[r]
// (every run but the last is full).  `run_state` holds local[r] on entry and start[r] on return.  A thread per element.
__global__ void __launch_bounds__(256)
linear_attention_starts_kernel(const float* __restrict__ decay, const int* __restrict__ seq_start,
                               const int* __restrict__ seq_slot, const float* __restrict__ state, size_t state_stride,
                               float* __restrict__ run_state, int heads, size_t head_floats, int run_rows, int max_runs) {
    chain_release();
    chain_wait();
    const size_t state_floats = (size_t)heads * head_floats;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int s = blockIdx.y;
    if (e >= state_floats) return;
    const int runs = (seq_start[s + 1] - seq_start[s] + run_rows - 1) / run_rows;
    const float dr = powf(decay[e / head_floats], (float)run_rows);
    float cur = state[(size_t)seq_slot[s] * state_stride + e];
    for (int r = 0; r < runs; ++r) {
        float* at = run_state + ((size_t)s * max_runs + r) * state_floats + e;
        const float local = r < runs - 1 ? *at : 0.f;
        *at = cur;
        cur = fmaf(dr, cur, local);
    }
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
    const size_t dimP = (dim + 3) & ~3, colsP = (cols + 3) & ~3;
    return sizeof(float) * (dimP * colsP + 2 * (size_t)kChunk * (dimP + 4) + (size_t)kChunk * colsP +
                            (size_t)kChunk * kAPitch + kChunk + 4);
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
// chunked != 0: a chunk of rows at a time, and with run_rows > 0 in runs of that many rows side by side
// (`max_runs`: the most runs of a sequence; `scratch`: n_seqs * max_runs * heads * dim * vdim floats).
int mdma_linear_attention(const void* proj, int dtype, int row_stride, int q_col, int k_col, int v_col, const float* decay,
                          const int* seq_start, const int* seq_slot, float* state, long state_stride, float* out,
                          int n_seqs, int heads, int dim, int vdim, int chunked, int run_rows, int max_runs,
                          float* scratch, long scratch_floats, cudaStream_t stream) {
    MDMA_REQUIRE(n_seqs >= 0 && heads > 0 && dim > 0 && vdim > 0, "linear_attention: bad sizes");
    MDMA_REQUIRE(n_seqs <= 65535 * 32 && heads <= 65535, "linear_attention: too many sequences or heads");
    if (n_seqs == 0) return 0;
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
#define MDMA_LA_CHUNK(PASS_, what)                                                                                        \
    MDMA_DISPATCH_DTYPE(dtype, T, {                                                                                       \
        static bool raised = false;                                                                                       \
        if (!raised) { cudaFuncSetAttribute(linear_attention_chunk_kernel<T, PASS_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLinSmemMost); raised = true; } \
        launch_chained(linear_attention_chunk_kernel<T, PASS_>, grid, dim3(256), smem, stream, (const T*)proj, row_stride, \
                       q_col, k_col, v_col, decay, seq_start, seq_slot, state, (size_t)state_stride, out, heads, dim, vdim, \
                       cols, run_rows, max_runs, scratch);                                                                \
    });                                                                                                                   \
    MDMA_LAUNCH_OK(what)
    if (run_rows > 0) {
        MDMA_LA_CHUNK(kLinLocal, "linear_attention (runs from zero)");
        launch_chained(linear_attention_starts_kernel, dim3((unsigned)((heads * head_floats + 255) / 256), n_seqs), dim3(256), 0,
                       stream, decay, seq_start, seq_slot, (const float*)state, (size_t)state_stride, scratch, heads, head_floats,
                       run_rows, max_runs);
        MDMA_LAUNCH_OK("linear_attention_starts");
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
