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
// Runs side by side (`linear_attention_chunk_kernel`, steps of many rows): the rows are walked kChunk at a time.
// Within a chunk  o_i = decay^(i+1) S^T q_i + sum_(j <= i) decay^(i-j) (q_i . k_j) v_j,  and afterwards
// S <- decay^n S + sum_j decay^(n-1-j) k_j v_j^T.  Equal to the walk row by row up to rounding.
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

// ---------------------------------------------------------------- runs side by side
// Block = (sequence, head, part of the columns), 256 threads.  A chunk of kChunk rows: q, k [kChunk][dim + 1] and
// v [kChunk][cols] are staged as floats; A[i][j] = decay^(i-j) (q_i . k_j) for j <= i is computed once (a thread per
// few (i, j)); then a thread owns column c of a few rows i: o_i[c] = decay^(i+1) sum_d q_i[d] S[d][c] + sum_j A[i][j] v_j[c];
// finally S[d][c] = decay^n S[d][c] + sum_j decay^(n-1-j) k_j[d] v_j[c].
constexpr int kChunk = 32;

template <typename T>
__global__ void __launch_bounds__(256)
linear_attention_chunk_kernel(const T* __restrict__ proj, int row_stride, int q_col, int k_col, int v_col,
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
    const int kd = dim + 1;
    float* S = sm;                               // [dim][cols]
    float* sq = S + (size_t)dim * cols;          // [kChunk][dim + 1]
    float* sk = sq + (size_t)kChunk * kd;        // [kChunk][dim + 1]
    float* sv = sk + (size_t)kChunk * kd;        // [kChunk][cols]
    float* sa = sv + (size_t)kChunk * cols;      // [kChunk][kChunk + 1]
    float* pw = sa + (size_t)kChunk * (kChunk + 1);   // decay^0 .. decay^kChunk
    float* st = state + (size_t)seq_slot[s] * state_stride + (size_t)h * dim * vdim;
    for (int e = threadIdx.x; e < dim * cw; e += blockDim.x) S[(e / cw) * cols + e % cw] = st[(size_t)(e / cw) * vdim + c0 + e % cw];
    const float dk = decay[h];
    if (threadIdx.x <= kChunk) pw[threadIdx.x] = powf(dk, (float)threadIdx.x);
    for (int r0 = t0; r0 < t1; r0 += kChunk) {
        const int n = min(kChunk, t1 - r0);
        __syncthreads();
        for (int e = threadIdx.x; e < n * dim; e += blockDim.x) {
            const int i = e / dim, d = e % dim;
            const T* row = proj + (size_t)(r0 + i) * row_stride;
            sq[i * kd + d] = silu_float(to_float(row[q_col + h * dim + d]));
            sk[i * kd + d] = silu_float(to_float(row[k_col + h * dim + d]));
        }
        for (int e = threadIdx.x; e < n * cw; e += blockDim.x) {
            const int i = e / cw, c = e % cw;
            sv[i * cols + c] = silu_float(to_float(proj[(size_t)(r0 + i) * row_stride + v_col + h * vdim + c0 + c]));
        }
        __syncthreads();
        for (int e = threadIdx.x; e < n * n; e += blockDim.x) {
            const int i = e / n, j = e % n;
            float a = 0.f;
            if (j <= i) {
                for (int d = 0; d < dim; ++d) a = fmaf(sq[i * kd + d], sk[j * kd + d], a);
                a *= pw[i - j];
            }
            sa[i * (kChunk + 1) + j] = a;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < n * cw; e += blockDim.x) {
            const int i = e / cw, c = e % cw;
            float carried = 0.f;
            for (int d = 0; d < dim; ++d) carried = fmaf(sq[i * kd + d], S[d * cols + c], carried);
            float o = carried * pw[i + 1];
            for (int j = 0; j <= i; ++j) o = fmaf(sa[i * (kChunk + 1) + j], sv[j * cols + c], o);
            out[(size_t)(r0 + i) * heads * vdim + (size_t)h * vdim + c0 + c] = o;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < dim * cw; e += blockDim.x) {
            const int d = e / cw, c = e % cw;
            float v = S[d * cols + c] * pw[n];
            for (int j = 0; j < n; ++j) v = fmaf(pw[n - 1 - j] * sk[j * kd + d], sv[j * cols + c], v);
            S[d * cols + c] = v;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < dim * cw; e += blockDim.x) st[(size_t)(e / cw) * vdim + c0 + e % cw] = S[(e / cw) * cols + e % cw];
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
    return sizeof(float) * ((size_t)dim * cols + 2 * (size_t)kChunk * (dim + 1) + (size_t)kChunk * cols +
                            (size_t)kChunk * (kChunk + 1) + kChunk + 1);
}

}  // namespace mdma

using namespace mdma;

extern "C" {

// How many of a head's columns a block takes: as many as keep its part of S within 48 KB, at most 64.
int mdma_linear_attention_cols(int dim, int vdim) {
    int cols = vdim < 64 ? vdim : 64;
    while (cols > 1 && (size_t)dim * cols > 12288) cols = (cols + 1) / 2;
    return cols;
}

// proj rows hold q at q_col + head * dim, k at k_col + head * dim, v at v_col + head * vdim (before their SiLU);
// state [slots][heads * dim * vdim] floats; out [n_tokens][heads * vdim] floats.  runs != 0: the side-by-side walk.
int mdma_linear_attention(const void* proj, int dtype, int row_stride, int q_col, int k_col, int v_col, const float* decay,
                          const int* seq_start, const int* seq_slot, float* state, long state_stride, float* out,
                          int n_seqs, int heads, int dim, int vdim, int runs, cudaStream_t stream) {
    MDMA_REQUIRE(n_seqs >= 0 && heads > 0 && dim > 0 && vdim > 0, "linear_attention: bad sizes");
    MDMA_REQUIRE(n_seqs <= 65535 * 32 && heads <= 65535, "linear_attention: too many sequences or heads");
    if (n_seqs == 0) return 0;
    const int cols = mdma_linear_attention_cols(dim, vdim);
    const size_t smem = runs ? chunk_smem(dim, cols) : scan_smem(dim, cols);
    MDMA_REQUIRE(smem <= 200 * 1024, "linear_attention: heads of %d x %d do not fit a block's shared memory", dim, vdim);
    const dim3 grid(n_seqs, heads, (vdim + cols - 1) / cols);
#define MDMA_LA_LAUNCH(KERNEL)                                                                                            \
    do {                                                                                                                  \
        static bool raised = false;                                                                                       \
        if (!raised) { cudaFuncSetAttribute(KERNEL<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); raised = true; } \
        launch_chained(KERNEL<T>, grid, dim3(256), smem, stream, (const T*)proj, row_stride, q_col, k_col, v_col, decay,  \
                       seq_start, seq_slot, state, (size_t)state_stride, out, heads, dim, vdim, cols);                    \
    } while (0)
    MDMA_DISPATCH_DTYPE(dtype, T, {
        if (runs) MDMA_LA_LAUNCH(linear_attention_chunk_kernel);
        else MDMA_LA_LAUNCH(linear_attention_scan_kernel);
    });
#undef MDMA_LA_LAUNCH
    MDMA_LAUNCH_OK("linear_attention");
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
