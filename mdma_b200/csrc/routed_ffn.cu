// A feed-forward made of many small gated feed-forwards ("experts") of which each token uses a few.
//
// Router (one block per token, float arithmetic):
//     z = R h                              logits over all routed outputs (experts, then identity experts)
//     s = softmax(z), or sigmoid(z) element by element (`scoring` 1)
//     c = s + correction                   choice scores
//     experts form `n_groups` equal groups of neighbours; a group's score is the sum of its `group_top`
//     largest c (1: its largest); only the `keep_groups` best groups stay eligible (the others count as
//     minus infinity)
//     the `top` eligible experts with the largest c are chosen (ties: the lower number)
//     weight_j = s[chosen_j] / (sum of the chosen s + 1e-20), or s[chosen_j] itself (`renormalize` 0)
// and, if the layer has a shared expert with a gate, sg = sigmoid(g . h), one number per token.
//
// Experts: expert e maps h to D_e pair(G_e h, U_e h), pair(g, u) = SiLU(g) * u or another gated form of
// `gated_pair`; the last `n_identity` routed
// outputs have no matrices, their output is h itself.  The matrices of all experts are stacked:
// G and U [experts * ff, width], D [experts * width, ff].
//
// Two ways to compute the chosen experts.  Token by token (steps of few tokens): a block per (token,
// choice) reads its expert's matrices; every output element is one warp's sum in a fixed order.  Expert
// by expert (steps of many tokens): the (token, choice) pairs are counted and sorted by expert on the
// device, and a block computes a tile of pairs x features of ONE expert with the expert's matrix tile
// staged in shared memory once for all its pairs.  No step of either way reads anything on the host.
#include "common.cuh"

namespace mdma {

constexpr int kMaxRouted = 1024, kMaxTop = 32, kMaxGroupTop = 8;

// eight consecutive elements as floats, by 16-byte loads (the address must be 16-byte aligned)
__device__ __forceinline__ void load8(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
}

// A warp's dot product over n elements; `vec`: n is a multiple of 8 and both rows start on 16-byte boundaries, so a lane
// takes eight consecutive elements at a time.  Either way the order of additions is fixed.
template <typename TA, typename TW>
__device__ __forceinline__ float warp_dot(const TA* __restrict__ a, const TW* __restrict__ w, int n, int lane, bool vec = false) {
    float acc = 0.f;
    if (vec) {
        for (int k = lane * 8; k < n; k += 256) {
            float x[8], y[8];
            load8(a + k, x);
            load8(w + k, y);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc = fmaf(x[i], y[i], acc);
        }
    } else {
        for (int k = lane; k < n; k += 32) acc = fmaf(to_float(a[k]), to_float(w[k]), acc);
    }
    return warp_sum(acc);
}

// ---------------------------------------------------------------- router
template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
route_kernel(const TA* __restrict__ h, int h_stride, const TW* __restrict__ router, const TC* __restrict__ correction,
             const TW* __restrict__ shared_gate, int width, int n_routed, int top, int n_groups, int keep_groups,
             int scoring, int group_top, int renormalize,
             int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ shared_scale) {
    chain_release();
    chain_wait();
    __shared__ float z[kMaxRouted];
    __shared__ float c[kMaxRouted];
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const TA* row = h + (size_t)t * h_stride;
    for (int e = warp; e < n_routed; e += n_warps) {
        const float v = warp_dot(row, router + (size_t)e * width, width, lane);
        if (lane == 0) z[e] = v;
    }
    if (shared_gate != nullptr && warp == n_warps - 1) {
        const float v = warp_dot(row, shared_gate, width, lane);
        if (lane == 0) shared_scale[t] = 1.0f / (1.0f + expf(-v));
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    // the rest is a few hundred operations: one thread, one order
    if (scoring == 1) {
        for (int e = 0; e < n_routed; ++e) z[e] = 1.0f / (1.0f + expf(-z[e]));
    } else {
        float m = -INFINITY;
        for (int e = 0; e < n_routed; ++e) m = fmaxf(m, z[e]);
        float sum = 0.f;
        for (int e = 0; e < n_routed; ++e) { z[e] = expf(z[e] - m); sum += z[e]; }
        for (int e = 0; e < n_routed; ++e) z[e] = z[e] / sum;
    }
    for (int e = 0; e < n_routed; ++e) c[e] = z[e] + (correction ? to_float(correction[e]) : 0.f);   // z: s; c: choice score
    if (n_groups > 1 && keep_groups < n_groups) {
        const int per = n_routed / n_groups;
        // the best group not yet kept is looked for keep_groups times (ties: the lower number); a bit per group
        unsigned kept[kMaxRouted / 32];
        for (int g = 0; g < (n_groups + 31) / 32; ++g) kept[g] = 0u;
        for (int k = 0; k < keep_groups; ++k) {
            int best = -1;
            float best_score = -INFINITY;
            for (int g = 0; g < n_groups; ++g) {
                if (kept[g >> 5] >> (g & 31) & 1u) continue;
                float gs = -INFINITY;
                if (group_top <= 1) {
                    for (int e = g * per; e < (g + 1) * per; ++e) gs = fmaxf(gs, c[e]);
                } else {
                    // the group's largest scores, largest first, are added up (a group of fewer members: all of them)
                    float best_of[kMaxGroupTop];
                    const int n_best = min(group_top, per);
                    for (int i = 0; i < n_best; ++i) best_of[i] = -INFINITY;
                    for (int e = g * per; e < (g + 1) * per; ++e) {
                        float v = c[e];
                        for (int i = 0; i < n_best; ++i)
                            if (v > best_of[i]) { const float tmp = best_of[i]; best_of[i] = v; v = tmp; }
                    }
                    gs = 0.f;
                    for (int i = 0; i < n_best; ++i) gs += best_of[i];
                }
                if (best < 0 || gs > best_score) { best = g; best_score = gs; }
            }
            if (best >= 0) kept[best >> 5] |= 1u << (best & 31);
        }
        for (int g = 0; g < n_groups; ++g)
            if (!(kept[g >> 5] >> (g & 31) & 1u))
                for (int e = g * per; e < (g + 1) * per; ++e) c[e] = -INFINITY;
    }
    int pick[kMaxTop];
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        int best = -1;
        float best_score = -INFINITY;
        for (int e = 0; e < n_routed; ++e)
            if (c[e] > best_score) { best = e; best_score = c[e]; }
        pick[k] = best;
        if (best >= 0) { c[best] = -INFINITY; total += z[best]; }
    }
    for (int k = 0; k < top; ++k) {
        chosen[(size_t)t * top + k] = pick[k];
        weights[(size_t)t * top + k] = pick[k] < 0 ? 0.f : renormalize ? z[pick[k]] / (total + 1e-20f) : z[pick[k]];
    }
}

// ---------------------------------------------------------------- token by token
// act[t * top + j, f] = silu(G_e[f] . h_t) * (U_e[f] . h_t), e = chosen[t, j] (nothing for identity experts)
template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
expert_gate_up_kernel(const TA* __restrict__ h, int h_stride, const TW* __restrict__ G, const TW* __restrict__ U,
                      const int* __restrict__ chosen, int n_experts, int top, int width, int ff, TA* __restrict__ act,
                      int pair_act, float act_limit, float act_alpha) {
    chain_release();
    chain_wait();
    extern __shared__ float hs[];
    const int pair = blockIdx.x;
    const int e = chosen[pair];
    if (e < 0 || e >= n_experts) return;
    const int t = pair / top;
    const TA* row = h + (size_t)t * h_stride;
    for (int k = threadIdx.x; k < width; k += blockDim.x) hs[k] = to_float(row[k]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const bool vec = width % 8 == 0 && (((uintptr_t)G | (uintptr_t)U) & 15) == 0;
    for (int f = blockIdx.y * n_warps + warp; f < ff; f += gridDim.y * n_warps) {
        const TW* g = G + ((size_t)e * ff + f) * width;
        const TW* u = U + ((size_t)e * ff + f) * width;
        float ag = 0.f, au = 0.f;
        if (vec) {
            for (int k = lane * 8; k < width; k += 256) {
                float x[8], a[8], b[8];
                load8(hs + k, x);
                load8(g + k, a);
                load8(u + k, b);
#pragma unroll
                for (int i = 0; i < 8; ++i) { ag = fmaf(x[i], a[i], ag); au = fmaf(x[i], b[i], au); }
            }
        } else {
            for (int k = lane; k < width; k += 32) {
                ag = fmaf(hs[k], to_float(g[k]), ag);
                au = fmaf(hs[k], to_float(u[k]), au);
            }
        }
        ag = warp_sum(ag);
        au = warp_sum(au);
        if (lane == 0) act[(size_t)pair * ff + f] = from_float<TA>(gated_pair(ag, au, pair_act, act_limit, act_alpha));
    }
}

// x[t, f] += sum_j w[t, j] * (D_e[f] . act[t * top + j]  or, for an identity expert,  h[t, f])
template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
expert_down_kernel(const TA* __restrict__ act, const TA* __restrict__ h, int h_stride, const TW* __restrict__ D,
                   const int* __restrict__ chosen, const float* __restrict__ weights, int n_experts, int top,
                   int width, int ff, float* __restrict__ x) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const bool vec = ff % 8 == 0 && (((uintptr_t)D | (uintptr_t)act) & 15) == 0;
    for (int f = blockIdx.y * n_warps + warp; f < width; f += gridDim.y * n_warps) {
        float total = 0.f;
        for (int j = 0; j < top; ++j) {
            const int e = chosen[(size_t)t * top + j];
            if (e < 0) continue;
            const float w = weights[(size_t)t * top + j];
            if (e >= n_experts) { total += w * to_float(h[(size_t)t * h_stride + f]); continue; }
            total += w * warp_dot(act + ((size_t)t * top + j) * ff, D + ((size_t)e * width + f) * ff, ff, lane, vec);
        }
        if (lane == 0) x[(size_t)t * width + f] += total;
    }
}

// ---------------------------------------------------------------- expert by expert
// The (token, choice) pairs sorted by expert: first[e] is where expert e's run starts in `order` (first[n_experts]: the
// total; identity experts are not counted), order[] lists the pairs expert after expert and where[] is its inverse.
// Three small kernels: every pair adds one to its expert's counter; one block turns the counters into starts (and
// clears them); every pair takes the next place of its expert's run.  The order inside a run depends on who comes
// first, the results do not: every pair's row is computed on its own.
__global__ void __launch_bounds__(256)
expert_count_kernel(const int* __restrict__ chosen, int n_pairs, int n_experts, int* __restrict__ counters) {
    chain_release();
    chain_wait();
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n_pairs) return;
    const int e = chosen[p];
    if (e >= 0 && e < n_experts) atomicAdd(&counters[e], 1);
}

__global__ void __launch_bounds__(32)
expert_starts_kernel(int n_experts, int* __restrict__ first, int* __restrict__ counters) {
    chain_release();
    chain_wait();
    if (threadIdx.x != 0) return;
    int run = 0;
    for (int e = 0; e < n_experts; ++e) { first[e] = run; run += counters[e]; counters[e] = 0; }
    first[n_experts] = run;
}

__global__ void __launch_bounds__(256)
expert_place_kernel(const int* __restrict__ chosen, int n_pairs, int n_experts, const int* __restrict__ first,
                    int* __restrict__ counters, int* __restrict__ order, int* __restrict__ where) {
    chain_release();
    chain_wait();
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n_pairs) return;
    const int e = chosen[p];
    if (e < 0 || e >= n_experts) return;
    const int at = first[e] + atomicAdd(&counters[e], 1);
    order[at] = p;
    if (where) where[p] = at;
}

// `first` holds 2 * (n_experts + 1) ints: the starts, then the counters
static int sort_pairs(const int* chosen, int n_pairs, int n_experts, int* first, int* order, int* where, cudaStream_t stream) {
    int* counters = first + n_experts + 1;
    if (cudaMemsetAsync(counters, 0, sizeof(int) * (size_t)(n_experts + 1), stream) != cudaSuccess) return fail("experts: memset failed");
    const int blocks = (n_pairs + 255) / 256;
    expert_count_kernel<<<blocks, 256, 0, stream>>>(chosen, n_pairs, n_experts, counters);
    expert_starts_kernel<<<1, 32, 0, stream>>>(n_experts, first, counters);
    expert_place_kernel<<<blocks, 256, 0, stream>>>(chosen, n_pairs, n_experts, first, counters, order, where);
    MDMA_LAUNCH_OK("expert sort");
    return 0;
}

// rows[i] = h[order[i] / top] for the sorted pairs i < first[n_experts]: the experts' inputs, expert after expert,
// as contiguous rows that a matrix product can take
template <typename TA>
__global__ void __launch_bounds__(256)
expert_gather_kernel(const TA* __restrict__ h, int h_stride, const int* __restrict__ first, const int* __restrict__ order,
                     int n_experts, int top, int width, TA* __restrict__ rows) {
    chain_release();
    chain_wait();
    const int i = blockIdx.x;
    if (i >= first[n_experts]) return;
    const TA* src = h + (size_t)(order[i] / top) * h_stride;
    TA* dst = rows + (size_t)i * width;
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < width; e += gridDim.y * blockDim.x) dst[e] = src[e];
}

// Tile sizes of the expert-by-expert products: kPairTile pairs x kFeatTile features per block, K walked kKTile at a time.
constexpr int kPairTile = 32, kFeatTile = 64, kKTile = 16;

// act[pair, f] = silu(G_e h) * (U_e h) for the pairs of expert blockIdx.z, tile blockIdx.y of its pairs
template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
expert_gate_up_sorted_kernel(const TA* __restrict__ h, int h_stride, const TW* __restrict__ G, const TW* __restrict__ U,
                             const int* __restrict__ first, const int* __restrict__ order, int top, int width, int ff,
                             TA* __restrict__ act, int pair_act, float act_limit, float act_alpha) {
    chain_release();
    chain_wait();
    const int e = blockIdx.z;
    const int begin = first[e] + blockIdx.y * kPairTile, end = first[e + 1];
    if (begin >= end) return;
    const int n = min(kPairTile, end - begin);
    const int f0 = blockIdx.x * kFeatTile;
    __shared__ float hs[kKTile][kPairTile + 1];
    __shared__ float gs[kKTile][kFeatTile + 1];
    __shared__ float us[kKTile][kFeatTile + 1];
    __shared__ int pair_of[kPairTile];
    if (threadIdx.x < kPairTile) pair_of[threadIdx.x] = threadIdx.x < n ? order[begin + threadIdx.x] : -1;
    __syncthreads();
    // thread (py, fx): pairs py*2 .. py*2+1, features fx*4 .. fx*4+3   (16 x 16 threads)
    const int py = threadIdx.x / 16, fx = threadIdx.x % 16;
    float ag[2][4] = {}, au[2][4] = {};
    for (int k0 = 0; k0 < width; k0 += kKTile) {
        for (int i = threadIdx.x; i < kKTile * kPairTile; i += 256) {
            const int p = i / kKTile, k = i % kKTile;
            const int pr = pair_of[p];
            hs[k][p] = (pr >= 0 && k0 + k < width) ? to_float(h[(size_t)(pr / top) * h_stride + k0 + k]) : 0.f;
        }
        for (int i = threadIdx.x; i < kKTile * kFeatTile; i += 256) {
            const int f = i / kKTile, k = i % kKTile;
            const bool ok = f0 + f < ff && k0 + k < width;
            const size_t at = ((size_t)e * ff + f0 + f) * width + k0 + k;
            gs[k][f] = ok ? to_float(G[at]) : 0.f;
            us[k][f] = ok ? to_float(U[at]) : 0.f;
        }
        __syncthreads();
        float pg[2][4] = {}, pu[2][4] = {};
#pragma unroll
        for (int k = 0; k < kKTile; ++k) {
            float a[2], g[4], u[4];
#pragma unroll
            for (int i = 0; i < 2; ++i) a[i] = hs[k][py * 2 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) { g[j] = gs[k][fx * 4 + j]; u[j] = us[k][fx * 4 + j]; }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) { pg[i][j] = fmaf(a[i], g[j], pg[i][j]); pu[i][j] = fmaf(a[i], u[j], pu[i][j]); }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) { ag[i][j] += pg[i][j]; au[i][j] += pu[i][j]; }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int pr = pair_of[py * 2 + i];
        if (pr < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int f = f0 + fx * 4 + j;
            if (f < ff) act[(size_t)pr * ff + f] = from_float<TA>(gated_pair(ag[i][j], au[i][j], pair_act, act_limit, act_alpha));
        }
    }
}

// y[pair, f] = D_e[f] . act[pair] for the pairs of expert blockIdx.z (float rows, one per pair)
template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
expert_down_sorted_kernel(const TA* __restrict__ act, const TW* __restrict__ D, const int* __restrict__ first,
                          const int* __restrict__ order, int width, int ff, float* __restrict__ y) {
    chain_release();
    chain_wait();
    const int e = blockIdx.z;
    const int begin = first[e] + blockIdx.y * kPairTile, end = first[e + 1];
    if (begin >= end) return;
    const int n = min(kPairTile, end - begin);
    const int f0 = blockIdx.x * kFeatTile;
    __shared__ float as[kKTile][kPairTile + 1];
    __shared__ float ds[kKTile][kFeatTile + 1];
    __shared__ int pair_of[kPairTile];
    if (threadIdx.x < kPairTile) pair_of[threadIdx.x] = threadIdx.x < n ? order[begin + threadIdx.x] : -1;
    __syncthreads();
    const int py = threadIdx.x / 16, fx = threadIdx.x % 16;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < ff; k0 += kKTile) {
        for (int i = threadIdx.x; i < kKTile * kPairTile; i += 256) {
            const int p = i / kKTile, k = i % kKTile;
            const int pr = pair_of[p];
            as[k][p] = (pr >= 0 && k0 + k < ff) ? to_float(act[(size_t)pr * ff + k0 + k]) : 0.f;
        }
        for (int i = threadIdx.x; i < kKTile * kFeatTile; i += 256) {
            const int f = i / kKTile, k = i % kKTile;
            ds[k][f] = (f0 + f < width && k0 + k < ff) ? to_float(D[((size_t)e * width + f0 + f) * ff + k0 + k]) : 0.f;
        }
        __syncthreads();
        float part[2][4] = {};
#pragma unroll
        for (int k = 0; k < kKTile; ++k) {
            float a[2], d[4];
#pragma unroll
            for (int i = 0; i < 2; ++i) a[i] = as[k][py * 2 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) d[j] = ds[k][fx * 4 + j];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[i][j] = fmaf(a[i], d[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int pr = pair_of[py * 2 + i];
        if (pr < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int f = f0 + fx * 4 + j;
            if (f < width) y[(size_t)pr * width + f] = acc[i][j];
        }
    }
}

// x[t, f] += sum_j w[t, j] * (y[row of pair t * top + j, f]  or, for an identity expert,  h[t, f]), j in order;
// the row of a pair is the pair's number, or where[pair] when y holds the sorted list's rows
template <typename TA>
__global__ void __launch_bounds__(256)
expert_combine_kernel(const float* __restrict__ y, const TA* __restrict__ h, int h_stride, const int* __restrict__ chosen,
                      const float* __restrict__ weights, const int* __restrict__ where, int n_experts, int top, int width,
                      float* __restrict__ x) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    for (int f = blockIdx.y * blockDim.x + threadIdx.x; f < width; f += gridDim.y * blockDim.x) {
        float total = 0.f;
        for (int j = 0; j < top; ++j) {
            const int e = chosen[(size_t)t * top + j];
            if (e < 0) continue;
            const size_t pair = (size_t)t * top + j;
            const float v = e >= n_experts ? to_float(h[(size_t)t * h_stride + f]) : y[(where ? (size_t)where[pair] : pair) * width + f];
            total += weights[(size_t)t * top + j] * v;
        }
        x[(size_t)t * width + f] += total;
    }
}

}  // namespace mdma

using namespace mdma;

#define MDMA_DISPATCH_2(a_code, TA, w_code, TW, ...) \
    MDMA_DISPATCH_DTYPE(a_code, TA, MDMA_DISPATCH_DTYPE(w_code, TW, __VA_ARGS__))

extern "C" {

int mdma_route(const void* h, int h_dtype, int h_stride, const void* router, int w_dtype, const void* correction,
               int c_dtype, const void* shared_gate, int n_tokens, int width, int n_routed, int top, int n_groups,
               int keep_groups, int scoring, int group_top, int renormalize, int* chosen, float* weights,
               float* shared_scale, cudaStream_t stream) {
    MDMA_REQUIRE(scoring >= 0 && scoring <= 1 && group_top >= 1 && group_top <= kMaxGroupTop,
                 "route: scoring %d, a group's score over its %d largest (at most %d)", scoring, group_top, kMaxGroupTop);
    MDMA_REQUIRE(n_tokens >= 0 && width > 0, "route: bad sizes");
    MDMA_REQUIRE(n_routed > 0 && n_routed <= kMaxRouted, "route: %d routed outputs, the kernel takes up to %d", n_routed, kMaxRouted);
    MDMA_REQUIRE(top > 0 && top <= kMaxTop && top <= n_routed, "route: top %d of %d (at most %d)", top, n_routed, kMaxTop);
    MDMA_REQUIRE(n_groups >= 1 && n_routed % n_groups == 0 && keep_groups >= 1 && keep_groups <= n_groups,
                 "route: %d groups (keep %d) over %d outputs", n_groups, keep_groups, n_routed);
    MDMA_REQUIRE(shared_gate == nullptr || shared_scale != nullptr, "route: the shared gate needs a place for its result");
    if (n_tokens == 0) return 0;
    MDMA_DISPATCH_2(h_dtype, TA, w_dtype, TW,
        MDMA_DISPATCH_DTYPE(c_dtype, TC,
            launch_chained(route_kernel<TA, TW, TC>, dim3(n_tokens), dim3(256), 0, stream, (const TA*)h, h_stride,
                           (const TW*)router, (const TC*)correction, (const TW*)shared_gate, width, n_routed, top,
                           n_groups, keep_groups, scoring, group_top, renormalize, chosen, weights, shared_scale)));
    MDMA_LAUNCH_OK("route");
    return 0;
}

// Token by token: act [n_tokens * top, ff] in h's dtype is scratch; x [n_tokens, width] float takes the sum.
int mdma_experts_by_token(const void* h, int h_dtype, int h_stride, const void* G, const void* U, const void* D,
                          int w_dtype, const int* chosen, const float* weights, int n_tokens, int n_experts, int top,
                          int width, int ff, void* act, float* x, int pair_act, float act_limit, float act_alpha,
                          cudaStream_t stream) {
    MDMA_REQUIRE(n_tokens >= 0 && width > 0 && ff > 0 && top > 0 && n_experts >= 0, "experts: bad sizes");
    MDMA_REQUIRE((size_t)width * sizeof(float) <= 160 * 1024, "experts: width %d is beyond the kernel's shared memory", width);
    if (n_tokens == 0) return 0;
    const int fparts = (ff + 7) / 8 > 64 ? 64 : (ff + 7) / 8;
    const int wparts = (width + 7) / 8 > 128 ? 128 : (width + 7) / 8;
    MDMA_DISPATCH_2(h_dtype, TA, w_dtype, TW, {
        if (n_experts > 0) {
            static bool raised = false;
            if (!raised) {
                cudaFuncSetAttribute(expert_gate_up_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
                raised = true;
            }
            launch_chained(expert_gate_up_kernel<TA, TW>, dim3(n_tokens * top, fparts), dim3(256),
                           (size_t)width * sizeof(float), stream, (const TA*)h, h_stride, (const TW*)G, (const TW*)U, chosen,
                           n_experts, top, width, ff, (TA*)act, pair_act, act_limit, act_alpha);
        }
        launch_chained(expert_down_kernel<TA, TW>, dim3(n_tokens, wparts), dim3(256), 0, stream, (const TA*)act, (const TA*)h,
                       h_stride, (const TW*)D, chosen, weights, n_experts, top, width, ff, x);
    });
    MDMA_LAUNCH_OK("experts_by_token");
    return 0;
}

// Expert by expert: first [2 * (n_experts + 1)] and order [n_tokens * top] ints, act [n_tokens * top, ff] in h's dtype and
// y [n_tokens * top, width] floats are scratch.
int mdma_experts_sorted(const void* h, int h_dtype, int h_stride, const void* G, const void* U, const void* D,
                        int w_dtype, const int* chosen, const float* weights, int n_tokens, int n_experts, int top,
                        int width, int ff, int* first, int* order, void* act, float* y, float* x, int pair_act,
                        float act_limit, float act_alpha, cudaStream_t stream) {
    MDMA_REQUIRE(n_tokens >= 0 && width > 0 && ff > 0 && top > 0 && n_experts >= 0 && n_experts <= kMaxRouted, "experts: bad sizes");
    if (n_tokens == 0) return 0;
    const int n_pairs = n_tokens * top;
    const int pair_tiles = (n_pairs + kPairTile - 1) / kPairTile;
    MDMA_REQUIRE(pair_tiles <= 65535 && n_experts <= 65535, "experts: too many pairs (%d)", n_pairs);
    const int wparts = (width + 255) / 256 > 64 ? 64 : (width + 255) / 256;
    MDMA_DISPATCH_2(h_dtype, TA, w_dtype, TW, {
        if (n_experts > 0) {
            if (int rc = sort_pairs(chosen, n_pairs, n_experts, first, order, nullptr, stream)) return rc;
            launch_chained(expert_gate_up_sorted_kernel<TA, TW>, dim3((ff + kFeatTile - 1) / kFeatTile, pair_tiles, n_experts),
                           dim3(256), 0, stream, (const TA*)h, h_stride, (const TW*)G, (const TW*)U, first, order, top, width,
                           ff, (TA*)act, pair_act, act_limit, act_alpha);
            launch_chained(expert_down_sorted_kernel<TA, TW>, dim3((width + kFeatTile - 1) / kFeatTile, pair_tiles, n_experts),
                           dim3(256), 0, stream, (const TA*)act, (const TW*)D, first, order, width, ff, y);
        }
        launch_chained(expert_combine_kernel<TA>, dim3(n_tokens, wparts), dim3(256), 0, stream, y, (const TA*)h, h_stride,
                       chosen, weights, (const int*)nullptr, n_experts, top, width, x);
    });
    MDMA_LAUNCH_OK("experts_sorted");
    return 0;
}

// The two ends of the expert-by-expert way when the products in between are the caller's (one matrix product per
// expert over its run of gathered rows).  Sort and gather: first [n_experts + 1], order and where [n_tokens * top],
// rows [n_tokens * top, width] in h's dtype.
int mdma_experts_gather(const void* h, int h_dtype, int h_stride, const int* chosen, int n_tokens, int n_experts, int top,
                        int width, int* first, int* order, int* where, void* rows, cudaStream_t stream) {
    MDMA_REQUIRE(n_tokens >= 0 && width > 0 && top > 0 && n_experts > 0 && n_experts <= kMaxRouted, "experts: bad sizes");
    if (n_tokens == 0) return 0;
    const int n_pairs = n_tokens * top;
    const int wparts = (width + 255) / 256 > 64 ? 64 : (width + 255) / 256;
    if (int rc = sort_pairs(chosen, n_pairs, n_experts, first, order, where, stream)) return rc;
    MDMA_DISPATCH_DTYPE(h_dtype, TA,
        launch_chained(expert_gather_kernel<TA>, dim3(n_pairs, wparts), dim3(256), 0, stream, (const TA*)h, h_stride,
                       (const int*)first, (const int*)order, n_experts, top, width, (TA*)rows));
    MDMA_LAUNCH_OK("experts_gather");
    return 0;
}

// Combine: y [sorted rows, width] floats hold the experts' results in the sorted list's order.
int mdma_experts_combine(const float* y, const void* h, int h_dtype, int h_stride, const int* chosen, const float* weights,
                         const int* where, int n_tokens, int n_experts, int top, int width, float* x, cudaStream_t stream) {
    MDMA_REQUIRE(n_tokens >= 0 && width > 0 && top > 0, "experts: bad sizes");
    if (n_tokens == 0) return 0;
    const int wparts = (width + 255) / 256 > 64 ? 64 : (width + 255) / 256;
    MDMA_DISPATCH_DTYPE(h_dtype, TA,
        launch_chained(expert_combine_kernel<TA>, dim3(n_tokens, wparts), dim3(256), 0, stream, y, (const TA*)h, h_stride,
                       chosen, weights, where, n_experts, top, width, x));
    MDMA_LAUNCH_OK("experts_combine");
    return 0;
}

}  // extern "C"
