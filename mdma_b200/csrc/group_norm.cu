// RMS norm in groups, and the weighted sum over the depth of the model.
//
// group_rmsnorm: a row of `width` floats is split into `groups` equal consecutive parts; every part is divided by
// its own sqrt(mean(part^2) + eps) and the whole row is multiplied by w.  Rows may be gathered by index.  Written
// in the compute dtype.  group_rmsnorm_add is the same norm on a sublayer's result y, added into the residual stream:
// x += norm(y); partial sums that a K-split product left of y are added up first.  All sums are float, in one fixed
// order: every warp sums a slice of a part, the slices of a part are added in slice order.
//
// depth_mix: the model keeps the result of every layer so far; after run i the stream that goes on is
// x <- w[0] x0 + sum_{j=1..i+1} w[j] X_j, x0 the embedding's rows and X_j the result of run j-1 (X_(i+1) is x as the
// run left it, stored first).  Float throughout, terms added in the order of j.
#include "common.cuh"

namespace mdma {

constexpr int kGroupNormMaxWarps = 16;

// Blocks of groups * slices warps (or fewer warps that walk the groups when there are more than 16 groups).
template <typename TW, typename TO, bool ADD>
__global__ void __launch_bounds__(kGroupNormMaxWarps * 32)
group_rmsnorm_kernel(const float* src, float* y_complete, const float* __restrict__ partial,
                     int splits, size_t split_stride, const int* __restrict__ rows, const TW* __restrict__ w,
                     TO* __restrict__ out, float* __restrict__ x_add, int width, int groups, int slices, float eps) {
    chain_release();
    chain_wait();
    __shared__ float sums[kGroupNormMaxWarps];
    const size_t t = blockIdx.x;
    const size_t r = rows ? (size_t)rows[t] : t;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const int part = width / groups;
    const int per_slice = (part + slices - 1) / slices;
    const float* xr = src + r * width;
    for (int g0 = 0; g0 < groups; g0 += n_warps / slices) {
        const int g = g0 + warp / slices, s = warp % slices;
        const int lo = g * part + s * per_slice, hi = min(g * part + part, lo + per_slice);
        float sq = 0.f;
        // four numbers a lane at a time where the slice allows 16-byte accesses; a K-split product's partial sums are
        // asked for four splits at a time (independent loads) and added in split order
        const bool vec = (width & 3) == 0 && (lo & 3) == 0 && (hi & 3) == 0;
        if (g < groups && vec) {
            for (int e = lo + lane * 4; e < hi; e += 128) {
                float4 v = *reinterpret_cast<const float4*>(xr + e);
                if (ADD && splits > 0) {
                    const float* pp = partial + r * width + e;
                    int k = 0;
                    for (; k + 4 <= splits; k += 4) {
                        const float4 p0 = *reinterpret_cast<const float4*>(pp + (size_t)k * split_stride);
                        const float4 p1 = *reinterpret_cast<const float4*>(pp + (size_t)(k + 1) * split_stride);
                        const float4 p2 = *reinterpret_cast<const float4*>(pp + (size_t)(k + 2) * split_stride);
                        const float4 p3 = *reinterpret_cast<const float4*>(pp + (size_t)(k + 3) * split_stride);
                        v.x = (((v.x + p0.x) + p1.x) + p2.x) + p3.x;
                        v.y = (((v.y + p0.y) + p1.y) + p2.y) + p3.y;
                        v.z = (((v.z + p0.z) + p1.z) + p2.z) + p3.z;
                        v.w = (((v.w + p0.w) + p1.w) + p2.w) + p3.w;
                    }
                    for (; k < splits; ++k) {
                        const float4 p0 = *reinterpret_cast<const float4*>(pp + (size_t)k * split_stride);
                        v.x += p0.x; v.y += p0.y; v.z += p0.z; v.w += p0.w;
                    }
                    *reinterpret_cast<float4*>(y_complete + r * width + e) = v;
                }
                sq = fmaf(v.x, v.x, sq); sq = fmaf(v.y, v.y, sq); sq = fmaf(v.z, v.z, sq); sq = fmaf(v.w, v.w, sq);
            }
        } else if (g < groups) {
            for (int e = lo + lane; e < hi; e += 32) {
                float v = xr[e];
                if (ADD) {
                    for (int k = 0; k < splits; ++k) v += partial[(size_t)k * split_stride + r * width + e];
                    if (splits > 0) y_complete[r * width + e] = v;
                }
                sq = fmaf(v, v, sq);
            }
        }
        sq = warp_sum(sq);
        __syncthreads();
        if (lane == 0) sums[warp] = sq;
        __syncthreads();
        if (g < groups) {
            float total = 0.f;
            for (int k = 0; k < slices; ++k) total += sums[(warp / slices) * slices + k];
            const float inv = 1.0f / sqrtf(total / (float)part + eps);
            for (int e = lo + lane; e < hi; e += 32) {
                const float v = (ADD && splits > 0) ? y_complete[r * width + e] : xr[e];
                if (ADD) x_add[r * width + e] += v * inv * to_float(w[e]);
                else out[t * width + e] = from_float<TO>(v * inv * to_float(w[e]));
            }
        }
    }
}

template <typename TW>
__global__ void __launch_bounds__(256)
depth_mix_kernel(float* __restrict__ x, const float* __restrict__ x0, float* __restrict__ history, int depth, int run,
                 const TW* __restrict__ w, int width) {
    chain_release();
    chain_wait();
    const size_t t = blockIdx.x;
    float* hist = history + t * (size_t)depth * width;
    if ((width & 3) == 0) {
        // four numbers a thread; the earlier results are asked for four at a time, added in the order of j
        const int e = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
        if (e >= width) return;
        const float4 mine = *reinterpret_cast<const float4*>(x + t * width + e);
        *reinterpret_cast<float4*>(hist + (size_t)run * width + e) = mine;
        const float4 first = *reinterpret_cast<const float4*>(x0 + t * width + e);
        const float w0 = to_float(w[0]);
        float4 acc = make_float4(w0 * first.x, w0 * first.y, w0 * first.z, w0 * first.w);
        int j = 0;
        for (; j + 4 <= run; j += 4) {
            float4 h[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) h[i] = *reinterpret_cast<const float4*>(hist + (size_t)(j + i) * width + e);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float wj = to_float(w[j + i + 1]);
                acc.x = fmaf(wj, h[i].x, acc.x); acc.y = fmaf(wj, h[i].y, acc.y);
                acc.z = fmaf(wj, h[i].z, acc.z); acc.w = fmaf(wj, h[i].w, acc.w);
            }
        }
        for (; j < run; ++j) {
            const float4 h = *reinterpret_cast<const float4*>(hist + (size_t)j * width + e);
            const float wj = to_float(w[j + 1]);
            acc.x = fmaf(wj, h.x, acc.x); acc.y = fmaf(wj, h.y, acc.y); acc.z = fmaf(wj, h.z, acc.z); acc.w = fmaf(wj, h.w, acc.w);
        }
        const float wl = to_float(w[run + 1]);
        acc.x = fmaf(wl, mine.x, acc.x); acc.y = fmaf(wl, mine.y, acc.y); acc.z = fmaf(wl, mine.z, acc.z); acc.w = fmaf(wl, mine.w, acc.w);
        *reinterpret_cast<float4*>(x + t * width + e) = acc;
        return;
    }
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < width; e += gridDim.y * blockDim.x) {
        const float mine = x[t * width + e];
        hist[(size_t)run * width + e] = mine;
        float acc = to_float(w[0]) * x0[t * width + e];
        for (int j = 0; j < run; ++j) acc = fmaf(to_float(w[j + 1]), hist[(size_t)j * width + e], acc);
        x[t * width + e] = fmaf(to_float(w[run + 1]), mine, acc);
    }
}

static inline void group_norm_shape(int width, int groups, int* slices, int* warps) {
    const int part = width / groups;
    int s = 1;
    if (groups <= kGroupNormMaxWarps) {
        s = kGroupNormMaxWarps / groups;
        while (s > 1 && part / s < 128) s >>= 1;      // a slice of fewer than 128 numbers is not worth a warp
        int p2 = 1;
        while (p2 * 2 <= s) p2 *= 2;
        s = p2;
    }
    *slices = s;
    *warps = groups <= kGroupNormMaxWarps ? groups * s : kGroupNormMaxWarps;
}

}  // namespace mdma

using namespace mdma;

extern "C" {

int mdma_group_rmsnorm(const float* x, const void* w, int w_dtype, const int* rows, void* out, int out_dtype, int n_rows,
                       int width, int groups, float eps, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0 && groups > 0 && width % groups == 0, "group_rmsnorm: %d numbers do not split into %d parts", width, groups);
    if (n_rows == 0) return 0;
    int slices, warps;
    group_norm_shape(width, groups, &slices, &warps);
    MDMA_DISPATCH_DTYPE(w_dtype, TW, MDMA_DISPATCH_DTYPE(out_dtype, TO,
        launch_chained(group_rmsnorm_kernel<TW, TO, false>, dim3(n_rows), dim3(warps * 32), 0, stream, x, (float*)nullptr,
                       (const float*)nullptr, 0, (size_t)0, rows, (const TW*)w, (TO*)out, (float*)nullptr, width, groups,
                       slices, eps)));
    MDMA_LAUNCH_OK("group_rmsnorm");
    return 0;
}

int mdma_group_rmsnorm_add(float* x, float* y, const float* partial, int splits, long split_stride, const void* w,
                           int w_dtype, int n_rows, int width, int groups, float eps, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0 && groups > 0 && width % groups == 0, "group_rmsnorm_add: %d numbers do not split into %d parts", width, groups);
    MDMA_REQUIRE(splits >= 0 && (splits == 0 || partial), "group_rmsnorm_add: partial sums need a pointer");
    MDMA_REQUIRE(splits == 0 || (((uintptr_t)partial & 15) == 0 && (split_stride & 3) == 0) || (width & 3) != 0, "group_rmsnorm_add: partial sums must be 16-byte aligned");
    if (n_rows == 0) return 0;
    int slices, warps;
    group_norm_shape(width, groups, &slices, &warps);
    MDMA_DISPATCH_DTYPE(w_dtype, TW,
        launch_chained(group_rmsnorm_kernel<TW, float, true>, dim3(n_rows), dim3(warps * 32), 0, stream, (const float*)y, y,
                       partial, splits, (size_t)split_stride, (const int*)nullptr, (const TW*)w, (float*)nullptr, x, width,
                       groups, slices, eps));
    MDMA_LAUNCH_OK("group_rmsnorm_add");
    return 0;
}

int mdma_depth_mix(float* x, const float* x0, float* history, int depth, int run, const void* w, int w_dtype, int n_rows,
                   int width, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0 && depth > 0 && run >= 0 && run < depth, "depth_mix: run %d of %d", run, depth);
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_DTYPE(w_dtype, TW,
        launch_chained(depth_mix_kernel<TW>, dim3(n_rows, (width & 3) == 0 ? (width / 4 + 255) / 256 : (width + 1023) / 1024),
                       dim3(256), 0, stream, x, x0, history, depth, run, (const TW*)w, width));
    MDMA_LAUNCH_OK("depth_mix");
    return 0;
}

}  // extern "C"
