// k-means (Lloyd iterations) for sample-tree clustering, sm_100a.
//
// The reference has no k-means function of its own: the only k-means near its
// path is the one inside nvGRAPH's spectral clustering, called from commented-out
// code (src/rsfk.cu:1521-1567, parameters at :1536-1539 and :1863-1868).  This
// file is therefore a new component with rules of its own, stated once in the CPU
// oracle (orc_kmeans_assign / orc_kmeans_update) and implemented here so that the
// result is a pure function of the input -- no atomics on floating-point sums, no
// dependence on scheduling:
//
//   assign : nearest centroid by squared distance in the reference's summation
//            order (the arithmetic of the query-bucket kernel: centroid rows staged
//            in shared memory, 32 distances per warp step), ties to the lower
//            centroid index;
//   update : points ordered by (label, index) with a stable radix sort, then one
//            CTA per (cluster, 32 dimensions): member j of the cluster goes to warp
//            j mod 8, every warp adds its members in order in double precision,
//            the eight partial sums are added in order; empty clusters keep their
//            centroid.
#include <cub/device/device_radix_sort.cuh>

#include "rsfk_context.h"

namespace rsfk {

constexpr int KM_THREADS = 256;
constexpr int KM_WARPS = KM_THREADS / 32;
constexpr int KM_PPW = 8; // points per warp and CTA pass

// Rows of the centroid tile a CTA stages at a time (a multiple of 32).
static int kmeans_tile_rows(int D)
{
    int groups = 16384 / (D > 0 ? D : 1) / 32;
    if (groups < 1) groups = 1;
    if (groups > 8) groups = 8;
    return 32 * groups;
}

template <bool VEC4>
__global__ void __launch_bounds__(KM_THREADS)
k_kmeans_assign(const float* __restrict__ pts, int N, int D, const float* __restrict__ cent, int C, int tile_rows,
                int* __restrict__ labels, float* __restrict__ sq_dist, int* __restrict__ changed)
{
    extern __shared__ float4 smem4[];
    float* X = reinterpret_cast<float*>(smem4);                 // [tile_rows][D] centroids
    float* xq_all = X + (size_t)tile_rows * D;                  // [KM_WARPS][D]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* xq = xq_all + (size_t)warp * D;
    const int per_cta = KM_WARPS * KM_PPW;
    const int n_blocks = (N + per_cta - 1) / per_cta;
    for (int blk = blockIdx.x; blk < n_blocks; blk += gridDim.x) {
        const int p0 = blk * per_cta + warp * KM_PPW;
        float best_d[KM_PPW];
        int best_c[KM_PPW];
#pragma unroll
        for (int u = 0; u < KM_PPW; ++u) { best_d[u] = CUDART_INF_F; best_c[u] = 0x7fffffff; }
        for (int c0 = 0; c0 < C; c0 += tile_rows) {
            const int rows = min(tile_rows, C - c0);
            __syncthreads();
            for (int e = threadIdx.x; e < rows * D; e += blockDim.x) X[e] = __ldg(cent + (size_t)c0 * D + e);
            __syncthreads();
#pragma unroll
            for (int u = 0; u < KM_PPW; ++u) {
                const int p = p0 + u;
                if (p >= N) break; // warp-uniform
                __syncwarp();
                for (int k = lane; k < D; k += 32) xq[k] = __ldg(pts + (size_t)p * D + k);
                __syncwarp();
                for (int b0 = 0; b0 < rows; b0 += 32) {
                    const int n = min(32, rows - b0);
                    int item;
                    const float d = VEC4 ? leaf_dist32_vec4(X, D, xq, b0, n, lane, item)
                                         : leaf_dist32_scalar(X, D, xq, b0, n, lane, item);
                    const int c = c0 + b0 + item;
                    if (item < n && (d < best_d[u] || (d == best_d[u] && c < best_c[u]))) {
                        best_d[u] = d;
                        best_c[u] = c;
                    }
                }
            }
        }
        int n_changed = 0;
#pragma unroll
        for (int u = 0; u < KM_PPW; ++u) {
            const int p = p0 + u;
            if (p >= N) break;
            float d = best_d[u];
            int c = best_c[u];
#pragma unroll
            for (int s = 16; s >= 1; s >>= 1) {
                const float od = __shfl_xor_sync(RSFK_FULL, d, s);
                const int oc = __shfl_xor_sync(RSFK_FULL, c, s);
                if (od < d || (od == d && oc < c)) { d = od; c = oc; }
            }
            if (lane == 0) {
                if (labels[p] != c) n_changed++;
                labels[p] = c;
                sq_dist[p] = d;
            }
        }
        if (lane == 0 && n_changed) atomicAdd(changed, n_changed);
    }
}

__global__ void k_kmeans_iota(int* __restrict__ a, int n)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) a[i] = i;
}

// start[c] = first position of label c in the sorted labels, start[C] = N.
__global__ void k_kmeans_bounds(const int* __restrict__ sorted, int N, int C, int* __restrict__ start)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < N; i += gridDim.x * blockDim.x) {
        const int k = min(max(sorted[i], 0), C - 1);
        const int kp = i > 0 ? min(max(sorted[i - 1], 0), C - 1) : -1;
        for (int c = kp + 1; c <= k; ++c) start[c] = i;
        if (i == N - 1)
            for (int c = k + 1; c <= C; ++c) start[c] = N;
    }
}

__global__ void __launch_bounds__(KM_THREADS)
k_kmeans_update(const float* __restrict__ pts, int D, const int* __restrict__ order, const int* __restrict__ start,
                float* __restrict__ cent)
{
    __shared__ double part[KM_WARPS][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.x;
    const int d = blockIdx.y * 32 + lane;
    const int s0 = start[c], count = start[c + 1] - s0;
    if (count <= 0) return;
    double acc = 0.0;
    if (d < D)
        for (int j = warp; j < count; j += KM_WARPS) acc += (double)__ldg(pts + (size_t)order[s0 + j] * D + d);
    part[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && d < D) {
        double s = part[0][lane];
#pragma unroll
        for (int w = 1; w < KM_WARPS; ++w) s += part[w][lane];
        cent[(size_t)c * D + d] = (float)(s / (double)count);
    }
}

// Means of the groups given by d_labels into d_centroids (groups without members keep
// their centroid).
static bool kmeans_update(Context& ctx, const float* d_points, int N, int D, int C, const int* d_labels,
                          float* d_centroids)
{
    cudaStream_t st = ctx.stream;
    int* iota = (int*)ctx.scratch(Context::KM_IOTA, sizeof(int) * (size_t)N);
    int* keys = (int*)ctx.scratch(Context::KM_KEYS, sizeof(int) * (size_t)N);
    int* order = (int*)ctx.scratch(Context::KM_ORDER, sizeof(int) * (size_t)N);
    int* start = (int*)ctx.scratch(Context::KM_START, sizeof(int) * (size_t)(C + 1));
    if (!iota || !keys || !order || !start) return false;
    int bits = 1;
    while (bits < 31 && (1 << bits) < C) ++bits;
    size_t temp_bytes = 0;
    if (!ctx.check(cub::DeviceRadixSort::SortPairs(nullptr, temp_bytes, d_labels, keys, iota, order, N, 0, bits, st),
                   "kmeans sort size"))
        return false;
    void* temp = ctx.scratch(Context::KM_TEMP, temp_bytes > 0 ? temp_bytes : 16);
    if (!temp) return false;
    int grid = (N + 255) / 256;
    if (grid > ctx.sm_count * 16) grid = ctx.sm_count * 16;
    k_kmeans_iota<<<grid, 256, 0, st>>>(iota, N);
    if (!ctx.check(cub::DeviceRadixSort::SortPairs(temp, temp_bytes, d_labels, keys, iota, order, N, 0, bits, st),
                   "kmeans sort"))
        return false;
    k_kmeans_bounds<<<grid, 256, 0, st>>>(keys, N, C, start);
    k_kmeans_update<<<dim3(C, (D + 31) / 32), KM_THREADS, 0, st>>>(d_points, D, order, start, d_centroids);
    count_launches(3);
    return ctx.check(cudaGetLastError(), "kmeans update launch");
}

bool kmeans(Context& ctx, const float* d_points, int N, int D, int C, int max_iter, bool init_from_labels,
            float* d_centroids, int* d_labels, float* d_sq_dist, int* iterations)
{
    TraceRange trace("rsfk kmeans");
    if (N <= 0 || D <= 0 || C <= 0 || max_iter < 0) return ctx.fail(RSFK_ERR_ARG, "kmeans: invalid argument");
    if (C > N) return ctx.fail(RSFK_ERR_ARG, "kmeans: more clusters than points");
    cudaStream_t st = ctx.stream;
    const int tile_rows = kmeans_tile_rows(D);
    const size_t smem = sizeof(float) * ((size_t)tile_rows + KM_WARPS) * D;
    if (smem > 200 * 1024) return ctx.fail(RSFK_ERR_UNSUPPORTED, "kmeans: D too large for the centroid tile");
    int* changed = (int*)ctx.scratch(Context::KM_CHANGED, sizeof(int));
    if (!changed) return false;
    const bool vec4 = (D % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_centroids) & 15) == 0);
    auto assign_kernel = vec4 ? k_kmeans_assign<true> : k_kmeans_assign<false>;
    if (smem > 48 * 1024 &&
        !ctx.check(cudaFuncSetAttribute(assign_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                   "kmeans smem attribute"))
        return false;
    const int per_cta = KM_WARPS * KM_PPW;
    long long blocks = ((long long)N + per_cta - 1) / per_cta;
    const int per_sm = smem > 100 * 1024 ? 1 : (smem > 48 * 1024 ? 2 : 4);
    if (blocks > (long long)ctx.sm_count * per_sm) blocks = (long long)ctx.sm_count * per_sm;
    int n_changed = 0;
    auto assign = [&]() -> bool {
        if (!ctx.check(cudaMemsetAsync(changed, 0, sizeof(int), st), "kmeans counter")) return false;
        assign_kernel<<<(int)blocks, KM_THREADS, smem, st>>>(d_points, N, D, d_centroids, C, tile_rows, d_labels,
                                                            d_sq_dist, changed);
        count_launches(1);
        return ctx.check(cudaGetLastError(), "kmeans assign launch") &&
               ctx.check(cudaMemcpyAsync(&n_changed, changed, sizeof(int), cudaMemcpyDeviceToHost, st), "kmeans D2H") &&
               ctx.check(cudaStreamSynchronize(st), "kmeans assign");
    };
    if (init_from_labels) {
        if (!kmeans_update(ctx, d_points, N, D, C, d_labels, d_centroids)) return false;
    } else if (!ctx.check(cudaMemsetAsync(d_labels, 0xff, sizeof(int) * (size_t)N, st), "kmeans labels")) {
        return false;
    }
    if (!assign()) return false;
    int done = 0;
    for (int it = 0; it < max_iter; ++it) {
        done = it + 1;
        if (it > 0 && n_changed == 0) break; // the labels of two assignments in a row agree
        if (!kmeans_update(ctx, d_points, N, D, C, d_labels, d_centroids)) return false;
        if (!assign()) return false;
    }
    if (iterations) *iterations = done;
    return true;
}

} // namespace rsfk
