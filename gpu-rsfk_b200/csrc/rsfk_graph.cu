// Symmetric closure of a K-NN graph in CSR form: row p holds p's own neighbours
// and every q that lists p without being listed by p.
//
// Reference: symmetric_knn_graph_edge_count / _offset / _add_edges
// (src/rsfk.cu:1229-1299), the step its spectral-clustering experiment ran after
// the forest.  There the offsets come from a single-thread loop and the edges of
// a row land in the order their atomics arrive; here the offsets are a parallel
// scan and every row is ordered by neighbour index, so the result is a function
// of the input.  Empty slots (-1) are skipped (the reference indexes with them).
#include "rsfk_common.cuh"
#include "rsfk_context.h"

namespace rsfk {

constexpr int SYM_THREADS = 256;

__device__ __forceinline__ bool row_lists(const int* __restrict__ row, int K, int target, int lane)
{
    bool hit = false;
    for (int e = lane; e < K; e += 32) hit |= (row[e] == target);
    return __any_sync(RSFK_FULL, hit);
}

// degree[p] = valid entries of row p  +  rows q (q != p's neighbours) that list p
__global__ void __launch_bounds__(SYM_THREADS)
k_sym_count(const int* __restrict__ idx, int N, int K, int* __restrict__ degree)
{
    const int lane = threadIdx.x & 31;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long p = warp0; p < N; p += n_warps) {
        const int* row = idx + p * K;
        int own = 0;
        for (int k0 = 0; k0 < K; k0 += 32) {
            const int k = k0 + lane;
            const int q = k < K ? row[k] : -1;
            const bool valid = q >= 0 && q < N;
            own += __popc(__ballot_sync(RSFK_FULL, valid));
            unsigned todo = __ballot_sync(RSFK_FULL, valid && q != (int)p);
            while (todo) {
                const int b = __ffs(todo) - 1;
                todo &= todo - 1;
                const int qq = __shfl_sync(RSFK_FULL, q, b);
                if (!row_lists(idx + (long long)qq * K, K, (int)p, lane) && lane == 0) atomicAdd(&degree[qq], 1);
            }
        }
        if (lane == 0) atomicAdd(&degree[p], own);
    }
}

// Exclusive scan of degree[N] into offsets[N+1] (64-bit), three passes over
// blocks of SCAN_ITEMS entries.
constexpr int SCAN_ITEMS = 4096;

__global__ void __launch_bounds__(SYM_THREADS)
k_scan_block_sums(const int* __restrict__ degree, int N, long long* __restrict__ block_sum)
{
    __shared__ long long sWarp[SYM_THREADS / 32];
    const long long base = (long long)blockIdx.x * SCAN_ITEMS;
    long long s = 0;
    for (int i = threadIdx.x; i < SCAN_ITEMS; i += blockDim.x)
        if (base + i < N) s += degree[base + i];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) s += __shfl_xor_sync(RSFK_FULL, s, o);
    if ((threadIdx.x & 31) == 0) sWarp[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        long long t = 0;
        for (int w = 0; w < SYM_THREADS / 32; ++w) t += sWarp[w];
        block_sum[blockIdx.x] = t;
    }
}

__global__ void k_scan_block_offsets(long long* __restrict__ block_sum, int n_blocks, long long* __restrict__ total)
{
    // one thread: a few thousand blocks at most (N / 4096)
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        long long run = 0;
        for (int b = 0; b < n_blocks; ++b) {
            const long long v = block_sum[b];
            block_sum[b] = run;
            run += v;
        }
        *total = run;
    }
}

__global__ void __launch_bounds__(SYM_THREADS)
k_scan_finish(const int* __restrict__ degree, int N, const long long* __restrict__ block_sum,
              const long long* __restrict__ total, long long* __restrict__ offsets)
{
    __shared__ long long sThread[SYM_THREADS];
    constexpr int PER = SCAN_ITEMS / SYM_THREADS; // consecutive entries per thread
    const long long base = (long long)blockIdx.x * SCAN_ITEMS + (long long)threadIdx.x * PER;
    long long s = 0;
    for (int i = 0; i < PER; ++i)
        if (base + i < N) s += degree[base + i];
    sThread[threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        long long run = block_sum[blockIdx.x];
        for (int t = 0; t < SYM_THREADS; ++t) {
            const long long v = sThread[t];
            sThread[t] = run;
            run += v;
        }
    }
    __syncthreads();
    long long run = sThread[threadIdx.x];
    for (int i = 0; i < PER; ++i)
        if (base + i < N) {
            offsets[base + i] = run;
            run += degree[base + i];
        }
    if (blockIdx.x == 0 && threadIdx.x == 0) offsets[N] = *total;
}

// Row p: its own valid entries first (in list order), then, through a cursor,
// the rows that list p without being listed.  cursor[p] starts at zero.
__global__ void __launch_bounds__(SYM_THREADS)
k_sym_fill(const int* __restrict__ idx, const float* __restrict__ dist, int N, int K,
           const long long* __restrict__ offsets, int* __restrict__ cursor, int* __restrict__ sym_idx,
           float* __restrict__ sym_dist)
{
    const int lane = threadIdx.x & 31;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long p = warp0; p < N; p += n_warps) {
        const int* row = idx + p * K;
        const float* drow = dist != nullptr ? dist + p * K : nullptr;
        // own entries take the first slots of the row: reserve them in one step
        int own = 0;
        for (int k0 = 0; k0 < K; k0 += 32) {
            const int k = k0 + lane;
            const int q = k < K ? row[k] : -1;
            own += __popc(__ballot_sync(RSFK_FULL, q >= 0 && q < N));
        }
        int first = 0;
        if (lane == 0) first = atomicAdd(&cursor[p], own);
        first = __shfl_sync(RSFK_FULL, first, 0);
        int placed = 0;
        for (int k0 = 0; k0 < K; k0 += 32) {
            const int k = k0 + lane;
            const int q = k < K ? row[k] : -1;
            const float d = (k < K && drow != nullptr) ? drow[k] : 0.0f;
            const bool valid = q >= 0 && q < N;
            const unsigned vmask = __ballot_sync(RSFK_FULL, valid);
            if (valid) {
                const long long at = offsets[p] + first + placed + __popc(vmask & ((1u << lane) - 1u));
                sym_idx[at] = q;
                if (sym_dist != nullptr) sym_dist[at] = d;
            }
            placed += __popc(vmask);
            unsigned todo = __ballot_sync(RSFK_FULL, valid && q != (int)p);
            while (todo) {
                const int b = __ffs(todo) - 1;
                todo &= todo - 1;
                const int qq = __shfl_sync(RSFK_FULL, q, b);
                const float dd = __shfl_sync(RSFK_FULL, d, b);
                if (!row_lists(idx + (long long)qq * K, K, (int)p, lane) && lane == 0) {
                    const long long at = offsets[qq] + atomicAdd(&cursor[qq], 1);
                    sym_idx[at] = (int)p;
                    if (sym_dist != nullptr) sym_dist[at] = dd;
                }
            }
        }
    }
}

// Every row ordered by neighbour index: a bitonic network over the row in global
// memory, one warp per row, comparisons ascending only, so that the positions
// beyond the row's length act as +infinity without being stored.
__global__ void __launch_bounds__(SYM_THREADS)
k_sym_sort(const long long* __restrict__ offsets, int N, int* __restrict__ sym_idx, float* __restrict__ sym_dist)
{
    const int lane = threadIdx.x & 31;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long p = warp0; p < N; p += n_warps) {
        const long long lo = offsets[p];
        const int L = (int)(offsets[p + 1] - lo);
        if (L < 2) continue;
        int* v = sym_idx + lo;
        float* w = sym_dist != nullptr ? sym_dist + lo : nullptr;
        int P = 2;
        while (P < L) P <<= 1;
        for (int k = 2; k <= P; k <<= 1) {
            for (int j = k >> 1; j > 0; j >>= 1) {
                __syncwarp();
                for (int i = lane; i < P; i += 32) {
                    // first step of a stage mirrors inside the block of k, later steps pair at distance j
                    const int l = (j == (k >> 1)) ? (i ^ (k - 1)) : (i ^ j);
                    if (l > i && l < L) {
                        const int a = v[i], b = v[l];
                        if (a > b) {
                            v[i] = b;
                            v[l] = a;
                            if (w != nullptr) {
                                const float t = w[i];
                                w[i] = w[l];
                                w[l] = t;
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
}

static int grid_for_rows(const Context& ctx, long long rows)
{
    long long blocks = (rows * 32 + SYM_THREADS - 1) / SYM_THREADS;
    if (blocks > (long long)ctx.sm_count * 16) blocks = (long long)ctx.sm_count * 16;
    return (int)(blocks < 1 ? 1 : blocks);
}

bool symmetrize_count(Context& ctx, const int* d_idx, int N, int K, long long* d_offsets, long long* nnz_host)
{
    if (N <= 0 || K <= 0) return ctx.fail(RSFK_ERR_ARG, "symmetrize: N and K must be positive");
    cudaStream_t st = ctx.stream;
    const int n_blocks = (N + SCAN_ITEMS - 1) / SCAN_ITEMS;
    int* degree = (int*)ctx.scratch(Context::SYM_DEGREE, sizeof(int) * (size_t)N);
    long long* block_sum = (long long*)ctx.scratch(Context::SYM_BLOCKS, sizeof(long long) * (size_t)(n_blocks + 1));
    if (!degree || !block_sum) return false;
    if (!ctx.check(cudaMemsetAsync(degree, 0, sizeof(int) * (size_t)N, st), "symmetrize memset")) return false;
    k_sym_count<<<grid_for_rows(ctx, N), SYM_THREADS, 0, st>>>(d_idx, N, K, degree);
    k_scan_block_sums<<<n_blocks, SYM_THREADS, 0, st>>>(degree, N, block_sum);
    k_scan_block_offsets<<<1, 32, 0, st>>>(block_sum, n_blocks, block_sum + n_blocks);
    k_scan_finish<<<n_blocks, SYM_THREADS, 0, st>>>(degree, N, block_sum, block_sum + n_blocks, d_offsets);
    count_launches(4);
    if (!ctx.check(cudaGetLastError(), "symmetrize launch")) return false;
    if (nnz_host != nullptr) {
        if (!ctx.check(cudaMemcpyAsync(nnz_host, block_sum + n_blocks, sizeof(long long), cudaMemcpyDeviceToHost, st),
                       "symmetrize D2H") ||
            !ctx.check(cudaStreamSynchronize(st), "symmetrize"))
            return false;
    }
    return true;
}

bool symmetrize_fill(Context& ctx, const int* d_idx, const float* d_dist, int N, int K, const long long* d_offsets,
                     int* d_sym_idx, float* d_sym_dist)
{
    if (N <= 0 || K <= 0) return ctx.fail(RSFK_ERR_ARG, "symmetrize: N and K must be positive");
    if (d_sym_dist != nullptr && d_dist == nullptr)
        return ctx.fail(RSFK_ERR_ARG, "symmetrize: distances asked for but none given");
    cudaStream_t st = ctx.stream;
    int* cursor = (int*)ctx.scratch(Context::SYM_DEGREE, sizeof(int) * (size_t)N);
    if (!cursor) return false;
    if (!ctx.check(cudaMemsetAsync(cursor, 0, sizeof(int) * (size_t)N, st), "symmetrize memset")) return false;
    k_sym_fill<<<grid_for_rows(ctx, N), SYM_THREADS, 0, st>>>(d_idx, d_dist, N, K, d_offsets, cursor, d_sym_idx,
                                                             d_sym_dist);
    k_sym_sort<<<grid_for_rows(ctx, N), SYM_THREADS, 0, st>>>(d_offsets, N, d_sym_idx, d_sym_dist);
    count_launches(2);
    return ctx.check(cudaGetLastError(), "symmetrize launch");
}

} // namespace rsfk
