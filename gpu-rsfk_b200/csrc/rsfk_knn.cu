// K-list kernels for sm_100a: canonical row sort, leaf-bucket all-pairs KNN,
// neighbour-of-neighbour exploration and the G-way list merge used when trees
// are sharded across GPUs.
//
// Every K-list row in device memory is kept canonical: ascending by
// (squared distance, index), distinct indices, unused slots (+inf, -1).  A
// row update is "the K smallest distinct of row + candidates", which equals
// the reference's replace-the-worst-slot rule
// (src/kernels/compute_knn_from_buckets.cu:1205-1285,
//  src/kernels/nearest_neighbors_exploring.cu:83-141) whenever no two
// competing distances tie; ties go to the lower index here.
//
// Squared distances keep the reference's summation order (term i in lane i%32,
// fused multiply-add, xor butterfly), so their bits equal the reference's.
#include <cstdlib>

#include "rsfk_context.h"

namespace rsfk {

constexpr int KNN_THREADS = 256;
constexpr int KNN_WARPS = KNN_THREADS / 32;
constexpr int MAX_KPL = 8; // K <= 256

int list_capacity() { return 32 * MAX_KPL; }

// ---------------------------------------------------------------------------
// sort_rows: one warp per row; entries are inserted in slot order into an
// empty list, so the first occurrence of a repeated index wins.
// ---------------------------------------------------------------------------
template <int KPL>
__global__ void __launch_bounds__(KNN_THREADS)
k_sort_rows(int* __restrict__ idx, float* __restrict__ dist, long long rows, int K)
{
    const int lane = threadIdx.x & 31;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long row = warp0; row < rows; row += n_warps) {
        int* gi = idx + row * K;
        float* gd = dist + row * K;
        float rd[KPL];
        int ri[KPL];
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
            int e = r * 32 + lane;
            rd[r] = e < K ? gd[e] : CUDART_INF_F;
            ri[r] = e < K ? gi[e] : -1;
        }
        WarpList<KPL> L;
        L.clear();
        bool sorted = true; // already canonical? then nothing to write
        float pd = -1.0f;
        int pi = -1;
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
            for (int b = 0; b < 32; ++b) {
                if (r * 32 + b >= K) break;
                float cd = __shfl_sync(RSFK_FULL, rd[r], b);
                int ci = __shfl_sync(RSFK_FULL, ri[r], b);
                if (ci < 0) {
                    if (!(cd == CUDART_INF_F)) sorted = false;
                    pd = CUDART_INF_F; pi = -1;
                    continue;
                }
                if (!key_less(pd, pi, cd, ci)) sorted = false;
                pd = cd; pi = ci;
                if (!L.try_insert(cd, ci, K, lane)) sorted = false; // repeated index
            }
        }
        if (!sorted) L.store(gi, gd, K, lane);
    }
}

// ---------------------------------------------------------------------------
// Leaf-bucket KNN.
//
// One CTA per leaf.  The leaf's rows are processed in blocks of B rows; for a
// block pair (I, J >= I) the rows are staged in shared memory, the B x B tile
// of squared distances is computed by warps in 4x4 register tiles (lane l owns
// dimensions l, l+32, ...; a transposed butterfly yields 16 distances per
// warp step in the reference's bit pattern), and then every row of I merges
// the tile row into its K-list (and, for J != I, every row of J the tile
// column).  Leaves that fit one block (the common case) stage each row once.
// ---------------------------------------------------------------------------
template <int KPL>
__device__ __forceinline__ void merge_candidates(WarpList<KPL>& L, const float* cand_d, int cand_stride,
                                                 const int* cand_ids, int n_cand, int self_id, int K,
                                                 int lane, bool& changed)
{
    for (int c0 = 0; c0 < n_cand; c0 += 32) {
        const int j = c0 + lane;
        float cd = CUDART_INF_F;
        int ci = -1;
        if (j < n_cand) {
            cd = cand_d[(size_t)j * cand_stride];
            ci = cand_ids[j];
        }
        bool pass = (j < n_cand) && ci != self_id && L.beats_threshold(cd, ci);
        unsigned mask = __ballot_sync(RSFK_FULL, pass);
        while (mask) {
            const int b = __ffs(mask) - 1;
            mask &= mask - 1;
            const float d = __shfl_sync(RSFK_FULL, cd, b);
            const int id = __shfl_sync(RSFK_FULL, ci, b);
            changed |= L.try_insert(d, id, K, lane);
        }
    }
}

// Rows ids[0..n) of the point array into X[n][D] (shared memory).  A warp takes
// rows warp, warp+8, ...; with 16-byte loads (VEC4: D % 4 == 0, aligned rows)
// four of its rows are in flight at a time, so that a 50-point bucket is fetched
// in two round trips instead of six.
template <bool VEC4>
__device__ __forceinline__ void stage_rows(const float* __restrict__ pts, int D, const int* ids, int n,
                                           float* X, int warp, int lane)
{
    if (VEC4) {
        const int D4 = D >> 2;
        float4* X4 = reinterpret_cast<float4*>(X);
        for (int rb = warp; rb < n; rb += 4 * KNN_WARPS) {
            const float4* src[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                src[u] = reinterpret_cast<const float4*>(pts + (size_t)ids[min(rb + u * KNN_WARPS, n - 1)] * D);
            for (int k4 = lane; k4 < D4; k4 += 32) {
                float4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = __ldg(src[u] + k4);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (rb + u * KNN_WARPS < n) X4[(size_t)(rb + u * KNN_WARPS) * D4 + k4] = v[u];
            }
        }
    } else {
        for (int r = warp; r < n; r += KNN_WARPS) {
            const float* src = pts + (size_t)ids[r] * D;
            float* dst = X + (size_t)r * D;
            for (int k = lane; k < D; k += 32) dst[k] = __ldg(src + k);
        }
    }
}

// Squared distance for D <= VL <= 16, one thread per pair.  In the reference's
// 32-lane sum every lane then holds at most one term (lanes >= D hold zero), so
// the result is the butterfly-ordered tree sum of the D squared differences.
template <int VL>
__device__ __forceinline__ float small_d_dist(const float* a, const float* b, int D)
{
    float acc[VL];
#pragma unroll
    for (int k = 0; k < VL; ++k) {
        const float df = k < D ? __fsub_rn(a[k], b[k]) : 0.0f;
        acc[k] = __fmaf_rn(df, df, 0.0f);
    }
#pragma unroll
    for (int stride = 1; stride < VL; stride <<= 1)
#pragma unroll
        for (int k = 0; k < VL; k += 2 * stride) acc[k] = __fadd_rn(acc[k], acc[k + stride]);
    return acc[0];
}

__device__ __forceinline__ float small_d_dist_any(const float* a, const float* b, int D)
{
    if (D <= 2) return small_d_dist<2>(a, b, D);
    if (D <= 4) return small_d_dist<4>(a, b, D);
    if (D <= 8) return small_d_dist<8>(a, b, D);
    return small_d_dist<16>(a, b, D);
}

template <int KPL, bool SMALL_D, bool VEC4>
__global__ void __launch_bounds__(KNN_THREADS, 3)
k_bucket_knn(const float* __restrict__ pts, int D, int K, const int* __restrict__ perm,
             const int* __restrict__ leaf_start, const int* __restrict__ leaf_count,
             int* __restrict__ knn_idx, float* __restrict__ knn_dist, int B, int two_blocks)
{
    extern __shared__ float4 smem4[];
    float* smem = reinterpret_cast<float*>(smem4);
    // layout: tile[B][B+1] | XI[B][D] | XJ[B][D] (only when two_blocks) | idsI[B] | idsJ[B]
    const int TS = B + 1;
    float* tile = smem;
    float* XI = tile + (size_t)B * TS;
    float* XJ = two_blocks ? XI + (size_t)B * D : XI;
    int* idsI = (int*)(XJ + (size_t)B * D);
    int* idsJ = two_blocks ? idsI + B : idsI;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int leaf = blockIdx.x;
    const int m = leaf_count[leaf];
    const int* ids = perm + leaf_start[leaf];
    const int n_blocks = (m + B - 1) / B;

    for (int bi = 0; bi < n_blocks; ++bi) {
        const int i0 = bi * B, mI = min(B, m - i0);
        __syncthreads();
        for (int r = threadIdx.x; r < mI; r += blockDim.x) idsI[r] = ids[i0 + r];
        __syncthreads();
        // A leaf that fits one block visits every row once: the first list of each warp is
        // requested now, before the rows and the distance tile, and each later one while
        // the previous row is merged, so that no warp waits for its list.
        const bool single = (n_blocks == 1);
        WarpList<KPL> Lnext;
        if (single && warp < mI) {
            const int first = idsI[warp];
            Lnext.load_raw(knn_idx + (size_t)first * K, knn_dist + (size_t)first * K, K, lane);
        }
        stage_rows<VEC4 && !SMALL_D>(pts, D, idsI, mI, XI, warp, lane);
        for (int bj = bi; bj < n_blocks; ++bj) {
            const int j0 = bj * B, mJ = min(B, m - j0);
            const bool diag = (bj == bi);
            if (!diag) {
                __syncthreads();
                for (int r = threadIdx.x; r < mJ; r += blockDim.x) idsJ[r] = ids[j0 + r];
                __syncthreads();
                stage_rows<VEC4 && !SMALL_D>(pts, D, idsJ, mJ, XJ, warp, lane);
            }
            __syncthreads();
            const float* XJc = diag ? XI : XJ;
            const int* idsJc = diag ? idsI : idsJ;
            // ---- distance tile ------------------------------------------------
            const int tI = (mI + 3) >> 2, tJ = (mJ + 3) >> 2;
            if (SMALL_D) {
                // few dimensions (D <= 16): one thread per pair
                for (int e = threadIdx.x; e < mI * mJ; e += blockDim.x) {
                    const int r = e / mJ, c = e - r * mJ;
                    if (diag && c < r) continue;
                    const float dsum = small_d_dist_any(XI + (size_t)r * D, XJc + (size_t)c * D, D);
                    tile[r * TS + c] = dsum;
                    if (diag) tile[c * TS + r] = dsum;
                }
            } else if (VEC4) {
                // 16-byte shared-memory loads: eight lanes share a 4x2 sub-tile of pairs, lane t
                // of the eight owns dimensions 4t..4t+3 (+32, ...), i.e. virtual lanes 4t..4t+3 of
                // the reference's sum; a warp covers an 8x4 tile.
                const int g = lane >> 3, t8 = lane & 7;
                const int D4 = D >> 2;
                const int sI = (mI + 7) >> 3, sJ = (mJ + 3) >> 2;
                const float4* XI4 = reinterpret_cast<const float4*>(XI);
                const float4* XJ4 = reinterpret_cast<const float4*>(XJc);
                for (int st = warp; st < sI * sJ; st += KNN_WARPS) {
                    const int ti = st / sJ, tj = st - ti * sJ;
                    if (diag && 4 * tj + 3 < 8 * ti) continue; // wholly below the diagonal
                    const int r0 = 8 * ti + 4 * (g >> 1), c0 = 4 * tj + 2 * (g & 1);
                    const float4* xi[4];
                    const float4* xj[2];
#pragma unroll
                    for (int u = 0; u < 4; ++u) xi[u] = XI4 + (size_t)min(r0 + u, mI - 1) * D4;
#pragma unroll
                    for (int v = 0; v < 2; ++v) xj[v] = XJ4 + (size_t)min(c0 + v, mJ - 1) * D4;
                    float acc[8][4];
#pragma unroll
                    for (int q = 0; q < 8; ++q)
#pragma unroll
                        for (int cc = 0; cc < 4; ++cc) acc[q][cc] = 0.0f;
                    for (int k4 = t8; k4 < D4; k4 += 8) {
                        float4 a[4], b[2];
#pragma unroll
                        for (int u = 0; u < 4; ++u) a[u] = xi[u][k4];
#pragma unroll
                        for (int v = 0; v < 2; ++v) b[v] = xj[v][k4];
#pragma unroll
                        for (int u = 0; u < 4; ++u)
#pragma unroll
                            for (int v = 0; v < 2; ++v) {
                                float df;
                                df = __fsub_rn(a[u].x, b[v].x); acc[u * 2 + v][0] = __fmaf_rn(df, df, acc[u * 2 + v][0]);
                                df = __fsub_rn(a[u].y, b[v].y); acc[u * 2 + v][1] = __fmaf_rn(df, df, acc[u * 2 + v][1]);
                                df = __fsub_rn(a[u].z, b[v].z); acc[u * 2 + v][2] = __fmaf_rn(df, df, acc[u * 2 + v][2]);
                                df = __fsub_rn(a[u].w, b[v].w); acc[u * 2 + v][3] = __fmaf_rn(df, df, acc[u * 2 + v][3]);
                            }
                    }
                    float part[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        part[q] = __fadd_rn(__fadd_rn(acc[q][0], acc[q][1]), __fadd_rn(acc[q][2], acc[q][3]));
                    halve_step<4, 1>(part, lane);
                    halve_step<2, 2>(part, lane);
                    halve_step<1, 4>(part, lane);
                    // lane t8 of the group now holds pair 4*bit0 + 2*bit1 + bit2 of its 4x2 sub-tile
                    const int item = ((t8 & 1) << 2) | (t8 & 2) | ((t8 & 4) >> 2);
                    const int r = r0 + (item >> 1), c = c0 + (item & 1);
                    if (r < mI && c < mJ) {
                        tile[r * TS + c] = part[0];
                        if (diag) tile[c * TS + r] = part[0];
                    }
                }
            } else
            for (int t = warp; t < tI * tJ; t += KNN_WARPS) {
                const int ti = t / tJ, tj = t - ti * tJ;
                if (diag && tj < ti) continue;
                const float* xi[4];
                const float* xj[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    xi[u] = XI + (size_t)min(ti * 4 + u, mI - 1) * D;
                    xj[u] = XJc + (size_t)min(tj * 4 + u, mJ - 1) * D;
                }
                float acc[16];
#pragma unroll
                for (int q = 0; q < 16; ++q) acc[q] = 0.0f;
                for (int k = lane; k < D; k += 32) {
                    float a[4], b[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) { a[u] = xi[u][k]; b[u] = xj[u][k]; }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            const float df = __fsub_rn(a[u], b[v]);
                            acc[u * 4 + v] = __fmaf_rn(df, df, acc[u * 4 + v]);
                        }
                }
                const float dsum = transposed_sum16(acc, lane);
                const int item = item16_of_lane(lane);
                const int r = ti * 4 + (item >> 2), c = tj * 4 + (item & 3);
                if (lane < 16 && r < mI && c < mJ) {
                    tile[r * TS + c] = dsum;
                    if (diag) tile[c * TS + r] = dsum;
                }
            }
            __syncthreads();
            // ---- rows of block I take the tile row ----------------------------
            for (int r = warp; r < mI; r += KNN_WARPS) {
                const int self = idsI[r];
                WarpList<KPL> L;
                if (single) {
                    L = Lnext;
                    L.refresh_threshold(K);
                    if (r + KNN_WARPS < mI) {
                        const int nxt = idsI[r + KNN_WARPS];
                        Lnext.load_raw(knn_idx + (size_t)nxt * K, knn_dist + (size_t)nxt * K, K, lane);
                    }
                } else {
                    L.load(knn_idx + (size_t)self * K, knn_dist + (size_t)self * K, K, lane);
                }
                bool changed = false;
                merge_candidates<KPL>(L, tile + r * TS, 1, idsJc, mJ, self, K, lane, changed);
                if (changed) L.store(knn_idx + (size_t)self * K, knn_dist + (size_t)self * K, K, lane);
            }
            // ---- rows of block J take the tile column -------------------------
            if (!diag) {
                for (int r = warp; r < mJ; r += KNN_WARPS) {
                    const int self = idsJ[r];
                    WarpList<KPL> L;
                    L.load(knn_idx + (size_t)self * K, knn_dist + (size_t)self * K, K, lane);
                    bool changed = false;
                    merge_candidates<KPL>(L, tile + r, TS, idsI, mI, self, K, lane, changed);
                    if (changed) L.store(knn_idx + (size_t)self * K, knn_dist + (size_t)self * K, K, lane);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Leaf-bucket KNN for few dimensions (D <= 16), leaves of any size whose rows fit
// shared memory.  With so few dimensions a distance costs less than a trip
// through a shared-memory tile: the leaf's rows are staged once, every warp owns
// rows warp, warp+8, ... and computes the distances of its row to 32 leaf members
// at a time (one pair per lane, the arithmetic of small_d_dist), feeding them
// straight into the row's list, which is read and written once per tree.  Each
// pair is evaluated from both ends (d(a,b) and d(b,a) carry the same bits).
// ---------------------------------------------------------------------------
template <int KPL>
__global__ void __launch_bounds__(KNN_THREADS, 3)
k_bucket_knn_lowd(const float* __restrict__ pts, int D, int K, const int* __restrict__ perm,
                  const int* __restrict__ leaf_start, const int* __restrict__ leaf_count,
                  int* __restrict__ knn_idx, float* __restrict__ knn_dist, int max_leaf)
{
    extern __shared__ float4 smem4[];
    float* X = reinterpret_cast<float*>(smem4);                  // [max_leaf][D]
    int* ids = reinterpret_cast<int*>(X + (size_t)max_leaf * D); // [max_leaf]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int leaf = blockIdx.x;
    const int m = min(leaf_count[leaf], max_leaf);
    const int* ids_g = perm + leaf_start[leaf];
    for (int r = threadIdx.x; r < m; r += blockDim.x) ids[r] = ids_g[r];
    __syncthreads();
    WarpList<KPL> Lnext;
    if (warp < m) {
        const int first = ids[warp];
        Lnext.load_raw(knn_idx + (size_t)first * K, knn_dist + (size_t)first * K, K, lane);
    }
    for (int e = threadIdx.x; e < m * D; e += blockDim.x) {
        const int r = e / D;
        X[e] = __ldg(pts + (size_t)ids[r] * D + (e - r * D));
    }
    __syncthreads();
    for (int r = warp; r < m; r += KNN_WARPS) {
        const int self = ids[r];
        WarpList<KPL> L = Lnext;
        L.refresh_threshold(K);
        if (r + KNN_WARPS < m) {
            const int nxt = ids[r + KNN_WARPS];
            Lnext.load_raw(knn_idx + (size_t)nxt * K, knn_dist + (size_t)nxt * K, K, lane);
        }
        const float* xr = X + (size_t)r * D;
        bool changed = false;
        for (int c0 = 0; c0 < m; c0 += 32) {
            const int j = c0 + lane;
            float cd = CUDART_INF_F;
            int ci = -1;
            if (j < m && j != r) {
                cd = small_d_dist_any(xr, X + (size_t)j * D, D);
                ci = ids[j];
            }
            unsigned mask = __ballot_sync(RSFK_FULL, ci >= 0 && L.beats_threshold(cd, ci));
            while (mask) {
                const int b = __ffs(mask) - 1;
                mask &= mask - 1;
                changed |= L.try_insert(__shfl_sync(RSFK_FULL, cd, b), __shfl_sync(RSFK_FULL, ci, b), K, lane);
            }
        }
        if (changed) L.store(knn_idx + (size_t)self * K, knn_dist + (size_t)self * K, K, lane);
    }
}

// ---------------------------------------------------------------------------
// Exploration sweep: one warp per point.  Candidates old[old[p][i]][k] that
// are not already in p's row are queued; every 32 queued candidates are
// evaluated together (each lane owns dimensions lane, lane+32, ... of all 32
// rows, a transposed butterfly leaves candidate c's distance in one lane).
// ---------------------------------------------------------------------------
constexpr int EXP_QUEUE = 64;

// Squared distances from the point (xp, shared memory) to up to 32 queued
// candidates; lane l returns the distance of candidate *cand (also returned).
// Scalar form: lane l owns dimensions l, l+32, ... of all 32 rows.
__device__ __forceinline__ float explore_dist32_scalar(const float* __restrict__ pts, int D, const float* xp,
                                                       const int* queue, int n, int lane, int& cand)
{
    float acc[32];
    const float* row[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) {
        acc[c] = 0.0f;
        row[c] = pts + (size_t)queue[min(c, n - 1)] * D;
    }
    for (int k = lane; k < D; k += 32) {
        const float x = xp[k];
        float v[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) v[c] = __ldg(row[c] + k);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            const float df = __fsub_rn(v[c], x);
            acc[c] = __fmaf_rn(df, df, acc[c]);
        }
    }
    const float dsum = transposed_sum32(acc, lane);
    cand = item32_of_lane(lane);
    return dsum;
}

// 16-byte loads (D % 4 == 0, aligned rows): eight lanes share a row; lane
// (g = lane/8, t = lane%8) owns terms 4t..4t+3 (+32, ...) of rows 4j+g, j=0..7,
// i.e. virtual lanes 4t..4t+3 of the reference's sum, and ends up with the
// distance of candidate 4t+g.
__device__ __forceinline__ float explore_dist32_vec4(const float* __restrict__ pts, int D, const float* xp,
                                                     const int* queue, int n, int lane, int& cand)
{
    const int g = lane >> 3, t = lane & 7;
    const float4* xp4 = reinterpret_cast<const float4*>(xp);
    const int D4 = D >> 2;
    float acc[8][4];
    const float4* row[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        row[j] = reinterpret_cast<const float4*>(pts + (size_t)queue[min(4 * j + g, n - 1)] * D);
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[j][q] = 0.0f;
    }
    for (int k4 = t; k4 < D4; k4 += 8) {
        const float4 x = xp4[k4];
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __ldg(row[j] + k4);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float df;
            df = __fsub_rn(v[j].x, x.x); acc[j][0] = __fmaf_rn(df, df, acc[j][0]);
            df = __fsub_rn(v[j].y, x.y); acc[j][1] = __fmaf_rn(df, df, acc[j][1]);
            df = __fsub_rn(v[j].z, x.z); acc[j][2] = __fmaf_rn(df, df, acc[j][2]);
            df = __fsub_rn(v[j].w, x.w); acc[j][3] = __fmaf_rn(df, df, acc[j][3]);
        }
    }
    float mine = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float s = __fadd_rn(__fadd_rn(acc[j][0], acc[j][1]), __fadd_rn(acc[j][2], acc[j][3]));
        s = __fadd_rn(s, __shfl_xor_sync(RSFK_FULL, s, 1));
        s = __fadd_rn(s, __shfl_xor_sync(RSFK_FULL, s, 2));
        s = __fadd_rn(s, __shfl_xor_sync(RSFK_FULL, s, 4));
        if (j == t) mine = s;
    }
    cand = 4 * t + g;
    return mine;
}

// The same distances for at most 4*J candidates with J in {2, 4}: a lane keeps J rows
// instead of eight and requests U = 8/J k-steps of each before it uses them, so that the
// number of dependent load rounds falls from D/32 to D/(32 U) -- what a batch of a few
// candidates of many dimensions waits for.  Every sum is formed in the same order.
template <int J, int U>
__device__ __forceinline__ float explore_dist_few_vec4(const float* __restrict__ pts, int D, const float* xp,
                                                       const int* queue, int n, int lane, int& cand)
{
    const int g = lane >> 3, t = lane & 7;
    const float4* xp4 = reinterpret_cast<const float4*>(xp);
    const int D4 = D >> 2;
    float acc[J][4];
    const float4* row[J];
#pragma unroll
    for (int j = 0; j < J; ++j) {
        row[j] = reinterpret_cast<const float4*>(pts + (size_t)queue[min(4 * j + g, n - 1)] * D);
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[j][q] = 0.0f;
    }
    for (int k4 = t; k4 < D4; k4 += 8 * U) {
        float4 v[U][J];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int j = 0; j < J; ++j)
                if (k4 + 8 * u < D4) v[u][j] = __ldg(row[j] + k4 + 8 * u);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (k4 + 8 * u < D4) {
                const float4 x = xp4[k4 + 8 * u];
#pragma unroll
                for (int j = 0; j < J; ++j) {
                    float df;
                    df = __fsub_rn(v[u][j].x, x.x); acc[j][0] = __fmaf_rn(df, df, acc[j][0]);
                    df = __fsub_rn(v[u][j].y, x.y); acc[j][1] = __fmaf_rn(df, df, acc[j][1]);
                    df = __fsub_rn(v[u][j].z, x.z); acc[j][2] = __fmaf_rn(df, df, acc[j][2]);
                    df = __fsub_rn(v[u][j].w, x.w); acc[j][3] = __fmaf_rn(df, df, acc[j][3]);
                }
            }
        }
    }
    float mine = 0.0f;
#pragma unroll
    for (int j = 0; j < J; ++j) {
        float s = __fadd_rn(__fadd_rn(acc[j][0], acc[j][1]), __fadd_rn(acc[j][2], acc[j][3]));
        s = __fadd_rn(s, __shfl_xor_sync(RSFK_FULL, s, 1));
        s = __fadd_rn(s, __shfl_xor_sync(RSFK_FULL, s, 2));
        s = __fadd_rn(s, __shfl_xor_sync(RSFK_FULL, s, 4));
        if (j == t) mine = s;
    }
    cand = 4 * t + g; // lanes with t >= J hold no candidate: 4t+g >= 4J >= n
    return mine;
}

// n candidates (1..32) with 16-byte loads: the routine with the fewest load rounds that holds them.
__device__ __forceinline__ float explore_dist_vec4_any(const float* __restrict__ pts, int D, const float* xp,
                                                       const int* queue, int n, int lane, int& cand)
{
    if (n <= 8) return explore_dist_few_vec4<2, 4>(pts, D, xp, queue, n, lane, cand);
    if (n <= 16) return explore_dist_few_vec4<4, 2>(pts, D, xp, queue, n, lane, cand);
    return explore_dist32_vec4(pts, D, xp, queue, n, lane, cand);
}

template <int KPL, bool VEC4>
__device__ __forceinline__ void explore_flush(WarpList<KPL>& L, const float* __restrict__ pts, int D,
                                              const float* xp, const int* queue, int n, int K,
                                              int lane, bool& changed)
{
    // n in [1,32] candidates at queue[0..n)
    int item;
    const float dsum = VEC4 ? explore_dist32_vec4(pts, D, xp, queue, n, lane, item)
                            : explore_dist32_scalar(pts, D, xp, queue, n, lane, item);
    const int ci = item < n ? queue[item] : -1;
    unsigned mask = __ballot_sync(RSFK_FULL, ci >= 0 && L.beats_threshold(dsum, ci));
    while (mask) {
        const int b = __ffs(mask) - 1;
        mask &= mask - 1;
        const float d = __shfl_sync(RSFK_FULL, dsum, b);
        const int id = __shfl_sync(RSFK_FULL, ci, b);
        changed |= L.try_insert(d, id, K, lane);
    }
}

// Per-warp set of the ids seen while one point is processed (open addressing
// in shared memory).  A candidate already in the set -- a member of the row or
// a candidate met before -- is not fetched again.  When a probe sequence finds
// no free slot the id is reported as new: a repeated evaluation is wasted work,
// never a wrong result (the list itself refuses repeated indices).
constexpr int EXP_PROBES = 16;

__device__ __forceinline__ bool seen_before(int* table, int table_log2, int c)
{
    unsigned h = ((unsigned)c * 2654435761u) >> (32 - table_log2);
    const unsigned wrap = (1u << table_log2) - 1u;
#pragma unroll 1
    for (int probe = 0; probe < EXP_PROBES; ++probe) {
        const int old = atomicCAS(&table[h], -1, c);
        if (old == -1) return false;
        if (old == c) return true;
        h = (h + 1) & wrap;
    }
    return false;
}

// Launch shape of the sweep: up to K*K candidates per point want a table of at
// least 2*K*K slots (capped at 4096); larger tables run four warps per CTA so
// that three CTAs still fit one SM.
struct ExploreShape {
    int warps, table_log2;
    size_t smem;
};
inline ExploreShape explore_shape(int D, int K)
{
    ExploreShape e;
    e.table_log2 = (K <= 32) ? 11 : 12;
    e.warps = (K <= 32) ? KNN_WARPS : 4;
    e.smem = sizeof(float) * (size_t)e.warps * D + sizeof(int) * (size_t)e.warps * (EXP_QUEUE + (1 << e.table_log2));
    return e;
}

template <int KPL, bool VEC4>
__global__ void __launch_bounds__(KNN_THREADS, 2)
k_explore(const float* __restrict__ pts, int N, int D, int K, const int* __restrict__ old_idx,
          int* __restrict__ knn_idx, float* __restrict__ knn_dist, int row_begin, int row_end,
          int list_row0, unsigned long long* __restrict__ evaluated, int table_log2)
{
    extern __shared__ float4 smem4[];
    float* smem = reinterpret_cast<float*>(smem4);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, cta_warps = blockDim.x >> 5;
    const int table_slots = 1 << table_log2;
    float* xp = smem + (size_t)warp * D;
    int* queue = (int*)(smem + (size_t)cta_warps * D) + warp * EXP_QUEUE;
    int* table = (int*)(smem + (size_t)cta_warps * D) + cta_warps * EXP_QUEUE + warp * table_slots;

    const int warp0 = blockIdx.x * cta_warps + warp;
    const int n_warps = gridDim.x * cta_warps;
    unsigned long long n_eval = 0;
    for (int p = row_begin + warp0; p < row_end; p += n_warps) {
        __syncwarp();
        for (int k = lane; k < D; k += 32) xp[k] = __ldg(pts + (size_t)p * D + k);
        for (int t = lane; t < table_slots; t += 32) table[t] = -1;
        WarpList<KPL> L;
        L.load(knn_idx + (size_t)(p - list_row0) * K, knn_dist + (size_t)(p - list_row0) * K, K, lane);
        int nb[KPL];
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
            int e = r * 32 + lane;
            nb[r] = e < K ? old_idx[(size_t)p * K + e] : -1;
        }
        __syncwarp();
        // members of the row are never candidates
#pragma unroll
        for (int r = 0; r < KPL; ++r)
            if (L.i[r] >= 0) seen_before(table, table_log2, L.i[r]);
        __syncwarp();
        bool changed = false;
        int qn = 0;
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
            for (int b = 0; b < 32; ++b) {
                if (r * 32 + b >= K) break;
                const int nbr = __shfl_sync(RSFK_FULL, nb[r], b);
                if (nbr < 0 || nbr >= N) continue;
                const int* nrow = old_idx + (size_t)nbr * K;
                for (int e0 = 0; e0 < K; e0 += 32) {
                    const int e = e0 + lane;
                    const int c = e < K ? nrow[e] : -1;
                    bool ok = c >= 0 && c < N;
                    if (ok) ok = !seen_before(table, table_log2, c);
                    const unsigned mask = __ballot_sync(RSFK_FULL, ok);
                    if (mask == 0) continue;
                    if (ok) queue[qn + __popc(mask & ((1u << lane) - 1u))] = c;
                    qn += __popc(mask);
                    __syncwarp();
                    if (qn >= 32) {
                        n_eval += 32;
                        explore_flush<KPL, VEC4>(L, pts, D, xp, queue, 32, K, lane, changed);
                        __syncwarp();
                        // move the tail to the front
                        const int rest = qn - 32;
                        int t = lane < rest ? queue[32 + lane] : -1;
                        __syncwarp();
                        if (lane < rest) queue[lane] = t;
                        qn = rest;
                        __syncwarp();
                    }
                }
            }
        }
        if (qn > 0) {
            n_eval += qn;
            explore_flush<KPL, VEC4>(L, pts, D, xp, queue, qn, K, lane, changed);
        }
        if (changed)
            L.store(knn_idx + (size_t)(p - list_row0) * K, knn_dist + (size_t)(p - list_row0) * K, K, lane);
    }
    if (lane == 0 && n_eval) atomicAdd(evaluated, n_eval);
}

// ---------------------------------------------------------------------------
// Query (ANN) bucket update (reference:
// compute_knn_from_buckets_perwarp_coalesced_ann,
// src/kernels/build_tree_update_parents_ann.cu:232-513): one warp per query,
// the base points of the bucket it was routed to are taken 32 at a time and
// merged into the query's list.  Queries are visited in leaf order
// (q_order), so the warps of a CTA read the same bucket rows.
// ---------------------------------------------------------------------------

// Exclusive prefix sum of counts[n] in place (one CTA); counts[n] = total.
__global__ void __launch_bounds__(1024)
k_leaf_offsets(int* __restrict__ counts, int n)
{
    __shared__ int sWarp[32];
    const int per = (n + blockDim.x - 1) / blockDim.x;
    const int lo = min(n, (int)threadIdx.x * per), hi = min(n, lo + per);
    int sum = 0;
    for (int i = lo; i < hi; ++i) sum += counts[i];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = sum;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        const int t = __shfl_up_sync(RSFK_FULL, incl, s);
        if (lane >= s) incl += t;
    }
    if (lane == 31) sWarp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = sWarp[lane], wi = w;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            const int t = __shfl_up_sync(RSFK_FULL, wi, s);
            if (lane >= s) wi += t;
        }
        sWarp[lane] = wi - w;
    }
    __syncthreads();
    int run = sWarp[warp] + incl - sum;
    for (int i = lo; i < hi; ++i) {
        const int c = counts[i];
        counts[i] = run;
        run += c;
    }
    if (threadIdx.x == blockDim.x - 1) counts[n] = run;
}

// q_order: queries grouped by leaf (any order inside a leaf: every query is
// independent of the others).  cursor = the offsets of k_leaf_offsets.
__global__ void k_place_queries(const int* __restrict__ q_leaf, int NQ, int* __restrict__ cursor,
                                int* __restrict__ q_order)
{
    for (int q = blockIdx.x * blockDim.x + threadIdx.x; q < NQ; q += gridDim.x * blockDim.x) {
        const int leaf = q_leaf[q];
        if (leaf < 0) continue;
        q_order[atomicAdd(&cursor[leaf], 1)] = q;
    }
}

template <int KPL, bool VEC4>
__global__ void __launch_bounds__(KNN_THREADS, 2)
k_ann_bucket(const float* __restrict__ pts, const float* __restrict__ queries, int D, int K,
             const int* __restrict__ perm, const int* __restrict__ leaf_start,
             const int* __restrict__ leaf_count, const int* __restrict__ q_leaf,
             const int* __restrict__ q_order, const int* __restrict__ n_order_ptr,
             int* __restrict__ knn_idx, float* __restrict__ knn_dist)
{
    extern __shared__ float4 smem4[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, cta_warps = blockDim.x >> 5;
    float* xq = reinterpret_cast<float*>(smem4) + (size_t)warp * D;
    const int warp0 = blockIdx.x * cta_warps + warp;
    const int n_warps = gridDim.x * cta_warps;
    const int n_order = *n_order_ptr; // queries that reached a leaf (all, unless the error flag is up)
    for (int o = warp0; o < n_order; o += n_warps) {
        const int q = q_order[o];
        const int leaf = q_leaf[q];
        const int* ids = perm + leaf_start[leaf];
        const int m = leaf_count[leaf];
        __syncwarp();
        for (int k = lane; k < D; k += 32) xq[k] = __ldg(queries + (size_t)q * D + k);
        WarpList<KPL> L;
        L.load(knn_idx + (size_t)q * K, knn_dist + (size_t)q * K, K, lane);
        __syncwarp();
        bool changed = false;
        for (int b0 = 0; b0 < m; b0 += 32)
            explore_flush<KPL, VEC4>(L, pts, D, xq, ids + b0, min(32, m - b0), K, lane, changed);
        if (changed) L.store(knn_idx + (size_t)q * K, knn_dist + (size_t)q * K, K, lane);
    }
}

// Query update, one CTA per leaf: the leaf's base rows are staged in shared
// memory once and every query routed to the leaf is compared with them there
// (same arithmetic, same lists as k_ann_bucket).  group_end[l] is the end of leaf
// l's group in q_order (groups in leaf order); a leaf without queries costs one
// load.  Used when the rows of the largest leaf fit shared memory.
template <int KPL, bool VEC4>
__global__ void __launch_bounds__(KNN_THREADS, KPL <= 1 ? 3 : 2)
k_ann_leaf(const float* __restrict__ pts, const float* __restrict__ queries, int D, int K,
           const int* __restrict__ perm, const int* __restrict__ leaf_start,
           const int* __restrict__ leaf_count, const int* __restrict__ group_end,
           const int* __restrict__ q_order, int max_leaf, int* __restrict__ knn_idx,
           float* __restrict__ knn_dist)
{
    extern __shared__ float4 smem4[];
    float* X = reinterpret_cast<float*>(smem4);                  // [max_leaf][D]
    float* xq_all = X + (size_t)max_leaf * D;                    // [KNN_WARPS][D]
    int* ids = reinterpret_cast<int*>(xq_all + (size_t)KNN_WARPS * D); // [max_leaf]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int leaf = blockIdx.x;
    const int q_end = group_end[leaf];
    const int q_beg = leaf > 0 ? group_end[leaf - 1] : 0;
    if (q_end <= q_beg) return;
    const int m = min(leaf_count[leaf], max_leaf);
    const int* ids_g = perm + leaf_start[leaf];
    for (int r = threadIdx.x; r < m; r += blockDim.x) ids[r] = ids_g[r];
    // the first query of each warp: its list and its row are requested before the leaf's rows
    WarpList<KPL> Lnext;
    int q_next = -1;
    if (q_beg + warp < q_end) {
        q_next = q_order[q_beg + warp];
        Lnext.load_raw(knn_idx + (size_t)q_next * K, knn_dist + (size_t)q_next * K, K, lane);
    }
    __syncthreads();
    stage_rows<VEC4>(pts, D, ids, m, X, warp, lane);
    __syncthreads();
    float* xq = xq_all + (size_t)warp * D;
    for (int o = q_beg + warp; o < q_end; o += KNN_WARPS) {
        const int q = q_next;
        __syncwarp();
        for (int k = lane; k < D; k += 32) xq[k] = __ldg(queries + (size_t)q * D + k);
        WarpList<KPL> L = Lnext;
        L.refresh_threshold(K);
        if (o + KNN_WARPS < q_end) {
            q_next = q_order[o + KNN_WARPS];
            Lnext.load_raw(knn_idx + (size_t)q_next * K, knn_dist + (size_t)q_next * K, K, lane);
        }
        __syncwarp();
        bool changed = false;
        for (int b0 = 0; b0 < m; b0 += 32) {
            const int n = min(32, m - b0);
            int item;
            const float dsum = VEC4 ? leaf_dist32_vec4(X, D, xq, b0, n, lane, item)
                                    : leaf_dist32_scalar(X, D, xq, b0, n, lane, item);
            const int ci = item < n ? ids[b0 + item] : -1;
            unsigned mask = __ballot_sync(RSFK_FULL, ci >= 0 && L.beats_threshold(dsum, ci));
            while (mask) {
                const int b = __ffs(mask) - 1;
                mask &= mask - 1;
                changed |= L.try_insert(__shfl_sync(RSFK_FULL, dsum, b), __shfl_sync(RSFK_FULL, ci, b), K, lane);
            }
        }
        if (changed) L.store(knn_idx + (size_t)q * K, knn_dist + (size_t)q * K, K, lane);
    }
}

// ---------------------------------------------------------------------------
// G-way merge of canonical lists: out = K smallest distinct of all G rows.
// ---------------------------------------------------------------------------
struct MergeArgs {
    const int* idx[16];
    const float* dist[16];
};

template <int KPL>
__global__ void __launch_bounds__(KNN_THREADS)
k_merge_lists(MergeArgs args, int G, long long rows, int K, int* __restrict__ out_idx,
              float* __restrict__ out_dist)
{
    const int lane = threadIdx.x & 31;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long row = warp0; row < rows; row += n_warps) {
        WarpList<KPL> L;
        L.load(args.idx[0] + row * K, args.dist[0] + row * K, K, lane);
        for (int g = 1; g < G; ++g) {
            const int* gi = args.idx[g] + row * K;
            const float* gd = args.dist[g] + row * K;
            for (int e0 = 0; e0 < K; e0 += 32) {
                const int e = e0 + lane;
                const float cd = e < K ? gd[e] : CUDART_INF_F;
                const int ci = e < K ? gi[e] : -1;
                unsigned mask = __ballot_sync(RSFK_FULL, ci >= 0 && L.beats_threshold(cd, ci));
                while (mask) {
                    const int b = __ffs(mask) - 1;
                    mask &= mask - 1;
                    L.try_insert(__shfl_sync(RSFK_FULL, cd, b), __shfl_sync(RSFK_FULL, ci, b), K, lane);
                }
            }
        }
        L.store(out_idx + row * K, out_dist + row * K, K, lane);
    }
}

#include "rsfk_bucket_tc.cuh"

// ---------------------------------------------------------------------------
// host launchers
// ---------------------------------------------------------------------------
static int kpl_for(int K)
{
    int kpl = 1;
    while (kpl * 32 < K) kpl <<= 1;
    return kpl;
}

#define RSFK_DISPATCH_KPL(K, ...)                                                     \
    switch (kpl_for(K)) {                                                             \
    case 1: { constexpr int KPL = 1; __VA_ARGS__; } break;                            \
    case 2: { constexpr int KPL = 2; __VA_ARGS__; } break;                            \
    case 4: { constexpr int KPL = 4; __VA_ARGS__; } break;                            \
    default: { constexpr int KPL = 8; __VA_ARGS__; } break;                           \
    }

static bool check_k(Context& ctx, int K)
{
    if (K < 1) return ctx.fail(RSFK_ERR_ARG, "K must be at least 1");
    if (K > list_capacity())
        return ctx.fail(RSFK_ERR_UNSUPPORTED, "K above 256 is not supported by this build");
    return true;
}

__global__ void k_fill_empty(int* __restrict__ idx, float* __restrict__ dist, long long n)
{
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {
        idx[e] = -1;
        dist[e] = CUDART_INF_F;
    }
}

bool fill_empty_lists(Context& ctx, int* d_idx, float* d_dist, long long n)
{
    if (n <= 0) return true;
    long long blocks = (n + 255) / 256;
    if (blocks > ctx.sm_count * 16) blocks = ctx.sm_count * 16;
    k_fill_empty<<<(int)blocks, 256, 0, ctx.stream>>>(d_idx, d_dist, n);
    count_launches(1);
    return ctx.check(cudaGetLastError(), "fill launch");
}

bool sort_rows(Context& ctx, int* d_idx, float* d_dist, long long rows, int K)
{
    if (!check_k(ctx, K)) return false;
    if (rows <= 0) return true;
    long long blocks = (rows + KNN_WARPS - 1) / KNN_WARPS;
    if (blocks > ctx.sm_count * 16) blocks = ctx.sm_count * 16;
    RSFK_DISPATCH_KPL(K, (k_sort_rows<KPL><<<(int)blocks, KNN_THREADS, 0, ctx.stream>>>(d_idx, d_dist, rows, K)));
    count_launches(1);
    return ctx.check(cudaGetLastError(), "sort_rows launch");
}

// The driver's tensor-map encoder, looked up once (the library does not link libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn tensor_map_encoder()
{
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// Bucket KNN on the tensor cores: leaf-ordered centred copy of the points, tile list,
// then the persistent pipeline kernel (rsfk_bucket_tc.cuh).
static bool bucket_knn_tc(Context& ctx, const float* d_points, int N, int D, int K, const TreeResult& tree,
                          int* d_idx, float* d_dist)
{
    cudaStream_t st = ctx.stream;
    const int Dp = (D + tc::KC - 1) / tc::KC * tc::KC;
    const int tile_cap = N / tc::BM + tree.n_leaves + 1;
    float* rows = (float*)ctx.scratch(Context::TC_ROWS, sizeof(float) * (size_t)N * Dp);
    float* rows_exact = (float*)ctx.scratch(Context::TC_EXACT, sizeof(float) * (size_t)N * D);
    float* norms = (float*)ctx.scratch(Context::TC_NORMS, sizeof(float) * (size_t)N);
    tc::Tile* tiles = (tc::Tile*)ctx.scratch(Context::TC_TILES, sizeof(tc::Tile) * (size_t)tile_cap);
    // [1]: rows left to k_tc_later, [2]: tiles with a row whose list is not full
    int* n_tiles = (int*)ctx.scratch(Context::TC_COUNT, 3 * sizeof(int));
    int* later_count = n_tiles ? n_tiles + 1 : nullptr;
    int* n_open = n_tiles ? n_tiles + 2 : nullptr;
    int* open_tile = (int*)ctx.scratch(Context::TC_OPEN, sizeof(int) * (size_t)tile_cap);
    float* thr0 = (float*)ctx.scratch(Context::TC_THR0, sizeof(float) * (size_t)N);
    int* later_rows = (int*)ctx.scratch(Context::TC_LATER_ROWS, sizeof(int) * (size_t)N);
    int* later_cand = (int*)ctx.scratch(Context::TC_LATER_CAND, sizeof(int) * (size_t)N * 32);
    unsigned long long* counters = ctx.tc_counters();
    int* flag = ctx.error_flag();
    if (!rows || !rows_exact || !norms || !tiles || !n_tiles || !later_rows || !later_cand || !open_tile || !thr0 ||
        !counters || !flag)
        return false;
    EncodeTiledFn encode = tensor_map_encoder();
    if (!encode) return ctx.fail(RSFK_ERR_CUDA, "bucket_knn: the driver offers no cuTensorMapEncodeTiled");
    // rows[N][Dp] fp32; a box is 32 floats (128 bytes, the swizzle span) by 128 rows
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)Dp, (cuuint64_t)N};
    const cuuint64_t strides[1] = {(cuuint64_t)Dp * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)tc::KC, (cuuint32_t)tc::BM};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, rows, dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return ctx.fail(RSFK_ERR_CUDA, "bucket_knn: cuTensorMapEncodeTiled failed");

    if (!ctx.check(cudaMemsetAsync(n_tiles, 0, 3 * sizeof(int), st), "clear tile count")) return false;
    tc::k_tc_tiles<<<(tree.n_leaves + 255) / 256, 256, 0, st>>>(tree.leaf_start, tree.leaf_count, tree.n_leaves,
                                                               tree.max_leaf, tiles, tile_cap, n_tiles);
    int row_grid = tile_cap < ctx.sm_count * 8 ? tile_cap : ctx.sm_count * 8;
    tc::k_tc_rows<<<row_grid, 256, sizeof(float) * (size_t)D, st>>>(d_points, D, Dp, tree.perm, tiles, n_tiles,
                                                                   tile_cap, rows, norms, rows_exact);
    const tc::Layout lay = tc::layout_for(D, tree.max_leaf);
    const bool vec4 = (D % 4 == 0) && ((reinterpret_cast<uintptr_t>(rows_exact) & 15) == 0);
    const float c_acc = tc::acc_margin(D);
    const int grid = tile_cap < ctx.sm_count ? tile_cap : ctx.sm_count;
    // Rows without a full list (a first tree): a first pass of the same pipeline over their tiles
    // derives each row's threshold from the approximate distances to its whole leaf; it leaves at
    // once when every list is full.
    {
        int open_grid = (tile_cap + 7) / 8;
        if (open_grid > ctx.sm_count * 8) open_grid = ctx.sm_count * 8;
        tc::k_tc_open_tiles<<<open_grid, 256, 0, st>>>(tiles, n_tiles, tile_cap, tree.perm, d_dist, K, open_tile, n_open);
        if (!ctx.check(cudaFuncSetAttribute(tc::k_tc_thresholds, cudaFuncAttributeMaxDynamicSharedMemorySize, lay.total),
                       "bucket_knn_tc smem attribute"))
            return false;
        tc::k_tc_thresholds<<<grid, tc::THREADS, lay.total, st>>>(map, D, Dp, K, tree.perm, norms, tiles, n_tiles,
                                                                  tile_cap, d_dist, tree.max_leaf, c_acc, flag,
                                                                  open_tile, n_open, thr0);
    }
    RSFK_DISPATCH_KPL(K, {
        auto kern = vec4 ? tc::k_bucket_knn_tc<KPL, true> : tc::k_bucket_knn_tc<KPL, false>;
        if (!ctx.check(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, lay.total),
                       "bucket_knn_tc smem attribute"))
            return false;
        kern<<<grid, tc::THREADS, lay.total, st>>>(map, rows_exact, D, Dp, K, tree.perm, norms, tiles, n_tiles,
                                                   tile_cap, d_idx, d_dist, tree.max_leaf, c_acc, counters, flag,
                                                   later_count, later_rows, later_cand, thr0);
        // the rows it left with less than a batch of candidates (a leaf's rows are disjoint from
        // every other leaf's, so nothing else touches their lists)
        auto later = vec4 ? tc::k_tc_later<KPL, true> : tc::k_tc_later<KPL, false>;
        const size_t later_smem = sizeof(float) * (size_t)tc::LATER_WARPS * (((D + 3) & ~3) + 32);
        if (later_smem > 48 * 1024 &&
            !ctx.check(cudaFuncSetAttribute(later, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)later_smem),
                       "bucket_knn_tc smem attribute"))
            return false;
        int per_sm = (int)(200 * 1024 / (later_smem + 1024));
        per_sm = per_sm < 1 ? 1 : (per_sm > 6 ? 6 : per_sm);
        const long long want = ((long long)N + tc::LATER_WARPS - 1) / tc::LATER_WARPS;
        const int later_grid = (int)(want < (long long)ctx.sm_count * per_sm ? want : (long long)ctx.sm_count * per_sm);
        later<<<later_grid, 32 * tc::LATER_WARPS, later_smem, st>>>(rows_exact, D, K, tree.perm, later_count,
                                                                    later_rows, later_cand, d_idx, d_dist);
    });
    count_launches(6);
    ctx.stats.tc_launches++;
    if (tree.sum_leaf_sq > 0) ctx.stats.tc_gram_flops += 2.0 * D * tree.sum_leaf_sq;
    return ctx.check(cudaGetLastError(), "bucket_knn_tc launch");
}

bool bucket_knn(Context& ctx, const float* d_points, int N, int D, int K, const TreeResult& tree,
                int* d_idx, float* d_dist)
{
    TraceRange trace("rsfk bucket knn");
    (void)N;
    cudaStream_t launch_stream = ctx.stream;
    if (!check_k(ctx, K)) return false;
    if (tree.n_leaves <= 0) return true;
    // few dimensions: every leaf's rows fit shared memory, distances are computed where they are used
    if (D <= 16 && (sizeof(float) * D + sizeof(int)) * (size_t)tree.max_leaf <= 72 * 1024) {
        const size_t smem = (sizeof(float) * D + sizeof(int)) * (size_t)tree.max_leaf;
        RSFK_DISPATCH_KPL(K, {
            auto kern = k_bucket_knn_lowd<KPL>;
            if (smem > 48 * 1024 &&
                !ctx.check(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                           "bucket_knn smem attribute"))
                return false;
            kern<<<tree.n_leaves, KNN_THREADS, smem, ctx.stream>>>(d_points, D, K, tree.perm, tree.leaf_start,
                                                                  tree.leaf_count, d_idx, d_dist, tree.max_leaf);
        });
        count_launches(1);
        return ctx.check(cudaGetLastError(), "bucket_knn launch");
    }
    const size_t budget = 200 * 1024;
    auto bytes = [&](int B, int two) {
        return sizeof(float) * ((size_t)B * (B + 1) + (size_t)(two ? 2 : 1) * B * D) + sizeof(int) * (size_t)(two ? 2 : 1) * B;
    };
    // D >= 64: Gram tiles on the tensor cores (the context's tc_mode: 1 always, 0 never;
    // by default where a leaf no longer fits the SIMT kernel's single shared-memory
    // block, which is where that kernel re-stages rows many times)
    const bool simt_single_block = bytes((tree.max_leaf + 3) & ~3, 0) <= budget;
    const bool want_tc = ctx.tc_mode == 1 || (ctx.tc_mode == -1 && !simt_single_block);
    if (want_tc && D >= 64 && N >= tc::BM && tree.max_leaf <= tc::MAX_LEAF &&
        tc::layout_for(D, tree.max_leaf).total <= 227 * 1024)
        return bucket_knn_tc(ctx, d_points, N, D, K, tree, d_idx, d_dist);
    // block size: the whole leaf when it fits, else the largest that fits twice
    int B = (tree.max_leaf + 3) & ~3;
    if (B < 4) B = 4;
    int two = 0;
    if (bytes(B, 0) > budget) {
        two = 1;
        B = 128;
        while (B > 4 && bytes(B, 1) > budget) B >>= 1;
        if (bytes(B, 1) > budget)
            return ctx.fail(RSFK_ERR_UNSUPPORTED, "bucket_knn: D too large for the shared-memory tile");
    }
    const size_t smem = bytes(B, two);
    RSFK_DISPATCH_KPL(K, {
        const bool v4 = (D % 4 == 0) && (B % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_points) & 15) == 0);
        auto kern = (D <= 16) ? k_bucket_knn<KPL, true, false>
                              : (v4 ? k_bucket_knn<KPL, false, true> : k_bucket_knn<KPL, false, false>);
        if (!ctx.check(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                       "bucket_knn smem attribute"))
            return false;
        kern<<<tree.n_leaves, KNN_THREADS, smem, launch_stream>>>(d_points, D, K, tree.perm, tree.leaf_start,
                                                              tree.leaf_count, d_idx, d_dist, B, two);
    });
    count_launches(1);
    return ctx.check(cudaGetLastError(), "bucket_knn launch");
}

// ---------------------------------------------------------------------------
// The sweep for long lists of medium-sized rows (32 < K <= 64, 64 <= D <= 128: 20 M x 128 with
// K = 64).  There the per-warp hash set takes 16 KiB, twelve warps fit an SM, and with register
// loads (k_explore) those twelve warps keep 48 KiB of rows in flight: 0.59 of the bandwidth that
// random row gathers reach.  Here a point is handled in two steps.  First all its candidates are
// gathered and made distinct (same hash set, same rule) and written to a list in global memory.
// Then the hash set's shared memory becomes two buffers of 16 whole rows each, filled by bulk
// copies (cp.async.bulk, one per row, completion counted on an mbarrier per buffer) while the
// other buffer is evaluated: up to 16 KiB in flight per warp, no registers held by loads.
// Distances are formed as k_explore's scalar routine forms them (lane l owns dimensions l, l+32,
// ..., transposed butterfly), so the bits are the same.
// Every wait is bounded; one that runs out raises the error flag and the warp leaves.
// Measured on 2 M x 128, K = 64 (one B200): 241 ms per sweep against 302 ms for k_explore.
// Tried and slower: four buffers of 8 rows with three in flight (314 ms: the work per batch of
// eight rows, not the bytes in flight, sets the pace) and 16-byte cp.async copies with commit
// groups instead of the bulk copies (262 ms).
// ---------------------------------------------------------------------------
constexpr int STAGED_WARPS = 4;
constexpr int STAGED_ROWS = 16; // rows per buffer

__device__ __forceinline__ void bulk_row_to_shared(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

template <int KPL>
__global__ void __launch_bounds__(32 * STAGED_WARPS, 3)
k_explore_staged(const float* __restrict__ pts, int N, int D, int K, const int* __restrict__ old_idx,
                 int* __restrict__ knn_idx, float* __restrict__ knn_dist, int row_begin, int row_end,
                 int list_row0, unsigned long long* __restrict__ evaluated, int table_log2,
                 int* __restrict__ cand_scratch, int cand_cap, int* __restrict__ error_flag)
{
    extern __shared__ float4 smem4[];
    __shared__ uint64_t sBar[STAGED_WARPS][2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int table_slots = 1 << table_log2;
    // per warp: xp[D] | table_slots words: the hash set, later 2 x 16 rows of D floats
    float* xp = reinterpret_cast<float*>(smem4) + (size_t)warp * (D + table_slots);
    int* table = reinterpret_cast<int*>(xp + D);
    const float* rows = xp + D;
    const uint32_t rows_addr = tc::smem_u32(rows);
    const uint32_t row_bytes = (uint32_t)D * 4u;
    const uint32_t bar[2] = {tc::smem_u32(&sBar[warp][0]), tc::smem_u32(&sBar[warp][1])};
    if (lane == 0) {
        tc::mbar_init(bar[0], 1);
        tc::mbar_init(bar[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    unsigned parity[2] = {0u, 0u};
    int* cand = cand_scratch + (size_t)(blockIdx.x * STAGED_WARPS + warp) * cand_cap;

    const int warp0 = blockIdx.x * STAGED_WARPS + warp;
    const int n_warps = gridDim.x * STAGED_WARPS;
    unsigned long long n_eval = 0;
    bool alive = true;
    for (int p = row_begin + warp0; p < row_end && alive; p += n_warps) {
        __syncwarp();
        // ---- the point's distinct candidates -> cand[0..n) -------------------
        for (int t = lane; t < table_slots; t += 32) table[t] = -1;
        WarpList<KPL> L;
        L.load(knn_idx + (size_t)(p - list_row0) * K, knn_dist + (size_t)(p - list_row0) * K, K, lane);
        int nb[KPL];
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
            const int e = r * 32 + lane;
            nb[r] = e < K ? old_idx[(size_t)p * K + e] : -1;
        }
        for (int k = lane; k < D; k += 32) xp[k] = __ldg(pts + (size_t)p * D + k);
        __syncwarp();
#pragma unroll
        for (int r = 0; r < KPL; ++r)
            if (L.i[r] >= 0) seen_before(table, table_log2, L.i[r]);
        __syncwarp();
        int n = 0;
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
            for (int b0 = 0; b0 < 32; b0 += 4) {
                if (r * 32 + b0 >= K) break;
                // four neighbours' lists are requested together
                int c[4][KPL];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int nbr = __shfl_sync(RSFK_FULL, nb[r], b0 + u);
                    const bool live = r * 32 + b0 + u < K && nbr >= 0 && nbr < N;
#pragma unroll
                    for (int q = 0; q < KPL; ++q) {
                        const int e = q * 32 + lane;
                        c[u][q] = (live && e < K) ? old_idx[(size_t)nbr * K + e] : -1;
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int q = 0; q < KPL; ++q) {
                        const int v = c[u][q];
                        bool ok = v >= 0 && v < N;
                        if (ok) ok = !seen_before(table, table_log2, v);
                        const unsigned mask = __ballot_sync(RSFK_FULL, ok);
                        const int at = n + __popc(mask & ((1u << lane) - 1u));
                        if (ok && at < cand_cap) cand[at] = v;
                        n = min(n + __popc(mask), cand_cap);
                    }
            }
        }
        n_eval += n;
        __syncwarp();
        if (n == 0) continue;
        // ---- evaluation: the hash set's memory becomes the row buffers --------
        __threadfence_block(); // the list written above is read back by other lanes below
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        const int n_batches = (n + STAGED_ROWS - 1) / STAGED_ROWS;
        // ids of the rows a buffer holds (lane j: row j), and of the rows it takes next
        int id_next[2], id_cur[2] = {-1, -1};
        id_next[0] = (lane < STAGED_ROWS && lane < n) ? cand[lane] : -1;
        id_next[1] = (lane < STAGED_ROWS && STAGED_ROWS + lane < n) ? cand[STAGED_ROWS + lane] : -1;
        auto issue = [&](int b) { // batch b -> buffer b & 1
            const int h = b & 1;
            const int m = min(STAGED_ROWS, n - STAGED_ROWS * b);
            id_cur[h] = id_next[h];
            if (lane == 0) tc::mbar_expect_tx(bar[h], (uint32_t)m * row_bytes);
            __syncwarp();
            if (lane < m)
                bulk_row_to_shared(rows_addr + (uint32_t)(h * STAGED_ROWS + lane) * row_bytes,
                                   pts + (size_t)id_cur[h] * D, row_bytes, bar[h]);
            const int later = STAGED_ROWS * (b + 2) + lane;
            id_next[h] = (lane < STAGED_ROWS && later < n) ? cand[later] : -1;
        };
        issue(0);
        if (n_batches > 1) issue(1);
        bool changed = false;
        for (int b = 0; b < n_batches; ++b) {
            const int h = b & 1;
            const int m = min(STAGED_ROWS, n - STAGED_ROWS * b);
            bool arrived = false;
            for (unsigned it = 0; it < tc::WAIT_LIMIT && !arrived; ++it) arrived = tc::mbar_try(bar[h], parity[h]);
            parity[h] ^= 1u;
            if (!__all_sync(RSFK_FULL, arrived)) { // give up: wait once more for what is in flight, then leave
                const int o = h ^ 1;
                if (b + 1 < n_batches)
                    for (unsigned it = 0; it < tc::WAIT_LIMIT; ++it)
                        if (tc::mbar_try(bar[o], parity[o])) break;
                if (lane == 0) atomicExch(error_flag, 1);
                alive = false;
                break;
            }
            const float* R = rows + (size_t)h * STAGED_ROWS * D;
            float acc[STAGED_ROWS];
#pragma unroll
            for (int c = 0; c < STAGED_ROWS; ++c) acc[c] = 0.0f;
            for (int k = lane; k < D; k += 32) {
                const float x = xp[k];
#pragma unroll
                for (int c = 0; c < STAGED_ROWS; ++c) {
                    const float df = __fsub_rn(R[(size_t)c * D + k], x);
                    acc[c] = __fmaf_rn(df, df, acc[c]);
                }
            }
            const float dsum = transposed_sum16(acc, lane);
            const int item = item16_of_lane(lane);
            int ci = __shfl_sync(RSFK_FULL, id_cur[h], item);
            if (lane >= 16 || item >= m) ci = -1;
            unsigned mask = __ballot_sync(RSFK_FULL, ci >= 0 && L.beats_threshold(dsum, ci));
            while (mask) {
                const int w = __ffs(mask) - 1;
                mask &= mask - 1;
                changed |= L.try_insert(__shfl_sync(RSFK_FULL, dsum, w), __shfl_sync(RSFK_FULL, ci, w), K, lane);
            }
            __syncwarp(); // the buffer's rows are read; it may be filled again
            if (b + 2 < n_batches) issue(b + 2);
        }
        if (alive && changed)
            L.store(knn_idx + (size_t)(p - list_row0) * K, knn_dist + (size_t)(p - list_row0) * K, K, lane);
    }
    if (lane == 0 && n_eval) atomicAdd(evaluated, n_eval);
}

// ---------------------------------------------------------------------------
// The sweep for wide rows (K <= 32, rows of 2 KiB and more: 1 M x 960).  The same two steps as
// k_explore_staged -- a point's distinct candidates are listed first (here in shared memory),
// then their rows come into shared memory by bulk copies -- but a buffer is ONE row and a warp
// has NBUF of them (the hash set's memory and what eight warps per SM instead of sixteen leave
// free): NBUF - 1 rows of 4 D bytes are in flight while one is evaluated, against 4 KiB per warp
// with register loads.  A row is evaluated by the whole warp in the reference's order (lane l
// takes dimensions l, l+32, ..., xor butterfly), one candidate at a time.  Every wait is bounded;
// one that runs out raises the error flag and the warp leaves.
// ---------------------------------------------------------------------------
constexpr int WIDE_WARPS = 4;
constexpr int WIDE_CAND = 1024; // K * K for K <= 32

template <int NBUF>
__global__ void __launch_bounds__(32 * WIDE_WARPS, 2)
k_explore_wide(const float* __restrict__ pts, int N, int D, int K, const int* __restrict__ old_idx,
               int* __restrict__ knn_idx, float* __restrict__ knn_dist, int row_begin, int row_end,
               int list_row0, unsigned long long* __restrict__ evaluated, int table_log2,
               int area_floats, int* __restrict__ error_flag)
{
    extern __shared__ float4 smem4[];
    __shared__ uint64_t sBar[WIDE_WARPS][NBUF];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // per warp: xp[D] | cand[WIDE_CAND] | area: the hash set (1 << table_log2 words), later NBUF rows of D floats
    float* xp = reinterpret_cast<float*>(smem4) + (size_t)warp * (D + WIDE_CAND + area_floats);
    int* cand = reinterpret_cast<int*>(xp + D);
    int* table = cand + WIDE_CAND;
    const float* rows = reinterpret_cast<const float*>(table);
    const uint32_t rows_addr = tc::smem_u32(rows);
    const uint32_t row_bytes = (uint32_t)D * 4u;
    uint32_t bar[NBUF];
    unsigned parity[NBUF];
#pragma unroll
    for (int u = 0; u < NBUF; ++u) {
        bar[u] = tc::smem_u32(&sBar[warp][u]);
        parity[u] = 0u;
        if (lane == 0) tc::mbar_init(bar[u], 1);
    }
    if (lane == 0) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();
    const int table_slots = 1 << table_log2;

    const int warp0 = blockIdx.x * WIDE_WARPS + warp;
    const int n_warps = gridDim.x * WIDE_WARPS;
    unsigned long long n_eval = 0;
    bool alive = true;
    for (int p = row_begin + warp0; p < row_end && alive; p += n_warps) {
        __syncwarp();
        // ---- the point's distinct candidates -> cand[0..n) -------------------
        for (int t = lane; t < table_slots; t += 32) table[t] = -1;
        WarpList<1> L;
        L.load(knn_idx + (size_t)(p - list_row0) * K, knn_dist + (size_t)(p - list_row0) * K, K, lane);
        const int nb = lane < K ? old_idx[(size_t)p * K + lane] : -1;
        for (int k = lane; k < D; k += 32) xp[k] = __ldg(pts + (size_t)p * D + k);
        __syncwarp();
        if (L.i[0] >= 0) seen_before(table, table_log2, L.i[0]);
        __syncwarp();
        int n = 0;
        for (int b0 = 0; b0 < K; b0 += 8) {
            int c[8]; // eight neighbours' lists are requested together
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int nbr = __shfl_sync(RSFK_FULL, nb, min(b0 + u, 31));
                const bool live = b0 + u < K && nbr >= 0 && nbr < N;
                c[u] = (live && lane < K) ? old_idx[(size_t)nbr * K + lane] : -1;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int v = c[u];
                bool ok = v >= 0 && v < N;
                if (ok) ok = !seen_before(table, table_log2, v);
                const unsigned mask = __ballot_sync(RSFK_FULL, ok);
                const int at = n + __popc(mask & ((1u << lane) - 1u));
                if (ok && at < WIDE_CAND) cand[at] = v;
                n = min(n + __popc(mask), WIDE_CAND);
            }
        }
        n_eval += n;
        __syncwarp();
        if (n == 0) continue;
        // ---- evaluation: the hash set's memory becomes the row buffers --------
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        auto issue = [&](int b, int u) { // candidate b -> buffer u
            if (lane == 0) {
                tc::mbar_expect_tx(bar[u], row_bytes);
                bulk_row_to_shared(rows_addr + (uint32_t)u * row_bytes, pts + (size_t)cand[b] * D, row_bytes, bar[u]);
            }
        };
#pragma unroll
        for (int u = 0; u < NBUF - 1; ++u)
            if (u < n) issue(u, u);
        bool changed = false;
        for (int b0 = 0; b0 < n && alive; b0 += NBUF) {
#pragma unroll
            for (int u = 0; u < NBUF; ++u) {
                const int b = b0 + u;
                if (b >= n || !alive) break;
                // all but one buffer in flight: the one candidate b-1 was read from is free again
                if (b + NBUF - 1 < n) issue(b + NBUF - 1, (u + NBUF - 1) % NBUF);
                const int ci = cand[b];
                bool arrived = false;
                for (unsigned it = 0; it < tc::WAIT_LIMIT && !arrived; ++it) arrived = tc::mbar_try(bar[u], parity[u]);
                parity[u] ^= 1u;
                if (!__all_sync(RSFK_FULL, arrived)) {
                    // give up: wait once more (bounded) for the copies still in flight, then leave
#pragma unroll
                    for (int o = 0; o < NBUF; ++o) {
                        const int ob = b + ((o - u + NBUF) % NBUF);
                        if (o != u && ob < n)
                            for (unsigned it = 0; it < tc::WAIT_LIMIT; ++it)
                                if (tc::mbar_try(bar[o], parity[o])) break;
                    }
                    if (lane == 0) atomicExch(error_flag, 1);
                    alive = false;
                    break;
                }
                const float* R = rows + (size_t)u * D;
                float acc = 0.0f;
                for (int k = lane; k < D; k += 32) {
                    const float df = __fsub_rn(R[k], xp[k]);
                    acc = __fmaf_rn(df, df, acc);
                }
                const float dsum = butterfly_sum(acc);
                if (L.beats_threshold(dsum, ci)) changed |= L.try_insert(dsum, ci, K, lane);
                __syncwarp(); // the buffer's row is read; it may be filled again
            }
        }
        if (alive && changed)
            L.store(knn_idx + (size_t)(p - list_row0) * K, knn_dist + (size_t)(p - list_row0) * K, K, lane);
    }
    if (lane == 0 && n_eval) atomicAdd(evaluated, n_eval);
}

bool explore_sweep(Context& ctx, const float* d_points, int N, int D, int K, const int* d_old_idx,
                   int* d_idx, float* d_dist, int row_begin, int row_end, int list_row0)
{
    TraceRange trace("rsfk exploration sweep");
    if (!check_k(ctx, K)) return false;
    if (row_end <= row_begin) return true;
    const ExploreShape shape = explore_shape(D, K);
    const size_t smem = shape.smem;
    if (smem > 200 * 1024) return ctx.fail(RSFK_ERR_UNSUPPORTED, "explore_sweep: D too large");
    long long rows = (long long)row_end - row_begin;
    long long blocks = (rows + shape.warps - 1) / shape.warps;
    if (blocks > ctx.sm_count * 8) blocks = ctx.sm_count * 8;
    unsigned long long* counter = ctx.explore_counter();
    if (!counter) return false;
    const bool vec4 = (D % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_points) & 15) == 0);
    // wide rows: one row per buffer, several buffers per warp (k_explore_wide)
    if (vec4 && K <= 32 && D >= 512 && D <= 1950) {
        const int per_warp = 110 * 1024 / 4 / WIDE_WARPS;              // floats a warp may use: two CTAs per SM
        const int fit = (per_warp - D - WIDE_CAND) / D;
        const int nbuf = fit >= 5 ? 5 : (fit >= 3 ? 3 : 2);
        const int table_slots = 1 << shape.table_log2;
        const int area = nbuf * D > table_slots ? nbuf * D : table_slots;
        const size_t w_smem = sizeof(float) * (size_t)WIDE_WARPS * (D + WIDE_CAND + area);
        long long w_blocks = (rows + WIDE_WARPS - 1) / WIDE_WARPS;
        if (w_blocks > ctx.sm_count * 2) w_blocks = ctx.sm_count * 2;
        int* flag = ctx.error_flag();
        if (!flag) return false;
        auto kern = nbuf == 5 ? k_explore_wide<5> : (nbuf == 3 ? k_explore_wide<3> : k_explore_wide<2>);
        if (!ctx.check(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)w_smem),
                       "explore smem attribute"))
            return false;
        kern<<<(int)w_blocks, 32 * WIDE_WARPS, w_smem, ctx.stream>>>(d_points, N, D, K, d_old_idx, d_idx, d_dist,
                                                                    row_begin, row_end, list_row0, counter,
                                                                    shape.table_log2, area, flag);
        count_launches(1);
        return ctx.check(cudaGetLastError(), "explore launch");
    }
    // long lists of medium rows: rows staged in shared memory by bulk copies (k_explore_staged)
    if (vec4 && K > 32 && K <= 64 && D >= 64 && 32 * D <= (1 << shape.table_log2)) {
        const size_t st_smem = sizeof(float) * (size_t)STAGED_WARPS * (D + (1 << shape.table_log2));
        long long st_blocks = (rows + STAGED_WARPS - 1) / STAGED_WARPS;
        if (st_blocks > ctx.sm_count * 3) st_blocks = ctx.sm_count * 3;
        const int cand_cap = K * K;
        int* cand = (int*)ctx.scratch(Context::EXPLORE_CAND, sizeof(int) * (size_t)st_blocks * STAGED_WARPS * cand_cap);
        int* flag = ctx.error_flag();
        if (!cand || !flag) return false;
        auto kern = k_explore_staged<2>;
        if (!ctx.check(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st_smem),
                       "explore smem attribute"))
            return false;
        kern<<<(int)st_blocks, 32 * STAGED_WARPS, st_smem, ctx.stream>>>(d_points, N, D, K, d_old_idx, d_idx, d_dist,
                                                                        row_begin, row_end, list_row0, counter,
                                                                        shape.table_log2, cand, cand_cap, flag);
        count_launches(1);
        return ctx.check(cudaGetLastError(), "explore launch");
    }
    RSFK_DISPATCH_KPL(K, {
        auto kern = vec4 ? k_explore<KPL, true> : k_explore<KPL, false>;
        if (!ctx.check(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                       "explore smem attribute"))
            return false;
        kern<<<(int)blocks, shape.warps * 32, smem, ctx.stream>>>(d_points, N, D, K, d_old_idx, d_idx, d_dist,
                                                                 row_begin, row_end, list_row0, counter,
                                                                 shape.table_log2);
    });
    count_launches(1);
    return ctx.check(cudaGetLastError(), "explore launch");
}

bool ann_bucket_knn(Context& ctx, const float* d_points, int N, const float* d_queries, int NQ, int D,
                    int K, const TreeResult& tree, int* d_idx, float* d_dist)
{
    TraceRange trace("rsfk query update");
    (void)N;
    if (!check_k(ctx, K)) return false;
    if (NQ <= 0) return true;
    if (tree.n_leaves < 1) return ctx.fail(RSFK_ERR_ARG, "ann_bucket_knn: no tree");
    cudaStream_t st = ctx.stream;
    int* q_leaf = (int*)ctx.scratch(Context::QUERY_LEAF, sizeof(int) * (size_t)NQ);
    int* q_order = (int*)ctx.scratch(Context::QUERY_ORDER, sizeof(int) * (size_t)NQ);
    int* leaf_queries = (int*)ctx.scratch(Context::LEAF_QUERIES, sizeof(int) * (size_t)(tree.n_leaves + 1));
    if (ctx.status != RSFK_OK) return false;
    cudaEvent_t* ev = ctx.next_ann_events();
    if (!ev) return ctx.fail(RSFK_ERR_CUDA, "ann_bucket_knn: cudaEventCreate failed");
    cudaEventRecord(ev[0], st);
    if (!ctx.check(cudaMemsetAsync(leaf_queries, 0, sizeof(int) * (size_t)(tree.n_leaves + 1), st),
                   "clear leaf counts"))
        return false;
    if (!tree_route(ctx, d_points, D, tree, d_queries, NQ, q_leaf, leaf_queries)) return false;
    k_leaf_offsets<<<1, 1024, 0, st>>>(leaf_queries, tree.n_leaves);
    int grid = (NQ + 255) / 256;
    if (grid > ctx.sm_count * 16) grid = ctx.sm_count * 16;
    k_place_queries<<<grid, 256, 0, st>>>(q_leaf, NQ, leaf_queries, q_order);
    count_launches(2);
    cudaEventRecord(ev[1], st);
    // leaf_queries[n_leaves] = number of queries that reached a leaf = entries of q_order
    const size_t smem = sizeof(float) * (size_t)KNN_WARPS * D;
    if (smem > 200 * 1024) return ctx.fail(RSFK_ERR_UNSUPPORTED, "ann_bucket_knn: D too large");
    long long blocks = ((long long)NQ + KNN_WARPS - 1) / KNN_WARPS;
    if (blocks > ctx.sm_count * 8) blocks = ctx.sm_count * 8;
    const bool vec4 = (D % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_points) & 15) == 0);
    // one CTA per leaf with the leaf's rows in shared memory, when they fit twice per SM and
    // leaves receive several queries each; else one warp per query reading rows through L2
    const size_t leaf_smem = sizeof(float) * ((size_t)tree.max_leaf + KNN_WARPS) * D + sizeof(int) * (size_t)tree.max_leaf;
    if (leaf_smem <= 100 * 1024 && (long long)NQ >= 4LL * tree.n_leaves) {
        RSFK_DISPATCH_KPL(K, {
            auto kern = vec4 ? k_ann_leaf<KPL, true> : k_ann_leaf<KPL, false>;
            if (leaf_smem > 48 * 1024 &&
                !ctx.check(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)leaf_smem),
                           "query leaf smem attribute"))
                return false;
            kern<<<tree.n_leaves, KNN_THREADS, leaf_smem, st>>>(d_points, d_queries, D, K, tree.perm, tree.leaf_start,
                                                                tree.leaf_count, leaf_queries, q_order,
                                                                tree.max_leaf, d_idx, d_dist);
        });
        count_launches(1);
        cudaEventRecord(ev[2], st);
        return ctx.check(cudaGetLastError(), "query leaf launch");
    }
    RSFK_DISPATCH_KPL(K, {
        auto kern = vec4 ? k_ann_bucket<KPL, true> : k_ann_bucket<KPL, false>;
        if (smem > 48 * 1024 &&
            !ctx.check(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                       "query bucket smem attribute"))
            return false;
        kern<<<(int)blocks, KNN_THREADS, smem, st>>>(d_points, d_queries, D, K, tree.perm, tree.leaf_start,
                                                     tree.leaf_count, q_leaf, q_order,
                                                     leaf_queries + tree.n_leaves, d_idx, d_dist);
    });
    count_launches(1);
    cudaEventRecord(ev[2], st);
    return ctx.check(cudaGetLastError(), "query bucket launch");
}

bool merge_lists(Context& ctx, long long rows, int K, int G, const int* const* d_idx_lists,
                 const float* const* d_dist_lists, int* d_out_idx, float* d_out_dist)
{
    TraceRange trace("rsfk merge lists");
    if (!check_k(ctx, K)) return false;
    if (G < 1 || G > 16) return ctx.fail(RSFK_ERR_ARG, "merge_lists: between 1 and 16 lists");
    if (rows <= 0) return true;
    MergeArgs a;
    for (int g = 0; g < 16; ++g) {
        a.idx[g] = g < G ? d_idx_lists[g] : nullptr;
        a.dist[g] = g < G ? d_dist_lists[g] : nullptr;
    }
    long long blocks = (rows + KNN_WARPS - 1) / KNN_WARPS;
    if (blocks > ctx.sm_count * 16) blocks = ctx.sm_count * 16;
    RSFK_DISPATCH_KPL(K, (k_merge_lists<KPL><<<(int)blocks, KNN_THREADS, 0, ctx.stream>>>(a, G, rows, K, d_out_idx, d_out_dist)));
    count_launches(1);
    return ctx.check(cudaGetLastError(), "merge_lists launch");
}

} // namespace rsfk

// ---------------------------------------------------------------------------
// Exploration sweep for callers that must not allocate.
//
// A sweep needs a frozen copy of the index lists (every point reads its
// neighbours' OLD rows while rows are being rewritten) and an 8-byte work
// counter.  The other entry points take that memory from the caller or from the
// context's pool (cudaMalloc).  This one keeps it in a fixed array that is part
// of the library image, so the call touches no allocator at all.
// ---------------------------------------------------------------------------
#include "../../include/rsfk_b200.h"

namespace {

constexpr long long STATIC_SNAPSHOT_INTS = RSFK_STATIC_SWEEP_MAX_ENTRIES;
constexpr int STATIC_MAX_DEVICES = 64;

// Snapshot of the index lists, then one 256-byte slot holding the work counter.
// In host code this name is only a handle for cudaGetSymbolAddress; it is not a
// device address and must never be handed to a kernel directly.
static __device__ __align__(256) int g_static_sweep_scratch[STATIC_SNAPSHOT_INTS + 64];

int* g_static_scratch_addr[STATIC_MAX_DEVICES]; // per device, filled on first use
int g_static_sm_count[STATIC_MAX_DEVICES];

int static_fail(int code, const char* msg)
{
    fprintf(stderr, "rsfk_explore_sweep_static: %s\n", msg);
    return code;
}

} // namespace

extern "C" int rsfk_explore_sweep_static(const float* d_points, int N, int D, int K, int* d_idx,
                                         float* d_dist, void* stream)
{
    using namespace rsfk;
    if (!d_points || !d_idx || !d_dist || N <= 0 || D <= 0 || K <= 0)
        return static_fail(RSFK_ERR_ARG, "invalid argument");
    if (K > list_capacity()) return static_fail(RSFK_ERR_UNSUPPORTED, "K above 256 is not supported");
    if ((long long)N * K > STATIC_SNAPSHOT_INTS)
        return static_fail(RSFK_ERR_ARG,
                           "N*K exceeds RSFK_STATIC_SWEEP_MAX_ENTRIES, the capacity of the built-in snapshot "
                           "buffer; use rsfk_dev_explore with a caller-provided snapshot instead");
    const ExploreShape shape = explore_shape(D, K);
    const size_t smem = shape.smem;
    if (smem > 200 * 1024) return static_fail(RSFK_ERR_UNSUPPORTED, "D too large for the sweep kernel");

    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return static_fail(RSFK_ERR_CUDA, cudaGetErrorString(err));
    if (dev < 0 || dev >= STATIC_MAX_DEVICES) return static_fail(RSFK_ERR_ARG, "device ordinal out of range");
    if (g_static_scratch_addr[dev] == nullptr) {
        // one-time set-up for this device (it is current): resolve the device
        // address of the built-in array and read the SM count
        int* addr = nullptr;
        err = cudaGetSymbolAddress((void**)&addr, g_static_sweep_scratch);
        if (err != cudaSuccess || addr == nullptr)
            return static_fail(RSFK_ERR_CUDA, err != cudaSuccess ? cudaGetErrorString(err) : "null symbol address");
        int sms = 0;
        err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (err != cudaSuccess) return static_fail(RSFK_ERR_CUDA, cudaGetErrorString(err));
        g_static_sm_count[dev] = sms > 0 ? sms : 148;
        g_static_scratch_addr[dev] = addr;
    }
    int* snapshot = g_static_scratch_addr[dev];
    unsigned long long* counter = reinterpret_cast<unsigned long long*>(snapshot + STATIC_SNAPSHOT_INTS);
    cudaStream_t st = (cudaStream_t)stream;

    // the array keeps whatever the previous call left: overwrite the part this
    // call reads and zero the counter
    err = cudaMemcpyAsync(snapshot, d_idx, sizeof(int) * (size_t)N * K, cudaMemcpyDeviceToDevice, st);
    if (err == cudaSuccess) err = cudaMemsetAsync(counter, 0, sizeof(unsigned long long), st);
    if (err != cudaSuccess) return static_fail(RSFK_ERR_CUDA, cudaGetErrorString(err));

    long long blocks = ((long long)N + shape.warps - 1) / shape.warps;
    if (blocks > (long long)g_static_sm_count[dev] * 8) blocks = (long long)g_static_sm_count[dev] * 8;
    const bool vec4 = (D % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_points) & 15) == 0);
    RSFK_DISPATCH_KPL(K, {
        auto kern = vec4 ? k_explore<KPL, true> : k_explore<KPL, false>;
        err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err == cudaSuccess) {
            kern<<<(int)blocks, shape.warps * 32, smem, st>>>(d_points, N, D, K, snapshot, d_idx, d_dist, 0, N, 0,
                                                             counter, shape.table_log2);
            err = cudaGetLastError();
        }
    });
    if (err != cudaSuccess) return static_fail(RSFK_ERR_CUDA, cudaGetErrorString(err));
    rsfk::count_launches(1);
    return RSFK_OK;
}
