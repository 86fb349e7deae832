// Shared device helpers of the sm_100a RSFK library: error plumbing, the
// counter hash that draws split pairs, the reference-order reductions and the
// per-warp sorted K-list.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <math_constants.h>

#define RSFK_FULL 0xffffffffu

enum rsfk_status_code {
    RSFK_OK = 0,
    RSFK_ERR_CUDA = 1,        // a CUDA runtime call failed
    RSFK_ERR_ARG = 2,         // invalid argument
    RSFK_ERR_UNSUPPORTED = 3, // feature not built (e.g. K above the list capacity)
    RSFK_ERR_OVERFLOW = 4,    // an internal table was too small
    RSFK_ERR_NOMEM = 5
};

namespace rsfk {

// ---------------------------------------------------------------------------
// Counter hash for split pairs.  Must stay bit-identical to the CPU oracle's
// orc_sample_positions: two distinct positions in [0,count) from
// (seed, depth, segment start).
// ---------------------------------------------------------------------------
__host__ __device__ inline uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__host__ __device__ inline void sample_positions(int seed, int depth, int start, int count,
                                                 int& r1, int& r2)
{
    uint64_t h = mix64(((uint64_t)(uint32_t)seed << 32) ^ (uint64_t)(uint32_t)start);
    h = mix64(h ^ ((uint64_t)(uint32_t)depth * 0xD6E8FEB86659FD93ull));
    uint32_t a = (uint32_t)(h & 0xffffffffu), b = (uint32_t)(h >> 32);
    int p = (int)(a % (uint32_t)count);
    int q = p;
    if (count > 1) q = (int)(((uint32_t)p + 1u + b % (uint32_t)(count - 1)) % (uint32_t)count);
    r1 = p;
    r2 = q;
}

// ---------------------------------------------------------------------------
// Reference-order reductions.  The reference sums D terms as 32 lane-strided
// partial sums (term i goes to lane i%32) combined by an xor butterfly with
// strides 1,2,4,8,16 (reference: src/kernels/compute_knn_from_buckets.cu:205-227).
// Every routine below reproduces exactly that association so that distances
// and projections carry the same bits as the reference's.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float butterfly_sum(float s)
{
    s = __fadd_rn(s, __shfl_xor_sync(RSFK_FULL, s, 1));
    s = __fadd_rn(s, __shfl_xor_sync(RSFK_FULL, s, 2));
    s = __fadd_rn(s, __shfl_xor_sync(RSFK_FULL, s, 4));
    s = __fadd_rn(s, __shfl_xor_sync(RSFK_FULL, s, 8));
    s = __fadd_rn(s, __shfl_xor_sync(RSFK_FULL, s, 16));
    return s;
}

// One halving step of a transposed butterfly: every lane holds 2*H partial
// sums (for 2*H different items); lanes l and l^STRIDE exchange halves so that
// afterwards each holds H sums over the lane pair.  Lanes with the STRIDE bit
// clear keep items [0,H), the others items [H,2H).
template <int H, int STRIDE>
__device__ __forceinline__ void halve_step(float* acc, int lane)
{
    const bool hi = (lane & STRIDE) != 0;
#pragma unroll
    for (int h = 0; h < H; ++h) {
        float send = hi ? acc[h] : acc[h + H];
        float keep = hi ? acc[h + H] : acc[h];
        acc[h] = __fadd_rn(keep, __shfl_xor_sync(RSFK_FULL, send, STRIDE));
    }
}

// 16 items per lane -> lane l ends with the full 32-lane sum of item
// item16_of_lane(l) (lanes l and l^16 hold the same item).
__device__ __forceinline__ float transposed_sum16(float* acc, int lane)
{
    halve_step<8, 1>(acc, lane);
    halve_step<4, 2>(acc, lane);
    halve_step<2, 4>(acc, lane);
    halve_step<1, 8>(acc, lane);
    return __fadd_rn(acc[0], __shfl_xor_sync(RSFK_FULL, acc[0], 16));
}
__device__ __forceinline__ int item16_of_lane(int lane)
{
    return ((lane & 1) << 3) | ((lane & 2) << 1) | ((lane & 4) >> 1) | ((lane & 8) >> 3);
}

// 32 items per lane -> lane l ends with the full sum of item item32_of_lane(l).
__device__ __forceinline__ float transposed_sum32(float* acc, int lane)
{
    halve_step<16, 1>(acc, lane);
    halve_step<8, 2>(acc, lane);
    halve_step<4, 4>(acc, lane);
    halve_step<2, 8>(acc, lane);
    halve_step<1, 16>(acc, lane);
    return acc[0];
}
__device__ __forceinline__ int item32_of_lane(int lane)
{
    return (int)(__brev((unsigned)lane) >> 27);
}

// ---------------------------------------------------------------------------
// (distance, index) ordering.  Distances are non-negative, so their bit
// patterns order like unsigned integers; index -1 (empty) orders last.
// ---------------------------------------------------------------------------
__device__ __forceinline__ bool key_less(float da, int ia, float db, int ib)
{
    return da < db || (da == db && (unsigned)ia < (unsigned)ib);
}

// ---------------------------------------------------------------------------
// A K-list held by one warp, ascending by (distance, index).  Entry e lives in
// register e/32 of lane e%32; entries at or beyond K are (+inf, -1) sentinels.
// ---------------------------------------------------------------------------
template <int KPL>
struct WarpList {
    float d[KPL];
    int i[KPL];
    float thr_d; // entry K-1, the one a new candidate must beat
    int thr_i;

    __device__ __forceinline__ void clear()
    {
#pragma unroll
        for (int r = 0; r < KPL; ++r) { d[r] = CUDART_INF_F; i[r] = -1; }
        thr_d = CUDART_INF_F;
        thr_i = -1;
    }
    __device__ __forceinline__ void refresh_threshold(int K)
    {
        const int e = K - 1;
#pragma unroll
        for (int r = 0; r < KPL; ++r)
            if (r == (e >> 5)) {
                thr_d = __shfl_sync(RSFK_FULL, d[r], e & 31);
                thr_i = __shfl_sync(RSFK_FULL, i[r], e & 31);
            }
    }
    // rows in memory are already canonical
    __device__ __forceinline__ void load(const int* gi, const float* gd, int K, int lane)
    {
        load_raw(gi, gd, K, lane);
        refresh_threshold(K);
    }
    // The loads alone, so that they can be issued early; refresh_threshold() must
    // follow before the list is used.
    __device__ __forceinline__ void load_raw(const int* gi, const float* gd, int K, int lane)
    {
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
            int e = r * 32 + lane;
            d[r] = e < K ? gd[e] : CUDART_INF_F;
            i[r] = e < K ? gi[e] : -1;
        }
    }
    __device__ __forceinline__ void store(int* gi, float* gd, int K, int lane) const
    {
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
            int e = r * 32 + lane;
            if (e < K) { gd[e] = d[r]; gi[e] = i[r]; }
        }
    }
    __device__ __forceinline__ bool beats_threshold(float cd, int ci) const
    {
        return key_less(cd, ci, thr_d, thr_i);
    }
    __device__ __forceinline__ bool contains(int ci) const
    {
        bool hit = false;
#pragma unroll
        for (int r = 0; r < KPL; ++r) hit |= (i[r] == ci);
        return __any_sync(RSFK_FULL, hit);
    }
    // Warp-uniform call: (cd, ci) identical in all lanes.  Inserts unless the
    // candidate does not beat entry K-1 or its index is already present.
    __device__ __forceinline__ bool try_insert(float cd, int ci, int K, int lane)
    {
        if (!beats_threshold(cd, ci)) return false;
        if (contains(ci)) return false;
        int pos = 0;
#pragma unroll
        for (int r = 0; r < KPL; ++r)
            pos += __popc(__ballot_sync(RSFK_FULL, key_less(d[r], i[r], cd, ci)));
#pragma unroll
        for (int r = KPL - 1; r >= 0; --r) {
            float ud = __shfl_up_sync(RSFK_FULL, d[r], 1);
            int ui = __shfl_up_sync(RSFK_FULL, i[r], 1);
            if (r > 0) {
                float pd = __shfl_sync(RSFK_FULL, d[r - 1], 31);
                int pi = __shfl_sync(RSFK_FULL, i[r - 1], 31);
                if (lane == 0) { ud = pd; ui = pi; }
            }
            int e = r * 32 + lane;
            if (e > pos) { d[r] = ud; i[r] = ui; }
            else if (e == pos) { d[r] = cd; i[r] = ci; }
            if (e >= K) { d[r] = CUDART_INF_F; i[r] = -1; }
        }
        refresh_threshold(K);
        return true;
    }
};

// ---------------------------------------------------------------------------
// Squared distances from the query (xq, shared memory) to rows row0 .. row0+n-1
// (n <= 32) of X[.][D] in shared memory, in the summation order of
// explore_dist32_*; lane l returns the distance of row row0 + item.
__device__ __forceinline__ float leaf_dist32_scalar(const float* X, int D, const float* xq, int row0, int n,
                                                    int lane, int& item)
{
    float acc[32];
    const float* row[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) {
        acc[c] = 0.0f;
        row[c] = X + (size_t)(row0 + min(c, n - 1)) * D;
    }
    for (int k = lane; k < D; k += 32) {
        const float x = xq[k];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            const float df = __fsub_rn(row[c][k], x);
            acc[c] = __fmaf_rn(df, df, acc[c]);
        }
    }
    const float dsum = transposed_sum32(acc, lane);
    item = item32_of_lane(lane);
    return dsum;
}

__device__ __forceinline__ float leaf_dist32_vec4(const float* X, int D, const float* xq, int row0, int n,
                                                  int lane, int& item)
{
    const int g = lane >> 3, t = lane & 7;
    const float4* xq4 = reinterpret_cast<const float4*>(xq);
    const int D4 = D >> 2;
    float acc[8][4];
    const float4* row[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        row[j] = reinterpret_cast<const float4*>(X) + (size_t)(row0 + min(4 * j + g, n - 1)) * D4;
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[j][q] = 0.0f;
    }
    for (int k4 = t; k4 < D4; k4 += 8) {
        const float4 x = xq4[k4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 v = row[j][k4];
            float df;
            df = __fsub_rn(v.x, x.x); acc[j][0] = __fmaf_rn(df, df, acc[j][0]);
            df = __fsub_rn(v.y, x.y); acc[j][1] = __fmaf_rn(df, df, acc[j][1]);
            df = __fsub_rn(v.z, x.z); acc[j][2] = __fmaf_rn(df, df, acc[j][2]);
            df = __fsub_rn(v.w, x.w); acc[j][3] = __fmaf_rn(df, df, acc[j][3]);
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
    item = 4 * t + g;
    return mine;
}

} // namespace rsfk
