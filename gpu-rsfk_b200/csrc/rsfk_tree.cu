// Random sample tree for sm_100a.
//
// The points of a node are one contiguous segment of a permutation array; a
// split is a stable partition of that segment (left side first), so a leaf's
// bucket is simply perm[start, start+count) and no per-point parent/depth
// bookkeeping exists.  Each level runs two kernels over the level's work
// chunks (CHUNK consecutive positions of one node):
//
//   project : side bit of every active point (n.x < c  =>  right) as one
//             32-bit mask per 32 positions, plus the chunk's left count; the
//             CTA that finishes the last chunk of a node then decides the node:
//             left total and per-chunk exclusive prefix, children, leaves and
//             the next level's chunk list;
//   scatter : stable partition into the other permutation buffer; points
//             whose child is a leaf are also written to the final array.
//
// The sizes of a level (nodes, chunks) live in device memory and the kernels
// loop over them, so the host enqueues several levels at a time and looks at
// the level mailbox once per batch.
//
// The rules (which side is right, when a child is a leaf, when a small child
// dissolves into its sibling) follow the reference's level kernels:
// src/kernels/build_tree_check_points_side.cu:131-151,
// src/kernels/build_tree_update_parents.cu:64-75,106-135,
// src/kernels/build_tree_create_nodes.cu:88-104, src/kernels/create_node.cu:60-66,120-134.
// The arithmetic keeps the reference's summation order so that the side of
// every point is bit-for-bit the reference's for the same split pair.
#include <chrono>
#include <cstdlib>
#include <cstring>

#include "rsfk_context.h"

namespace rsfk {

constexpr int CHUNK = 512;           // positions per work chunk
constexpr int CHUNK_WORDS = CHUNK / 32;
static_assert(CHUNK % 32 == 0 && CHUNK_WORDS <= 32, "one warp scans the words of a chunk");
constexpr int TREE_THREADS = 256;

struct NodeSplit {
    int n_left;
    int flags; // bit0: left side is final (leaf), bit1: right side is final
};

// ---------------------------------------------------------------------------
__device__ __forceinline__ void node_pair(const Node& nd, const int* __restrict__ perm,
                                          const int4* __restrict__ table, int n_table, int seed,
                                          int level, int& p1, int& p2)
{
    if (table != nullptr && nd.tbl >= 0 && nd.tbl < n_table) {
        int4 t = table[nd.tbl];
        p1 = t.x;
        p2 = t.y;
        return;
    }
    int r1, r2;
    sample_positions(seed, level, nd.pstart, nd.pcount, r1, r2);
    p1 = perm[nd.pstart + r1];
    p2 = perm[nd.pstart + r2];
}

// Hyperplane of the chunk's node into shared memory: normal sN[D] and offset.
// Root offset is a serial sum, every other node's is lane-strided + butterfly.
__device__ __forceinline__ float load_hyperplane(const float* __restrict__ pts, int D, int p1, int p2,
                                                 bool is_root, float* sN, float* sC)
{
    const float* x1 = pts + (size_t)p1 * D;
    const float* x2 = pts + (size_t)p2 * D;
    for (int k = threadIdx.x; k < D; k += blockDim.x) sN[k] = __fsub_rn(x1[k], x2[k]);
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float c = 0.0f;
        if (is_root) {
            if (lane == 0)
                for (int k = 0; k < D; ++k)
                    c = __fadd_rn(c, __fmul_rn(__fmul_rn(sN[k], __fadd_rn(x1[k], x2[k])), 0.5f));
            c = __shfl_sync(RSFK_FULL, c, 0);
        } else {
            for (int k = lane; k < D; k += 32)
                c = __fadd_rn(c, __fmul_rn(__fmul_rn(sN[k], __fadd_rn(x1[k], x2[k])), 0.5f));
            c = butterfly_sum(c);
        }
        if (lane == 0) *sC = c;
    }
    __syncthreads();
    return *sC;
}

// ---------------------------------------------------------------------------
// Side bits of up to 32 rows against the hyperplane (sN[D] in shared memory, c).
// Lane q < here holds the id of row q in my_id.  Returns the mask of rows with
// n.x < c.  Both variants accumulate term k in "virtual lane" k%32 and combine
// the 32 partial sums in the xor-butterfly order, so the projection carries the
// bits of the reference's warp-per-point sum.
// ---------------------------------------------------------------------------

// Scalar loads: the warp takes four rows at a time, lane l owns terms l, l+32, ...
__device__ __forceinline__ unsigned project_group_scalar(const float* __restrict__ pts, int D,
                                                         const float* sN, float c, int my_id, int here,
                                                         int lane)
{
    unsigned mask = 0;
    for (int q = 0; q < here; q += 4) {
        float acc[4];
        const float* row[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int id = __shfl_sync(RSFK_FULL, my_id, min(q + u, here - 1));
            row[u] = pts + (size_t)id * D;
            acc[u] = 0.0f;
        }
        for (int k = lane; k < D; k += 32) {
            const float nk = sN[k];
            float x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) x[u] = __ldg(row[u] + k);
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[u] = __fmaf_rn(nk, x[u], acc[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float pr = butterfly_sum(acc[u]);
            if (q + u < here && pr < c) mask |= 1u << (q + u);
        }
    }
    return mask;
}

// 16-byte loads (D % 4 == 0, 16-byte aligned rows): eight lanes share a row,
// lane g of the eight owns terms 4g..4g+3 (+32, +64, ...), i.e. virtual lanes
// 4g..4g+3; sixteen rows are in flight per warp.
__device__ __forceinline__ unsigned project_group_vec4(const float* __restrict__ pts, int D,
                                                       const float* sN, float c, int my_id, int here,
                                                       int lane)
{
    const int g = lane & 7, rr = lane >> 3;
    const float4* sN4 = reinterpret_cast<const float4*>(sN);
    const int D4 = D >> 2;
    unsigned mask = 0;
    for (int q0 = 0; q0 < here; q0 += 16) {
        float acc[4][4];
        const float4* row[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int q = q0 + 4 * r + rr;
            const int id = __shfl_sync(RSFK_FULL, my_id, min(q, here - 1));
            row[r] = reinterpret_cast<const float4*>(pts + (size_t)id * D);
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[r][j] = 0.0f;
        }
#pragma unroll 2
        for (int k4 = g; k4 < D4; k4 += 8) {
            const float4 n = sN4[k4];
            float4 x[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) x[r] = __ldg(row[r] + k4);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                acc[r][0] = __fmaf_rn(n.x, x[r].x, acc[r][0]);
                acc[r][1] = __fmaf_rn(n.y, x[r].y, acc[r][1]);
                acc[r][2] = __fmaf_rn(n.z, x[r].z, acc[r][2]);
                acc[r][3] = __fmaf_rn(n.w, x[r].w, acc[r][3]);
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            float t = __fadd_rn(__fadd_rn(acc[r][0], acc[r][1]), __fadd_rn(acc[r][2], acc[r][3]));
            t = __fadd_rn(t, __shfl_xor_sync(RSFK_FULL, t, 1));
            t = __fadd_rn(t, __shfl_xor_sync(RSFK_FULL, t, 2));
            t = __fadd_rn(t, __shfl_xor_sync(RSFK_FULL, t, 4));
            const int q = q0 + 4 * r + rr;
            const unsigned bal = __ballot_sync(RSFK_FULL, g == 0 && q < here && t < c);
            // lanes 0, 8, 16, 24 carry rows q0+4r+0..3
            mask |= (((bal >> 0) & 1u) | (((bal >> 8) & 1u) << 1) | (((bal >> 16) & 1u) << 2) |
                     (((bal >> 24) & 1u) << 3)) << (q0 + 4 * r);
        }
    }
    return mask;
}

__device__ __forceinline__ unsigned project_group(const float* __restrict__ pts, int D, bool vec4,
                                                  const float* sN, float c, int my_id, int here, int lane)
{
    return vec4 ? project_group_vec4(pts, D, sN, c, my_id, here, lane)
                : project_group_scalar(pts, D, sN, c, my_id, here, lane);
}

// ---------------------------------------------------------------------------
// decide: what becomes of a node once all its chunks are projected (one warp).
// ---------------------------------------------------------------------------
__device__ __forceinline__ int emit_leaf(int start, int count, int* leaf_start, int* leaf_count,
                                         int leaf_cap, LevelCounters* cnt)
{
    int slot = atomicAdd(&cnt->n_leaves, 1);
    if (slot < leaf_cap) {
        leaf_start[slot] = start;
        leaf_count[slot] = count;
    } else {
        cnt->error = RSFK_ERR_OVERFLOW;
    }
    atomicMax(&cnt->max_leaf, count);
    atomicMin(&cnt->min_leaf, count);
    atomicAdd(&cnt->leaf_sq, (unsigned long long)count * (unsigned long long)count);
    return slot;
}

// A new row of the tree index (lane 0 only), or 0 when no index is kept.
__device__ __forceinline__ int new_record(int4* records, int rec_cap, LevelCounters* cnt)
{
    if (records == nullptr) return 0;
    const int r = atomicAdd(&cnt->n_recs, 1);
    if (r >= rec_cap) {
        cnt->error = RSFK_ERR_OVERFLOW;
        return 0;
    }
    return r;
}

// Child refs of a row: a node with one child sends both sides to it.
__device__ __forceinline__ void file_refs(int4* records, int rec, int n_children, const int* ref)
{
    if (records == nullptr) return;
    records[rec].z = ref[0];
    records[rec].w = n_children == 2 ? ref[1] : ref[0];
}

// Children of a node whose stable partition put n_left points on the left.
struct Children {
    int n;            // 1 or 2
    int start[2], count[2];
    int pstart[2], pcount[2]; // segment the child's own split pair is drawn from
    int side[2];      // which side of the parent the child (or the survivor of a merge) is
    bool leaf[2];
    int final_flags;  // bit0: left points are final, bit1: right points are final
};

__device__ __forceinline__ Children decide_children(int start, int count, int nL, int min_children,
                                                    int max_children)
{
    Children c;
    const int nR = count - nL;
    if (nL > 0 && nR > 0 && nL >= min_children && nR >= min_children) {
        c.n = 2;
        c.start[0] = c.pstart[0] = start;      c.count[0] = c.pcount[0] = nL; c.side[0] = 0;
        c.start[1] = c.pstart[1] = start + nL; c.count[1] = c.pcount[1] = nR; c.side[1] = 1;
        c.leaf[0] = nL <= max_children - 2;
        c.leaf[1] = nR <= max_children - 2;
    } else if (nL > 0 && nR > 0) {
        // the side with fewer than min_children points dissolves into the other,
        // which keeps the split pair drawn from its own segment
        int keep = (nL < min_children) ? 1 : 0;
        if (nL < min_children && nR < min_children) keep = 0;
        c.n = 1;
        c.start[0] = start; c.count[0] = count;
        c.pstart[0] = keep ? start + nL : start;
        c.pcount[0] = keep ? nR : nL;
        c.side[0] = keep;
        c.leaf[0] = count <= max_children;
        c.leaf[1] = c.leaf[0];
    } else {
        c.n = 1;
        c.start[0] = c.pstart[0] = start; c.count[0] = c.pcount[0] = count;
        c.side[0] = nL > 0 ? 0 : 1;
        c.leaf[0] = count <= max_children - 2;
        c.leaf[1] = c.leaf[0];
    }
    c.final_flags = 0;
    return c;
}

__device__ __forceinline__ int child_table_row(const int4* __restrict__ table, int n_table, int tbl, int side)
{
    if (table == nullptr || tbl < 0 || tbl >= n_table) return -1;
    const int4 t = table[tbl];
    return side ? t.w : t.z;
}

// Everything a level kernel needs besides the points.
struct LevelArgs {
    const int* perm;            // this level's permutation
    const Node* nodes;          // this level's open nodes
    const int* chunk_node;      // node of every work chunk
    unsigned* side_bits;
    int* chunk_left;            // left count per chunk, then the exclusive prefix inside the node
    int* node_done;             // chunks of a node projected so far (all zero between levels)
    Node* nodes_out;
    int node_cap;
    int* chunk_node_out;
    int chunk_cap;
    NodeSplit* split;
    int* leaf_start;
    int* leaf_count;
    int leaf_cap;
    Node* small_nodes;
    int small_cap, small_limit;
    LevelCounters* cnt;
    const int4* table;
    int n_table;
    int seed, level;
    int min_children, max_children;
    int4* records;
    int rec_cap;
};

// One warp; every chunk of the node has posted its left count.
__device__ __forceinline__ void decide_node(const LevelArgs& a, int node, const Node& nd, int lane)
{
    LevelCounters* cnt = a.cnt;
    LevelState* next = &cnt->lvl[(a.level + 1) % 3];
    const int n_chunks = (nd.count + CHUNK - 1) / CHUNK;
    // left total; chunk_left becomes the exclusive prefix inside the node.  Eight rounds of
    // loads are requested together: a node of the first levels has thousands of chunks and
    // one warp walks them, so the loads must not wait for one another.
    int carry = 0;
    for (int c0 = 0; c0 < n_chunks; c0 += 32 * 8) {
        int v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int c = c0 + 32 * u + lane;
            v[u] = c < n_chunks ? __ldcg(a.chunk_left + nd.chunk_base + c) : 0;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int c = c0 + 32 * u + lane;
            if (c0 + 32 * u >= n_chunks) break; // warp-uniform
            int incl = v[u];
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                int t = __shfl_up_sync(RSFK_FULL, incl, s);
                if (lane >= s) incl += t;
            }
            if (c < n_chunks) a.chunk_left[nd.chunk_base + c] = carry + incl - v[u];
            carry += __shfl_sync(RSFK_FULL, incl, 31);
        }
    }
    const int nL = carry;
    const Children ch = decide_children(nd.start, nd.count, nL, a.min_children, a.max_children);

    // a child's points are final (copied to perm_final by the scatter) when it
    // is a leaf or small enough to be finished inside one CTA
    int flags = 0;
    int ref[2] = {0, 0}; // lane 0: where each child went (row, or -1-leaf slot)
    for (int k = 0; k < ch.n; ++k) {
        const bool small = !ch.leaf[k] && ch.count[k] <= a.small_limit;
        const bool fin = ch.leaf[k] || small;
        if (fin) flags |= (ch.n == 2) ? (1 << k) : 3;
        if (ch.leaf[k]) {
            if (lane == 0)
                ref[k] = -1 - emit_leaf(ch.start[k], ch.count[k], a.leaf_start, a.leaf_count, a.leaf_cap, cnt);
            continue;
        }
        Node o;
        o.start = ch.start[k];   o.count = ch.count[k];
        o.pstart = ch.pstart[k]; o.pcount = ch.pcount[k];
        o.tbl = child_table_row(a.table, a.n_table, nd.tbl, ch.side[k]);
        o.chunk_base = 0;
        o.level = a.level + 1;
        o.rec = 0;
        // an only child takes over its parent's row: both sides of the parent lead to it, so a
        // query loses nothing by starting at the child's split, and a node that fails to split
        // again and again (coincident points) does not use up a row per attempt
        if (lane == 0) ref[k] = o.rec = (ch.n == 1) ? nd.rec : new_record(a.records, a.rec_cap, cnt);
        if (small) {
            if (lane == 0) {
                const int slot = atomicAdd(&cnt->n_small, 1);
                if (slot < a.small_cap) a.small_nodes[slot] = o;
                else cnt->error = RSFK_ERR_OVERFLOW;
            }
            continue;
        }
        const int nch = (ch.count[k] + CHUNK - 1) / CHUNK;
        int slot = 0, cb = 0;
        if (lane == 0) {
            slot = atomicAdd(&next->n_nodes, 1);
            cb = atomicAdd(&next->n_chunks, nch);
            atomicAdd(&next->active, ch.count[k]);
        }
        slot = __shfl_sync(RSFK_FULL, slot, 0);
        cb = __shfl_sync(RSFK_FULL, cb, 0);
        if (slot >= a.node_cap || cb + nch > a.chunk_cap) {
            if (lane == 0) cnt->error = RSFK_ERR_OVERFLOW;
            continue;
        }
        if (lane == 0) {
            o.chunk_base = cb;
            a.nodes_out[slot] = o;
        }
        for (int c = lane; c < nch; c += 32) a.chunk_node_out[cb + c] = slot;
    }
    if (lane == 0) {
        a.split[node].n_left = nL;
        a.split[node].flags = flags;
        if (ch.n == 2 || ch.leaf[0]) file_refs(a.records, nd.rec, ch.n, ref); // else the child rewrites the row
    }
}

// Start of a level kernel: the sizes of this level; one thread clears the state two
// levels ahead (nobody reads or writes it during this level) and books the level.
__device__ __forceinline__ LevelState level_begin(const LevelArgs& a)
{
    LevelCounters* cnt = a.cnt;
    const LevelState ls = cnt->lvl[a.level % 3];
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        LevelState* far = &cnt->lvl[(a.level + 2) % 3];
        far->n_nodes = 0; far->n_chunks = 0; far->active = 0;
        if (ls.n_nodes > 0) {
            cnt->lvl_active += (unsigned long long)ls.active;
            cnt->lvl_nodes += (unsigned long long)ls.n_nodes;
            cnt->last_depth = a.level + 1;
        }
        if (a.level < LEVEL_HISTORY) cnt->level_chunks[a.level] = ls.n_chunks;
    }
    return ls;
}

// End of a chunk (all threads): post the chunk's left count; the CTA that posts the
// last chunk of a node decides the node.  sLast is a shared flag.
__device__ __forceinline__ void chunk_done(const LevelArgs& a, int chunk, int node, const Node& nd, int left,
                                           int* sLast)
{
    if (threadIdx.x == 0) {
        a.chunk_left[chunk] = left;
        __threadfence();
        const int nch = (nd.count + CHUNK - 1) / CHUNK;
        *sLast = (atomicAdd(&a.node_done[node], 1) == nch - 1) ? 1 : 0;
    }
    __syncthreads();
    if (*sLast && threadIdx.x < 32) {
        __threadfence();
        decide_node(a, node, nd, threadIdx.x);
        if (threadIdx.x == 0) a.node_done[node] = 0;
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------
// project, any D: one warp per point, four (or sixteen) points in flight per warp.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(TREE_THREADS)
k_project_wide(const float* __restrict__ pts, int D, int vec4, LevelArgs a)
{
    extern __shared__ float4 smem4[];
    float* sN = reinterpret_cast<float*>(smem4);
    __shared__ float sC;
    __shared__ int sPair[2];
    __shared__ int sLeft;
    __shared__ int sLast;

    const LevelState ls = level_begin(a);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int chunk = blockIdx.x; chunk < ls.n_chunks; chunk += gridDim.x) {
        const int node = a.chunk_node[chunk];
        const Node nd = a.nodes[node];
        const int off = (chunk - nd.chunk_base) * CHUNK;
        const int cnt = min(CHUNK, nd.count - off);
        if (threadIdx.x == 0) {
            int p1, p2;
            node_pair(nd, a.perm, a.table, a.n_table, a.seed, a.level, p1, p2);
            sPair[0] = p1;
            sPair[1] = p2;
            sLeft = 0;
            if (a.records != nullptr && off == 0) { // the node's first chunk files the split pair
                a.records[nd.rec].x = p1;
                a.records[nd.rec].y = p2;
            }
        }
        __syncthreads();
        const float c = load_hyperplane(pts, D, sPair[0], sPair[1], a.level == 0, sN, &sC);

        const int* ids = a.perm + nd.start + off;
        int left_total = 0;
        for (int w = warp; w * 32 < cnt; w += n_warps) {
            const int base = w * 32;
            const int here = min(32, cnt - base);
            const int my_id = lane < here ? ids[base + lane] : -1;
            const unsigned mask = project_group(pts, D, vec4 != 0, sN, c, my_id, here, lane);
            if (lane == 0) {
                a.side_bits[(size_t)chunk * CHUNK_WORDS + w] = mask;
                left_total += here - __popc(mask);
            }
        }
        if (lane == 0 && left_total) atomicAdd(&sLeft, left_total);
        __syncthreads();
        chunk_done(a, chunk, node, nd, sLeft, &sLast);
    }
}

// ---------------------------------------------------------------------------
// project, D <= 16: one thread per point.  Lanes >= D of the reference's
// 32-lane sum hold zero, and adding zero changes no comparison, so only
// VL = next power of two >= D partial sums are kept and combined in the
// butterfly's order.
// ---------------------------------------------------------------------------
template <int VL>
__global__ void __launch_bounds__(TREE_THREADS)
k_project_small(const float* __restrict__ pts, int D, LevelArgs a)
{
    __shared__ float sN[VL];
    __shared__ float sC;
    __shared__ int sPair[2];
    __shared__ int sLeft;
    __shared__ int sLast;

    const LevelState ls = level_begin(a);
    const int lane = threadIdx.x & 31;
    for (int chunk = blockIdx.x; chunk < ls.n_chunks; chunk += gridDim.x) {
        const int node = a.chunk_node[chunk];
        const Node nd = a.nodes[node];
        const int off = (chunk - nd.chunk_base) * CHUNK;
        const int cnt = min(CHUNK, nd.count - off);
        if (threadIdx.x == 0) {
            int p1, p2;
            node_pair(nd, a.perm, a.table, a.n_table, a.seed, a.level, p1, p2);
            sPair[0] = p1;
            sPair[1] = p2;
            sLeft = 0;
            if (a.records != nullptr && off == 0) { // the node's first chunk files the split pair
                a.records[nd.rec].x = p1;
                a.records[nd.rec].y = p2;
            }
        }
        __syncthreads();
        const float c = load_hyperplane(pts, D, sPair[0], sPair[1], a.level == 0, sN, &sC);

        const int* ids = a.perm + nd.start + off;
        int left_total = 0;
        for (int base = (threadIdx.x >> 5) * 32; base < cnt; base += blockDim.x) {
            const int i = base + lane;
            bool right = false;
            if (i < cnt) {
                const float* x = pts + (size_t)ids[i] * D;
                float acc[VL];
#pragma unroll
                for (int k = 0; k < VL; ++k) acc[k] = k < D ? __fmaf_rn(sN[k], __ldg(x + k), 0.0f) : 0.0f;
#pragma unroll
                for (int stride = 1; stride < VL; stride <<= 1)
#pragma unroll
                    for (int k = 0; k < VL; k += 2 * stride) acc[k] = __fadd_rn(acc[k], acc[k + stride]);
                right = acc[0] < c;
            }
            const unsigned mask = __ballot_sync(RSFK_FULL, right);
            if (lane == 0) {
                a.side_bits[(size_t)chunk * CHUNK_WORDS + (base >> 5)] = mask;
                left_total += min(32, cnt - base) - __popc(mask);
            }
        }
        if (lane == 0 && left_total) atomicAdd(&sLeft, left_total);
        __syncthreads();
        chunk_done(a, chunk, node, nd, sLeft, &sLast);
    }
}

// ---------------------------------------------------------------------------
// scatter: stable partition of one chunk.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(TREE_THREADS)
k_scatter(const int* __restrict__ perm_in, int* __restrict__ perm_out, int* __restrict__ perm_final,
          const Node* __restrict__ nodes, const int* __restrict__ chunk_node,
          const unsigned* __restrict__ side_bits, const int* __restrict__ chunk_lprefix,
          const NodeSplit* __restrict__ split, const LevelCounters* counters, int level,
          volatile LevelMail* mail, int seq)
{
    __shared__ unsigned sMask[CHUNK_WORDS];
    __shared__ int sWordLeft[CHUNK_WORDS];

    // Every node of the level is decided (stream order): post the next level's sizes
    // to the host mailbox.
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        const LevelState* next = &counters->lvl[(level + 1) % 3];
        mail->n_nodes = next->n_nodes;
        mail->n_chunks = next->n_chunks;
        mail->active = next->active;
        mail->n_small = counters->n_small;
        mail->error = counters->error;
        __threadfence_system();
        mail->seq = seq;
    }

    const int n_chunks = counters->lvl[level % 3].n_chunks;
    for (int chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
        const int node = chunk_node[chunk];
        const Node nd = nodes[node];
        const NodeSplit sp = split[node];
        const int off = (chunk - nd.chunk_base) * CHUNK;
        const int cnt = min(CHUNK, nd.count - off);
        const int lprefix = chunk_lprefix[chunk];

        if (threadIdx.x < 32) {
            const int w = threadIdx.x;
            const int here = max(0, min(32, cnt - w * 32));
            const unsigned valid = here >= 32 ? 0xffffffffu : ((1u << here) - 1u);
            const unsigned m = here > 0 ? (side_bits[(size_t)chunk * CHUNK_WORDS + w] & valid) : 0u;
            const int lefts = __popc(~m & valid);
            int incl = lefts;
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                int t = __shfl_up_sync(RSFK_FULL, incl, s);
                if (w >= s) incl += t;
            }
            if (w < CHUNK_WORDS) { // the scan runs on all 32 lanes; a chunk has CHUNK_WORDS words
                sMask[w] = m;
                sWordLeft[w] = incl - lefts;
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
            const int w = i >> 5, b = i & 31;
            const unsigned m = sMask[w];
            const bool right = (m >> b) & 1u;
            const int lrank = sWordLeft[w] + __popc(~m & ((1u << b) - 1u));
            const int lefts_before = lprefix + lrank;
            const int dest = right ? nd.start + sp.n_left + (off + i - lefts_before)
                                   : nd.start + lefts_before;
            const int id = perm_in[nd.start + off + i];
            perm_out[dest] = id;
            if (sp.flags & (right ? 2 : 1)) perm_final[dest] = id;
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// subtree: one CTA finishes a node of at most SUB_MAX points, all its levels,
// without leaving the SM: ids ping-pong in shared memory, rows are read from
// global memory (L2 after the first level).  Same rules and arithmetic as the
// level kernels, so the buckets are identical to a level-synchronous build.
// ---------------------------------------------------------------------------
constexpr int SUB_MAX = 2048;        // largest node a CTA takes
constexpr int SUB_NODES = 128;       // open nodes a CTA can hold per level
constexpr int SUB_GROUPS = SUB_MAX / 32 + SUB_NODES;

struct SubNode {
    int start, count;   // relative to the CTA's segment
    int pstart, pcount; // relative
    int tbl;
    int rec;            // row of the tree index
};

__global__ void __launch_bounds__(TREE_THREADS, 4)
k_subtree(const float* __restrict__ pts, int D, int* __restrict__ perm_final,
          const Node* __restrict__ small_nodes, int* __restrict__ leaf_start,
          int* __restrict__ leaf_count, int leaf_cap, LevelCounters* __restrict__ cnt,
          const int4* __restrict__ table, int n_table, int seed, int min_children, int max_children,
          int max_depth, int vec4, int4* __restrict__ records, int rec_cap)
{
    extern __shared__ float4 smem4[]; // per-warp normal vectors: n_warps * D floats
    float* smem = reinterpret_cast<float*>(smem4);
    __shared__ int sIds[2][SUB_MAX];
    __shared__ unsigned sMask[SUB_GROUPS];
    __shared__ int sGroupNode[SUB_GROUPS];
    __shared__ SubNode sOpen[2][SUB_NODES];
    __shared__ int sGroupBase[SUB_NODES];
    __shared__ int sCount[2];          // open nodes of the next level, total groups

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    float* sN = smem + (size_t)warp * D;
    const Node root = small_nodes[blockIdx.x];
    int* seg = perm_final + root.start;

    for (int i = threadIdx.x; i < root.count; i += blockDim.x) sIds[0][i] = seg[i];
    if (threadIdx.x == 0) {
        SubNode r;
        r.start = 0; r.count = root.count;
        r.pstart = root.pstart - root.start; r.pcount = root.pcount;
        r.tbl = root.tbl;
        r.rec = root.rec;
        sOpen[0][0] = r;
    }
    int n_open = 1, cur = 0, level = root.level;
    unsigned long long my_active = 0, my_nodes = 0;
    __syncthreads();

    while (n_open > 0) {
        if (level + 1 >= max_depth) {
            // depth limit: open nodes become leaves of at most max_children points
            for (int i = warp; i < n_open; i += n_warps) {
                const SubNode nd = sOpen[cur][i];
                for (int k = lane; k < nd.count; k += 32) seg[nd.start + k] = sIds[cur][nd.start + k];
                if (lane == 0) {
                    const int piece = max(1, max_children);
                    const int q = (nd.count + piece - 1) / piece;
                    int first = 0;
                    for (int j = 0; j < q; ++j) {
                        int a = (int)((long long)nd.count * j / q), b = (int)((long long)nd.count * (j + 1) / q);
                        const int slot = emit_leaf(root.start + nd.start + a, b - a, leaf_start, leaf_count, leaf_cap, cnt);
                        if (j == 0) first = slot;
                    }
                    if (records != nullptr) // no split: queries go to the first piece
                        records[nd.rec] = make_int4(-1, -1, -1 - first, -1 - first);
                }
            }
            break;
        }
        // ---- group list: 32 consecutive positions of one open node ----------
        if (warp == 0) {
            int carry = 0;
            for (int i0 = 0; i0 < n_open; i0 += 32) {
                const int i = i0 + lane;
                const int g = i < n_open ? (sOpen[cur][i].count + 31) >> 5 : 0;
                int incl = g;
#pragma unroll
                for (int s = 1; s < 32; s <<= 1) {
                    int t = __shfl_up_sync(RSFK_FULL, incl, s);
                    if (lane >= s) incl += t;
                }
                if (i < n_open) sGroupBase[i] = carry + incl - g;
                carry += __shfl_sync(RSFK_FULL, incl, 31);
            }
            if (lane == 0) { sCount[0] = 0; sCount[1] = carry; }
        }
        __syncthreads();
        const int n_groups = sCount[1];
        for (int i = warp; i < n_open; i += n_warps) {
            const int g0 = sGroupBase[i], ng = (sOpen[cur][i].count + 31) >> 5;
            for (int g = lane; g < ng; g += 32) sGroupNode[g0 + g] = i;
            if (lane == 0) { my_active += sOpen[cur][i].count; my_nodes += 1; }
        }
        __syncthreads();
        // ---- projection: one warp per group ---------------------------------
        for (int g = warp; g < n_groups; g += n_warps) {
            const int i = sGroupNode[g];
            const SubNode nd = sOpen[cur][i];
            const int off = (g - sGroupBase[i]) * 32;
            const int here = min(32, nd.count - off);
            int p1, p2;
            if (table != nullptr && nd.tbl >= 0 && nd.tbl < n_table) {
                const int4 t = table[nd.tbl];
                p1 = t.x; p2 = t.y;
            } else {
                int r1, r2;
                sample_positions(seed, level, root.start + nd.pstart, nd.pcount, r1, r2);
                p1 = sIds[cur][nd.pstart + r1];
                p2 = sIds[cur][nd.pstart + r2];
            }
            if (records != nullptr && off == 0 && lane == 0) {
                records[nd.rec].x = p1;
                records[nd.rec].y = p2;
            }
            const float* x1 = pts + (size_t)p1 * D;
            const float* x2 = pts + (size_t)p2 * D;
            float c = 0.0f;
            __syncwarp();
            if (level == 0) {
                for (int k = lane; k < D; k += 32) sN[k] = __fsub_rn(__ldg(x1 + k), __ldg(x2 + k));
                __syncwarp();
                if (lane == 0)
                    for (int k = 0; k < D; ++k)
                        c = __fadd_rn(c, __fmul_rn(__fmul_rn(sN[k], __fadd_rn(__ldg(x1 + k), __ldg(x2 + k))), 0.5f));
                c = __shfl_sync(RSFK_FULL, c, 0);
            } else {
                for (int k = lane; k < D; k += 32) {
                    const float a = __ldg(x1 + k), b = __ldg(x2 + k);
                    const float nk = __fsub_rn(a, b);
                    sN[k] = nk;
                    c = __fadd_rn(c, __fmul_rn(__fmul_rn(nk, __fadd_rn(a, b)), 0.5f));
                }
                c = butterfly_sum(c);
            }
            __syncwarp();
            const int my_id = lane < here ? sIds[cur][nd.start + off + lane] : -1;
            const unsigned mask = project_group(pts, D, vec4 != 0, sN, c, my_id, here, lane);
            if (lane == 0) sMask[g] = mask;
        }
        __syncthreads();
        // ---- partition + decision: one warp per open node -------------------
        const int nxt = cur ^ 1;
        for (int i = warp; i < n_open; i += n_warps) {
            const SubNode nd = sOpen[cur][i];
            const int g0 = sGroupBase[i], ng = (nd.count + 31) >> 5;
            int nL = 0;
            for (int g = lane; g < ng; g += 32) {
                const int here = min(32, nd.count - g * 32);
                const unsigned valid = here >= 32 ? 0xffffffffu : ((1u << here) - 1u);
                nL += __popc(~sMask[g0 + g] & valid);
            }
#pragma unroll
            for (int s = 16; s >= 1; s >>= 1) nL += __shfl_xor_sync(RSFK_FULL, nL, s);
            int lefts = 0;
            for (int g = 0; g < ng; ++g) {
                const int here = min(32, nd.count - g * 32);
                const unsigned valid = here >= 32 ? 0xffffffffu : ((1u << here) - 1u);
                const unsigned m = sMask[g0 + g] & valid;
                if (lane < here) {
                    const bool right = (m >> lane) & 1u;
                    const int lb = lefts + __popc(~m & ((1u << lane) - 1u));
                    const int pos = g * 32 + lane;
                    const int dest = right ? nL + (pos - lb) : lb;
                    sIds[nxt][nd.start + dest] = sIds[cur][nd.start + pos];
                }
                lefts += __popc(~m & valid);
            }
            __syncwarp();
            const Children ch = decide_children(nd.start, nd.count, nL, min_children, max_children);
            int ref[2] = {0, 0};
            for (int k = 0; k < ch.n; ++k) {
                if (ch.leaf[k]) {
                    for (int q = lane; q < ch.count[k]; q += 32)
                        seg[ch.start[k] + q] = sIds[nxt][ch.start[k] + q];
                    if (lane == 0)
                        ref[k] = -1 - emit_leaf(root.start + ch.start[k], ch.count[k], leaf_start, leaf_count, leaf_cap, cnt);
                } else if (lane == 0) {
                    const int slot = atomicAdd(&sCount[0], 1);
                    if (slot < SUB_NODES) {
                        SubNode o;
                        o.start = ch.start[k];   o.count = ch.count[k];
                        o.pstart = ch.pstart[k]; o.pcount = ch.pcount[k];
                        o.tbl = child_table_row(table, n_table, nd.tbl, ch.side[k]);
                        ref[k] = o.rec = (ch.n == 1) ? nd.rec : new_record(records, rec_cap, cnt);
                        sOpen[nxt][slot] = o;
                    } else {
                        cnt->error = RSFK_ERR_OVERFLOW;
                    }
                }
            }
            if (lane == 0 && (ch.n == 2 || ch.leaf[0])) file_refs(records, nd.rec, ch.n, ref);
        }
        __syncthreads();
        n_open = min(sCount[0], SUB_NODES);
        cur = nxt;
        level++;
        __syncthreads();
    }
    if (lane == 0) {
        if (my_active) atomicAdd(&cnt->sub_active, my_active);
        if (my_nodes) atomicAdd(&cnt->sub_nodes, my_nodes);
    }
    if (threadIdx.x == 0) atomicMax(&cnt->max_level, level);
}

// Depth limit reached: every open node becomes leaves of at most max_children
// points (consecutive pieces of its segment).
__global__ void k_force_leaves(const Node* __restrict__ nodes, const LevelCounters* counters, int level,
                               const int* __restrict__ perm, int* __restrict__ perm_final,
                               int* __restrict__ leaf_start, int* __restrict__ leaf_count, int leaf_cap,
                               LevelCounters* cnt, int max_children, int4* __restrict__ records)
{
    const int n_nodes = counters->lvl[level % 3].n_nodes;
    for (int node = blockIdx.x; node < n_nodes; node += gridDim.x) {
        const Node nd = nodes[node];
        for (int i = threadIdx.x; i < nd.count; i += blockDim.x) perm_final[nd.start + i] = perm[nd.start + i];
        if (threadIdx.x == 0) {
            const int piece = max(1, max_children);
            const int q = (nd.count + piece - 1) / piece;
            int first = 0;
            for (int i = 0; i < q; ++i) {
                int a = (int)((long long)nd.count * i / q), b = (int)((long long)nd.count * (i + 1) / q);
                const int slot = emit_leaf(nd.start + a, b - a, leaf_start, leaf_count, leaf_cap, cnt);
                if (i == 0) first = slot;
            }
            if (records != nullptr) // no split: queries go to the first piece
                records[nd.rec] = make_int4(-1, -1, -1 - first, -1 - first);
        }
    }
}

__global__ void k_iota(int* p, int n)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) p[i] = i;
}

__device__ __forceinline__ void clear_counters(LevelCounters* cnt)
{
    for (int l = 0; l < 3; ++l) { cnt->lvl[l].n_nodes = 0; cnt->lvl[l].n_chunks = 0; cnt->lvl[l].active = 0; cnt->lvl[l].pad = 0; }
    cnt->n_leaves = 0; cnt->max_leaf = 0; cnt->min_leaf = 0x7fffffff; cnt->error = 0;
    cnt->n_small = 0; cnt->max_level = 0; cnt->n_recs = 1; // row 0 is the root
    cnt->last_depth = 0;
    cnt->sub_active = 0; cnt->sub_nodes = 0; cnt->lvl_active = 0; cnt->lvl_nodes = 0; cnt->leaf_sq = 0;
    for (int l = 0; l < LEVEL_HISTORY; ++l) cnt->level_chunks[l] = 0;
}

__global__ void k_tree_init(Node* nodes, int* chunk_node, int* node_done, int node_cap, int n_chunks, int N,
                            int has_table, LevelCounters* cnt)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t == 0) {
        Node r;
        r.start = 0; r.count = N; r.pstart = 0; r.pcount = N;
        r.tbl = has_table ? 0 : -1;
        r.chunk_base = 0; r.level = 0; r.rec = 0;
        nodes[0] = r;
        clear_counters(cnt);
        cnt->lvl[0].n_nodes = 1; cnt->lvl[0].n_chunks = n_chunks; cnt->lvl[0].active = N;
    }
    for (int c = t; c < n_chunks; c += gridDim.x * blockDim.x) chunk_node[c] = 0;
    for (int c = t; c < node_cap; c += gridDim.x * blockDim.x) node_done[c] = 0;
}

__global__ void k_single_leaf(int* leaf_start, int* leaf_count, int N, LevelCounters* cnt, int4* records)
{
    leaf_start[0] = 0;
    leaf_count[0] = N;
    clear_counters(cnt);
    if (records != nullptr) records[0] = make_int4(-1, -1, -1, -1); // every query: leaf slot 0
    cnt->n_leaves = 1; cnt->max_leaf = N; cnt->min_leaf = N;
    cnt->leaf_sq = (unsigned long long)N * (unsigned long long)N;
}

// ---------------------------------------------------------------------------
static void launch_project(Context& ctx, const float* pts, int D, int grid, const LevelArgs& a)
{
    cudaStream_t st = ctx.stream;
    if (D <= 2) k_project_small<2><<<grid, TREE_THREADS, 0, st>>>(pts, D, a);
    else if (D <= 4) k_project_small<4><<<grid, TREE_THREADS, 0, st>>>(pts, D, a);
    else if (D <= 8) k_project_small<8><<<grid, TREE_THREADS, 0, st>>>(pts, D, a);
    else if (D <= 16) k_project_small<16><<<grid, TREE_THREADS, 0, st>>>(pts, D, a);
    else
        k_project_wide<<<grid, TREE_THREADS, (size_t)D * sizeof(float), st>>>(
            pts, D, (D % 4 == 0 && ((uintptr_t)pts & 15) == 0) ? 1 : 0, a);
    count_launches(1);
}

static double host_now()
{
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// Waits (bounded) until the scatter kernel of tree depth `depth` has posted the level
// mailbox.  limit_ms == 0 gives up at once, without looking.
static bool wait_for_level(Context& ctx, int depth, int limit_ms)
{
    cudaStream_t st = ctx.stream;
    volatile LevelMail* mail = ctx.mail;
    const auto t_start = std::chrono::steady_clock::now();
    unsigned spins = 0;
    bool got = false;
    if (limit_ms != 0) {
        while (!(got = (mail->seq == depth))) {
            if ((++spins & 0x3ff) == 0) {
                const cudaError_t q = cudaStreamQuery(st);
                if (q != cudaErrorNotReady) { // finished or failed: the mail is there now or never
                    got = (mail->seq == depth);
                    if (!got) ctx.check(q == cudaSuccess ? cudaErrorUnknown : q, "tree level");
                    break;
                }
                if (std::chrono::steady_clock::now() - t_start > std::chrono::milliseconds(limit_ms)) break;
            }
        }
    }
    std::atomic_thread_fence(std::memory_order_acquire);
    if (!got) {
        cudaStreamSynchronize(st); // nothing of this tree is left in flight when the call returns
        return ctx.fail(RSFK_ERR_CUDA, "tree_build: the level mailbox did not arrive within its time limit");
    }
    return true;
}

bool tree_build(Context& ctx, const float* d_points, int N, int D, int min_children,
                int max_children, int max_depth, int seed, const int* d_table, int n_table,
                TreeResult& out)
{
    TraceRange trace("rsfk tree build");
    out = TreeResult();
    if (N <= 0 || D <= 0) return ctx.fail(RSFK_ERR_ARG, "tree_build: N and D must be positive");
    if (D > 12000) return ctx.fail(RSFK_ERR_UNSUPPORTED, "tree_build: D above 12000 is not supported");
    if (min_children < 0 || max_children < 1)
        return ctx.fail(RSFK_ERR_ARG, "tree_build: invalid min/max_tree_children");
    cudaStream_t st = ctx.stream;
    const double t_enter = host_now();
    const double alloc_before = ctx.alloc_seconds;

    // capacities: an open node holds more than max_children-2 points, a leaf
    // normally at least min_children
    const long long open_min = max_children - 1 > 1 ? max_children - 1 : 1;
    const int node_cap = (int)(N / open_min + 2);
    const int chunk_cap = (int)(N / CHUNK + node_cap + 2);
    const long long leaf_min = min_children / 2 > 1 ? min_children / 2 : 1;
    const int leaf_cap = (int)(N / leaf_min + 16 < N ? N / leaf_min + 16 : N + 16);

    int* perm[2];
    perm[0] = (int*)ctx.scratch(Context::PERM_A, sizeof(int) * (size_t)N);
    perm[1] = (int*)ctx.scratch(Context::PERM_B, sizeof(int) * (size_t)N);
    int* perm_final = (int*)ctx.scratch(Context::PERM_FINAL, sizeof(int) * (size_t)N);
    unsigned* side_bits = (unsigned*)ctx.scratch(Context::SIDE_BITS, sizeof(unsigned) * (size_t)chunk_cap * CHUNK_WORDS);
    int* chunk_node[2];
    chunk_node[0] = (int*)ctx.scratch(Context::CHUNK_NODE_A, sizeof(int) * (size_t)chunk_cap);
    chunk_node[1] = (int*)ctx.scratch(Context::CHUNK_NODE_B, sizeof(int) * (size_t)chunk_cap);
    int* chunk_left = (int*)ctx.scratch(Context::CHUNK_LEFT, sizeof(int) * (size_t)chunk_cap);
    int* node_done = (int*)ctx.scratch(Context::NODE_DONE, sizeof(int) * (size_t)node_cap);
    Node* nodes[2];
    nodes[0] = (Node*)ctx.scratch(Context::NODES_A, sizeof(Node) * (size_t)node_cap);
    nodes[1] = (Node*)ctx.scratch(Context::NODES_B, sizeof(Node) * (size_t)node_cap);
    NodeSplit* split = (NodeSplit*)ctx.scratch(Context::NODE_SPLIT, sizeof(NodeSplit) * (size_t)node_cap);
    // nodes at or below small_limit points are finished inside one CTA each
    int small_limit = 262144 / D;
    if (small_limit > SUB_MAX) small_limit = SUB_MAX;
    const long long node_room = (long long)SUB_NODES * open_min;
    if (small_limit > node_room) small_limit = (int)node_room;
    const size_t sub_smem = sizeof(float) * (size_t)(TREE_THREADS / 32) * D;
    if (small_limit < max_children - 1 || sub_smem > 64 * 1024) small_limit = 0; // nothing would qualify
    const int small_cap = node_cap;
    Node* small_nodes = (Node*)ctx.scratch(Context::SMALL_NODES, sizeof(Node) * (size_t)small_cap);
    int* leaf_start = (int*)ctx.scratch(Context::LEAF_START, sizeof(int) * (size_t)leaf_cap);
    int* leaf_count = (int*)ctx.scratch(Context::LEAF_COUNT, sizeof(int) * (size_t)leaf_cap);
    LevelCounters* cnt = (LevelCounters*)ctx.scratch(Context::COUNTERS, sizeof(LevelCounters));
    // tree index: a row per node with two children (an only child reuses its parent's row),
    // i.e. one row less than there are leaves
    const int rec_cap = ctx.keep_index ? leaf_cap + 64 : 0;
    int4* records = ctx.keep_index ? (int4*)ctx.scratch(Context::RECORDS, sizeof(int4) * (size_t)rec_cap) : nullptr;
    ctx.planes_ready = false;
    if (ctx.status != RSFK_OK) return false;
    if (!ctx.host_counters &&
        !ctx.check(cudaMallocHost((void**)&ctx.host_counters, sizeof(LevelCounters)), "cudaMallocHost"))
        return false;
    if (!ctx.mail) {
        if (!ctx.check(cudaHostAlloc((void**)&ctx.mail, sizeof(LevelMail), cudaHostAllocMapped), "cudaHostAlloc(mail)"))
            return false;
    }
    memset(ctx.mail, 0, sizeof(LevelMail)); // seq 0 is never a loop depth
    const int4* table = (const int4*)d_table;
    const int wait_ms = ctx.level_wait_ms >= 0 ? ctx.level_wait_ms : 30000;

    const int grid_n = (int)(((long long)N + 255) / 256 < 4096 ? ((long long)N + 255) / 256 : 4096);
    k_iota<<<grid_n, 256, 0, st>>>(perm[0], N);
    count_launches(1);

    const int n_chunks0 = (N + CHUNK - 1) / CHUNK;
    bool open = true;
    if (N == 1) {
        k_iota<<<1, 32, 0, st>>>(perm_final, 1);
        k_single_leaf<<<1, 1, 0, st>>>(leaf_start, leaf_count, N, cnt, records);
        count_launches(2);
        open = false;
    } else {
        const int init_items = n_chunks0 > node_cap ? n_chunks0 : node_cap;
        k_tree_init<<<(init_items + 255) / 256, 256, 0, st>>>(nodes[0], chunk_node[0], node_done, node_cap,
                                                              n_chunks0, N, table != nullptr, cnt);
        count_launches(1);
    }

    LevelArgs a;
    a.side_bits = side_bits;     a.chunk_left = chunk_left;   a.node_done = node_done;
    a.node_cap = node_cap;       a.chunk_cap = chunk_cap;     a.split = split;
    a.leaf_start = leaf_start;   a.leaf_count = leaf_count;   a.leaf_cap = leaf_cap;
    a.small_nodes = small_nodes; a.small_cap = small_cap;     a.small_limit = small_limit;
    a.cnt = cnt;                 a.table = table;             a.n_table = n_table;
    a.seed = seed;               a.min_children = min_children; a.max_children = max_children;
    a.records = records;         a.rec_cap = rec_cap;

    // The level kernels loop over as many chunks as the level turns out to have, so any grid is
    // correct; one CTA per chunk is fastest.  The grid of a level is sized from the chunks the
    // previous tree of this context had at that level (trees over the same points are alike),
    // else from what the level can hold at most.
    if (ctx.hint_points != N) {
        for (int l = 0; l < LEVEL_HISTORY; ++l) ctx.level_chunks_hint[l] = 0;
        ctx.level_hint = 0;
        ctx.hint_points = N;
    }
    auto grid_of_level = [&](int level) {
        long long g;
        if (level < LEVEL_HISTORY && ctx.level_chunks_hint[level] > 0) {
            g = ctx.level_chunks_hint[level] + ctx.level_chunks_hint[level] / 4 + 16;
        } else if (ctx.level_hint > 0 && level >= ctx.level_hint) {
            g = 64; // deeper than the previous tree went: most likely nothing is left to split
        } else {
            const long long nodes_most = level < 30 ? (1LL << level) : (long long)node_cap;
            g = (long long)n_chunks0 + (nodes_most < node_cap ? nodes_most : node_cap);
        }
        if (g > chunk_cap) g = chunk_cap;
        if (g > ctx.sm_count * 32) g = ctx.sm_count * 32;
        return (int)(g < 1 ? 1 : g);
    };

    const double t_levels = host_now();
    double wait_s = 0.0;
    int depth = 1; // depth of the children the next level creates
    int cur = 0;
    int timed_levels = 0;
    int n_small_seen = 0;
    // Levels are enqueued in batches; the host reads the mailbox of a batch's last level
    // only.  The first batch is as long as the previous tree of this context was deep
    // (less one), the following ones are short: a level enqueued after the tree has ended
    // costs two empty launches.
    int batch = ctx.level_hint > 3 ? ctx.level_hint - 1 : 4;
    while (open && depth < max_depth) {
        int enq = 0;
        for (; enq < batch && depth < max_depth; ++enq, ++depth) {
            a.level = depth - 1; // level of the nodes being split
            a.perm = perm[cur];
            a.nodes = nodes[cur];       a.chunk_node = chunk_node[cur];
            a.nodes_out = nodes[cur ^ 1]; a.chunk_node_out = chunk_node[cur ^ 1];
            while ((int)ctx.level_ev.size() < 3 * (timed_levels + 1)) {
                cudaEvent_t e;
                cudaEventCreate(&e);
                ctx.level_ev.push_back(e);
            }
            const int level_grid = grid_of_level(a.level);
            cudaEventRecord(ctx.level_ev[3 * timed_levels], st);
            launch_project(ctx, d_points, D, level_grid, a);
            cudaEventRecord(ctx.level_ev[3 * timed_levels + 1], st);
            k_scatter<<<level_grid, TREE_THREADS, 0, st>>>(perm[cur], perm[cur ^ 1], perm_final, nodes[cur],
                                                           chunk_node[cur], side_bits, chunk_left, split, cnt,
                                                           a.level, ctx.mail, depth);
            cudaEventRecord(ctx.level_ev[3 * timed_levels + 2], st);
            count_launches(1);
            timed_levels++;
            cur ^= 1;
        }
        const double w0 = host_now();
        const bool got = wait_for_level(ctx, depth - 1, wait_ms);
        wait_s += host_now() - w0;
        if (!got) return false;
        if (ctx.mail->error) {
            cudaStreamSynchronize(st);
            return ctx.fail(ctx.mail->error, "tree_build: internal table overflow");
        }
        open = ctx.mail->n_nodes > 0;
        n_small_seen = ctx.mail->n_small;
        batch = 2;
    }
    const double t_levels_end = host_now();
    if (ctx.levels_done_event) {
        cudaEventRecord(ctx.levels_done_event, st);
        if (ctx.levels_done_flag) ctx.levels_done_flag->store(1, std::memory_order_release);
        ctx.levels_done_event = nullptr;
        ctx.levels_done_flag = nullptr;
    }
    if (open) { // depth limit: nodes[cur] still holds open nodes (level depth-1)
        int grid = node_cap < ctx.sm_count * 8 ? node_cap : ctx.sm_count * 8;
        k_force_leaves<<<grid, 256, 0, st>>>(nodes[cur], cnt, depth - 1, perm[cur], perm_final, leaf_start,
                                             leaf_count, leaf_cap, cnt, max_children, records);
        count_launches(1);
    }
    const int n_small = N > 1 ? n_small_seen : 0;
    if (n_small > 0) {
        if (sub_smem > 16 * 1024 &&
            !ctx.check(cudaFuncSetAttribute(k_subtree, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sub_smem),
                       "subtree smem attribute"))
            return false;
        if (!ctx.sub_ev[0]) { cudaEventCreate(&ctx.sub_ev[0]); cudaEventCreate(&ctx.sub_ev[1]); }
        cudaEventRecord(ctx.sub_ev[0], st);
        k_subtree<<<n_small, TREE_THREADS, sub_smem, st>>>(d_points, D, perm_final, small_nodes, leaf_start,
                                                           leaf_count, leaf_cap, cnt, table, n_table, seed,
                                                           min_children, max_children, max_depth,
                                                           (D % 4 == 0 && ((uintptr_t)d_points & 15) == 0) ? 1 : 0,
                                                           records, rec_cap);
        cudaEventRecord(ctx.sub_ev[1], st);
        count_launches(1);
    }
    const double t_end0 = host_now();
    if (!ctx.check(cudaMemcpyAsync(ctx.host_counters, cnt, sizeof(LevelCounters),
                                   cudaMemcpyDeviceToHost, st), "counters D2H") ||
        !ctx.check(cudaStreamSynchronize(st), "tree end"))
        return false;
    const LevelCounters& hc = *ctx.host_counters;
    if (hc.error) return ctx.fail(hc.error, "tree_build: internal table overflow");

    float project_ms = 0.0f, scatter_ms = 0.0f;
    for (int l = 0; l < timed_levels; ++l) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, ctx.level_ev[3 * l], ctx.level_ev[3 * l + 1]) == cudaSuccess) project_ms += ms;
        if (cudaEventElapsedTime(&ms, ctx.level_ev[3 * l + 1], ctx.level_ev[3 * l + 2]) == cudaSuccess) scatter_ms += ms;
    }
    int levels = hc.last_depth; // levels the level kernels split
    ctx.level_hint = levels;
    for (int l = 0; l < LEVEL_HISTORY; ++l) ctx.level_chunks_hint[l] = hc.level_chunks[l];
    ctx.stats.project_us += project_ms * 1e3;
    ctx.stats.project_launches += levels;
    ctx.stats.trees++;
    ctx.stats.tree_active_points += (long long)(hc.lvl_active + hc.sub_active);
    ctx.stats.tree_nodes += (long long)(hc.lvl_nodes + hc.sub_nodes);
    ctx.stats.sub_active_points += (long long)hc.sub_active;
    ctx.stats.sub_nodes += (long long)hc.sub_nodes;
    float sub_ms = 0.0f;
    if (n_small > 0 && cudaEventElapsedTime(&sub_ms, ctx.sub_ev[0], ctx.sub_ev[1]) == cudaSuccess)
        ctx.stats.subtree_us += sub_ms * 1e3;
    if (hc.max_level > levels) levels = hc.max_level;
    out.perm = perm_final;
    out.leaf_start = leaf_start;
    out.leaf_count = leaf_count;
    out.n_leaves = hc.n_leaves;
    out.max_leaf = hc.max_leaf;
    out.min_leaf = hc.min_leaf;
    out.levels = N == 1 ? 0 : levels + 1;
    out.records = records;
    out.n_records = records ? hc.n_recs : 0;
    out.sum_leaf_sq = (double)hc.leaf_sq;
    const double t_exit = host_now();
    out.times.init_s = (float)(t_levels - t_enter);
    out.times.build_s = (float)(t_levels_end - t_levels);
    out.times.project_s = project_ms * 1e-3f;
    out.times.scatter_s = scatter_ms * 1e-3f;
    out.times.wait_s = (float)wait_s;
    out.times.alloc_s = (float)(ctx.alloc_seconds - alloc_before);
    out.times.subtree_s = sub_ms * 1e-3f;
    out.times.end_s = (float)(t_exit - t_end0);
    return true;
}

// ---------------------------------------------------------------------------
// Query routing over the tree index (reference: the query descent of
// RSFK::knn_gpu_rsfk_forest_ann_tree, src/rsfk.cu:270-347, which runs
// build_tree_check_points_side over the query array level by level and
// build_tree_update_parents_ann.cu:150-160 to step to the child, or to its
// sibling when the side a query falls on holds no node).
// ---------------------------------------------------------------------------

// Hyperplane of every row: normal n = x[p1]-x[p2] and offset c, in the
// arithmetic of load_hyperplane (row 0, the root, sums serially).
__global__ void __launch_bounds__(TREE_THREADS)
k_planes(const float* __restrict__ pts, int D, const int4* __restrict__ records, int n_recs,
         float* __restrict__ normals, float* __restrict__ offsets)
{
    const int lane = threadIdx.x & 31;
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (r >= n_recs) return;
    const int4 rec = records[r];
    if (rec.x < 0 || rec.y < 0) {
        if (lane == 0) offsets[r] = 0.0f;
        return;
    }
    const float* x1 = pts + (size_t)rec.x * D;
    const float* x2 = pts + (size_t)rec.y * D;
    float* nrm = normals + (size_t)r * D;
    float c = 0.0f;
    if (r == 0) {
        for (int k = lane; k < D; k += 32) nrm[k] = __fsub_rn(__ldg(x1 + k), __ldg(x2 + k));
        if (lane == 0)
            for (int k = 0; k < D; ++k) {
                const float a = __ldg(x1 + k), b = __ldg(x2 + k);
                c = __fadd_rn(c, __fmul_rn(__fmul_rn(__fsub_rn(a, b), __fadd_rn(a, b)), 0.5f));
            }
    } else {
        for (int k = lane; k < D; k += 32) {
            const float a = __ldg(x1 + k), b = __ldg(x2 + k);
            const float nk = __fsub_rn(a, b);
            nrm[k] = nk;
            c = __fadd_rn(c, __fmul_rn(__fmul_rn(nk, __fadd_rn(a, b)), 0.5f));
        }
        c = butterfly_sum(c);
    }
    if (lane == 0) offsets[r] = c;
}

// Descent from row 0 to a leaf slot.  The projection is the reference's warp sum
// (term k on lane k%32, fused multiply-add, xor butterfly), the comparison
// `n.x < c` sends the query right.  The descent is bounded by max_steps; a query
// that does not reach a leaf raises the error flag.
//
// VEC4 (D % 4 == 0, 16-byte aligned rows): eight lanes per query, four queries
// per warp; lane t of the eight owns terms 4t..4t+3 (+32, ...), i.e. virtual
// lanes 4t..4t+3 of that sum (the layout of project_group_vec4), so a warp keeps
// four independent descents in flight.  Otherwise one warp per query.
constexpr int ROUTE_WARPS = 8;

template <bool VEC4>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
k_route(const float* __restrict__ queries, int NQ, int D, const int4* __restrict__ records, int n_recs,
        const float* __restrict__ normals, const float* __restrict__ offsets, int max_steps,
        int n_leaves, int* __restrict__ q_leaf, int* __restrict__ leaf_queries, int* __restrict__ error_flag)
{
    constexpr int QPW = VEC4 ? 4 : 1;       // queries per warp
    constexpr int GL = 32 / QPW;            // lanes per query
    extern __shared__ float4 smem4[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane / GL, t = lane % GL;
    float* xq = reinterpret_cast<float*>(smem4) + ((size_t)warp * QPW + g) * D;
    const int warp0 = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    const int D4 = D >> 2;
    for (int q0 = warp0 * QPW; q0 < NQ; q0 += n_warps * QPW) {
        const int q = q0 + g;
        const bool live = q < NQ;
        __syncwarp();
        if (live) {
            if (VEC4) {
                const float4* src = reinterpret_cast<const float4*>(queries + (size_t)q * D);
                for (int k4 = t; k4 < D4; k4 += GL) reinterpret_cast<float4*>(xq)[k4] = __ldg(src + k4);
            } else {
                for (int k = t; k < D; k += GL) xq[k] = __ldg(queries + (size_t)q * D + k);
            }
        }
        __syncwarp();
        int cur = 0, leaf = -1;
        bool done = !live;
        for (int step = 0; step < max_steps && __any_sync(RSFK_FULL, !done); ++step) {
            int4 rec = make_int4(-1, -1, -1, -1);
            if (!done) rec = records[cur];
            float pr = 0.0f;
            if (VEC4) {
                float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
                if (!done && rec.x >= 0) {
                    const float4* nrm = reinterpret_cast<const float4*>(normals + (size_t)cur * D);
                    const float4* x4 = reinterpret_cast<const float4*>(xq);
                    for (int k4 = t; k4 < D4; k4 += GL) {
                        const float4 n = __ldg(nrm + k4);
                        const float4 x = x4[k4];
                        a0 = __fmaf_rn(n.x, x.x, a0);
                        a1 = __fmaf_rn(n.y, x.y, a1);
                        a2 = __fmaf_rn(n.z, x.z, a2);
                        a3 = __fmaf_rn(n.w, x.w, a3);
                    }
                }
                pr = __fadd_rn(__fadd_rn(a0, a1), __fadd_rn(a2, a3));
                pr = __fadd_rn(pr, __shfl_xor_sync(RSFK_FULL, pr, 1));
                pr = __fadd_rn(pr, __shfl_xor_sync(RSFK_FULL, pr, 2));
                pr = __fadd_rn(pr, __shfl_xor_sync(RSFK_FULL, pr, 4));
            } else {
                float acc = 0.0f;
                if (!done && rec.x >= 0) {
                    const float* nrm = normals + (size_t)cur * D;
                    for (int k = t; k < D; k += GL) acc = __fmaf_rn(__ldg(nrm + k), xq[k], acc);
                }
                pr = butterfly_sum(acc);
            }
            if (!done) {
                int ref = rec.z;
                if (rec.x >= 0 && pr < offsets[cur]) ref = rec.w;
                if (ref < 0) {
                    leaf = -1 - ref;
                    done = true;
                } else if (ref >= n_recs) {
                    done = true;
                } else {
                    cur = ref;
                }
            }
        }
        if (live && t == 0) {
            if (leaf < 0 || leaf >= n_leaves) {
                q_leaf[q] = -1;
                atomicExch(error_flag, RSFK_ERR_OVERFLOW);
            } else {
                q_leaf[q] = leaf;
                if (leaf_queries != nullptr) atomicAdd(&leaf_queries[leaf], 1);
            }
        }
    }
}

bool tree_route(Context& ctx, const float* d_points, int D, const TreeResult& tree,
                const float* d_queries, int NQ, int* d_q_leaf, int* d_leaf_queries)
{
    if (tree.records == nullptr || tree.n_records < 1)
        return ctx.fail(RSFK_ERR_ARG, "tree_route: the tree was built without its index");
    if (NQ <= 0) return true;
    cudaStream_t st = ctx.stream;
    const int n_recs = tree.n_records;
    float* normals = (float*)ctx.scratch(Context::PLANE_NORMALS, sizeof(float) * (size_t)n_recs * D);
    float* offsets = (float*)ctx.scratch(Context::PLANE_OFFSETS, sizeof(float) * (size_t)n_recs);
    int* error_flag = ctx.error_flag();
    if (ctx.status != RSFK_OK || !error_flag) return false;
    if (!ctx.planes_ready) {
        k_planes<<<(n_recs * 32 + TREE_THREADS - 1) / TREE_THREADS, TREE_THREADS, 0, st>>>(
            d_points, D, tree.records, n_recs, normals, offsets);
        count_launches(1);
        ctx.planes_ready = true;
    }
    const bool vec4 = (D % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_queries) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(normals) & 15) == 0);
    const int qpw = vec4 ? 4 : 1;
    const size_t smem = sizeof(float) * (size_t)ROUTE_WARPS * qpw * D;
    if (smem > 200 * 1024) return ctx.fail(RSFK_ERR_UNSUPPORTED, "tree_route: D too large");
    auto kern = vec4 ? k_route<true> : k_route<false>;
    if (smem > 48 * 1024 &&
        !ctx.check(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                   "route smem attribute"))
        return false;
    long long blocks = ((long long)NQ + ROUTE_WARPS * qpw - 1) / (ROUTE_WARPS * qpw);
    if (blocks > ctx.sm_count * 8) blocks = ctx.sm_count * 8;
    // a descent takes at most one step per tree level; the limit bounds the kernel's loop
    const int max_steps = ctx.route_step_limit >= 0 ? ctx.route_step_limit : tree.levels + 8;
    kern<<<(int)blocks, ROUTE_WARPS * 32, smem, st>>>(d_queries, NQ, D, tree.records, n_recs, normals, offsets,
                                                       max_steps, tree.n_leaves, d_q_leaf, d_leaf_queries,
                                                       error_flag);
    count_launches(1);
    return ctx.check(cudaGetLastError(), "route launch");
}

} // namespace rsfk
