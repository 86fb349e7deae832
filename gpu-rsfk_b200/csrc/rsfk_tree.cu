// Random sample tree for sm_100a.
//
// The points of a node are one contiguous segment of a permutation array; a
// split is a stable partition of that segment (left side first), so a leaf's
// bucket is simply perm[start, start+count) and no per-point parent/depth
// bookkeeping exists.  Each level runs three kernels over the level's work
// chunks (CHUNK consecutive positions of one node):
//
//   project : side bit of every active point (n.x < c  =>  right) as one
//             32-bit mask per 32 positions, plus the chunk's left count;
//   decide  : per node, the left total and the per-chunk exclusive prefix;
//             children, leaves and next level's chunk list;
//   scatter : stable partition into the other permutation buffer; points
//             whose child is a leaf are also written to the final array.
//
// The rules (which side is right, when a child is a leaf, when a small child
// dissolves into its sibling) follow the reference's level kernels:
// src/kernels/build_tree_check_points_side.cu:131-151,
// src/kernels/build_tree_update_parents.cu:64-75,106-135,
// src/kernels/build_tree_create_nodes.cu:88-104, src/kernels/create_node.cu:60-66,120-134.
// The arithmetic keeps the reference's summation order so that the side of
// every point is bit-for-bit the reference's for the same split pair.
#include "rsfk_context.h"

namespace rsfk {

constexpr int CHUNK = 1024;          // positions per work chunk
constexpr int CHUNK_WORDS = CHUNK / 32;
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
// project, any D: one warp per point, four points in flight per warp.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(TREE_THREADS)
k_project_wide(const float* __restrict__ pts, int D, const int* __restrict__ perm,
               const Node* __restrict__ nodes, const int* __restrict__ chunk_node,
               unsigned* __restrict__ side_bits, int* __restrict__ chunk_left,
               const int4* __restrict__ table, int n_table, int seed, int level)
{
    extern __shared__ float smem[];
    float* sN = smem;
    __shared__ float sC;
    __shared__ int sPair[2];
    __shared__ int sLeft;

    const int chunk = blockIdx.x;
    const Node nd = nodes[chunk_node[chunk]];
    const int off = (chunk - nd.chunk_base) * CHUNK;
    const int cnt = min(CHUNK, nd.count - off);
    if (threadIdx.x == 0) {
        int p1, p2;
        node_pair(nd, perm, table, n_table, seed, level, p1, p2);
        sPair[0] = p1;
        sPair[1] = p2;
        sLeft = 0;
    }
    __syncthreads();
    const float c = load_hyperplane(pts, D, sPair[0], sPair[1], level == 0, sN, &sC);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int* ids = perm + nd.start + off;
    int left_total = 0;
    for (int w = warp; w * 32 < cnt; w += n_warps) {
        const int base = w * 32;
        const int here = min(32, cnt - base);
        const int my_id = lane < here ? ids[base + lane] : -1;
        unsigned mask = 0;
        for (int q = 0; q < here; q += 4) {
            float acc[4];
            const float* row[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                int id = __shfl_sync(RSFK_FULL, my_id, min(q + u, here - 1));
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
                float pr = butterfly_sum(acc[u]);
                if (q + u < here && pr < c) mask |= 1u << (q + u);
            }
        }
        if (lane == 0) {
            side_bits[(size_t)chunk * CHUNK_WORDS + w] = mask;
            left_total += here - __popc(mask);
        }
    }
    if (lane == 0 && left_total) atomicAdd(&sLeft, left_total);
    __syncthreads();
    if (threadIdx.x == 0) chunk_left[chunk] = sLeft;
}

// ---------------------------------------------------------------------------
// project, D <= 16: one thread per point.  Lanes >= D of the reference's
// 32-lane sum hold zero, and adding zero changes no comparison, so only
// VL = next power of two >= D partial sums are kept and combined in the
// butterfly's order.
// ---------------------------------------------------------------------------
template <int VL>
__global__ void __launch_bounds__(TREE_THREADS)
k_project_small(const float* __restrict__ pts, int D, const int* __restrict__ perm,
                const Node* __restrict__ nodes, const int* __restrict__ chunk_node,
                unsigned* __restrict__ side_bits, int* __restrict__ chunk_left,
                const int4* __restrict__ table, int n_table, int seed, int level)
{
    __shared__ float sN[VL];
    __shared__ float sC;
    __shared__ int sPair[2];
    __shared__ int sLeft;

    const int chunk = blockIdx.x;
    const Node nd = nodes[chunk_node[chunk]];
    const int off = (chunk - nd.chunk_base) * CHUNK;
    const int cnt = min(CHUNK, nd.count - off);
    if (threadIdx.x == 0) {
        int p1, p2;
        node_pair(nd, perm, table, n_table, seed, level, p1, p2);
        sPair[0] = p1;
        sPair[1] = p2;
        sLeft = 0;
    }
    __syncthreads();
    const float c = load_hyperplane(pts, D, sPair[0], sPair[1], level == 0, sN, &sC);

    const int lane = threadIdx.x & 31;
    const int* ids = perm + nd.start + off;
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
            side_bits[(size_t)chunk * CHUNK_WORDS + (base >> 5)] = mask;
            left_total += min(32, cnt - base) - __popc(mask);
        }
    }
    if (lane == 0 && left_total) atomicAdd(&sLeft, left_total);
    __syncthreads();
    if (threadIdx.x == 0) chunk_left[chunk] = sLeft;
}

// ---------------------------------------------------------------------------
// decide: one warp per node.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void emit_leaf(int start, int count, int* leaf_start, int* leaf_count,
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
}

__global__ void __launch_bounds__(TREE_THREADS)
k_decide(const Node* __restrict__ nodes, int n_nodes, int* __restrict__ chunk_left,
         Node* __restrict__ nodes_out, int node_cap, int* __restrict__ chunk_node_out, int chunk_cap,
         NodeSplit* __restrict__ split, int* __restrict__ leaf_start, int* __restrict__ leaf_count,
         int leaf_cap, LevelCounters* __restrict__ cnt, const int4* __restrict__ table, int n_table,
         int min_children, int max_children)
{
    const int lane = threadIdx.x & 31;
    const int node = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (node >= n_nodes) return;
    const Node nd = nodes[node];
    const int n_chunks = (nd.count + CHUNK - 1) / CHUNK;

    // left total; chunk_left becomes the exclusive prefix inside the node
    int carry = 0;
    for (int c0 = 0; c0 < n_chunks; c0 += 32) {
        const int c = c0 + lane;
        int v = c < n_chunks ? chunk_left[nd.chunk_base + c] : 0;
        int incl = v;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            int t = __shfl_up_sync(RSFK_FULL, incl, s);
            if (lane >= s) incl += t;
        }
        if (c < n_chunks) chunk_left[nd.chunk_base + c] = carry + incl - v;
        carry += __shfl_sync(RSFK_FULL, incl, 31);
    }
    const int nL = carry, nR = nd.count - nL;

    // children: {start, count, own segment, side, leaf}
    int n_ch = 0;
    int ch_start[2], ch_count[2], ch_pstart[2], ch_pcount[2], ch_side[2], ch_leaf[2];
    int flags = 0;
    if (nL > 0 && nR > 0 && nL >= min_children && nR >= min_children) {
        n_ch = 2;
        ch_start[0] = ch_pstart[0] = nd.start;      ch_count[0] = ch_pcount[0] = nL; ch_side[0] = 0;
        ch_start[1] = ch_pstart[1] = nd.start + nL; ch_count[1] = ch_pcount[1] = nR; ch_side[1] = 1;
        ch_leaf[0] = nL <= max_children - 2;
        ch_leaf[1] = nR <= max_children - 2;
        flags = (ch_leaf[0] ? 1 : 0) | (ch_leaf[1] ? 2 : 0);
    } else if (nL > 0 && nR > 0) {
        // the side with fewer than min_children points dissolves into the other,
        // which keeps the split pair drawn from its own segment
        int keep = (nL < min_children) ? 1 : 0;
        if (nL < min_children && nR < min_children) keep = 0;
        n_ch = 1;
        ch_start[0] = nd.start; ch_count[0] = nd.count;
        ch_pstart[0] = keep ? nd.start + nL : nd.start;
        ch_pcount[0] = keep ? nR : nL;
        ch_side[0] = keep;
        ch_leaf[0] = nd.count <= max_children;
        flags = ch_leaf[0] ? 3 : 0;
    } else {
        n_ch = 1;
        ch_start[0] = ch_pstart[0] = nd.start; ch_count[0] = ch_pcount[0] = nd.count;
        ch_side[0] = nL > 0 ? 0 : 1;
        ch_leaf[0] = nd.count <= max_children - 2;
        flags = ch_leaf[0] ? 3 : 0;
    }
    if (lane == 0) {
        split[node].n_left = nL;
        split[node].flags = flags;
    }
    for (int k = 0; k < n_ch; ++k) {
        if (ch_leaf[k]) {
            if (lane == 0) emit_leaf(ch_start[k], ch_count[k], leaf_start, leaf_count, leaf_cap, cnt);
            continue;
        }
        const int nch = (ch_count[k] + CHUNK - 1) / CHUNK;
        int slot = 0, cb = 0;
        if (lane == 0) {
            slot = atomicAdd(&cnt->n_nodes_next, 1);
            cb = atomicAdd(&cnt->n_chunks_next, nch);
            atomicAdd(&cnt->active_next, ch_count[k]);
        }
        slot = __shfl_sync(RSFK_FULL, slot, 0);
        cb = __shfl_sync(RSFK_FULL, cb, 0);
        if (slot >= node_cap || cb + nch > chunk_cap) {
            if (lane == 0) cnt->error = RSFK_ERR_OVERFLOW;
            continue;
        }
        if (lane == 0) {
            Node o;
            o.start = ch_start[k];   o.count = ch_count[k];
            o.pstart = ch_pstart[k]; o.pcount = ch_pcount[k];
            o.tbl = -1;
            if (table != nullptr && nd.tbl >= 0 && nd.tbl < n_table) {
                int4 t = table[nd.tbl];
                o.tbl = ch_side[k] ? t.w : t.z;
            }
            o.chunk_base = cb;
            o.pad0 = o.pad1 = 0;
            nodes_out[slot] = o;
        }
        for (int c = lane; c < nch; c += 32) chunk_node_out[cb + c] = slot;
    }
}

// ---------------------------------------------------------------------------
// scatter: stable partition of one chunk.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(TREE_THREADS)
k_scatter(const int* __restrict__ perm_in, int* __restrict__ perm_out, int* __restrict__ perm_final,
          const Node* __restrict__ nodes, const int* __restrict__ chunk_node,
          const unsigned* __restrict__ side_bits, const int* __restrict__ chunk_lprefix,
          const NodeSplit* __restrict__ split)
{
    __shared__ unsigned sMask[CHUNK_WORDS];
    __shared__ int sWordLeft[CHUNK_WORDS];

    const int chunk = blockIdx.x;
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
        sMask[w] = m;
        sWordLeft[w] = incl - lefts;
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
}

// Depth limit reached: every open node becomes leaves of at most max_children
// points (consecutive pieces of its segment).
__global__ void k_force_leaves(const Node* __restrict__ nodes, int n_nodes, const int* __restrict__ perm,
                               int* __restrict__ perm_final, int* __restrict__ leaf_start,
                               int* __restrict__ leaf_count, int leaf_cap, LevelCounters* cnt,
                               int max_children)
{
    const int node = blockIdx.x;
    if (node >= n_nodes) return;
    const Node nd = nodes[node];
    for (int i = threadIdx.x; i < nd.count; i += blockDim.x) perm_final[nd.start + i] = perm[nd.start + i];
    if (threadIdx.x == 0) {
        const int piece = max(1, max_children);
        const int q = (nd.count + piece - 1) / piece;
        for (int i = 0; i < q; ++i) {
            int a = (int)((long long)nd.count * i / q), b = (int)((long long)nd.count * (i + 1) / q);
            emit_leaf(nd.start + a, b - a, leaf_start, leaf_count, leaf_cap, cnt);
        }
    }
}

__global__ void k_iota(int* p, int n)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) p[i] = i;
}

__global__ void k_tree_init(Node* nodes, int* chunk_node, int n_chunks, int N, int has_table,
                            LevelCounters* cnt)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t == 0) {
        Node r;
        r.start = 0; r.count = N; r.pstart = 0; r.pcount = N;
        r.tbl = has_table ? 0 : -1;
        r.chunk_base = 0; r.pad0 = r.pad1 = 0;
        nodes[0] = r;
        cnt->n_nodes_next = 0; cnt->n_chunks_next = 0; cnt->n_leaves = 0;
        cnt->max_leaf = 0; cnt->min_leaf = 0x7fffffff; cnt->error = 0; cnt->active_next = 0;
    }
    for (int c = t; c < n_chunks; c += gridDim.x * blockDim.x) chunk_node[c] = 0;
}

__global__ void k_reset_level(LevelCounters* cnt)
{
    cnt->n_nodes_next = 0;
    cnt->n_chunks_next = 0;
    cnt->active_next = 0;
}

__global__ void k_single_leaf(int* leaf_start, int* leaf_count, int N, LevelCounters* cnt)
{
    leaf_start[0] = 0;
    leaf_count[0] = N;
    cnt->n_leaves = 1; cnt->max_leaf = N; cnt->min_leaf = N; cnt->error = 0;
    cnt->n_nodes_next = 0; cnt->n_chunks_next = 0;
}

// ---------------------------------------------------------------------------
static void launch_project(Context& ctx, const float* pts, int D, const int* perm, const Node* nodes,
                           const int* chunk_node, int n_chunks, unsigned* side_bits, int* chunk_left,
                           const int4* table, int n_table, int seed, int level)
{
    cudaStream_t st = ctx.stream;
#define RSFK_SMALL(VL)                                                                              \
    k_project_small<VL><<<n_chunks, TREE_THREADS, 0, st>>>(pts, D, perm, nodes, chunk_node,         \
                                                           side_bits, chunk_left, table, n_table,   \
                                                           seed, level)
    if (D <= 2) RSFK_SMALL(2);
    else if (D <= 4) RSFK_SMALL(4);
    else if (D <= 8) RSFK_SMALL(8);
    else if (D <= 16) RSFK_SMALL(16);
    else
        k_project_wide<<<n_chunks, TREE_THREADS, (size_t)D * sizeof(float), st>>>(
            pts, D, perm, nodes, chunk_node, side_bits, chunk_left, table, n_table, seed, level);
#undef RSFK_SMALL
    count_launches(1);
}

bool tree_build(Context& ctx, const float* d_points, int N, int D, int min_children,
                int max_children, int max_depth, int seed, const int* d_table, int n_table,
                TreeResult& out)
{
    out = TreeResult();
    if (N <= 0 || D <= 0) return ctx.fail(RSFK_ERR_ARG, "tree_build: N and D must be positive");
    if (D > 12000) return ctx.fail(RSFK_ERR_UNSUPPORTED, "tree_build: D above 12000 is not supported");
    if (min_children < 0 || max_children < 1)
        return ctx.fail(RSFK_ERR_ARG, "tree_build: invalid min/max_tree_children");
    cudaStream_t st = ctx.stream;

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
    Node* nodes[2];
    nodes[0] = (Node*)ctx.scratch(Context::NODES_A, sizeof(Node) * (size_t)node_cap);
    nodes[1] = (Node*)ctx.scratch(Context::NODES_B, sizeof(Node) * (size_t)node_cap);
    NodeSplit* split = (NodeSplit*)ctx.scratch(Context::NODE_SPLIT, sizeof(NodeSplit) * (size_t)node_cap);
    int* leaf_start = (int*)ctx.scratch(Context::LEAF_START, sizeof(int) * (size_t)leaf_cap);
    int* leaf_count = (int*)ctx.scratch(Context::LEAF_COUNT, sizeof(int) * (size_t)leaf_cap);
    LevelCounters* cnt = (LevelCounters*)ctx.scratch(Context::COUNTERS, sizeof(LevelCounters));
    if (ctx.status != RSFK_OK) return false;
    if (!ctx.host_counters &&
        !ctx.check(cudaMallocHost((void**)&ctx.host_counters, sizeof(LevelCounters)), "cudaMallocHost"))
        return false;
    const int4* table = (const int4*)d_table;

    const int grid_n = (int)(((long long)N + 255) / 256 < 4096 ? ((long long)N + 255) / 256 : 4096);
    k_iota<<<grid_n, 256, 0, st>>>(perm[0], N);
    count_launches(1);

    int levels = 0;
    int n_nodes = 1, n_chunks = (N + CHUNK - 1) / CHUNK;
    int cur = 0;
    if (N == 1) {
        k_iota<<<1, 32, 0, st>>>(perm_final, 1);
        k_single_leaf<<<1, 1, 0, st>>>(leaf_start, leaf_count, N, cnt);
        count_launches(2);
        n_nodes = 0;
    } else {
        k_tree_init<<<(n_chunks + 255) / 256, 256, 0, st>>>(nodes[0], chunk_node[0], n_chunks, N,
                                                            table != nullptr, cnt);
        count_launches(1);
    }

    int depth = 1;
    long long active = N;
    for (; depth < max_depth && n_nodes > 0; ++depth) {
        const int level = depth - 1; // level of the nodes being split
        ctx.stats.tree_active_points += active;
        ctx.stats.tree_nodes += n_nodes;
        launch_project(ctx, d_points, D, perm[cur], nodes[cur], chunk_node[cur], n_chunks, side_bits,
                       chunk_left, table, n_table, seed, level);
        k_reset_level<<<1, 1, 0, st>>>(cnt);
        k_decide<<<(n_nodes * 32 + TREE_THREADS - 1) / TREE_THREADS, TREE_THREADS, 0, st>>>(
            nodes[cur], n_nodes, chunk_left, nodes[cur ^ 1], node_cap, chunk_node[cur ^ 1], chunk_cap,
            split, leaf_start, leaf_count, leaf_cap, cnt, table, n_table, min_children, max_children);
        k_scatter<<<n_chunks, TREE_THREADS, 0, st>>>(perm[cur], perm[cur ^ 1], perm_final, nodes[cur],
                                                     chunk_node[cur], side_bits, chunk_left, split);
        count_launches(3);
        if (!ctx.check(cudaMemcpyAsync(ctx.host_counters, cnt, sizeof(LevelCounters),
                                       cudaMemcpyDeviceToHost, st), "counters D2H") ||
            !ctx.check(cudaStreamSynchronize(st), "tree level"))
            return false;
        if (ctx.host_counters->error)
            return ctx.fail(ctx.host_counters->error, "tree_build: internal table overflow");
        n_nodes = ctx.host_counters->n_nodes_next;
        n_chunks = ctx.host_counters->n_chunks_next;
        active = ctx.host_counters->active_next;
        cur ^= 1;
        levels = depth;
    }
    if (n_nodes > 0) {
        k_force_leaves<<<n_nodes, 256, 0, st>>>(nodes[cur], n_nodes, perm[cur], perm_final, leaf_start,
                                                leaf_count, leaf_cap, cnt, max_children);
        count_launches(1);
    }
    if (!ctx.check(cudaMemcpyAsync(ctx.host_counters, cnt, sizeof(LevelCounters),
                                   cudaMemcpyDeviceToHost, st), "counters D2H") ||
        !ctx.check(cudaStreamSynchronize(st), "tree end"))
        return false;
    if (ctx.host_counters->error)
        return ctx.fail(ctx.host_counters->error, "tree_build: internal table overflow");

    ctx.stats.trees++;
    out.perm = perm_final;
    out.leaf_start = leaf_start;
    out.leaf_count = leaf_count;
    out.n_leaves = ctx.host_counters->n_leaves;
    out.max_leaf = ctx.host_counters->max_leaf;
    out.min_leaf = ctx.host_counters->min_leaf;
    out.levels = N == 1 ? 0 : levels + 1;
    return true;
}

} // namespace rsfk
