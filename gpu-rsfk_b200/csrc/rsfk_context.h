// Host-side context of the sm_100a RSFK library: one device, one stream, a
// grow-only pool of scratch buffers (no allocation inside the per-tree loop),
// pinned mailboxes for the few counters the host reads back, and the status
// word the C ABI exposes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <atomic>
#include <chrono>
#include <string>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "rsfk_common.cuh"

namespace rsfk {

// Named range on the calling host thread for timeline tools (NVTX, header-only: costs a
// few nanoseconds when no tool is attached).  The reference brackets the same phases with
// its Cron timers (src/rsfk.cu:509-512, 2076-2147).
struct TraceRange {
    explicit TraceRange(const char* name) { nvtxRangePushA(name); }
    ~TraceRange() { nvtxRangePop(); }
    TraceRange(const TraceRange&) = delete;
    TraceRange& operator=(const TraceRange&) = delete;
};

// kernels of this library launched so far in this process
inline std::atomic<long long> g_kernel_launches{0};
inline void count_launches(int n) { g_kernel_launches.fetch_add(n, std::memory_order_relaxed); }

struct Buffer {
    void* ptr = nullptr;
    size_t bytes = 0;
};

// Active node of the level being split.  Its points are perm[start, start+count).
// The split pair is drawn from perm[pstart, pstart+pcount) (the node's own
// segment before a sibling was merged into it).
struct Node {
    int start, count;
    int pstart, pcount;
    int tbl;        // row of the replay table, or -1
    int chunk_base; // first work chunk of this node in the level's chunk list
    int level;      // depth of the node (root = 0)
    int rec;        // row of the node in the tree index (when one is kept)
};

constexpr int LEVEL_HISTORY = 64;

// Sizes of one tree level: how many open nodes it splits, how many work chunks
// they make, how many points they hold.
struct LevelState {
    int n_nodes, n_chunks, active, pad;
};

struct LevelCounters {
    // Level L reads lvl[L % 3], collects the next level in lvl[(L+1) % 3] and clears
    // lvl[(L+2) % 3], so that a batch of levels can be enqueued without the host.
    LevelState lvl[3];
    int n_leaves;
    int max_leaf;
    int min_leaf;
    int error;
    int n_small;     // nodes handed to the in-CTA subtree kernel
    int max_level;   // deepest level any subtree reached
    int n_recs;      // rows of the tree index handed out so far
    int last_depth;  // 1 + the deepest level the level kernels split
    unsigned long long sub_active; // points projected inside subtree CTAs (all levels)
    unsigned long long sub_nodes;  // nodes split inside subtree CTAs
    unsigned long long lvl_active; // points projected by the level kernels (all levels)
    unsigned long long lvl_nodes;  // nodes split by the level kernels
    unsigned long long leaf_sq;    // sum over leaves of count^2
    int level_chunks[LEVEL_HISTORY]; // work chunks of the first levels (sizes the next tree's grids)
};

// Per-level mailbox in pinned, device-mapped host memory: the scatter kernel of a
// level posts the next level's sizes here and the host picks them up by polling
// `seq`, without a copy or a stream synchronisation.
struct LevelMail {
    int n_nodes, n_chunks, active, n_small, error;
    int seq; // written last: the loop depth these numbers belong to
    int pad0, pad1;
};

// Work counters a benchmark reads to turn kernel times into achieved bytes/s.
struct Stats {
    long long trees = 0;              // trees built
    long long tree_active_points = 0; // sum over levels of the points projected
    long long tree_nodes = 0;         // nodes split (hyperplanes formed)
    double bucket_knn_us = 0.0;       // device time of the bucket-KNN kernels
    double subtree_us = 0.0;          // device time of the subtree kernels
    double project_us = 0.0;          // device time of the projection kernels of the tree levels
    long long project_launches = 0;
    double tree_build_us = 0.0;       // host-observed time of the tree builds (each ends with a stream sync)
    long long sub_active_points = 0;  // part of tree_active_points projected inside subtree CTAs
    long long sub_nodes = 0;          // part of tree_nodes split inside subtree CTAs
    void add(const Stats& o)
    {
        trees += o.trees; tree_active_points += o.tree_active_points; tree_nodes += o.tree_nodes;
        bucket_knn_us += o.bucket_knn_us; subtree_us += o.subtree_us; project_us += o.project_us;
        project_launches += o.project_launches; tree_build_us += o.tree_build_us;
        sub_active_points += o.sub_active_points; sub_nodes += o.sub_nodes;
        route_us += o.route_us; query_update_us += o.query_update_us;
        tc_launches += o.tc_launches; tc_gram_flops += o.tc_gram_flops;
    }
    double route_us = 0.0;            // query path: device time of hyperplanes + descent + grouping by leaf
    double query_update_us = 0.0;     // query path: device time of the query-bucket kernels
    long long tc_launches = 0;        // bucket-KNN launches that took the tensor-core kernel
    double tc_gram_flops = 0.0;       // 2*D*sum(m_b^2) over the leaves of those launches
};

// Host-observed and device-measured parts of one tree build, in seconds; they fill
// the per-tree rows of the forest log.
struct TreeTimes {
    float init_s = 0, build_s = 0, project_s = 0, decide_s = 0, scatter_s = 0, wait_s = 0, alloc_s = 0,
          subtree_s = 0, end_s = 0;
};

struct TreeResult {
    const int* perm = nullptr;       // device, [N]: points ordered by leaf
    const int* leaf_start = nullptr; // device, [n_leaves] (unordered)
    const int* leaf_count = nullptr; // device, [n_leaves]
    int n_leaves = 0;
    int max_leaf = 0;
    int min_leaf = 0;
    int levels = 0;
    // Tree index (kept on request): row r = {p1, p2, left ref, right ref}; the split
    // pair is (p1, p2) (p1 < 0: no split, follow the left ref); a ref >= 0 is a row,
    // a ref < 0 names the leaf slot -1-ref.  Row 0 is the root.
    const int4* records = nullptr;
    int n_records = 0;
    TreeTimes times;
    double sum_leaf_sq = 0.0; // sum over leaves of (points in the leaf)^2
};

struct Context {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 148;
    int status = RSFK_OK;
    std::string message;

    enum Slot {
        PERM_A, PERM_B, PERM_FINAL, SIDE_BITS, CHUNK_NODE_A, CHUNK_NODE_B, CHUNK_LEFT, NODE_DONE,
        NODES_A, NODES_B, NODE_SPLIT, SMALL_NODES, LEAF_START, LEAF_COUNT, COUNTERS, TABLE,
        SNAPSHOT, EXPLORE_COUNT, EXPLORE_CAND, ERROR_FLAG, HOST_POINTS, HOST_IDX, HOST_DIST,
        RECORDS, PLANE_NORMALS, PLANE_OFFSETS, QUERY_LEAF, QUERY_ORDER, LEAF_QUERIES, HOST_QUERIES,
        LANE_IDX, LANE_DIST, SYM_DEGREE, SYM_BLOCKS, TC_ROWS, TC_EXACT, TC_NORMS, TC_TILES, TC_COUNT, TC_STATS, TC_LATER_ROWS, TC_LATER_CAND, TC_OPEN, TC_THR0,
        PEER_IDX, PEER_DIST,
        KM_IOTA, KM_KEYS, KM_ORDER, KM_START, KM_TEMP, KM_CHANGED, KM_POINTS, KM_CENTROIDS, KM_LABELS, KM_DIST,
        N_SLOTS
    };
    // When set, tree_build keeps the tree index (TreeResult::records) that the
    // query path descends.
    bool keep_index = false;
    bool planes_ready = false; // hyperplanes of the current tree index are materialised
    // Bucket KNN on the tensor cores: 1 always (where the shape allows it), 0 never,
    // -1 the library's choice.
    int tc_mode = -1;
    // Limits of the bounded waits (negative: the built-in value).  route_step_limit is the
    // number of tree levels a query may descend before its kernel gives up and raises the
    // error flag; level_wait_ms is how long the host waits for a tree level's mailbox.
    int route_step_limit = -1;
    int level_wait_ms = -1;
    double alloc_seconds = 0.0; // host time spent growing scratch buffers
    Stats stats;
    Buffer slots[N_SLOTS];
    LevelCounters* host_counters = nullptr; // pinned
    LevelMail* mail = nullptr;              // pinned + mapped
    cudaEvent_t sub_ev[2] = {nullptr, nullptr};
    // Query path: three events per query update (before routing, after grouping, after the
    // update), taken from a pool and turned into times only when somebody asks for the stats
    // or the forest ends, so that no tree waits for the previous tree's update.
    std::vector<cudaEvent_t> ann_ev;
    size_t ann_ev_used = 0;
    cudaEvent_t* next_ann_events()
    {
        if (ann_ev_used + 3 > 3 * 256) resolve_ann_events();
        while (ann_ev.size() < ann_ev_used + 3) {
            cudaEvent_t e = nullptr;
            if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
            ann_ev.push_back(e);
        }
        cudaEvent_t* p = &ann_ev[ann_ev_used];
        ann_ev_used += 3;
        return p;
    }
    // adds the pending query updates' device times to the stats (waits for the last event)
    void resolve_ann_events()
    {
        for (size_t i = 0; i + 3 <= ann_ev_used; i += 3) {
            float a = 0.0f, b = 0.0f;
            if (cudaEventSynchronize(ann_ev[i + 2]) == cudaSuccess &&
                cudaEventElapsedTime(&a, ann_ev[i], ann_ev[i + 1]) == cudaSuccess &&
                cudaEventElapsedTime(&b, ann_ev[i + 1], ann_ev[i + 2]) == cudaSuccess) {
                stats.route_us += a * 1e3;
                stats.query_update_us += b * 1e3;
            }
        }
        ann_ev_used = 0;
    }
    std::vector<cudaEvent_t> level_ev; // three per tree level, reused by every tree
    // When set, the next tree build records this event on the stream right after its level
    // loop is enqueued, raises the flag, and clears both (forest lanes start one after the
    // other on the GPU with it, so that they do not run the same phase at the same time).
    cudaEvent_t levels_done_event = nullptr;
    std::atomic<int>* levels_done_flag = nullptr;
    int level_hint = 0;                // levels the previous tree of this context needed
    int level_chunks_hint[LEVEL_HISTORY] = {}; // and the work chunks of its first levels (0: unknown)
    long long hint_points = 0;         // the N those hints belong to
    bool fail(int code, const std::string& msg)
    {
        if (status == RSFK_OK) { status = code; message = msg; }
        fprintf(stderr, "rsfk: %s\n", msg.c_str());
        return false;
    }
    bool check(cudaError_t e, const char* what)
    {
        if (e == cudaSuccess) return true;
        return fail(RSFK_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
    }
    // grow-only scratch; contents are not preserved across growth
    void* scratch(Slot s, size_t bytes)
    {
        Buffer& b = slots[s];
        if (b.bytes >= bytes && b.ptr) return b.ptr;
        const auto t0 = std::chrono::steady_clock::now();
        if (b.ptr) cudaFree(b.ptr);
        b.ptr = nullptr;
        b.bytes = 0;
        size_t want = bytes + bytes / 8 + 256;
        if (!check(cudaMalloc(&b.ptr, want), "cudaMalloc(scratch)")) { status = RSFK_ERR_NOMEM; return nullptr; }
        b.bytes = want;
        alloc_seconds += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        return b.ptr;
    }
    // device counter of candidates evaluated by exploration sweeps (zeroed once)
    unsigned long long* explore_counter()
    {
        const bool fresh = slots[EXPLORE_COUNT].ptr == nullptr;
        auto* p = (unsigned long long*)scratch(EXPLORE_COUNT, sizeof(unsigned long long));
        if (p && fresh) cudaMemsetAsync(p, 0, sizeof(unsigned long long), stream);
        return p;
    }
    // device counters of the tensor-core bucket kernel: pairs passed by its filter, pairs seen
    unsigned long long* tc_counters()
    {
        const bool fresh = slots[TC_STATS].ptr == nullptr;
        auto* p = (unsigned long long*)scratch(TC_STATS, 2 * sizeof(unsigned long long));
        if (p && fresh) cudaMemsetAsync(p, 0, 2 * sizeof(unsigned long long), stream);
        return p;
    }
    // device word a kernel sets when one of its bounded waits gave up (zeroed once)
    int* error_flag()
    {
        const bool fresh = slots[ERROR_FLAG].ptr == nullptr;
        int* p = (int*)scratch(ERROR_FLAG, sizeof(int));
        if (p && fresh) cudaMemsetAsync(p, 0, sizeof(int), stream);
        return p;
    }
    // reads the flag back (synchronizes the stream); false and a failure status when set
    bool check_error_flag()
    {
        if (!slots[ERROR_FLAG].ptr) return true;
        int v = 0;
        if (!check(cudaMemcpyAsync(&v, slots[ERROR_FLAG].ptr, sizeof(int), cudaMemcpyDeviceToHost, stream), "flag D2H") ||
            !check(cudaStreamSynchronize(stream), "flag sync"))
            return false;
        if (v != 0) {
            cudaMemsetAsync(slots[ERROR_FLAG].ptr, 0, sizeof(int), stream);
            return fail(RSFK_ERR_CUDA, "a device-side check failed (a bounded wait of the tensor-core bucket "
                                       "kernel ran out, or a query reached no leaf)");
        }
        return true;
    }
    void release()
    {
        for (auto& b : slots) { if (b.ptr) cudaFree(b.ptr); b.ptr = nullptr; b.bytes = 0; }
        if (host_counters) { cudaFreeHost(host_counters); host_counters = nullptr; }
        if (mail) { cudaFreeHost(mail); mail = nullptr; }
        for (auto& e : sub_ev) { if (e) cudaEventDestroy(e); e = nullptr; }
        for (auto& e : ann_ev) cudaEventDestroy(e);
        ann_ev.clear();
        ann_ev_used = 0;
        for (auto& e : level_ev) cudaEventDestroy(e);
        level_ev.clear();
        if (owns_stream && stream) { cudaStreamDestroy(stream); stream = nullptr; }
    }
};

// rsfk_tree.cu
bool tree_build(Context& ctx, const float* d_points, int N, int D, int min_children,
                int max_children, int max_depth, int seed, const int* d_table, int n_table,
                TreeResult& out);
// Leaf slot of every query row (d_q_leaf[NQ], -1 on failure) by descending the tree
// index; d_leaf_queries[n_leaves], when given, is incremented once per query.
bool tree_route(Context& ctx, const float* d_points, int D, const TreeResult& tree,
                const float* d_queries, int NQ, int* d_q_leaf, int* d_leaf_queries);

// rsfk_knn.cu
int list_capacity();                      // largest supported K
bool sort_rows(Context& ctx, int* d_idx, float* d_dist, long long rows, int K);
// n list entries set to empty: index -1, distance +inf
bool fill_empty_lists(Context& ctx, int* d_idx, float* d_dist, long long n);
bool bucket_knn(Context& ctx, const float* d_points, int N, int D, int K, const TreeResult& tree,
                int* d_idx, float* d_dist);
// Query lists (rows of d_idx/d_dist, NQ x K, indices of base points) merged with the
// bucket of base points each query is routed to.
bool ann_bucket_knn(Context& ctx, const float* d_points, int N, const float* d_queries, int NQ, int D,
                    int K, const TreeResult& tree, int* d_idx, float* d_dist);
bool explore_sweep(Context& ctx, const float* d_points, int N, int D, int K, const int* d_old_idx,
                   int* d_idx, float* d_dist, int row_begin, int row_end, int list_row0);
// rsfk_graph.cu: symmetric closure of a K-NN graph as CSR (offsets are 64-bit, [N+1])
bool symmetrize_count(Context& ctx, const int* d_idx, int N, int K, long long* d_offsets, long long* nnz_host);
bool symmetrize_fill(Context& ctx, const int* d_idx, const float* d_dist, int N, int K, const long long* d_offsets,
                     int* d_sym_idx, float* d_sym_dist);
// rsfk_kmeans.cu: Lloyd iterations from d_centroids (or from the means of the groups in
// d_labels); stops after max_iter iterations or when two assignments in a row agree
bool kmeans(Context& ctx, const float* d_points, int N, int D, int C, int max_iter, bool init_from_labels,
            float* d_centroids, int* d_labels, float* d_sq_dist, int* iterations);
bool merge_lists(Context& ctx, long long rows, int K, int G, const int* const* d_idx_lists,
                 const float* const* d_dist_lists, int* d_out_idx, float* d_out_dist);

} // namespace rsfk
