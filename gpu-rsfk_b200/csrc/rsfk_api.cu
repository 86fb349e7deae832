// C ABI of librsfk.so (declarations and reference citations: include/rsfk_b200.h).
#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <map>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include "../../include/rsfk_b200.h"
#include "rsfk_context.h"

using rsfk::Context;
using rsfk::TreeResult;

struct rsfk_ctx {
    Context c;
    TreeResult tree;
    bool has_tree = false;
    // Helper contexts (own stream, own scratch) that build part of a forest beside
    // this one on the same GPU; created on first use, destroyed with the context.
    std::vector<rsfk_ctx*> lanes;
    cudaEvent_t lane_ready = nullptr;
    int lanes_wanted = 0; // 0: the library's default (RSFK_LANES, else by the size of the call)
};

namespace {

std::mutex g_mutex;
rsfk_ctx* g_default = nullptr; // context behind the host-pointer entry points
int g_last_status = RSFK_OK;
std::string g_last_message;


// Host <-> device copies of caller-owned (pageable) arrays.  The driver's own
// pageable path moves about 10 GB/s here; four host threads that each pump their
// share of the array through two pinned 8 MiB buffers on a stream of their own
// overlap the host-side memcpy with the DMA and with each other.
class StagedCopier {
public:
    static constexpr int THREADS = 4;
    static constexpr size_t CHUNK = 8u << 20;
    bool ready = false;

    bool init()
    {
        if (ready) return true;
        for (int t = 0; t < THREADS; ++t) {
            if (cudaStreamCreateWithFlags(&stream_[t], cudaStreamNonBlocking) != cudaSuccess) return false;
            for (int b = 0; b < 2; ++b) {
                if (cudaMallocHost(&pinned_[t][b], CHUNK) != cudaSuccess) return false;
                if (cudaEventCreateWithFlags(&event_[t][b], cudaEventDisableTiming) != cudaSuccess) return false;
            }
        }
        ready = true;
        return true;
    }
    // to_device: host -> device, else device -> host.  Blocks until done.
    bool copy(void* dev, void* host, size_t bytes, bool to_device, int device)
    {
        if (bytes < 4 * CHUNK || !init()) {
            return cudaMemcpy(to_device ? dev : host, to_device ? host : dev, bytes,
                              to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost) == cudaSuccess;
        }
        const size_t n_chunks = (bytes + CHUNK - 1) / CHUNK;
        bool ok[THREADS];
        std::thread workers[THREADS];
        for (int t = 0; t < THREADS; ++t) {
            ok[t] = true;
            workers[t] = std::thread([&, t] {
                cudaSetDevice(device);
                int use = 0;
                size_t pending_off[2] = {0, 0}, pending_n[2] = {0, 0};
                auto drain = [&](int b) { // device -> host: finish the chunk that went through buffer b
                    if (pending_n[b] == 0) return;
                    if (cudaEventSynchronize(event_[t][b]) != cudaSuccess) ok[t] = false;
                    memcpy((char*)host + pending_off[b], pinned_[t][b], pending_n[b]);
                    pending_n[b] = 0;
                };
                for (size_t c = t; c < n_chunks; c += THREADS, use ^= 1) {
                    const size_t off = c * CHUNK, n = std::min(CHUNK, bytes - off);
                    if (to_device) {
                        if (cudaEventSynchronize(event_[t][use]) != cudaSuccess) ok[t] = false; // buffer free?
                        memcpy(pinned_[t][use], (const char*)host + off, n);
                        if (cudaMemcpyAsync((char*)dev + off, pinned_[t][use], n, cudaMemcpyHostToDevice, stream_[t]) != cudaSuccess)
                            ok[t] = false;
                    } else {
                        drain(use);
                        if (cudaMemcpyAsync(pinned_[t][use], (const char*)dev + off, n, cudaMemcpyDeviceToHost, stream_[t]) != cudaSuccess)
                            ok[t] = false;
                        pending_off[use] = off;
                        pending_n[use] = n;
                    }
                    cudaEventRecord(event_[t][use], stream_[t]);
                }
                if (!to_device) { drain(use); drain(use ^ 1); }
                if (cudaStreamSynchronize(stream_[t]) != cudaSuccess) ok[t] = false;
            });
        }
        bool all = true;
        for (int t = 0; t < THREADS; ++t) { workers[t].join(); all = all && ok[t]; }
        return all;
    }

private:
    cudaStream_t stream_[THREADS] = {};
    void* pinned_[THREADS][2] = {};
    cudaEvent_t event_[THREADS][2] = {};
};
StagedCopier g_copier;
// Copiers of the devices a multi-GPU call uses (streams and events belong to one device);
// entries are created before the per-GPU host threads start.
std::map<int, StagedCopier*> g_device_copier;

double now_s()
{
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

rsfk_ctx* make_ctx(int device, void* stream, bool private_stream)
{
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        fprintf(stderr, "rsfk: no CUDA device available\n");
        return nullptr;
    }
    if (device < 0 || device >= count) {
        fprintf(stderr, "rsfk: device %d out of range\n", device);
        return nullptr;
    }
    if (cudaSetDevice(device) != cudaSuccess) return nullptr;
    rsfk_ctx* h = new rsfk_ctx();
    h->c.device = device;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) h->c.sm_count = prop.multiProcessorCount;
    if (!private_stream) {
        h->c.stream = (cudaStream_t)stream; // NULL is the legacy default stream
        h->c.owns_stream = false;
    } else {
        if (cudaStreamCreateWithFlags(&h->c.stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete h;
            return nullptr;
        }
        h->c.owns_stream = true;
    }
    return h;
}

rsfk_ctx* default_ctx()
{
    if (!g_default) {
        int device = 0;
        if (const char* e = getenv("RSFK_DEVICE")) device = atoi(e);
        g_default = make_ctx(device, nullptr, true);
    }
    if (g_default) {
        cudaSetDevice(g_default->c.device);
        g_default->c.status = RSFK_OK;
        g_default->c.message.clear();
    }
    return g_default;
}

void publish(const Context& c)
{
    g_last_status = c.status;
    g_last_message = c.message;
}

// Number of lanes a forest is split over on one GPU.  The trees of a forest are
// independent and several of their kernels are latency-bound (the host round trip
// of every tree level, the first levels' small grids, the subtree kernel), so two
// tree sequences on two streams fill each other's gaps.  Each lane merges its trees
// into a list of its own; the lists are combined at the end, which gives the same
// rows as one sequence (the row of a point is the K smallest distinct of everything
// it met, in whatever order).  Three lanes by default: two sometimes fall into step
// with each other (both in the same phase at the same time) and then gain nothing.
// Lanes pay where a tree's kernels are short (a tree level of 1 M x 100 points takes 80 us);
// where every kernel already fills the GPU
// for a millisecond or more the sequences only compete for cache (measured: 1 M x 960
// 3.7 -> 4.7 s, 20 M x 128 22.2 -> 23.8 s with three lanes), so by default lanes are used up
// to 2^28 coordinates (1 GiB of points).  rsfk_ctx_set_lanes or RSFK_LANES set the number
// outright (1 = off, at most 4).  list_rows x K is the size of one list.
int forest_lanes(const rsfk_ctx* h, int n_trees, size_t N, int D, size_t list_rows, int K)
{
    static const int by_env = [] {
        const char* e = getenv("RSFK_LANES");
        const int v = e ? atoi(e) : 0;
        return v < 0 ? 0 : (v > 4 ? 4 : v);
    }();
    int g = h->lanes_wanted > 0 ? h->lanes_wanted : by_env;
    if (g == 0) {
        g = (N * (size_t)D <= ((size_t)1 << 28)) ? 3 : 1;
        // a lane's own list and the final combination want a few trees to pay for them
        // (eight ranks with six trees each: 46.3 ms with three lanes, 44.5 ms with one)
        while (g > 1 && n_trees < 4 * g) --g;
    }
    while (g > 1 && n_trees < 2 * g) --g; // at least two trees per lane
    // every lane holds a list of its own and tree scratch (about 64 bytes per point):
    // stay within half of the memory that is free now
    size_t free_b = 0, total_b = 0;
    if (g > 1 && cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) {
        const size_t per_lane = list_rows * (size_t)K * 8 + N * 64;
        size_t held = 0; // lanes that exist already hold their memory
        for (const rsfk_ctx* l : h->lanes)
            for (const auto& b : l->c.slots) held += b.bytes;
        held += h->c.slots[Context::LANE_IDX].bytes + h->c.slots[Context::LANE_DIST].bytes;
        while (g > 1 && per_lane * g > (free_b + held) / 2) --g;
    }
    return g;
}

// Rows 0-14 of the forest log for tree i of n_trees (layout: src/include/rsfk.h:274-392 of the
// reference, flattened [attribute][tree] as src/rsfk.cu:2148-2173 does; times in seconds).
// Attributes without a counterpart here stay 0: there is no "check active points" pass (a
// node's points are a contiguous segment), split pairs need no preprocessing (a counter hash
// inside the projection kernel draws them) and child nodes are created in the tail of the
// projection kernel, whose time is booked under "check points side".
void log_tree(float* log_forest, int n_trees, int i, const TreeResult& t, double build_s)
{
    if (!log_forest) return;
    log_forest[0 * n_trees + i] = (float)t.levels;
    log_forest[1 * n_trees + i] = (float)t.max_leaf;
    log_forest[2 * n_trees + i] = (float)t.min_leaf;
    log_forest[3 * n_trees + i] = (float)t.n_leaves;
    log_forest[4 * n_trees + i] = t.times.init_s;     // buffers, identity permutation, root
    log_forest[5 * n_trees + i] = (float)build_s;     // the whole build as the host saw it
    log_forest[7 * n_trees + i] = t.times.project_s;  // projection kernels (device)
    log_forest[8 * n_trees + i] = t.times.wait_s;     // host waiting for the levels' node counts
    log_forest[9 * n_trees + i] = t.times.alloc_s;    // growth of the scratch pool
    log_forest[12 * n_trees + i] = t.times.scatter_s; // partition kernels (device)
    log_forest[13 * n_trees + i] = t.times.subtree_s; // in-CTA subtrees down to the leaf buckets (device)
    log_forest[14 * n_trees + i] = t.times.end_s;     // counters read back, final synchronisation
}

void destroy_lanes(rsfk_ctx* h)
{
    for (rsfk_ctx* l : h->lanes) {
        cudaStreamSynchronize(l->c.stream);
        l->c.release();
        delete l;
    }
    h->lanes.clear();
    if (h->lane_ready) { cudaEventDestroy(h->lane_ready); h->lane_ready = nullptr; }
}

// One lane's share of a forest: trees lane, lane+G, ... of the call, on the lane's
// context and stream, merged into the lane's lists.
// With d_queries the lists are query lists (NQ rows) and every tree is followed by the
// query update instead of the bucket KNN.
// Stagger of the lanes: lane g+1 starts on the GPU when lane g has finished the level loop of
// its first tree (and goes on to the latency-bound subtree and bucket kernels), so that the
// lanes do not walk through the same phase side by side.
struct LaneStagger {
    std::vector<cudaEvent_t> levels_done; // per lane
    std::vector<std::atomic<int>> recorded;
    explicit LaneStagger(int G) : levels_done(G, nullptr), recorded(G)
    {
        for (int g = 0; g < G; ++g) {
            recorded[g].store(0);
            cudaEventCreateWithFlags(&levels_done[g], cudaEventDisableTiming);
        }
    }
    ~LaneStagger()
    {
        for (auto& e : levels_done)
            if (e) cudaEventDestroy(e);
    }
};

void lane_forest(rsfk_ctx* l, int lane, int G, const float* d_points, int N, int D, int K, int n_trees,
                 int first_tree, int tree_stride, int min_children, int max_children, int max_depth, int seed,
                 int* idx, float* dist, float* log_forest, int verbose, std::vector<cudaEvent_t>* ev,
                 const float* d_queries, int NQ, LaneStagger* stagger)
{
    Context& c = l->c;
    cudaSetDevice(c.device);
    if (stagger) {
        if (lane + 1 < G) { // the next lane waits for this one
            c.levels_done_event = stagger->levels_done[lane];
            c.levels_done_flag = &stagger->recorded[lane];
        }
        if (lane > 0) {
            // bounded host wait until the previous lane has recorded its event (or given up)
            const double t0 = now_s();
            while (stagger->recorded[lane - 1].load(std::memory_order_acquire) == 0 && now_s() - t0 < 0.2)
                std::this_thread::yield();
            if (stagger->recorded[lane - 1].load(std::memory_order_acquire) == 1)
                cudaStreamWaitEvent(c.stream, stagger->levels_done[lane - 1], 0);
        }
    }
    const bool keep_before = c.keep_index;
    c.keep_index = keep_before || d_queries != nullptr;
    bool ok = true;
    for (int i = lane; i < n_trees && ok; i += G) {
        const int t = first_tree + i * tree_stride;
        const double tb0 = now_s();
        ok = rsfk::tree_build(c, d_points, N, D, min_children, max_children, max_depth, seed + t, nullptr, 0,
                              l->tree);
        l->has_tree = ok;
        const double tb1 = now_s();
        c.stats.tree_build_us += (tb1 - tb0) * 1e6;
        if (!ok) break;
        cudaEventRecord((*ev)[2 * i], c.stream);
        ok = d_queries ? rsfk::ann_bucket_knn(c, d_points, N, d_queries, NQ, D, K, l->tree, idx, dist)
                       : rsfk::bucket_knn(c, d_points, N, D, K, l->tree, idx, dist);
        cudaEventRecord((*ev)[2 * i + 1], c.stream);
        log_tree(log_forest, n_trees, i, l->tree, tb1 - tb0);
        if (verbose >= 2)
            printf("tree %d: depth %d, leaves %d, leaf size %d..%d, build %.6f s\n", t, l->tree.levels,
                   l->tree.n_leaves, l->tree.min_leaf, l->tree.max_leaf, tb1 - tb0);
    }
    if (stagger && lane + 1 < G && stagger->recorded[lane].load() == 0)
        stagger->recorded[lane].store(2, std::memory_order_release); // nothing to wait for: this lane built no tree
    c.levels_done_event = nullptr;
    c.levels_done_flag = nullptr;
    ok = ok && c.check(cudaStreamSynchronize(c.stream), "forest lane");
    ok = ok && c.check_error_flag();
    c.resolve_ann_events();
    c.keep_index = keep_before;
}

bool run_forest_lanes(rsfk_ctx* h, int G, const float* d_points, int N, int D, int K, int n_trees,
                      int first_tree, int tree_stride, int min_children, int max_children, int max_depth,
                      int seed, int* d_idx, float* d_dist, float* log_forest, int verbose,
                      const float* d_queries = nullptr, int NQ = 0,
                      const std::function<bool()>* lists_ready = nullptr)
{
    Context& c = h->c;
    while ((int)h->lanes.size() < G) {
        rsfk_ctx* l = make_ctx(c.device, nullptr, true);
        if (!l) return c.fail(RSFK_ERR_CUDA, "forest lanes: no stream for a lane");
        h->lanes.push_back(l);
    }
    if (!h->lane_ready &&
        !c.check(cudaEventCreateWithFlags(&h->lane_ready, cudaEventDisableTiming), "cudaEventCreate"))
        return false;
    const long long list_rows = d_queries ? NQ : N;
    const size_t list_elems = (size_t)list_rows * K;
    // every lane works on a stream and lists of its own; the caller's stream only empties the
    // lane lists before and combines them with the caller's lists after
    int* lane_idx = (int*)c.scratch(Context::LANE_IDX, sizeof(int) * list_elems * G);
    float* lane_dist = (float*)c.scratch(Context::LANE_DIST, sizeof(float) * list_elems * G);
    if (!lane_idx || !lane_dist) return false;
    if (!rsfk::fill_empty_lists(c, lane_idx, lane_dist, (long long)list_elems * G)) return false;
    // the points and the emptied lane lists are ready once the main stream gets here
    cudaEventRecord(h->lane_ready, c.stream);
    std::vector<cudaEvent_t> ev(2 * (size_t)n_trees);
    for (auto& e : ev) cudaEventCreate(&e);
    if (log_forest) memset(log_forest, 0, sizeof(float) * (size_t)(16 * n_trees + 2));
    const double t0 = now_s();
    LaneStagger stagger(G);
    std::vector<std::thread> workers;
    for (int g = 0; g < G; ++g) {
        rsfk_ctx* l = h->lanes[g];
        l->c.status = RSFK_OK;
        l->c.message.clear();
        // a lane builds its trees as the caller's context would
        l->c.keep_index = c.keep_index;
        l->c.tc_mode = c.tc_mode;
        l->c.route_step_limit = c.route_step_limit;
        l->c.level_wait_ms = c.level_wait_ms;
        cudaStreamWaitEvent(l->c.stream, h->lane_ready, 0);
        if (g == 0) continue; // lane 0 runs on the calling thread
        workers.emplace_back(lane_forest, l, g, G, d_points, N, D, K, n_trees, first_tree, tree_stride,
                             min_children, max_children, max_depth, seed, lane_idx + list_elems * g,
                             lane_dist + list_elems * g, log_forest, verbose, &ev, d_queries, NQ, &stagger);
    }
    lane_forest(h->lanes[0], 0, G, d_points, N, D, K, n_trees, first_tree, tree_stride, min_children,
                max_children, max_depth, seed, lane_idx, lane_dist, log_forest, verbose, &ev, d_queries, NQ,
                &stagger);
    for (auto& w : workers) w.join();
    bool ok = c.status == RSFK_OK;
    for (int g = 0; g < G; ++g) {
        Context& lc = h->lanes[g]->c;
        if (ok && lc.status != RSFK_OK) ok = c.fail(lc.status, lc.message);
        c.stats.add(lc.stats);
        lc.stats = rsfk::Stats();
    }
    // the context's tree is the last one its first lane built; hyperplanes the context
    // materialised for an earlier tree do not belong to it
    h->tree = h->lanes[0]->tree;
    h->has_tree = ok && h->lanes[0]->has_tree;
    c.planes_ready = false;
    // the caller's lists take part from here on only
    if (lists_ready != nullptr && !(*lists_ready)()) ok = false;
    if (ok) {
        // every lane's stream is idle now; combine on the main stream, in place over the caller's lists
        const int* ip[5];
        const float* dp[5];
        ip[0] = d_idx;
        dp[0] = d_dist;
        for (int g = 0; g < G; ++g) {
            ip[g + 1] = lane_idx + list_elems * g;
            dp[g + 1] = lane_dist + list_elems * g;
        }
        ok = rsfk::merge_lists(c, list_rows, K, G + 1, ip, dp, d_idx, d_dist) &&
             c.check(cudaStreamSynchronize(c.stream), "forest merge");
    }
    if (ok && !d_queries)
        for (int i = 0; i < n_trees; ++i) {
            float ms = 0.0f;
            if (cudaEventElapsedTime(&ms, ev[2 * i], ev[2 * i + 1]) == cudaSuccess) {
                c.stats.bucket_knn_us += ms * 1e3;
                if (log_forest) log_forest[15 * n_trees + i] = ms * 1e-3f;
            }
        }
    for (auto& e : ev) cudaEventDestroy(e);
    if (log_forest) log_forest[16 * n_trees] = (float)(now_s() - t0);
    return ok;
}

// Trees + bucket KNN into canonical device lists; fills the ForestLog rows.
// lists_ready (optional) is called once, on the calling thread, before the first use of
// d_idx/d_dist: a host entry point finishes uploading the caller's lists there, so that the
// upload runs beside the trees when the forest works on lane lists of its own.
bool run_forest(rsfk_ctx* h, const float* d_points, int N, int D, int K, int n_trees, int first_tree,
                int tree_stride, int min_children, int max_children, int max_depth, int seed,
                int* d_idx, float* d_dist, float* log_forest, int verbose,
                const std::function<bool()>* lists_ready = nullptr)
{
    Context& c = h->c;
    {
        const int G = forest_lanes(h, n_trees, (size_t)N, D, (size_t)N, K);
        if (G > 1)
            return run_forest_lanes(h, G, d_points, N, D, K, n_trees, first_tree, tree_stride, min_children,
                                    max_children, max_depth, seed, d_idx, d_dist, log_forest, verbose,
                                    nullptr, 0, lists_ready);
    }
    if (lists_ready != nullptr && !(*lists_ready)()) return false;
    std::vector<cudaEvent_t> ev(2 * (size_t)n_trees);
    for (auto& e : ev) cudaEventCreate(&e);
    if (log_forest) memset(log_forest, 0, sizeof(float) * (size_t)(16 * n_trees + 2));
    const double t0 = now_s();
    bool ok = true;
    for (int i = 0; i < n_trees && ok; ++i) {
        const int t = first_tree + i * tree_stride;
        const double tb0 = now_s();
        ok = rsfk::tree_build(c, d_points, N, D, min_children, max_children, max_depth, seed + t,
                              nullptr, 0, h->tree);
        h->has_tree = ok;
        const double tb1 = now_s();
        c.stats.tree_build_us += (tb1 - tb0) * 1e6;
        if (!ok) break;
        cudaEventRecord(ev[2 * i], c.stream);
        ok = rsfk::bucket_knn(c, d_points, N, D, K, h->tree, d_idx, d_dist);
        cudaEventRecord(ev[2 * i + 1], c.stream);
        log_tree(log_forest, n_trees, i, h->tree, tb1 - tb0);
        if (verbose >= 2)
            printf("tree %d: depth %d, leaves %d, leaf size %d..%d, build %.6f s\n", t, h->tree.levels,
                   h->tree.n_leaves, h->tree.min_leaf, h->tree.max_leaf, tb1 - tb0);
    }
    ok = ok && c.check(cudaStreamSynchronize(c.stream), "forest");
    ok = ok && c.check_error_flag();
    if (ok)
        for (int i = 0; i < n_trees; ++i) {
            float ms = 0.0f;
            if (cudaEventElapsedTime(&ms, ev[2 * i], ev[2 * i + 1]) == cudaSuccess) {
                c.stats.bucket_knn_us += ms * 1e3;
                if (log_forest) log_forest[15 * n_trees + i] = ms * 1e-3f;
            }
        }
    for (auto& e : ev) cudaEventDestroy(e);
    if (log_forest) log_forest[16 * n_trees] = (float)(now_s() - t0);
    return ok;
}

// Query path: every tree is built over the base points with its index kept, the
// queries descend it and their lists take in the bucket they land in.
bool run_forest_ann(rsfk_ctx* h, const float* d_points, int N, const float* d_queries, int NQ, int D,
                    int K, int n_trees, int first_tree, int tree_stride, int min_children,
                    int max_children, int max_depth, int seed, int* d_idx, float* d_dist, int verbose)
{
    Context& c = h->c;
    {
        // lanes only on request (rsfk_ctx_set_lanes): the query update is issue-bound and takes
        // most of a tree's time here, so sequences side by side gain nothing (measured)
        const int G = h->lanes_wanted > 1 ? forest_lanes(h, n_trees, (size_t)N, D, (size_t)NQ, K) : 1;
        if (G > 1)
            return run_forest_lanes(h, G, d_points, N, D, K, n_trees, first_tree, tree_stride, min_children,
                                    max_children, max_depth, seed, d_idx, d_dist, nullptr, verbose, d_queries, NQ);
    }
    const bool keep_before = c.keep_index;
    c.keep_index = true;
    bool ok = true;
    for (int i = 0; i < n_trees && ok; ++i) {
        const int t = first_tree + i * tree_stride;
        const double tb0 = now_s();
        ok = rsfk::tree_build(c, d_points, N, D, min_children, max_children, max_depth, seed + t,
                              nullptr, 0, h->tree);
        h->has_tree = ok;
        c.stats.tree_build_us += (now_s() - tb0) * 1e6;
        if (!ok) break;
        ok = rsfk::ann_bucket_knn(c, d_points, N, d_queries, NQ, D, K, h->tree, d_idx, d_dist);
        if (verbose >= 2)
            printf("tree %d: depth %d, leaves %d, leaf size %d..%d, index rows %d\n", t, h->tree.levels,
                   h->tree.n_leaves, h->tree.min_leaf, h->tree.max_leaf, h->tree.n_records);
    }
    c.keep_index = keep_before;
    ok = ok && c.check(cudaStreamSynchronize(c.stream), "query forest");
    ok = ok && c.check_error_flag();
    return ok;
}

bool run_sweeps(rsfk_ctx* h, const float* d_points, int N, int D, int K, int sweeps, int* d_idx,
                float* d_dist)
{
    Context& c = h->c;
    if (sweeps <= 0) return true;
    int* snap = (int*)c.scratch(Context::SNAPSHOT, sizeof(int) * (size_t)N * K);
    if (!snap) return false;
    for (int s = 0; s < sweeps; ++s) {
        if (!c.check(cudaMemcpyAsync(snap, d_idx, sizeof(int) * (size_t)N * K, cudaMemcpyDeviceToDevice,
                                     c.stream), "snapshot"))
            return false;
        if (!rsfk::explore_sweep(c, d_points, N, D, K, snap, d_idx, d_dist, 0, N, 0)) return false;
    }
    return true;
}

// ---------------------------------------------------------------------------
// Several GPUs inside one host-pointer call (one process, one host thread per GPU).
// The trees of the forest are dealt out round-robin; every GPU holds all the points
// (its own slice uploaded over PCIe, the others' fetched from their owners over
// NVLink) and builds its trees into lists of its own.  GPU g then owns rows
// [N g / G, N (g+1) / G): it fetches those rows of every other GPU's lists, merges
// them with its own and with the caller's, runs the sweeps on them (a sweep's
// snapshot of the whole graph is gathered from the owners) and writes them back to
// the caller.  The lists are canonical, so the result is the one a single GPU gives,
// bit for bit.
// ---------------------------------------------------------------------------
std::vector<int> g_devices;                  // rsfk_set_devices
std::map<int, rsfk_ctx*> g_device_ctx;       // one context per device used that way

std::vector<int> devices_for_call()
{
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) count = 0;
    std::vector<int> devs = g_devices;
    if (devs.empty()) {
        if (const char* e = getenv("RSFK_DEVICES")) {
            for (const char* p = e; *p;) {
                char* end = nullptr;
                const long v = strtol(p, &end, 10);
                if (end == p) break;
                devs.push_back((int)v);
                p = *end == ',' ? end + 1 : end;
            }
        } else if (const char* e = getenv("RSFK_NUM_GPUS")) {
            const int n = std::min(atoi(e), count);
            for (int g = 0; g < n; ++g) devs.push_back(g);
        }
    }
    for (int d : devs)
        if (d < 0 || d >= count) return {}; // a list that names a missing device is ignored
    std::sort(devs.begin(), devs.end());
    devs.erase(std::unique(devs.begin(), devs.end()), devs.end());
    return devs;
}

// Rendezvous of the per-GPU host threads; a failure anywhere is seen by everybody at
// the next rendezvous, where they all leave together.
struct HostBarrier {
    explicit HostBarrier(int n) : n_(n) {}
    bool wait(bool my_ok)
    {
        std::unique_lock<std::mutex> lock(m_);
        ok_ = ok_ && my_ok;
        if (++waiting_ == n_) {
            waiting_ = 0;
            ++phase_;
            cv_.notify_all();
        } else {
            const int p = phase_;
            cv_.wait(lock, [&] { return phase_ != p; });
        }
        return ok_;
    }
private:
    std::mutex m_;
    std::condition_variable cv_;
    int n_, waiting_ = 0, phase_ = 0;
    bool ok_ = true;
};

struct DeviceShare {
    rsfk_ctx* h = nullptr;
    float* d_points = nullptr;
    int* d_idx = nullptr;
    float* d_dist = nullptr;
    std::vector<float> log;   // this GPU's trees, [attribute][tree] as the caller's log
    int n_trees = 0;
};

void knn_on_devices(const std::vector<int>& devs, int n_trees, int K, int N, int D, int min_children,
                    int max_children, int max_depth, int verbose, int seed, int sweeps, float* points,
                    int* knn_indices, float* knn_sqr_distances, float* log_forest)
{
    const int G = (int)devs.size();
    std::vector<DeviceShare> share(G);
    for (int g = 0; g < G; ++g) {
        auto it = g_device_ctx.find(devs[g]);
        if (it == g_device_ctx.end()) {
            rsfk_ctx* h = make_ctx(devs[g], nullptr, true);
            if (!h) {
                g_last_status = RSFK_ERR_CUDA;
                g_last_message = "no usable CUDA device";
                return;
            }
            it = g_device_ctx.emplace(devs[g], h).first;
        }
        // direct copies from the other GPUs' memory where the machine allows it (every call: the
        // list of devices may have grown; asking again for access that exists is an error to forget)
        cudaSetDevice(devs[g]);
        for (int p = 0; p < G; ++p) {
            int can = 0;
            if (p != g && cudaDeviceCanAccessPeer(&can, devs[g], devs[p]) == cudaSuccess && can)
                if (cudaDeviceEnablePeerAccess(devs[p], 0) != cudaSuccess) cudaGetLastError();
        }
        if (!g_device_copier.count(devs[g])) g_device_copier[devs[g]] = new StagedCopier();
        share[g].h = it->second;
        share[g].h->c.status = RSFK_OK;
        share[g].h->c.message.clear();
        share[g].n_trees = n_trees > g ? (n_trees - g + G - 1) / G : 0;
        share[g].log.assign((size_t)16 * share[g].n_trees + 2, 0.0f);
    }
    auto row_lo = [&](int g) { return (long long)N * g / G; };
    HostBarrier barrier(G);
    double t_forest = 0.0, t_sweeps = 0.0;
    const double t_begin = now_s();

    auto body = [&](int g) {
        DeviceShare& me = share[g];
        Context& c = me.h->c;
        const int dev = c.device;
        cudaSetDevice(dev);
        const long long lo = row_lo(g), hi = row_lo(g + 1), rows = hi - lo;
        const size_t list_elems = (size_t)N * K;
        long long max_rows = 0;
        for (int p = 0; p < G; ++p) max_rows = std::max(max_rows, row_lo(p + 1) - row_lo(p));
        const size_t stage_elems = (size_t)max_rows * K;
        me.d_points = (float*)c.scratch(Context::HOST_POINTS, sizeof(float) * (size_t)N * D);
        me.d_idx = (int*)c.scratch(Context::HOST_IDX, sizeof(int) * list_elems);
        me.d_dist = (float*)c.scratch(Context::HOST_DIST, sizeof(float) * list_elems);
        // rows [lo, hi) of the G-1 other GPUs' lists and of the caller's
        int* peer_idx = (int*)c.scratch(Context::PEER_IDX, sizeof(int) * stage_elems * G);
        float* peer_dist = (float*)c.scratch(Context::PEER_DIST, sizeof(float) * stage_elems * G);
        bool ok = me.d_points && me.d_idx && me.d_dist && peer_idx && peer_dist;
        StagedCopier* copier = g_device_copier.find(dev)->second; // the map is not modified while the threads run
        auto copy = [&](void* d, void* h, size_t n, bool to_device, const char* what) {
            if (n == 0) return true;
            if (copier->copy(d, h, n, to_device, dev)) return true;
            return c.fail(RSFK_ERR_CUDA, std::string(what) + " failed");
        };
        // 1. this GPU's slice of the points
        ok = ok && copy(me.d_points + (size_t)lo * D, points + (size_t)lo * D, sizeof(float) * (size_t)rows * D, true,
                        "H2D points");
        if (!barrier.wait(ok)) return;
        // the caller's lists for this GPU's rows are needed at the merge only: they travel beside the trees
        bool lists_up = true;
        std::thread uploader([&] {
            cudaSetDevice(dev);
            if (rows > 0) // the context's status belongs to the GPU's own thread: only the flag is set here
                lists_up = copier->copy(peer_idx + stage_elems * (G - 1), knn_indices + (size_t)lo * K,
                                        sizeof(int) * (size_t)rows * K, true, dev) &&
                           copier->copy(peer_dist + stage_elems * (G - 1), knn_sqr_distances + (size_t)lo * K,
                                        sizeof(float) * (size_t)rows * K, true, dev);
        });
        // 2. the other slices from their owners
        for (int p = 0; p < G && ok; ++p) {
            if (p == g) continue;
            const long long plo = row_lo(p), prow = row_lo(p + 1) - plo;
            if (prow > 0)
                ok = c.check(cudaMemcpyPeerAsync(me.d_points + (size_t)plo * D, dev, share[p].d_points + (size_t)plo * D,
                                                 share[p].h->c.device, sizeof(float) * (size_t)prow * D, c.stream),
                             "points from a peer");
        }
        // 3. this GPU's trees into empty lists
        const double t0 = now_s();
        ok = ok && rsfk::fill_empty_lists(c, me.d_idx, me.d_dist, (long long)list_elems);
        ok = ok && run_forest(me.h, me.d_points, N, D, K, me.n_trees, g, G, min_children, max_children, max_depth,
                              seed, me.d_idx, me.d_dist, me.log.data(), g == 0 ? verbose : 0, nullptr);
        ok = ok && c.check(cudaStreamSynchronize(c.stream), "forest");
        uploader.join();
        if (!lists_up) ok = c.fail(RSFK_ERR_CUDA, "H2D lists failed");
        if (!barrier.wait(ok)) return;
        if (g == 0) t_forest = now_s() - t0;
        // 4. rows [lo, hi) of everybody's lists, merged in place over this GPU's own
        {
            const int* ip[10];
            const float* dp[10];
            int n_lists = 0;
            ip[n_lists] = me.d_idx + (size_t)lo * K;
            dp[n_lists++] = me.d_dist + (size_t)lo * K;
            int slot = 0;
            for (int p = 0; p < G && ok && rows > 0; ++p) {
                if (p == g) continue;
                int* si = peer_idx + stage_elems * slot;
                float* sd = peer_dist + stage_elems * slot;
                ok = c.check(cudaMemcpyPeerAsync(si, dev, share[p].d_idx + (size_t)lo * K, share[p].h->c.device,
                                                 sizeof(int) * (size_t)rows * K, c.stream), "lists from a peer") &&
                     c.check(cudaMemcpyPeerAsync(sd, dev, share[p].d_dist + (size_t)lo * K, share[p].h->c.device,
                                                 sizeof(float) * (size_t)rows * K, c.stream), "lists from a peer");
                ip[n_lists] = si;
                dp[n_lists++] = sd;
                ++slot;
            }
            // the caller's rows in canonical form
            ok = ok && rsfk::sort_rows(c, peer_idx + stage_elems * (G - 1), peer_dist + stage_elems * (G - 1), rows, K);
            ip[n_lists] = peer_idx + stage_elems * (G - 1);
            dp[n_lists++] = peer_dist + stage_elems * (G - 1);
            ok = ok && rsfk::merge_lists(c, rows, K, n_lists, ip, dp, me.d_idx + (size_t)lo * K,
                                         me.d_dist + (size_t)lo * K);
            ok = ok && c.check(cudaStreamSynchronize(c.stream), "list exchange");
        }
        if (!barrier.wait(ok)) return;
        // 5. sweeps over this GPU's rows; the snapshot of the whole graph comes from the owners
        const double t1 = now_s();
        int* snap = sweeps > 0 ? (int*)c.scratch(Context::SNAPSHOT, sizeof(int) * list_elems) : nullptr;
        ok = ok && (sweeps <= 0 || snap != nullptr);
        for (int s = 0; s < sweeps; ++s) {
            for (int p = 0; p < G && ok; ++p) {
                const long long plo = row_lo(p), prow = row_lo(p + 1) - plo;
                if (prow <= 0) continue;
                ok = c.check(cudaMemcpyPeerAsync(snap + (size_t)plo * K, dev, share[p].d_idx + (size_t)plo * K,
                                                 share[p].h->c.device, sizeof(int) * (size_t)prow * K, c.stream),
                             "snapshot");
            }
            ok = ok && c.check(cudaStreamSynchronize(c.stream), "snapshot");
            if (!barrier.wait(ok)) return; // nobody changes its rows before everybody has the snapshot
            if (rows > 0)
                ok = rsfk::explore_sweep(c, me.d_points, N, D, K, snap, me.d_idx, me.d_dist, (int)lo, (int)hi, 0);
            ok = ok && c.check(cudaStreamSynchronize(c.stream), "exploration");
            if (!barrier.wait(ok)) return;
        }
        ok = ok && c.check_error_flag();
        if (g == 0) t_sweeps = now_s() - t1;
        // 6. this GPU's rows back to the caller
        ok = ok && copy(me.d_idx + (size_t)lo * K, knn_indices + (size_t)lo * K, sizeof(int) * (size_t)rows * K, false,
                        "D2H indices");
        ok = ok && copy(me.d_dist + (size_t)lo * K, knn_sqr_distances + (size_t)lo * K,
                        sizeof(float) * (size_t)rows * K, false, "D2H distances");
        barrier.wait(ok);
    };

    std::vector<std::thread> workers;
    for (int g = 1; g < G; ++g) workers.emplace_back(body, g);
    body(0);
    for (auto& w : workers) w.join();

    g_last_status = RSFK_OK;
    g_last_message.clear();
    for (int g = 0; g < G; ++g) {
        const Context& c = share[g].h->c;
        if (c.status != RSFK_OK && g_last_status == RSFK_OK) publish(c);
    }
    if (log_forest) {
        memset(log_forest, 0, sizeof(float) * (size_t)(16 * n_trees + 2));
        for (int g = 0; g < G; ++g)
            for (int i = 0; i < share[g].n_trees; ++i)
                for (int a = 0; a < 16; ++a)
                    log_forest[(size_t)a * n_trees + g + (size_t)i * G] = share[g].log[(size_t)a * share[g].n_trees + i];
        log_forest[16 * n_trees] = (float)t_forest;
        log_forest[16 * n_trees + 1] = (float)t_sweeps;
    }
    if (verbose >= 1 && g_last_status == RSFK_OK) {
        printf("Creating RSFK forest takes %lf seconds\n", t_forest);
        printf("Nearest Neighbors Exploring computation Kernel takes %lf seconds\n", t_sweeps);
        printf("%d GPUs, whole call %lf seconds\n", G, now_s() - t_begin);
    }
}

} // namespace

extern "C" {

int rsfk_last_status(void) { return g_last_status; }
const char* rsfk_last_message(void) { return g_last_message.c_str(); }
void rsfk_free(void* p) { free(p); }
int rsfk_max_neighbors(void) { return rsfk::list_capacity(); }

void rsfk_release_memory(void)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    std::vector<rsfk_ctx*> all;
    if (g_default) all.push_back(g_default);
    for (auto& kv : g_device_ctx) all.push_back(kv.second);
    for (rsfk_ctx* h : all) {
        cudaSetDevice(h->c.device);
        cudaStreamSynchronize(h->c.stream);
        destroy_lanes(h);
        for (auto& b : h->c.slots) {
            if (b.ptr) cudaFree(b.ptr);
            b.ptr = nullptr;
            b.bytes = 0;
        }
        h->has_tree = false;
    }
    if (g_default) cudaSetDevice(g_default->c.device);
}

int rsfk_set_devices(int n, const int* devices)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    if (n < 0 || n > 8 || (n > 0 && !devices)) return RSFK_ERR_ARG;
    if (n == 0) { // back to one GPU; needs no device to say so
        g_devices.clear();
        return RSFK_OK;
    }
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) return RSFK_ERR_ARG;
    for (int i = 0; i < n; ++i)
        if (devices[i] < 0 || devices[i] >= count) return RSFK_ERR_ARG;
    g_devices.assign(devices, devices + n);
    return RSFK_OK;
}

long long rsfk_kernel_launches(void) { return rsfk::g_kernel_launches.load(); }

void pymodule_rsfk_knn(int n_trees, int num_neighbors, int N, int D, int MIN_TREE_CHILD,
                       int MAX_TREE_CHILD, int MAX_DEPTH, int VERBOSE, int RANDOM_STATE,
                       int nn_exploring_factor, float* points, int* knn_indices,
                       float* knn_sqr_distances, float* log_forest)
{
    rsfk::TraceRange trace("pymodule_rsfk_knn");
    std::lock_guard<std::mutex> lock(g_mutex);
    rsfk_ctx* h = default_ctx();
    if (!h) {
        g_last_status = RSFK_ERR_CUDA;
        g_last_message = "no usable CUDA device";
        return;
    }
    Context& c = h->c;
    const int K = num_neighbors;
    if (N <= 0 || D <= 0 || K <= 0 || n_trees < 0 || !points || !knn_indices || !knn_sqr_distances) {
        c.fail(RSFK_ERR_ARG, "pymodule_rsfk_knn: invalid argument");
        publish(c);
        return;
    }
    if (K > rsfk::list_capacity()) {
        c.fail(RSFK_ERR_UNSUPPORTED, "pymodule_rsfk_knn: K above 256 is not supported");
        publish(c);
        return;
    }
    {
        // several GPUs when the caller asked for them (rsfk_set_devices, RSFK_DEVICES, RSFK_NUM_GPUS)
        const std::vector<int> devs = devices_for_call();
        if (devs.size() > 1 && (long long)N >= (long long)devs.size()) {
            knn_on_devices(devs, n_trees, K, N, D, MIN_TREE_CHILD, MAX_TREE_CHILD, MAX_DEPTH, VERBOSE, RANDOM_STATE,
                           nn_exploring_factor, points, knn_indices, knn_sqr_distances, log_forest);
            return;
        }
    }
    const size_t pts_bytes = sizeof(float) * (size_t)N * D, list_elems = (size_t)N * K;
    const double ta0 = now_s();
    float* d_points = nullptr;
    int* d_idx = nullptr;
    float* d_dist = nullptr;
    // device copies live in the context's grow-only pool: no cudaMalloc/cudaFree per call
    // (rsfk_release_memory() returns the pool to the driver)
    d_points = (float*)c.scratch(Context::HOST_POINTS, pts_bytes);
    d_idx = (int*)c.scratch(Context::HOST_IDX, sizeof(int) * list_elems);
    d_dist = (float*)c.scratch(Context::HOST_DIST, sizeof(float) * list_elems);
    bool ok = d_points && d_idx && d_dist;
    if (ok && VERBOSE >= 1) printf("Device allocations take %lf seconds\n", now_s() - ta0);
    const int dev_id = c.device;
    auto h2d = [&](void* d, void* h, size_t n, const char* what) {
        if (g_copier.copy(d, h, n, true, dev_id)) return true;
        return c.fail(RSFK_ERR_CUDA, std::string(what) + " failed");
    };
    auto d2h = [&](void* d, void* h, size_t n, const char* what) {
        if (g_copier.copy(d, h, n, false, dev_id)) return true;
        return c.fail(RSFK_ERR_CUDA, std::string(what) + " failed");
    };
    const double th0 = now_s();
    ok = ok && h2d(d_points, points, pts_bytes, "H2D points");
    const double t0 = now_s();
    if (ok && VERBOSE >= 1) printf("Host to device copy of the points takes %lf seconds\n", t0 - th0);
    // The caller's lists are needed only where the forest first touches them (with lanes: at the
    // final combination), so they travel on a thread of their own beside the trees.
    bool lists_up = true, joined = true;
    std::thread uploader;
    if (ok) {
        joined = false;
        uploader = std::thread([&] {
            cudaSetDevice(dev_id);
            lists_up = g_copier.copy(d_idx, knn_indices, sizeof(int) * list_elems, true, dev_id) &&
                       g_copier.copy(d_dist, knn_sqr_distances, sizeof(float) * list_elems, true, dev_id);
        });
    }
    const std::function<bool()> lists_ready = [&]() -> bool {
        if (!joined) { uploader.join(); joined = true; }
        if (!lists_up) return c.fail(RSFK_ERR_CUDA, "H2D lists failed");
        return rsfk::sort_rows(c, d_idx, d_dist, N, K);
    };
    ok = ok && run_forest(h, d_points, N, D, K, n_trees, 0, 1, MIN_TREE_CHILD, MAX_TREE_CHILD, MAX_DEPTH,
                          RANDOM_STATE, d_idx, d_dist, log_forest, VERBOSE, &lists_ready);
    if (!joined) { uploader.join(); joined = true; }
    const double t1 = now_s();
    if (ok && VERBOSE >= 1) printf("Creating RSFK forest takes %lf seconds\n", t1 - t0);
    ok = ok && run_sweeps(h, d_points, N, D, K, nn_exploring_factor, d_idx, d_dist);
    ok = ok && c.check(cudaStreamSynchronize(c.stream), "exploration");
    const double t2 = now_s();
    if (ok && VERBOSE >= 1)
        printf("Nearest Neighbors Exploring computation Kernel takes %lf seconds\n", t2 - t1);
    if (ok && log_forest) log_forest[16 * n_trees + 1] = (float)(t2 - t1);
    // outputs are written only when every step succeeded
    ok = ok && d2h(d_idx, knn_indices, sizeof(int) * list_elems, "D2H indices");
    ok = ok && d2h(d_dist, knn_sqr_distances, sizeof(float) * list_elems, "D2H distances");
    ok = ok && c.check(cudaStreamSynchronize(c.stream), "D2H");
    if (ok && VERBOSE >= 1) printf("Device to host copies take %lf seconds\n", now_s() - t2);
    cudaStreamSynchronize(c.stream);
    publish(c);
}

void pymodule_cluster_by_sample_tree(int N, int D, int MIN_TREE_CHILD, int MAX_TREE_CHILD,
                                     int MAX_DEPTH, int VERBOSE, int RANDOM_STATE, float* points,
                                     int** nodes_buckets, int** bucket_sizes, int* total_leaves,
                                     int* max_child)
{
    rsfk::TraceRange trace("pymodule_cluster_by_sample_tree");
    std::lock_guard<std::mutex> lock(g_mutex);
    rsfk_ctx* h = default_ctx();
    if (!h) {
        g_last_status = RSFK_ERR_CUDA;
        g_last_message = "no usable CUDA device";
        return;
    }
    Context& c = h->c;
    if (N <= 0 || D <= 0 || !points || !nodes_buckets || !bucket_sizes || !total_leaves || !max_child) {
        c.fail(RSFK_ERR_ARG, "pymodule_cluster_by_sample_tree: invalid argument");
        publish(c);
        return;
    }
    const double t0 = now_s();
    float* d_points = nullptr;
    d_points = (float*)c.scratch(Context::HOST_POINTS, sizeof(float) * (size_t)N * D);
    bool ok = d_points != nullptr;
    ok = ok && c.check(cudaMemcpyAsync(d_points, points, sizeof(float) * (size_t)N * D, cudaMemcpyHostToDevice, c.stream), "H2D points");
    ok = ok && rsfk::tree_build(c, d_points, N, D, MIN_TREE_CHILD, MAX_TREE_CHILD, MAX_DEPTH, RANDOM_STATE,
                                nullptr, 0, h->tree);
    h->has_tree = ok;
    if (ok) {
        const TreeResult& t = h->tree;
        std::vector<int> perm(N), ls(t.n_leaves), lc(t.n_leaves);
        ok = c.check(cudaMemcpyAsync(perm.data(), t.perm, sizeof(int) * (size_t)N, cudaMemcpyDeviceToHost, c.stream), "D2H perm") &&
             c.check(cudaMemcpyAsync(ls.data(), t.leaf_start, sizeof(int) * (size_t)t.n_leaves, cudaMemcpyDeviceToHost, c.stream), "D2H leaves") &&
             c.check(cudaMemcpyAsync(lc.data(), t.leaf_count, sizeof(int) * (size_t)t.n_leaves, cudaMemcpyDeviceToHost, c.stream), "D2H leaves") &&
             c.check(cudaStreamSynchronize(c.stream), "D2H tree");
        if (ok) {
            std::vector<int> order(t.n_leaves);
            for (int i = 0; i < t.n_leaves; ++i) order[i] = i;
            std::sort(order.begin(), order.end(), [&](int a, int b) { return ls[a] < ls[b]; });
            const int mc = t.max_leaf;
            int* table = (int*)malloc(sizeof(int) * (size_t)std::max(1, t.n_leaves) * (size_t)std::max(1, mc));
            int* sizes = (int*)malloc(sizeof(int) * (size_t)std::max(1, t.n_leaves));
            if (!table || !sizes) {
                free(table);
                free(sizes);
                ok = c.fail(RSFK_ERR_NOMEM, "pymodule_cluster_by_sample_tree: malloc failed");
            } else {
                for (int b = 0; b < t.n_leaves; ++b) {
                    const int s = ls[order[b]], n = lc[order[b]];
                    sizes[b] = n;
                    memcpy(table + (size_t)b * mc, perm.data() + s, sizeof(int) * (size_t)n);
                    for (int k = n; k < mc; ++k) table[(size_t)b * mc + k] = -1;
                }
                *nodes_buckets = table;
                *bucket_sizes = sizes;
                *total_leaves = t.n_leaves;
                *max_child = mc;
                if (VERBOSE >= 1) {
                    printf("Tree depth: %d\nMax child count: %d\nMin child count: %d\nTotal leaves: %d\n",
                           t.levels, t.max_leaf, t.min_leaf, t.n_leaves);
                    printf("Creating cluster with one tree takes %lf seconds\n", now_s() - t0);
                }
            }
        }
    }
    cudaStreamSynchronize(c.stream);
    publish(c);
}

void pymodule_rsfk_knn_ann(int n_trees, int num_neighbors, int N, int NQ, int D, int MIN_TREE_CHILD,
                           int MAX_TREE_CHILD, int MAX_DEPTH, int VERBOSE, int RANDOM_STATE,
                           int nn_exploring_factor, float* points, float* query_points,
                           int* knn_indices, float* knn_sqr_distances, float* log_forest)
{
    rsfk::TraceRange trace("pymodule_rsfk_knn_ann");
    (void)nn_exploring_factor; // the reference's query path runs no exploration (src/rsfk.cu:98-152)
    (void)log_forest;          // nor does it write the log (its ForestLog is a local, src/rsfk.cu:169)
    std::lock_guard<std::mutex> lock(g_mutex);
    rsfk_ctx* h = default_ctx();
    if (!h) {
        g_last_status = RSFK_ERR_CUDA;
        g_last_message = "no usable CUDA device";
        return;
    }
    Context& c = h->c;
    const int K = num_neighbors;
    if (N <= 0 || NQ <= 0 || D <= 0 || K <= 0 || n_trees < 0 || !points || !query_points || !knn_indices ||
        !knn_sqr_distances) {
        c.fail(RSFK_ERR_ARG, "pymodule_rsfk_knn_ann: invalid argument");
        publish(c);
        return;
    }
    if (K > rsfk::list_capacity()) {
        c.fail(RSFK_ERR_UNSUPPORTED, "pymodule_rsfk_knn_ann: K above 256 is not supported");
        publish(c);
        return;
    }
    const size_t pts_bytes = sizeof(float) * (size_t)N * D, q_bytes = sizeof(float) * (size_t)NQ * D;
    const size_t list_elems = (size_t)NQ * K;
    float* d_points = (float*)c.scratch(Context::HOST_POINTS, pts_bytes);
    float* d_queries = (float*)c.scratch(Context::HOST_QUERIES, q_bytes);
    int* d_idx = (int*)c.scratch(Context::HOST_IDX, sizeof(int) * list_elems);
    float* d_dist = (float*)c.scratch(Context::HOST_DIST, sizeof(float) * list_elems);
    bool ok = d_points && d_queries && d_idx && d_dist;
    const int dev_id = c.device;
    auto h2d = [&](void* d, void* hp, size_t n, const char* what) {
        if (g_copier.copy(d, hp, n, true, dev_id)) return true;
        return c.fail(RSFK_ERR_CUDA, std::string(what) + " failed");
    };
    auto d2h = [&](void* d, void* hp, size_t n, const char* what) {
        if (g_copier.copy(d, hp, n, false, dev_id)) return true;
        return c.fail(RSFK_ERR_CUDA, std::string(what) + " failed");
    };
    const double t0 = now_s();
    ok = ok && h2d(d_points, points, pts_bytes, "H2D points");
    ok = ok && h2d(d_queries, query_points, q_bytes, "H2D query points");
    const double t1 = now_s();
    if (ok && VERBOSE >= 2) printf("Allocate+copy points takes: %lf seconds\n", t1 - t0);
    // The trees work on lists of their own that start empty on the device; the caller's lists
    // travel beside them on a thread of their own and are combined with the result at the end
    // (a row is the K smallest distinct of everything it met, in whatever order).
    int* d_work_idx = (int*)c.scratch(Context::LANE_IDX, sizeof(int) * list_elems);
    float* d_work_dist = (float*)c.scratch(Context::LANE_DIST, sizeof(float) * list_elems);
    ok = ok && d_work_idx && d_work_dist && rsfk::fill_empty_lists(c, d_work_idx, d_work_dist, (long long)list_elems);
    bool lists_up = true;
    std::thread uploader;
    if (ok)
        uploader = std::thread([&] {
            cudaSetDevice(dev_id);
            lists_up = g_copier.copy(d_idx, knn_indices, sizeof(int) * list_elems, true, dev_id) &&
                       g_copier.copy(d_dist, knn_sqr_distances, sizeof(float) * list_elems, true, dev_id);
        });
    // lanes, when asked for, keep their lists in the same scratch slots: one sequence here
    const int lanes_before = h->lanes_wanted;
    h->lanes_wanted = 1;
    ok = ok && run_forest_ann(h, d_points, N, d_queries, NQ, D, K, n_trees, 0, 1, MIN_TREE_CHILD,
                              MAX_TREE_CHILD, MAX_DEPTH, RANDOM_STATE, d_work_idx, d_work_dist, VERBOSE);
    h->lanes_wanted = lanes_before;
    if (uploader.joinable()) uploader.join();
    if (ok && !lists_up) ok = c.fail(RSFK_ERR_CUDA, "H2D lists failed");
    ok = ok && rsfk::sort_rows(c, d_idx, d_dist, NQ, K);
    if (ok) {
        const int* ip[2] = {d_idx, d_work_idx};
        const float* dp[2] = {d_dist, d_work_dist};
        ok = rsfk::merge_lists(c, NQ, K, 2, ip, dp, d_idx, d_dist) &&
             c.check(cudaStreamSynchronize(c.stream), "list combination");
    }
    const double t2 = now_s();
    if (ok && VERBOSE >= 1) printf("Creating RSFK forest and updating the query lists takes %lf seconds\n", t2 - t1);
    // outputs are written only when every step succeeded
    ok = ok && d2h(d_idx, knn_indices, sizeof(int) * list_elems, "D2H indices");
    ok = ok && d2h(d_dist, knn_sqr_distances, sizeof(float) * list_elems, "D2H distances");
    ok = ok && c.check(cudaStreamSynchronize(c.stream), "D2H");
    if (ok && VERBOSE >= 2) printf("Copy KNN takes: %lf seconds\n", now_s() - t2);
    cudaStreamSynchronize(c.stream);
    publish(c);
}

void rsfk_kmeans(int N, int D, int C, int max_iter, int init_from_labels, float* points, float* centroids,
                 int* labels, float* sq_dist, int* iterations)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    rsfk_ctx* h = default_ctx();
    if (!h) {
        g_last_status = RSFK_ERR_CUDA;
        g_last_message = "no usable CUDA device";
        return;
    }
    Context& c = h->c;
    if (N <= 0 || D <= 0 || C <= 0 || C > N || max_iter < 0 || !points || !centroids || !labels || !sq_dist) {
        c.fail(RSFK_ERR_ARG, "rsfk_kmeans: invalid argument");
        publish(c);
        return;
    }
    if (init_from_labels)
        for (int p = 0; p < N; ++p)
            if (labels[p] < 0 || labels[p] >= C) {
                c.fail(RSFK_ERR_ARG, "rsfk_kmeans: a label is outside [0, n_clusters)");
                publish(c);
                return;
            }
    float* d_points = (float*)c.scratch(Context::KM_POINTS, sizeof(float) * (size_t)N * D);
    float* d_cent = (float*)c.scratch(Context::KM_CENTROIDS, sizeof(float) * (size_t)C * D);
    int* d_labels = (int*)c.scratch(Context::KM_LABELS, sizeof(int) * (size_t)N);
    float* d_dist = (float*)c.scratch(Context::KM_DIST, sizeof(float) * (size_t)N);
    bool ok = d_points && d_cent && d_labels && d_dist;
    ok = ok && c.check(cudaMemcpyAsync(d_points, points, sizeof(float) * (size_t)N * D, cudaMemcpyHostToDevice, c.stream), "H2D points");
    ok = ok && c.check(cudaMemcpyAsync(d_cent, centroids, sizeof(float) * (size_t)C * D, cudaMemcpyHostToDevice, c.stream), "H2D centroids");
    if (init_from_labels)
        ok = ok && c.check(cudaMemcpyAsync(d_labels, labels, sizeof(int) * (size_t)N, cudaMemcpyHostToDevice, c.stream), "H2D labels");
    int done = 0;
    ok = ok && rsfk::kmeans(c, d_points, N, D, C, max_iter, init_from_labels != 0, d_cent, d_labels, d_dist, &done);
    // outputs are written only when every step succeeded
    ok = ok && c.check(cudaStreamSynchronize(c.stream), "kmeans");
    ok = ok && c.check(cudaMemcpyAsync(centroids, d_cent, sizeof(float) * (size_t)C * D, cudaMemcpyDeviceToHost, c.stream), "D2H centroids");
    ok = ok && c.check(cudaMemcpyAsync(labels, d_labels, sizeof(int) * (size_t)N, cudaMemcpyDeviceToHost, c.stream), "D2H labels");
    ok = ok && c.check(cudaMemcpyAsync(sq_dist, d_dist, sizeof(float) * (size_t)N, cudaMemcpyDeviceToHost, c.stream), "D2H distances");
    ok = ok && c.check(cudaStreamSynchronize(c.stream), "D2H");
    if (ok && iterations) *iterations = done;
    cudaStreamSynchronize(c.stream);
    publish(c);
}

// ------------------------------------------------------------------ part 3 --

rsfk_ctx* rsfk_ctx_create(int device, void* stream) { return make_ctx(device, stream, false); }

void rsfk_ctx_destroy(rsfk_ctx* ctx)
{
    if (!ctx) return;
    cudaSetDevice(ctx->c.device);
    destroy_lanes(ctx);
    cudaStreamSynchronize(ctx->c.stream);
    ctx->c.release();
    delete ctx;
}

int rsfk_ctx_status(const rsfk_ctx* ctx) { return ctx ? ctx->c.status : RSFK_ERR_ARG; }

int rsfk_ctx_stats(rsfk_ctx* ctx, double* out, int n)
{
    if (!ctx || !out) return RSFK_ERR_ARG;
    Context& c = ctx->c;
    cudaSetDevice(c.device);
    unsigned long long evaluated = 0;
    if (c.slots[Context::EXPLORE_COUNT].ptr) {
        if (!c.check(cudaMemcpyAsync(&evaluated, c.slots[Context::EXPLORE_COUNT].ptr, sizeof(evaluated),
                                     cudaMemcpyDeviceToHost, c.stream), "stats D2H") ||
            !c.check(cudaStreamSynchronize(c.stream), "stats"))
            return c.status;
    }
    unsigned long long tc_pairs[2] = {0, 0};
    if (c.slots[Context::TC_STATS].ptr) {
        if (!c.check(cudaMemcpyAsync(tc_pairs, c.slots[Context::TC_STATS].ptr, sizeof(tc_pairs),
                                     cudaMemcpyDeviceToHost, c.stream), "stats D2H") ||
            !c.check(cudaStreamSynchronize(c.stream), "stats"))
            return c.status;
    }
    for (rsfk_ctx* l : ctx->lanes) { // lanes keep device counters of their own
        unsigned long long lp[2] = {0, 0};
        if (l->c.slots[Context::TC_STATS].ptr &&
            cudaMemcpy(lp, l->c.slots[Context::TC_STATS].ptr, sizeof(lp), cudaMemcpyDeviceToHost) == cudaSuccess) {
            tc_pairs[0] += lp[0];
            tc_pairs[1] += lp[1];
        }
    }
    c.resolve_ann_events();
    const double v[17] = {(double)c.stats.trees, (double)c.stats.tree_active_points, (double)c.stats.tree_nodes,
                         c.stats.bucket_knn_us, (double)evaluated, c.stats.subtree_us,
                         (double)c.stats.sub_active_points, (double)c.stats.sub_nodes, c.stats.tree_build_us,
                         c.stats.project_us, (double)c.stats.project_launches, c.stats.route_us,
                         c.stats.query_update_us, (double)c.stats.tc_launches, c.stats.tc_gram_flops,
                         (double)tc_pairs[0], (double)tc_pairs[1]};
    for (int i = 0; i < n && i < 17; ++i) out[i] = v[i];
    return RSFK_OK;
}

int rsfk_ctx_synchronize(rsfk_ctx* ctx)
{
    if (!ctx) return RSFK_ERR_ARG;
    ctx->c.check(cudaStreamSynchronize(ctx->c.stream), "synchronize");
    ctx->c.check_error_flag();
    return ctx->c.status;
}

#define RSFK_ENTER(ctx)                   \
    if (!(ctx)) return RSFK_ERR_ARG;      \
    cudaSetDevice((ctx)->c.device);       \
    (ctx)->c.status = RSFK_OK;            \
    (ctx)->c.message.clear();

int rsfk_dev_sort_rows(rsfk_ctx* ctx, int* d_idx, float* d_dist, long long rows, int K)
{
    RSFK_ENTER(ctx);
    rsfk::sort_rows(ctx->c, d_idx, d_dist, rows, K);
    return ctx->c.status;
}

int rsfk_dev_tree_build(rsfk_ctx* ctx, const float* d_points, int N, int D, int min_children,
                        int max_children, int max_depth, int seed, const int* d_table, int n_table,
                        int* n_leaves, int* max_leaf, int* min_leaf, int* levels)
{
    RSFK_ENTER(ctx);
    ctx->has_tree = rsfk::tree_build(ctx->c, d_points, N, D, min_children, max_children, max_depth, seed,
                                     d_table, n_table, ctx->tree);
    if (ctx->has_tree) {
        if (n_leaves) *n_leaves = ctx->tree.n_leaves;
        if (max_leaf) *max_leaf = ctx->tree.max_leaf;
        if (min_leaf) *min_leaf = ctx->tree.min_leaf;
        if (levels) *levels = ctx->tree.levels;
    }
    return ctx->c.status;
}

int rsfk_dev_tree_export(rsfk_ctx* ctx, int N, int* perm, int* leaf_start, int* leaf_count)
{
    RSFK_ENTER(ctx);
    Context& c = ctx->c;
    if (!ctx->has_tree) {
        c.fail(RSFK_ERR_ARG, "rsfk_dev_tree_export: no tree in this context");
        return c.status;
    }
    const TreeResult& t = ctx->tree;
    std::vector<int> ls(t.n_leaves), lc(t.n_leaves);
    bool ok = c.check(cudaMemcpyAsync(perm, t.perm, sizeof(int) * (size_t)N, cudaMemcpyDeviceToHost, c.stream), "D2H perm") &&
              c.check(cudaMemcpyAsync(ls.data(), t.leaf_start, sizeof(int) * (size_t)t.n_leaves, cudaMemcpyDeviceToHost, c.stream), "D2H leaves") &&
              c.check(cudaMemcpyAsync(lc.data(), t.leaf_count, sizeof(int) * (size_t)t.n_leaves, cudaMemcpyDeviceToHost, c.stream), "D2H leaves") &&
              c.check(cudaStreamSynchronize(c.stream), "D2H tree");
    if (ok) {
        std::vector<int> order(t.n_leaves);
        for (int i = 0; i < t.n_leaves; ++i) order[i] = i;
        std::sort(order.begin(), order.end(), [&](int a, int b) { return ls[a] < ls[b]; });
        for (int b = 0; b < t.n_leaves; ++b) {
            leaf_start[b] = ls[order[b]];
            leaf_count[b] = lc[order[b]];
        }
    }
    return c.status;
}

int rsfk_dev_bucket_knn(rsfk_ctx* ctx, const float* d_points, int N, int D, int K, int* d_idx,
                        float* d_dist)
{
    RSFK_ENTER(ctx);
    if (!ctx->has_tree) {
        ctx->c.fail(RSFK_ERR_ARG, "rsfk_dev_bucket_knn: no tree in this context");
        return ctx->c.status;
    }
    rsfk::bucket_knn(ctx->c, d_points, N, D, K, ctx->tree, d_idx, d_dist);
    return ctx->c.status;
}

int rsfk_dev_bucket_knn_table(rsfk_ctx* ctx, const float* d_points, int N, int D, int K,
                              const int* d_perm, const int* d_leaf_start, const int* d_leaf_count,
                              int n_leaves, int max_leaf, int* d_idx, float* d_dist)
{
    RSFK_ENTER(ctx);
    TreeResult t;
    t.perm = d_perm;
    t.leaf_start = d_leaf_start;
    t.leaf_count = d_leaf_count;
    t.n_leaves = n_leaves;
    t.max_leaf = max_leaf;
    t.sum_leaf_sq = -1.0; // not known for a caller's table
    rsfk::bucket_knn(ctx->c, d_points, N, D, K, t, d_idx, d_dist);
    return ctx->c.status;
}

int rsfk_ctx_set_lanes(rsfk_ctx* ctx, int lanes)
{
    if (!ctx || lanes < 0 || lanes > 4) return RSFK_ERR_ARG;
    ctx->lanes_wanted = lanes;
    return RSFK_OK;
}

int rsfk_ctx_set_tc(rsfk_ctx* ctx, int mode)
{
    if (!ctx || mode < -1 || mode > 1) return RSFK_ERR_ARG;
    ctx->c.tc_mode = mode;
    return RSFK_OK;
}

int rsfk_ctx_set_wait_limits(rsfk_ctx* ctx, int route_max_steps, int level_wait_ms)
{
    if (!ctx) return RSFK_ERR_ARG;
    ctx->c.route_step_limit = route_max_steps;
    ctx->c.level_wait_ms = level_wait_ms;
    return RSFK_OK;
}

int rsfk_ctx_keep_index(rsfk_ctx* ctx, int on)
{
    if (!ctx) return RSFK_ERR_ARG;
    ctx->c.keep_index = on != 0;
    return RSFK_OK;
}

int rsfk_dev_route_queries(rsfk_ctx* ctx, const float* d_points, int N, int D, const float* d_queries,
                           int NQ, int* q_start, int* q_count)
{
    RSFK_ENTER(ctx);
    Context& c = ctx->c;
    (void)N;
    if (!ctx->has_tree || ctx->tree.records == nullptr) {
        c.fail(RSFK_ERR_ARG, "rsfk_dev_route_queries: build a tree with rsfk_ctx_keep_index(ctx, 1) first");
        return c.status;
    }
    if (NQ <= 0) return c.status;
    const TreeResult& t = ctx->tree;
    int* q_leaf = (int*)c.scratch(Context::QUERY_LEAF, sizeof(int) * (size_t)NQ);
    if (!q_leaf || !rsfk::tree_route(c, d_points, D, t, d_queries, NQ, q_leaf, nullptr)) return c.status;
    std::vector<int> leaf(NQ), ls(t.n_leaves), lc(t.n_leaves);
    bool ok = c.check(cudaMemcpyAsync(leaf.data(), q_leaf, sizeof(int) * (size_t)NQ, cudaMemcpyDeviceToHost, c.stream), "D2H query leaves") &&
              c.check(cudaMemcpyAsync(ls.data(), t.leaf_start, sizeof(int) * (size_t)t.n_leaves, cudaMemcpyDeviceToHost, c.stream), "D2H leaves") &&
              c.check(cudaMemcpyAsync(lc.data(), t.leaf_count, sizeof(int) * (size_t)t.n_leaves, cudaMemcpyDeviceToHost, c.stream), "D2H leaves") &&
              c.check(cudaStreamSynchronize(c.stream), "D2H route");
    ok = ok && c.check_error_flag();
    if (ok)
        for (int q = 0; q < NQ; ++q) {
            const int l = leaf[q];
            q_start[q] = (l >= 0 && l < t.n_leaves) ? ls[l] : -1;
            q_count[q] = (l >= 0 && l < t.n_leaves) ? lc[l] : 0;
        }
    return c.status;
}

int rsfk_dev_ann_bucket_knn(rsfk_ctx* ctx, const float* d_points, int N, const float* d_queries, int NQ,
                            int D, int K, int* d_idx, float* d_dist)
{
    RSFK_ENTER(ctx);
    if (!ctx->has_tree || ctx->tree.records == nullptr) {
        ctx->c.fail(RSFK_ERR_ARG, "rsfk_dev_ann_bucket_knn: build a tree with rsfk_ctx_keep_index(ctx, 1) first");
        return ctx->c.status;
    }
    rsfk::ann_bucket_knn(ctx->c, d_points, N, d_queries, NQ, D, K, ctx->tree, d_idx, d_dist);
    return ctx->c.status;
}

int rsfk_dev_forest_ann(rsfk_ctx* ctx, const float* d_points, int N, const float* d_queries, int NQ, int D,
                        int K, int n_trees, int first_tree, int tree_stride, int min_children,
                        int max_children, int max_depth, int seed, int* d_idx, float* d_dist)
{
    RSFK_ENTER(ctx);
    if (N <= 0 || NQ < 0 || D <= 0 || K <= 0 || n_trees < 0 || tree_stride < 1) {
        ctx->c.fail(RSFK_ERR_ARG, "rsfk_dev_forest_ann: invalid argument");
        return ctx->c.status;
    }
    run_forest_ann(ctx, d_points, N, d_queries, NQ, D, K, n_trees, first_tree, tree_stride, min_children,
                   max_children, max_depth, seed, d_idx, d_dist, 0);
    return ctx->c.status;
}

int rsfk_dev_forest(rsfk_ctx* ctx, const float* d_points, int N, int D, int K, int n_trees,
                    int first_tree, int tree_stride, int min_children, int max_children,
                    int max_depth, int seed, int* d_idx, float* d_dist, float* log_forest)
{
    RSFK_ENTER(ctx);
    if (N <= 0 || D <= 0 || K <= 0 || n_trees < 0 || tree_stride < 1) {
        ctx->c.fail(RSFK_ERR_ARG, "rsfk_dev_forest: invalid argument");
        return ctx->c.status;
    }
    run_forest(ctx, d_points, N, D, K, n_trees, first_tree, tree_stride, min_children, max_children,
               max_depth, seed, d_idx, d_dist, log_forest, 0);
    return ctx->c.status;
}

int rsfk_dev_explore(rsfk_ctx* ctx, const float* d_points, int N, int D, int K, const int* d_old_idx,
                     int* d_idx, float* d_dist, int row_begin, int row_end, int list_row0)
{
    RSFK_ENTER(ctx);
    if (row_begin < 0 || row_end > N || row_begin > row_end || list_row0 < 0 || list_row0 > row_begin) {
        ctx->c.fail(RSFK_ERR_ARG, "rsfk_dev_explore: invalid row range");
        return ctx->c.status;
    }
    rsfk::explore_sweep(ctx->c, d_points, N, D, K, d_old_idx, d_idx, d_dist, row_begin, row_end, list_row0);
    return ctx->c.status;
}

int rsfk_dev_symmetrize_count(rsfk_ctx* ctx, int N, int K, const int* d_idx, long long* d_offsets, long long* nnz)
{
    RSFK_ENTER(ctx);
    rsfk::symmetrize_count(ctx->c, d_idx, N, K, d_offsets, nnz);
    return ctx->c.status;
}

int rsfk_dev_symmetrize_fill(rsfk_ctx* ctx, int N, int K, const int* d_idx, const float* d_dist,
                             const long long* d_offsets, int* d_sym_idx, float* d_sym_dist)
{
    RSFK_ENTER(ctx);
    rsfk::symmetrize_fill(ctx->c, d_idx, d_dist, N, K, d_offsets, d_sym_idx, d_sym_dist);
    return ctx->c.status;
}

int rsfk_dev_kmeans(rsfk_ctx* ctx, const float* d_points, int N, int D, int C, int max_iter,
                    int init_from_labels, float* d_centroids, int* d_labels, float* d_sq_dist, int* iterations)
{
    RSFK_ENTER(ctx);
    if (!d_points || !d_centroids || !d_labels || !d_sq_dist) {
        ctx->c.fail(RSFK_ERR_ARG, "rsfk_dev_kmeans: invalid argument");
        return ctx->c.status;
    }
    rsfk::kmeans(ctx->c, d_points, N, D, C, max_iter, init_from_labels != 0, d_centroids, d_labels, d_sq_dist,
                 iterations);
    return ctx->c.status;
}

int rsfk_dev_merge_lists(rsfk_ctx* ctx, long long rows, int K, int G, const int* const* d_idx_lists,
                         const float* const* d_dist_lists, int* d_out_idx, float* d_out_dist)
{
    RSFK_ENTER(ctx);
    rsfk::merge_lists(ctx->c, rows, K, G, d_idx_lists, d_dist_lists, d_out_idx, d_out_dist);
    return ctx->c.status;
}

} // extern "C"
