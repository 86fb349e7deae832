/*
 * C ABI of librsfk.so, the sm_100a implementation of the RSFK K-NN-graph path.
 *
 * Part 1 re-exports, with identical signatures, the entry points the reference
 * library exposes to its ctypes wrapper, so the wrapper can load this library
 * in place of the reference's.  Part 2 adds status reporting (the reference
 * calls exit(1) on a CUDA error; this library never exits).  Part 3 is the
 * device-resident interface the multi-GPU driver and the parity tests use:
 * every pointer named d_* is a device pointer on the context's device.
 *
 * All functions of parts 2 and 3 that return int return 0 on success or an
 * rsfk_status code.
 */
#ifndef RSFK_B200_H
#define RSFK_B200_H

#if defined(__GNUC__)
#define RSFK_EXPORT __attribute__((visibility("default")))
#else
#define RSFK_EXPORT
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- part 1 -- */

/* Replaces pymodule_rsfk_knn (reference: src/python/pymodule_ext.cu:45-59,124-147;
 * bound at python/gpu_rsfk/RSFK.py:115-133).  Host pointers.  Builds n_trees random
 * sample trees (tree t uses seed RANDOM_STATE+t), merges every leaf bucket's
 * all-pairs candidates into the caller's K-lists, then runs nn_exploring_factor
 * neighbour-of-neighbour sweeps.  knn_indices/knn_sqr_distances are IN/OUT
 * ([N*K]; -1 / +inf or FLT_MAX mark an empty slot) and come back ordered by
 * (distance, index).  log_forest receives 16*n_trees+2 floats laid out as the
 * reference's ForestLog (src/rsfk.cu:2148-2173). */
RSFK_EXPORT void pymodule_rsfk_knn(int n_trees, int num_neighbors, int N, int D,
                       int MIN_TREE_CHILD, int MAX_TREE_CHILD, int MAX_DEPTH, int VERBOSE,
                       int RANDOM_STATE, int nn_exploring_factor,
                       float* points, int* knn_indices, float* knn_sqr_distances,
                       float* log_forest);

/* Replaces pymodule_cluster_by_sample_tree (reference: src/python/pymodule_ext.cu:79-91,
 * 183-212; bound at python/gpu_rsfk/RSFK.py:153-168).  One tree; returns malloc()ed
 * nodes_buckets[total_leaves*max_child] (-1 padded) and bucket_sizes[total_leaves];
 * release them with rsfk_free (or free). */
RSFK_EXPORT void pymodule_cluster_by_sample_tree(int N, int D, int MIN_TREE_CHILD, int MAX_TREE_CHILD,
                                     int MAX_DEPTH, int VERBOSE, int RANDOM_STATE,
                                     float* points, int** nodes_buckets, int** bucket_sizes,
                                     int* total_leaves, int* max_child);

/* Replaces pymodule_rsfk_knn_ann (reference: src/python/pymodule_ext.cu:61-77, 149-181;
 * bound at python/gpu_rsfk/RSFK.py:134-152, called at :498-514; driver
 * RSFK::knn_gpu_rsfk_forest_ann, src/rsfk.cu:98-498).  n_trees trees over the N base
 * points (tree t seeded RANDOM_STATE+t); every query row descends each tree to a leaf
 * and its list -- knn_indices/knn_sqr_distances[NQ*K], IN/OUT, indices of BASE points,
 * -1 / +inf (or FLT_MAX) = empty -- takes in the base points of that leaf.  As in the
 * reference, nn_exploring_factor is not used and log_forest is not written on this
 * path.  Rows come back ordered by (distance, index). */
RSFK_EXPORT void pymodule_rsfk_knn_ann(int n_trees, int num_neighbors, int N, int NQ, int D,
                           int MIN_TREE_CHILD, int MAX_TREE_CHILD, int MAX_DEPTH, int VERBOSE,
                           int RANDOM_STATE, int nn_exploring_factor,
                           float* points, float* query_points, int* knn_indices,
                           float* knn_sqr_distances, float* log_forest);

/* k-means (Lloyd iterations) on host buffers, for clustering on top of a sample tree:
 * the groups of pymodule_cluster_by_sample_tree as starting labels (init_from_labels = 1:
 * centroids start as the means of the groups given in labels[N], values in [0, C)) or
 * caller-chosen starting centroids (init_from_labels = 0: centroids[C*D] is read).
 * Runs until two assignments in a row agree or max_iter iterations; writes the final
 * centroids[C*D], labels[N], squared distance of every point to its centroid sq_dist[N]
 * and the iterations run.  Nearest centroid by squared distance in the library's usual
 * summation order, ties to the lower cluster index; a cluster that loses all its points
 * keeps its centroid; the result is a pure function of the input.
 * The reference has no such function: the k-means of its sample-tree clustering sits
 * inside nvGRAPH's spectral clustering and is reached from commented-out code only
 * (src/rsfk.cu:1521-1567, parameters at :1536-1539,1863-1868). */
RSFK_EXPORT void rsfk_kmeans(int N, int D, int C, int max_iter, int init_from_labels,
                 float* points, float* centroids, int* labels, float* sq_dist, int* iterations);

/* ---------------------------------------------------------------- part 2 -- */

/* Status of the most recent part-1 call on this thread's process (0 = ok).
 * Stands in for the reference's CudaTest()/exit(1) (src/rsfk.cu:40-50). */
RSFK_EXPORT int rsfk_last_status(void);
RSFK_EXPORT const char* rsfk_last_message(void);
/* Frees memory returned by pymodule_cluster_by_sample_tree. */
RSFK_EXPORT void rsfk_free(void* p);
/* Number of this library's kernels launched so far in this process. */
RSFK_EXPORT long long rsfk_kernel_launches(void);
/* The host-pointer entry points keep their device buffers (points, lists, tree
 * scratch) between calls, so repeated calls do not pay cudaMalloc/cudaFree (the
 * reference allocates and frees per call, src/rsfk.cu:2039-2067,2175-2181).
 * This returns that memory to the driver. */
RSFK_EXPORT void rsfk_release_memory(void);
/* Largest K the K-list kernels support. */
RSFK_EXPORT int rsfk_max_neighbors(void);
/* GPUs that pymodule_rsfk_knn spreads one call over (one process, one host thread
 * per GPU).  The trees are dealt out round-robin, every GPU holds all the points
 * (its slice comes from the host, the rest from the other GPUs), GPU g merges and
 * sweeps rows [N g / G, N (g+1) / G) of the graph, fetched from the other GPUs'
 * lists; the result is the single-GPU result bit for bit.  n = 0 or 1 returns to
 * one GPU (RSFK_DEVICE).  Without this call the environment decides:
 * RSFK_DEVICES="0,1,..." or RSFK_NUM_GPUS=G (devices 0..G-1).  At most 8 devices.
 * No reference counterpart: the reference runs on one GPU (it calls no
 * cudaSetDevice anywhere; src/rsfk.cu:2033-2228).  Returns RSFK_OK or
 * RSFK_ERR_ARG. */
RSFK_EXPORT int rsfk_set_devices(int n, const int* devices);

/* ---------------------------------------------------------------- part 3 -- */

typedef struct rsfk_ctx rsfk_ctx;

/* A context owns scratch memory on `device` and issues all work on `stream`
 * (a cudaStream_t passed as void*; NULL is the legacy default stream).
 * rsfk_dev_forest and rsfk_dev_forest_ann may in addition run tree sequences on
 * streams and host threads of their own (rsfk_ctx_set_lanes); they start after
 * everything queued on `stream` and the call returns when they are done.
 * No reference counterpart: the reference hard-codes device 0 and the default
 * stream (src/rsfk.cu:679-684). */
RSFK_EXPORT rsfk_ctx* rsfk_ctx_create(int device, void* stream);
RSFK_EXPORT void rsfk_ctx_destroy(rsfk_ctx* ctx);
RSFK_EXPORT int rsfk_ctx_status(const rsfk_ctx* ctx);
RSFK_EXPORT int rsfk_ctx_synchronize(rsfk_ctx* ctx);
/* Work counters since the context was created, for turning kernel times into
 * achieved bytes/s: out[0] trees built, out[1] points projected summed over
 * tree levels, out[2] nodes split, out[3] device microseconds spent in the
 * bucket-KNN kernels, out[4] candidates whose distance the exploration sweeps
 * evaluated, out[5] device microseconds spent in the subtree kernels, out[6] and
 * out[7] the part of out[1] and out[2] done inside subtree kernels, out[8] microseconds
 * the tree builds took as seen from the host, out[9] device microseconds spent in the
 * projection kernels of the tree levels and out[10] their launch count; query path:
 * out[11] device microseconds of hyperplanes + descent + grouping by leaf, out[12] of
 * the query-bucket kernels; out[13] bucket-KNN launches that ran on the tensor cores and
 * out[14] the Gram-matrix flops of those launches, 2*D*sum(leaf size^2), out[15] the pairs
 * the tensor-core filter let through to the exact evaluation and out[16] the pairs it
 * looked at.  The reference's
 * counterpart is its ForestLog of per-phase wall-clock times (src/include/rsfk.h:274-392). */
RSFK_EXPORT int rsfk_ctx_stats(rsfk_ctx* ctx, double* out, int n);

/* Orders every row by (distance, index), dropping repeated indices; the other
 * device entry points expect and keep rows in this form.  The reference leaves
 * rows unordered (src/include/rsfk.h:404-411). */
RSFK_EXPORT int rsfk_dev_sort_rows(rsfk_ctx* ctx, int* d_idx, float* d_dist, long long rows, int K);

/* One random sample tree (reference: RSFK::create_bucket_from_sample_tree,
 * src/rsfk.cu:500-1207).  d_table, when not NULL, supplies the split pairs
 * explicitly: n_table rows of {p1, p2, row of left child, row of right child},
 * row 0 the root; otherwise pairs come from a counter hash of
 * (seed, depth, segment start).  The tree stays inside the context. */
RSFK_EXPORT int rsfk_dev_tree_build(rsfk_ctx* ctx, const float* d_points, int N, int D,
                        int min_children, int max_children, int max_depth, int seed,
                        const int* d_table, int n_table,
                        int* n_leaves, int* max_leaf, int* min_leaf, int* levels);
/* Copies the context's tree to host arrays: perm[N], leaves ordered by start. */
RSFK_EXPORT int rsfk_dev_tree_export(rsfk_ctx* ctx, int N, int* perm, int* leaf_start, int* leaf_count);

/* Leaf-bucket KNN over the context's tree (reference: RSFK::update_knn_indice_with_buckets,
 * src/rsfk.cu:1967-2030, kernel src/kernels/compute_knn_from_buckets.cu:998-1378). */
RSFK_EXPORT int rsfk_dev_bucket_knn(rsfk_ctx* ctx, const float* d_points, int N, int D, int K,
                        int* d_idx, float* d_dist);
/* Same over an explicit bucket table: leaf b holds points
 * d_perm[d_leaf_start[b] .. +d_leaf_count[b]). */
RSFK_EXPORT int rsfk_dev_bucket_knn_table(rsfk_ctx* ctx, const float* d_points, int N, int D, int K,
                              const int* d_perm, const int* d_leaf_start,
                              const int* d_leaf_count, int n_leaves, int max_leaf,
                              int* d_idx, float* d_dist);

/* How many tree sequences ("lanes") a forest call of this context runs side by side on
 * the GPU, each on a stream of its own with lists of its own that are combined at the
 * end: 1..4, or 0 for the default (environment variable RSFK_LANES, else three where
 * N*D <= 2^28 and the call has at least twelve trees, two from eight trees, else one; a
 * number set here is used as long as every lane gets two trees).  The result does not depend
 * on it.  No reference counterpart (the
 * reference builds its trees one after another, src/rsfk.cu:2073-2088). */
RSFK_EXPORT int rsfk_ctx_set_lanes(rsfk_ctx* ctx, int lanes);

/* Which kernel the bucket KNN of this context takes where D >= 64: 1 = the tcgen05 Gram
 * filter (128-row tiles, TMA-fed) wherever the shape allows it, 0 = the exact SIMT kernel
 * only, -1 = the library's choice: the tcgen05 kernel where a leaf no longer fits one CTA's
 * shared memory, else the exact kernel.  Either way the lists are the same bit for bit.  No reference counterpart (the reference has one
 * SIMT kernel, src/kernels/compute_knn_from_buckets.cu:998-1378). */
RSFK_EXPORT int rsfk_ctx_set_tc(rsfk_ctx* ctx, int mode);

/* Limits of the library's bounded waits; a negative value restores the built-in limit.
 * route_max_steps: tree levels a query may descend (rsfk_dev_route_queries and the query
 * updates) before the kernel gives up, marks the query as lost and the call returns
 * RSFK_ERR_CUDA; built-in: the tree's depth + 8.  level_wait_ms: how long the host waits for
 * the node counts of a batch of tree levels before rsfk_dev_tree_build returns RSFK_ERR_CUDA
 * (0 = do not wait at all); built-in: 30 s.  After either failure the stream is idle and the
 * context stays usable.  The reference has no counterpart: it blocks in
 * cudaDeviceSynchronize and calls exit(1) on errors (src/rsfk.cu:40-50). */
RSFK_EXPORT int rsfk_ctx_set_wait_limits(rsfk_ctx* ctx, int route_max_steps, int level_wait_ms);

/* Trees first_tree, first_tree+tree_stride, ... (n_trees of them), tree t with
 * seed `seed`+t, each followed by its bucket KNN (reference: the tree loop of
 * RSFK::knn_gpu_rsfk_forest, src/rsfk.cu:2073-2088).  log_forest (host,
 * 16*n_trees+2 floats) may be NULL. */
RSFK_EXPORT int rsfk_dev_forest(rsfk_ctx* ctx, const float* d_points, int N, int D, int K,
                    int n_trees, int first_tree, int tree_stride,
                    int min_children, int max_children, int max_depth, int seed,
                    int* d_idx, float* d_dist, float* log_forest);

/* One neighbour-of-neighbour sweep over rows [row_begin,row_end), candidates
 * read from the snapshot d_old_idx ([N*K], all rows) (reference:
 * src/kernels/nearest_neighbors_exploring.cu:41-146, driven at src/rsfk.cu:2117-2126).
 * d_idx/d_dist hold the lists being updated starting at row list_row0
 * (0 for full [N*K] arrays; row_begin when a rank keeps only its own rows). */
RSFK_EXPORT int rsfk_dev_explore(rsfk_ctx* ctx, const float* d_points, int N, int D, int K,
                     const int* d_old_idx, int* d_idx, float* d_dist,
                     int row_begin, int row_end, int list_row0);

/* Query (base/query) path on device memory.
 *
 * rsfk_ctx_keep_index(ctx, 1) makes every later tree build of the context keep its
 * tree index (one row per split: the pair of sample points and where each side
 * leads), which the two calls below descend; 0 (the default) turns that off.
 * Reference: the per-level arrays the reference keeps in RSFKIndexTree when
 * create_bucket_from_sample_tree runs with free_index=false
 * (src/include/rsfk.h:92-160, src/rsfk.cu:176-178). */
RSFK_EXPORT int rsfk_ctx_keep_index(rsfk_ctx* ctx, int on);
/* Leaf bucket of every query row under the context's tree: q_start/q_count (HOST,
 * [NQ]) receive the segment of perm (rsfk_dev_tree_export) that is the bucket
 * (reference: the query descent, src/rsfk.cu:270-347, ending in
 * compute_bucket_for_query_points, build_tree_update_parents_ann.cu:76-91). */
RSFK_EXPORT int rsfk_dev_route_queries(rsfk_ctx* ctx, const float* d_points, int N, int D,
                           const float* d_queries, int NQ, int* q_start, int* q_count);
/* Routes the queries and merges each query's list (d_idx/d_dist, [NQ*K], canonical,
 * indices of base points) with the base points of its bucket (reference:
 * compute_knn_from_buckets_perwarp_coalesced_ann,
 * src/kernels/build_tree_update_parents_ann.cu:232-513). */
RSFK_EXPORT int rsfk_dev_ann_bucket_knn(rsfk_ctx* ctx, const float* d_points, int N,
                            const float* d_queries, int NQ, int D, int K,
                            int* d_idx, float* d_dist);
/* Trees first_tree, first_tree+tree_stride, ... (n_trees of them, tree t seeded
 * seed+t) over the base points, each followed by the query update (reference: the
 * tree loop of RSFK::knn_gpu_rsfk_forest_ann, src/rsfk.cu:116-126). */
RSFK_EXPORT int rsfk_dev_forest_ann(rsfk_ctx* ctx, const float* d_points, int N,
                        const float* d_queries, int NQ, int D, int K,
                        int n_trees, int first_tree, int tree_stride,
                        int min_children, int max_children, int max_depth, int seed,
                        int* d_idx, float* d_dist);

/* Symmetric closure of a K-NN graph in CSR form: row p holds p's valid entries and every
 * q that lists p without being listed by p, ordered by neighbour index (reference: the
 * kernels symmetric_knn_graph_edge_count / _offset / _add_edges, src/rsfk.cu:1229-1299,
 * which leave a row in atomic arrival order).  Two steps, so that the caller owns the
 * output: _count writes the row offsets d_offsets[N+1] (64-bit) and returns the number
 * of entries in *nnz (host); _fill writes d_sym_idx[nnz] and, when d_sym_dist is not
 * NULL, the squared distance of every entry taken from d_dist.  Rows of d_idx must hold
 * distinct indices (as every list this library returns does); -1 entries are skipped. */
RSFK_EXPORT int rsfk_dev_symmetrize_count(rsfk_ctx* ctx, int N, int K, const int* d_idx,
                              long long* d_offsets, long long* nnz);
RSFK_EXPORT int rsfk_dev_symmetrize_fill(rsfk_ctx* ctx, int N, int K, const int* d_idx, const float* d_dist,
                             const long long* d_offsets, int* d_sym_idx, float* d_sym_dist);

/* rsfk_kmeans on device memory (same rules; d_labels is read only when
 * init_from_labels is set; iterations is a host pointer and may be NULL). */
RSFK_EXPORT int rsfk_dev_kmeans(rsfk_ctx* ctx, const float* d_points, int N, int D, int C, int max_iter,
                    int init_from_labels, float* d_centroids, int* d_labels, float* d_sq_dist,
                    int* iterations);

/* out = the K smallest distinct entries of G canonical lists per row.
 * d_idx_lists/d_dist_lists are HOST arrays of G device pointers (G <= 16).
 * No reference counterpart (the reference is single-GPU); used to combine the
 * lists of trees built on different GPUs. */
RSFK_EXPORT int rsfk_dev_merge_lists(rsfk_ctx* ctx, long long rows, int K, int G,
                         const int* const* d_idx_lists, const float* const* d_dist_lists,
                         int* d_out_idx, float* d_out_dist);

/* ---------------------------------------------------------------- part 4 -- */

/* Capacity, in K-list entries (N*K), of the snapshot buffer built into the
 * library for rsfk_explore_sweep_static: 4 Mi entries = 16 MiB of device memory
 * that every GPU using the library holds from load until the process exits. */
#define RSFK_STATIC_SWEEP_MAX_ENTRIES (4 * 1024 * 1024)

/* One neighbour-of-neighbour sweep over all N rows, in place, WITHOUT touching
 * any allocator.  This entry point has no counterpart in the reference.
 *
 * It exists for hosts that cannot call cudaMalloc where the sweep runs: an
 * application that hands its whole device-memory budget to its own arena at
 * start-up, a service whose latency rules forbid the device-wide
 * synchronisation cudaMalloc/cudaFree imply, or a plug-in API that bans
 * allocation after initialisation.  Everything else the sweep needs -- the
 * frozen copy of the index lists and a work counter -- lives in a fixed array
 * inside the library image, so the call makes no cudaMalloc, cudaFree or other
 * allocating call and needs no rsfk_ctx.
 *
 *   d_points [N*D], d_idx / d_dist [N*K]: device pointers on the CURRENT
 *   device; rows must be canonical (see rsfk_dev_sort_rows); they are updated
 *   in place exactly as rsfk_dev_explore would update them from a snapshot
 *   taken at the start of the call.  stream: cudaStream_t as void*
 *   (NULL = legacy default stream); the work is enqueued, not awaited.
 *
 * Limits and rules:
 *  - N*K <= RSFK_STATIC_SWEEP_MAX_ENTRIES, K <= rsfk_max_neighbors(); larger
 *    problems are refused with RSFK_ERR_ARG and a message on stderr (use
 *    rsfk_dev_explore with your own snapshot buffer).
 *  - The first call on each device looks up the built-in array's device
 *    address; make that first call outside any stream capture.
 *  - All calls on a device share the one array and it keeps the previous
 *    call's contents (each call overwrites what it reads).  Two calls whose GPU
 *    work overlaps -- different streams, or different host threads -- race on
 *    it: serialise them.
 * Returns 0 or an rsfk_status code. */
RSFK_EXPORT int rsfk_explore_sweep_static(const float* d_points, int N, int D, int K,
                                          int* d_idx, float* d_dist, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RSFK_B200_H */
