/*
 * CPU oracle for the RSFK K-NN-graph path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic and the update rules of the
 * reference CUDA kernels so that the sm_100a kernels can be checked against
 * it.  Nothing in the product path links or calls it: only the test-suite, the
 * smoke check and the CPU-baseline leg of the benchmark load it.
 *
 * Every function names the reference file:line it follows (paths are relative
 * to the reference project's root).
 *
 * Compile with -ffp-contract=off: every fused multiply-add the reference's
 * compiler emits (nvcc contracts a*b+c by default) is written here as an
 * explicit fmaf(), and nothing else may be fused.
 *
 * Parity status: pinned.  The distance function, the bucket update rule, the
 * exploration sweep, and the tree rules (split side with the root's serial and
 * the other nodes' lane-strided offset, minimum side size, leaf sizes) are all
 * checked against outputs of the reference binary itself (fixtures under
 * tests/golden/, produced by tests/golden/make_ref_golden.py).  The query
 * (base/query) update is checked slot for slot against the reference binary
 * run over its own base points (tests/golden/make_ref_ann_golden.py), the only
 * shape its query driver handles within bounds; the descent of a query that is
 * not a base point is pinned through its parts (the split rule above, the
 * follow-the-sibling rule read from build_tree_update_parents_ann.cu:150-160),
 * not end to end.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* 32-lane emulation helpers                                                  */
/* ------------------------------------------------------------------------- */

/* The reference reduces 32 per-lane partial sums with
 *   s += shfl_xor(s,1); s += shfl_xor(s,2); ... s += shfl_xor(s,16);
 * (src/kernels/compute_knn_from_buckets.cu:219-223,
 *  src/kernels/build_tree_check_points_side.cu:139-143,
 *  src/kernels/create_node.cu:128-132).  Every lane ends with the same value;
 * the association is the balanced tree reproduced here. */
static float butterfly32(float acc[32])
{
    float tmp[32];
    for (int stride = 1; stride < 32; stride <<= 1) {
        for (int l = 0; l < 32; ++l) tmp[l] = acc[l] + acc[l ^ stride];
        memcpy(acc, tmp, sizeof(tmp));
    }
    return acc[0];
}

/* Squared L2 distance in the reference's summation order:
 * lane l accumulates i = l, l+32, ... with diff*diff fused into the running
 * sum, then the butterfly (src/kernels/compute_knn_from_buckets.cu:205-227;
 * same body inlined at :1176-1186). */
ORC_API float orc_dist_sqr(const float* a, const float* b, int D)
{
    float acc[32];
    for (int l = 0; l < 32; ++l) acc[l] = 0.0f;
    for (int i = 0; i < D; ++i) {
        float diff = a[i] - b[i];
        acc[i & 31] = fmaf(diff, diff, acc[i & 31]);
    }
    return butterfly32(acc);
}

/* Hyperplane of a split pair: normal n = x1 - x2 and offset
 * c = sum n_i * (x1_i + x2_i) / 2.
 * Root: serial sum over i = 0..D-1 (src/kernels/create_node.cu:60-66).
 * Other nodes: lane-strided partial sums and the butterfly
 * (src/kernels/create_node.cu:120-134).
 * The product n_i*(x1_i+x2_i) is rounded, halved exactly, then added, so no
 * contraction changes the bits. */
ORC_API float orc_hyperplane(const float* x1, const float* x2, int D, int is_root, float* n)
{
    for (int i = 0; i < D; ++i) n[i] = x1[i] - x2[i];
    if (is_root) {
        float c = 0.0f;
        for (int i = 0; i < D; ++i) {
            float t = n[i] * (x1[i] + x2[i]);
            c = c + t / 2;
        }
        return c;
    }
    float acc[32];
    for (int l = 0; l < 32; ++l) acc[l] = 0.0f;
    for (int i = 0; i < D; ++i) {
        float t = n[i] * (x1[i] + x2[i]);
        acc[i & 31] = acc[i & 31] + t / 2;
    }
    return butterfly32(acc);
}

/* Projection n.x, lane-strided fused multiply-adds then the butterfly
 * (src/kernels/build_tree_check_points_side.cu:131-143). */
ORC_API float orc_project(const float* n, const float* x, int D)
{
    float acc[32];
    for (int l = 0; l < 32; ++l) acc[l] = 0.0f;
    for (int i = 0; i < D; ++i) acc[i & 31] = fmaf(n[i], x[i], acc[i & 31]);
    return butterfly32(acc);
}

/* ------------------------------------------------------------------------- */
/* Split-pair sampling shared with the CUDA build                             */
/* ------------------------------------------------------------------------- */

/* The reference draws the pair with cuRAND XORWOW from positions in an array
 * whose order depends on atomic arrival order
 * (src/kernels/build_tree_create_nodes.cu:90-100, build_tree_init.cu:66-72),
 * so it is not reproducible.  Both this oracle and the CUDA build instead draw
 * two distinct positions inside the node's segment of the stably partitioned
 * permutation from a counter hash of (seed, depth, segment start). */
static uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

ORC_API void orc_sample_positions(int seed, int depth, int start, int count, int* r1, int* r2)
{
    uint64_t h = mix64(((uint64_t)(uint32_t)seed << 32) ^ (uint64_t)(uint32_t)start);
    h = mix64(h ^ ((uint64_t)(uint32_t)depth * 0xD6E8FEB86659FD93ull));
    uint32_t a = (uint32_t)(h & 0xffffffffu), b = (uint32_t)(h >> 32);
    int p = (int)(a % (uint32_t)count);
    int q = p;
    if (count > 1) q = (int)(((uint32_t)p + 1u + b % (uint32_t)(count - 1)) % (uint32_t)count);
    *r1 = p;
    *r2 = q;
}

/* ------------------------------------------------------------------------- */
/* Random sample tree                                                         */
/* ------------------------------------------------------------------------- */

typedef struct {
    int start, count, p1, p2, tbl;
    int qs, qc; /* segment of the query permutation routed to this node */
} orc_node;

typedef struct {
    int* data;
    int n, cap;
} ivec;

static void ivec_push(ivec* v, int x)
{
    if (v->n == v->cap) {
        v->cap = v->cap ? 2 * v->cap : 1024;
        v->data = (int*)realloc(v->data, sizeof(int) * (size_t)v->cap);
    }
    v->data[v->n++] = x;
}

static void emit_leaf(ivec* ls, ivec* lc, int start, int count, int max_piece)
{
    /* A node that is still too large when the depth limit is hit is cut into
     * consecutive pieces of at most max_piece points.  The reference has no
     * such path: it indexes its leaf table with -1 there
     * (src/kernels/build_tree_bucket_points.cu:51-54). */
    if (max_piece <= 0 || count <= max_piece) {
        ivec_push(ls, start);
        ivec_push(lc, count);
        return;
    }
    int q = (count + max_piece - 1) / max_piece;
    for (int i = 0; i < q; ++i) {
        int a = (int)((int64_t)count * i / q), b = (int)((int64_t)count * (i + 1) / q);
        ivec_push(ls, start + a);
        ivec_push(lc, b - a);
    }
}

static void pick_pair(orc_node* nd, const int* perm, int seed, int depth, const int* table, int n_table)
{
    if (table && nd->tbl >= 0 && nd->tbl < n_table) {
        nd->p1 = table[4 * nd->tbl + 0];
        nd->p2 = table[4 * nd->tbl + 1];
        return;
    }
    int r1, r2;
    orc_sample_positions(seed, depth, nd->start, nd->count, &r1, &r2);
    nd->p1 = perm[nd->start + r1];
    nd->p2 = perm[nd->start + r2];
}

static int table_child(const int* table, int n_table, int tbl, int side)
{
    if (!table || tbl < 0 || tbl >= n_table) return -1;
    return table[4 * tbl + 2 + side];
}

/*
 * One random sample tree over points[N][D].
 *
 * Rules restated (level by level, as src/rsfk.cu:719-931 drives them):
 *  - the root is never a leaf and always splits (build_tree_init.cu:76-79);
 *  - a point goes RIGHT iff n.x < c (build_tree_check_points_side.cu:149);
 *  - every non-empty side becomes a child (build_tree_create_nodes.cu:88-104);
 *    the child is a leaf iff its count <= MAX-2 (build_tree_update_parents.cu:69-71);
 *  - a child with fewer than MIN points is emptied into its sibling, which is a
 *    leaf iff the merged count <= MAX and is split again otherwise
 *    (build_tree_update_parents.cu:106-133);
 *  - a child's split pair is drawn from the child's own points when the child
 *    is created, i.e. before any merge (build_tree_create_nodes.cu:90-100).
 *
 * Points of a node are one contiguous segment of `perm`; each split is a
 * stable partition (left side first).  `table`, when given, supplies the split
 * pairs explicitly: row t = {p1, p2, table row of the left child, of the right
 * child}, row 0 is the root; a row index of -1 falls back to the counter hash.
 * `table_out` (capacity table_out_cap rows) records the tree that was built in
 * the same format.
 *
 * Outputs: perm[N]; leaf_start/leaf_count (caller frees with orc_free), leaves
 * ordered by segment start; returns the number of levels processed.
 *
 * Query routing (the ANN path, src/rsfk.cu:270-347): queries[NQ][D] descend the
 * tree level by level beside the base points.  A query takes the side the
 * split rule gives it (the same kernel as for base points,
 * build_tree_check_points_side.cu:131-151, run over the query array); where
 * that side holds no node of its own -- it was empty or it dissolved into its
 * sibling -- the query follows to the sibling
 * (build_tree_update_parents_ann.cu:150-160).  q_start[q]/q_count[q] receive
 * the segment of `perm` that is the leaf bucket query q ends in.
 */
static int build_tree_impl(const float* points, int N, int D, int MIN, int MAX, int MAX_DEPTH,
                           int seed, const int* table, int n_table, int* perm,
                           int** leaf_start_out, int** leaf_count_out, int* n_leaves_out,
                           int* table_out, int table_out_cap, int* n_table_out,
                           const float* queries, int NQ, int* q_start, int* q_count)
{
    ivec ls = {0, 0, 0}, lc = {0, 0, 0};
    int n_rec = 0;
    for (int i = 0; i < N; ++i) perm[i] = i;
    if (!queries) NQ = 0;
    int* qperm = (int*)malloc(sizeof(int) * (size_t)(NQ > 0 ? NQ : 1));
    int* qtmp = (int*)malloc(sizeof(int) * (size_t)(NQ > 0 ? NQ : 1));
    for (int i = 0; i < NQ; ++i) { qperm[i] = i; q_start[i] = -1; q_count[i] = 0; }
    int* tmp = (int*)malloc(sizeof(int) * (size_t)(N > 0 ? N : 1));
    unsigned char* side = (unsigned char*)malloc((size_t)(N > 0 ? N : 1));
    float* nrm = (float*)malloc(sizeof(float) * (size_t)(D > 0 ? D : 1));
    int cap = 1024, n_act = 0;
    orc_node* act = (orc_node*)malloc(sizeof(orc_node) * (size_t)cap);
    orc_node* nxt = (orc_node*)malloc(sizeof(orc_node) * (size_t)cap);
    int* rec_of = NULL; /* record row of each active node */
    int* rec_nxt = NULL;
    rec_of = (int*)malloc(sizeof(int) * (size_t)cap);
    rec_nxt = (int*)malloc(sizeof(int) * (size_t)cap);
    int depth = 0;

    if (N <= 0) goto done;
    if (N == 1) {
        emit_leaf(&ls, &lc, 0, 1, 0);
        for (int i = 0; i < NQ; ++i) { q_start[i] = 0; q_count[i] = 1; }
        goto done;
    }

    act[0].start = 0; act[0].count = N; act[0].tbl = table ? 0 : -1;
    act[0].qs = 0; act[0].qc = NQ;
    pick_pair(&act[0], perm, seed, 0, table, n_table);
    n_act = 1;
    if (table_out && n_rec < table_out_cap) {
        table_out[0] = act[0].p1; table_out[1] = act[0].p2; table_out[2] = -1; table_out[3] = -1;
    }
    rec_of[0] = 0;
    n_rec = 1;

    for (depth = 1; depth < MAX_DEPTH && n_act > 0; ++depth) {
        int n_nxt = 0;
        for (int a = 0; a < n_act; ++a) {
            orc_node nd = act[a];
            float c = orc_hyperplane(points + (size_t)nd.p1 * D, points + (size_t)nd.p2 * D, D,
                                     depth == 1, nrm);
            int nL = 0;
            for (int i = 0; i < nd.count; ++i) {
                int p = perm[nd.start + i];
                float pr = orc_project(nrm, points + (size_t)p * D, D);
                side[i] = pr < c;
                nL += !side[i];
            }
            int nR = nd.count - nL;
            {   /* stable partition, left side first */
                int l = 0, r = nL;
                for (int i = 0; i < nd.count; ++i) {
                    if (side[i]) tmp[r++] = perm[nd.start + i];
                    else tmp[l++] = perm[nd.start + i];
                }
                memcpy(perm + nd.start, tmp, sizeof(int) * (size_t)nd.count);
            }
            int nQL = 0;
            if (nd.qc > 0) { /* the queries of this node, same rule, same stable order */
                int l = 0, r = 0;
                for (int i = 0; i < nd.qc; ++i) {
                    int q = qperm[nd.qs + i];
                    float pr = orc_project(nrm, queries + (size_t)q * D, D);
                    nQL += !(pr < c);
                }
                r = nQL;
                for (int i = 0; i < nd.qc; ++i) {
                    int q = qperm[nd.qs + i];
                    float pr = orc_project(nrm, queries + (size_t)q * D, D);
                    if (pr < c) qtmp[r++] = q;
                    else qtmp[l++] = q;
                }
                memcpy(qperm + nd.qs, qtmp, sizeof(int) * (size_t)nd.qc);
            }
            orc_node ch[2];
            int n_ch = 0, leaf[2] = {0, 0}, chside[2] = {0, 0};
            if (nL > 0 && nR > 0 && nL >= MIN && nR >= MIN) {
                ch[0].start = nd.start;      ch[0].count = nL; chside[0] = 0;
                ch[1].start = nd.start + nL; ch[1].count = nR; chside[1] = 1;
                leaf[0] = nL <= MAX - 2;
                leaf[1] = nR <= MAX - 2;
                ch[0].qs = nd.qs;       ch[0].qc = nQL;
                ch[1].qs = nd.qs + nQL; ch[1].qc = nd.qc - nQL;
                n_ch = 2;
            } else if (nL > 0 && nR > 0) {
                /* the side with fewer than MIN points dissolves into the other */
                int keep = (nL < MIN) ? 1 : 0;
                if (nL < MIN && nR < MIN) keep = 0;
                /* the survivor's pair comes from its own, pre-merge, segment */
                ch[0].start = keep ? nd.start + nL : nd.start;
                ch[0].count = keep ? nR : nL;
                chside[0] = keep;
                leaf[0] = nd.count <= MAX;
                ch[0].qs = nd.qs; ch[0].qc = nd.qc;
                n_ch = 1;
            } else {
                ch[0].start = nd.start; ch[0].count = nd.count;
                chside[0] = (nL > 0) ? 0 : 1;
                leaf[0] = nd.count <= MAX - 2;
                ch[0].qs = nd.qs; ch[0].qc = nd.qc;
                n_ch = 1;
            }
            for (int k = 0; k < n_ch; ++k) {
                ch[k].tbl = table_child(table, n_table, nd.tbl, chside[k]);
                int merged = (n_ch == 1 && nL > 0 && nR > 0);
                int rec = -1;
                if (!leaf[k]) {
                    pick_pair(&ch[k], perm, seed, depth, table, n_table);
                    if (table_out && n_rec < table_out_cap) {
                        rec = n_rec;
                        table_out[4 * rec + 0] = ch[k].p1; table_out[4 * rec + 1] = ch[k].p2;
                        table_out[4 * rec + 2] = -1;       table_out[4 * rec + 3] = -1;
                        if (rec_of[a] >= 0) table_out[4 * rec_of[a] + 2 + chside[k]] = rec;
                    }
                    if (table_out) n_rec++;
                }
                if (merged) { ch[k].start = nd.start; ch[k].count = nd.count; }
                if (leaf[k]) {
                    emit_leaf(&ls, &lc, ch[k].start, ch[k].count, 0);
                    for (int i = 0; i < ch[k].qc; ++i) {
                        q_start[qperm[ch[k].qs + i]] = ch[k].start;
                        q_count[qperm[ch[k].qs + i]] = ch[k].count;
                    }
                } else {
                    if (n_nxt == cap) {
                        cap *= 2;
                        act = (orc_node*)realloc(act, sizeof(orc_node) * (size_t)cap);
                        nxt = (orc_node*)realloc(nxt, sizeof(orc_node) * (size_t)cap);
                        rec_of = (int*)realloc(rec_of, sizeof(int) * (size_t)cap);
                        rec_nxt = (int*)realloc(rec_nxt, sizeof(int) * (size_t)cap);
                    }
                    rec_nxt[n_nxt] = rec;
                    nxt[n_nxt++] = ch[k];
                }
            }
        }
        { orc_node* t = act; act = nxt; nxt = t; }
        { int* t = rec_of; rec_of = rec_nxt; rec_nxt = t; }
        n_act = n_nxt;
    }
    /* depth limit: whatever is still open becomes leaves, cut to <= MAX */
    for (int a = 0; a < n_act; ++a) {
        int before = ls.n;
        emit_leaf(&ls, &lc, act[a].start, act[a].count, MAX);
        for (int i = 0; i < act[a].qc; ++i) { /* queries of a cut node go to its first piece */
            q_start[qperm[act[a].qs + i]] = ls.data[before];
            q_count[qperm[act[a].qs + i]] = lc.data[before];
        }
    }

done:
    {   /* order leaves by segment start (insertion order is level order) */
        int n = ls.n;
        int* order = (int*)malloc(sizeof(int) * (size_t)(n > 0 ? n : 1));
        int* first = (int*)malloc(sizeof(int) * (size_t)(N + 1));
        for (int i = 0; i <= N; ++i) first[i] = -1;
        for (int i = 0; i < n; ++i) first[ls.data[i]] = i;
        int m = 0;
        for (int i = 0; i < N; ++i) if (first[i] >= 0) order[m++] = first[i];
        int* s = (int*)malloc(sizeof(int) * (size_t)(n > 0 ? n : 1));
        int* c = (int*)malloc(sizeof(int) * (size_t)(n > 0 ? n : 1));
        for (int i = 0; i < m; ++i) { s[i] = ls.data[order[i]]; c[i] = lc.data[order[i]]; }
        free(order); free(first);
        *leaf_start_out = s; *leaf_count_out = c; *n_leaves_out = m;
    }
    if (n_table_out) *n_table_out = n_rec;
    free(ls.data); free(lc.data); free(tmp); free(side); free(nrm); free(act); free(nxt);
    free(rec_of); free(rec_nxt); free(qperm); free(qtmp);
    return depth;
}

ORC_API int orc_build_tree(const float* points, int N, int D, int MIN, int MAX, int MAX_DEPTH,
                           int seed, const int* table, int n_table, int* perm,
                           int** leaf_start_out, int** leaf_count_out, int* n_leaves_out,
                           int* table_out, int table_out_cap, int* n_table_out)
{
    return build_tree_impl(points, N, D, MIN, MAX, MAX_DEPTH, seed, table, n_table, perm,
                           leaf_start_out, leaf_count_out, n_leaves_out, table_out, table_out_cap,
                           n_table_out, NULL, 0, NULL, NULL);
}

/* The same tree, with queries[NQ][D] routed to their leaf buckets:
 * q_start[q], q_count[q] = the bucket's segment of perm. */
ORC_API int orc_build_tree_route(const float* points, int N, int D, int MIN, int MAX, int MAX_DEPTH,
                                 int seed, const int* table, int n_table, int* perm,
                                 int** leaf_start_out, int** leaf_count_out, int* n_leaves_out,
                                 const float* queries, int NQ, int* q_start, int* q_count)
{
    return build_tree_impl(points, N, D, MIN, MAX, MAX_DEPTH, seed, table, n_table, perm,
                           leaf_start_out, leaf_count_out, n_leaves_out, NULL, 0, NULL,
                           queries, NQ, q_start, q_count);
}

ORC_API void orc_free(void* p) { free(p); }

/* ------------------------------------------------------------------------- */
/* Leaf-bucket KNN                                                            */
/* ------------------------------------------------------------------------- */

/* Slot of the largest distance of a K-list as the reference's warp finds it:
 * lane l scans slots l, l+32, ... keeping the first strictly larger value, then
 * a shfl_down tree (16,8,4,2,1) keeps the lower lane on ties
 * (src/kernels/compute_knn_from_buckets.cu:1058-1099). */
static int argmax_warp(const float* d, int K, float* val_out)
{
    float lv[32];
    int lp[32];
    for (int l = 0; l < 32; ++l) {
        lv[l] = -1.0f; lp[l] = -1;
        for (int j = l; j < K; j += 32)
            if (d[j] > lv[l]) { lv[l] = d[j]; lp[l] = j; }
    }
    for (int off = 16; off >= 1; off >>= 1) {
        for (int l = 0; l < 32; ++l) {
            /* lanes l+off beyond 31 return the lane's own value: no change */
            if (l + off < 32 && lv[l + off] > lv[l]) { lv[l] = lv[l + off]; lp[l] = lp[l + off]; }
        }
    }
    *val_out = lv[0];
    return lp[0];
}

static int row_has(const int* idx, int K, int v)
{
    for (int k = 0; k < K; ++k) if (idx[k] == v) return 1;
    return 0;
}

/* Reference-order bucket update: for every diagonal d of the bucket's pair
 * matrix, first every row i takes candidate i+d, then every row i+d takes
 * candidate i; a candidate replaces the row's current worst slot iff it is
 * strictly closer and not already in the row
 * (src/kernels/compute_knn_from_buckets.cu:1121-1376). */
ORC_API void orc_bucket_knn_ref(const float* points, int N, int D, int K, const int* perm,
                                const int* leaf_start, const int* leaf_count, int n_leaves,
                                int* idx, float* dist)
{
    (void)N;
    #pragma omp parallel for schedule(dynamic, 16)
    for (int b = 0; b < n_leaves; ++b) {
        int m = leaf_count[b];
        const int* ids = perm + leaf_start[b];
        float* maxv = (float*)malloc(sizeof(float) * (size_t)m);
        int* maxp = (int*)malloc(sizeof(int) * (size_t)m);
        float* cand = (float*)malloc(sizeof(float) * (size_t)m);
        for (int i = 0; i < m; ++i) maxp[i] = argmax_warp(dist + (size_t)ids[i] * K, K, &maxv[i]);
        for (int d = 1; d < m; ++d) {
            for (int i = 0; i + d < m; ++i)
                cand[i] = orc_dist_sqr(points + (size_t)ids[i] * D, points + (size_t)ids[i + d] * D, D);
            for (int i = 0; i + d < m; ++i) {
                int r = ids[i], c = ids[i + d];
                if (!(cand[i] >= maxv[i]) && !row_has(idx + (size_t)r * K, K, c)) {
                    idx[(size_t)r * K + maxp[i]] = c;
                    dist[(size_t)r * K + maxp[i]] = cand[i];
                    maxp[i] = argmax_warp(dist + (size_t)r * K, K, &maxv[i]);
                }
            }
            for (int i = 0; i + d < m; ++i) {
                int r = ids[i + d], c = ids[i];
                if (!(cand[i] >= maxv[i + d]) && !row_has(idx + (size_t)r * K, K, c)) {
                    idx[(size_t)r * K + maxp[i + d]] = c;
                    dist[(size_t)r * K + maxp[i + d]] = cand[i];
                    maxp[i + d] = argmax_warp(dist + (size_t)r * K, K, &maxv[i + d]);
                }
            }
        }
        free(maxv); free(maxp); free(cand);
    }
}

typedef struct { float d; int i; } orc_entry;

static int entry_less(orc_entry a, orc_entry b)
{
    if (a.d < b.d) return 1;
    if (a.d > b.d) return 0;
    return (uint32_t)a.i < (uint32_t)b.i;
}

static int entry_cmp(const void* x, const void* y)
{
    orc_entry a = *(const orc_entry*)x, b = *(const orc_entry*)y;
    return entry_less(a, b) ? -1 : (entry_less(b, a) ? 1 : 0);
}

/* Canonical row: the K smallest entries of (row entries with idx >= 0) united
 * with `cands`, distinct by index (an index already in the row keeps the row's
 * distance), ordered by (distance, index); unused slots are (-1, +inf). */
static void canonical_row(int* ridx, float* rdist, int K, const orc_entry* cands, int n_c)
{
    orc_entry* all = (orc_entry*)malloc(sizeof(orc_entry) * (size_t)(K + n_c + 1));
    int n = 0;
    for (int k = 0; k < K; ++k) {
        if (ridx[k] < 0) continue;
        int dup = 0;
        for (int j = 0; j < n; ++j) if (all[j].i == ridx[k]) { dup = 1; break; }
        if (!dup) { all[n].d = rdist[k]; all[n].i = ridx[k]; n++; }
    }
    int n_row = n;
    for (int c = 0; c < n_c; ++c) {
        int dup = 0;
        for (int j = 0; j < n_row; ++j) if (all[j].i == cands[c].i) { dup = 1; break; }
        if (!dup) all[n++] = cands[c];
    }
    qsort(all, (size_t)n, sizeof(orc_entry), entry_cmp);
    /* duplicates among candidates share index and distance bits: adjacent now */
    int o = 0;
    for (int j = 0; j < n && o < K; ++j) {
        int dup = 0;
        for (int q = 0; q < o; ++q) if (ridx[q] == all[j].i) { dup = 1; break; }
        if (dup) continue;
        ridx[o] = all[j].i; rdist[o] = all[j].d; o++;
    }
    for (; o < K; ++o) { ridx[o] = -1; rdist[o] = INFINITY; }
    free(all);
}

/* Order every row by (distance, index), dropping repeated indices. */
ORC_API void orc_sort_rows(int N, int K, int* idx, float* dist)
{
    #pragma omp parallel for schedule(static)
    for (int p = 0; p < N; ++p) canonical_row(idx + (size_t)p * K, dist + (size_t)p * K, K, NULL, 0);
}

/* Tie-free statement of the bucket update: same candidate set and distance
 * bits as orc_bucket_knn_ref, result rows in canonical order.  Equal to the
 * reference-order result as a set whenever no two competing distances tie. */
ORC_API void orc_bucket_knn(const float* points, int N, int D, int K, const int* perm,
                            const int* leaf_start, const int* leaf_count, int n_leaves,
                            int* idx, float* dist)
{
    (void)N;
    #pragma omp parallel for schedule(dynamic, 16)
    for (int b = 0; b < n_leaves; ++b) {
        int m = leaf_count[b];
        const int* ids = perm + leaf_start[b];
        orc_entry* cands = (orc_entry*)malloc(sizeof(orc_entry) * (size_t)(m > 0 ? m : 1));
        for (int i = 0; i < m; ++i) {
            int n_c = 0;
            for (int j = 0; j < m; ++j) {
                if (j == i) continue;
                cands[n_c].i = ids[j];
                cands[n_c].d = (i < j)
                    ? orc_dist_sqr(points + (size_t)ids[i] * D, points + (size_t)ids[j] * D, D)
                    : orc_dist_sqr(points + (size_t)ids[j] * D, points + (size_t)ids[i] * D, D);
                n_c++;
            }
            canonical_row(idx + (size_t)ids[i] * K, dist + (size_t)ids[i] * K, K, cands, n_c);
        }
        free(cands);
    }
}

/* ------------------------------------------------------------------------- */
/* Query (ANN) bucket update                                                  */
/* ------------------------------------------------------------------------- */

/* Reference-order update of the query lists: one warp per query, its bucket's
 * base points taken 32 at a time in bucket order; a candidate already in the
 * row when its batch starts is dropped, the batch's distances are computed,
 * then the candidates replace the row's worst slot, one after another, when
 * strictly closer (src/kernels/build_tree_update_parents_ann.cu:271-513).
 * The distance is Sum (q_i - b_i)^2 in the order of orc_dist_sqr
 * (:205-228: term i on lane i%32, xor butterfly).  List indices are indices of
 * base points. */
ORC_API void orc_ann_bucket_knn_ref(const float* points, const float* queries, int NQ, int D, int K,
                                    const int* perm, const int* q_start, const int* q_count,
                                    int* idx, float* dist)
{
    #pragma omp parallel for schedule(dynamic, 64)
    for (int q = 0; q < NQ; ++q) {
        int* ridx = idx + (size_t)q * K;
        float* rdist = dist + (size_t)q * K;
        const int* ids = perm + q_start[q];
        const int m = q_count[q];
        float maxv;
        int maxp = argmax_warp(rdist, K, &maxv);
        for (int b0 = 0; b0 < m; b0 += 32) {
            int cand[32];
            float cd[32];
            const int nb = m - b0 < 32 ? m - b0 : 32;
            for (int j = 0; j < nb; ++j) {
                cand[j] = row_has(ridx, K, ids[b0 + j]) ? -1 : ids[b0 + j];
                if (cand[j] >= 0)
                    cd[j] = orc_dist_sqr(queries + (size_t)q * D, points + (size_t)cand[j] * D, D);
            }
            for (int j = 0; j < nb; ++j) {
                if (cand[j] < 0) continue;
                if (cd[j] < maxv) {
                    ridx[maxp] = cand[j];
                    rdist[maxp] = cd[j];
                    maxp = argmax_warp(rdist, K, &maxv);
                }
            }
        }
    }
}

/* Tie-free statement of the same update: every query row becomes the K
 * smallest distinct of (row united with its bucket's base points) by
 * (distance, index). */
ORC_API void orc_ann_bucket_knn(const float* points, const float* queries, int NQ, int D, int K,
                                const int* perm, const int* q_start, const int* q_count,
                                int* idx, float* dist)
{
    #pragma omp parallel for schedule(dynamic, 64)
    for (int q = 0; q < NQ; ++q) {
        const int* ids = perm + q_start[q];
        const int m = q_count[q];
        orc_entry* cands = (orc_entry*)malloc(sizeof(orc_entry) * (size_t)(m > 0 ? m : 1));
        for (int j = 0; j < m; ++j) {
            cands[j].i = ids[j];
            cands[j].d = orc_dist_sqr(queries + (size_t)q * D, points + (size_t)ids[j] * D, D);
        }
        canonical_row(idx + (size_t)q * K, dist + (size_t)q * K, K, cands, m);
        free(cands);
    }
}

/* Exact K nearest base points of every query row (distance in the order of
 * orc_dist_sqr), ordered by (distance, index): the recall denominator of the
 * query path. */
ORC_API void orc_bruteforce_ann(const float* points, int N, const float* queries, int NQ, int D,
                                int K, int* idx, float* dist)
{
    #pragma omp parallel for schedule(dynamic, 8)
    for (int q = 0; q < NQ; ++q) {
        orc_entry* all = (orc_entry*)malloc(sizeof(orc_entry) * (size_t)(N > 0 ? N : 1));
        for (int p = 0; p < N; ++p) {
            all[p].i = p;
            all[p].d = orc_dist_sqr(queries + (size_t)q * D, points + (size_t)p * D, D);
        }
        qsort(all, (size_t)N, sizeof(orc_entry), entry_cmp);
        for (int k = 0; k < K; ++k) {
            idx[(size_t)q * K + k] = k < N ? all[k].i : -1;
            dist[(size_t)q * K + k] = k < N ? all[k].d : INFINITY;
        }
        free(all);
    }
}

/* ------------------------------------------------------------------------- */
/* Symmetric closure of the graph                                             */
/* ------------------------------------------------------------------------- */

/* Row p of the result: p's valid entries and every q that lists p without being
 * listed by p (src/rsfk.cu:1229-1299: symmetric_knn_graph_edge_count counts one
 * entry per listed neighbour plus one in the neighbour's row when the edge is
 * not mutual; symmetric_knn_graph_add_edges writes them).  Rows are ordered by
 * neighbour index here (the reference leaves them in atomic arrival order);
 * -1 entries are skipped.  offsets has N+1 entries; with sym_idx == NULL only
 * the offsets are computed.  Returns the number of entries. */
ORC_API long long orc_symmetrize(int N, int K, const int* idx, const float* dist, long long* offsets,
                                 int* sym_idx, float* sym_dist)
{
    long long* deg = (long long*)calloc((size_t)N + 1, sizeof(long long));
    for (int p = 0; p < N; ++p)
        for (int k = 0; k < K; ++k) {
            int q = idx[(size_t)p * K + k];
            if (q < 0 || q >= N) continue;
            deg[p]++;
            if (q != p && !row_has(idx + (size_t)q * K, K, p)) deg[q]++;
        }
    long long run = 0;
    for (int p = 0; p < N; ++p) { offsets[p] = run; run += deg[p]; }
    offsets[N] = run;
    if (sym_idx) {
        long long* cur = (long long*)calloc((size_t)N + 1, sizeof(long long));
        orc_entry* tmp;
        for (int p = 0; p < N; ++p)
            for (int k = 0; k < K; ++k) {
                int q = idx[(size_t)p * K + k];
                if (q < 0 || q >= N) continue;
                float d = dist ? dist[(size_t)p * K + k] : 0.0f;
                sym_idx[offsets[p] + cur[p]] = q;
                if (sym_dist) sym_dist[offsets[p] + cur[p]] = d;
                cur[p]++;
                if (q != p && !row_has(idx + (size_t)q * K, K, p)) {
                    sym_idx[offsets[q] + cur[q]] = p;
                    if (sym_dist) sym_dist[offsets[q] + cur[q]] = d;
                    cur[q]++;
                }
            }
        /* order every row by neighbour index (entries of a row are distinct) */
        long long longest = 0;
        for (int p = 0; p < N; ++p) if (deg[p] > longest) longest = deg[p];
        tmp = (orc_entry*)malloc(sizeof(orc_entry) * (size_t)(longest > 0 ? longest : 1));
        for (int p = 0; p < N; ++p) {
            long long L = deg[p];
            for (long long e = 0; e < L; ++e) {
                tmp[e].i = sym_idx[offsets[p] + e];
                tmp[e].d = sym_dist ? sym_dist[offsets[p] + e] : 0.0f;
            }
            for (long long a = 1; a < L; ++a) { /* insertion sort by index */
                orc_entry x = tmp[a];
                long long b = a - 1;
                while (b >= 0 && tmp[b].i > x.i) { tmp[b + 1] = tmp[b]; --b; }
                tmp[b + 1] = x;
            }
            for (long long e = 0; e < L; ++e) {
                sym_idx[offsets[p] + e] = tmp[e].i;
                if (sym_dist) sym_dist[offsets[p] + e] = tmp[e].d;
            }
        }
        free(tmp);
        free(cur);
    }
    free(deg);
    return run;
}

/* ------------------------------------------------------------------------- */
/* Neighbour-of-neighbour exploration                                         */
/* ------------------------------------------------------------------------- */

/* Reference-order sweep: one point at a time, candidates old[old[p][i]][k] in
 * (i,k) order, skipped when already in the row being updated, inserted over
 * the current worst slot when strictly closer; the worst slot is the first
 * maximum of a serial scan
 * (src/kernels/nearest_neighbors_exploring.cu:66-145).  Negative ids are
 * skipped here; the reference indexes with them (:83-88). */
ORC_API void orc_explore_ref(const float* points, int N, int D, int K, const int* old_idx,
                             int* idx, float* dist)
{
    #pragma omp parallel for schedule(dynamic, 64)
    for (int p = 0; p < N; ++p) {
        int* ri = idx + (size_t)p * K;
        float* rd = dist + (size_t)p * K;
        int mp = 0;
        float mv = rd[0];
        for (int j = 1; j < K; ++j) if (rd[j] > mv) { mv = rd[j]; mp = j; }
        for (int i = 0; i < K; ++i) {
            int nb = old_idx[(size_t)p * K + i];
            if (nb < 0 || nb >= N) continue;
            for (int k = 0; k < K; ++k) {
                int c = old_idx[(size_t)nb * K + k];
                if (c < 0 || c >= N) continue;
                if (row_has(ri, K, c)) continue;
                float d = orc_dist_sqr(points + (size_t)c * D, points + (size_t)p * D, D);
                if (d < mv) {
                    ri[mp] = c; rd[mp] = d;
                    mp = 0; mv = rd[0];
                    for (int j = 1; j < K; ++j) if (rd[j] > mv) { mv = rd[j]; mp = j; }
                }
            }
        }
    }
}

/* Tie-free statement of the sweep for rows [row_begin, row_end): canonical
 * rows over (row united with all neighbour-of-neighbour candidates). */
ORC_API void orc_explore(const float* points, int N, int D, int K, const int* old_idx,
                         int* idx, float* dist, int row_begin, int row_end)
{
    #pragma omp parallel for schedule(dynamic, 64)
    for (int p = row_begin; p < row_end; ++p) {
        orc_entry* cands = (orc_entry*)malloc(sizeof(orc_entry) * (size_t)K * (size_t)K + 16);
        int n_c = 0;
        for (int i = 0; i < K; ++i) {
            int nb = old_idx[(size_t)p * K + i];
            if (nb < 0 || nb >= N) continue;
            for (int k = 0; k < K; ++k) {
                int c = old_idx[(size_t)nb * K + k];
                if (c < 0 || c >= N) continue;
                cands[n_c].i = c;
                cands[n_c].d = orc_dist_sqr(points + (size_t)c * D, points + (size_t)p * D, D);
                n_c++;
            }
        }
        canonical_row(idx + (size_t)p * K, dist + (size_t)p * K, K, cands, n_c);
        free(cands);
    }
}

/* Merge G canonical K-lists per row (lists[g] = idx_g, dists[g] = dist_g, each
 * [rows][K]) into out: K smallest distinct by (distance, index). */
ORC_API void orc_merge_lists(int rows, int K, int G, const int* const* lists,
                             const float* const* dists, int* out_idx, float* out_dist)
{
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        orc_entry* cands = (orc_entry*)malloc(sizeof(orc_entry) * (size_t)K * (size_t)G + 16);
        int n_c = 0;
        for (int g = 1; g < G; ++g)
            for (int k = 0; k < K; ++k) {
                int c = lists[g][(size_t)r * K + k];
                if (c < 0) continue;
                cands[n_c].i = c; cands[n_c].d = dists[g][(size_t)r * K + k]; n_c++;
            }
        for (int k = 0; k < K; ++k) {
            out_idx[(size_t)r * K + k] = lists[0][(size_t)r * K + k];
            out_dist[(size_t)r * K + k] = dists[0][(size_t)r * K + k];
        }
        canonical_row(out_idx + (size_t)r * K, out_dist + (size_t)r * K, K, cands, n_c);
        free(cands);
    }
}

/* ------------------------------------------------------------------------- */
/* Exact brute-force KNN (recall oracle and CPU baseline)                     */
/* ------------------------------------------------------------------------- */

/* Exact K nearest neighbours of the rows queries[0..nq) of `points` among all
 * N points (self included), rows in canonical order.  Plain serial fmaf sum
 * per pair, eight interleaved accumulators; all host threads. */
ORC_API int orc_bruteforce_knn(const float* points, int N, int D, const int* queries, int nq,
                               int K, int* out_idx, float* out_dist)
{
    int threads = 1;
    #ifdef _OPENMP
    threads = omp_get_max_threads();
    #endif
    #pragma omp parallel for schedule(dynamic, 4)
    for (int qi = 0; qi < nq; ++qi) {
        const float* q = points + (size_t)queries[qi] * D;
        orc_entry* heap = (orc_entry*)malloc(sizeof(orc_entry) * (size_t)K);
        int hn = 0;
        for (int j = 0; j < N; ++j) {
            const float* x = points + (size_t)j * D;
            float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            int i = 0;
            for (; i + 8 <= D; i += 8)
                for (int u = 0; u < 8; ++u) { float t = q[i + u] - x[i + u]; a[u] = fmaf(t, t, a[u]); }
            for (; i < D; ++i) { float t = q[i] - x[i]; a[i & 7] = fmaf(t, t, a[i & 7]); }
            orc_entry e;
            e.d = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
            e.i = j;
            if (hn < K) {
                /* max-heap insert */
                int c = hn++;
                heap[c] = e;
                while (c > 0) {
                    int par = (c - 1) / 2;
                    if (entry_less(heap[par], heap[c])) { orc_entry t = heap[par]; heap[par] = heap[c]; heap[c] = t; c = par; }
                    else break;
                }
            } else if (entry_less(e, heap[0])) {
                heap[0] = e;
                int c = 0;
                for (;;) {
                    int l = 2 * c + 1, r = l + 1, big = c;
                    if (l < hn && entry_less(heap[big], heap[l])) big = l;
                    if (r < hn && entry_less(heap[big], heap[r])) big = r;
                    if (big == c) break;
                    orc_entry t = heap[big]; heap[big] = heap[c]; heap[c] = t; c = big;
                }
            }
        }
        qsort(heap, (size_t)hn, sizeof(orc_entry), entry_cmp);
        for (int k = 0; k < K; ++k) {
            out_idx[(size_t)qi * K + k] = k < hn ? heap[k].i : -1;
            out_dist[(size_t)qi * K + k] = k < hn ? heap[k].d : INFINITY;
        }
        free(heap);
    }
    return threads;
}

/* Recall as the reference's experiments define it: shared neighbours per row
 * summed over rows, divided by rows*K (examples/utils/knn_compare.py:46-62). */
ORC_API double orc_recall(const int* truth, const int* approx, int rows, int K)
{
    long long hit = 0;
    #pragma omp parallel for reduction(+ : hit) schedule(static)
    for (int r = 0; r < rows; ++r) {
        const int* t = truth + (size_t)r * K;
        const int* a = approx + (size_t)r * K;
        for (int i = 0; i < K; ++i) {
            if (t[i] < 0) continue;
            int seen = 0;
            for (int q = 0; q < i; ++q) if (t[q] == t[i]) { seen = 1; break; }
            if (seen) continue;
            for (int j = 0; j < K; ++j) if (a[j] == t[i]) { hit++; break; }
        }
    }
    return (double)hit / ((double)rows * K);
}

/* ------------------------------------------------------------------------- */
/* Recovering split pairs of a reference tree from its leaves (tests only)    */
/* ------------------------------------------------------------------------- */

/* The reference does not report which pairs it sampled.  Given the points of a
 * node (ids[0..n)) and the leaf each point finally landed in (leaf[0..n), small
 * non-negative labels < n_leaves <= 64), this enumerates the distinct ways a
 * pair (p1, p2) of the node's own points can separate the node's LEAVES with the
 * restated split rule (n.x < c goes right; offset summed serially when is_root,
 * lane-strided otherwise): every leaf entirely on one side, both sides non-empty.
 * Each separation is returned once as the 64-bit mask of the leaves that go
 * right, with the first pair found for it.  Returns the number of separations
 * (at most cap). */
ORC_API int orc_find_leaf_separations(const float* points, int D, const int* ids, const int* leaf, int n,
                                      int n_leaves, int is_root, int min_side, uint64_t* masks_out,
                                      int* pairs_out, int cap)
{
    int found = 0;
    #pragma omp parallel
    {
        float* nrm = (float*)malloc(sizeof(float) * (size_t)D);
        #pragma omp for schedule(dynamic, 4)
        for (int a = 0; a < n; ++a) {
            for (int b = 0; b < n; ++b) {
                if (a == b || leaf[a] == leaf[b]) continue;
                const float* x1 = points + (size_t)ids[a] * D;
                const float* x2 = points + (size_t)ids[b] * D;
                float c = orc_hyperplane(x1, x2, D, is_root, nrm);
                uint64_t right = 0, left = 0;
                int n_right = 0, ok = 1;
                for (int q = 0; q < n && ok; ++q) {
                    int r = orc_project(nrm, points + (size_t)ids[q] * D, D) < c;
                    if (r) { right |= 1ull << leaf[q]; n_right++; } else left |= 1ull << leaf[q];
                    if (right & left) ok = 0;
                }
                if (!ok || right == 0 || left == 0) continue;
                if (n_right < min_side || n - n_right < min_side) continue;
                #pragma omp critical
                {
                    int known = 0;
                    for (int k = 0; k < found; ++k) if (masks_out[k] == right) { known = 1; break; }
                    if (!known && found < cap) {
                        masks_out[found] = right;
                        pairs_out[2 * found] = ids[a];
                        pairs_out[2 * found + 1] = ids[b];
                        found++;
                    }
                }
            }
        }
        free(nrm);
    }
    (void)n_leaves;
    return found;
}

/* ------------------------------------------------------------------------- */
/* k-means (Lloyd) for sample-tree clustering                                 */
/* ------------------------------------------------------------------------- */
/* PARITY UNPINNED: the reference has no k-means function.  The only k-means near its
 * path is the one inside nvGRAPH's spectral clustering, which it calls from
 * commented-out code (src/rsfk.cu:1521-1567, parameters at :1536-1539 and :1863-1868);
 * nvGRAPH is neither part of the reference tree nor of current toolkits.  What follows
 * states the rules the sm_100a kernels of this repository implement, so that they can
 * be checked against something; it is not a restatement of reference code.
 *
 * Assignment: the nearest centroid by squared distance in the reference's summation
 * order (orc_dist_sqr), ties to the lower centroid index.
 * Update: centroid c = mean of its members; the sum runs in double precision over the
 * members in ascending point index, member number j going to partial sum j mod 8, the
 * eight partial sums added in order 0..7; a cluster without members keeps its centroid. */
ORC_API void orc_kmeans_assign(const float* points, int N, int D, const float* centroids, int C,
                               int* assign, float* dist)
{
#pragma omp parallel for schedule(static)
    for (int p = 0; p < N; ++p) {
        int best = -1;
        float bd = INFINITY;
        for (int c = 0; c < C; ++c) {
            const float d = orc_dist_sqr(points + (size_t)p * D, centroids + (size_t)c * D, D);
            if (best < 0 || d < bd) { bd = d; best = c; }
        }
        assign[p] = best;
        dist[p] = bd;
    }
}

ORC_API void orc_kmeans_update(const float* points, int N, int D, const int* assign, int C,
                               float* centroids, int* counts)
{
    double* part = (double*)calloc((size_t)C * D * 8, sizeof(double));
    int* seen = (int*)calloc((size_t)C, sizeof(int));
    for (int p = 0; p < N; ++p) {
        const int c = assign[p];
        if (c < 0 || c >= C) continue;
        double* dst = part + ((size_t)c * 8 + (size_t)(seen[c] & 7)) * D;
        for (int k = 0; k < D; ++k) dst[k] += (double)points[(size_t)p * D + k];
        seen[c]++;
    }
    for (int c = 0; c < C; ++c) {
        if (counts) counts[c] = seen[c];
        if (seen[c] == 0) continue;
        for (int k = 0; k < D; ++k) {
            double s = 0.0;
            for (int w = 0; w < 8; ++w) s += part[((size_t)c * 8 + w) * D + k];
            centroids[(size_t)c * D + k] = (float)(s / (double)seen[c]);
        }
    }
    free(part);
    free(seen);
}
