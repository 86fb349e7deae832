"""Makes the scratch copy of the reference's driver that writes out the tree it built.

    python oracle/patch_ref_dump.py <reference root> <output rsfk.cu>

The reference keeps a tree only on the query path (its RSFKIndexTree, src/include/rsfk.h:89-127,
filled at src/rsfk.cu:1117-1150) and hands it to nobody.  This script copies src/rsfk.cu and
adds, in the copy only, a function of this repository's own that copies those arrays to the
host and writes them to the file named by the environment variable RSFK_DUMP_TREE, called right
after the tree is built (after the call at src/rsfk.cu:177-178).  Nothing else is changed;
the copy lives under oracle/_ref/ (git-ignored) and is compiled by `make -C oracle ref_dump`.
tests/golden/make_ref_tree_golden.py turns a dump into a fixture.

File layout (little endian): int32 magic 0x52534654, D, depths, total_leaves, max_child; then per
depth: int32 n (entries kept for the level), float32 planes[n][D+1], int32 parents[n],
int32 children[n][2], uint8 is_leaf[n], int32 child_count[n]; then int32 level_count[depths],
int32 buckets[total_leaves][max_child], int32 bucket_sizes[total_leaves].
"""
import sys

DUMP_FN = r'''
#include <cstdio>
#include <cstdlib>
#include <thrust/host_vector.h>
// added by oracle/patch_ref_dump.py (not part of the reference): writes the index tree to a file
static void rsfk_b200_dump_tree(const char* path, RSFKIndexTree* t, int D)
{
    FILE* f = fopen(path, "wb");
    if (!f) return;
    cudaDeviceSynchronize();
    const int depths = t->reached_max_depth;
    int head[5] = {0x52534654, D, depths, t->total_leaves, t->max_child};
    fwrite(head, sizeof(int), 5, f);
    thrust::host_vector<int> level_count(*t->device_depth_level_count);
    for (int d = 0; d < depths; ++d) {
        thrust::host_vector<RSFK_typepoints> planes(*t->device_tree[d]);
        thrust::host_vector<int> parents(*t->device_tree_parents[d]);
        thrust::host_vector<int> children(*t->device_tree_children[d]);
        thrust::host_vector<bool> leaf(*t->device_is_leaf[d]);
        thrust::host_vector<int> count(*t->device_child_count[d]);
        int n = level_count[d];
        if (n < 0) n = 0;
        if ((size_t)n > parents.size()) n = (int)parents.size();
        if ((size_t)n * (D + 1) > planes.size()) n = (int)(planes.size() / (D + 1));
        if ((size_t)2 * n > children.size()) n = (int)(children.size() / 2);
        if ((size_t)n > leaf.size()) n = (int)leaf.size();
        if ((size_t)n > count.size()) n = (int)count.size();
        fwrite(&n, sizeof(int), 1, f);
        for (int i = 0; i < n * (D + 1); ++i) { float v = (float)planes[i]; fwrite(&v, sizeof(float), 1, f); }
        fwrite(parents.data(), sizeof(int), n, f);
        fwrite(children.data(), sizeof(int), 2 * (size_t)n, f);
        for (int i = 0; i < n; ++i) { unsigned char b = leaf[i] ? 1 : 0; fwrite(&b, 1, 1, f); }
        fwrite(count.data(), sizeof(int), n, f);
    }
    fwrite(level_count.data(), sizeof(int), depths, f);
    thrust::host_vector<int> buckets(*t->device_nodes_buckets);
    thrust::host_vector<int> sizes(*t->device_bucket_sizes);
    fwrite(buckets.data(), sizeof(int), (size_t)t->total_leaves * t->max_child, f);
    fwrite(sizes.data(), sizeof(int), t->total_leaves, f);
    fclose(f);
}
'''

CALL = r'''
    if (const char* rsfk_b200_dump_path = getenv("RSFK_DUMP_TREE")) rsfk_b200_dump_tree(rsfk_b200_dump_path, rsfkindextree, D);
'''


def main(ref_root, out_path):
    src = open(ref_root + "/src/rsfk.cu").read()
    # the function goes in front of the first member function of the driver class
    anchor_fn = "TreeInfo RSFK::create_bucket_from_sample_tree("
    first = src.find("RSFK::")
    line_start = src.rfind("\n", 0, first) + 1
    assert first >= 0 and anchor_fn in src
    src = src[:line_start] + DUMP_FN + "\n" + src[line_start:]
    # the call goes after the tree of the query path is built
    anchor = "device_points, N, D, VERBOSE, forest_log, run_name, false, rsfkindextree);"
    assert src.count(anchor) == 1, "the query path's tree call was not found exactly once"
    at = src.index(anchor) + len(anchor)
    stop = "tree_bucket_construction.stop();"
    at2 = src.index(stop, at) + len(stop)
    src = src[:at2] + CALL + src[at2:]
    open(out_path, "w").write(src)


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
