// Leaf-bucket KNN with the bucket's Gram matrix on the 5th-generation tensor
// cores (tcgen05, sm_100a).  Included by rsfk_knn.cu.
//
// For D >= 64 the all-pairs distances of a bucket are a dense contraction:
// d2(i,j) = |yi|^2 + |yj|^2 - 2 yi.yj.  The tensor cores compute the Gram tile
// Y Y^T in TF32 with fp32 accumulation in tensor memory.  That value is used ONLY
// to decide which pairs can possibly enter a K-list: a pair passes when its
// approximate distance, lowered by a margin that covers the TF32 and accumulation
// error, is below the row's current K-th distance.  Every passing candidate is
// then evaluated again on the original coordinates in the reference's exact
// summation order (the routine the exploration sweep uses) and merged with the
// usual list rule, so the stored distances and the selected indices are the ones
// the SIMT kernel gives, bit for bit.
//
// Data path.  Once per tree k_tc_rows writes the points in leaf order, centred on
// the first point of their leaf (y = x - x_first: distances are unchanged, norms
// and with them the error margin shrink from |x| to the leaf's spread) and rounded
// to the nearest TF32 value, rows padded to a multiple of 32 floats, plus the squared
// norm of every (rounded) row.  A work item ("tile") is a
// block of 128 consecutive rows of one leaf against all the rows of that leaf, taken
// in column groups of 256.  The kernel is persistent, one CTA per SM, and
// warp-specialised:
//
//   warp 0    one thread issues 2-D TMA tile loads (cp.async.bulk.tensor, 128-byte
//             swizzle, no multicast) of 32-dimension chunks of the 128 A rows and
//             the 256 B rows into a ring of shared-memory stages;
//   warp 1    one thread issues tcgen05.mma (kind::tf32, M=128, N=256, K=8) on the
//             stages as they fill, frees a stage with tcgen05.commit, and hands a
//             finished 128 x 256 accumulator (one of two in tensor memory) to the
//             epilogue with another commit;
//   warps 2-9 read the accumulator with tcgen05.ld, turn it into one pass bit per
//             pair, and evaluate the passing pairs exactly -- while the tensor
//             cores already work on the next column group.
//
// Three kernels share the work of a tree.  k_tc_thresholds (the same pipeline, another
// epilogue) runs first and only over tiles with a row whose list is not full: it gives
// such rows a threshold from the approximate distances to their whole leaf.
// k_bucket_knn_tc filters and evaluates whatever comes in batches of 32 while a row's
// threshold can still tighten the filter of the following column groups; what is left
// of a row after the last group (fewer than 32 candidates) goes to a work list that
// k_tc_later evaluates with more warps in flight.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises an abort flag
// that all roles poll, the MMA thread drains its outstanding work with a last
// commit before tensor memory is released, the producer waits (bounded) for the
// loads still in flight, and the kernel sets the context's error flag.
#pragma once

#include <cuda.h>

namespace tc {

constexpr int BM = 128;                 // rows of a tile (MMA M)
constexpr int BN = 256;                 // columns of a group (MMA N)
constexpr int KC = 32;                  // dimensions per stage: 32 floats = one 128-byte swizzle row
constexpr int STAGES = 3;
constexpr int A_BYTES = BM * KC * 4;    // 16 KiB
constexpr int B_BYTES = BN * KC * 4;    // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 32 * (2 + EPI_WARPS);
constexpr int MAX_LEAF = 2048;          // pass bits of a row: one per leaf member
constexpr int TMEM_COLS = 512;          // two 128 x 256 fp32 accumulators
constexpr unsigned WAIT_LIMIT = 1u << 22; // polls before a wait gives up

struct Tile {
    int row0;   // first row of the leaf in leaf order
    int m;      // rows of the leaf
    int i0;     // first row of this tile inside the leaf
    int pad;
};

// How far the Gram distance can be from the true squared distance.  The rows the tensor
// cores see are y~ = rn_tf32(fl(x - c)), off from the exact centred row by at most
// 2^-11 (1 + 2^-12) of each coordinate, so |y~i - y~j| differs from the true distance d by
// at most delta = DELTA_REL (|y~i| + |y~j|).  What the kernel forms is
// t2 = |y~i|^2 + |y~j|^2 - 2 y~i.y~j = |y~i - y~j|^2 up to the fp32 accumulation of D
// products in the tensor core and of the norms (two units in the last place per addition
// allowed): e1 = acc_margin(D) (|y~i|^2 + |y~j|^2).  Hence
//     d^2 >= (sqrt(t2 + e1) - delta)^2 >= t2 - e1 - 2 sqrt(t2 + e1) delta =: lowered(t2)
//     d^2 <= (sqrt(t2 + e1) + delta)^2  =  t2 + e1 + 2 sqrt(t2 + e1) delta + delta^2
// The first is what a pair is filtered by, the second bounds the true distance of pairs used
// to derive a threshold for rows whose list is not full.
constexpr float DELTA_REL = 4.8828125e-4f * 1.002f; // 2^-11 and the centring's own rounding
__host__ __device__ inline float acc_margin(int D)
{
    return 1.25f * (2.5e-7f * (float)D + 1e-6f);
}

struct Layout {
    int pass_words;                 // 32-bit words of pass bits per row
    int off_pass, off_xp, off_queue, off_thr, off_nrm_a, off_nrm_b, off_sq_a, off_sq_b, off_boot, off_bar, total;
    int xp_floats;
};
__host__ __device__ inline Layout layout_for(int D, int max_leaf)
{
    Layout l;
    const int groups = (max_leaf + BN - 1) / BN;
    l.pass_words = groups * (BN / 32);
    l.xp_floats = (D + 3) & ~3;
    int o = STAGES * STAGE_BYTES;
    l.off_pass = o;  o += BM * l.pass_words * 4;
    l.off_xp = o;    o += EPI_WARPS * l.xp_floats * 4;
    l.off_queue = o; o += EPI_WARPS * EXP_QUEUE * 4;
    l.off_thr = o;   o += BM * 4;
    l.off_nrm_a = o; o += BM * 4;
    l.off_nrm_b = o; o += 2 * BN * 4;
    l.off_sq_a = o;  o += BM * 4;
    l.off_sq_b = o;  o += 2 * BN * 4;
    l.off_boot = o;  o += 4 * BM * 4;
    l.off_bar = o;   o += 128;
    l.total = o + 1024; // slack to align the stages to 1024 bytes
    return l;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred P1;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P1;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait; gives up when the limit runs out (and then raises the abort flag)
// or when another role has raised it.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag)
{
    for (unsigned it = 0; it < WAIT_LIMIT; ++it) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 31u) == 31u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// ---- TMA --------------------------------------------------------------------
// One 2-D tile (the box of the tensor map: 32 floats x 128 rows) at column x, row y
// into shared memory; completion is counted in bytes on the mbarrier.  x must be a
// multiple of 4 floats (16 bytes); rows outside the tensor read as zeros.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"((uint64_t)map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// ---- tcgen05 ----------------------------------------------------------------
// Shared-memory operand descriptor: K-major, 128-byte swizzle (the layout a TMA box of
// 128-byte rows produces): 8-row groups 1024 bytes apart, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr)
{
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}
// kind::tf32, fp32 accumulator, both operands K-major.
__device__ __forceinline__ uint32_t umma_idesc(int M, int N)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v)
{
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// barrier of the epilogue warps only (hardware barrier 1)
__device__ __forceinline__ void epi_barrier()
{
    asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
}

// ---------------------------------------------------------------------------
// Tile list of a tree: every leaf contributes ceil(m / 128) consecutive tiles.
// ---------------------------------------------------------------------------
__global__ void k_tc_tiles(const int* __restrict__ leaf_start, const int* __restrict__ leaf_count, int n_leaves,
                           int max_leaf, Tile* __restrict__ tiles, int tile_cap, int* __restrict__ n_tiles)
{
    const int leaf = blockIdx.x * blockDim.x + threadIdx.x;
    if (leaf >= n_leaves) return;
    const int m = min(leaf_count[leaf], max_leaf);
    const int nb = (m + BM - 1) / BM;
    const int base = atomicAdd(n_tiles, nb);
    for (int b = 0; b < nb; ++b)
        if (base + b < tile_cap) tiles[base + b] = Tile{leaf_start[leaf], m, b * BM, 0};
}

// ---------------------------------------------------------------------------
// Leaf-ordered copies of the points: rows[r][0..Dp) = x[perm[r]] - x[perm[row0]] rounded to
// TF32 (zeros beyond D) for the tensor cores, norms[r] = |row|^2, and rows_exact[r][0..D) =
// x[perm[r]] unchanged, from which the exact evaluation reads (the rows of a leaf lie together
// there and stay in L2 while the leaf's tiles are at work; gathered through the permutation
// they would come from all over the point array).  One CTA per tile, one warp per row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_tc_rows(const float* __restrict__ pts, int D, int Dp, const int* __restrict__ perm,
          const Tile* __restrict__ tiles, const int* __restrict__ n_tiles_ptr, int tile_cap,
          float* __restrict__ rows, float* __restrict__ norms, float* __restrict__ rows_exact)
{
    extern __shared__ float4 smem4[];
    float* centre = reinterpret_cast<float*>(smem4); // [D]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int n_tiles = min(*n_tiles_ptr, tile_cap);
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const Tile tl = tiles[t];
        __syncthreads();
        const float* c = pts + (size_t)perm[tl.row0] * D;
        for (int k = threadIdx.x; k < D; k += blockDim.x) centre[k] = __ldg(c + k);
        __syncthreads();
        const int n = min(BM, tl.m - tl.i0);
        for (int r = warp; r < n; r += n_warps) {
            const size_t row = (size_t)tl.row0 + tl.i0 + r;
            const float* x = pts + (size_t)perm[row] * D;
            float* y = rows + row * Dp;
            float* z = rows_exact + row * D;
            float nrm = 0.0f;
            for (int k = lane; k < Dp; k += 32) {
                const float xv = k < D ? __ldg(x + k) : 0.0f;
                if (k < D) z[k] = xv; // the untouched coordinates, for the exact evaluation
                float v = k < D ? __fsub_rn(xv, centre[k]) : 0.0f;
                // nearest value with 10 explicit mantissa bits: what kind::tf32 reads anyway
                v = __uint_as_float((__float_as_uint(v) + 0x1000u) & 0xffffe000u);
                y[k] = v;
                nrm = __fmaf_rn(v, v, nrm);
            }
#pragma unroll
            for (int s = 16; s >= 1; s >>= 1) nrm += __shfl_xor_sync(RSFK_FULL, nrm, s);
            if (lane == 0) norms[row] = nrm;
        }
    }
}

// ---------------------------------------------------------------------------
// The pipeline kernel.  stats[0] += pairs that passed the filter, stats[1] += pairs
// looked at.
// ---------------------------------------------------------------------------
// MODE 0: the filter and the exact evaluation.  MODE 1: the same pipeline over the tiles
// flagged in open_tile (tiles with a row whose list is not full), whose epilogue only
// derives a threshold for every row from the approximate distances of the WHOLE leaf
// (thr0[row], see the MODE 1 block below); nothing is evaluated and no list is touched.
template <int KPL, bool VEC4, int MODE>
__device__ __forceinline__ void
tc_pipeline(const CUtensorMap* map, const float* __restrict__ rows_exact, int D, int Dp, int K,
            const int* __restrict__ perm, const float* __restrict__ norms, const Tile* __restrict__ tiles,
            const int* __restrict__ n_tiles_ptr, int tile_cap, int* __restrict__ knn_idx,
            float* __restrict__ knn_dist, int max_leaf, float c_acc, unsigned long long* __restrict__ stats,
            int* __restrict__ error_flag, int* __restrict__ later_count, int* __restrict__ later_rows,
            int* __restrict__ later_cand, const int* __restrict__ open_tile, float* __restrict__ thr0)
{
    extern __shared__ unsigned char smem_raw[];
    // the swizzled operand tiles want 1024-byte alignment
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const Layout L0 = layout_for(D, max_leaf);
    unsigned* sPass = reinterpret_cast<unsigned*>(smem + L0.off_pass);
    float* sThr = reinterpret_cast<float*>(smem + L0.off_thr);
    float* sNrmA = reinterpret_cast<float*>(smem + L0.off_nrm_a);
    float* sNrmB = reinterpret_cast<float*>(smem + L0.off_nrm_b);
    float* sSqA = reinterpret_cast<float*>(smem + L0.off_sq_a);   // |y~| of the tile's rows
    float* sSqB = reinterpret_cast<float*>(smem + L0.off_sq_b);   // and of the group's columns
    uint64_t* sBar = reinterpret_cast<uint64_t*>(smem + L0.off_bar);
    // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], drain
    const uint32_t bar_full = smem_u32(sBar), bar_empty = smem_u32(sBar + STAGES);
    const uint32_t bar_acc_full = smem_u32(sBar + 2 * STAGES), bar_acc_empty = smem_u32(sBar + 2 * STAGES + 2);
    const uint32_t bar_drain = smem_u32(sBar + 2 * STAGES + 4);
    uint32_t* sTmem = reinterpret_cast<uint32_t*>(sBar + 2 * STAGES + 5);
    volatile int* sAbort = reinterpret_cast<volatile int*>(sTmem + 1);
    volatile int* sOpen = sAbort + 1; // [2]: does the tile (by parity) have a row whose list is not full?
    float* sBootT = reinterpret_cast<float*>(smem + L0.off_boot); // [2][BM] per column half
    float* sBootN = sBootT + 2 * BM;                              // [2][BM]
    const int PW = L0.pass_words;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_tiles = min(*n_tiles_ptr, tile_cap);
    const int n_chunks = Dp / KC;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full + 8 * b, 1); mbar_init(bar_acc_empty + 8 * b, EPI_WARPS); }
        mbar_init(bar_drain, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *sAbort = 0;
        sOpen[0] = 0;
        sOpen[1] = 0;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(sTmem)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *sTmem;

    if (warp == 0) {
        // ================= producer =================
        if (lane == 0) {
            unsigned it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                if (MODE == 1 && !open_tile[t]) continue;
                const Tile tl = tiles[t];
                const int n_groups = (tl.m + BN - 1) / BN;
                for (int g = 0; g < n_groups && ok; ++g) {
                    for (int c = 0; c < n_chunks; ++c, ++it) {
                        const int s = it % STAGES;
                        if (!mbar_wait(bar_empty + 8 * s, ((it / STAGES) & 1u) ^ 1u, sAbort)) { ok = false; break; }
                        const uint32_t dst = smem_u32(smem + s * STAGE_BYTES);
                        mbar_expect_tx(bar_full + 8 * s, STAGE_BYTES);
                        tma_load_2d(dst, map, c * KC, tl.row0 + tl.i0, bar_full + 8 * s);
                        tma_load_2d(dst + A_BYTES, map, c * KC, tl.row0 + g * BN, bar_full + 8 * s);
                        tma_load_2d(dst + 2 * A_BYTES, map, c * KC, tl.row0 + g * BN + BM, bar_full + 8 * s);
                    }
                }
            }
            // The MMA thread waits for every stage that was filled unless the kernel aborts;
            // then the loads still in flight are waited for here (bounded) so that nothing
            // writes shared memory after the CTA has left.
            if (!ok || *sAbort) {
                for (unsigned back = 0; back < (unsigned)STAGES && back < it; ++back) {
                    const unsigned j = it - 1 - back;
                    for (unsigned p = 0; p < WAIT_LIMIT; ++p)
                        if (mbar_try(bar_full + 8 * (j % STAGES), (j / STAGES) & 1u)) break;
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(BM, BN);
            unsigned it = 0, gc = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                if (MODE == 1 && !open_tile[t]) continue;
                const Tile tl = tiles[t];
                const int n_groups = (tl.m + BN - 1) / BN;
                for (int g = 0; g < n_groups && ok; ++g, ++gc) {
                    const int ab = gc & 1;
                    // the epilogue has read this accumulator's previous contents
                    if (!mbar_wait(bar_acc_empty + 8 * ab, ((gc >> 1) & 1u) ^ 1u, sAbort)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t tmem_d = tmem_base + (uint32_t)(ab * BN);
                    for (int c = 0; c < n_chunks; ++c, ++it) {
                        const int s = it % STAGES;
                        if (!mbar_wait(bar_full + 8 * s, (it / STAGES) & 1u, sAbort)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t a = smem_u32(smem + s * STAGE_BYTES), b = a + A_BYTES;
#pragma unroll
                        for (int k8 = 0; k8 < KC / 8; ++k8)
                            umma_tf32(tmem_d, umma_desc_sw128(a + k8 * 32), umma_desc_sw128(b + k8 * 32), idesc,
                                      (c > 0 || k8 > 0) ? 1u : 0u);
                        umma_commit(bar_empty + 8 * s); // the stage is free once these MMAs have read it
                    }
                    if (ok) umma_commit(bar_acc_full + 8 * ab);
                }
            }
            // nothing may still write tensor memory or read shared memory when the CTA ends:
            // a last commit completes after everything issued before it
            umma_commit(bar_drain);
            for (unsigned p = 0; p < WAIT_LIMIT; ++p)
                if (mbar_try(bar_drain, 0)) break;
        }
    } else {
        // ================= epilogue + exact evaluation =================
        const int ew = warp - 2;                  // 0..7
        const int quarter = warp & 3;             // tensor-memory lanes this warp may read
        const int half = ew >> 2;                 // which 128 of the group's 256 columns
        const int erow = 32 * quarter + lane;     // this thread's row of the tile
        const int et = threadIdx.x - 64;          // 0..255
        float* xp = reinterpret_cast<float*>(smem + L0.off_xp) + (size_t)ew * L0.xp_floats;
        int* queue = reinterpret_cast<int*>(smem + L0.off_queue) + ew * EXP_QUEUE;
        unsigned gc = 0;
        bool ok = true;
        unsigned long long n_passed = 0, n_pairs = 0;
        int tile_parity = 0;
        // MODE 1: what a thread keeps of its row from the first column group on
        float h_lo = 0.0f, h_hi = CUDART_INF_F, h_scale = 0.0f, h_nbmax = 0.0f;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, tile_parity ^= 1) {
            if (MODE == 1 && !open_tile[t]) continue;
            const Tile tl = tiles[t];
            const int n_groups = (tl.m + BN - 1) / BN;
            const int mI = min(BM, tl.m - tl.i0);
            const int* ids = perm + tl.row0;      // the leaf's members in leaf order
            epi_barrier();                        // the previous tile's rows are done with sPass / sThr
            for (int w = et; w < BM * PW; w += EPI_WARPS * 32) sPass[w] = 0u;
            if (et == 0) sOpen[tile_parity ^ 1] = 0; // the next tile's flag; nobody looks at it during this tile
            if (et < BM) {
                float thr = -1.0f, nrm = 0.0f;
                if (et < mI) {
                    const int id = ids[tl.i0 + et];
                    thr = __ldcg(knn_dist + (size_t)id * K + (K - 1));
                    nrm = norms[tl.row0 + tl.i0 + et];
                    // a row without a full list takes the threshold the first pass derived for it
                    if (MODE == 0 && thr0 != nullptr && thr == CUDART_INF_F) thr = thr0[tl.row0 + tl.i0 + et];
                    if (thr == CUDART_INF_F) sOpen[tile_parity] = 1;
                }
                sThr[et] = thr;
                sNrmA[et] = nrm;
                sSqA[et] = sqrtf(nrm);
            }
            for (int g = 0; g < n_groups && ok; ++g, ++gc) {
                const int ab = gc & 1;
                const int j0 = g * BN;
                float* nB = sNrmB + ab * BN;
                float* qB = sSqB + ab * BN;
                nB[et] = (j0 + et < tl.m) ? norms[tl.row0 + j0 + et] : 0.0f;
                qB[et] = sqrtf(nB[et]);
                // the wait of every thread is bounded; whether to go on is decided together
                // after the barrier, so that no warp leaves the others at a barrier
                mbar_wait(bar_acc_full + 8 * ab, (gc >> 1) & 1u, sAbort);
                epi_barrier();                    // also: sThr (row phase), sNrm*, cleared sPass
                if (*sAbort) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if constexpr (MODE == 1) {
                    // Threshold of a row from the approximate distances v = |y~i|^2 + |y~j|^2 - 2 y~i.y~j to
                    // ALL the leaf's rows.  The first group gives [lo, hi]: lo its smallest v, hi the larger
                    // of the two column halves' ceil(K/2)-th smallest (bisection, as in MODE 0), so at least
                    // K pairs have v <= hi.  Every group then counts its v <= hi in NB bins over [lo, hi]
                    // (shared memory, the pass-bit array).  After the last group the first bin edge with at
                    // least K pairs at or below it is a v that K pairs do not exceed; their true distances
                    // are then at most (sqrt(v + e1) + delta)^2, which is the threshold (e1 and delta with
                    // the largest column norm among the counted pairs).
                    const int NB = PW >= 64 ? 64 : (PW >= 32 ? 32 : (PW >= 16 ? 16 : 8));
                    const float n_row = sNrmA[erow];
                    const uint32_t trow = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(ab * BN + 128 * half);
                    if (g == 0) {
                        const int need = (K + 1) >> 1;
                        int n_valid = 0;
                        float vmin = CUDART_INF_F, vmax = -CUDART_INF_F;
#pragma unroll 1
                        for (int sb = 0; sb < 4; ++sb) {
                            float gv[32];
                            tmem_ld32(trow + (uint32_t)(32 * sb), gv);
#pragma unroll
                            for (int c = 0; c < 32; ++c) {
                                const int j = j0 + 128 * half + 32 * sb + c;
                                const float v = __fmaf_rn(-2.0f, gv[c], n_row + nB[128 * half + 32 * sb + c]);
                                if (j < tl.m && j != tl.i0 + erow) {
                                    n_valid++;
                                    vmin = fminf(vmin, v);
                                    vmax = fmaxf(vmax, v);
                                }
                            }
                        }
                        float lo = vmin, hi = vmax;
#pragma unroll 1
                        for (int it = 0; it < 12; ++it) {
                            const float mid = 0.5f * (lo + hi);
                            int below = 0;
#pragma unroll 1
                            for (int sb = 0; sb < 4; ++sb) {
                                float gv[32];
                                tmem_ld32(trow + (uint32_t)(32 * sb), gv);
#pragma unroll
                                for (int c = 0; c < 32; ++c) {
                                    const int j = j0 + 128 * half + 32 * sb + c;
                                    const float v = __fmaf_rn(-2.0f, gv[c], n_row + nB[128 * half + 32 * sb + c]);
                                    below += (j < tl.m && j != tl.i0 + erow && v <= mid) ? 1 : 0;
                                }
                            }
                            if (below >= need) hi = mid; else lo = mid;
                        }
                        sBootT[half * BM + erow] = n_valid >= need ? hi : CUDART_INF_F;
                        sBootN[half * BM + erow] = vmin;
                        epi_barrier();
                        h_hi = fmaxf(sBootT[erow], sBootT[BM + erow]);
                        h_lo = fminf(sBootN[erow], sBootN[BM + erow]);
                        h_scale = (h_hi < CUDART_INF_F && h_hi > h_lo) ? (float)NB / (h_hi - h_lo) : 0.0f;
                        h_nbmax = 0.0f;
                        epi_barrier(); // sBoot* are written again at the end of the tile
                    }
#pragma unroll 1
                    for (int sb = 0; sb < 4; ++sb) { // every lane takes part in the loads
                        float gv[32];
                        tmem_ld32(trow + (uint32_t)(32 * sb), gv);
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            const int j = j0 + 128 * half + 32 * sb + c;
                            const float nb = nB[128 * half + 32 * sb + c];
                            const float v = __fmaf_rn(-2.0f, gv[c], n_row + nb);
                            if (j < tl.m && j != tl.i0 + erow && v <= h_hi) {
                                int bin = (int)((v - h_lo) * h_scale);
                                bin = bin < 0 ? 0 : (bin > NB - 1 ? NB - 1 : bin);
                                atomicAdd(&sPass[erow * PW + ((bin + erow) & (NB - 1))], 1u);
                                h_nbmax = fmaxf(h_nbmax, nb);
                            }
                        }
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_acc_empty + 8 * ab);
                    if (g == n_groups - 1) {
                        sBootN[half * BM + erow] = h_nbmax;
                        epi_barrier(); // both halves' counts and largest norms are in
                        if (half == 0 && erow < mI) {
                            float thr_row = CUDART_INF_F;
                            if (h_hi < CUDART_INF_F) {
                                unsigned cum = 0;
                                int edge = NB;
                                for (int bin = 0; bin < NB; ++bin) {
                                    cum += sPass[erow * PW + ((bin + erow) & (NB - 1))];
                                    if (cum >= (unsigned)K) { edge = bin + 1; break; }
                                }
                                // a v counted in bins < edge is below lo + edge (hi - lo) / NB up to the
                                // rounding of the bin index (a few units in the last place of v - lo)
                                float v_k = h_hi;
                                if (edge < NB && h_scale > 0.0f)
                                    v_k = fminf(h_hi, h_lo + ((float)edge / h_scale) * 1.00001f);
                                const float nb_most = fmaxf(sBootN[erow], sBootN[BM + erow]);
                                const float e1 = c_acc * (n_row + nb_most);
                                const float delta = DELTA_REL * (sSqA[erow] + sqrtf(nb_most));
                                const float root = sqrtf(fmaxf(v_k + e1, 0.0f)) + delta;
                                thr_row = root * root * 1.000001f + 1e-30f;
                            }
                            thr0[tl.row0 + tl.i0 + erow] = thr_row;
                        }
                    }
                    continue;
                }
                {
                    float thr = sThr[erow];
                    const float n_row = sNrmA[erow];
                    const float q_row = sSqA[erow];
                    const bool live = erow < mI;
                    // Rows whose list is not full yet have no threshold, and every pair of the first
                    // column group would go on to the exact evaluation.  The approximate distances
                    // themselves give one: with T the larger of the two column halves'
                    // ceil(K/2)-th smallest Gram distance, at least K candidates have a true distance
                    // of at most upper(T), so no pair beyond that (by its lowered distance) can end
                    // up among the K nearest.  T is found by bisection over the tile row in tensor
                    // memory.
                    if (g == 0 && sOpen[tile_parity]) { // the same decision in every epilogue warp
                        const uint32_t trow = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(ab * BN + 128 * half);
                        const int need = (K + 1) >> 1;
                        int n_valid = 0;
                        float vmin = CUDART_INF_F, vmax = -CUDART_INF_F, nbmax = 0.0f;
#pragma unroll 1
                        for (int sb = 0; sb < 4; ++sb) {
                            float gv[32];
                            tmem_ld32(trow + (uint32_t)(32 * sb), gv);
#pragma unroll
                            for (int c = 0; c < 32; ++c) {
                                const int j = j0 + 128 * half + 32 * sb + c;
                                const float nb = nB[128 * half + 32 * sb + c];
                                const float v = __fmaf_rn(-2.0f, gv[c], n_row + nb);
                                if (j < tl.m && j != tl.i0 + erow) {
                                    n_valid++;
                                    vmin = fminf(vmin, v);
                                    vmax = fmaxf(vmax, v);
                                    nbmax = fmaxf(nbmax, nb);
                                }
                            }
                        }
                        float lo = vmin, hi = vmax;
#pragma unroll 1
                        for (int it = 0; it < 12; ++it) { // every lane takes part in the loads
                            const float mid = 0.5f * (lo + hi);
                            int below = 0;
#pragma unroll 1
                            for (int sb = 0; sb < 4; ++sb) {
                                float gv[32];
                                tmem_ld32(trow + (uint32_t)(32 * sb), gv);
#pragma unroll
                                for (int c = 0; c < 32; ++c) {
                                    const int j = j0 + 128 * half + 32 * sb + c;
                                    const float v = __fmaf_rn(-2.0f, gv[c], n_row + nB[128 * half + 32 * sb + c]);
                                    below += (j < tl.m && j != tl.i0 + erow && v <= mid) ? 1 : 0;
                                }
                            }
                            if (below >= need) hi = mid; else lo = mid;
                        }
                        // hi always has at least `need` candidates at or below it (it starts at the maximum)
                        sBootT[half * BM + erow] = n_valid >= need ? hi : CUDART_INF_F;
                        sBootN[half * BM + erow] = nbmax;
                        epi_barrier();
                        const float T = fmaxf(sBootT[erow], sBootT[BM + erow]);
                        const float nb_most = fmaxf(sBootN[erow], sBootN[BM + erow]);
                        if (thr == CUDART_INF_F && T < CUDART_INF_F) {
                            const float e1 = c_acc * (n_row + nb_most);
                            const float delta = DELTA_REL * (q_row + sqrtf(nb_most));
                            const float root = sqrtf(fmaxf(T + e1, 0.0f)) + delta;
                            thr = root * root * 1.000001f + 1e-30f;
                        }
                    }
#pragma unroll 1
                    for (int sb = 0; sb < 4; ++sb) {
                        const int c0 = 128 * half + 32 * sb;
                        float gv[32];
                        tmem_ld32(tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(ab * BN + c0), gv);
                        unsigned word = 0;
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            const int j = j0 + c0 + c;
                            const float nn = n_row + nB[c0 + c];
                            const float t2 = __fmaf_rn(-2.0f, gv[c], nn);
                            const float e1 = c_acc * nn;
                            const float two_delta = (2.0f * DELTA_REL) * (q_row + qB[c0 + c]);
                            const float d2 = t2 - e1 - sqrtf(fmaxf(t2 + e1, 0.0f)) * two_delta;
                            // a pair whose lowered distance EQUALS the K-th distance passes too (the margin is zero
                            // for coincident points, and a tie with a lower index enters the list);
                            // !(d2 > thr) also keeps the candidate when anything is not a number
                            if (j < tl.m && j != tl.i0 + erow && !(d2 > thr)) word |= 1u << c;
                        }
                        if (live) {
                            sPass[erow * PW + (j0 >> 5) + (c0 >> 5)] = word;
                            n_passed += __popc(word);
                            n_pairs += max(0, min(32, tl.m - (j0 + c0)));
                        }
                    }
                }
                // the accumulator may be overwritten once every warp has read its part
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * ab);
                epi_barrier();                    // pass words of this group complete

                // ---- rows of the tile: exact distances of passing candidates ----
                // A row is flushed as soon as 32 candidates wait (its K-th distance then
                // tightens the filter of the following groups) and after the last group.
                const bool last_group = (g == n_groups - 1);
                const int n_words = min((tl.m + 31) >> 5, (g + 1) * (BN / 32));
                // queue[0..n) of row r becomes an entry of k_tc_later's work list (a row at most once per tree)
                auto hand_over = [&](int r, int n) {
                    __syncwarp();
                    int slot = 0;
                    if (lane == 0) slot = atomicAdd(later_count, 1);
                    slot = __shfl_sync(RSFK_FULL, slot, 0);
                    if (lane == 0) later_rows[slot] = tl.row0 + tl.i0 + r;
                    later_cand[(size_t)slot * 32 + lane] = lane < n ? queue[lane] : -1;
                    __syncwarp();
                };
                for (int r = ew; r < mI; r += EPI_WARPS) {
                    int pending = 0;
                    for (int w = lane; w < n_words; w += 32) pending += __popc(sPass[r * PW + w]);
#pragma unroll
                    for (int sft = 16; sft >= 1; sft >>= 1) pending += __shfl_xor_sync(RSFK_FULL, pending, sft);
                    if (pending == 0 || (pending < 32 && !last_group)) continue;
                    if (pending < 32 && later_cand != nullptr) {
                        // fewer than a batch after the last group: handed to k_tc_later, which has the
                        // warps in flight that these short, latency-bound evaluations want
                        int qn = 0;
                        for (int w = 0; w < n_words; ++w) {
                            const unsigned bits = sPass[r * PW + w];
                            if ((bits >> lane) & 1u) queue[qn + __popc(bits & ((1u << lane) - 1u))] = tl.row0 + 32 * w + lane;
                            qn += __popc(bits);
                        }
                        hand_over(r, qn);
                        continue;
                    }
                    const int self = ids[tl.i0 + r];
                    __syncwarp();
                    for (int k = lane; k < D; k += 32)
                        xp[k] = rows_exact[(size_t)(tl.row0 + tl.i0 + r) * D + k];
                    WarpList<KPL> L;
                    L.load(knn_idx + (size_t)self * K, knn_dist + (size_t)self * K, K, lane);
                    __syncwarp();
                    bool changed = false;
                    int qn = 0;
                    // the first n (<= 32) queued rows (leaf order): exact distances in the sweep's
                    // arithmetic from the leaf-ordered copy, then the usual merge under their point ids
                    auto merge = [&](float dsum, int item, int n) {
                        const int ci = item < n ? perm[queue[item]] : -1;
                        unsigned mask = __ballot_sync(RSFK_FULL, ci >= 0 && L.beats_threshold(dsum, ci));
                        while (mask) {
                            const int b = __ffs(mask) - 1;
                            mask &= mask - 1;
                            changed |= L.try_insert(__shfl_sync(RSFK_FULL, dsum, b), __shfl_sync(RSFK_FULL, ci, b), K, lane);
                        }
                    };
                    for (int w = 0; w < n_words; ++w) {
                        const unsigned bits = sPass[r * PW + w];
                        if (bits == 0) continue;
                        __syncwarp();
                        if (lane == 0) sPass[r * PW + w] = 0u;
                        const bool pass = (bits >> lane) & 1u;
                        if (pass) queue[qn + __popc(bits & ((1u << lane) - 1u))] = tl.row0 + 32 * w + lane;
                        qn += __popc(bits);
                        __syncwarp();
                        if (qn >= 32) {
                            int item;
                            const float dsum = VEC4 ? explore_dist32_vec4(rows_exact, D, xp, queue, 32, lane, item)
                                                    : explore_dist32_scalar(rows_exact, D, xp, queue, 32, lane, item);
                            merge(dsum, item, 32);
                            __syncwarp();
                            const int rest = qn - 32;
                            const int tmp = lane < rest ? queue[32 + lane] : -1;
                            __syncwarp();
                            if (lane < rest) queue[lane] = tmp;
                            qn = rest;
                            __syncwarp();
                        }
                    }
                    if (qn > 0 && last_group && later_cand != nullptr) {
                        hand_over(r, qn); // the rest after the full batches
                    } else if (qn > 0) {
                        int item;
                        const float dsum = VEC4 ? explore_dist32_vec4(rows_exact, D, xp, queue, qn, lane, item)
                                                : explore_dist32_scalar(rows_exact, D, xp, queue, qn, lane, item);
                        merge(dsum, item, qn);
                    }
                    if (changed) {
                        L.store(knn_idx + (size_t)self * K, knn_dist + (size_t)self * K, K, lane);
                        if (lane == 0) sThr[r] = fminf(sThr[r], L.thr_d); // a first-pass threshold stays until the list is full
                    }
                }
            }
        }
        if (stats != nullptr) {
#pragma unroll
            for (int sft = 16; sft >= 1; sft >>= 1) {
                n_passed += __shfl_xor_sync(RSFK_FULL, n_passed, sft);
                n_pairs += __shfl_xor_sync(RSFK_FULL, n_pairs, sft);
            }
            if (lane == 0 && n_pairs) {
                atomicAdd(&stats[0], n_passed);
                atomicAdd(&stats[1], n_pairs);
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
    if (threadIdx.x == 0 && *sAbort) atomicExch(error_flag, 1);
}

template <int KPL, bool VEC4>
__global__ void __launch_bounds__(THREADS, 1)
k_bucket_knn_tc(const __grid_constant__ CUtensorMap map, const float* __restrict__ rows_exact, int D, int Dp, int K,
                const int* __restrict__ perm, const float* __restrict__ norms, const Tile* __restrict__ tiles,
                const int* __restrict__ n_tiles_ptr, int tile_cap, int* __restrict__ knn_idx,
                float* __restrict__ knn_dist, int max_leaf, float c_acc, unsigned long long* __restrict__ stats,
                int* __restrict__ error_flag, int* __restrict__ later_count, int* __restrict__ later_rows,
                int* __restrict__ later_cand, const float* __restrict__ thr0)
{
    tc_pipeline<KPL, VEC4, 0>(&map, rows_exact, D, Dp, K, perm, norms, tiles, n_tiles_ptr, tile_cap, knn_idx, knn_dist,
                              max_leaf, c_acc, stats, error_flag, later_count, later_rows, later_cand, nullptr,
                              const_cast<float*>(thr0));
}

// First pass over the tiles that have a row without a full list (open_tile, n_open of them):
// thr0[row] for every row of those tiles.  Leaves at once when there is no such tile.
__global__ void __launch_bounds__(THREADS, 1)
k_tc_thresholds(const __grid_constant__ CUtensorMap map, int D, int Dp, int K, const int* __restrict__ perm,
                const float* __restrict__ norms, const Tile* __restrict__ tiles, const int* __restrict__ n_tiles_ptr,
                int tile_cap, float* __restrict__ knn_dist, int max_leaf, float c_acc, int* __restrict__ error_flag,
                const int* __restrict__ open_tile, const int* __restrict__ n_open, float* __restrict__ thr0)
{
    if (*n_open == 0) return;
    tc_pipeline<1, false, 1>(&map, nullptr, D, Dp, K, perm, norms, tiles, n_tiles_ptr, tile_cap, nullptr, knn_dist,
                             max_leaf, c_acc, nullptr, error_flag, nullptr, nullptr, nullptr, open_tile, thr0);
}

// open_tile[t] = 1 when tile t has a row whose list is not full; *n_open counts them.  One warp per tile.
__global__ void k_tc_open_tiles(const Tile* __restrict__ tiles, const int* __restrict__ n_tiles_ptr, int tile_cap,
                                const int* __restrict__ perm, const float* __restrict__ knn_dist, int K,
                                int* __restrict__ open_tile, int* __restrict__ n_open)
{
    const int lane = threadIdx.x & 31;
    const int n_tiles = min(*n_tiles_ptr, tile_cap);
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < n_tiles; t += (gridDim.x * blockDim.x) >> 5) {
        const Tile tl = tiles[t];
        const int n = min(BM, tl.m - tl.i0);
        bool open = false;
        for (int r = lane; r < n; r += 32)
            open |= knn_dist[(size_t)perm[tl.row0 + tl.i0 + r] * K + (K - 1)] == CUDART_INF_F;
        open = __any_sync(RSFK_FULL, open);
        if (lane == 0) {
            open_tile[t] = open ? 1 : 0;
            if (open) atomicAdd(n_open, 1);
        }
    }
}

// ---------------------------------------------------------------------------
// Rows that the pipeline kernel left with fewer than 32 candidates: one warp per row
// evaluates them exactly and merges them.  Every row occurs at most once per tree, so
// no two warps touch one list.  later_cand[slot][0..n) are rows in leaf order.
// ---------------------------------------------------------------------------
constexpr int LATER_WARPS = 4;
template <int KPL, bool VEC4>
__global__ void __launch_bounds__(32 * LATER_WARPS, VEC4 ? 6 : 1)
k_tc_later(const float* __restrict__ rows_exact, int D, int K, const int* __restrict__ perm,
           const int* __restrict__ later_count, const int* __restrict__ later_rows,
           const int* __restrict__ later_cand, int* __restrict__ knn_idx, float* __restrict__ knn_dist)
{
    extern __shared__ float4 later_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int xp_floats = (D + 3) & ~3;
    float* xp = reinterpret_cast<float*>(later_smem) + (size_t)warp * (xp_floats + 32);
    int* queue = reinterpret_cast<int*>(xp + xp_floats);
    const int n_rows = *later_count;
    const int step = gridDim.x * LATER_WARPS;
    int slot = blockIdx.x * LATER_WARPS + warp;
    // the next row's position, point and candidates are requested one row ahead
    int pos_next = slot < n_rows ? later_rows[slot] : 0;
    int self_next = slot < n_rows ? perm[pos_next] : 0;
    int cand_next = slot < n_rows ? later_cand[(size_t)slot * 32 + lane] : -1;
    for (; slot < n_rows; slot += step) {
        const int pos = pos_next, self = self_next, cand = cand_next;
        if (slot + step < n_rows) {
            pos_next = later_rows[slot + step];
            cand_next = later_cand[(size_t)(slot + step) * 32 + lane];
        }
        const int qn = __popc(__ballot_sync(RSFK_FULL, cand >= 0));
        __syncwarp();
        queue[lane] = cand;
        if (VEC4) {
            const float4* src = reinterpret_cast<const float4*>(rows_exact + (size_t)pos * D);
            for (int k4 = lane; k4 < (D >> 2); k4 += 32) reinterpret_cast<float4*>(xp)[k4] = src[k4];
        } else {
            for (int k = lane; k < D; k += 32) xp[k] = rows_exact[(size_t)pos * D + k];
        }
        WarpList<KPL> L;
        L.load(knn_idx + (size_t)self * K, knn_dist + (size_t)self * K, K, lane);
        __syncwarp();
        bool changed = false;
        // eight candidates at a time: two rows per lane group and four k-steps requested together, so
        // that few dependent load rounds are left, in few enough registers for 24 warps per SM
        for (int base = 0; base < qn; base += (VEC4 ? 8 : 32)) {
            const int m = min(qn - base, VEC4 ? 8 : 32);
            int item;
            float dsum;
            if (VEC4)
                dsum = explore_dist_few_vec4<2, 4>(rows_exact, D, xp, queue + base, m, lane, item);
            else
                dsum = explore_dist32_scalar(rows_exact, D, xp, queue + base, m, lane, item);
            const int ci = item < m ? perm[queue[base + item]] : -1;
            unsigned mask = __ballot_sync(RSFK_FULL, ci >= 0 && L.beats_threshold(dsum, ci));
            while (mask) {
                const int b = __ffs(mask) - 1;
                mask &= mask - 1;
                changed |= L.try_insert(__shfl_sync(RSFK_FULL, dsum, b), __shfl_sync(RSFK_FULL, ci, b), K, lane);
            }
        }
        if (changed) L.store(knn_idx + (size_t)self * K, knn_dist + (size_t)self * K, K, lane);
        if (slot + step < n_rows) self_next = perm[pos_next];
    }
}

} // namespace tc
