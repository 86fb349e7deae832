// Leaf-bucket KNN with the bucket's Gram matrix on the 5th-generation tensor
// cores (tcgen05, sm_100a).  Included by rsfk_knn.cu.
//
// For D >= 64 the all-pairs distances of a bucket are a dense contraction:
// d2(i,j) = |xi|^2 + |xj|^2 - 2 xi.xj.  The Gram tile X X^T is computed by
// tcgen05.mma kind::tf32 with a 3xTF32 split (x = big + small, three products
// big.big + big.small + small.big, fp32 accumulation in tensor memory), which
// keeps about 21 mantissa bits.  That value is used ONLY to decide which pairs
// can possibly enter a K-list: a pair passes when its approximate distance,
// lowered by a safety margin that covers the split and accumulation error, is
// below the row's current K-th distance.  Every passing candidate is then
// evaluated again in the reference's exact summation order (the same routine
// the exploration sweep uses) and merged with the usual list rule, so the
// stored distances and the selected indices are the ones the SIMT path gives.
//
// One CTA per leaf.  The leaf's rows are cut into blocks of 128; for a block
// pair (I, J) the 128 x 128 Gram tile accumulates in tensor memory over K-chunks
// of 32 dimensions.  Operands are staged by the threads themselves (rows are
// gathered through the permutation, so no 2-D TMA tile exists): a chunk is split
// into big/small TF32 and stored in the K-major, no-swizzle core-matrix layout
// the UMMA shared-memory descriptor addresses (8 rows x 16 bytes per core
// matrix).  After all J the rows of block I hold one pass bit per leaf member.
#pragma once

namespace tc {

constexpr int TC_ROWS = 128;            // MMA M and N: rows of one leaf block
constexpr int TC_KC = 32;               // dimensions staged per chunk
constexpr int TC_LBO = 128;             // bytes between K-adjacent core matrices
constexpr int TC_SBO = (TC_KC / 4) * 128; // bytes between 8-row groups
constexpr int TC_OPERAND_BYTES = TC_ROWS * TC_KC * 4; // one of big / small
constexpr unsigned TC_WAIT_LIMIT = 1u << 22;          // polls before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

// K-major, no swizzle: start address, leading (K) byte offset, stride (8-row
// group) byte offset, all in 16-byte units; descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr)
{
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)(TC_LBO >> 4) << 16) |
           ((uint64_t)(TC_SBO >> 4) << 32) | (1ull << 46);
}

// kind::tf32, fp32 accumulator, both operands K-major, M = N = 128.
__device__ __forceinline__ uint32_t umma_idesc()
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TC_ROWS >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);
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

// Bounded wait on an mbarrier phase; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t phase)
{
    for (unsigned it = 0; it < TC_WAIT_LIMIT; ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred P1;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, P1;\n\t"
            "}"
            : "=r"(done)
            : "r"(bar), "r"(phase)
            : "memory");
        if (done) return true;
    }
    return false;
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

// Relative safety margin of the 3xTF32 Gram distance, applied to |xi|^2+|xj|^2:
// dropped small.small terms and truncated small parts (each below 2^-20 of the
// product) plus fp32 accumulation over up to 3*D terms.
constexpr float TC_MARGIN = 1.5e-4f;

constexpr int TC_MAX_BLOCKS = 16; // leaves of up to 2048 points

// Shared-memory layout of one CTA (bytes).  Leaves that fit one block need a
// single operand pair (the Gram tile is X_I X_I^T); larger leaves also stage the
// J block.
struct Layout {
    int two_operands, pass_words; // pass_words: 32-bit words of pass bits per row
    int off_b, off_norm, off_ids, off_pass, off_xp, off_queue, off_misc, total;
};
__host__ __device__ inline Layout layout_for(int D, int max_leaf)
{
    Layout l;
    const int n_blocks = (max_leaf + TC_ROWS - 1) / TC_ROWS;
    l.two_operands = n_blocks > 1;
    l.pass_words = n_blocks * (TC_ROWS / 32);
    int o = 2 * TC_OPERAND_BYTES;
    l.off_b = o;     o += l.two_operands ? 2 * TC_OPERAND_BYTES : 0;
    l.off_norm = o;  o += 2 * TC_ROWS * 4;
    l.off_ids = o;   o += 2 * TC_ROWS * 4;
    l.off_pass = o;  o += TC_ROWS * l.pass_words * 4;
    // the per-warp copy of a row (exact distances, row phase) reuses the operand
    // area, which is idle then, when it fits there
    const int xp_bytes = KNN_WARPS * ((D + 3) & ~3) * 4;
    const int operand_area = (l.two_operands ? 4 : 2) * TC_OPERAND_BYTES;
    if (xp_bytes <= operand_area) l.off_xp = 0;
    else { l.off_xp = o; o += xp_bytes; }
    l.off_queue = o; o += KNN_WARPS * EXP_QUEUE * 4;
    l.off_misc = o;  o += 64;
    l.total = o;
    return l;
}

// Stages dimensions [k0, k0+TC_KC) of the 128 rows whose ids are in sIds (-1 =
// padding row, staged as zeros) as big/small TF32 in the core-matrix layout,
// and adds this thread's share of |x|^2 to nrm[0..1].
// Thread map: lane = 8*q + t handles row 8*rg + t and dimensions 4*q.. of every
// 16-dimension step, so the 8 lanes with equal q write one 128-byte core matrix.
template <bool VEC4>
__device__ __forceinline__ void stage_chunk(const float* __restrict__ pts, int D, const int* sIds, int k0,
                                            unsigned char* sBig, unsigned char* sSmall, float* nrm, int warp,
                                            int lane)
{
    const int t = lane & 7, q = lane >> 3;
#pragma unroll
    for (int g2 = 0; g2 < 2; ++g2) {
        const int rg = warp + g2 * KNN_WARPS; // 16 groups of 8 rows
        const int id = sIds[rg * 8 + t];
        const float* src = pts + (size_t)(id < 0 ? 0 : id) * D;
#pragma unroll
        for (int kk = 0; kk < TC_KC; kk += 16) {
            const int k = k0 + kk + 4 * q;
            float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (id >= 0) {
                if (VEC4) {
                    if (k < D) x = __ldg(reinterpret_cast<const float4*>(src + k));
                } else {
                    if (k + 0 < D) x.x = __ldg(src + k + 0);
                    if (k + 1 < D) x.y = __ldg(src + k + 1);
                    if (k + 2 < D) x.z = __ldg(src + k + 2);
                    if (k + 3 < D) x.w = __ldg(src + k + 3);
                }
            }
            nrm[g2] = __fmaf_rn(x.x, x.x, nrm[g2]);
            nrm[g2] = __fmaf_rn(x.y, x.y, nrm[g2]);
            nrm[g2] = __fmaf_rn(x.z, x.z, nrm[g2]);
            nrm[g2] = __fmaf_rn(x.w, x.w, nrm[g2]);
            float4 b, s;
            b.x = __uint_as_float(__float_as_uint(x.x) & 0xffffe000u); s.x = x.x - b.x;
            b.y = __uint_as_float(__float_as_uint(x.y) & 0xffffe000u); s.y = x.y - b.y;
            b.z = __uint_as_float(__float_as_uint(x.z) & 0xffffe000u); s.z = x.z - b.z;
            b.w = __uint_as_float(__float_as_uint(x.w) & 0xffffe000u); s.w = x.w - b.w;
            s.x = __uint_as_float(__float_as_uint(s.x) & 0xffffe000u);
            s.y = __uint_as_float(__float_as_uint(s.y) & 0xffffe000u);
            s.z = __uint_as_float(__float_as_uint(s.z) & 0xffffe000u);
            s.w = __uint_as_float(__float_as_uint(s.w) & 0xffffe000u);
            const int off = rg * TC_SBO + ((kk >> 2) + q) * TC_LBO + t * 16;
            *reinterpret_cast<float4*>(sBig + off) = b;
            *reinterpret_cast<float4*>(sSmall + off) = s;
        }
    }
}

// |x|^2 of the 128 staged rows from the per-thread shares (lanes t, t+8, t+16,
// t+24 hold the four quarters of a row).
__device__ __forceinline__ void store_norms(const float* nrm, float* sNorm, int warp, int lane)
{
#pragma unroll
    for (int g2 = 0; g2 < 2; ++g2) {
        float v = nrm[g2];
        v += __shfl_xor_sync(RSFK_FULL, v, 8);
        v += __shfl_xor_sync(RSFK_FULL, v, 16);
        if ((lane >> 3) == 0) sNorm[(warp + g2 * KNN_WARPS) * 8 + (lane & 7)] = v;
    }
}

template <int KPL, bool VEC4>
__global__ void __launch_bounds__(KNN_THREADS)
k_bucket_knn_tc(const float* __restrict__ pts, int D, int K, const int* __restrict__ perm,
                const int* __restrict__ leaf_start, const int* __restrict__ leaf_count,
                int* __restrict__ knn_idx, float* __restrict__ knn_dist, int max_leaf,
                int* __restrict__ error_flag)
{
    extern __shared__ float4 smem4[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(smem4);
    const Layout L0 = layout_for(D, max_leaf);
    unsigned char* sBigA = smem;
    unsigned char* sSmallA = smem + TC_OPERAND_BYTES;
    unsigned char* sBigB = L0.two_operands ? smem + L0.off_b : sBigA;
    unsigned char* sSmallB = L0.two_operands ? smem + L0.off_b + TC_OPERAND_BYTES : sSmallA;
    float* sNormA = reinterpret_cast<float*>(smem + L0.off_norm);
    float* sNormB = sNormA + TC_ROWS;
    int* sIdsA = reinterpret_cast<int*>(smem + L0.off_ids);
    int* sIdsB = sIdsA + TC_ROWS;
    unsigned* sPass = reinterpret_cast<unsigned*>(smem + L0.off_pass);
    uint64_t* sBar = reinterpret_cast<uint64_t*>(smem + L0.off_misc);
    uint32_t* sTmem = reinterpret_cast<uint32_t*>(smem + L0.off_misc + 16);
    int* sFail = reinterpret_cast<int*>(smem + L0.off_misc + 32);
    const int PW = L0.pass_words;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* xp = reinterpret_cast<float*>(smem + L0.off_xp) + (size_t)warp * ((D + 3) & ~3);
    int* queue = reinterpret_cast<int*>(smem + L0.off_queue) + warp * EXP_QUEUE;

    const int leaf = blockIdx.x;
    const int m = leaf_count[leaf];
    const int* ids = perm + leaf_start[leaf];
    const int n_blocks = (m + TC_ROWS - 1) / TC_ROWS;

    // ---- set-up: barrier and tensor memory --------------------------------
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(sBar)), "r"(1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *sFail = 0;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(sTmem)),
                     "r"((uint32_t)TC_ROWS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *sTmem;
    const uint32_t bar = smem_u32(sBar);
    const uint32_t idesc = umma_idesc();
    const int n_chunks = (D + TC_KC - 1) / TC_KC;
    uint32_t phase = 0;
    bool failed = false;

    for (int bi = 0; bi < n_blocks && !failed; ++bi) {
        const int i0 = bi * TC_ROWS;
        __syncthreads(); // the previous block's row phase has finished with sIdsA / sPass
        for (int r = threadIdx.x; r < TC_ROWS; r += blockDim.x) sIdsA[r] = i0 + r < m ? ids[i0 + r] : -1;
        for (int w = threadIdx.x; w < TC_ROWS * PW; w += blockDim.x) sPass[w] = 0u;
        __syncthreads();
        // this thread's epilogue row: tensor-memory lane 32*(warp%4)+lane
        const int erow = 32 * (warp & 3) + lane;
        const int eid = sIdsA[erow];
        const int mI = min(TC_ROWS, m - i0);

        for (int bj = 0; bj < n_blocks && !failed; ++bj) {
            const int j0 = bj * TC_ROWS;
            const bool diag = (bj == bi);
            __syncthreads(); // the previous tile's row phase used the operand area for its row copies
            if (!diag) {
                for (int r = threadIdx.x; r < TC_ROWS; r += blockDim.x) sIdsB[r] = j0 + r < m ? ids[j0 + r] : -1;
                __syncthreads();
            }
            // ---- Gram tile (I, J) over K chunks ---------------------------
            float nrmA[2] = {0.0f, 0.0f}, nrmB[2] = {0.0f, 0.0f};
            for (int ch = 0; ch < n_chunks; ++ch) {
                stage_chunk<VEC4>(pts, D, sIdsA, ch * TC_KC, sBigA, sSmallA, nrmA, warp, lane);
                if (!diag) stage_chunk<VEC4>(pts, D, sIdsB, ch * TC_KC, sBigB, sSmallB, nrmB, warp, lane);
                // generic-proxy writes must be visible to the tensor core (async proxy)
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncthreads();
                if (threadIdx.x == 0) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t aB = smem_u32(sBigA), aS = smem_u32(sSmallA);
                    const uint32_t bB = diag ? aB : smem_u32(sBigB), bS = diag ? aS : smem_u32(sSmallB);
#pragma unroll
                    for (int pass = 0; pass < 3; ++pass) {
                        const uint32_t a = (pass == 2) ? aS : aB; // big.big, big.small, small.big
                        const uint32_t b = (pass == 1) ? bS : bB;
#pragma unroll
                        for (int s8 = 0; s8 < TC_KC / 8; ++s8)
                            umma_tf32(tmem_d, umma_desc(a + s8 * 2 * TC_LBO), umma_desc(b + s8 * 2 * TC_LBO), idesc,
                                      (ch > 0 || pass > 0 || s8 > 0) ? 1u : 0u);
                    }
                    umma_commit(bar);
                }
                // the operands may be overwritten only after the MMAs have read them
                if (!mbar_wait(bar, phase)) *sFail = 1;
                phase ^= 1u;
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncthreads();
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (*sFail) { failed = true; break; }
            }
            if (failed) break;
            store_norms(nrmA, sNormA, warp, lane);
            if (!diag) store_norms(nrmB, sNormB, warp, lane);
            __syncthreads();
            // ---- epilogue: pass bits of rows I against columns J ------------
            // warp w reads tensor-memory lanes 32*(w%4).. (rows) and columns 64*(w/4)..
            {
                // current K-th distance of the row (rows flushed after earlier tiles have tightened it)
                const float thr = eid >= 0 ? __ldcg(knn_dist + (size_t)eid * K + (K - 1)) : -1.0f;
                const float* nJ = diag ? sNormA : sNormB;
                const float n_row = sNormA[erow];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int c0 = 64 * (warp >> 2) + 32 * half;
                    float g[32];
                    tmem_ld32(tmem_d + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)c0, g);
                    unsigned word = 0;
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int j = c0 + c;
                        const float nn = n_row + nJ[j];
                        const float d2 = __fmaf_rn(-2.0f, g[c], nn) - TC_MARGIN * nn;
                        // !(d2 >= thr) keeps the candidate when anything is not a number
                        if (j0 + j < m && j0 + j != i0 + erow && !(d2 >= thr)) word |= 1u << c;
                    }
                    if (eid >= 0) sPass[erow * PW + bj * (TC_ROWS / 32) + (c0 >> 5)] = word;
                }
            }
            // the next tile's MMAs overwrite tensor memory and sIdsB: order after the loads
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

            // ---- rows of block I: exact distances of passing candidates ----
            // A row is flushed as soon as 32 candidates wait (its K-th distance then
            // tightens the filter of the following tiles) and after the last tile.
            const bool last_tile = (bj == n_blocks - 1);
            const int n_words = min((m + 31) >> 5, (bj + 1) * (TC_ROWS / 32));
            for (int r = warp; r < mI; r += KNN_WARPS) {
                int pending = 0;
                for (int w = lane; w < n_words; w += 32) pending += __popc(sPass[r * PW + w]);
#pragma unroll
                for (int sft = 16; sft >= 1; sft >>= 1) pending += __shfl_xor_sync(RSFK_FULL, pending, sft);
                if (pending == 0 || (pending < 32 && !last_tile)) continue;
                const int self = sIdsA[r];
                __syncwarp();
                for (int k = lane; k < D; k += 32) xp[k] = __ldg(pts + (size_t)self * D + k);
                WarpList<KPL> L;
                L.load(knn_idx + (size_t)self * K, knn_dist + (size_t)self * K, K, lane);
                __syncwarp();
                bool changed = false;
                int qn = 0;
                for (int w = 0; w < n_words; ++w) {
                    const unsigned bits = sPass[r * PW + w];
                    if (bits == 0) continue;
                    __syncwarp();
                    if (lane == 0) sPass[r * PW + w] = 0u;
                    const bool ok = (bits >> lane) & 1u;
                    if (ok) queue[qn + __popc(bits & ((1u << lane) - 1u))] = ids[32 * w + lane];
                    qn += __popc(bits);
                    __syncwarp();
                    if (qn >= 32) {
                        explore_flush<KPL, VEC4>(L, pts, D, xp, queue, 32, K, lane, changed);
                        __syncwarp();
                        const int rest = qn - 32;
                        const int tmp = lane < rest ? queue[32 + lane] : -1;
                        __syncwarp();
                        if (lane < rest) queue[lane] = tmp;
                        qn = rest;
                        __syncwarp();
                    }
                }
                if (qn > 0) explore_flush<KPL, VEC4>(L, pts, D, xp, queue, qn, K, lane, changed);
                if (changed) L.store(knn_idx + (size_t)self * K, knn_dist + (size_t)self * K, K, lane);
            }
        }
        if (failed) break;
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)TC_ROWS)
                     : "memory");
    }
    if (failed && threadIdx.x == 0) atomicExch(error_flag, 1);
}

} // namespace tc
