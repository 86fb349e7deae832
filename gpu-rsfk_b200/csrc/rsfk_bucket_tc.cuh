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
// One CTA per leaf of at most 128 points.  Operands are staged by the threads
// themselves (rows are gathered through the permutation, so no 2-D TMA tile
// exists): a K-chunk of 64 dimensions of all rows is split into big/small TF32
// and stored in the K-major, no-swizzle core-matrix layout the UMMA shared
// memory descriptor addresses (8 rows x 16 bytes per core matrix).
#pragma once

namespace tc {

constexpr int TC_ROWS = 128;            // MMA M and N: rows of one leaf block
constexpr int TC_KC = 64;               // dimensions staged per chunk
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

// Shared-memory layout of one CTA (bytes), after the two operand arrays.
struct Layout {
    int off_norm, off_ids, off_pass, off_xp, off_queue, off_misc, total;
};
__host__ __device__ inline Layout layout_for(int D)
{
    Layout l;
    int o = 2 * TC_OPERAND_BYTES;
    l.off_norm = o;  o += TC_ROWS * 4;
    l.off_ids = o;   o += TC_ROWS * 4;
    l.off_pass = o;  o += TC_ROWS * (TC_ROWS / 32) * 4;
    l.off_xp = o;    o += KNN_WARPS * ((D + 3) & ~3) * 4;
    l.off_queue = o; o += KNN_WARPS * EXP_QUEUE * 4;
    l.off_misc = o;  o += 64;
    l.total = o;
    return l;
}

template <int KPL, bool VEC4>
__global__ void __launch_bounds__(KNN_THREADS)
k_bucket_knn_tc(const float* __restrict__ pts, int D, int K, const int* __restrict__ perm,
                const int* __restrict__ leaf_start, const int* __restrict__ leaf_count,
                int* __restrict__ knn_idx, float* __restrict__ knn_dist, int* __restrict__ error_flag)
{
    extern __shared__ float4 smem4[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(smem4);
    const Layout L0 = layout_for(D);
    unsigned char* sBig = smem;
    unsigned char* sSmall = smem + TC_OPERAND_BYTES;
    float* sNorm = reinterpret_cast<float*>(smem + L0.off_norm);
    int* sIds = reinterpret_cast<int*>(smem + L0.off_ids);
    unsigned* sPass = reinterpret_cast<unsigned*>(smem + L0.off_pass);
    uint64_t* sBar = reinterpret_cast<uint64_t*>(smem + L0.off_misc);
    uint32_t* sTmem = reinterpret_cast<uint32_t*>(smem + L0.off_misc + 16);
    int* sFail = reinterpret_cast<int*>(smem + L0.off_misc + 32);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* xp = reinterpret_cast<float*>(smem + L0.off_xp) + (size_t)warp * ((D + 3) & ~3);
    int* queue = reinterpret_cast<int*>(smem + L0.off_queue) + warp * EXP_QUEUE;

    const int leaf = blockIdx.x;
    const int m = leaf_count[leaf];
    const int* ids = perm + leaf_start[leaf];

    // ---- set-up: barrier, tensor memory, ids ------------------------------
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
    for (int r = threadIdx.x; r < TC_ROWS; r += blockDim.x) sIds[r] = r < m ? ids[r] : -1;
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *sTmem;
    const uint32_t bar = smem_u32(sBar);
    const uint32_t idesc = umma_idesc();

    // ---- Gram tile: K chunks of 64 dimensions -----------------------------
    // staging map: lane = 8*q + t handles row 8*rg + t and the four dimensions
    // 4*q.. of every 16-dimension step (8 lanes with equal q write 128
    // contiguous bytes: one core matrix)
    const int t = lane & 7, q = lane >> 3;
    float nrm[2] = {0.0f, 0.0f}; // this thread's part of |x|^2 for its two row groups
    uint32_t phase = 0;
    bool alive = true;
    const int n_chunks = (D + TC_KC - 1) / TC_KC;
    for (int ch = 0; ch < n_chunks; ++ch) {
        const int k0 = ch * TC_KC;
#pragma unroll
        for (int g2 = 0; g2 < 2; ++g2) {
            const int rg = warp + g2 * KNN_WARPS; // 16 groups of 8 rows
            const int row = rg * 8 + t;
            const int id = sIds[row];
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
        // generic-proxy writes must be visible to the tensor core (async proxy)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (threadIdx.x == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t aB = smem_u32(sBig), aS = smem_u32(sSmall);
#pragma unroll
            for (int pass = 0; pass < 3; ++pass) {
                const uint32_t a = (pass == 2) ? aS : aB; // big.big, big.small, small.big
                const uint32_t b = (pass == 1) ? aS : aB;
#pragma unroll
                for (int s8 = 0; s8 < TC_KC / 8; ++s8)
                    umma_tf32(tmem_d, umma_desc(a + s8 * 2 * TC_LBO), umma_desc(b + s8 * 2 * TC_LBO), idesc,
                              (ch > 0 || pass > 0 || s8 > 0) ? 1u : 0u);
            }
            umma_commit(bar);
        }
        // everyone waits: the operands may be overwritten only after the MMAs read them
        if (alive && !mbar_wait(bar, phase)) alive = false;
        phase ^= 1u;
        if (!alive) *sFail = 1;
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (*sFail) break;
    }
    const bool failed = *sFail != 0;

    // ---- norms ------------------------------------------------------------
#pragma unroll
    for (int g2 = 0; g2 < 2; ++g2) {
        float v = nrm[g2];
        v += __shfl_xor_sync(RSFK_FULL, v, 8);
        v += __shfl_xor_sync(RSFK_FULL, v, 16);
        if (q == 0) sNorm[(warp + g2 * KNN_WARPS) * 8 + t] = v;
    }
    __syncthreads();

    // ---- epilogue: pass bits ------------------------------------------------
    // warp w reads tensor-memory lanes 32*(w%4).. (rows) and columns 64*(w/4)..
    if (!failed) {
        const int row = 32 * (warp & 3) + lane;
        const int id_row = sIds[row];
        float thr = -1.0f;
        if (id_row >= 0) thr = knn_dist[(size_t)id_row * K + (K - 1)];
        const float n_row = sNorm[row];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int c0 = 64 * (warp >> 2) + 32 * half;
            float g[32];
            tmem_ld32(tmem_d + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)c0, g);
            unsigned word = 0;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const int j = c0 + c;
                const float nn = n_row + sNorm[j];
                const float d2 = __fmaf_rn(-2.0f, g[c], nn) - TC_MARGIN * nn;
                // !(d2 >= thr) keeps candidates when anything is not a number
                if (j < m && j != row && !(d2 >= thr)) word |= 1u << c;
            }
            if (id_row >= 0) sPass[row * (TC_ROWS / 32) + (c0 >> 5)] = word;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)TC_ROWS)
                     : "memory");
    }
    if (failed) {
        if (threadIdx.x == 0) atomicExch(error_flag, 1);
        return;
    }

    // ---- rows: exact distances of the passing candidates, list update -----
    for (int r = warp; r < m; r += KNN_WARPS) {
        const int self = sIds[r];
        const unsigned any = sPass[r * 4 + 0] | sPass[r * 4 + 1] | sPass[r * 4 + 2] | sPass[r * 4 + 3];
        if (any == 0) continue;
        __syncwarp();
        for (int k = lane; k < D; k += 32) xp[k] = __ldg(pts + (size_t)self * D + k);
        WarpList<KPL> L;
        L.load(knn_idx + (size_t)self * K, knn_dist + (size_t)self * K, K, lane);
        __syncwarp();
        bool changed = false;
        int qn = 0;
        for (int w = 0; w < TC_ROWS / 32; ++w) {
            const unsigned bits = sPass[r * (TC_ROWS / 32) + w];
            if (bits == 0) continue;
            const bool ok = (bits >> lane) & 1u;
            if (ok) queue[qn + __popc(bits & ((1u << lane) - 1u))] = sIds[32 * w + lane];
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

} // namespace tc
