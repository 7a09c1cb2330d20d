// Distance GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), operands
// staged by TMA, with the top-k selection fused into the epilogue so that the
// nq x nb score matrix is never written to HBM.
//
// Replaces the reference's simdgroup_gemm_* kernels (shaders/simdgroup_gemm.metal:26-481,
// shaders/simdgroup_gemm_bf16.metal:23-242, shaders/simdgroup_gemm_family9.metal:27-470),
// their host dispatch (src/MetalDistance.mm:225-323) and, through the fused
// epilogue, fused_l2_topk_* (shaders/fused_l2_topk.metal:19-444).
//
// Two shapes of one kernel (352 threads, one CTA per SM, persistent over work items):
//  * single CTA (up to 128 queries): tile 128 x 256, cta_group::1, two TMEM accumulators;
//  * CTA pair (more queries): a cluster of two CTAs computes a 256 x 512 tile with
//    cta_group::2 MMAs (M = 256); each CTA stages its own 128 query rows and half of the X
//    rows of every k-block, and holds two 256-column accumulators (all 512 TMEM columns).
// Roles of the warps:
//   warp 0      TMA producer: Q tile (128 x 64) and X tile per k-block, 128-byte swizzle,
//               4-stage mbarrier ring
//   warps 1,10  MMA issuers: tcgen05.mma kind::f16, N = 256, K = 16, fp32 accumulators in
//               TMEM.  A chain of MMAs on one accumulator runs at about half the tensor rate,
//               so the pair shape runs two chains (columns 0-255 and 256-511 of the tile),
//               one issuing thread each.
//   warps 2-9   epilogue: tcgen05.ld (thread t owns query row t of the tile, two warps per
//               TMEM lane quarter, half of the tile's columns each), one max per column (the
//               L2 bias -||x||^2/2 is part of the dot product: 8 extra K columns, see
//               rows.cu), filter against the row's bound, hits staged in shared memory and
//               worked off after the accumulator has been released.
// Epilogue modes:
//   top-k   a sorted list of up to 32 entries per (row, column range, column half) in the
//           thread's registers; every item yields partial lists, merged afterwards
//   filter  a fixed per-row threshold; every column under it is appended to the row's
//           candidate buffer in global memory
//   store   the keys are written out as a matrix (k beyond the list paths, pairwise distances)
// The mode is a template parameter (six instantiations with the two shapes): the filter and
// store kernels carry no list registers, which lets the filter kernel read 64 accumulator
// columns per TMEM load.  A work item is (query block, column range).
//
// FP32 storage: both operands are split into three bf16 planes
// (x = x0 + x1 + x2 exactly to 24 bits) and six plane products
// (0,0) (0,1) (1,0) (0,2) (2,0) (1,1) are accumulated in the same fp32 TMEM
// accumulator; the dropped products are below 2^-24 relative.
//
// Every wait on an mbarrier is bounded: after ~1 s of clock the waiting thread
// records kDevErrBarrierWait in the status word, raises the CTA abort flag and
// all roles drain out, TMEM is released and the kernel returns.
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace b200f {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;  // 16-bit elements: 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int KMAX = B200F_FUSED_MAX_K;
constexpr int NUM_EPI_WARPS = 8;   // two per TMEM lane quarter: each takes half of the tile's columns
constexpr int MMA2_WARP = 2 + NUM_EPI_WARPS;   // second MMA issuer (pair shape): one thread per accumulator chain
constexpr int NUM_THREADS = 32 * (3 + NUM_EPI_WARPS);
constexpr int TMEM_COLS = 512;

// Two shapes of the same kernel:
//  PAIR = false  one CTA per tile: M = 128 queries, N = 256 rows of X, cta_group::1
//  PAIR = true   two CTAs of a cluster share a 256 x 256 tile (cta_group::2): each CTA stages
//                its own 128 query rows and HALF of the X rows of every k-block, so the
//                shared-memory fill per FLOP is halved; the MMA is issued by the even CTA.
template <bool PAIR>
struct Cfg {
    static constexpr int STAGES = 4;
    static constexpr int B_ROWS = PAIR ? 128 : 256;        // rows of X this CTA stages per sub-tile
    // A dependent chain of MMAs on ONE accumulator runs at about half the tensor rate (each
    // MMA waits out the read-modify-write turnaround of the one before it); two chains on two
    // accumulators, one issuing thread each, come close to the full rate.  The pair shape
    // therefore computes two 256-column sub-tiles at once (same query k-block, two X k-blocks,
    // both TMEM halves); the price is that a chain's epilogue no longer overlaps its next MMAs.
    // Each chain has its own accumulator-full / accumulator-free barriers and its own four
    // epilogue warps per CTA, so one chain's MMAs do run beside the other chain's epilogue.
    static constexpr int NSUB = PAIR ? 2 : 1;              // 256-column sub-tiles per tile
    static constexpr int TILE_N = NSUB * BN;               // columns of X per tile: 512 / 256
    static constexpr int ACC_BUFS = PAIR ? 1 : 2;          // TMEM accumulator buffers of TILE_N columns
    static constexpr int B_SUB_BYTES = B_ROWS * BK * 2;    // 16 / 32 KiB
    static constexpr int B_STAGE_BYTES = NSUB * B_SUB_BYTES;  // 32 KiB either way
    static constexpr int QB = PAIR ? 256 : 128;            // query rows per work item
    // shared memory map (bytes from the 1024-aligned dynamic base)
    static constexpr int SM_A = 0;
    static constexpr int SM_B = SM_A + STAGES * A_STAGE_BYTES;
    static constexpr int SM_LKEY = SM_B + STAGES * B_STAGE_BYTES;
    // store mode transposes 32 x 32 blocks per epilogue warp here (32 x 33 floats each)
    static constexpr int SM_BAR = SM_LKEY + ((NUM_EPI_WARPS * 32 * 33 * 4 + 127) / 128) * 128;
    // barriers: full[STAGES] empty[STAGES] tfull[2] tempty[2]
    static constexpr int SM_TMEMPTR = SM_BAR + (2 * STAGES + 4) * 8;
    static constexpr int SM_ABORT = SM_TMEMPTR + 4;
    static constexpr int SMEM_BYTES = SM_ABORT + 4 + 8;
};

enum { MODE_TOPK = 0, MODE_STORE = 1, MODE_FILTER = 2 };

struct GemmParams {
    int64_t nq;
    int64_t col0;        // first global column (row of X) of this launch
    int64_t ncols_end;   // one past the last valid global column of this launch
    int64_t ntiles;      // column tiles in this launch
    int64_t tiles_per_range;
    int nqb;
    int P;
    int kb_per_pass;     // k-blocks of 64 per plane product
    int k_extent;        // valid K elements per plane product (multiple of 8)
    int npass;
    uint32_t pass_a;     // 4 bits per pass: plane index of A
    uint32_t pass_b;
    uint32_t idesc;
    int mode;
    int k;
    float kscale;        // key = -kscale * t  (2 for L2, 1 for inner product)
    // optional per-row factor on kscale (operands scaled per query row: fp16x2 planes); row j of
    // this launch is row rowscale_map[j] of the array when the map is set (redone rows)
    const float* rowscale;
    const int32_t* rowscale_map;
    float sign;
    const float* rowadd; // per query row, may be null (0)
    float* part_key;
    int32_t* part_idx;
    uint32_t* gthr;      // [nq][gslots] ordered-float 32nd-best keys published by the lists of a row
    int gslots;          // lists publish to slot (list number % gslots); the row's bound is the
                         // largest slot: gslots full lists hold 32 * gslots distinct candidates
    const int* nq_dev;   // when set: the number of live query rows is read from device memory
    int64_t tile_stride; // tile t of the launch is tile t * tile_stride of X (sampling passes)
    // MODE_FILTER: every column whose key is <= the row's threshold is appended to the row's
    // candidate buffer (position from an atomic counter; entries past cand_cap are only counted)
    const float* fthr;   // threshold of row q in scaled key units: fthr[q * fthr_stride + fthr_pos]
    int fthr_stride, fthr_pos;
    float* cand_key;     // [nq][cand_cap]
    int32_t* cand_idx;
    int32_t* cand_cnt;   // [nq]
    int cand_cap;
    int wide;            // MODE_FILTER: 64 columns per TMEM load (few hits expected), else 32
    float* out;
    int64_t ld;
    int32_t* status;
};

// ---- PTX wrappers (mbarrier and bounded-wait helpers come from ptx.cuh) -----------------

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int32_t* status) {
    return mbar_wait_bounded(bar, parity, abort_flag, status, kDevErrBarrierWait);
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2) {
    asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
            : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// arrive on an mbarrier given by a shared::cluster address (own or peer CTA)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMA load issued inside a CTA pair: the mbarrier may live in the peer CTA
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 int c0, int c1, int c2) {
    asm volatile(
            "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
            : "memory");
}

__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
                 : "memory");
}

__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b,
                                                uint32_t idesc, uint32_t accumulate) {
    asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(d_tmem),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
}

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(d_tmem),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
}

// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
              "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
              "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
              "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
              "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
              "=r"(r[31])
            : "r"(taddr)
            : "memory");
}
// 32 lanes x 64 consecutive fp32 columns -> 64 registers per thread
__device__ __forceinline__ void tc_ld64(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
            "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
            "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
              "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
              "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
              "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
              "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
              "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]),
              "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]),
              "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),
              "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]),
              "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]),
              "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
            : "r"(taddr)
            : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major operand tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t desc = 0;
    desc |= (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address
    desc |= (uint64_t)1 << 16;                    // leading byte offset (unused with swizzle)
    desc |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset between 8-row groups
    desc |= (uint64_t)1 << 46;                    // descriptor version (sm_100)
    desc |= (uint64_t)2 << 61;                    // SWIZZLE_128B
    return desc;
}

// Per-row candidate list held in REGISTERS by the thread that owns the row: 32 (key, id)
// pairs sorted ascending by key, every index static so nothing spills.  Inserting s drops
// the largest element: slot j takes the old slot j-1 if that is greater than s, keeps its
// value if it is <= s, and takes s otherwise.  Elements equal to s stay in front of it
// (ids arrive ascending).  For k < 32 the first 32-k slots hold -INF sentinels, so the
// k-th best key is always slot 31.
__device__ __forceinline__ void reglist_insert(float (&lk)[KMAX], int32_t (&li)[KMAX], float s,
                                               int32_t id) {
    float pk = -CUDART_INF_F;
    int32_t pi = -1;
#pragma unroll
    for (int j = 0; j < KMAX; j++) {
        const float cur = lk[j];
        const int32_t ci = li[j];
        const bool shift = pk > s;
        const bool keep = cur <= s;
        lk[j] = shift ? pk : (keep ? cur : s);
        li[j] = shift ? pi : (keep ? ci : id);
        pk = cur;
        pi = ci;
    }
}

// Hits of the tile in flight are staged per thread in shared memory (entry i of a thread at
// [i * STAGE_LD]: raw key s = -t and column) and worked off AFTER the accumulator has been handed
// back to the MMA issuers, so that list insertion and buffer appends run beside the next
// tile's MMAs instead of in front of them.  Only a thread whose stage fills up inside one
// tile (list warm-up, massive ties) drains it on the spot.
constexpr int STAGE_N = 16;
constexpr int STAGE_LD = 32 * NUM_EPI_WARPS;

__device__ __forceinline__ void drain_to_list(float (&lk)[KMAX], int32_t (&li)[KMAX], const float* sk,
                                              const int32_t* si, int n, float& thr, float& thr_eff) {
    for (int i = 0; i < n; i++) {
        const float sc = sk[i * STAGE_LD];
        if (sc < thr_eff) {  // the list may have tightened since the entry was staged
            reglist_insert(lk, li, sc, si[i * STAGE_LD]);
            thr = lk[KMAX - 1];
            thr_eff = fminf(thr_eff, thr);
        }
    }
}

// MODE_FILTER: one atomic takes n slots of the row's candidate buffer; the counter also counts
// entries that no longer fit.
__device__ __forceinline__ void drain_to_buffer(int32_t* cnt, float* ck, int32_t* ci, int cap,
                                                float kscale, const float* sk, const int32_t* si, int n) {
    if (n <= 0) return;
    const int base = atomicAdd(cnt, n);
    for (int i = 0; i < n; i++) {
        if (base + i < cap) {
            ck[base + i] = kscale * sk[i * STAGE_LD];
            ci[base + i] = si[i * STAGE_LD];
        }
    }
}

// MODE is a template parameter: the filter and store instantiations carry no list registers.
template <bool PAIR, int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_topk_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
    using C = Cfg<PAIR>;
    constexpr int STAGES = C::STAGES;
    constexpr int B_STAGE_BYTES = C::B_STAGE_BYTES;
    constexpr int TILE_N = C::TILE_N;
    constexpr int SM_A = C::SM_A, SM_B = C::SM_B, SM_LKEY = C::SM_LKEY;
    constexpr int SM_BAR = C::SM_BAR, SM_TMEMPTR = C::SM_TMEMPTR, SM_ABORT = C::SM_ABORT;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;   // 0 = MMA issuer of the pair
    const int64_t unit = PAIR ? (blockIdx.x >> 1) : blockIdx.x;  // work is dealt to CTAs / CTA pairs
    const int64_t nunits = PAIR ? (gridDim.x >> 1) : gridDim.x;

    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(smem + SM_TMEMPTR);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM_ABORT);

    const uint32_t bar_full = sbase + SM_BAR;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_tfull = bar_empty + STAGES * 8;
    const uint32_t bar_tempty = bar_tfull + 2 * 8;

    // A launch that redoes rows counted on the device usually finds none: leave before any
    // barrier or TMEM allocation (the value is the same for every thread of every CTA).
    if (p.nq_dev && *p.nq_dev <= 0) return;

    if ((sbase & 1023u) != 0) {  // swizzled tiles need a 1024-byte aligned base (same in both CTAs)
        if (threadIdx.x == 0 && p.status) atomicOr(p.status, kDevErrSmemAlign);
        return;
    }

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, PAIR ? 2 : 1);   // one commit per issuing thread
        }
        for (int s = 0; s < 2; s++) {
            // single CTA: barrier s = accumulator buffer s, all epilogue warps;
            // pair: barrier s = chain s, the warps of that column half in both CTAs
            mbar_init(bar_tfull + s * 8, 1);
            mbar_init(bar_tempty + s * 8, NUM_EPI_WARPS);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                                 sbase + SM_TMEMPTR),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                                 sbase + SM_TMEMPTR),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    // live query rows: known to the host, or left in device memory by an earlier kernel
    const int64_t nq_live = p.nq_dev ? min((int64_t)*p.nq_dev, p.nq) : p.nq;
    const int nqb = p.nq_dev ? (int)((nq_live + C::QB - 1) / C::QB) : p.nqb;
    const int64_t nitems = (int64_t)nqb * p.P;
    const int kb_total = p.kb_per_pass * p.npass;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t item = unit; item < nitems && ok; item += nunits) {
                const int qb = (int)(item % nqb);
                const int64_t xr = item / nqb;
                const int64_t t0 = xr * p.tiles_per_range;
                const int64_t t1 = min(t0 + p.tiles_per_range, p.ntiles);
                for (int64_t t = t0; t < t1 && ok; t++) {
                    const int xrow = (int)(p.col0 + t * p.tile_stride * TILE_N);
                    for (int kb = 0; kb < kb_total; kb++) {
                        if (!mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, p.status)) {
                            ok = false;
                            break;
                        }
                        const int pass = kb / p.kb_per_pass;
                        const int kk = (kb - pass * p.kb_per_pass) * BK;
                        const int pa = (p.pass_a >> (4 * pass)) & 15;
                        const int pb = (p.pass_b >> (4 * pass)) & 15;
                        if (PAIR) {
                            // both CTAs' copies complete on the issuer's barrier
                            const uint32_t fb = map_to_cta(bar_full + stage * 8, 0);
                            if (cta_rank == 0)
                                mbar_arrive_expect_tx(bar_full + stage * 8,
                                                      2 * (A_STAGE_BYTES + B_STAGE_BYTES));
                            tma_load_3d_pair(sbase + SM_A + stage * A_STAGE_BYTES, &tmap_a, fb, kk,
                                             qb * C::QB + (int)cta_rank * BM, pa);
#pragma unroll
                            for (int sub = 0; sub < C::NSUB; sub++)
                                tma_load_3d_pair(sbase + SM_B + stage * B_STAGE_BYTES + sub * C::B_SUB_BYTES,
                                                 &tmap_b, fb, kk, xrow + sub * BN + (int)cta_rank * C::B_ROWS, pb);
                        } else {
                            mbar_arrive_expect_tx(bar_full + stage * 8, A_STAGE_BYTES + B_STAGE_BYTES);
                            tma_load_3d(sbase + SM_A + stage * A_STAGE_BYTES, &tmap_a,
                                        bar_full + stage * 8, kk, qb * BM, pa);
                            tma_load_3d(sbase + SM_B + stage * B_STAGE_BYTES, &tmap_b,
                                        bar_full + stage * 8, kk, xrow, pb);
                        }
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                }
            }
            // Let every copy this thread issued land before the CTA's shared memory goes
            // away: wait (bounded) until the consumer released, or the data arrived in,
            // each stage that is still in flight.
            if (!ok) {
                long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) {
                }
            }
        }
    } else if (warp == 1 || warp == MMA2_WARP) {
        // ------------------------------ MMA issuer --------------------------------
        // The tensor pipe idles whenever this thread is not issuing, so the loop carries
        // nothing but the barrier wait, four MMAs and the commit(s) per k-block:
        // descriptors, barrier addresses and the shape of the last k-block are set up once.
        // One thread sustains about one MMA per 190 cycles, and a chain of MMAs on one
        // accumulator about one per 290; in the pair shape the two accumulator chains of a tile
        // are therefore issued by two threads (warp 1: columns 0-255, warp MMA2_WARP: 256-511).
        const int chain = (warp == 1) ? 0 : 1;
        if (lane == 0 && cta_rank == 0 && (chain == 0 || PAIR)) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            const uint64_t da0 = make_smem_desc(sbase + SM_A);
            const uint64_t db0 = make_smem_desc(sbase + SM_B);
            const uint32_t empty0 = PAIR ? map_to_cta(bar_empty, 0) : bar_empty;
            const uint32_t empty1 = PAIR ? map_to_cta(bar_empty, 1) : 0;
            const uint32_t tfull0 = PAIR ? map_to_cta(bar_tfull, 0) : bar_tfull;
            const uint32_t tfull1 = PAIR ? map_to_cta(bar_tfull, 1) : 0;
            // the last k-block of a plane product may hold fewer than 64 valid K elements
            // (TMA zero-fills the rest): skip the all-zero sub-steps
            const int klast_valid = p.k_extent - (p.kb_per_pass - 1) * BK;
            const int nk4_last = klast_valid >= BK ? BK / UMMA_K : (klast_valid + UMMA_K - 1) / UMMA_K;
            for (int64_t item = unit; item < nitems && ok; item += nunits) {
                const int64_t xr = item / nqb;
                const int64_t t0 = xr * p.tiles_per_range;
                const int64_t t1 = min(t0 + p.tiles_per_range, p.ntiles);
                for (int64_t t = t0; t < t1 && ok; t++) {
                    const int bi = PAIR ? chain : acc;  // barrier pair of this chain / buffer
                    if (!mbar_wait(bar_tempty + bi * 8, acc_phase ^ 1, abort_flag, p.status)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + acc * TILE_N;
                    int kin = 0;
                    uint32_t accumulate = 0;
                    for (int kb = 0; kb < kb_total; kb++) {
                        if (!mbar_try_wait(bar_full + stage * 8, phase) &&
                            !mbar_wait(bar_full + stage * 8, phase, abort_flag, p.status)) {
                            ok = false;
                            break;
                        }
                        const uint64_t da = da0 + (uint64_t)(stage * (A_STAGE_BYTES >> 4));
                        const uint64_t db = db0 + (uint64_t)(stage * (B_STAGE_BYTES >> 4));
                        const bool last = ++kin == p.kb_per_pass;
                        if (last) kin = 0;
                        const int nk4 = last ? nk4_last : BK / UMMA_K;
#pragma unroll
                        for (int k4 = 0; k4 < BK / UMMA_K; k4++) {
                            // advance 32 bytes (16 elements) along K inside the swizzle row
                            if (k4 < nk4) {
                                if (PAIR) {
                                    tc_mma_f16_pair(d_tmem + chain * BN, da + (uint64_t)(k4 * 2),
                                                    db + (uint64_t)(chain * (C::B_SUB_BYTES >> 4) + k4 * 2),
                                                    p.idesc, accumulate);
                                } else {
                                    tc_mma_f16(d_tmem, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2),
                                               p.idesc, accumulate);
                                }
                                accumulate = 1;
                            }
                        }
                        // frees the stage (in both CTAs of a pair) when the MMAs retire
                        if (PAIR) {
                            tc_commit_pair(empty0 + stage * 8);
                            tc_commit_pair(empty1 + stage * 8);
                        } else {
                            tc_commit(empty0 + stage * 8);
                        }
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                    if (!ok) break;
                    if (PAIR) {  // this chain's accumulator complete, in both CTAs
                        tc_commit_pair(tfull0 + chain * 8);
                        tc_commit_pair(tfull1 + chain * 8);
                    } else {
                        tc_commit(tfull0 + acc * 8);
                    }
                    if (C::ACC_BUFS == 2) {
                        acc ^= 1;
                        if (acc == 0) acc_phase ^= 1;
                    } else {
                        acc_phase ^= 1;
                    }
                }
            }
        }
    } else if (warp >= 2 && warp < 2 + NUM_EPI_WARPS) {
        // ------------------------------ epilogue -----------------------------------
        const int ew = warp & 3;              // TMEM lane quarter this warp may read
        const int eh = (warp - 2) >> 2;       // which half of the tile's columns this warp scans
        constexpr int CH_PER_HALF = TILE_N / 64;
        const int row = ew * 32 + lane;       // row of the tile owned by this thread
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const int k = p.k;
        float lk[KMAX];     // this thread's row list (see reglist_insert)
        int32_t li[KMAX];
        // this thread's stage (see drain_to_list); the area serves the transposes in store mode
        float* const stage_key = reinterpret_cast<float*>(smem + SM_LKEY) + (threadIdx.x - 64);
        int32_t* const stage_idx =
                reinterpret_cast<int32_t*>(smem + SM_LKEY) + STAGE_N * STAGE_LD + (threadIdx.x - 64);
        int nstaged = 0;
        for (int64_t item = unit; item < nitems && ok; item += nunits) {
            const int qb = (int)(item % nqb);
            const int64_t xr = item / nqb;
            const int64_t t0 = xr * p.tiles_per_range;
            const int64_t t1 = min(t0 + p.tiles_per_range, p.ntiles);
            const int64_t grow = (int64_t)qb * C::QB + (int64_t)cta_rank * BM + row;
            const bool row_live = grow < nq_live;
            // slot of the row's bound array this list publishes to
            uint32_t* const gslot = p.gthr ? p.gthr + grow * p.gslots + (int)((2 * xr + eh) % p.gslots) : nullptr;
            float ksc = p.kscale;          // this row's key scale
            if (p.rowscale && row_live) ksc *= __ldg(p.rowscale + (p.rowscale_map ? (int64_t)__ldg(p.rowscale_map + grow) : grow));
            float thr = CUDART_INF_F;      // worst key of this thread's list (k-th best of the range)
            float thr_eff = CUDART_INF_F;  // filter: min(thr, bound shared by all ranges of the row)
            float thr_pub = CUDART_INF_F;  // last value published to gthr
            float radd = 0.f;
            if (MODE == MODE_TOPK) {
#pragma unroll
                for (int j = 0; j < KMAX; j++) {
                    lk[j] = (j >= KMAX - k) ? CUDART_INF_F : -CUDART_INF_F;
                    li[j] = -1;
                }
            } else if (MODE == MODE_FILTER) {
                // keys <= threshold pass: the filter below is exclusive, so take the next float up
                // (+INF, the threshold of a row whose sample was too small, stays; -INF passes nothing)
                thr_eff = -CUDART_INF_F;
                if (row_live) {
                    const float t = p.fthr[grow * p.fthr_stride + p.fthr_pos] / ksc;
                    const uint32_t o = float_to_ordered(t);
                    thr_eff = (o >= 0xff800000u) ? t : ordered_to_float(o + 1u);
                }
            } else if (row_live && p.rowadd) {
                radd = p.rowadd[grow];
            }
            for (int64_t t = t0; t < t1 && ok; t++) {
                const int64_t c_tile = p.col0 + t * p.tile_stride * TILE_N;
                {
                    const bool w = mbar_wait(bar_tfull + (PAIR ? eh : acc) * 8, acc_phase, abort_flag, p.status);
                    if (!__all_sync(0xffffffffu, w)) {  // keep the warp converged for tcgen05.ld
                        ok = false;
                        break;
                    }
                }
                tc_fence_after();
                if (MODE == MODE_TOPK && row_live) {
                    // A full list's worst key bounds the row's 32nd best from above; the largest
                    // of gslots such keys (distinct lists) bounds the (32 * gslots)-th best, which
                    // is at or beyond the k-th.  Publish ours, adopt the bound.  A key equal to
                    // the bound may still win a tie on the id, so the filter admits s <= bound.
                    if (thr < thr_pub) {
                        atomicMin(gslot, float_to_ordered(thr));
                        thr_pub = thr;
                    }
                    uint32_t g = 0;
                    for (int sidx = 0; sidx < p.gslots; sidx++)
                        g = max(g, __ldcg(p.gthr + grow * p.gslots + sidx));
                    const float gnext = (g >= 0xff800000u) ? CUDART_INF_F : ordered_to_float(g + 1u);
                    thr_eff = fminf(thr, gnext);
                }
                // The accumulator holds t = q.x (- ||x||^2/2 for L2): larger is better; the
                // lists keep s = -t (smaller is better).  Rows of X beyond the last valid
                // column are zero-filled by TMA (t = 0) and must be masked out.
                const bool partial = c_tile + TILE_N > p.ncols_end;
                const uint32_t taddr = tmem_base + ((uint32_t)(ew * 32) << 16) + acc * TILE_N;
                if constexpr (MODE != MODE_STORE) {
                // CW columns per TMEM load.  64 saves ~3 % of the tile time when hits are rare
                // (filter mode has the registers for it: no lists to keep); with a hit in most
                // chunks the 64-column masks cost more than the wider load saves.
                auto scan = [&](auto cw_tag) {
                constexpr int CW = decltype(cw_tag)::value;
#pragma unroll 1
                for (int ch = 0; ch < CH_PER_HALF * 32 / CW; ch++) {
                    uint32_t r[CW];
                    const int col = eh * CH_PER_HALF * 32 + ch * CW;  // first column inside the tile
                    if constexpr (CW == 64) tc_ld64(taddr + col, r);
                    else tc_ld32(taddr + col, r);
                    tc_wait_ld();
                    const int64_t cbase = c_tile + col;
                    {
                        if (partial) {
#pragma unroll
                            for (int c = 0; c < CW; c++)
                                if (cbase + c >= p.ncols_end) r[c] = 0xff800000u;  // -INF
                        }
                        // one max per column (tree), one compare per CW columns
                        float m[CW / 2];
#pragma unroll
                        for (int c = 0; c < CW / 2; c++)
                            m[c] = fmaxf(__uint_as_float(r[c]), __uint_as_float(r[c + CW / 2]));
#pragma unroll
                        for (int w2 = CW / 4; w2 > 0; w2 >>= 1)
#pragma unroll
                            for (int c = 0; c < w2; c++) m[c] = fmaxf(m[c], m[c + w2]);
                        // Slow path, entered by the whole warp when any row has a candidate in
                        // this chunk: a lane marks its hit columns and moves them to its stage.
                        const bool any_hit = row_live && (-m[0] < thr_eff);
                        if (__any_sync(0xffffffffu, any_hit)) {
                            if (any_hit) {
#pragma unroll
                                for (int h = 0; h < CW / 32; h++) {
                                    uint32_t mask = 0;
#pragma unroll
                                    for (int c = 0; c < 32; c++)
                                        mask |= (-__uint_as_float(r[h * 32 + c]) < thr_eff ? 1u : 0u) << c;
                                    while (mask != 0) {
                                        const int cc = __ffs(mask) - 1;
                                        mask &= mask - 1;
                                        uint32_t bits = 0;
#pragma unroll
                                        for (int c = 0; c < 32; c++) bits = (c == cc) ? r[h * 32 + c] : bits;
                                        if (nstaged == STAGE_N) {  // rare: list warm-up, massive ties
                                            if (MODE == MODE_TOPK)
                                                drain_to_list(lk, li, stage_key, stage_idx, nstaged, thr, thr_eff);
                                            else
                                                drain_to_buffer(p.cand_cnt + grow, p.cand_key + grow * p.cand_cap,
                                                                p.cand_idx + grow * p.cand_cap, p.cand_cap,
                                                                ksc, stage_key, stage_idx, nstaged);
                                            nstaged = 0;
                                        }
                                        stage_key[nstaged * STAGE_LD] = -__uint_as_float(bits);
                                        stage_idx[nstaged * STAGE_LD] = (int32_t)cbase + h * 32 + cc;
                                        nstaged++;
                                    }
                                }
                            }
                            __syncwarp();
                        }
                    }
                }
                };
                if constexpr (MODE == MODE_FILTER) {
                    if (p.wide) scan(std::integral_constant<int, 64>{});
                    else scan(std::integral_constant<int, 32>{});
                } else {
                    scan(std::integral_constant<int, 32>{});
                }
                } else {
#pragma unroll 1
                for (int ch = eh * CH_PER_HALF; ch < (eh + 1) * CH_PER_HALF; ch++) {
                    uint32_t r[32];
                    tc_ld32(taddr + ch * 32, r);
                    tc_wait_ld();
                    const int64_t cbase = c_tile + ch * 32;
                    {
                        // Store mode: thread t holds 32 consecutive columns of ITS row; writing
                        // them directly would touch 32 different rows per instruction.  The warp
                        // transposes the 32 x 32 block through shared memory (the list area is
                        // idle in this mode) and writes one 128-byte row segment per instruction.
                        float* tbuf = reinterpret_cast<float*>(smem + SM_LKEY) + (warp - 2) * (32 * 33);
#pragma unroll
                        for (int c = 0; c < 32; c++) {
                            const float key = -ksc * __uint_as_float(r[c]);
                            tbuf[lane * 33 + c] = fmaf(p.sign, key, radd);
                        }
                        __syncwarp();
                        const int64_t grow0 = grow - lane;  // first row of this warp's 32 rows
                        const bool col_ok = cbase + lane < p.ncols_end;
                        float* obase = p.out + (t * TILE_N + ch * 32) + lane;   // tiles lie side by side, whatever the stride
#pragma unroll 8
                        for (int rr = 0; rr < 32; rr++) {
                            const float v = tbuf[rr * 33 + lane];
                            if (col_ok && grow0 + rr < nq_live) obase[(grow0 + rr) * p.ld] = v;
                        }
                        __syncwarp();
                    }
                }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(map_to_cta(bar_tempty + eh * 8, 0));
                    else mbar_arrive(bar_tempty + acc * 8);
                }
                // the accumulator is back with the MMA issuers: now work off the staged hits
                if (nstaged > 0) {
                    if (MODE == MODE_TOPK)
                        drain_to_list(lk, li, stage_key, stage_idx, nstaged, thr, thr_eff);
                    else
                        drain_to_buffer(p.cand_cnt + grow, p.cand_key + grow * p.cand_cap,
                                        p.cand_idx + grow * p.cand_cap, p.cand_cap, ksc, stage_key,
                                        stage_idx, nstaged);
                    nstaged = 0;
                }
                __syncwarp();
                if (C::ACC_BUFS == 2) {
                    acc ^= 1;
                    if (acc == 0) acc_phase ^= 1;
                } else {
                    acc_phase ^= 1;
                }
            }
            if (MODE == MODE_TOPK && row_live && ok) {
                if (thr < thr_pub) atomicMin(gslot, float_to_ordered(thr));
                // two lists per (row, column range): one per column half
                float* okey = p.part_key + (grow * (2 * p.P) + 2 * xr + eh) * k - (KMAX - k);
                int32_t* oidx = p.part_idx + (grow * (2 * p.P) + 2 * xr + eh) * k - (KMAX - k);
#pragma unroll
                for (int j = 0; j < KMAX; j++) {
                    if (j >= KMAX - k) {
                        okey[j] = ksc * lk[j];  // INF stays INF for empty slots
                        oidx[j] = li[j];
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // the peer may still read this CTA's tiles / signal its barriers
    if (warp == 1) {
        __syncwarp();
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                         "r"(TMEM_COLS)
                         : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                         "r"(TMEM_COLS)
                         : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
                    cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
        else
            (void)cudaGetLastError();
    }
    return fn;
}

// 3-D map {k, row, plane} over a [planes][rows][pitch] 16-bit array; box {64, box_rows, 1}.
int make_operand_map(CUtensorMap* map, const uint16_t* base, int is_bf16, int64_t k_extent,
                     int64_t rows, int64_t pitch, int planes, int64_t plane_stride, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return B200F_ERR_CUDA;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (pitch % 8) != 0 ||
        (planes > 1 && (plane_stride % 8) != 0))
        return B200F_ERR_BAD_ARG;
    cuuint64_t dims[3] = {(cuuint64_t)k_extent, (cuuint64_t)rows, (cuuint64_t)planes};
    cuuint64_t pstride = (planes > 1) ? (cuuint64_t)plane_stride * 2 : (cuuint64_t)pitch * 2 * (cuuint64_t)(rows > 0 ? rows : 1);
    cuuint64_t strides[2] = {(cuuint64_t)pitch * 2, pstride};
    cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                    3, const_cast<uint16_t*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? B200F_OK : B200F_ERR_CUDA;
}

int launch_common(const GemmOperands& op, const GemmPlan& plan, GemmParams& p, int64_t col0,
                  int64_t ncols, cudaStream_t stream) {
    if (op.nq <= 0 || ncols <= 0) return B200F_OK;
    if (col0 + ncols > op.nb || op.nb > 0x7fffffffLL) return B200F_ERR_BAD_ARG;
    CUtensorMap ma, mb;
    int rc = make_operand_map(&ma, op.a_planes, op.is_bf16, op.d_pad, op.nq, op.a_pitch, op.npl,
                              op.a_plane_stride, BM);
    if (rc != B200F_OK) return rc;
    rc = make_operand_map(&mb, op.b_planes, op.is_bf16, op.d_pad, op.nb, op.b_pitch, op.npl,
                          op.b_plane_stride, plan.pair ? Cfg<true>::B_ROWS : Cfg<false>::B_ROWS);
    if (rc != B200F_OK) return rc;

    p.nq = op.nq;
    p.nq_dev = op.nq_dev;
    if (p.tile_stride < 1) p.tile_stride = 1;
    p.col0 = col0;
    p.ncols_end = col0 + ncols;
    p.ntiles = plan.ntiles;
    p.tiles_per_range = plan.tiles_per_range;
    p.nqb = plan.nqb;
    p.P = plan.P;
    p.kb_per_pass = (int)ceil_div64(op.d_pad, BK);
    p.k_extent = op.d_pad;
    p.rowscale = op.rowscale;
    p.rowscale_map = op.rowscale_map;
    if (op.npl == 1) {
        p.npass = 1;
        p.pass_a = 0;
        p.pass_b = 0;
    } else if (op.npl == 2) {
        // two fp16 planes (22 bits): (1,0) (0,1) (0,0), smallest first; (1,1) is below 2^-22
        p.npass = 3;
        p.pass_a = 0x001u;
        p.pass_b = 0x010u;
    } else {
        // smallest products first: (1,1) (0,2) (2,0) (0,1) (1,0) (0,0)
        p.npass = 6;
        p.pass_a = 0x010201u;  // nibble i = plane of A in pass i (pass 0 is the lowest nibble)
        p.pass_b = 0x001021u;
    }
    const uint32_t fmt = op.is_bf16 ? 1u : 0u;
    // fp32 accumulate, K-major operands, N = 256, M = 128 (one CTA) or 256 (CTA pair)
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) |
              ((uint32_t)((plan.pair ? 2 * BM : BM) >> 4) << 24);

    typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const GemmParams);
    static const KernelFn kernels[2][3] = {
            {gemm_topk_kernel<false, MODE_TOPK>, gemm_topk_kernel<false, MODE_STORE>,
             gemm_topk_kernel<false, MODE_FILTER>},
            {gemm_topk_kernel<true, MODE_TOPK>, gemm_topk_kernel<true, MODE_STORE>,
             gemm_topk_kernel<true, MODE_FILTER>}};
    static bool attr_set[kMaxDevices] = {false};   // the shared-memory opt-in is per device
    const int slot = device_slot();
    if (!attr_set[slot]) {
        for (int pr = 0; pr < 2; pr++)
            for (int m = 0; m < 3; m++)
                B200F_CUDA_TRY(cudaFuncSetAttribute(reinterpret_cast<const void*>(kernels[pr][m]),
                                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    pr ? Cfg<true>::SMEM_BYTES : Cfg<false>::SMEM_BYTES));
        attr_set[slot] = true;
    }
    if (p.mode < 0 || p.mode > 2) return B200F_ERR_BAD_ARG;
    const KernelFn kernel = kernels[plan.pair ? 1 : 0][p.mode];
    main_kernel_begin(stream);
    if (plan.pair) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)plan.grid, 1, 1);
        cfg.blockDim = dim3(NUM_THREADS, 1, 1);
        cfg.dynamicSmemBytes = Cfg<true>::SMEM_BYTES;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ma, mb, p);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            main_kernel_end(stream);
            return B200F_ERR_CUDA;
        }
    } else {
        kernel<<<plan.grid, NUM_THREADS, Cfg<false>::SMEM_BYTES, stream>>>(ma, mb, p);
    }
    main_kernel_end(stream);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

}  // namespace

// Shape override (testing): b200f_set_gemm_shape, default from the environment variable
// B200F_GEMM_PAIR=0 / 1 read ONCE at the first plan.  -1 = choose by the number of queries.
static std::atomic<int> g_pair_override{-2};

static int pair_override() {
    int v = g_pair_override.load(std::memory_order_relaxed);
    if (v == -2) {
        const char* e = getenv("B200F_GEMM_PAIR");
        v = (e && (e[0] == '0' || e[0] == '1')) ? e[0] - '0' : -1;
        int expected = -2;
        if (!g_pair_override.compare_exchange_strong(expected, v)) v = expected;
    }
    return v;
}

// CTA pairs that can be resident at once (GPC boundaries may leave a few SMs unpaired).
static int max_active_pairs(int sm_count) {
    static int per_device[kMaxDevices] = {0};   // 0 = not asked yet on that device
    int& cached = per_device[device_slot()];
    if (cached <= 0) {
        cached = sm_count / 2;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(sm_count / 2 * 2), 1, 1);
        cfg.blockDim = dim3(NUM_THREADS, 1, 1);
        cfg.dynamicSmemBytes = Cfg<true>::SMEM_BYTES;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaFuncSetAttribute(gemm_topk_kernel<true, MODE_TOPK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<true>::SMEM_BYTES) == cudaSuccess &&
            cudaOccupancyMaxActiveClusters(&n, gemm_topk_kernel<true, MODE_TOPK>, &cfg) == cudaSuccess && n > 0) {
            if (n < cached) cached = n;
        } else {
            (void)cudaGetLastError();
        }
    }
    return cached;
}

GemmPlan plan_gemm(int64_t nq, int64_t ncols, int sm_count) {
    GemmPlan g;
    const int ov = pair_override();
    g.pair = ov >= 0 ? ov : (nq > BM ? 1 : 0);       // a pair covers 256 query rows
    const int qb = g.pair ? 2 * BM : BM;
    const int units = g.pair ? max_active_pairs(sm_count) : sm_count;  // CTAs or CTA pairs that run at once
    g.nqb = (int)ceil_div64(nq, qb);
    g.tile_n = g.pair ? Cfg<true>::TILE_N : Cfg<false>::TILE_N;
    g.ntiles = ceil_div64(ncols, g.tile_n);
    if (g.nqb <= 0 || g.ntiles <= 0) {
        g.nqb = 0; g.ntiles = 0; g.P = 0; g.tiles_per_range = 0; g.grid = 0;
        return g;
    }
    // Number of column ranges: make nqb * P a multiple of the unit count when there is
    // enough work, keep at least ~32 tiles per range so list warm-up stays cheap.
    auto gcd = [](int64_t a, int64_t b) { while (b) { int64_t t = a % b; a = b; b = t; } return a; };
    int64_t P0 = units / gcd(units, g.nqb);
    int64_t P;
    if (P0 >= g.ntiles) {
        P = g.ntiles;
    } else {
        int64_t max_mult = g.ntiles / (P0 * 32);
        int64_t want_waves = 8;
        int64_t mult = (want_waves * units) / (P0 * g.nqb);
        if (mult < 1) mult = 1;
        if (max_mult < 1) max_mult = 1;
        if (mult > max_mult) mult = max_mult;
        P = P0 * mult;
    }
    if (P > 4096) P = 4096;
    g.tiles_per_range = ceil_div64(g.ntiles, P);
    g.P = (int)ceil_div64(g.ntiles, g.tiles_per_range);
    int64_t items = (int64_t)g.nqb * g.P;
    int64_t u = items < units ? items : units;
    g.grid = (int)(g.pair ? 2 * u : u);
    return g;
}

int launch_gemm_topk(const GemmOperands& op, const GemmPlan& plan, int64_t col0, int64_t ncols,
                     int64_t tile_stride, float kscale, int k, int gslots, float* part_key,
                     int32_t* part_idx, uint32_t* gthr, int32_t* status, cudaStream_t stream) {
    if (k <= 0 || k > KMAX || gslots < 1) return B200F_ERR_UNSUPPORTED;
    if (!gthr) return B200F_ERR_BAD_ARG;
    // all-ones is above every ordered float: no bound yet
    B200F_CUDA_TRY(cudaMemsetAsync(gthr, 0xff, (size_t)op.nq * gslots * sizeof(uint32_t), stream));
    GemmParams p{};
    p.mode = MODE_TOPK;
    p.tile_stride = tile_stride;
    p.gslots = gslots;
    p.k = k;
    p.kscale = kscale;
    p.sign = 1.f;
    p.rowadd = nullptr;
    p.part_key = part_key;
    p.part_idx = part_idx;
    p.gthr = gthr;
    p.out = nullptr;
    p.ld = 0;
    p.status = status;
    return launch_common(op, plan, p, col0, ncols, stream);
}

int launch_gemm_filter(const GemmOperands& op, const GemmPlan& plan, float kscale, const float* thr,
                       int thr_stride, int thr_pos, float* cand_key, int32_t* cand_idx,
                       int32_t* cand_cnt, int cand_cap, int few_hits, int32_t* status,
                       cudaStream_t stream) {
    if (!thr || !cand_key || !cand_idx || !cand_cnt || cand_cap < 1) return B200F_ERR_BAD_ARG;
    B200F_CUDA_TRY(cudaMemsetAsync(cand_cnt, 0, (size_t)op.nq * sizeof(int32_t), stream));
    GemmParams p{};
    p.mode = MODE_FILTER;
    p.kscale = kscale;
    p.sign = 1.f;
    p.fthr = thr;
    p.fthr_stride = thr_stride;
    p.fthr_pos = thr_pos;
    p.cand_key = cand_key;
    p.cand_idx = cand_idx;
    p.cand_cnt = cand_cnt;
    p.cand_cap = cand_cap;
    p.wide = few_hits ? 1 : 0;
    p.status = status;
    return launch_common(op, plan, p, 0, op.nb, stream);
}

int launch_gemm_store(const GemmOperands& op, const GemmPlan& plan, int64_t col0, int64_t ncols,
                      int64_t tile_stride, float kscale, float sign, const float* rowadd, float* out,
                      int64_t ld, int32_t* status, cudaStream_t stream) {
    GemmParams p{};
    p.mode = MODE_STORE;
    p.tile_stride = tile_stride;
    p.k = 0;
    p.kscale = kscale;
    p.sign = sign;
    p.rowadd = rowadd;
    p.part_key = nullptr;
    p.part_idx = nullptr;
    p.out = out;
    p.ld = ld;
    p.status = status;
    return launch_common(op, plan, p, col0, ncols, stream);
}

}  // namespace b200f

extern "C" int b200f_set_gemm_shape(int shape) {
    if (shape < B200F_GEMM_SHAPE_AUTO || shape > B200F_GEMM_SHAPE_PAIR) return B200F_ERR_BAD_ARG;
    b200f::g_pair_override.store(shape, std::memory_order_relaxed);
    return B200F_OK;
}
