// Streaming search for small query batches: HBM-bound.  Two kernels:
//   scan_mma_kernel  16-bit rows, up to 8 queries per pass: rows staged through a
//                    cp.async.bulk ring, scores by mma.sync (described further down)
//   scan_kernel      the plain version (fp32 rows, shards too small for the ring, and the
//                    store mode that writes keys for k > 32): up to 4 queries per pass
//
// Replaces fused_l2_topk_min / fused_ip_topk_max and their f16storage variants
// (shaders/fused_l2_topk.metal:19-444, gate in src/MetalDistance.mm:341-354) and the
// tiny-database direct kernels l2_distance_direct_f16[storage]
// (shaders/l2_norm_f16.metal:74-123).  Differences by design: every lane streams
// 128-bit pieces of consecutive rows (the reference walks one whole row per lane),
// the dot product is fp32, BF16 rows are handled natively, and the per-warp top-k is
// a sorted warp list (one slot per lane) updated by ballot + shuffle insertion so no
// candidate is dropped.
//
// Work layout of scan_kernel: a row of C 16-byte pieces is covered by LPR = min(8, pow2(C))
// lanes (ITERS = ceil(C / LPR) pieces per lane); a warp therefore covers 32 / LPR rows per
// step and U steps per block, keeping U independent 16-byte loads in flight per lane.
#include "common.cuh"
#include "ptx.cuh"

namespace b200f {

namespace {

constexpr int SCAN_THREADS = 256;
constexpr int SCAN_WARPS = SCAN_THREADS / 32;
constexpr int SCAN_U = 8;
constexpr unsigned FULL = 0xffffffffu;

struct ScanParams {
    const float* queries;   // [nq][d]
    const void* rows;
    int64_t pitch_bytes;
    const float* norms;     // null for inner product
    int64_t nb;
    int64_t col0, col1;     // rows [col0, col1) are scanned
    int d;
    int nq;
    int k;
    int metric;
    int C;                  // 16-byte pieces per row
    int lpr;                // lanes per row (power of two)
    int iters;              // pieces per lane
    int qstride;            // floats per query in shared memory (C * E)
    int norm_cols;          // 16-bit rows carry -||x||^2/2 in 8 columns after d8 (see rows.cu)
    float nscale[4];        // scales the query side puts into those columns
    float* part_key;        // top-k mode: [nq][P][k]
    int32_t* part_idx;
    float* out;             // store mode: [nq][ld]
    int64_t ld;
    // bulk-copy pipeline (scan_bulk_kernel)
    int rb;                 // rows per consumer warp per stage
    int stage_rows;         // rows per stage = SB_NW * rb
    int stage_stride;       // bytes between stages in shared memory
    int nstage;
    int32_t* status;
};

template <int STORAGE>
struct Piece {
    static constexpr int E = (STORAGE == B200F_STORAGE_F32) ? 4 : 8;
};

template <int STORAGE>
__device__ __forceinline__ void unpack(const uint4& v, float (&x)[Piece<STORAGE>::E]) {
    if (STORAGE == B200F_STORAGE_F32) {
        x[0] = __uint_as_float(v.x);
        x[1] = __uint_as_float(v.y);
        x[2] = __uint_as_float(v.z);
        x[3] = __uint_as_float(v.w);
    } else if (STORAGE == B200F_STORAGE_BF16) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int t = 0; t < 4; t++) {
            x[2 * t] = __uint_as_float(w[t] << 16);
            x[2 * t + 1] = __uint_as_float(w[t] & 0xffff0000u);
        }
    } else {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int t = 0; t < 4; t++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
            x[2 * t] = f.x;
            x[2 * t + 1] = f.y;
        }
    }
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ unsigned long long pack2(uint32_t lo, uint32_t hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
// d = a * b + c on both fp32 halves of the 64-bit operands
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// (key, id) lexicographic "a before b"
__device__ __forceinline__ bool before(float ka, int ia, float kb, int ib) {
    return (ka < kb) || (ka == kb && (unsigned)ia < (unsigned)ib);
}

// Sorted warp list: lane j holds rank j.  All 32 lanes call this together.
__device__ __forceinline__ void warp_insert(float& lk, int& li, float s, int id, int lane) {
    const bool stays = before(lk, li, s, id);
    const int pos = __popc(__ballot_sync(FULL, stays));
    const float upk = __shfl_up_sync(FULL, lk, 1);
    const int upi = __shfl_up_sync(FULL, li, 1);
    if (lane == pos) {
        lk = s;
        li = id;
    } else if (lane > pos) {
        lk = upk;
        li = upi;
    }
}

template <int STORAGE, int NQ, bool STORE>
// Three CTAs per SM where 80 registers suffice; four queries, and two queries on fp32 rows (paired
// accumulators), take 128 registers and two CTAs; the grid is exactly one such wave.  Measured on
// 12.5 M fp32 rows of d = 128: 6.90 / 5.64 / 4.06 TB/s for one / two / four queries (4.98 / 4.58 /
// 3.53 with plain FMAs and a grid of four CTAs per SM, whose last wave ran a third full).
__global__ void __launch_bounds__(SCAN_THREADS, (NQ == 4 || (NQ == 2 && STORAGE == B200F_STORAGE_F32 && !STORE)) ? 2 : 3)
scan_kernel(const ScanParams p) {
    constexpr int E = Piece<STORAGE>::E;
    // rows per lane and block; fp32 rows keep two partial sums per (row, query), so fewer rows fit the registers
    constexpr int U = (STORAGE == B200F_STORAGE_F32 && !STORE && NQ == 4) ? 6 : SCAN_U;
    extern __shared__ __align__(16) float sq[];  // [NQ][qstride] queries, then merge area
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

    // stage the queries (zero padded to whole pieces)
    for (int i = threadIdx.x; i < NQ * p.qstride; i += SCAN_THREADS) {
        const int qi = i / p.qstride;
        const int j = i - qi * p.qstride;
        float v = 0.f;
        if (qi < p.nq) {
            const int d8 = (p.d + 7) & ~7;
            if (j < p.d) v = p.queries[(int64_t)qi * p.d + j];
            else if (p.norm_cols && j >= d8 && j < d8 + 4) v = p.nscale[j - d8];
        }
        sq[i] = v;
    }
    __syncthreads();

    const int lpr = p.lpr;
    const int rps = 32 / lpr;            // rows per warp step
    const int cl = lane & (lpr - 1);     // piece lane inside the row
    const int sub = lane / lpr;          // which of the rps rows
    const int rows_per_block = rps * U;
    const int64_t nrows = p.col1 - p.col0;
    const int64_t nblocks = ceil_div64(nrows, rows_per_block);
    const int64_t gw = (int64_t)blockIdx.x * SCAN_WARPS + warp;
    const int64_t total_warps = (int64_t)gridDim.x * SCAN_WARPS;
    const uint8_t* base = reinterpret_cast<const uint8_t*>(p.rows);
    const bool l2 = p.metric == B200F_METRIC_L2;

    float lk[NQ];
    int li[NQ];
    float thr[NQ];
    int thr_id[NQ];
#pragma unroll
    for (int qi = 0; qi < NQ; qi++) {
        lk[qi] = CUDART_INF_F;
        li[qi] = -1;
        thr[qi] = CUDART_INF_F;
        thr_id[qi] = -1;
    }

    for (int64_t blk = gw; blk < nblocks; blk += total_warps) {
        const int64_t row_base = p.col0 + blk * rows_per_block;
        float acc[U][NQ];
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int qi = 0; qi < NQ; qi++) acc[u][qi] = 0.f;
        // fp32 rows: two partial sums per (row, query) in one 64-bit register, advanced by packed
        // FMAs (fma.rn.f32x2: half the FMA instructions of the plain loop, which is what limits
        // this kernel before the memory system does)
        [[maybe_unused]] unsigned long long acc2[STORAGE == B200F_STORAGE_F32 ? U : 1][NQ];
        if constexpr (STORAGE == B200F_STORAGE_F32) {
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int qi = 0; qi < NQ; qi++) acc2[u][qi] = 0ull;
        }

        for (int it = 0; it < p.iters; it++) {
            const int piece = it * lpr + cl;
            const bool pv = piece < p.C;
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int64_t row = row_base + u * rps + sub;
                if (pv && row < p.col1)
                    v[u] = ldg_stream(base + row * p.pitch_bytes + (int64_t)piece * 16);
                else
                    v[u] = make_uint4(0, 0, 0, 0);
            }
            if constexpr (STORAGE == B200F_STORAGE_F32) {
                unsigned long long q01[NQ], q23[NQ];
#pragma unroll
                for (int qi = 0; qi < NQ; qi++) {
                    const uint4 f = *reinterpret_cast<const uint4*>(sq + qi * p.qstride + (pv ? piece : 0) * E);
                    q01[qi] = pack2(f.x, f.y);
                    q23[qi] = pack2(f.z, f.w);
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const unsigned long long x01 = pack2(v[u].x, v[u].y);
                    const unsigned long long x23 = pack2(v[u].z, v[u].w);
#pragma unroll
                    for (int qi = 0; qi < NQ; qi++) {
                        acc2[u][qi] = fma2(x01, q01[qi], acc2[u][qi]);
                        acc2[u][qi] = fma2(x23, q23[qi], acc2[u][qi]);
                    }
                }
                continue;
            }
            float qf[NQ][E];
#pragma unroll
            for (int qi = 0; qi < NQ; qi++) {
                const float4* src = reinterpret_cast<const float4*>(sq + qi * p.qstride + (pv ? piece : 0) * E);
#pragma unroll
                for (int e4 = 0; e4 < E / 4; e4++) {
                    const float4 f = src[e4];
                    qf[qi][4 * e4] = f.x;
                    qf[qi][4 * e4 + 1] = f.y;
                    qf[qi][4 * e4 + 2] = f.z;
                    qf[qi][4 * e4 + 3] = f.w;
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                float x[E];
                unpack<STORAGE>(v[u], x);
#pragma unroll
                for (int qi = 0; qi < NQ; qi++)
#pragma unroll
                    for (int e = 0; e < E; e++) acc[u][qi] = fmaf(qf[qi][e], x[e], acc[u][qi]);
            }
        }
        if constexpr (STORAGE == B200F_STORAGE_F32) {
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int qi = 0; qi < NQ; qi++)
                    acc[u][qi] = __uint_as_float((uint32_t)acc2[u][qi]) + __uint_as_float((uint32_t)(acc2[u][qi] >> 32));
        }
        // reduce the partial dot products over the lpr lanes of each row
        for (int o = lpr >> 1; o > 0; o >>= 1) {
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int qi = 0; qi < NQ; qi++)
                    acc[u][qi] += __shfl_xor_sync(FULL, acc[u][qi], o);
        }
        // lane cl == 0 of each row group owns the row's candidates.  With several queries the
        // dot products are first turned into keys and ONE vote decides whether any row of the block
        // has a candidate for any query (a single query measured slower with the extra pass).
        constexpr bool PREVOTE = (NQ > 1) && !STORE;
        if (PREVOTE) {
            bool any_hit = false;
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int64_t row = row_base + u * rps + sub;
                const bool owner = (cl == 0) && row < p.col1;
                float nrm = 0.f;
                if (owner && l2) nrm = __ldg(p.norms + row);
#pragma unroll
                for (int qi = 0; qi < NQ; qi++) {
                    acc[u][qi] = l2 ? fmaf(-2.f, acc[u][qi], nrm) : -acc[u][qi];
                    any_hit |= owner && before(acc[u][qi], (int)row, thr[qi], thr_id[qi]);
                }
            }
            if (!__any_sync(FULL, any_hit)) continue;
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int64_t row = row_base + u * rps + sub;
            const bool owner = (cl == 0) && row < p.col1;
            float nrm = 0.f;
            if (!PREVOTE && owner && l2) nrm = __ldg(p.norms + row);
#pragma unroll
            for (int qi = 0; qi < NQ; qi++) {
                const float key = PREVOTE ? acc[u][qi] : (l2 ? fmaf(-2.f, acc[u][qi], nrm) : -acc[u][qi]);
                if (STORE) {
                    if (owner && qi < p.nq) p.out[(int64_t)qi * p.ld + (row - p.col0)] = key;
                } else {
                    const bool hit = owner && before(key, (int)row, thr[qi], thr_id[qi]);
                    unsigned m = __ballot_sync(FULL, hit);
                    while (m) {
                        const int src = __ffs(m) - 1;
                        m &= m - 1;
                        const float s = __shfl_sync(FULL, key, src);
                        const int id = __shfl_sync(FULL, (int)row, src);
                        if (before(s, id, thr[qi], thr_id[qi])) {
                            warp_insert(lk[qi], li[qi], s, id, lane);
                            thr[qi] = __shfl_sync(FULL, lk[qi], p.k - 1);
                            thr_id[qi] = __shfl_sync(FULL, li[qi], p.k - 1);
                        }
                    }
                }
            }
        }
    }

    if (STORE) return;

    // CTA merge: every warp publishes its lists, warp qi folds them for query qi.
    __syncthreads();  // queries in shared memory are no longer needed
    float* mk = sq;                                                  // [SCAN_WARPS][NQ][32]
    int* mi = reinterpret_cast<int*>(sq + SCAN_WARPS * NQ * 32);
#pragma unroll
    for (int qi = 0; qi < NQ; qi++) {
        mk[(warp * NQ + qi) * 32 + lane] = lk[qi];
        mi[(warp * NQ + qi) * 32 + lane] = li[qi];
    }
    __syncthreads();
    if (warp < NQ && warp < p.nq) {
        const int qi = warp;
        float k0 = mk[(0 * NQ + qi) * 32 + lane];
        int i0 = mi[(0 * NQ + qi) * 32 + lane];
        float t = __shfl_sync(FULL, k0, p.k - 1);
        int tid = __shfl_sync(FULL, i0, p.k - 1);
        for (int w = 1; w < SCAN_WARPS; w++) {
            for (int j = 0; j < p.k; j++) {
                const float s = mk[(w * NQ + qi) * 32 + j];
                const int id = mi[(w * NQ + qi) * 32 + j];
                if (id < 0) break;  // sorted: the rest of this list is empty
                if (before(s, id, t, tid)) {
                    warp_insert(k0, i0, s, id, lane);
                    t = __shfl_sync(FULL, k0, p.k - 1);
                    tid = __shfl_sync(FULL, i0, p.k - 1);
                } else {
                    break;  // sorted: nothing later in this list can enter either
                }
            }
        }
        if (lane < p.k) {
            const int64_t o = ((int64_t)qi * gridDim.x + blockIdx.x) * p.k + lane;
            p.part_key[o] = k0;
            p.part_idx[o] = i0;
        }
    }
}


// ---------------------------------------------------------------------------------------
// Streaming pipeline for 16-bit storage (top-k mode, up to 8 queries per pass): one CTA per
// SM.  Warp 0 streams whole blocks of rows (contiguous in memory) into a shared-memory ring
// with cp.async.bulk + mbarriers, so the bytes in flight are set by the ring depth.  The
// SM_NW consumer warps take 16-row tiles and evaluate them with mma.sync m16n8k16
// (A = 16 stored rows, B = the queries as 8 columns, fp32 accumulate): about two
// instructions per row instead of a convert + FMA per element, and no shuffle reduction --
// the accumulator fragment leaves the score of (row g / g+8, query 2t / 2t+1) in lane 4g+t.
// The dot product is invariant under a permutation of K applied to both operands, so each
// lane simply takes 16 contiguous bytes per 32-column chunk (row g and row g+8 at column
// 32c + 8t) and the query matrix in shared memory is read with the same pattern.  With
// norm columns in the rows the L2 term -||x||^2/2 is part of the same dot product.
// ---------------------------------------------------------------------------------------
constexpr int SM_NW = 8;            // consumer warps of the ring kernels (scan_mma_kernel: for one or two queries)
constexpr int SM_NW_MANY = 12;      // scan_mma_kernel with three to eight queries
constexpr int SM_THREADS = 32 * (1 + SM_NW);
constexpr int SM_MAX_STAGES = 8;
constexpr int SM_NQ = 8;

template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    if (BF16) {
        asm volatile(
                "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                "{%8,%9}, {%0,%1,%2,%3};"
                : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile(
                "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                "{%8,%9}, {%0,%1,%2,%3};"
                : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// NW consumer warps: 8 for one or two queries (6.80 / 6.62 TB/s on 25 M fp16 rows; 12 warps: 6.55 at
// one), 12 beyond (four queries 6.24 -> 6.53 TB/s, eight 5.44 -> 6.08).
template <bool BF16, int NW>
__global__ void __launch_bounds__(32 * (1 + NW), 1) scan_mma_kernel(const ScanParams p) {
    extern __shared__ __align__(128) uint8_t sm[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint32_t sbase = smem_u32(sm);
    const int ring_bytes = p.nstage * p.stage_stride;
    // query matrix [8][kq] in the storage format, kq = 32 * nchunk (zero padded)
    const int nchunk = p.iters;          // 32-column chunks per row, norm columns included
    const int kq = nchunk * 32;
    uint16_t* sqh = reinterpret_cast<uint16_t*>(sm + ring_bytes);
    const int qbytes = SM_NQ * kq * 2;
    const uint32_t bar_full = sbase + ring_bytes + qbytes;
    const uint32_t bar_empty = bar_full + SM_MAX_STAGES * 8;
    volatile int* abort_flag =
            reinterpret_cast<volatile int*>(sm + ring_bytes + qbytes + 2 * SM_MAX_STAGES * 8);
    const int d8 = (p.d + 7) & ~7;
    const int kext = d8 + (p.norm_cols ? 8 : 0);  // valid columns of a stored row

    for (int i = threadIdx.x; i < SM_NQ * kq; i += 32 * (1 + NW)) {
        const int qi = i / kq;
        const int j = i - qi * kq;
        float v = 0.f;
        if (qi < p.nq) {
            if (j < p.d) v = p.queries[(int64_t)qi * p.d + j];
            else if (p.norm_cols && j >= d8 && j < d8 + 4) v = p.nscale[j - d8];
        }
        sqh[i] = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
    }
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < p.nstage; s++) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, NW);
        }
        mbar_fence_init();
    }
    __syncthreads();

    const int64_t nrows_total = p.col1 - p.col0;
    const int64_t nchunks = ceil_div64(nrows_total, p.stage_rows);
    const uint8_t* base = reinterpret_cast<const uint8_t*>(p.rows);
    const float kmul = p.metric == B200F_METRIC_L2 ? -2.f : -1.f;

    float lk[SM_NQ];
    int li[SM_NQ];
    float thr[SM_NQ];
    int thr_id[SM_NQ];
#pragma unroll
    for (int qi = 0; qi < SM_NQ; qi++) {
        lk[qi] = CUDART_INF_F;
        li[qi] = -1;
        thr[qi] = CUDART_INF_F;
        thr_id[qi] = -1;
    }

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
                if (!mbar_wait_bounded(bar_empty + stage * 8, phase ^ 1, abort_flag, p.status,
                                       kDevErrBarrierWait)) {
                    ok = false;
                    break;
                }
                const int64_t row0 = p.col0 + c * p.stage_rows;
                const int64_t nr = min((int64_t)p.stage_rows, p.col1 - row0);
                const uint32_t bytes = (uint32_t)(nr * p.pitch_bytes);
                mbar_arrive_expect_tx(bar_full + stage * 8, bytes);
                bulk_load(sbase + stage * p.stage_stride, base + row0 * p.pitch_bytes, bytes,
                          bar_full + stage * 8);
                if (++stage == p.nstage) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (!ok) {  // let copies already issued land before shared memory goes away
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) {
                }
            }
        }
    } else {
        const int wc = warp - 1;
        const int g = lane >> 2;
        const int t = lane & 3;
        int stage = 0;
        uint32_t phase = 0;
        // Bounds of the two queries whose scores land in this lane (2t and 2t+1), so that ONE vote
        // per tile tells whether any of its 16 x nq scores is a candidate; a query beyond nq
        // gets -INF and never is.
        float mta, mtb;
        int mia, mib;
        auto refresh_bounds = [&]() {
            mta = t == 0 ? thr[0] : t == 1 ? thr[2] : t == 2 ? thr[4] : thr[6];
            mtb = t == 0 ? thr[1] : t == 1 ? thr[3] : t == 2 ? thr[5] : thr[7];
            mia = t == 0 ? thr_id[0] : t == 1 ? thr_id[2] : t == 2 ? thr_id[4] : thr_id[6];
            mib = t == 0 ? thr_id[1] : t == 1 ? thr_id[3] : t == 2 ? thr_id[5] : thr_id[7];
            if (2 * t >= p.nq) mta = -CUDART_INF_F;
            if (2 * t + 1 >= p.nq) mtb = -CUDART_INF_F;
        };
        refresh_bounds();
        // a stage may hold fewer 16-row tiles than there are consumer warps: the first tile's owner
        // moves on by that many warps from stage to stage, so all of them work (eight warps: stages of
        // 128 or 256 rows are the rule, and the single-query stream keeps its measured loop)
        constexpr bool ROTATE = NW != 8;
        const int tiles_full = p.stage_rows >> 4;
        int shift = 0;
        for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
            const bool w = mbar_wait_bounded(bar_full + stage * 8, phase, abort_flag, p.status,
                                             kDevErrBarrierWait);
            if (!__all_sync(FULL, w)) break;
            const int64_t row0 = p.col0 + c * p.stage_rows;
            const int nr = (int)min((int64_t)p.stage_rows, p.col1 - row0);
            const uint32_t sstage = sbase + stage * p.stage_stride;
            const int ntiles = (nr + 15) >> 4;
            for (int tile = ROTATE ? (wc - shift + NW) % NW : wc; tile < ntiles; tile += NW) {
                const int r0 = tile * 16 + g;      // local rows of this lane
                const int r1 = r0 + 8;
                const bool v0 = r0 < nr, v1 = r1 < nr;
                const uint32_t a_row0 = sstage + (uint32_t)r0 * (uint32_t)p.pitch_bytes + t * 16;
                const uint32_t a_row1 = sstage + (uint32_t)r1 * (uint32_t)p.pitch_bytes + t * 16;
                const uint32_t b_row = sbase + ring_bytes + (uint32_t)(g * kq * 2) + t * 16;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
                for (int ch = 0; ch < nchunk; ch++) {
                    const bool kv = ch * 32 + t * 8 < kext;  // beyond the row: the next row's bytes
                    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = make_uint4(0, 0, 0, 0);
                    if (kv && v0) x0 = lds128(a_row0 + ch * 64);
                    if (kv && v1) x1 = lds128(a_row1 + ch * 64);
                    const uint4 q = lds128(b_row + ch * 64);
                    // A fragment: a0 = row g cols k, a1 = row g+8 cols k, a2 = row g cols k+8, a3 = row g+8 cols k+8
                    mma16816<BF16>(acc, x0.x, x1.x, x0.y, x1.y, q.x, q.y);
                    mma16816<BF16>(acc, x0.z, x1.z, x0.w, x1.w, q.z, q.w);
                }
                // acc[0]: (row r0, query 2t)  acc[1]: (r0, 2t+1)  acc[2]: (r1, 2t)  acc[3]: (r1, 2t+1)
                // One vote tells whether the tile has a candidate at all; if so, one vote per accumulator
                // register: bit l of mj[j] = lane l's key j is a candidate (lane 4g + t holds query 2t
                // in keys 0 / 2 and query 2t + 1 in keys 1 / 3).
                const int row_a = (int)(row0 + r0), row_b = (int)(row0 + r1);
                float key[4];
#pragma unroll
                for (int j = 0; j < 4; j++) key[j] = kmul * acc[j];
                const bool h0 = v0 && before(key[0], row_a, mta, mia), h1 = v0 && before(key[1], row_a, mtb, mib);
                const bool h2 = v1 && before(key[2], row_b, mta, mia), h3 = v1 && before(key[3], row_b, mtb, mib);
                if (!__any_sync(FULL, h0 || h1 || h2 || h3)) continue;  // the usual case: nothing for any query
                unsigned mj[4];
                mj[0] = __ballot_sync(FULL, h0);
                mj[1] = __ballot_sync(FULL, h1);
                mj[2] = __ballot_sync(FULL, h2);
                mj[3] = __ballot_sync(FULL, h3);
#pragma unroll
                for (int qi = 0; qi < SM_NQ; qi++) {
                    if (qi >= p.nq) break;
                    const unsigned lanes_q = 0x11111111u << (qi >> 1);   // the lanes with t = qi / 2
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const float kk = key[2 * h + (qi & 1)];
                        const int row = h ? row_b : row_a;
                        unsigned m = mj[2 * h + (qi & 1)] & lanes_q;
                        while (m) {
                            const int src = __ffs(m) - 1;
                            m &= m - 1;
                            const float s = __shfl_sync(FULL, kk, src);
                            const int id = __shfl_sync(FULL, row, src);
                            if (before(s, id, thr[qi], thr_id[qi])) {
                                warp_insert(lk[qi], li[qi], s, id, lane);
                                thr[qi] = __shfl_sync(FULL, lk[qi], p.k - 1);
                                thr_id[qi] = __shfl_sync(FULL, li[qi], p.k - 1);
                            }
                        }
                    }
                }
                refresh_bounds();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + stage * 8);
            if (ROTATE) shift = (shift + tiles_full) % NW;
            if (++stage == p.nstage) {
                stage = 0;
                phase ^= 1;
            }
        }
    }

    // CTA merge in the (now idle) ring memory: consumer warp wc publishes its lists,
    // warp 1 + qi folds them for query qi.
    __syncthreads();
    float* mk = reinterpret_cast<float*>(sm);                        // [NW][SM_NQ][32]
    int* mi = reinterpret_cast<int*>(sm) + NW * SM_NQ * 32;
    if (warp > 0) {
#pragma unroll
        for (int qi = 0; qi < SM_NQ; qi++) {
            mk[((warp - 1) * SM_NQ + qi) * 32 + lane] = lk[qi];
            mi[((warp - 1) * SM_NQ + qi) * 32 + lane] = li[qi];
        }
    }
    __syncthreads();
    if (warp >= 1 && warp - 1 < p.nq) {
        const int qi = warp - 1;
        float k0 = mk[qi * 32 + lane];
        int i0 = mi[qi * 32 + lane];
        float tk = __shfl_sync(FULL, k0, p.k - 1);
        int tid = __shfl_sync(FULL, i0, p.k - 1);
        for (int w2 = 1; w2 < NW; w2++) {
            for (int j = 0; j < p.k; j++) {
                const float s = mk[(w2 * SM_NQ + qi) * 32 + j];
                const int id = mi[(w2 * SM_NQ + qi) * 32 + j];
                if (id < 0 || !before(s, id, tk, tid)) break;
                warp_insert(k0, i0, s, id, lane);
                tk = __shfl_sync(FULL, k0, p.k - 1);
                tid = __shfl_sync(FULL, i0, p.k - 1);
            }
        }
        if (lane < p.k) {
            const int64_t o = ((int64_t)qi * gridDim.x + blockIdx.x) * p.k + lane;
            p.part_key[o] = k0;
            p.part_idx[o] = i0;
        }
    }
}

// ---------------------------------------------------------------------------------------
// The same streaming pipeline for FP32 rows: mma.sync m16n8k8 on a tf32 split.  A value is
// x = hi + lo with hi = x cut to tf32's bits, lo = x - hi (of which the MMA reads the top bits: 21
// mantissa bits between them); the three products hi*hi, lo*hi, hi*lo accumulate in fp32 and leave
// about 2^-21 of the result out, as an fp32 FMA chain would.  The rows are split on the fly (a
// mask and a subtraction per element), the queries once into two matrices.  K is permuted as in the 16-bit kernel: per
// 16-column chunk a lane takes the 16 bytes at column 16c + 4t of rows g and g+8, floats 0 / 1 feed
// k-slots t / t+4 of the first MMA, floats 2 / 3 those of the second, and the query matrices are read
// with the same pattern.  ||x||^2 comes from the norm array (FP32 rows carry no norm columns).
// Up to 8 queries per pass, one dot product per (row, query) on the tensor pipe instead of d FMAs
// and a shuffle reduction: what held the FMA kernel to 86 % / 62 % of the copy bandwidth at 2 / 4
// queries (this kernel: 108 / 103 / 94 % at 2 / 4 / 8).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ void mma1688_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
            "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int ST_QPAD = 16;   // floats between query rows beyond kq: rows 64 bytes apart in bank space
constexpr int ST_NW = 15;     // consumer warps: the split and the three MMA chains of a tile are latency, not issue, bound
constexpr int ST_THREADS = 32 * (1 + ST_NW);

__global__ void __launch_bounds__(ST_THREADS, 1) scan_tf32_kernel(const ScanParams p) {
    extern __shared__ __align__(128) uint8_t sm[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint32_t sbase = smem_u32(sm);
    const int ring_bytes = p.nstage * p.stage_stride;
    const int nchunk = p.iters;          // 16-column chunks per row
    const int kq = nchunk * 16;
    const int qpitch = kq + ST_QPAD;     // floats
    float* sqh = reinterpret_cast<float*>(sm + ring_bytes);      // [8][qpitch] hi parts
    float* sql = sqh + SM_NQ * qpitch;                           // [8][qpitch] lo parts
    const int qbytes = 2 * SM_NQ * qpitch * 4;
    const uint32_t bar_full = sbase + ring_bytes + qbytes;
    const uint32_t bar_empty = bar_full + SM_MAX_STAGES * 8;
    volatile int* abort_flag =
            reinterpret_cast<volatile int*>(sm + ring_bytes + qbytes + 2 * SM_MAX_STAGES * 8);
    const int kext = (p.d + 3) & ~3;     // floats of a row that are read (zero padded by the store)

    for (int i = threadIdx.x; i < SM_NQ * qpitch; i += ST_THREADS) {
        const int qi = i / qpitch;
        const int j = i - qi * qpitch;
        float v = 0.f;
        if (qi < p.nq && j < p.d) v = p.queries[(int64_t)qi * p.d + j];
        const float hi = __uint_as_float(to_tf32(v));
        sqh[i] = hi;
        sql[i] = __uint_as_float(to_tf32(v - hi));
    }
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < p.nstage; s++) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, ST_NW);
        }
        mbar_fence_init();
    }
    __syncthreads();

    const int64_t nrows_total = p.col1 - p.col0;
    const int64_t nchunks = ceil_div64(nrows_total, p.stage_rows);
    const uint8_t* base = reinterpret_cast<const uint8_t*>(p.rows);
    const bool l2 = p.metric == B200F_METRIC_L2;
    const uint32_t norm_off = (uint32_t)p.stage_rows * (uint32_t)p.pitch_bytes;   // norms of a stage, behind its rows

    float lk[SM_NQ];
    int li[SM_NQ];
    float thr[SM_NQ];
    int thr_id[SM_NQ];
#pragma unroll
    for (int qi = 0; qi < SM_NQ; qi++) {
        lk[qi] = CUDART_INF_F;
        li[qi] = -1;
        thr[qi] = CUDART_INF_F;
        thr_id[qi] = -1;
    }

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
                if (!mbar_wait_bounded(bar_empty + stage * 8, phase ^ 1, abort_flag, p.status,
                                       kDevErrBarrierWait)) {
                    ok = false;
                    break;
                }
                const int64_t row0 = p.col0 + c * p.stage_rows;
                const int64_t nr = min((int64_t)p.stage_rows, p.col1 - row0);
                const uint32_t bytes = (uint32_t)(nr * p.pitch_bytes);
                // the stage's norms ride behind its rows: whole 16-byte pieces by bulk copy, the
                // up to three floats left of a last, ragged stage by plain stores (made visible
                // by the arrive that follows them)
                const uint32_t nbytes = l2 ? (uint32_t)(nr * 4) & ~15u : 0u;
                if (l2) {
                    float* sn = reinterpret_cast<float*>(sm + stage * p.stage_stride + norm_off);
                    for (int64_t r = nbytes / 4; r < nr; r++) sn[r] = __ldg(p.norms + row0 + r);
                }
                mbar_arrive_expect_tx(bar_full + stage * 8, bytes + nbytes);
                bulk_load(sbase + stage * p.stage_stride, base + row0 * p.pitch_bytes, bytes,
                          bar_full + stage * 8);
                if (nbytes)
                    bulk_load(sbase + stage * p.stage_stride + norm_off, p.norms + row0, nbytes,
                              bar_full + stage * 8);
                if (++stage == p.nstage) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (!ok) {  // let copies already issued land before shared memory goes away
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) {
                }
            }
        }
    } else {
        const int wc = warp - 1;
        const int g = lane >> 2;
        const int t = lane & 3;
        int stage = 0;
        uint32_t phase = 0;
        float mta, mtb;
        int mia, mib;
        auto refresh_bounds = [&]() {
            mta = t == 0 ? thr[0] : t == 1 ? thr[2] : t == 2 ? thr[4] : thr[6];
            mtb = t == 0 ? thr[1] : t == 1 ? thr[3] : t == 2 ? thr[5] : thr[7];
            mia = t == 0 ? thr_id[0] : t == 1 ? thr_id[2] : t == 2 ? thr_id[4] : thr_id[6];
            mib = t == 0 ? thr_id[1] : t == 1 ? thr_id[3] : t == 2 ? thr_id[5] : thr_id[7];
            if (2 * t >= p.nq) mta = -CUDART_INF_F;
            if (2 * t + 1 >= p.nq) mtb = -CUDART_INF_F;
        };
        refresh_bounds();
        const uint32_t bh_row = sbase + ring_bytes + (uint32_t)(g * qpitch * 4) + t * 16;
        const uint32_t bl_row = bh_row + (uint32_t)(SM_NQ * qpitch * 4);
        // A stage of wide rows holds fewer 16-row tiles than there are consumer warps: the first
        // tile's owner moves on by that many warps from stage to stage, so all of them work.
        const int tiles_full = p.stage_rows >> 4;
        int shift = 0;
        for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
            const bool w = mbar_wait_bounded(bar_full + stage * 8, phase, abort_flag, p.status,
                                             kDevErrBarrierWait);
            if (!__all_sync(FULL, w)) break;
            const int64_t row0 = p.col0 + c * p.stage_rows;
            const int nr = (int)min((int64_t)p.stage_rows, p.col1 - row0);
            const uint32_t sstage = sbase + stage * p.stage_stride;
            const float* snorm = reinterpret_cast<const float*>(sm + stage * p.stage_stride + norm_off);
            const int ntiles = (nr + 15) >> 4;
            for (int tile = (wc - shift + ST_NW) % ST_NW; tile < ntiles; tile += ST_NW) {
                const int r0 = tile * 16 + g;      // local rows of this lane
                const int r1 = r0 + 8;
                const bool v0 = r0 < nr, v1 = r1 < nr;
                float n0 = 0.f, n1 = 0.f;
                if (l2) {
                    if (v0) n0 = snorm[r0];
                    if (v1) n1 = snorm[r1];
                }
                const uint32_t a_row0 = sstage + (uint32_t)r0 * (uint32_t)p.pitch_bytes + t * 16;
                const uint32_t a_row1 = sstage + (uint32_t)r1 * (uint32_t)p.pitch_bytes + t * 16;
                // one accumulator per product kind: three short dependent MMA chains, not one long
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                float acc_lh[4] = {0.f, 0.f, 0.f, 0.f};
                float acc_hl[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
                for (int ch = 0; ch < nchunk; ch++) {
                    const bool kv = ch * 16 + t * 4 < kext;  // beyond the row: the next row's bytes
                    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = make_uint4(0, 0, 0, 0);
                    if (kv && v0) x0 = lds128(a_row0 + ch * 64);
                    if (kv && v1) x1 = lds128(a_row1 + ch * 64);
                    const uint4 qh = lds128(bh_row + ch * 64);
                    const uint4 ql = lds128(bl_row + ch * 64);
                    const uint32_t xs0[4] = {x0.x, x0.y, x0.z, x0.w};
                    const uint32_t xs1[4] = {x1.x, x1.y, x1.z, x1.w};
                    uint32_t h0[4], l0[4], h1[4], l1[4];
                    // hi = the value cut to tf32's 10 mantissa bits (a mask: the MMA reads no more of
                    // its operands anyway), lo = the exact remainder, of which the MMA again reads
                    // the top 10 bits: 2^-21 of the value is left out, as with rounded halves, for
                    // two instructions per element instead of three
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        h0[e] = xs0[e] & 0xffffe000u;
                        h1[e] = xs1[e] & 0xffffe000u;
                        l0[e] = __float_as_uint(__uint_as_float(xs0[e]) - __uint_as_float(h0[e]));
                        l1[e] = __float_as_uint(__uint_as_float(xs1[e]) - __uint_as_float(h1[e]));
                    }
                    // A fragment: a0 = row g slot t, a1 = row g+8 slot t, a2 = row g slot t+4,
                    // a3 = row g+8 slot t+4
                    mma1688_tf32(acc_lh, l0[0], l1[0], l0[1], l1[1], qh.x, qh.y);
                    mma1688_tf32(acc_hl, h0[0], h1[0], h0[1], h1[1], ql.x, ql.y);
                    mma1688_tf32(acc, h0[0], h1[0], h0[1], h1[1], qh.x, qh.y);
                    mma1688_tf32(acc_lh, l0[2], l1[2], l0[3], l1[3], qh.z, qh.w);
                    mma1688_tf32(acc_hl, h0[2], h1[2], h0[3], h1[3], ql.z, ql.w);
                    mma1688_tf32(acc, h0[2], h1[2], h0[3], h1[3], qh.z, qh.w);
                }
#pragma unroll
                for (int e = 0; e < 4; e++) acc[e] += acc_lh[e] + acc_hl[e];
                // acc[0]: (row r0, query 2t)  acc[1]: (r0, 2t+1)  acc[2]: (r1, 2t)  acc[3]: (r1, 2t+1)
                float key[4];
                key[0] = l2 ? fmaf(-2.f, acc[0], n0) : -acc[0];
                key[1] = l2 ? fmaf(-2.f, acc[1], n0) : -acc[1];
                key[2] = l2 ? fmaf(-2.f, acc[2], n1) : -acc[2];
                key[3] = l2 ? fmaf(-2.f, acc[3], n1) : -acc[3];
                // one vote tells whether the tile has a candidate at all; if so, one vote per accumulator
                // register: bit l of mj[j] = lane l's key j is a candidate (lane 4g + t holds query 2t
                // in keys 0 / 2 and query 2t + 1 in keys 1 / 3)
                const int row_a = (int)(row0 + r0), row_b = (int)(row0 + r1);
                const bool h0 = v0 && before(key[0], row_a, mta, mia), h1 = v0 && before(key[1], row_a, mtb, mib);
                const bool h2 = v1 && before(key[2], row_b, mta, mia), h3 = v1 && before(key[3], row_b, mtb, mib);
                if (!__any_sync(FULL, h0 || h1 || h2 || h3)) continue;  // the usual case: nothing for any query
                unsigned mj[4];
                mj[0] = __ballot_sync(FULL, h0);
                mj[1] = __ballot_sync(FULL, h1);
                mj[2] = __ballot_sync(FULL, h2);
                mj[3] = __ballot_sync(FULL, h3);
#pragma unroll
                for (int qi = 0; qi < SM_NQ; qi++) {
                    if (qi >= p.nq) break;
                    const unsigned lanes_q = 0x11111111u << (qi >> 1);   // the lanes with t = qi / 2
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const float kk = key[2 * h + (qi & 1)];
                        const int row = h ? row_b : row_a;
                        unsigned m = mj[2 * h + (qi & 1)] & lanes_q;
                        while (m) {
                            const int src = __ffs(m) - 1;
                            m &= m - 1;
                            const float s = __shfl_sync(FULL, kk, src);
                            const int id = __shfl_sync(FULL, row, src);
                            if (before(s, id, thr[qi], thr_id[qi])) {
                                warp_insert(lk[qi], li[qi], s, id, lane);
                                thr[qi] = __shfl_sync(FULL, lk[qi], p.k - 1);
                                thr_id[qi] = __shfl_sync(FULL, li[qi], p.k - 1);
                            }
                        }
                    }
                }
                refresh_bounds();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + stage * 8);
            shift = (shift + tiles_full) % ST_NW;
            if (++stage == p.nstage) {
                stage = 0;
                phase ^= 1;
            }
        }
    }

    // CTA merge in the (now idle) ring memory, as in scan_mma_kernel
    __syncthreads();
    float* mk = reinterpret_cast<float*>(sm);                        // [ST_NW][SM_NQ][32]
    int* mi = reinterpret_cast<int*>(sm) + ST_NW * SM_NQ * 32;
    if (warp > 0) {
#pragma unroll
        for (int qi = 0; qi < SM_NQ; qi++) {
            mk[((warp - 1) * SM_NQ + qi) * 32 + lane] = lk[qi];
            mi[((warp - 1) * SM_NQ + qi) * 32 + lane] = li[qi];
        }
    }
    __syncthreads();
    if (warp >= 1 && warp - 1 < p.nq) {
        const int qi = warp - 1;
        float k0 = mk[qi * 32 + lane];
        int i0 = mi[qi * 32 + lane];
        float tk = __shfl_sync(FULL, k0, p.k - 1);
        int tid = __shfl_sync(FULL, i0, p.k - 1);
        for (int w2 = 1; w2 < ST_NW; w2++) {
            for (int j = 0; j < p.k; j++) {
                const float s = mk[(w2 * SM_NQ + qi) * 32 + j];
                const int id = mi[(w2 * SM_NQ + qi) * 32 + j];
                if (id < 0 || !before(s, id, tk, tid)) break;
                warp_insert(k0, i0, s, id, lane);
                tk = __shfl_sync(FULL, k0, p.k - 1);
                tid = __shfl_sync(FULL, i0, p.k - 1);
            }
        }
        if (lane < p.k) {
            const int64_t o = ((int64_t)qi * gridDim.x + blockIdx.x) * p.k + lane;
            p.part_key[o] = k0;
            p.part_idx[o] = i0;
        }
    }
}

// Stage geometry of the FP32 streaming pipeline; false when it does not apply.
bool plan_stream_f32(ScanParams& p, int d) {
    if ((p.pitch_bytes % 16) != 0 || (reinterpret_cast<uintptr_t>(p.rows) & 15) != 0) return false;
    if (p.norms && (reinterpret_cast<uintptr_t>(p.norms) & 15) != 0) return false;
    if ((int64_t)((d + 3) & ~3) * 4 > p.pitch_bytes) return false;
    p.norm_cols = 0;
    p.iters = (d + 15) / 16;                    // 16-column chunks
    int64_t rows = (36 * 1024) / p.pitch_bytes; // ~36 KiB per stage
    rows = rows / 16 * 16;
    if (rows < 16) rows = 16;
    if (rows > 16 * ST_NW * 2) rows = 16 * ST_NW * 2;
    p.stage_rows = (int)rows;
    p.rb = 16;
    p.stage_stride = (int)round_up64((int64_t)p.stage_rows * (p.pitch_bytes + 4) + 64, 128);   // rows, then their norms
    const int64_t fixed = (int64_t)2 * SM_NQ * (p.iters * 16 + ST_QPAD) * 4 + 2 * SM_MAX_STAGES * 8 + 16;
    int64_t ns = (220 * 1024 - fixed) / p.stage_stride;
    if (ns > SM_MAX_STAGES) ns = SM_MAX_STAGES;
    p.nstage = (int)ns;
    // the CTA merge reuses the ring: SM_NW * SM_NQ * 32 (key, id) pairs
    return ns >= 3 && (int64_t)p.nstage * p.stage_stride >= (int64_t)ST_NW * SM_NQ * 32 * 8;
}

size_t scan_smem_bytes(int nq_t, int qstride) {
    size_t a = (size_t)nq_t * qstride * 4;
    size_t b = (size_t)SCAN_WARPS * nq_t * 32 * 8;
    return a > b ? a : b;
}

void fill_geometry(ScanParams& p, int storage, int d, int64_t row_pitch, int norm_cols, int lpr_cap) {
    const int E = storage == B200F_STORAGE_F32 ? 4 : 8;
    const int es = storage == B200F_STORAGE_F32 ? 4 : 2;
    p.pitch_bytes = row_pitch * es;
    p.norm_cols = (norm_cols && storage != B200F_STORAGE_F32) ? 1 : 0;
    p.C = (d + E - 1) / E;  // data pieces; the norm piece (if any) follows them in the row
    if (storage == B200F_STORAGE_F16) {
        p.nscale[0] = 4096.f; p.nscale[1] = 2.f; p.nscale[2] = 9.765625e-4f; p.nscale[3] = 4.76837158203125e-7f;
    } else {
        p.nscale[0] = 1.f; p.nscale[1] = 1.f; p.nscale[2] = 1.f; p.nscale[3] = 0.f;
    }
    // lanes per row: at most lpr_cap (8: a warp step covers at least 4 rows and the shuffle
    // reduction has 3 levels; with 32 lanes on one row the reduction and the candidate votes
    // cost more instructions than the dot products).
    int lpr = 1;
    while (lpr < p.C && lpr < lpr_cap) lpr <<= 1;
    p.lpr = lpr;
    p.iters = (p.C + lpr - 1) / lpr;
    p.qstride = p.C * E;
}

template <int STORAGE, bool STORE>
int launch_nq(const ScanParams& p, int grid, size_t smem, cudaStream_t stream) {
#define B200F_SCAN_CASE(NQ)                                                                      \
    {                                                                                            \
        if (smem > 48 * 1024)                                                                    \
            B200F_CUDA_TRY(cudaFuncSetAttribute(scan_kernel<STORAGE, NQ, STORE>,                 \
                                                cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                                (int)smem));                                     \
        main_kernel_begin(stream);                                                               \
        scan_kernel<STORAGE, NQ, STORE><<<grid, SCAN_THREADS, smem, stream>>>(p);                \
        main_kernel_end(stream);                                                                 \
        count_launch();                                                                          \
    }
    if (p.nq == 1) B200F_SCAN_CASE(1)
    else if (p.nq == 2) B200F_SCAN_CASE(2)
    else B200F_SCAN_CASE(4)
#undef B200F_SCAN_CASE
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

template <bool STORE>
int launch_storage(const ScanParams& p, int storage, int grid, cudaStream_t stream) {
    const int nq_t = p.nq == 1 ? 1 : (p.nq == 2 ? 2 : 4);
    const size_t smem = scan_smem_bytes(nq_t, p.qstride);
    if (smem > 200 * 1024) return B200F_ERR_UNSUPPORTED;
    switch (storage) {
        case B200F_STORAGE_F32: return launch_nq<B200F_STORAGE_F32, STORE>(p, grid, smem, stream);
        case B200F_STORAGE_F16: return launch_nq<B200F_STORAGE_F16, STORE>(p, grid, smem, stream);
        case B200F_STORAGE_BF16: return launch_nq<B200F_STORAGE_BF16, STORE>(p, grid, smem, stream);
    }
    return B200F_ERR_BAD_ARG;
}


// Stage geometry of the streaming pipeline; returns false when it does not apply.
bool plan_stream(ScanParams& p, int storage, int d, int norm_cols) {
    if (storage == B200F_STORAGE_F32 || (p.pitch_bytes % 16) != 0) return false;
    const int d8 = (d + 7) & ~7;
    const int kext = d8 + (norm_cols ? 8 : 0);
    p.norm_cols = norm_cols ? 1 : 0;
    p.iters = (kext + 31) / 32;                 // 32-column chunks
    int64_t rows = (36 * 1024) / p.pitch_bytes; // ~36 KiB per stage
    rows = rows / 16 * 16;
    if (rows < 16) rows = 16;
    if (rows > 256) rows = 256;
    p.stage_rows = (int)rows;
    p.rb = 16;
    p.stage_stride = (int)round_up64((int64_t)p.stage_rows * p.pitch_bytes + 64, 128);
    const int64_t fixed = (int64_t)SM_NQ * p.iters * 32 * 2 + 2 * SM_MAX_STAGES * 8 + 16;
    int64_t ns = (220 * 1024 - fixed) / p.stage_stride;
    if (ns > SM_MAX_STAGES) ns = SM_MAX_STAGES;
    p.nstage = (int)ns;
    return ns >= 3;
}

int lanes_per_row_cap(int64_t nq) { (void)nq; return 8; }

// CTAs of scan_kernel that are resident per SM (its launch bounds): the grid is one full wave of
// them.  A grid of 4 per SM with 3 resident ran a second, third-empty wave: measured 66 % of the
// DRAM peak in the profile of one fp32 query where one wave reaches more.
int resident_ctas(int64_t nq, int storage, bool store) {
    const int64_t group = nq < 4 ? nq : 4;   // queries per launch: 1, 2 or 4 (three run as four)
    if (group >= 3) return 2;
    if (group == 2 && storage == B200F_STORAGE_F32 && !store) return 2;
    return 3;
}

int scan_grid(int64_t nrows, int d, int storage, int sm_count, int lpr_cap, int per_sm) {
    ScanParams t{};
    fill_geometry(t, storage, d, d, 0, lpr_cap);
    const int rows_per_block = (32 / t.lpr) * SCAN_U;
    const int64_t nblocks = ceil_div64(nrows, rows_per_block);
    int64_t g = ceil_div64(nblocks, SCAN_WARPS);
    const int64_t cap = (int64_t)sm_count * per_sm;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace

ScanPlan plan_scan(int64_t nq, int64_t nb, int d, int storage, int sm_count) {
    ScanPlan s;
    s.lpr_cap = lanes_per_row_cap(nq);  // of the whole search: every query group uses the same geometry
    s.grid = scan_grid(nb, d, storage, sm_count, s.lpr_cap, resident_ctas(nq, storage, false));
    s.threads = SCAN_THREADS;
    return s;
}

int launch_scan_topk(const B200FSearchArgs& a, const ScanPlan& plan, float* part_key,
                     int32_t* part_idx, int* out_P, bool stream_f32, cudaStream_t stream) {
    if (a.nq < 1 || a.nq > 8 || a.k < 1 || a.k > 32) return B200F_ERR_UNSUPPORTED;
    ScanParams p{};
    fill_geometry(p, a.storage, a.d, a.row_pitch, a.metric == B200F_METRIC_L2 ? a.norm_cols : 0,
                  plan.lpr_cap);
    p.queries = a.queries;
    p.rows = a.rows;
    p.norms = a.norms;
    p.nb = a.nb;
    p.col0 = 0;
    p.col1 = a.nb;
    p.d = a.d;
    p.nq = (int)a.nq;
    p.k = a.k;
    p.metric = a.metric;
    p.part_key = part_key;
    p.part_idx = part_idx;
    p.status = a.status;
    const int sm = cached_sm_count();
    {
        ScanParams ps = p;
        const int nc = (a.metric == B200F_METRIC_L2 && a.norm_cols) ? 1 : 0;
        if ((a.metric != B200F_METRIC_L2 || nc) && plan_stream(ps, a.storage, a.d, nc) &&
            a.nb >= (int64_t)ps.stage_rows * sm) {
            // streaming pipeline: one CTA per SM, one partial list per CTA
            const int64_t nchunks = ceil_div64(a.nb, ps.stage_rows);
            const int grid = (int)(nchunks < sm ? nchunks : sm);
            const size_t smem = (size_t)ps.nstage * ps.stage_stride + (size_t)SM_NQ * ps.iters * 32 * 2 +
                                2 * SM_MAX_STAGES * 8 + 16;
            *out_P = grid;
            // macro: the kernel is a template over (format, consumer warps)
#define B200F_SCAN_MMA(BF, NW)                                                                            \
    {                                                                                                     \
        B200F_CUDA_TRY(cudaFuncSetAttribute(scan_mma_kernel<BF, NW>,                                      \
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));     \
        main_kernel_begin(stream);                                                                        \
        scan_mma_kernel<BF, NW><<<grid, 32 * (1 + NW), smem, stream>>>(ps);                               \
    }
            const bool bf = a.storage == B200F_STORAGE_BF16;
            if (a.nq <= 2) {
                if (bf) B200F_SCAN_MMA(true, 8) else B200F_SCAN_MMA(false, 8)
            } else {
                if (bf) B200F_SCAN_MMA(true, SM_NW_MANY) else B200F_SCAN_MMA(false, SM_NW_MANY)
            }
#undef B200F_SCAN_MMA
            main_kernel_end(stream);
            count_launch();
            B200F_LAUNCH_CHECK();
            return B200F_OK;
        }
    }
    if (a.storage == B200F_STORAGE_F32 && stream_f32 && (a.metric != B200F_METRIC_L2 || a.norms)) {
        ScanParams ps = p;
        // no minimum shard size: a row's distance must not depend on how the rows are sharded,
        // and this kernel and the FMA kernel round differently
        if (plan_stream_f32(ps, a.d)) {
            const int64_t nchunks = ceil_div64(a.nb, ps.stage_rows);
            const int grid = (int)(nchunks < sm ? nchunks : sm);
            const size_t smem = (size_t)ps.nstage * ps.stage_stride +
                                (size_t)2 * SM_NQ * (ps.iters * 16 + ST_QPAD) * 4 + 2 * SM_MAX_STAGES * 8 + 16;
            *out_P = grid;
            B200F_CUDA_TRY(cudaFuncSetAttribute(scan_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                (int)smem));
            main_kernel_begin(stream);
            scan_tf32_kernel<<<grid, ST_THREADS, smem, stream>>>(ps);
            main_kernel_end(stream);
            count_launch();
            B200F_LAUNCH_CHECK();
            return B200F_OK;
        }
    }
    if (a.nq > 4) return B200F_ERR_UNSUPPORTED;
    *out_P = plan.grid;
    return launch_storage<false>(p, a.storage, plan.grid, stream);
}

int launch_scan_store(const B200FSearchArgs& a, int64_t col0, int64_t ncols, float* out, int64_t ld,
                      int sm_count, cudaStream_t stream) {
    if (a.nq < 1 || a.nq > 4) return B200F_ERR_UNSUPPORTED;
    if (ncols <= 0) return B200F_OK;
    ScanParams p{};
    fill_geometry(p, a.storage, a.d, a.row_pitch, a.metric == B200F_METRIC_L2 ? a.norm_cols : 0,
                  lanes_per_row_cap(a.nq));
    p.queries = a.queries;
    p.rows = a.rows;
    p.norms = a.norms;
    p.nb = a.nb;
    p.col0 = col0;
    p.col1 = col0 + ncols;
    p.d = a.d;
    p.nq = (int)a.nq;
    p.k = 1;
    p.metric = a.metric;
    p.out = out;
    p.ld = ld;
    return launch_storage<true>(p, a.storage,
                                scan_grid(ncols, a.d, a.storage, sm_count, lanes_per_row_cap(a.nq),
                                          resident_ctas(a.nq, a.storage, true)),
                                stream);
}

}  // namespace b200f
