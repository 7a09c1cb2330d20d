// Selection and merge kernels.
//
// Replaces warp_select_min/max (shaders/warp_select.metal:11-114), block_select_min/max
// (shaders/block_select.metal:111-274), their dispatch (src/MetalSelect.mm:34-108) and the
// final list merge inside the fused kernels (shaders/fused_l2_topk.metal:88-131).
//
// Building blocks:
//  * merge_small: k <= 32.  One CTA per query; each warp folds a subset of sorted input
//    lists into a sorted warp list (lane j = rank j) by ballot + shuffle insertion with
//    early exit, then warp 0 folds the warp lists.
//  * sort_select: any k <= 4096.  One CTA per query streams candidates, keeps those under
//    the current k-th best in a shared-memory buffer of 8192 packed (key, payload) words
//    and compacts with a bitonic sort whenever the buffer could overflow.  Results are
//    exact for every k (the reference's block_select keeps only 8 real results per row).
//    Sources: a key matrix chunk, sorted lists of other ranks, the fused kernel's 32-entry
//    lists, or a threshold-filtered candidate buffer; the last two also report rows whose
//    result is not proven exact.
//  * select_small: k <= 32 from a candidate buffer, one warp per query.
//  * compact_rows / gather_rows: the rows to redo, counted and gathered on the device.
//
// Keys are "smaller is better" everywhere: L2 key = distance, inner product key = -dot.
// Ties go to the lower id.
#include "common.cuh"

namespace b200f {

namespace {

constexpr unsigned FULL = 0xffffffffu;

// ---------------------------------------------------------------------------------------
// merge_small
// ---------------------------------------------------------------------------------------
constexpr int MS_THREADS = 256;
constexpr int MS_WARPS = MS_THREADS / 32;

template <typename IdT>
__device__ __forceinline__ bool before_id(float ka, IdT ia, float kb, IdT ib) {
    // negative ids are empty slots and sort last among equal keys
    typedef typename std::conditional<sizeof(IdT) == 8, unsigned long long, unsigned>::type U;
    return (ka < kb) || (ka == kb && (U)ia < (U)ib);
}

template <typename IdT>
__device__ __forceinline__ IdT shfl_id(IdT v, int src) {
    if (sizeof(IdT) == 8) {
        unsigned long long u = (unsigned long long)v;
        unsigned lo = __shfl_sync(FULL, (unsigned)u, src);
        unsigned hi = __shfl_sync(FULL, (unsigned)(u >> 32), src);
        return (IdT)(((unsigned long long)hi << 32) | lo);
    } else {
        return (IdT)__shfl_sync(FULL, (int)v, src);
    }
}
template <typename IdT>
__device__ __forceinline__ IdT shfl_up_id(IdT v) {
    if (sizeof(IdT) == 8) {
        unsigned long long u = (unsigned long long)v;
        unsigned lo = __shfl_up_sync(FULL, (unsigned)u, 1);
        unsigned hi = __shfl_up_sync(FULL, (unsigned)(u >> 32), 1);
        return (IdT)(((unsigned long long)hi << 32) | lo);
    } else {
        return (IdT)__shfl_up_sync(FULL, (int)v, 1);
    }
}

template <typename IdT>
__device__ __forceinline__ void warp_insert_id(float& lk, IdT& li, float s, IdT id, int lane) {
    const bool stays = before_id<IdT>(lk, li, s, id);
    const int pos = __popc(__ballot_sync(FULL, stays));
    const float upk = __shfl_up_sync(FULL, lk, 1);
    const IdT upi = shfl_up_id<IdT>(li);
    if (lane == pos) {
        lk = s;
        li = id;
    } else if (lane > pos) {
        lk = upk;
        li = upi;
    }
}

// Input list p of query q lives at in_key/in_id + (q*q_stride + p*p_stride) (k entries).
// key = key_sign * in_key.  Output: dist = out_sign * key + qnorm[q] (clamped at 0 when
// clamp), label = id + label_base; empty slots give (pad, -1).
template <typename IdT>
struct MergeSmallParams {
    const float* in_key;
    const IdT* in_id;
    int64_t q_stride, p_stride;   // elements: between queries, between lists (keys)
    int64_t p_stride_id;          // between lists (ids)
    int P;
    int64_t nq;
    const int* nq_dev;        // optional: live rows (<= nq), read on the device
    const int32_t* row_map;   // optional: lists of row j belong to query row_map[j]
    int k;
    float key_sign;
    float out_sign;
    const float* qnorm;
    int clamp;
    float pad;
    int64_t label_base;
    float* out_dist;
    int64_t* out_labels;
};

template <typename IdT>
__global__ void __launch_bounds__(MS_THREADS) merge_small_kernel(const MergeSmallParams<IdT> p) {
    __shared__ float sk[MS_WARPS][32];
    __shared__ IdT si[MS_WARPS][32];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t nq_live = p.nq_dev ? min((int64_t)*p.nq_dev, p.nq) : p.nq;
    for (int64_t q = blockIdx.x; q < nq_live; q += gridDim.x) {
        float lk = CUDART_INF_F;
        IdT li = (IdT)-1;
        float thr = CUDART_INF_F;
        IdT thr_id = (IdT)-1;
        for (int l = warp; l < p.P; l += MS_WARPS) {
            const float* lkey = p.in_key + q * p.q_stride + (int64_t)l * p.p_stride;
            const IdT* lid = p.in_id + q * p.q_stride + (int64_t)l * p.p_stride_id;
            // lane j prefetches entry j, entries are then consumed in order
            float myk = CUDART_INF_F;
            IdT myi = (IdT)-1;
            if (lane < p.k) {
                myk = p.key_sign * lkey[lane];
                myi = lid[lane];
            }
            for (int j = 0; j < p.k; j++) {
                const float s = __shfl_sync(FULL, myk, j);
                const IdT id = shfl_id<IdT>(myi, j);
                if (id < 0 || !before_id<IdT>(s, id, thr, thr_id)) break;
                warp_insert_id<IdT>(lk, li, s, id, lane);
                thr = __shfl_sync(FULL, lk, p.k - 1);
                thr_id = shfl_id<IdT>(li, p.k - 1);
            }
        }
        __syncthreads();  // previous query's shared lists fully consumed
        sk[warp][lane] = lk;
        si[warp][lane] = li;
        __syncthreads();
        if (warp == 0) {
            for (int w = 1; w < MS_WARPS; w++) {
                for (int j = 0; j < p.k; j++) {
                    const float s = sk[w][j];
                    const IdT id = si[w][j];
                    if (id < 0 || !before_id<IdT>(s, id, thr, thr_id)) break;
                    warp_insert_id<IdT>(lk, li, s, id, lane);
                    thr = __shfl_sync(FULL, lk, p.k - 1);
                    thr_id = shfl_id<IdT>(li, p.k - 1);
                }
            }
            if (lane < p.k) {
                const int64_t qo = p.row_map ? (int64_t)p.row_map[q] : q;
                float dist = p.pad;
                int64_t label = -1;
                if (li >= 0) {
                    dist = p.out_sign * lk + (p.qnorm ? p.qnorm[qo] : 0.f);
                    if (p.clamp && dist < 0.f) dist = 0.f;
                    label = (int64_t)li + p.label_base;
                }
                p.out_dist[qo * p.k + lane] = dist;
                if (p.out_labels) p.out_labels[qo * p.k + lane] = label;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// sort_select
// ---------------------------------------------------------------------------------------
constexpr int SS_THREADS = 1024;
constexpr int SS_CAP = 8192;
constexpr int SS_ITEMS = 4;
constexpr int SS_BATCH = SS_THREADS * SS_ITEMS;  // 4096 candidates per batch
constexpr uint64_t SS_EMPTY = ~0ull;

enum { SRC_MATRIX = 0, SRC_LISTS = 1, SRC_PARTS = 2 };

struct SortSelectParams {
    // SRC_MATRIX: keys[q*ld + c], c in [0, ncand); payload = col0 + c
    // SRC_LISTS : keys[(l*nq + q)*k + j] over l in [0, P); payload = l*k + j; labels != -1 live
    // SRC_PARTS : keys[q*ld + c], ids part_idx[same] (-1 = empty); payload = id.  Either P
    //             sorted lists of 32 entries (ld = 32 P), or, with cand_cnt, an unordered
    //             candidate buffer of min(cand_cnt[q], ld) entries
    const float* keys;
    const int64_t* labels;
    int64_t ld;
    int64_t ncand;
    int64_t col0;
    int64_t list_stride_k;   // SRC_LISTS: elements between consecutive lists in keys
    int64_t list_stride_l;   // SRC_LISTS: elements between consecutive lists in labels
    int P;
    int64_t nq;
    const int* nq_dev;    // optional: live rows (<= nq), read on the device
    const int32_t* part_idx;  // SRC_PARTS
    const int32_t* cand_cnt;  // SRC_PARTS: candidates counted per row (may exceed ld: overflow)
    int64_t nb_total;     // SRC_PARTS with cand_cnt: rows in the shard
    int32_t* dirty;       // SRC_PARTS: per row, 1 when the result is not proven exact
    int k;
    float key_sign;       // key = key_sign * input
    int has_prev;
    float* run_key;       // [nq][k] in/out running lists (may be null when finalising directly)
    int32_t* run_idx;
    // finalisation (out_dist != null): dist = out_sign*key + qnorm[q]
    float out_sign;
    const float* qnorm;
    int clamp;
    float pad;
    int64_t label_base;
    float* out_dist;
    int64_t* out_labels;
};

__device__ __forceinline__ uint64_t pack(float key, uint32_t payload) {
    return ((uint64_t)float_to_ordered(key) << 32) | payload;
}

// ascending bitonic sort of buf[0..n), n a power of two, all threads of the CTA
__device__ void bitonic_sort(uint64_t* buf, int n) {
    for (int size = 2; size <= n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int i = threadIdx.x; i < (n >> 1); i += blockDim.x) {
                const int pos = 2 * i - (i & (stride - 1));
                const uint64_t a = buf[pos];
                const uint64_t b = buf[pos + stride];
                const bool up = (pos & size) == 0;
                if ((a > b) == up) {
                    buf[pos] = b;
                    buf[pos + stride] = a;
                }
            }
        }
    }
    __syncthreads();
}

template <int SRC>
__global__ void __launch_bounds__(SS_THREADS) sort_select_kernel(const SortSelectParams p) {
    extern __shared__ __align__(16) uint64_t buf[];  // SS_CAP entries
    __shared__ int s_count;
    __shared__ uint64_t s_thr;
    __shared__ int s_pending[2];
    const int tid = threadIdx.x;
    if (tid == 0) {
        s_pending[0] = 0;
        s_pending[1] = 0;
    }

    const int64_t nq_live = p.nq_dev ? min((int64_t)*p.nq_dev, p.nq) : p.nq;
    for (int64_t q = blockIdx.x; q < nq_live; q += gridDim.x) {
        __syncthreads();
        // the buffer is not cleared up front: slots past the live count are set to EMPTY
        // right before each sort that would read them
        if (tid == 0) {
            s_count = 0;
            s_thr = SS_EMPTY;
            s_pending[0] = 0;
            s_pending[1] = 0;
        }
        __syncthreads();
        if (p.has_prev) {
            for (int j = tid; j < p.k; j += SS_THREADS) {
                const int32_t id = p.run_idx[q * p.k + j];
                buf[j] = (id >= 0) ? pack(p.run_key[q * p.k + j], (uint32_t)id) : SS_EMPTY;
            }
            __syncthreads();
            if (tid == 0) {
                // live entries form a prefix of the sorted previous list
                int c = 0;
                // binary search for the first empty slot
                int lo = 0, hi = p.k;
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (buf[mid] != SS_EMPTY) lo = mid + 1; else hi = mid;
                }
                c = lo;
                s_count = c;
                s_thr = (c >= p.k) ? buf[p.k - 1] : SS_EMPTY;
            }
            __syncthreads();
        }

        int64_t total = (SRC == SRC_MATRIX) ? p.ncand : (SRC == SRC_LISTS) ? (int64_t)p.P * p.k : p.ld;
        if (SRC == SRC_PARTS && p.cand_cnt) total = min((int64_t)__ldg(p.cand_cnt + q), p.ld);
        // Merging result lists: equal keys must come out in label order, whichever list they
        // sit in (lists of interleaved row shards do not hold ascending label ranges).  Labels
        // below 2^32 ride in the low word of the sort key; should a row hold a larger one, its
        // ties fall back to list order.
        bool wide_labels = false;
        if (SRC == SRC_LISTS) {
            int big = 0;
            for (int64_t c = tid; c < total; c += SS_THREADS) {
                const int64_t l = c / p.k;
                const int64_t lab = __ldg(p.labels + l * p.list_stride_l + q * p.k + (c - l * p.k));
                big |= (lab >= 0 && (lab >> 32) != 0) ? 1 : 0;   // -1 marks an empty slot
            }
            wide_labels = __syncthreads_or(big) != 0;
        }
        // Wide streaming path (key matrix with 16-byte aligned rows): every thread loads
        // 8 x float4 = 32 columns up front, counts its hits against the current threshold, and
        // the CTA appends them after ONE count check per 32,768 columns.  Only when the buffer
        // could overflow (no threshold yet, or adversarial order) the batch is replayed in
        // eight 4,096-column steps with a compaction check before each.
        const bool wide = (SRC == SRC_MATRIX) && ((p.ld & 3) == 0) &&
                          ((reinterpret_cast<uintptr_t>(p.keys) & 15) == 0);
        int64_t b_start = 0;
        if (wide) {
            constexpr int WV = 8;
            constexpr int64_t WIDE = (int64_t)SS_THREADS * 4 * WV;
            const float* rowp = p.keys + q * p.ld;
            int par = 0;
            for (int64_t w0 = 0; w0 < total; w0 += WIDE) {
                float4 v[WV];
#pragma unroll
                for (int i = 0; i < WV; i++) {
                    const int64_t c = w0 + ((int64_t)i * SS_THREADS + tid) * 4;
                    if (c + 4 <= total) {
                        v[i] = __ldg(reinterpret_cast<const float4*>(rowp + c));
                    } else {
                        float t4[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) t4[e] = (c + e < total) ? __ldg(rowp + c + e) : CUDART_NAN_F;
                        v[i] = make_float4(t4[0], t4[1], t4[2], t4[3]);
                    }
                }
                const uint64_t thr0 = s_thr;
                const uint32_t thr_hi = (uint32_t)(thr0 >> 32);
                uint32_t hits = 0;
#pragma unroll
                for (int i = 0; i < WV; i++) {
                    const float e4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float key = p.key_sign * e4[e];
                        // NaN (also the out-of-range filler) never qualifies
                        const bool h = (key == key) && float_to_ordered(key) <= thr_hi;
                        hits |= (h ? 1u : 0u) << (i * 4 + e);
                    }
                }
                if (hits) atomicAdd(&s_pending[par], __popc(hits));
                __syncthreads();
                const int cnt = s_count;
                const int pend = s_pending[par];
                // the other counter belongs to the next batch: its last readers are behind the
                // previous batch's second barrier, its next writers behind the one below
                if (tid == 0) s_pending[par ^ 1] = 0;
                __syncthreads();
                if (cnt + pend <= SS_CAP) {
                    // fast path: room for every hit
                    while (hits) {
                        const int b = __ffs(hits) - 1;
                        hits &= hits - 1;
                        const int i = b >> 2, e = b & 3;
                        float val = 0.f;
#pragma unroll
                        for (int ii = 0; ii < WV; ii++) {
                            const float e4[4] = {v[ii].x, v[ii].y, v[ii].z, v[ii].w};
#pragma unroll
                            for (int ee = 0; ee < 4; ee++) val = (ii == i && ee == e) ? e4[ee] : val;
                        }
                        const int64_t c = w0 + ((int64_t)i * SS_THREADS + tid) * 4 + e;
                        const uint64_t w = pack(p.key_sign * val, (uint32_t)(p.col0 + c));
                        if (w < thr0) {
                            const int pos = atomicAdd(&s_count, 1);
                            buf[pos] = w;
                        }
                    }
                } else {
                    // replay in 4,096-column steps (vector i of every thread), compacting as needed
#pragma unroll
                    for (int i = 0; i < WV; i++) {
                        __syncthreads();
                        const int cnt2 = s_count;
                        __syncthreads();
                        if (cnt2 > SS_CAP - SS_BATCH) {
                            for (int j = cnt2 + tid; j < SS_CAP; j += SS_THREADS) buf[j] = SS_EMPTY;
                            bitonic_sort(buf, SS_CAP);
                            for (int j = p.k + tid; j < SS_CAP; j += SS_THREADS) buf[j] = SS_EMPTY;
                            if (tid == 0) {
                                s_count = p.k;
                                s_thr = buf[p.k - 1];
                            }
                            __syncthreads();
                        }
                        const uint64_t thr = s_thr;
                        const float e4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int64_t c = w0 + ((int64_t)i * SS_THREADS + tid) * 4 + e;
                            const float key = p.key_sign * e4[e];
                            if (c < total && key == key) {
                                const uint64_t w = pack(key, (uint32_t)(p.col0 + c));
                                if (w < thr) {
                                    const int pos = atomicAdd(&s_count, 1);
                                    buf[pos] = w;  // at most 4,096 appends per step
                                }
                            }
                        }
                    }
                }
                par ^= 1;
            }
            b_start = total;  // everything consumed
        }
        for (int64_t b0 = b_start; b0 < total; b0 += SS_BATCH) {
            // Every thread must take the same branch below: read the count between two
            // barriers, so that no thread of the next batch has appended yet.
            __syncthreads();
            const int cnt = s_count;
            __syncthreads();
            // make room: after compaction at most k <= 4096 entries remain
            if (cnt > SS_CAP - SS_BATCH) {
                for (int i = cnt + tid; i < SS_CAP; i += SS_THREADS) buf[i] = SS_EMPTY;
                bitonic_sort(buf, SS_CAP);
                for (int i = p.k + tid; i < SS_CAP; i += SS_THREADS) buf[i] = SS_EMPTY;
                if (tid == 0) {
                    s_count = p.k;
                    s_thr = buf[p.k - 1];
                }
                __syncthreads();
            }
            const uint64_t thr = s_thr;
#pragma unroll
            for (int it = 0; it < SS_ITEMS; it++) {
                const int64_t c = b0 + (int64_t)it * SS_THREADS + tid;
                if (c < total) {
                    float key;
                    uint32_t payload;
                    bool live = true;
                    if (SRC == SRC_MATRIX) {
                        key = p.key_sign * __ldg(p.keys + q * p.ld + c);
                        payload = (uint32_t)(p.col0 + c);
                    } else if (SRC == SRC_PARTS) {
                        const int64_t off = q * p.ld + c;
                        const int32_t id = __ldg(p.part_idx + off);
                        key = p.key_sign * __ldg(p.keys + off);
                        live = id >= 0;
                        payload = (uint32_t)id;
                    } else {
                        const int64_t l = c / p.k;
                        const int64_t j = c - l * p.k;
                        const int64_t off = q * p.k + j;
                        key = p.key_sign * __ldg(p.keys + l * p.list_stride_k + off);
                        const int64_t lab = __ldg(p.labels + l * p.list_stride_l + off);
                        live = lab >= 0;
                        payload = wide_labels ? (uint32_t)c : (uint32_t)lab;
                    }
                    const uint64_t w = pack(key, payload);
                    if (live && w < thr) {
                        const int pos = atomicAdd(&s_count, 1);
                        buf[pos] = w;  // pos < SS_CAP by construction
                    }
                }
            }
        }
        __syncthreads();
        // final ordering
        {
            const int cnt = s_count;
            int n = 64;
            while (n < cnt) n <<= 1;
            for (int i = cnt + tid; i < n; i += SS_THREADS) buf[i] = SS_EMPTY;
            bitonic_sort(buf, n);
        }
        for (int j = tid; j < p.k; j += SS_THREADS) {
            const uint64_t w = buf[j];
            const bool live = (w != SS_EMPTY) && j < s_count;
            const float key = ordered_to_float((uint32_t)(w >> 32));
            const uint32_t payload = (uint32_t)w;
            if (p.out_dist) {
                float dist = p.pad;
                int64_t label = -1;
                if (live) {
                    dist = p.out_sign * key + (p.qnorm ? p.qnorm[q] : 0.f);
                    if (p.clamp && dist < 0.f) dist = 0.f;
                    if (SRC != SRC_LISTS) {
                        label = (int64_t)payload + p.label_base;
                    } else if (!wide_labels) {
                        label = (int64_t)payload;
                    } else {
                        const int64_t l = payload / p.k;
                        const int64_t jj = payload - l * p.k;
                        label = p.labels[l * p.list_stride_l + q * p.k + jj];
                    }
                }
                p.out_dist[q * p.k + j] = dist;
                p.out_labels[q * p.k + j] = label;
            } else {
                p.run_key[q * p.k + j] = live ? key : CUDART_INF_F;
                p.run_idx[q * p.k + j] = live ? (int32_t)payload : -1;
            }
        }
        if (SRC == SRC_PARTS && p.dirty) {
            // Entries a list dropped sort behind its worst kept entry.  They cannot belong to
            // the result when that entry itself sorts behind the k-th selected candidate.
            const uint64_t kth = (s_count >= p.k) ? buf[p.k - 1] : SS_EMPTY;
            int bad = 0;
            if (p.cand_cnt) {
                // threshold-filtered candidates: exact when nothing overflowed and either k of
                // them were found or every row of the shard is a candidate
                const int64_t cnt = __ldg(p.cand_cnt + q);
                bad = (cnt > p.ld) || (cnt < p.k && cnt < p.nb_total);
            } else {
                for (int l = tid; l < p.P; l += SS_THREADS) {
                    const int64_t off = q * p.ld + (int64_t)l * 32 + 31;
                    const int32_t id = __ldg(p.part_idx + off);
                    if (id >= 0 && pack(p.key_sign * __ldg(p.keys + off), (uint32_t)id) <= kth) bad = 1;
                }
            }
            bad = __syncthreads_or(bad);
            if (tid == 0) p.dirty[q] = bad ? 1 : 0;
        }
    }
}

// k <= 32 from an unordered candidate buffer of a few hundred to a few thousand entries per
// row: one WARP per row.  The lanes read 32 candidates at a time; those that beat the current
// k-th best are inserted one after the other into the warp's sorted list (lane j = rank j).
// About 32 ln(n / 32) + 32 insertions per row; a 1024-thread bitonic sort per row would cost
// fifty barrier rounds for the same result.
constexpr int SEL_WARPS = 8;
__global__ void __launch_bounds__(SEL_WARPS * 32) select_small_kernel(const SortSelectParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * SEL_WARPS + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * SEL_WARPS;
    const int64_t nq_live = p.nq_dev ? min((int64_t)*p.nq_dev, p.nq) : p.nq;
    for (int64_t q = warp0; q < nq_live; q += nwarps) {
        const int64_t cnt = __ldg(p.cand_cnt + q);
        const int n = (int)min(cnt, p.ld);
        const float* keys = p.keys + q * p.ld;
        const int32_t* ids = p.part_idx + q * p.ld;
        float lk = CUDART_INF_F;
        int32_t li = -1;
        float thr = CUDART_INF_F;
        int32_t thr_id = -1;
        for (int base = 0; base < n; base += 32) {
            const int c = base + lane;
            const float key = c < n ? p.key_sign * __ldg(keys + c) : CUDART_INF_F;
            const int32_t id = c < n ? __ldg(ids + c) : -1;
            unsigned m = __ballot_sync(FULL, id >= 0 && before_id<int32_t>(key, id, thr, thr_id));
            while (m) {
                const int src = __ffs(m) - 1;
                m &= m - 1;
                const float s = __shfl_sync(FULL, key, src);
                const int32_t sid = __shfl_sync(FULL, id, src);
                if (before_id<int32_t>(s, sid, thr, thr_id)) {  // the bound moved since the ballot
                    warp_insert_id<int32_t>(lk, li, s, sid, lane);
                    thr = __shfl_sync(FULL, lk, p.k - 1);
                    thr_id = __shfl_sync(FULL, li, p.k - 1);
                }
            }
        }
        if (lane < p.k) {
            float dist = p.pad;
            int64_t label = -1;
            if (li >= 0) {
                dist = p.out_sign * lk + (p.qnorm ? p.qnorm[q] : 0.f);
                if (p.clamp && dist < 0.f) dist = 0.f;
                label = (int64_t)li + p.label_base;
            }
            p.out_dist[q * p.k + lane] = dist;
            p.out_labels[q * p.k + lane] = label;
        }
        if (lane == 0 && p.dirty) p.dirty[q] = ((cnt > p.ld) || (cnt < p.k && cnt < p.nb_total)) ? 1 : 0;
    }
}

// The r <= 32 smallest keys of a matrix row (the pilot sample of the threshold filter): one warp
// per row reads 128 columns at a time; a key under the current r-th best is inserted into the
// warp's sorted list (lane j = rank j).  About r ln(n / r) + r insertions per row.
__global__ void __launch_bounds__(SEL_WARPS * 32) select_keys_kernel(const float* __restrict__ keys, int64_t nq,
                                                                     int64_t ncols, int64_t ld, int r,
                                                                     float* __restrict__ out_key) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * SEL_WARPS + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * SEL_WARPS;
    const bool vec = ((ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(keys) & 15) == 0);
    for (int64_t q = warp0; q < nq; q += nwarps) {
        const float* row = keys + q * ld;
        float lk = CUDART_INF_F;
        float thr = CUDART_INF_F;
        for (int64_t base = 0; base < ncols; base += 128) {
            const int64_t c = base + lane * 4;
            float v[4];
            if (vec && c + 4 <= ncols) {
                const float4 f = __ldg(reinterpret_cast<const float4*>(row + c));
                v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; e++) v[e] = (c + e < ncols) ? __ldg(row + c + e) : CUDART_INF_F;
            }
#pragma unroll
            for (int e = 0; e < 4; e++) {
                unsigned m = __ballot_sync(FULL, v[e] < thr);   // NaN never qualifies
                while (m) {
                    const int src = __ffs(m) - 1;
                    m &= m - 1;
                    const float s = __shfl_sync(FULL, v[e], src);
                    if (s < thr) {   // the bound moved since the ballot
                        const int pos = __popc(__ballot_sync(FULL, lk <= s));
                        const float up = __shfl_up_sync(FULL, lk, 1);
                        if (lane == pos) lk = s;
                        else if (lane > pos) lk = up;
                        thr = __shfl_sync(FULL, lk, r - 1);
                    }
                }
            }
        }
        if (lane < r) out_key[q * r + lane] = lk;
    }
}

// rows[0 .. n) = ascending q with flag[q] != 0, n -> *count (one CTA)
__global__ void __launch_bounds__(1024) compact_rows_kernel(const int32_t* __restrict__ flag, int64_t nq,
                                                            int32_t* __restrict__ rows,
                                                            int32_t* __restrict__ count,
                                                            int32_t* __restrict__ count_copy) {
    __shared__ int s_warp[32];
    __shared__ int s_base;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_base = 0;
    __syncthreads();
    for (int64_t q0 = 0; q0 < nq; q0 += 1024) {
        const int64_t q = q0 + tid;
        const bool f = q < nq && flag[q] != 0;
        const unsigned b = __ballot_sync(FULL, f);
        if (lane == 0) s_warp[warp] = __popc(b);
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; w++) before += s_warp[w];
        const int base = s_base;
        if (f) rows[base + before + __popc(b & ((1u << lane) - 1u))] = (int32_t)q;
        __syncthreads();
        if (tid == 1023) s_base = base + before + __popc(b);
        __syncthreads();
    }
    if (tid == 0) {
        *count = s_base;
        if (count_copy) *count_copy = s_base;
    }
}

__global__ void gather_rows_kernel(const uint16_t* __restrict__ a, int npl, int64_t plane_stride,
                                   int64_t pitch, const int32_t* __restrict__ rows,
                                   const int32_t* __restrict__ count, uint16_t* __restrict__ out) {
    const int n = *count;
    const int64_t vec_per_row = pitch / 8;  // 16-byte vectors
    for (int64_t j = blockIdx.x; j < n; j += gridDim.x) {
        const int64_t src = rows[j];
        for (int pl = 0; pl < npl; pl++) {
            const uint4* s4 = reinterpret_cast<const uint4*>(a + pl * plane_stride + src * pitch);
            uint4* d4 = reinterpret_cast<uint4*>(out + pl * plane_stride + j * pitch);
            for (int64_t v = threadIdx.x; v < vec_per_row; v += blockDim.x) d4[v] = s4[v];
        }
    }
}

template <int SRC>
int launch_sort_select(const SortSelectParams& p, cudaStream_t stream) {
    if (p.nq <= 0) return B200F_OK;
    if (p.k < 1 || p.k > B200F_MAX_K) return B200F_ERR_UNSUPPORTED;
    const int smem = SS_CAP * 8;
    static bool attr_set[kMaxDevices] = {false};   // the opt-in is per device
    const int slot = device_slot();
    if (!attr_set[slot]) {
        B200F_CUDA_TRY(cudaFuncSetAttribute(sort_select_kernel<SRC>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_set[slot] = true;
    }
    int64_t g = p.nq;
    const int64_t cap = (int64_t)cached_sm_count() * 2 * 8;
    if (g > cap) g = cap;
    // rows counted on the device are usually few or none: idle CTAs leave at once
    if (p.nq_dev && g > cached_sm_count()) g = cached_sm_count();
    sort_select_kernel<SRC><<<(int)g, SS_THREADS, smem, stream>>>(p);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

__global__ void finalize_lists_kernel(const float* __restrict__ run_key,
                                      const int32_t* __restrict__ run_idx, int64_t nq, int k,
                                      float out_sign, const float* __restrict__ qnorm, int clamp,
                                      float pad, int64_t label_base, float* __restrict__ out_dist,
                                      int64_t* __restrict__ out_labels,
                                      const int* __restrict__ nq_dev,
                                      const int32_t* __restrict__ row_map) {
    if (nq_dev) nq = min((int64_t)*nq_dev, nq);
    const int64_t total = nq * k;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t q = i / k;
        const int64_t qo = row_map ? (int64_t)row_map[q] : q;  // output row
        const int32_t id = run_idx[i];
        float dist = pad;
        int64_t label = -1;
        if (id >= 0) {
            dist = out_sign * run_key[i] + (qnorm ? qnorm[qo] : 0.f);
            if (clamp && dist < 0.f) dist = 0.f;
            label = (int64_t)id + label_base;
        }
        out_dist[qo * k + (i - q * k)] = dist;
        out_labels[qo * k + (i - q * k)] = label;
    }
}

}  // namespace

int launch_merge_partials(const float* part_key, const int32_t* part_idx, int P, int64_t nq, int k,
                          int metric, const float* qnorm, int64_t label_base, float* out_dist,
                          int64_t* out_labels, const int* nq_dev, const int32_t* row_map,
                          cudaStream_t stream) {
    if (nq <= 0) return B200F_OK;
    if (k < 1 || k > 32 || P < 1) return B200F_ERR_UNSUPPORTED;
    MergeSmallParams<int32_t> p{};
    p.nq_dev = nq_dev;
    p.row_map = row_map;
    p.in_key = part_key;
    p.in_id = part_idx;
    p.q_stride = (int64_t)P * k;
    p.p_stride = k;
    p.p_stride_id = k;
    p.P = P;
    p.nq = nq;
    p.k = k;
    p.key_sign = 1.f;
    const bool l2 = metric == B200F_METRIC_L2;
    p.out_sign = l2 ? 1.f : -1.f;
    p.qnorm = l2 ? qnorm : nullptr;
    p.clamp = l2 ? 1 : 0;
    p.pad = l2 ? kHostInf : -kHostInf;
    p.label_base = label_base;
    p.out_dist = out_dist;
    p.out_labels = out_labels;
    int64_t g = nq;
    const int64_t cap = (int64_t)cached_sm_count() * 32;
    if (g > cap) g = cap;
    if (nq_dev && g > cached_sm_count()) g = cached_sm_count();
    merge_small_kernel<int32_t><<<(int)g, MS_THREADS, 0, stream>>>(p);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

int launch_merge_keys(const float* part_key, const int32_t* part_idx, int P, int64_t nq, int k,
                      float* out_key, cudaStream_t stream) {
    if (nq <= 0) return B200F_OK;
    if (k < 1 || k > 32 || P < 1) return B200F_ERR_UNSUPPORTED;
    MergeSmallParams<int32_t> p{};
    p.in_key = part_key;
    p.in_id = part_idx;
    p.q_stride = (int64_t)P * k;
    p.p_stride = k;
    p.p_stride_id = k;
    p.P = P;
    p.nq = nq;
    p.k = k;
    p.key_sign = 1.f;
    p.out_sign = 1.f;
    p.pad = kHostInf;
    p.out_dist = out_key;
    p.out_labels = nullptr;
    int64_t g = nq;
    const int64_t cap = (int64_t)cached_sm_count() * 32;
    if (g > cap) g = cap;
    merge_small_kernel<int32_t><<<(int)g, MS_THREADS, 0, stream>>>(p);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

int launch_select_keys(const float* keys, int64_t nq, int64_t ncols, int64_t ld, int r, float* out_key,
                       cudaStream_t stream) {
    if (r < 1 || r > 32 || ncols < 0 || ld < ncols || !keys || !out_key) return B200F_ERR_BAD_ARG;
    if (nq <= 0) return B200F_OK;
    int64_t g = ceil_div64(nq, SEL_WARPS);
    const int64_t gcap = (int64_t)cached_sm_count() * 8;
    if (g > gcap) g = gcap;
    select_keys_kernel<<<(int)g, SEL_WARPS * 32, 0, stream>>>(keys, nq, ncols, ld, r, out_key);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

int launch_select_chunk(const float* keys, int64_t nq, int64_t ncols, int64_t ld, int64_t col0,
                        int k, int has_prev, float* run_key, int32_t* run_idx, const int* nq_dev,
                        cudaStream_t stream) {
    SortSelectParams p{};
    p.nq_dev = nq_dev;
    p.keys = keys;
    p.ld = ld;
    p.ncand = ncols;
    p.col0 = col0;
    p.nq = nq;
    p.k = k;
    p.key_sign = 1.f;
    p.has_prev = has_prev;
    p.run_key = run_key;
    p.run_idx = run_idx;
    p.out_dist = nullptr;
    return launch_sort_select<SRC_MATRIX>(p, stream);
}

int launch_select_parts(const float* part_key, const int32_t* part_idx, int nlists, int64_t nq,
                        int k, int metric, const float* qnorm, int64_t label_base, float* out_dist,
                        int64_t* out_labels, int32_t* dirty, cudaStream_t stream) {
    if (nlists < 1 || (int64_t)nlists * 32 > 0x7fffffffLL) return B200F_ERR_UNSUPPORTED;
    const bool l2 = metric == B200F_METRIC_L2;
    SortSelectParams p{};
    p.keys = part_key;
    p.part_idx = part_idx;
    p.P = nlists;
    p.ld = (int64_t)nlists * 32;
    p.nq = nq;
    p.k = k;
    p.key_sign = 1.f;
    p.has_prev = 0;
    p.out_sign = l2 ? 1.f : -1.f;
    p.qnorm = l2 ? qnorm : nullptr;
    p.clamp = l2 ? 1 : 0;
    p.pad = l2 ? kHostInf : -kHostInf;
    p.label_base = label_base;
    p.out_dist = out_dist;
    p.out_labels = out_labels;
    p.dirty = dirty;
    return launch_sort_select<SRC_PARTS>(p, stream);
}

int launch_select_candidates(const float* cand_key, const int32_t* cand_idx, const int32_t* cand_cnt,
                             int cap, int64_t nb, int64_t nq, int k, int metric, const float* qnorm,
                             int64_t label_base, float* out_dist, int64_t* out_labels, int32_t* dirty,
                             cudaStream_t stream) {
    if (cap < 1 || !cand_cnt) return B200F_ERR_BAD_ARG;
    if (rank_select_enabled() && rank_select_fits(cap, k) && dirty)
        return launch_rank_select(cand_key, cand_idx, cand_cnt, cap, nb, nq, k, metric, qnorm, label_base,
                                  out_dist, out_labels, dirty, stream);
    const bool l2 = metric == B200F_METRIC_L2;
    SortSelectParams p{};
    p.keys = cand_key;
    p.part_idx = cand_idx;
    p.cand_cnt = cand_cnt;
    p.nb_total = nb;
    p.ld = cap;
    p.nq = nq;
    p.k = k;
    p.key_sign = 1.f;
    p.has_prev = 0;
    p.out_sign = l2 ? 1.f : -1.f;
    p.qnorm = l2 ? qnorm : nullptr;
    p.clamp = l2 ? 1 : 0;
    p.pad = l2 ? kHostInf : -kHostInf;
    p.label_base = label_base;
    p.out_dist = out_dist;
    p.out_labels = out_labels;
    p.dirty = dirty;
    if (k <= 32) {
        if (nq <= 0) return B200F_OK;
        int64_t g = ceil_div64(nq, SEL_WARPS);
        const int64_t gcap = (int64_t)cached_sm_count() * 8;
        if (g > gcap) g = gcap;
        select_small_kernel<<<(int)g, SEL_WARPS * 32, 0, stream>>>(p);
        count_launch();
        B200F_LAUNCH_CHECK();
        return B200F_OK;
    }
    return launch_sort_select<SRC_PARTS>(p, stream);
}

int launch_compact_rows(const int32_t* dirty, int64_t nq, int32_t* rows, int32_t* count,
                        int32_t* count_copy, cudaStream_t stream) {
    if (nq <= 0) return B200F_OK;
    compact_rows_kernel<<<1, 1024, 0, stream>>>(dirty, nq, rows, count, count_copy);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

int launch_gather_rows(const uint16_t* a, int npl, int64_t plane_stride, int64_t pitch,
                       const int32_t* rows, const int32_t* count, int64_t nq_max, uint16_t* out,
                       cudaStream_t stream) {
    if (nq_max <= 0) return B200F_OK;
    if ((pitch % 8) != 0 || (plane_stride % 8) != 0) return B200F_ERR_BAD_ARG;
    int64_t g = nq_max < 2 * (int64_t)cached_sm_count() ? nq_max : 2 * (int64_t)cached_sm_count();
    gather_rows_kernel<<<(int)g, 128, 0, stream>>>(a, npl, plane_stride, pitch, rows, count, out);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

int launch_finalize_lists(const float* run_key, const int32_t* run_idx, int64_t nq, int k,
                          int metric, const float* qnorm, int64_t label_base, float* out_dist,
                          int64_t* out_labels, const int* nq_dev, const int32_t* row_map,
                          cudaStream_t stream) {
    if (nq <= 0) return B200F_OK;
    const bool l2 = metric == B200F_METRIC_L2;
    int64_t g = ceil_div64(nq * k, 256);
    const int64_t cap = (int64_t)cached_sm_count() * 16;
    if (g > cap) g = cap;
    finalize_lists_kernel<<<(int)g, 256, 0, stream>>>(run_key, run_idx, nq, k, l2 ? 1.f : -1.f,
                                                      l2 ? qnorm : nullptr, l2 ? 1 : 0,
                                                      l2 ? kHostInf : -kHostInf, label_base,
                                                      out_dist, out_labels, nq_dev, row_map);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

}  // namespace b200f

using namespace b200f;

extern "C" size_t b200f_select_scratch_bytes(int64_t nq, int k) {
    (void)nq;
    (void)k;
    return 256;  // the selection kernel keeps all of its state in shared memory
}

extern "C" int b200f_select_rows(const float* scores, int64_t nq, int64_t ncols, int64_t ld,
                                 int metric, int k, float* out_dist, int64_t* out_labels,
                                 void* scratch, size_t scratch_bytes, void* stream) {
    (void)scratch;
    (void)scratch_bytes;
    if (nq < 0 || ncols < 0 || ld < ncols || k <= 0 ||
        (metric != B200F_METRIC_L2 && metric != B200F_METRIC_INNER_PRODUCT))
        return B200F_ERR_BAD_ARG;
    if (k > B200F_MAX_K || ncols > 0x7fffffffLL) return B200F_ERR_UNSUPPORTED;
    if (nq == 0) return B200F_OK;
    if (!scores || !out_dist || !out_labels) return B200F_ERR_BAD_ARG;
    const bool l2 = metric == B200F_METRIC_L2;
    SortSelectParams p{};
    p.keys = scores;
    p.ld = ld;
    p.ncand = ncols;
    p.col0 = 0;
    p.nq = nq;
    p.k = k;
    p.key_sign = l2 ? 1.f : -1.f;
    p.has_prev = 0;
    p.out_sign = l2 ? 1.f : -1.f;
    p.qnorm = nullptr;
    p.clamp = 0;
    p.pad = l2 ? kHostInf : -kHostInf;
    p.label_base = 0;
    p.out_dist = out_dist;
    p.out_labels = out_labels;
    return launch_sort_select<SRC_MATRIX>(p, static_cast<cudaStream_t>(stream));
}

// Row shards laid out block-cyclically: global row g lives on shard (g / B) % S at local row
// (g / (B * S)) * B + g % B.  The inverse, applied to the labels a shard-local search returned.
__global__ void remap_labels_kernel(int64_t* __restrict__ labels, int64_t n, int64_t block, int64_t nshards,
                                    int64_t shard) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t l = labels[i];
        if (l >= 0) labels[i] = ((l / block) * nshards + shard) * block + l % block;
    }
}

extern "C" int b200f_remap_labels_block_cyclic(int64_t* labels, int64_t count, int64_t block_rows, int nshards,
                                               int shard, void* stream) {
    if (count < 0 || block_rows < 1 || nshards < 1 || shard < 0 || shard >= nshards) return B200F_ERR_BAD_ARG;
    if (count == 0) return B200F_OK;
    if (!labels) return B200F_ERR_BAD_ARG;
    int64_t g = ceil_div64(count, 256);
    const int64_t cap = (int64_t)cached_sm_count() * 8;
    if (g > cap) g = cap;
    remap_labels_kernel<<<(int)g, 256, 0, static_cast<cudaStream_t>(stream)>>>(labels, count, block_rows, nshards, shard);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

extern "C" int b200f_merge_lists_strided(const float* dist, const int64_t* labels,
                                         int64_t list_stride_dist, int64_t list_stride_labels, int P,
                                         int64_t nq, int k, int metric, float* out_dist,
                                         int64_t* out_labels, void* stream) {
    if (P <= 0 || nq < 0 || k <= 0 ||
        (metric != B200F_METRIC_L2 && metric != B200F_METRIC_INNER_PRODUCT))
        return B200F_ERR_BAD_ARG;
    if (k > B200F_MAX_K || (int64_t)P * k > 0x7fffffffLL) return B200F_ERR_UNSUPPORTED;
    if (nq == 0) return B200F_OK;
    if (!dist || !labels || !out_dist || !out_labels) return B200F_ERR_BAD_ARG;
    if (list_stride_dist < nq * (int64_t)k || list_stride_labels < nq * (int64_t)k) return B200F_ERR_BAD_ARG;
    const bool l2 = metric == B200F_METRIC_L2;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (k <= 32) {
        MergeSmallParams<int64_t> p{};
        p.in_key = dist;
        p.in_id = labels;
        p.q_stride = k;
        p.p_stride = list_stride_dist;
        p.p_stride_id = list_stride_labels;
        p.P = P;
        p.nq = nq;
        p.k = k;
        p.key_sign = l2 ? 1.f : -1.f;
        p.out_sign = l2 ? 1.f : -1.f;
        p.qnorm = nullptr;
        p.clamp = 0;
        p.pad = l2 ? kHostInf : -kHostInf;
        p.label_base = 0;
        p.out_dist = out_dist;
        p.out_labels = out_labels;
        int64_t g = nq;
        const int64_t cap = (int64_t)cached_sm_count() * 32;
        if (g > cap) g = cap;
        merge_small_kernel<int64_t><<<(int)g, MS_THREADS, 0, st>>>(p);
        count_launch();
        B200F_LAUNCH_CHECK();
        return B200F_OK;
    }
    if (rank_select_enabled() && rank_merge_fits(P, k))
        return launch_rank_merge(dist, labels, list_stride_dist, list_stride_labels, P, nq, k, metric, out_dist,
                                 out_labels, st);
    SortSelectParams p{};
    p.keys = dist;
    p.labels = labels;
    p.list_stride_k = list_stride_dist;
    p.list_stride_l = list_stride_labels;
    p.P = P;
    p.nq = nq;
    p.k = k;
    p.key_sign = l2 ? 1.f : -1.f;
    p.has_prev = 0;
    p.out_sign = l2 ? 1.f : -1.f;
    p.qnorm = nullptr;
    p.clamp = 0;
    p.pad = l2 ? kHostInf : -kHostInf;
    p.out_dist = out_dist;
    p.out_labels = out_labels;
    return launch_sort_select<SRC_LISTS>(p, st);
}

extern "C" int b200f_merge_lists(const float* dist, const int64_t* labels, int P, int64_t nq, int k,
                                 int metric, float* out_dist, int64_t* out_labels, void* stream) {
    return b200f_merge_lists_strided(dist, labels, nq * (int64_t)k, nq * (int64_t)k, P, nq, k, metric,
                                     out_dist, out_labels, stream);
}
