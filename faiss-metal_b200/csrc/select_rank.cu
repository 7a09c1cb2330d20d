// Selection by rank: radix threshold, sorting in registers, merging by binary search.
//
// Covers the same ground as block_select_min/max (shaders/block_select.metal:111-274) and the
// list merge of the fused kernels (shaders/fused_l2_topk.metal:88-131) for the two inputs that
// are small enough to need no streaming:
//
//  * rank_select: the k best (32 < k <= 4096) of a row's threshold-filtered candidates, an
//    unordered buffer of at most 8192 (key, id) pairs, typically several times k.  A CTA of W
//    warps takes one row.  (1) The k-th smallest key is found exactly by a radix select over the
//    keys' spread (8 bits a pass, histogram in shared memory).  (2) The candidates up to that key
//    (k of them plus ties) are compacted.  (3) Every warp sorts its share of them in registers
//    (bitonic network over 32 R elements, R per lane: strides below R are register swaps, the
//    others one shuffle pair), the sorted runs go to shared memory, and every element finds its
//    final position as its own index plus its lower bounds in the other runs.
//  * rank_merge: P sorted result lists of k entries (other shards' answers), P k <= 8192.
//    The lists are runs already.  Only entries up to the largest of the lists' (k / P)-th keys
//    can belong to the result; each of those finds its position by binary search in the other
//    lists.  Final distances can tie where the keys a shard sorted by did not, so equal
//    distances need not come in label order inside a list: short runs of them are put in order
//    first, and a row that still is not strictly ordered is sorted outright in shared memory.
//
// Both write exactly what sort_select_kernel writes for the same input: ascending key, ties to the
// lower id / label.
#include <atomic>

#include "common.cuh"

namespace b200f {

namespace {

constexpr unsigned FULL = 0xffffffffu;
constexpr uint64_t RS_EMPTY = ~0ull;
constexpr int RS_MAX_WARPS = 8;
constexpr int RS_RUN = 512;    // most elements one warp sorts (16 per lane)

std::atomic<int> g_rank_select{1};

__device__ __forceinline__ uint64_t shfl_xor64(uint64_t v, int m) {
    const unsigned lo = __shfl_xor_sync(FULL, (unsigned)v, m);
    const unsigned hi = __shfl_xor_sync(FULL, (unsigned)(v >> 32), m);
    return ((uint64_t)hi << 32) | lo;
}

// Ascending sort of the 32 R words a warp holds; element e = lane * R + r sits in v[r] of lane.
template <int R>
__device__ __forceinline__ void warp_sort(uint64_t (&v)[R], int lane) {
#pragma unroll
    for (int size = 2; size <= 32 * R; size <<= 1) {
#pragma unroll
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (stride >= R) {
                const int ls = stride / R;
                const bool up = ((lane * R) & size) == 0;
                const bool keep_min = ((lane & ls) == 0) == up;
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const uint64_t o = shfl_xor64(v[r], ls);
                    const bool less = v[r] < o;
                    v[r] = (less == keep_min) ? v[r] : o;
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; r++) {
                    if ((r & stride) == 0) {
                        const bool up = (size < R) ? ((r & size) == 0) : (((lane * R) & size) == 0);
                        constexpr int RM = R - 1;   // no-op mask: keeps the index in range where the branch is dead
                        const uint64_t a = v[r], b = v[(r | stride) & RM];
                        const bool swap = (a > b) == up;
                        v[r] = swap ? b : a;
                        v[(r | stride) & RM] = swap ? a : b;
                    }
                }
            }
        }
    }
}

struct RankSelectParams {
    const float* keys;        // [nq][ld] candidate keys, smaller is better
    const int32_t* ids;       // [nq][ld] row ids (-1 = empty)
    const int32_t* cnt;       // [nq] candidates counted (may exceed ld: overflow)
    int64_t ld;
    int64_t nb_total;
    int64_t nq;
    int k;
    float out_sign;
    const float* qnorm;
    int clamp;
    float pad;
    int64_t label_base;
    float* out_dist;
    int64_t* out_labels;
    int32_t* dirty;
};

__device__ __forceinline__ void rs_write(const RankSelectParams& p, int64_t q, int rank, uint64_t w) {
    float dist = p.out_sign * ordered_to_float((uint32_t)(w >> 32)) + (p.qnorm ? p.qnorm[q] : 0.f);
    if (p.clamp && dist < 0.f) dist = 0.f;
    p.out_dist[q * p.k + rank] = dist;
    p.out_labels[q * p.k + rank] = (int64_t)(uint32_t)w + p.label_base;
}

// Sort and place the c words staged in `runs` (all distinct); warp w takes words [w m, w m + m).
// The staging area becomes the sorted runs, 32 R words per warp.
template <int R>
__device__ __forceinline__ void rank_place(const RankSelectParams& p, int64_t q, int c, int m,
                                           uint64_t* runs, int W) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    uint64_t v[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int t = r * 32 + lane;
        const int i = warp * m + t;
        v[r] = (t < m && i < c) ? runs[i] : RS_EMPTY;
    }
    __syncthreads();   // everybody holds their share: the area may be overwritten
    warp_sort<R>(v, lane);
    constexpr int N = 32 * R;
#pragma unroll
    for (int r = 0; r < R; r++) runs[warp * N + lane * R + r] = v[r];
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int e = lane * R + r;
        const uint64_t w = v[r];
        if (w != RS_EMPTY && e < p.k) {
            int rank = e;
            for (int o = 0; o < W && rank < p.k; o++) {
                if (o == warp) continue;
                const uint64_t* run = runs + o * N;
                int lo = 0, hi = N;       // words are distinct: the lower bound is the count
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (run[mid] < w) lo = mid + 1; else hi = mid;
                }
                rank += lo;
            }
            if (rank < p.k) rs_write(p, q, rank, w);
        }
    }
}

// W warps; at most W * RS_RUN candidates up to the k-th key are sorted here.  A row with more
// (k-th key shared by hundreds of candidates) is reported through dirty[] like an overflowed
// one, and the caller's exact redo pass takes it.
__global__ void __launch_bounds__(RS_MAX_WARPS * 32, 4) rank_select_kernel(const RankSelectParams p) {
    extern __shared__ __align__(16) uint64_t rs_runs[];   // W * RS_RUN words
    __shared__ int s_hist[256];
    __shared__ uint32_t s_min[RS_MAX_WARPS], s_max[RS_MAX_WARPS];
    __shared__ int s_live[RS_MAX_WARPS];
    __shared__ int s_sel[2];
    __shared__ int s_count;
    const int W = blockDim.x >> 5;
    const int T = blockDim.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int bound = W * RS_RUN;
    for (int64_t q = blockIdx.x; q < p.nq; q += gridDim.x) {
        const int64_t cnt = __ldg(p.cnt + q);
        const int n = (int)min(cnt, p.ld);
        const float* keys = p.keys + q * p.ld;
        const int32_t* ids = p.ids + q * p.ld;
        // spread of the live keys (the row's few KB stay in L1 for the passes below)
        int live = 0;
        uint32_t mn = 0xffffffffu, mx = 0;
#pragma unroll 4
        for (int c = tid; c < n; c += T) {
            const int32_t id = __ldg(ids + c);     // both loads issued before either is used
            const uint32_t key = float_to_ordered(__ldg(keys + c));
            if (id >= 0) {
                live++;
                mn = min(mn, key);
                mx = max(mx, key);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            live += __shfl_xor_sync(FULL, live, o);
            mn = min(mn, __shfl_xor_sync(FULL, mn, o));
            mx = max(mx, __shfl_xor_sync(FULL, mx, o));
        }
        if (lane == 0) {
            s_live[warp] = live;
            s_min[warp] = mn;
            s_max[warp] = mx;
        }
        if (tid == 0) s_count = 0;
        __syncthreads();
        live = 0;
        for (int w = 0; w < W; w++) {
            live += s_live[w];
            mn = min(mn, s_min[w]);
            mx = max(mx, s_max[w]);
        }
        // x = key - mn; the k-th smallest x of the live candidates, exactly
        uint32_t thr_x = live > 0 ? mx - mn : 0;
        if (live > p.k) {
            int hi = 32 - __clz(thr_x);   // significant bits of the spread; 0: all keys equal
            uint32_t prefix = 0;
            int kk = p.k;
            while (hi > 0) {
                const int lo = hi > 8 ? hi - 8 : 0;
                const uint32_t mask = (1u << (hi - lo)) - 1u;
                for (int i = tid; i < 256; i += T) s_hist[i] = 0;
                __syncthreads();
#pragma unroll 4
                for (int c = tid; c < n; c += T) {
                    const int32_t id = __ldg(ids + c);
                    const uint32_t x = float_to_ordered(__ldg(keys + c)) - mn;
                    if (id >= 0 && (uint32_t)((uint64_t)x >> hi) == prefix)
                        atomicAdd(&s_hist[(x >> lo) & mask], 1);
                }
                __syncthreads();
                if (warp == 0) {
                    int h[8], sum = 0;
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        h[i] = s_hist[lane * 8 + i];
                        sum += h[i];
                    }
                    int incl = sum;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int up = __shfl_up_sync(FULL, incl, o);
                        if (lane >= o) incl += up;
                    }
                    int below = incl - sum;
                    if (below < kk && kk <= incl) {   // exactly one lane
                        int digit = 0;
#pragma unroll
                        for (int i = 0; i < 7; i++) {
                            if (digit == i && below + h[i] < kk) {
                                below += h[i];
                                digit = i + 1;
                            }
                        }
                        s_sel[0] = lane * 8 + digit;
                        s_sel[1] = kk - below;
                    }
                }
                __syncthreads();
                prefix = (prefix << (hi - lo)) | (uint32_t)s_sel[0];
                kk = s_sel[1];
                hi = lo;
            }
            thr_x = prefix;
        }
        // compaction of the candidates up to the threshold (k of them plus ties, or all)
        for (int c0 = warp * 32; c0 < n; c0 += T) {
            const int c = c0 + lane;
            bool keep = false;
            uint64_t word = 0;
            if (c < n) {
                const int32_t id = __ldg(ids + c);
                const uint32_t key = float_to_ordered(__ldg(keys + c));
                keep = id >= 0 && key - mn <= thr_x;   // live keys are >= mn
                word = ((uint64_t)key << 32) | (uint32_t)id;
            }
            const unsigned b = __ballot_sync(FULL, keep);
            int base = 0;
            if (lane == 0 && b) base = atomicAdd(&s_count, __popc(b));
            base = __shfl_sync(FULL, base, 0);
            const int pos = base + __popc(b & ((1u << lane) - 1u));
            if (keep && pos < bound) rs_runs[pos] = word;
        }
        __syncthreads();
        const int c = s_count;
        const bool too_many = c > bound;
        if (!too_many) {
            const int m = (c + W - 1) / W;    // <= RS_RUN
            if (m <= 32) rank_place<1>(p, q, c, m, rs_runs, W);
            else if (m <= 64) rank_place<2>(p, q, c, m, rs_runs, W);
            else if (m <= 128) rank_place<4>(p, q, c, m, rs_runs, W);
            else if (m <= 256) rank_place<8>(p, q, c, m, rs_runs, W);
            else rank_place<16>(p, q, c, m, rs_runs, W);
            for (int j = c + tid; j < p.k; j += T) {
                p.out_dist[q * p.k + j] = p.pad;
                p.out_labels[q * p.k + j] = -1;
            }
        }
        if (tid == 0) p.dirty[q] = (too_many || (cnt > p.ld) || (cnt < p.k && cnt < p.nb_total)) ? 1 : 0;
        __syncthreads();   // the shared arrays are rewritten by the next row
    }
}

// ---------------------------------------------------------------------------------------
// rank_merge
// ---------------------------------------------------------------------------------------
struct RankMergeParams {
    const float* dist;       // list l of query q at dist + l * stride_d + q * k
    const int64_t* labels;   // same layout with stride_l; -1 = empty slot
    int64_t stride_d, stride_l;
    int P;
    int64_t nq;
    int k;
    int Tp;                  // P k rounded up to a power of two (entries of the shared arrays)
    float key_sign;          // key = key_sign * dist, smaller is better
    float pad;
    float* out_dist;
    int64_t* out_labels;
};

constexpr int RM_MAX_LISTS = 256;   // P <= 8192 / 33

// (key, label) of a before (key, label) of b; an empty slot (label -1) is the largest label
__device__ __forceinline__ bool rm_before(uint32_t ka, uint64_t la, uint32_t kb, uint64_t lb) {
    return ka < kb || (ka == kb && la < lb);
}

__global__ void __launch_bounds__(512, 2) rank_merge_kernel(const RankMergeParams p) {
    extern __shared__ __align__(16) uint64_t rm_lab[];    // [Tp] labels, then [Tp] ordered keys
    __shared__ int s_live;
    __shared__ int s_start[RM_MAX_LISTS + 1];   // entries up to tau: list l holds [s_start[l], s_start[l+1]) of them
    const int T = p.P * p.k;
    uint32_t* rm_key = reinterpret_cast<uint32_t*>(rm_lab + p.Tp);
    const int tid = threadIdx.x;
    const int kp = (p.k + p.P - 1) / p.P;
    for (int64_t q = blockIdx.x; q < p.nq; q += gridDim.x) {
        __syncthreads();   // the previous row's readers are done
        if (tid == 0) s_live = 0;
        __syncthreads();
        // flat index over all lists: every thread's loads are in flight together
        int live = 0;
#pragma unroll 4
        for (int c = tid; c < p.Tp; c += blockDim.x) {
            uint64_t lab = RS_EMPTY;
            uint32_t key = 0xffffffffu;
            if (c < T) {
                const int l = c / p.k;
                const int64_t off = q * p.k + (c - l * p.k);
                const int64_t lb = __ldg(p.labels + (int64_t)l * p.stride_l + off);
                const float d = __ldg(p.dist + (int64_t)l * p.stride_d + off);
                if (lb >= 0) {
                    lab = (uint64_t)lb;
                    key = float_to_ordered(p.key_sign * d);
                    live++;
                }
            }
            rm_lab[c] = lab;
            rm_key[c] = key;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) live += __shfl_xor_sync(FULL, live, o);
        if ((tid & 31) == 0 && live) atomicAdd(&s_live, live);
        __syncthreads();
        // every list must ascend strictly in (key, label), empty slots last
        int bad = 0;
        for (int c = tid; c < T; c += blockDim.x) {
            if (c % p.k == 0) continue;
            const bool both_empty = rm_lab[c] == RS_EMPTY && rm_lab[c - 1] == RS_EMPTY;
            if (!both_empty && !rm_before(rm_key[c - 1], rm_lab[c - 1], rm_key[c], rm_lab[c])) bad = 1;
        }
        bad = __syncthreads_or(bad);
        if (bad) {
            // equal keys next to each other in label order: four odd-even rounds settle runs of
            // up to four (final distances that tie although the shard's keys did not)
            for (int phase = 0; phase < 4; phase++) {
                for (int l = 0; l < p.P; l++) {
                    for (int j = (phase & 1) + 2 * tid; j + 1 < p.k; j += 2 * blockDim.x) {
                        const int c = l * p.k + j;
                        if (rm_key[c] == rm_key[c + 1]) {
                            const uint64_t a = rm_lab[c], b = rm_lab[c + 1];
                            if (a > b) {
                                rm_lab[c] = b;
                                rm_lab[c + 1] = a;
                            }
                        }
                    }
                }
                __syncthreads();
            }
            bad = 0;
            for (int l = 0; l < p.P; l++) {
                for (int j = 1 + tid; j < p.k; j += blockDim.x) {
                    const int c = l * p.k + j;
                    const bool both_empty = rm_lab[c] == RS_EMPTY && rm_lab[c - 1] == RS_EMPTY;
                    if (!both_empty && !rm_before(rm_key[c - 1], rm_lab[c - 1], rm_key[c], rm_lab[c])) bad = 1;
                }
            }
            bad = __syncthreads_or(bad);
        }
        if (!bad) {
            // at least P * kp >= k entries have a key up to tau: nothing beyond it is in the result
            uint32_t tau = 0;
            for (int l = 0; l < p.P; l++) tau = max(tau, rm_key[l * p.k + kp - 1]);
            for (int l = tid; l < p.P; l += blockDim.x) {
                const uint32_t* run = rm_key + l * p.k;
                int lo = 0, hi = p.k;
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (run[mid] <= tau) lo = mid + 1; else hi = mid;
                }
                s_start[l + 1] = lo;   // a count for now
            }
            __syncthreads();
            if (tid == 0) {
                s_start[0] = 0;
                for (int l = 0; l < p.P; l++) s_start[l + 1] += s_start[l];
            }
            __syncthreads();
            const int S = s_start[p.P];
            for (int e = tid; e < S; e += blockDim.x) {
                int l = 0;
                while (s_start[l + 1] <= e) l++;
                const int j = e - s_start[l];
                const uint64_t lab = rm_lab[l * p.k + j];
                const uint32_t key = rm_key[l * p.k + j];
                if (lab == RS_EMPTY) continue;
                int rank = j;
                for (int o = 0; o < p.P && rank < p.k; o++) {
                    if (o == l) continue;
                    // entries of list o that come first: an equal (key, label) in a lower list does
                    const int base = o * p.k;
                    int lo = 0, hi = s_start[o + 1] - s_start[o];
                    while (lo < hi) {
                        const int mid = (lo + hi) >> 1;
                        const uint32_t km = rm_key[base + mid];
                        bool first = km < key;
                        if (km == key) {
                            const uint64_t lm = rm_lab[base + mid];
                            first = lm < lab || (lm == lab && o < l);
                        }
                        if (first) lo = mid + 1; else hi = mid;
                    }
                    rank += lo;
                }
                if (rank < p.k) {
                    p.out_dist[q * p.k + rank] = p.key_sign * ordered_to_float(key);
                    p.out_labels[q * p.k + rank] = (int64_t)lab;
                }
            }
        } else {
            // any order at all: bitonic sort of the (key, label) records
            for (int size = 2; size <= p.Tp; size <<= 1) {
                for (int stride = size >> 1; stride > 0; stride >>= 1) {
                    for (int i = tid; i < (p.Tp >> 1); i += blockDim.x) {
                        const int pos = 2 * i - (i & (stride - 1));
                        const uint32_t ka = rm_key[pos], kb = rm_key[pos + stride];
                        const uint64_t la = rm_lab[pos], lb = rm_lab[pos + stride];
                        const bool up = (pos & size) == 0;
                        if (rm_before(kb, lb, ka, la) == up && !(ka == kb && la == lb)) {
                            rm_key[pos] = kb;
                            rm_key[pos + stride] = ka;
                            rm_lab[pos] = lb;
                            rm_lab[pos + stride] = la;
                        }
                    }
                    __syncthreads();
                }
            }
            for (int j = tid; j < p.k; j += blockDim.x) {
                const uint64_t lab = rm_lab[j];
                if (lab != RS_EMPTY) {
                    p.out_dist[q * p.k + j] = p.key_sign * ordered_to_float(rm_key[j]);
                    p.out_labels[q * p.k + j] = (int64_t)lab;
                }
            }
        }
        const int total = s_live;
        for (int j = total + tid; j < p.k; j += blockDim.x) {
            p.out_dist[q * p.k + j] = p.pad;
            p.out_labels[q * p.k + j] = -1;
        }
    }
}

}  // namespace

bool rank_select_enabled() { return g_rank_select.load(std::memory_order_relaxed) != 0; }

bool rank_select_fits(int cap, int k) { return k > 32 && k <= 1024 && cap >= 1; }

int launch_rank_select(const float* cand_key, const int32_t* cand_idx, const int32_t* cand_cnt, int cap,
                       int64_t nb, int64_t nq, int k, int metric, const float* qnorm, int64_t label_base,
                       float* out_dist, int64_t* out_labels, int32_t* dirty, cudaStream_t stream) {
    if (!rank_select_fits(cap, k) || !cand_cnt || !dirty) return B200F_ERR_BAD_ARG;
    if (nq <= 0) return B200F_OK;
    const bool l2 = metric == B200F_METRIC_L2;
    RankSelectParams p{};
    p.keys = cand_key;
    p.ids = cand_idx;
    p.cnt = cand_cnt;
    p.ld = cap;
    p.nb_total = nb;
    p.nq = nq;
    p.k = k;
    p.out_sign = l2 ? 1.f : -1.f;
    p.qnorm = l2 ? qnorm : nullptr;
    p.clamp = l2 ? 1 : 0;
    p.pad = l2 ? kHostInf : -kHostInf;
    p.label_base = label_base;
    p.out_dist = out_dist;
    p.out_labels = out_labels;
    p.dirty = dirty;
    // room for 4 k candidates up to the k-th key: 2048 (4 warps) or 4096 (8 warps)
    const int W = k <= 512 ? 4 : RS_MAX_WARPS;
    const int smem = W * RS_RUN * 8;
    int64_t g = nq;
    const int64_t gcap = (int64_t)cached_sm_count() * 8;
    if (g > gcap) g = gcap;
    rank_select_kernel<<<(int)g, W * 32, smem, stream>>>(p);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

bool rank_merge_fits(int P, int k) { return k > 32 && P >= 1 && (int64_t)P * k <= 8192; }

int launch_rank_merge(const float* dist, const int64_t* labels, int64_t stride_d, int64_t stride_l, int P,
                      int64_t nq, int k, int metric, float* out_dist, int64_t* out_labels,
                      cudaStream_t stream) {
    if (!rank_merge_fits(P, k)) return B200F_ERR_BAD_ARG;
    if (nq <= 0) return B200F_OK;
    const bool l2 = metric == B200F_METRIC_L2;
    RankMergeParams p{};
    p.dist = dist;
    p.labels = labels;
    p.stride_d = stride_d;
    p.stride_l = stride_l;
    p.P = P;
    p.nq = nq;
    p.k = k;
    p.key_sign = l2 ? 1.f : -1.f;
    p.pad = l2 ? kHostInf : -kHostInf;
    p.out_dist = out_dist;
    p.out_labels = out_labels;
    const int T = P * k;
    int Tp = 64;
    while (Tp < T) Tp <<= 1;
    p.Tp = Tp;
    const int smem = Tp * 12;
    static bool attr_set[kMaxDevices] = {false};
    const int slot = device_slot();
    if (!attr_set[slot]) {
        B200F_CUDA_TRY(cudaFuncSetAttribute(rank_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            8192 * 12));
        attr_set[slot] = true;
    }
    const int threads = T > 4096 ? 512 : T > 1024 ? 256 : 128;
    int64_t g = nq;
    const int64_t gcap = (int64_t)cached_sm_count() * (threads == 128 ? 16 : 8);
    if (g > gcap) g = gcap;
    rank_merge_kernel<<<(int)g, threads, smem, stream>>>(p);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

}  // namespace b200f

extern "C" int b200f_set_rank_select(int on) {
    b200f::g_rank_select.store(on ? 1 : 0, std::memory_order_relaxed);
    return B200F_OK;
}
