// Shard-local search driver: path choice, scratch layout, kernel sequencing.
//
// Replaces the encode sequence of MetalIndexFlat::search (src/MetalIndexFlat.mm:358-378)
// and the path selection of MetalDistance / MetalSelect (src/MetalDistance.mm:107-128,
// 327-363; src/MetalSelect.mm:34-89).  Paths here depend on (nq, k) only:
//   nq <= 4 (8 on 16-bit rows)   streaming scan (scan.cu)
//   more queries                 tensor-core GEMM (gemm_topk.cu)
//   k  <= 32           top-k fused into the distance kernel, partial lists merged after
//   k  <= 1024         (tensor path, shard of >= 64k / 128k rows) threshold filter: a pilot pass
//                      over every 64th / 128th column tile gives each query a key threshold
//                      that admits a few times k rows; the full pass appends every column under
//                      the threshold to the query's candidate buffer (no lists, no matrix);
//                      the k best candidates are selected.  A row whose buffer overflowed or
//                      holds fewer than k candidates is redone by the paths below.
//   32 < k <= 1024     (tensor path, enough column ranges) the fused kernel keeps 32 entries
//                      per list, the k best of all lists are selected, and a row is redone
//                      through the key matrix only when a full list could have dropped one of
//                      its k results (rows counted and compacted on the device, no host sync)
//   k   > 32 otherwise distance keys written per column chunk, running sort-select
#include <atomic>
#include <cstdio>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"
#include "ptx.cuh"

namespace b200f {

namespace {

constexpr int64_t MATRIX_BUDGET_BYTES = 1024ll << 20;  // key-matrix chunk of the k > 32 path
constexpr int SCAN_GROUP = 4;

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

struct ProfileState {
    bool enabled = false;
    long long launches = 0;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pending;  // recorded, not yet read
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pool;
    long long main_launches = 0;
    double main_ms = 0.0;
};
ProfileState g_prof;
std::mutex g_prof_mu;

constexpr int kMaxGuards = 32;
constexpr uint32_t kCanaryWord = 0xC0DEFACEu;

struct SearchPlan {
    int path;         // B200F_PATH_SCAN or B200F_PATH_TENSOR
    bool fused;       // k <= 32
    bool lists;       // k > 32 selected from the fused kernel's 32-entry lists, matrix fallback per row
    int gslots;       // words per query row in the shared bound array
    bool filter;      // pilot threshold + candidate buffers, fused / matrix fallback per row
    int fstride;      // pilot pass: every fstride-th column tile
    int frank;        // threshold = frank-th best key of the pilot sample
    int fcap;         // candidate buffer entries per query
    GemmPlan pilot;
    bool pilot_matrix; // pilot sample as a key matrix (store mode + key selection) instead of lists
    int npl;
    int64_t a_pitch, a_plane_stride;
    GemmPlan gemm;    // tensor path (fused: whole shard; chunked: per chunk)
    ScanPlan scan;
    int64_t chunk_cols;
    int64_t ngroups;  // scan path: query groups of SCAN_GROUP
    size_t off_qscale;
    size_t off_qnorm, off_gthr, off_a, off_part_key, off_part_idx, off_matrix, off_run_key, off_run_idx;
    size_t off_dirty, off_rows, off_count, off_a2;
    size_t off_pilot_key, off_pilot_idx, off_thr, off_cand_key, off_cand_idx, off_cand_cnt;
    size_t total;
    // debug canaries: a 256-byte guard behind every slice of the scratch region
    int nguards;
    uint32_t guard_off[kMaxGuards];   // in units of 256 bytes
};

// Which optimistic selection stages of the tensor path may run (B200F_SELECT_*): set by
// b200f_set_selection_mode; until then the default comes from the environment variable
// B200F_SELECT_MODE (auto | filter | no_filter | matrix), read ONCE at the first search.
std::atomic<int> g_select_mode{-1};
std::atomic<int> g_canaries{0};   // b200f_set_debug_canaries

int select_mode() {
    int m = g_select_mode.load(std::memory_order_relaxed);
    if (m < 0) {
        m = B200F_SELECT_AUTO;
        if (const char* e = getenv("B200F_SELECT_MODE")) {
            if (!strcmp(e, "filter")) m = B200F_SELECT_FILTER;
            else if (!strcmp(e, "no_filter")) m = B200F_SELECT_NO_FILTER;
            else if (!strcmp(e, "matrix")) m = B200F_SELECT_MATRIX;
        }
        int expected = -1;
        if (!g_select_mode.compare_exchange_strong(expected, m)) m = expected;
    }
    return m;
}
bool filter_disabled() { const int m = select_mode(); return m == B200F_SELECT_NO_FILTER || m == B200F_SELECT_MATRIX; }
bool filter_forced() { return select_mode() == B200F_SELECT_FILTER; }
bool lists_disabled() { return select_mode() == B200F_SELECT_MATRIX; }

// The pilot pass costs 0.1 - 0.2 ms whatever the size (a handful of work items, each warming up
// its lists on a single tile).  Measured: at 2.6e8 (query, row) pairs the filter path is 19 - 47 %
// faster than the lists (d = 768 / 1536, 16-bit rows), at 1e8 - 4e8 pairs of fp32 rows with
// d = 128 the two are level; below this many pairs the lists are used.
// fp32 rows: five to eight queries take the scan path where the tf32 streaming scan pays and fits (three
// stages of 16 rows and two query matrices in shared memory: d up to 768)
constexpr int64_t F32_STREAM_MIN_ROWS = 65536;
constexpr int F32_STREAM_MAX_D = 768;
constexpr int64_t FILTER_MIN_PAIRS = 1ll << 27;
constexpr int64_t FILTER_MIN_PAIRS_MATRIX = 1ll << 22;
constexpr int64_t PILOT_MATRIX_BYTES = 256ll << 20;   // k <= 32: largest pilot sample kept as a key matrix

// columns of the key matrix slice: at most MATRIX_BUDGET_BYTES, at least 1024, never more than the shard
static int64_t matrix_chunk_cols(int64_t nq, int64_t nb) {
    int64_t cols = MATRIX_BUDGET_BYTES / (4 * (nq > 0 ? nq : 1));
    cols &= ~(int64_t)255;
    if (cols < 1024) cols = 1024;
    const int64_t nb_pad = round_up64(nb > 0 ? nb : 1, 256);
    if (cols > nb_pad) cols = nb_pad;
    return cols;
}

bool make_plan(int64_t nq, int64_t nb, int d, int k, int storage, int path, bool pairwise,
               SearchPlan& pl) {
    // the query operand always reserves the 8 norm columns (used for L2 only)
    if (nq < 0 || nb < 0 || d <= 0 || k <= 0 || storage < 0 || storage > 2) return false;
    const int sm = cached_sm_count();
    pl = SearchPlan{};
    pl.path = path;
    // the streaming scans take up to 8 queries per pass, which beats a 128-row tensor tile that is
    // mostly padding (measured on 12.5 M fp32 rows of d = 128, 8 queries: 1.1 against 4.1 ms); fp32
    // shards under 64 Ki rows or wider than the streaming kernel takes: 4 per pass (the reference's
    // limit, src/MetalDistance.mm:346-354)
    const bool f32_stream = nb >= F32_STREAM_MIN_ROWS && d <= F32_STREAM_MAX_D;
    const int64_t scan_limit = (storage == B200F_STORAGE_F32 && !f32_stream) ? SCAN_GROUP : 2 * SCAN_GROUP;
    if (path == B200F_PATH_AUTO) pl.path = (nq <= scan_limit) ? B200F_PATH_SCAN : B200F_PATH_TENSOR;
    pl.fused = (k <= B200F_FUSED_MAX_K) && !pairwise;
    pl.npl = (storage == B200F_STORAGE_F32) ? 3 : 1;
    pl.a_pitch = round_up64(d, 8) + 8;
    pl.a_plane_stride = round_up64((nq > 0 ? nq : 1) * pl.a_pitch, 128);
    pl.ngroups = ceil_div64(nq, SCAN_GROUP);
    size_t off = 0;
    const bool canaries = g_canaries.load(std::memory_order_relaxed) != 0;
    // every slice ends on a 256-byte boundary; with canaries on, a guard follows it
    auto adv = [&](size_t bytes) {
        off += align256(bytes);
        if (canaries && pl.nguards < kMaxGuards) {
            pl.guard_off[pl.nguards++] = (uint32_t)(off / 256);
            off += 256;
        }
    };
    pl.off_qnorm = off;
    adv((size_t)(nq > 0 ? nq : 1) * 4);
    pl.off_qscale = off;   // per-row key scales of the fp16x2 plane format
    adv((size_t)(nq > 0 ? nq : 1) * 4);
    pl.gslots = 1;
    if (!pairwise && pl.path == B200F_PATH_TENSOR && k <= B200F_LIST_MAX_K && !filter_disabled()) {
        // The pilot sample holds nb / stride rows and, on average, e = k / stride of a query's k
        // best.  The threshold is the sample's r-th best key with r = e + 4.5 sqrt(e) + 3: fewer
        // than k rows of the shard lie under it only if the sample caught r of the k best, which
        // is about one row in a million; about r * stride rows do lie under it.
        const int stride = k <= 128 ? 64 : 128;
        // with the pilot sample kept as a key matrix (no list warm-up) the filter wins from far
        // fewer pairs: measured 26 - 36 % faster than the lists at 3e7 - 1.3e8 pairs (d = 128, k = 10)
        int64_t min_pairs = FILTER_MIN_PAIRS;
        if (nb >= (int64_t)stride * 1024 && rank_select_enabled()) {
            const GemmPlan g0 = plan_gemm(nq, nb, sm);
            const int64_t pcols = ceil_div64(g0.ntiles, stride) * g0.tile_n;
            const int64_t n1 = nq > 0 ? nq : 1;
            const bool as_matrix = (k <= B200F_FUSED_MAX_K) ? n1 * pcols * 4 <= PILOT_MATRIX_BYTES
                                                            : pcols <= matrix_chunk_cols(nq, nb);
            if (as_matrix) min_pairs = FILTER_MIN_PAIRS_MATRIX;
        }
        if (nb >= (int64_t)stride * 1024 && (nq * nb >= min_pairs || filter_forced())) {
            const double e = (double)k / stride;
            int r = (int)(e + 4.5 * std::sqrt(e) + 3.0 + 0.999);
            if (r > B200F_FUSED_MAX_K) r = B200F_FUSED_MAX_K;
            int cap = 1024;
            while (cap < 4 * r * stride && cap < 8192) cap <<= 1;
            pl.filter = true;
            pl.fstride = stride;
            pl.frank = r;
            pl.fcap = cap;
        }
    }
    if (!pl.filter && !pl.fused && !pairwise && pl.path == B200F_PATH_TENSOR && k <= B200F_LIST_MAX_K &&
        !lists_disabled()) {
        // lists must be able to hold the result four times over, else the fallback would be the rule
        const GemmPlan g = plan_gemm(nq, nb, sm);
        if ((int64_t)2 * g.P * B200F_FUSED_MAX_K >= 4 * (int64_t)k) {
            pl.lists = true;
            pl.gslots = (k + B200F_FUSED_MAX_K - 1) / B200F_FUSED_MAX_K;
        }
    }
    pl.off_gthr = off;
    adv((size_t)(nq > 0 ? nq : 1) * pl.gslots * 4);
    if (pl.path == B200F_PATH_TENSOR) {
        pl.off_a = off;
        adv((size_t)pl.npl * pl.a_plane_stride * 2);
    }
    if (pairwise) {
        pl.gemm = plan_gemm(nq, nb, sm);
        pl.total = off;
        return true;
    }
    if (pl.fused || pl.lists) {
        const int kl = pl.fused ? k : B200F_FUSED_MAX_K;  // entries per list
        int64_t P;
        if (pl.path == B200F_PATH_TENSOR) {
            pl.gemm = plan_gemm(nq, nb, sm);
            P = 2 * pl.gemm.P;  // the tensor kernel writes two lists per column range
        } else {
            pl.scan = plan_scan(nq, nb, d, storage, sm);
            // room for either scan kernel: the streaming one writes one list per SM
            P = pl.scan.grid > sm ? pl.scan.grid : sm;
        }
        if (P < 1) P = 1;
        pl.off_part_key = off;
        adv((size_t)(nq > 0 ? nq : 1) * P * kl * 4);
        pl.off_part_idx = off;
        adv((size_t)(nq > 0 ? nq : 1) * P * kl * 4);
    }
    if (pl.filter) {
        const int64_t n1 = nq > 0 ? nq : 1;
        if (!pl.fused) pl.gemm = plan_gemm(nq, nb, sm);
        pl.pilot = plan_gemm(nq, ceil_div64(pl.gemm.ntiles, pl.fstride) * pl.gemm.tile_n, sm);
        pl.off_pilot_key = off;
        adv((size_t)n1 * 2 * (pl.pilot.P > 0 ? pl.pilot.P : 1) * pl.frank * 4);
        pl.off_pilot_idx = off;
        adv((size_t)n1 * 2 * (pl.pilot.P > 0 ? pl.pilot.P : 1) * pl.frank * 4);
        pl.off_thr = off;
        adv((size_t)n1 * pl.frank * 4);
        pl.off_cand_key = off;
        adv((size_t)n1 * pl.fcap * 4);
        pl.off_cand_idx = off;
        adv((size_t)n1 * pl.fcap * 4);
        pl.off_cand_cnt = off;
        adv((size_t)n1 * 4);
    }
    if (pl.filter && pl.fused && rank_select_enabled()) {
        // k <= 32 has no matrix slice of its own: a small one for the pilot sample alone (the lists'
        // first-tile cost, ~0.1 ms per work item, is most of a small search)
        const int64_t pcols = pl.pilot.ntiles * pl.pilot.tile_n;
        const int64_t n1 = nq > 0 ? nq : 1;
        if (pcols > 0 && n1 * pcols * 4 <= PILOT_MATRIX_BYTES) {
            pl.pilot_matrix = true;
            pl.off_matrix = off;
            adv((size_t)(n1 * pcols * 4));
        }
    }
    if (pl.lists || pl.filter) {
        pl.off_dirty = off;
        adv((size_t)(nq > 0 ? nq : 1) * 4);
        pl.off_rows = off;
        adv((size_t)(nq > 0 ? nq : 1) * 4);
        pl.off_count = off;
        adv(256);
        pl.off_a2 = off;
        adv((size_t)pl.npl * pl.a_plane_stride * 2);
    }
    if (!pl.fused) {
        const int64_t cols = matrix_chunk_cols(nq, nb);
        pl.chunk_cols = cols;
        if (!pl.lists && !pl.filter) pl.gemm = plan_gemm(nq, cols, sm);
        // A list starts empty and takes every key of its first tile: ~0.1 ms per work item, and a
        // small shard's pilot is all first tiles.  Where the sample's keys fit the matrix slice
        // they are written out instead and the frank best picked by a selection kernel.
        pl.pilot_matrix = pl.filter && rank_select_enabled() &&
                          pl.pilot.ntiles * pl.pilot.tile_n <= cols;
        pl.off_matrix = off;
        adv((size_t)(nq > 0 ? nq : 1) * cols * 4);
        pl.off_run_key = off;
        adv((size_t)(nq > 0 ? nq : 1) * k * 4);
        pl.off_run_idx = off;
        adv((size_t)(nq > 0 ? nq : 1) * k * 4);
    }
    pl.total = off;
    return true;
}

__global__ void fill_pad_kernel(float* dist, int64_t* labels, int64_t n, float pad) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        dist[i] = pad;
        labels[i] = -1;
    }
}

// scan path of b200f_pairwise: keys -> scores
__global__ void finish_matrix_kernel(float* m, int64_t nq, int64_t ncols, int64_t ld, float sign,
                                     const float* qnorm) {
    const int64_t total = nq * ncols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t q = i / ncols;
        const int64_t c = i - q * ncols;
        m[q * ld + c] = sign * m[q * ld + c] + (qnorm ? qnorm[q] : 0.f);
    }
}

int validate(const B200FSearchArgs* a, bool pairwise) {
    if (!a) return B200F_ERR_BAD_ARG;
    if (a->nq < 0 || a->nb < 0 || a->d <= 0) return B200F_ERR_BAD_ARG;
    if (a->storage < 0 || a->storage > 2) return B200F_ERR_BAD_ARG;
    if (a->metric != B200F_METRIC_L2 && a->metric != B200F_METRIC_INNER_PRODUCT)
        return B200F_ERR_BAD_ARG;
    if (!pairwise && a->k <= 0) return B200F_ERR_BAD_ARG;
    if (!pairwise && a->k > B200F_MAX_K) return B200F_ERR_UNSUPPORTED;
    if (a->nb > 0x7fffffffLL) return B200F_ERR_UNSUPPORTED;  // int32 row numbers inside a shard
    if (a->path < B200F_PATH_AUTO || a->path > B200F_PATH_TENSOR) return B200F_ERR_BAD_ARG;
    if (a->plane_format != B200F_PLANES_BF16X3 && a->plane_format != B200F_PLANES_FP16X2) return B200F_ERR_BAD_ARG;
    if (a->plane_scale_log2 < -126 || a->plane_scale_log2 > 126) return B200F_ERR_BAD_ARG;
    if (a->nq > 0 && !a->queries) return B200F_ERR_BAD_ARG;
    if (!pairwise && a->nq > 0 && (!a->out_dist || !a->out_labels)) return B200F_ERR_BAD_ARG;
    if (a->nb > 0) {
        if (!a->rows) return B200F_ERR_BAD_ARG;
        const int e = a->storage == B200F_STORAGE_F32 ? 4 : 8;
        if (a->row_pitch < a->d || (a->row_pitch % e) != 0 ||
            (reinterpret_cast<uintptr_t>(a->rows) & 15) != 0)
            return B200F_ERR_BAD_ARG;
        if (a->metric == B200F_METRIC_L2 && !a->norms) return B200F_ERR_BAD_ARG;
    }
    if ((reinterpret_cast<uintptr_t>(a->scratch) & 255) != 0) return B200F_ERR_BAD_ARG;
    return B200F_OK;
}

int fill_operands(const B200FSearchArgs& a, const SearchPlan& pl, uint8_t* scratch,
                  GemmOperands& op) {
    op.a_planes = reinterpret_cast<const uint16_t*>(scratch + pl.off_a);
    op.a_pitch = pl.a_pitch;
    op.a_plane_stride = pl.a_plane_stride;
    op.npl = pl.npl;
    op.nq = a.nq;
    op.nb = a.nb;
    const bool l2 = a.metric == B200F_METRIC_L2;
    if (l2 && !a.norm_cols) return B200F_ERR_BAD_ARG;  // the tensor path takes ||x||^2 from the rows
    op.d_pad = (int)round_up64(a.d, 8) + (l2 ? 8 : 0);
    if (a.storage == B200F_STORAGE_F32) {
        if (!a.planes || a.plane_pitch < op.d_pad || (a.plane_pitch % 8) != 0 ||
            (a.plane_stride % 8) != 0)
            return B200F_ERR_BAD_ARG;
        op.b_planes = a.planes;
        op.b_pitch = a.plane_pitch;
        op.b_plane_stride = a.plane_stride;
        if (a.plane_format == B200F_PLANES_FP16X2) {
            op.npl = 2;
            op.is_bf16 = 0;
            op.rowscale = reinterpret_cast<const float*>(scratch + pl.off_qscale);
        } else {
            op.is_bf16 = 1;
        }
    } else {
        if (a.row_pitch < op.d_pad) return B200F_ERR_BAD_ARG;
        op.b_planes = reinterpret_cast<const uint16_t*>(a.rows);
        op.b_pitch = a.row_pitch;
        op.b_plane_stride = 0;
        op.is_bf16 = a.storage == B200F_STORAGE_BF16;
    }
    return B200F_OK;
}

}  // namespace

void count_launch(int n) {
    std::lock_guard<std::mutex> g(g_prof_mu);
    g_prof.launches += n;
}

void main_kernel_begin(cudaStream_t stream) {
    std::lock_guard<std::mutex> g(g_prof_mu);
    if (!g_prof.enabled) return;
    // a launch that is being captured into a graph is not timed (its events would belong to the graph)
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        (void)cudaGetLastError();
        return;
    }
    std::pair<cudaEvent_t, cudaEvent_t> ev;
    if (!g_prof.pool.empty()) {
        ev = g_prof.pool.back();
        g_prof.pool.pop_back();
    } else {
        if (cudaEventCreate(&ev.first) != cudaSuccess || cudaEventCreate(&ev.second) != cudaSuccess) {
            (void)cudaGetLastError();
            return;
        }
    }
    cudaEventRecord(ev.first, stream);
    g_prof.pending.push_back(ev);
}

void main_kernel_end(cudaStream_t stream) {
    std::lock_guard<std::mutex> g(g_prof_mu);
    if (!g_prof.enabled || g_prof.pending.empty()) return;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        (void)cudaGetLastError();
        return;
    }
    cudaEventRecord(g_prof.pending.back().second, stream);
}

}  // namespace b200f

using namespace b200f;

extern "C" int b200f_profile_enable(int on) {
    std::lock_guard<std::mutex> g(g_prof_mu);
    g_prof.enabled = on != 0;
    return B200F_OK;
}

extern "C" int b200f_profile_read(int64_t* launches, int64_t* main_launches, double* main_ms,
                                  int reset) {
    std::lock_guard<std::mutex> g(g_prof_mu);
    for (auto& ev : g_prof.pending) {
        float ms = 0.f;
        if (cudaEventSynchronize(ev.second) == cudaSuccess &&
            cudaEventElapsedTime(&ms, ev.first, ev.second) == cudaSuccess) {
            g_prof.main_ms += ms;
            g_prof.main_launches++;
        } else {
            (void)cudaGetLastError();
        }
        g_prof.pool.push_back(ev);
    }
    g_prof.pending.clear();
    if (launches) *launches = g_prof.launches;
    if (main_launches) *main_launches = g_prof.main_launches;
    if (main_ms) *main_ms = g_prof.main_ms;
    if (reset) {
        g_prof.launches = 0;
        g_prof.main_launches = 0;
        g_prof.main_ms = 0.0;
    }
    return B200F_OK;
}

extern "C" int b200f_set_selection_mode(int mode) {
    if (mode < B200F_SELECT_AUTO || mode > B200F_SELECT_MATRIX) return B200F_ERR_BAD_ARG;
    g_select_mode.store(mode, std::memory_order_relaxed);
    return B200F_OK;
}

extern "C" int b200f_get_selection_mode(void) { return select_mode(); }

// One CTA waits, with the library's bounded-wait helper, on an mbarrier that nothing arrives
// at.  The wait runs out after limit_cycles, the status word gets kDevErrBarrierWait and the
// kernel returns normally: the expiry path without any fault.
__global__ void wait_expiry_kernel(int32_t* status, long long limit_cycles) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        mbar_fence_init();
    }
    __syncthreads();
    // every thread of the warp waits: the first one to give up raises the abort flag, the
    // others leave through it, as the roles of the search kernels do
    (void)mbar_wait_bounded(smem_u32(&bar), 0, &abort_flag, status, kDevErrBarrierWait, limit_cycles);
    __syncthreads();
}

extern "C" int b200f_debug_wait_expiry(int32_t* status, int64_t limit_cycles, void* stream) {
    if (!status || limit_cycles < 1 || limit_cycles > kWaitLimitCycles) return B200F_ERR_BAD_ARG;
    wait_expiry_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, (long long)limit_cycles);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

extern "C" int b200f_set_debug_canaries(int on) {
    g_canaries.store(on ? 1 : 0, std::memory_order_relaxed);
    return B200F_OK;
}

extern "C" const char* b200f_status_string(int status) {
    switch (status) {
        case B200F_OK: return "ok";
        case B200F_ERR_BAD_ARG: return "bad argument";
        case B200F_ERR_UNSUPPORTED: return "unsupported size (k > 4096 or more than 2^31-1 rows in a shard)";
        case B200F_ERR_SCRATCH: return "scratch buffer too small";
        case B200F_ERR_CUDA: return "CUDA call failed";
        case B200F_ERR_DEVICE_WAIT: return "a bounded device-side wait ran out";
        case B200F_ERR_NO_DEVICE: return "no sm_100 device (there is no CPU fallback)";
        case B200F_ERR_OOM: return "out of device or pinned host memory";
        case B200F_ERR_RANGE: return "key out of range";
        case B200F_ERR_STATE: return "token already consumed";
        case B200F_ERR_DEVICE_CHECK: return "a device-side self-check failed";
    }
    return "unknown status";
}

extern "C" int b200f_device_count(int* count) {
    if (!count) return B200F_ERR_BAD_ARG;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        *count = 0;
        return B200F_ERR_NO_DEVICE;
    }
    *count = n;
    return B200F_OK;
}

extern "C" int b200f_device_caps(int device, B200FCaps* caps) {
    if (!caps) return B200F_ERR_BAD_ARG;
    std::memset(caps, 0, sizeof(*caps));
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        (void)cudaGetLastError();
        return B200F_ERR_NO_DEVICE;
    }
    if (device < 0) {
        if (cudaGetDevice(&device) != cudaSuccess) return B200F_ERR_CUDA;
    }
    if (device >= n) return B200F_ERR_BAD_ARG;
    cudaDeviceProp prop;
    B200F_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    caps->device = device;
    caps->cc_major = prop.major;
    caps->cc_minor = prop.minor;
    caps->sm_count = prop.multiProcessorCount;
    caps->max_smem_per_block = (int32_t)prop.sharedMemPerBlockOptin;
    caps->l2_bytes = prop.l2CacheSize;
    caps->hbm_bytes = (int64_t)prop.totalGlobalMem;
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, device) == cudaSuccess) caps->sm_clock_khz = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, device) == cudaSuccess) caps->mem_clock_khz = v;
    (void)cudaGetLastError();
    caps->supported = (prop.major == 10) ? 1 : 0;
    std::snprintf(caps->name, sizeof(caps->name), "%s", prop.name);
    return B200F_OK;
}

extern "C" size_t b200f_search_scratch_bytes(int64_t nq, int64_t nb, int d, int k, int storage,
                                             int path) {
    SearchPlan pl;
    if (!make_plan(nq, nb, d, k, storage, path, false, pl)) return 0;
    return pl.total + 256;
}

// Debug canaries: the guards behind the scratch slices are filled before the search and
// compared after it; a changed word means some kernel wrote past its slice.  status == nullptr
// fills, otherwise checks (status[0] |= kDevErrCanary, status[2] = 1 + number of the first bad guard).
struct GuardList {
    int n;
    uint32_t off[kMaxGuards];
};
__global__ void canary_kernel(uint8_t* scratch, GuardList g, int32_t* status) {
    const int gi = blockIdx.x;
    if (gi >= g.n) return;
    uint32_t* w = reinterpret_cast<uint32_t*>(scratch + (size_t)g.off[gi] * 256);
    const int t = threadIdx.x;   // 64 threads: one word each
    if (!status) {
        w[t] = kCanaryWord ^ (uint32_t)(gi * 64 + t);
    } else if (w[t] != (kCanaryWord ^ (uint32_t)(gi * 64 + t))) {
        atomicOr(status, kDevErrCanary);
        atomicMax(status + 2, gi + 1);
    }
}
static int launch_canaries(const SearchPlan& pl, uint8_t* scratch, int32_t* status, cudaStream_t st) {
    GuardList g;
    g.n = pl.nguards;
    for (int i = 0; i < kMaxGuards; i++) g.off[i] = i < pl.nguards ? pl.guard_off[i] : 0;
    if (status == nullptr) {
        canary_kernel<<<g.n, 64, 0, st>>>(scratch, g, nullptr);
    } else {
        canary_kernel<<<g.n, 64, 0, st>>>(scratch, g, status);
    }
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

static int run_search(const B200FSearchArgs* a, const SearchPlan& pl);

extern "C" int b200f_search(const B200FSearchArgs* a) {
    int rc = validate(a, false);
    if (rc != B200F_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(a->stream);
    if (a->nq == 0) return B200F_OK;
    if (a->status) B200F_CUDA_TRY(cudaMemsetAsync(a->status, 0, 4 * sizeof(int32_t), st));
    const bool l2 = a->metric == B200F_METRIC_L2;
    if (a->nb == 0) {
        const int64_t n = a->nq * a->k;
        fill_pad_kernel<<<(int)(ceil_div64(n, 256) < 1024 ? ceil_div64(n, 256) : 1024), 256, 0, st>>>(
                a->out_dist, a->out_labels, n, l2 ? kHostInf : -kHostInf);
        count_launch();
        B200F_LAUNCH_CHECK();
        return B200F_OK;
    }
    SearchPlan pl;
    if (!make_plan(a->nq, a->nb, a->d, a->k, a->storage, a->path, false, pl)) return B200F_ERR_BAD_ARG;
    if (!a->scratch || a->scratch_bytes < pl.total) return B200F_ERR_SCRATCH;
    if (pl.nguards > 0) {
        rc = launch_canaries(pl, static_cast<uint8_t*>(a->scratch), nullptr, st);
        if (rc != B200F_OK) return rc;
    }
    rc = run_search(a, pl);
    if (rc == B200F_OK && pl.nguards > 0 && a->status)
        rc = launch_canaries(pl, static_cast<uint8_t*>(a->scratch), a->status, st);
    return rc;
}

// The kernel sequence of one planned search (everything is enqueued on a->stream).
static int run_search(const B200FSearchArgs* a, const SearchPlan& pl) {
    int rc = B200F_OK;
    cudaStream_t st = static_cast<cudaStream_t>(a->stream);
    const bool l2 = a->metric == B200F_METRIC_L2;
    uint8_t* scratch = static_cast<uint8_t*>(a->scratch);
    float* qnorm = reinterpret_cast<float*>(scratch + pl.off_qnorm);
    const int sm = cached_sm_count();
    const float kscale = l2 ? 2.f : 1.f;
    const int qnc = l2 ? 1 : 0;

    GemmOperands op{};
    if (pl.path == B200F_PATH_TENSOR) {
        rc = fill_operands(*a, pl, scratch, op);
        if (rc != B200F_OK) return rc;
        rc = launch_prepare_queries(a->queries, a->nq, a->d, a->storage,
                                    reinterpret_cast<uint16_t*>(scratch + pl.off_a), pl.a_pitch,
                                    pl.a_plane_stride, qnorm, qnc, a->plane_format, a->plane_scale_log2,
                                    reinterpret_cast<float*>(scratch + pl.off_qscale), st);
    } else {
        rc = launch_prepare_queries(a->queries, a->nq, a->d, a->storage, nullptr, 0, 0, qnorm, 0, 0, 0, nullptr, st);
    }
    if (rc != B200F_OK) return rc;

    // rows (counted and listed on the device) that an optimistic stage could not prove exact
    const int* nq_dev = nullptr;
    const int32_t* row_map = nullptr;
    uint32_t* gthr = reinterpret_cast<uint32_t*>(scratch + pl.off_gthr);
    auto redo_setup = [&](int32_t* dirty) -> int {
        int32_t* rows = reinterpret_cast<int32_t*>(scratch + pl.off_rows);
        int32_t* count = reinterpret_cast<int32_t*>(scratch + pl.off_count);
        uint16_t* a2 = reinterpret_cast<uint16_t*>(scratch + pl.off_a2);
        // the number of redone rows is left in status word 1 for whoever wants to know
        int r2 = launch_compact_rows(dirty, a->nq, rows, count, a->status ? a->status + 1 : nullptr, st);
        if (r2 != B200F_OK) return r2;
        r2 = launch_gather_rows(op.a_planes, op.npl, op.a_plane_stride, op.a_pitch, rows, count, a->nq,
                                a2, st);
        if (r2 != B200F_OK) return r2;
        op.a_planes = a2;
        op.rowscale_map = rows;   // row j of the gathered operand is query rows[j]
        op.nq_dev = count;
        nq_dev = count;
        row_map = rows;
        return B200F_OK;
    };

    if (pl.filter) {
        float* pkey = reinterpret_cast<float*>(scratch + pl.off_pilot_key);
        int32_t* pidx = reinterpret_cast<int32_t*>(scratch + pl.off_pilot_idx);
        float* thr = reinterpret_cast<float*>(scratch + pl.off_thr);
        float* ckey = reinterpret_cast<float*>(scratch + pl.off_cand_key);
        int32_t* cidx = reinterpret_cast<int32_t*>(scratch + pl.off_cand_idx);
        int32_t* ccnt = reinterpret_cast<int32_t*>(scratch + pl.off_cand_cnt);
        int32_t* dirty = reinterpret_cast<int32_t*>(scratch + pl.off_dirty);
        if (pl.pilot_matrix) {
            // every fstride-th column tile, side by side in the matrix slice; the last one may be partial
            float* matrix = reinterpret_cast<float*>(scratch + pl.off_matrix);
            const int64_t pcols = pl.pilot.ntiles * pl.pilot.tile_n;
            const int64_t last0 = (pl.pilot.ntiles - 1) * pl.fstride * pl.pilot.tile_n;
            int64_t last_valid = a->nb - last0;
            if (last_valid > pl.pilot.tile_n) last_valid = pl.pilot.tile_n;
            const int64_t valid = (pl.pilot.ntiles - 1) * pl.pilot.tile_n + last_valid;
            rc = launch_gemm_store(op, pl.pilot, 0, a->nb, pl.fstride, kscale, 1.f, nullptr, matrix, pcols,
                                   a->status, st);
            if (rc != B200F_OK) return rc;
            rc = launch_select_keys(matrix, a->nq, valid, pcols, pl.frank, thr, st);
            if (rc != B200F_OK) return rc;
        } else {
            rc = launch_gemm_topk(op, pl.pilot, 0, a->nb, pl.fstride, kscale, pl.frank, 1, pkey, pidx, gthr,
                                  a->status, st);
            if (rc != B200F_OK) return rc;
            rc = launch_merge_keys(pkey, pidx, 2 * pl.pilot.P, a->nq, pl.frank, thr, st);
            if (rc != B200F_OK) return rc;
        }
        // candidates per row ~ frank * fstride: a few hundred for k <= 128, thousands beyond
        rc = launch_gemm_filter(op, pl.gemm, kscale, thr, pl.frank, pl.frank - 1, ckey, cidx, ccnt,
                                pl.fcap, pl.fstride == 64 ? 1 : 0, a->status, st);
        if (rc != B200F_OK) return rc;
        rc = launch_select_candidates(ckey, cidx, ccnt, pl.fcap, a->nb, a->nq, a->k, a->metric, qnorm,
                                      a->label_base, a->out_dist, a->out_labels, dirty, st);
        if (rc != B200F_OK) return rc;
        rc = redo_setup(dirty);
        if (rc != B200F_OK) return rc;
    }

    if (pl.fused) {
        float* part_key = reinterpret_cast<float*>(scratch + pl.off_part_key);
        int32_t* part_idx = reinterpret_cast<int32_t*>(scratch + pl.off_part_idx);
        int P;
        if (pl.path == B200F_PATH_TENSOR) {
            P = 2 * pl.gemm.P;
            rc = launch_gemm_topk(op, pl.gemm, 0, a->nb, 1, kscale, a->k, 1, part_key, part_idx, gthr,
                                  a->status, st);
            if (rc != B200F_OK) return rc;
        } else {
            // every group of queries writes the same number of lists (same shard, same
            // geometry); the first launch reports it.  Groups of 8 where a streaming kernel
            // applies (shard large enough), else of 4.
            P = pl.scan.grid;
            // FP32 rows: the streaming tf32 kernel for two queries and more (7.1 - 6.1 TB/s for 2 - 8
            // per pass; the FMA kernel: 6.9 / 5.6 / 4.1 TB/s for 1 / 2 / 4)
            const bool stream_f32 = a->nq >= 2;
            int64_t group = a->nq > SCAN_GROUP ? 2 * SCAN_GROUP : SCAN_GROUP;
            for (int64_t q0 = 0; q0 < a->nq;) {
                B200FSearchArgs sub = *a;
                sub.queries = a->queries + q0 * (int64_t)a->d;
                sub.nq = (a->nq - q0) < group ? (a->nq - q0) : group;
                int Pg = P;
                rc = launch_scan_topk(sub, pl.scan, part_key + q0 * (int64_t)P * a->k,
                                      part_idx + q0 * (int64_t)P * a->k, &Pg, stream_f32, st);
                if (rc == B200F_ERR_UNSUPPORTED && q0 == 0 && group > SCAN_GROUP) {
                    group = SCAN_GROUP;  // no streaming kernel for this shape: nothing was launched
                    continue;
                }
                if (rc != B200F_OK) return rc;
                if (q0 == 0) P = Pg;
                q0 += sub.nq;
            }
        }
        return launch_merge_partials(part_key, part_idx, P, a->nq, a->k, a->metric, qnorm,
                                     a->label_base, a->out_dist, a->out_labels, nq_dev, row_map, st);
    }

    // k > 32 from 32-entry lists: select, find the rows that are not proven exact, and send only
    // those (gathered into a second query operand, counted on the device) through the key matrix
    if (pl.lists) {
        float* part_key = reinterpret_cast<float*>(scratch + pl.off_part_key);
        int32_t* part_idx = reinterpret_cast<int32_t*>(scratch + pl.off_part_idx);
        int32_t* dirty = reinterpret_cast<int32_t*>(scratch + pl.off_dirty);
        rc = launch_gemm_topk(op, pl.gemm, 0, a->nb, 1, kscale, B200F_FUSED_MAX_K, pl.gslots, part_key,
                              part_idx, gthr, a->status, st);
        if (rc != B200F_OK) return rc;
        rc = launch_select_parts(part_key, part_idx, 2 * pl.gemm.P, a->nq, a->k, a->metric, qnorm,
                                 a->label_base, a->out_dist, a->out_labels, dirty, st);
        if (rc != B200F_OK) return rc;
        rc = redo_setup(dirty);
        if (rc != B200F_OK) return rc;
    }

    // k > 32: distance keys per column chunk + running selection
    float* matrix = reinterpret_cast<float*>(scratch + pl.off_matrix);
    float* run_key = reinterpret_cast<float*>(scratch + pl.off_run_key);
    int32_t* run_idx = reinterpret_cast<int32_t*>(scratch + pl.off_run_idx);
    int has_prev = 0;
    for (int64_t c0 = 0; c0 < a->nb; c0 += pl.chunk_cols) {
        const int64_t nc = (a->nb - c0) < pl.chunk_cols ? (a->nb - c0) : pl.chunk_cols;
        if (pl.path == B200F_PATH_TENSOR) {
            GemmPlan g = plan_gemm(a->nq, nc, sm);
            rc = launch_gemm_store(op, g, c0, nc, 1, kscale, 1.f, nullptr, matrix, pl.chunk_cols,
                                   a->status, st);
            if (rc != B200F_OK) return rc;
        } else {
            for (int64_t g = 0; g < pl.ngroups; g++) {
                B200FSearchArgs sub = *a;
                sub.queries = a->queries + g * SCAN_GROUP * (int64_t)a->d;
                sub.nq = (a->nq - g * SCAN_GROUP) < SCAN_GROUP ? (a->nq - g * SCAN_GROUP) : SCAN_GROUP;
                rc = launch_scan_store(sub, c0, nc, matrix + g * SCAN_GROUP * pl.chunk_cols,
                                       pl.chunk_cols, sm, st);
                if (rc != B200F_OK) return rc;
            }
        }
        rc = launch_select_chunk(matrix, a->nq, nc, pl.chunk_cols, c0, a->k, has_prev, run_key,
                                 run_idx, nq_dev, st);
        if (rc != B200F_OK) return rc;
        has_prev = 1;
    }
    return launch_finalize_lists(run_key, run_idx, a->nq, a->k, a->metric, qnorm, a->label_base,
                                 a->out_dist, a->out_labels, nq_dev, row_map, st);
}

__global__ void poke_kernel(uint32_t* word) { *word = 0; }

extern "C" int b200f_debug_canary_selftest(void* scratch, size_t scratch_bytes, int corrupt, int32_t* status,
                                           void* stream) {
    if (!scratch || scratch_bytes < 4 * 1024 || !status || (reinterpret_cast<uintptr_t>(scratch) & 255) != 0)
        return B200F_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    SearchPlan pl{};
    pl.nguards = 3;
    pl.guard_off[0] = 1;   // guards at bytes 256, 1536 and 3584 of the region
    pl.guard_off[1] = 6;
    pl.guard_off[2] = 14;
    int rc = launch_canaries(pl, static_cast<uint8_t*>(scratch), nullptr, st);
    if (rc != B200F_OK) return rc;
    if (corrupt) {   // what a kernel running past its slice would do: one word of guard 1
        poke_kernel<<<1, 1, 0, st>>>(reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(scratch) + 6 * 256 + 40));
        B200F_LAUNCH_CHECK();
    }
    return launch_canaries(pl, static_cast<uint8_t*>(scratch), status, st);
}

extern "C" int b200f_pairwise(const B200FSearchArgs* a, float* out_matrix, int64_t ld_out) {
    int rc = validate(a, true);
    if (rc != B200F_OK) return rc;
    if (a->nq == 0 || a->nb == 0) return B200F_OK;
    if (!out_matrix || ld_out < a->nb) return B200F_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(a->stream);
    if (a->status) B200F_CUDA_TRY(cudaMemsetAsync(a->status, 0, 4 * sizeof(int32_t), st));
    SearchPlan pl;
    if (!make_plan(a->nq, a->nb, a->d, 1, a->storage, a->path, true, pl)) return B200F_ERR_BAD_ARG;
    if (!a->scratch || a->scratch_bytes < pl.total) return B200F_ERR_SCRATCH;
    uint8_t* scratch = static_cast<uint8_t*>(a->scratch);
    float* qnorm = reinterpret_cast<float*>(scratch + pl.off_qnorm);
    const bool l2 = a->metric == B200F_METRIC_L2;
    const float kscale = l2 ? 2.f : 1.f;
    const int sm = cached_sm_count();
    if (pl.path == B200F_PATH_TENSOR) {
        GemmOperands op{};
        rc = fill_operands(*a, pl, scratch, op);
        if (rc != B200F_OK) return rc;
        rc = launch_prepare_queries(a->queries, a->nq, a->d, a->storage,
                                    reinterpret_cast<uint16_t*>(scratch + pl.off_a), pl.a_pitch,
                                    pl.a_plane_stride, qnorm, l2 ? 1 : 0, a->plane_format, a->plane_scale_log2,
                                    reinterpret_cast<float*>(scratch + pl.off_qscale), st);
        if (rc != B200F_OK) return rc;
        return launch_gemm_store(op, pl.gemm, 0, a->nb, 1, kscale, l2 ? 1.f : -1.f,
                                 l2 ? qnorm : nullptr, out_matrix, ld_out, a->status, st);
    }
    rc = launch_prepare_queries(a->queries, a->nq, a->d, a->storage, nullptr, 0, 0, qnorm, 0, 0, 0, nullptr, st);
    if (rc != B200F_OK) return rc;
    for (int64_t g = 0; g < pl.ngroups; g++) {
        B200FSearchArgs sub = *a;
        sub.queries = a->queries + g * SCAN_GROUP * (int64_t)a->d;
        sub.nq = (a->nq - g * SCAN_GROUP) < SCAN_GROUP ? (a->nq - g * SCAN_GROUP) : SCAN_GROUP;
        rc = launch_scan_store(sub, 0, a->nb, out_matrix + g * SCAN_GROUP * ld_out, ld_out, sm, st);
        if (rc != B200F_OK) return rc;
    }
    const int64_t total = a->nq * a->nb;
    int64_t g = ceil_div64(total, 256);
    if (g > (int64_t)sm * 16) g = (int64_t)sm * 16;
    finish_matrix_kernel<<<(int)g, 256, 0, st>>>(out_matrix, a->nq, a->nb, ld_out, l2 ? 1.f : -1.f,
                                                 l2 ? qnorm : nullptr);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

// ---------------------------------------------------------------------------------------
// Search without any allocation
// ---------------------------------------------------------------------------------------
namespace {

// Scratch of b200f_search_small_noalloc: lives in the module image of every GPU that loads
// the library until the process exits.  1 MiB covers the streaming-scan path for
// nq <= 4, k <= 32 (query norms + at most 592 partial lists of 32 entries per query).
constexpr size_t kNoAllocScratchBytes = 1u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

void* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mu;

// Device address of the array on the CURRENT device.  In host code the symbol's name is only
// a stand-in, never an address a kernel may use: the real address is asked for once per device.
int noalloc_scratch_for_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        return B200F_ERR_CUDA;
    }
    std::lock_guard<std::mutex> g(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || !ptr) {
            (void)cudaGetLastError();
            return B200F_ERR_CUDA;
        }
        g_noalloc_ptr[dev] = ptr;
    }
    *out = g_noalloc_ptr[dev];
    return B200F_OK;
}

}  // namespace

extern "C" size_t b200f_noalloc_scratch_capacity(void) { return kNoAllocScratchBytes; }

extern "C" int b200f_search_small_noalloc(const B200FSearchArgs* a) {
    if (!a) return B200F_ERR_BAD_ARG;
    if (a->nq < 0 || a->k < 1) return B200F_ERR_BAD_ARG;   // same codes as b200f_search
    if (a->nq > 4 || a->k > B200F_FUSED_MAX_K) return B200F_ERR_UNSUPPORTED;
    B200FSearchArgs c = *a;
    c.path = B200F_PATH_SCAN;
    const size_t need = b200f_search_scratch_bytes(c.nq, c.nb, c.d, c.k, c.storage, c.path);
    if (need == 0) return B200F_ERR_BAD_ARG;
    if (need > kNoAllocScratchBytes) return B200F_ERR_SCRATCH;  // shape beyond the built-in scratch
    void* ptr = nullptr;
    const int rc = noalloc_scratch_for_current_device(&ptr);
    if (rc != B200F_OK) return rc;
    c.scratch = ptr;
    c.scratch_bytes = kNoAllocScratchBytes;
    return b200f_search(&c);
}
