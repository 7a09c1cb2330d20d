// Shared device/host helpers for the flat k-NN kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../../include/b200_flat.h"

namespace b200f {

constexpr int kNumSMsDefault = 148;
constexpr float kHostInf = __builtin_huge_valf();

// Bits OR-ed into the device status word (B200FSearchArgs::status[0]).
constexpr int kDevErrBarrierWait = 1;   // a bounded mbarrier wait ran out
constexpr int kDevErrSmemAlign = 2;     // dynamic shared memory base not 1024-byte aligned
constexpr int kDevErrOverflow = 4;      // a candidate buffer overflowed (never expected)
constexpr int kDevErrCanary = 8;        // debug canaries: a kernel wrote past its scratch slice

#define B200F_CUDA_TRY(expr)                         \
    do {                                             \
        cudaError_t _e = (expr);                     \
        if (_e != cudaSuccess) {                     \
            (void)cudaGetLastError();                \
            return B200F_ERR_CUDA;                   \
        }                                            \
    } while (0)

#define B200F_LAUNCH_CHECK()                         \
    do {                                             \
        cudaError_t _e = cudaGetLastError();         \
        if (_e != cudaSuccess) return B200F_ERR_CUDA; \
    } while (0)

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ inline int64_t round_up64(int64_t a, int64_t b) { return ceil_div64(a, b) * b; }

// Monotone map float -> uint32 (ascending float order == ascending unsigned order;
// NaN sorts after +INF).
__device__ __forceinline__ uint32_t float_to_ordered(float f) {
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ordered_to_float(uint32_t u) {
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Launchers implemented in the other translation units ------------------------

// rows.cu: queries fp32 [nq][d] -> A planes (16-bit, [npl][nq][d_pad]) + squared norms.
// FP32 storage, plane_format B200F_PLANES_FP16X2: two fp16 planes of the row scaled by its own
// power of two, and rowscale[r] = 1 / (row scale * 2^x_scale_log2) (what turns the kernel's
// accumulator back into key units).  Otherwise rowscale is not written.
int launch_prepare_queries(const float* q, int64_t nq, int d, int storage, uint16_t* a_planes,
                           int64_t a_pitch, int64_t a_plane_stride, float* qnorm, int norm_cols,
                           int plane_format, int x_scale_log2, float* rowscale, cudaStream_t stream);

// scan.cu: streaming search for small nq, k <= 32.  Writes P = *out_P partial lists.
struct ScanPlan {
    int grid;        // CTAs == number of partial lists per query
    int threads;
    int lpr_cap;     // plain kernel: upper limit of the lanes that share one row
};
ScanPlan plan_scan(int64_t nq, int64_t nb, int d, int storage, int sm_count);
// *out_P receives the number of partial lists per query actually written (<= plan.grid).
// stream_f32: FP32 rows may take the streaming tf32 kernel (up to 8 queries); the caller must pass
// the same value for every query group of a search, since the kernels write different list counts.
int launch_scan_topk(const B200FSearchArgs& a, const ScanPlan& plan, float* part_key,
                     int32_t* part_idx, int* out_P, bool stream_f32, cudaStream_t stream);
// Scan that stores keys (smaller = better) to a matrix [nq][ld] for columns [col0, col0+ncols).
int launch_scan_store(const B200FSearchArgs& a, int64_t col0, int64_t ncols, float* out,
                      int64_t ld, int sm_count, cudaStream_t stream);

// gemm_topk.cu
struct GemmPlan {
    int pair;            // 1: CTA pairs (cta_group::2), query blocks of 256 rows
    int nqb;             // query blocks of 128 (256) rows
    int tile_n;          // columns of X per tile: 256, or 512 for pairs
    int64_t ntiles;      // column tiles in the launch
    int P;               // column ranges == partial lists per query
    int64_t tiles_per_range;
    int grid;
};
GemmPlan plan_gemm(int64_t nq, int64_t ncols, int sm_count);
struct GemmOperands {
    const uint16_t* a_planes;  // [npl][nq][a_pitch]
    int64_t a_pitch, a_plane_stride;
    const uint16_t* b_planes;  // [npl][nb][b_pitch]
    int64_t b_pitch, b_plane_stride;
    int npl;                   // 1 (fp16 / bf16 storage), 3 (fp32 storage, bf16 split) or 2 (fp16 split)
    int is_bf16;               // element format of both operands
    const float* rowscale;     // optional, per query row: keys are the accumulator times kscale * rowscale[row]
    const int32_t* rowscale_map;  // optional: row j of A is row rowscale_map[j] of rowscale (redone rows)
    int64_t nq, nb;
    int d_pad;                 // K extent (multiple of 8), norm columns included
    const int* nq_dev;         // optional: live rows of A (<= nq) left in device memory by a kernel
};
// Fused top-k (k <= 32): partial lists part_key/part_idx [nq][2 * P][k] (two per column range).
// gthr holds nq * gslots words; with gslots = s the shared filter bounds the (32 * s)-th best
// key of a row, so lists of k = 32 entries can feed a later selection of up to 32 * s results.
// tile_stride > 1 visits only every tile_stride-th column tile (plan made for that many tiles).
int launch_gemm_topk(const GemmOperands& op, const GemmPlan& plan, int64_t col0, int64_t ncols,
                     int64_t tile_stride, float kscale, int k, int gslots, float* part_key,
                     int32_t* part_idx, uint32_t* gthr, int32_t* status, cudaStream_t stream);
// Threshold filter over the whole shard: column c of row q with scaled key <= thr[q * thr_stride +
// thr_pos] is appended to the row's candidate buffer cand_key/cand_idx [nq][cand_cap] in any
// order; cand_cnt[q] counts every hit, also those beyond cand_cap, which are not stored.
// few_hits: the threshold admits well under one column in a thousand (tunes the scan width).
int launch_gemm_filter(const GemmOperands& op, const GemmPlan& plan, float kscale, const float* thr,
                       int thr_stride, int thr_pos, float* cand_key, int32_t* cand_idx,
                       int32_t* cand_cnt, int cand_cap, int few_hits, int32_t* status,
                       cudaStream_t stream);
// Store mode: out[row*ld + (col-col0)] = sign*(-kscale*t) + rowadd[row], t = q.x (- ||x||^2/2).
// tile_stride > 1 visits only every tile_stride-th column tile (plan made for that many tiles);
// the visited tiles lie side by side in out.
int launch_gemm_store(const GemmOperands& op, const GemmPlan& plan, int64_t col0, int64_t ncols,
                      int64_t tile_stride, float kscale, float sign, const float* rowadd, float* out,
                      int64_t ld, int32_t* status, cudaStream_t stream);

// select.cu
// Merge P sorted partial lists (key smaller=better, int32 local ids; -1 = empty) per
// query and finalise: L2 dist = max(key + qnorm, 0), IP dist = -key; labels = id + base.
// nq_dev / row_map (optional): live rows counted on the device; lists of row j belong to query
// row_map[j].  out_labels may be null (keys only).
int launch_merge_partials(const float* part_key, const int32_t* part_idx, int P, int64_t nq, int k,
                          int metric, const float* qnorm, int64_t label_base, float* out_dist,
                          int64_t* out_labels, const int* nq_dev, const int32_t* row_map,
                          cudaStream_t stream);
// Running top-k over a key matrix chunk: run lists [nq][k] (key, int32 id) are read
// (if has_prev) and rewritten with the best k of (previous list U chunk columns).
// Merged raw keys only: out_key[q][k], best first, +INF where fewer than k entries exist.
int launch_merge_keys(const float* part_key, const int32_t* part_idx, int P, int64_t nq, int k,
                      float* out_key, cudaStream_t stream);
// The r <= 32 smallest keys of every row of a key matrix (no ids): out_key[q][r], best first,
// +INF where the row has fewer.  One warp per row.
int launch_select_keys(const float* keys, int64_t nq, int64_t ncols, int64_t ld, int r, float* out_key,
                       cudaStream_t stream);
// nq_dev (optional): number of live rows, read on the device.
int launch_select_chunk(const float* keys, int64_t nq, int64_t ncols, int64_t ld, int64_t col0,
                        int k, int has_prev, float* run_key, int32_t* run_idx, const int* nq_dev,
                        cudaStream_t stream);
// row_map (optional): list j belongs to query row_map[j] (output row and query norm).
int launch_finalize_lists(const float* run_key, const int32_t* run_idx, int64_t nq, int k,
                          int metric, const float* qnorm, int64_t label_base, float* out_dist,
                          int64_t* out_labels, const int* nq_dev, const int32_t* row_map,
                          cudaStream_t stream);
// Selection of k > 32 results from nlists sorted 32-entry lists per query (the fused kernel's
// output).  A list that is full may have dropped candidates; when its worst entry is not
// behind the k-th selected one the row's result is not proven exact and dirty[q] is set to 1
// (else 0).  Results are written for every row.
int launch_select_parts(const float* part_key, const int32_t* part_idx, int nlists, int64_t nq,
                        int k, int metric, const float* qnorm, int64_t label_base, float* out_dist,
                        int64_t* out_labels, int32_t* dirty, cudaStream_t stream);
// Selection of the k best of a row's threshold-filtered candidates (unordered buffer of
// min(cand_cnt[q], cap) entries).  dirty[q] = 1 when entries were lost to overflow or fewer than
// k candidates were found although the shard has more rows.
int launch_select_candidates(const float* cand_key, const int32_t* cand_idx, const int32_t* cand_cnt,
                             int cap, int64_t nb, int64_t nq, int k, int metric, const float* qnorm,
                             int64_t label_base, float* out_dist, int64_t* out_labels, int32_t* dirty,
                             cudaStream_t stream);
// select_rank.cu: the same selection / merge for inputs of at most 8192 entries per row, sorted in
// registers and placed by binary search; results identical to the kernels of select.cu.
bool rank_select_enabled();
bool rank_select_fits(int cap, int k);
int launch_rank_select(const float* cand_key, const int32_t* cand_idx, const int32_t* cand_cnt, int cap,
                       int64_t nb, int64_t nq, int k, int metric, const float* qnorm, int64_t label_base,
                       float* out_dist, int64_t* out_labels, int32_t* dirty, cudaStream_t stream);
bool rank_merge_fits(int P, int k);
int launch_rank_merge(const float* dist, const int64_t* labels, int64_t stride_d, int64_t stride_l, int P,
                      int64_t nq, int k, int metric, float* out_dist, int64_t* out_labels,
                      cudaStream_t stream);
// rows[0 .. *count) = ascending indices q with dirty[q] != 0; *count also goes to *count_copy.
int launch_compact_rows(const int32_t* dirty, int64_t nq, int32_t* rows, int32_t* count,
                        int32_t* count_copy, cudaStream_t stream);
// out[pl][j][:] = a[pl][rows[j]][:] for j < *count (16-bit elements, pitch a multiple of 8).
int launch_gather_rows(const uint16_t* a, int npl, int64_t plane_stride, int64_t pitch,
                       const int32_t* rows, const int32_t* count, int64_t nq_max, uint16_t* out,
                       cudaStream_t stream);

// Per-device state: function attributes (the opt-in to more than 48 KiB of dynamic shared
// memory), SM counts and occupancy figures belong to a device, and one process may hold
// resources on several.  device_slot() is the current device's index into such tables.
constexpr int kMaxDevices = 64;
int device_slot();
int cached_sm_count();

// Profiling (off by default): counts kernel launches of this library and, when enabled,
// brackets every launch of the dominant distance kernel (tensor GEMM or scan) with CUDA
// events on the launching stream.
void count_launch(int n = 1);
void main_kernel_begin(cudaStream_t stream);
void main_kernel_end(cudaStream_t stream);

}  // namespace b200f
