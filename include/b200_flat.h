/*
 * b200_flat.h -- C-ABI of the B200 (sm_100a) flat k-NN search backend.
 *
 * This is the whole drop-in boundary: plain C types, caller-owned pointers,
 * status codes instead of exceptions.  Two groups of entry points:
 *
 *   1. "op" entry points: one launcher per device operation.  They are what the
 *      reference's op wrappers (MetalL2Norm, MetalDistance, MetalSelect) were to
 *      its index class.  Pointers are DEVICE pointers, work is enqueued on the
 *      given CUDA stream and nothing is allocated inside.
 *   2. "index" entry points: a handle-based mirror of the reference's plugin
 *      class (faiss_metal::MetalIndexFlat) for bindings that cannot hold a C++
 *      object (ctypes, cgo, JNI, N-API).  Pointers are HOST pointers unless the
 *      comment says "host or device".
 *
 * Each declaration cites the reference interface it replaces
 * (path inside the reference project : line).
 */
#ifndef B200_FLAT_H
#define B200_FLAT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- enums ------------------------------------------------------------ */

/* faiss::MetricType values used by the reference (src/MetalDistance.h:21-22). */
#define B200F_METRIC_INNER_PRODUCT 0
#define B200F_METRIC_L2 1

/* faiss_metal::StorageType (include/faiss-metal/MetalIndexFlat.h:39-43). */
#define B200F_STORAGE_F32 0
#define B200F_STORAGE_F16 1
#define B200F_STORAGE_BF16 2

/* Status codes (the reference throws: src/MetalIndexFlat.mm:321-326,
 * src/MetalSelect.mm:67-70, src/StandardMetalResources.mm:21-23,71-74). */
#define B200F_OK 0
#define B200F_ERR_BAD_ARG 1      /* null pointer, k <= 0, bad enum, misaligned pitch   */
#define B200F_ERR_UNSUPPORTED 2  /* k above B200F_MAX_K, ntotal above 2^31-1            */
#define B200F_ERR_SCRATCH 3      /* scratch buffer smaller than *_scratch_bytes()       */
#define B200F_ERR_CUDA 4         /* CUDA runtime / driver call failed                   */
#define B200F_ERR_DEVICE_WAIT 5  /* a bounded device-side wait ran out (status word)    */
#define B200F_ERR_NO_DEVICE 6    /* no sm_100 device; there is no CPU fallback          */
#define B200F_ERR_OOM 7          /* device or pinned-host allocation failed             */
#define B200F_ERR_RANGE 8        /* reconstruct key out of range                        */
#define B200F_ERR_STATE 9        /* token already consumed / moved-from                 */
#define B200F_ERR_DEVICE_CHECK 10 /* a device-side self-check failed: shared-memory base misaligned,
                                     candidate buffer overflow, debug canary overwritten   */

/* Split planes FP32 storage keeps for the tensor path (the reference multiplies FP32 storage in
 * half precision, shaders/simdgroup_gemm.metal:62-69, ~1e-2 relative; the contract here is 1e-4):
 *   BF16X3  x = b0 + b1 + b2, three bf16 planes, six plane products, exact to 2^-24.
 *   FP16X2  2^s x = h0 + h1, two fp16 planes of the row scaled by the index's power of two 2^s
 *           (largest element near 2^6), three plane products, exact to 2^-22: half the tensor
 *           work, two thirds of the plane bytes.  Valid while every row fits fp16's range
 *           (elements below 2^15 after scaling, no non-zero row whose largest element is below
 *           2^-4); b200f_store_rows_fp32 reports rows that do not through range_flag, and the
 *           index then re-splits itself into BF16X3.  Queries are scaled per row inside
 *           b200f_search, so their magnitude does not matter. */
#define B200F_PLANES_BF16X3 0
#define B200F_PLANES_FP16X2 1

/* Largest k any path accepts (README.md:218-219 / src/MetalSelect.mm:65-70: 4096 on M3+). */
#define B200F_MAX_K 4096
/* Largest k served by the fused (no distance matrix) epilogue and scan kernels
 * (src/MetalDistance.mm:346-354: k <= 32). */
#define B200F_FUSED_MAX_K 32
/* Largest k the tensor path serves from the fused kernel's 32-entry lists (no distance
 * matrix unless a row's lists overflow; no counterpart in the reference, whose k > 32 path
 * always writes the matrix, src/MetalIndexFlat.mm:358-378). */
#define B200F_LIST_MAX_K 1024

/* Path override for tests, the analogue of MetalIndexFlat::setForceMPS
 * (include/faiss-metal/MetalIndexFlat.h:106): 0 = choose by (nq, k). */
#define B200F_PATH_AUTO 0
#define B200F_PATH_SCAN 1    /* streaming CUDA-core scan (small nq)          */
#define B200F_PATH_TENSOR 2  /* tcgen05 GEMM with fused top-k / select      */

const char* b200f_status_string(int status);

/* ---- library-wide switches (testing aids) ------------------------------- */
/* The counterpart of MetalIndexFlat::setForceMPS (include/faiss-metal/MetalIndexFlat.h:106)
 * one level down: which selection scheme the tensor path uses.  Results are identical in
 * every mode; only the kernel sequence differs.  Process-wide, read by every later search.
 * Until the setter is called the default comes from the environment variable
 * B200F_SELECT_MODE (auto | filter | no_filter | matrix), which is read once, at the first
 * search; nothing else in the search path reads the environment. */
#define B200F_SELECT_AUTO 0       /* threshold filter from 2^27 (query, row) pairs (2^22 where the pilot sample fits a key matrix), 32-entry lists below */
#define B200F_SELECT_FILTER 1     /* threshold filter wherever the shard allows a pilot sample */
#define B200F_SELECT_NO_FILTER 2  /* never the threshold filter                                */
#define B200F_SELECT_MATRIX 3     /* neither filter nor lists: fused lists (k <= 32), key matrix beyond */
int b200f_set_selection_mode(int mode);
int b200f_get_selection_mode(void);
/* Shape of the tensor kernel: one CTA per 128 x 256 tile, or a CTA pair per 256 x 512 tile.
 * Default: by the number of queries (environment default B200F_GEMM_PAIR=0|1, read once). */
#define B200F_GEMM_SHAPE_AUTO (-1)
#define B200F_GEMM_SHAPE_SINGLE 0
#define B200F_GEMM_SHAPE_PAIR 1
int b200f_set_gemm_shape(int shape);
/* Selection of more than 32 results from at most 8192 entries per row (a row's threshold-filtered
 * candidates; the sorted lists of up to 8192 / k shards): with on != 0 (the default) the kernels
 * that sort in registers and place every entry by binary search, else the shared-memory sorting
 * kernel that also serves larger inputs.  The same switch decides how the threshold filter takes
 * its pilot sample: on, as a key matrix picked over by a selection kernel wherever it fits (and the
 * filter is then used from 2^22 pairs); off, always as 32-entry lists.  Results are identical
 * either way; a testing aid.  No counterpart in the reference (its block_select,
 * shaders/block_select.metal:111-274, is the one kernel). */
int b200f_set_rank_select(int on);
/* Debug canaries, the stand-in for a memory checker on the scratch arena: with on != 0 every
 * slice of a search's scratch region is followed by a 256-byte guard that is filled before the
 * search and compared after it; a kernel that wrote past its slice sets bit 8 of status[0]
 * (B200F_ERR_DEVICE_CHECK at the index level).  Changes b200f_search_scratch_bytes(): set it
 * before sizing scratch, not between sizing and searching.  No counterpart in the reference. */
int b200f_set_debug_canaries(int on);
/* Self-test of the canary checker on a caller-provided device region (>= 4 KiB, 256-byte
 * aligned): three guards are filled, with corrupt != 0 one word of the second guard is
 * overwritten the way a kernel running past its slice would, and the guards are compared:
 * status[0] gets bit 8 and status[2] = 2 exactly when corrupt != 0.  status is not cleared. */
int b200f_debug_canary_selftest(void* scratch, size_t scratch_bytes, int corrupt, int32_t* status, void* stream);
/* Runs the bounded-wait helper every kernel of this library waits with, on a barrier that
 * nothing will ever signal, with a limit of limit_cycles SM clocks (about a millisecond is
 * plenty): one CTA, the wait gives up, records bit 1 in status[0] and the kernel returns
 * normally.  It exists so that the expiry path (status word, B200F_ERR_DEVICE_WAIT) can be
 * exercised without a fault, trap or hang.  status: device int32[4], not cleared by the call.
 * No counterpart in the reference. */
int b200f_debug_wait_expiry(int32_t* status, int64_t limit_cycles, void* stream);

/* ---- device capabilities ----------------------------------------------- */
/* Replaces MetalDeviceCapabilities / queryDeviceCapabilities
 * (include/faiss-metal/MetalDeviceCapabilities.h:23-61,
 *  src/MetalDeviceCapabilities.mm:8-96). */
typedef struct B200FCaps {
    int32_t device;
    int32_t cc_major, cc_minor;
    int32_t sm_count;
    int32_t max_smem_per_block;   /* opt-in bytes */
    int32_t l2_bytes;
    int64_t hbm_bytes;
    int32_t sm_clock_khz;
    int32_t mem_clock_khz;
    int32_t supported;            /* 1 when the device is sm_100 */
    char name[128];
} B200FCaps;

int b200f_device_count(int* count);
int b200f_device_caps(int device, B200FCaps* caps);

/* ---- op entry points (device pointers, async on `stream`) --------------- */

/* out[r] = sum_j rows[r][j]^2 in fp32.
 * Replaces MetalL2Norm::encode (src/MetalL2Norm.mm:42-74) and kernels
 * l2_norm / l2_norm_large / l2_norm_f16 / l2_norm_f16_large
 * (shaders/l2_norm.metal:7-66, shaders/l2_norm_f16.metal:10-67). */
int b200f_row_norms(const void* rows, int storage, int64_t n, int d, int64_t pitch_elems,
                    float* out, void* stream);

/* Append-time conversion: src fp32 [n][d] (pitch d) -> dst rows in `storage`
 * precision (pitch dst_pitch elements, pad columns zeroed), optional squared
 * norms of the STORED values, and for FP32 storage the three bf16 split
 * planes the tensor path multiplies (planes[p][r][plane_pitch], plane p at
 * p*plane_stride elements).  With norm_cols = 1 the 16-bit row (or split plane 0)
 * also receives, in the 8 columns after round_up(d, 8), the value -||x||^2/2 split
 * into 16-bit pieces, so that the distance GEMM / scan obtains q.x - ||x||^2/2 from
 * one dot product (the pitch must then be >= round_up(d, 8) + 8).
 * Replaces the conversion loops and the per-add norm pass of
 * MetalIndexFlat::add (src/MetalIndexFlat.mm:224-255,259-268,296-307). */
int b200f_store_rows(const float* src, int64_t n, int d, int storage, void* dst_rows,
                     int64_t dst_pitch, uint16_t* planes, int64_t plane_pitch,
                     int64_t plane_stride, float* norms_or_null, int norm_cols, void* stream);
/* The same for FP32 storage with a choice of plane format (B200F_PLANES_*) and, for FP16X2, the
 * index's scale 2^plane_scale_log2.  src rows are src_pitch elements apart; src == dst_rows
 * (with src_pitch == dst_pitch) re-splits rows that are stored already.  range_flag (device
 * int32, may be NULL): bit 1 is OR-ed in when a row does not fit the FP16X2 format. */
int b200f_store_rows_fp32(const float* src, int64_t src_pitch, int64_t n, int d, float* dst_rows,
                          int64_t dst_pitch, uint16_t* planes, int64_t plane_pitch, int64_t plane_stride,
                          int plane_format, int plane_scale_log2, int32_t* range_flag, float* norms_or_null,
                          int norm_cols, void* stream);
/* *max_bits = bit pattern of the largest finite |element| of the fp32 rows (0 when all are zero):
 * what an index derives its FP16X2 scale from.  Device pointers.  No counterpart in the reference. */
int b200f_rows_absmax(const float* rows, int64_t n, int d, int64_t pitch_elems, uint32_t* max_bits, void* stream);

/* Stored rows -> fp32 [n][d] (pitch d).
 * Replaces the per-element conversions of MetalIndexFlat::reconstruct
 * (src/MetalIndexFlat.mm:508-527). */
int b200f_load_rows(const void* rows, int storage, int64_t n, int d, int64_t pitch_elems,
                    float* dst, void* stream);

/* Arguments of one shard-local search. */
typedef struct B200FSearchArgs {
    const float* queries;    /* device fp32 [nq][d], pitch d                                */
    int64_t nq;
    int32_t d;
    int32_t storage;         /* B200F_STORAGE_*                                             */
    const void* rows;        /* device stored rows [nb][row_pitch]                          */
    int64_t row_pitch;       /* elements; 16-bit: multiple of 8, fp32: multiple of 4        */
    const uint16_t* planes;  /* FP32 storage: bf16 split planes, else NULL                  */
    int64_t plane_pitch;     /* elements, multiple of 8                                     */
    int64_t plane_stride;    /* elements between planes                                     */
    const float* norms;      /* device [nb] squared norms (L2), NULL for inner product      */
    int64_t nb;              /* rows in this shard, <= 2^31-1                               */
    int32_t metric;          /* B200F_METRIC_*                                              */
    int32_t k;
    int64_t label_base;      /* added to local row numbers to form labels                   */
    float* out_dist;         /* device [nq][k], best first; tail (+/-INF) when k > nb       */
    int64_t* out_labels;     /* device [nq][k]; tail -1                                     */
    void* scratch;           /* device, >= b200f_search_scratch_bytes(), 256-byte aligned   */
    size_t scratch_bytes;
    int32_t* status;         /* device int32[4], zeroed by the call; [0] != 0 after the
                                stream drains means a bounded device wait ran out          */
    void* stream;
    int32_t path;            /* B200F_PATH_*                                                */
    int32_t norm_cols;       /* 1: 16-bit rows / split plane 0 carry the 8 norm columns
                                written by b200f_store_rows(norm_cols = 1); required for
                                L2 on 16-bit storage and on the tensor path                */
    int32_t plane_format;    /* FP32 storage: B200F_PLANES_* of `planes` (0 = three bf16 planes) */
    int32_t plane_scale_log2; /* FP16X2: the planes hold 2^plane_scale_log2 * x                  */
} B200FSearchArgs;

/* Scratch bytes b200f_search needs for this shape (0 on bad arguments).
 * Replaces the grow-only scratch getters of the reference's index
 * (src/MetalIndexFlat.mm:102-142). */
size_t b200f_search_scratch_bytes(int64_t nq, int64_t nb, int d, int k, int storage, int path);

/* Shard-local k-NN: query norms, distance (tensor-core GEMM or streaming scan)
 * fused with top-k, and the merge of per-range partial lists.
 * Replaces MetalDistance::encodeFused / encode + MetalSelect::encode as driven
 * by MetalIndexFlat::search (src/MetalIndexFlat.mm:358-378,
 * src/MetalDistance.mm:107-128,225-408, src/MetalSelect.mm:34-89) and kernels
 * simdgroup_gemm_* (shaders/simdgroup_gemm*.metal), fused_*_topk_*
 * (shaders/fused_l2_topk.metal:19-444), warp_select_* / block_select_*
 * (shaders/warp_select.metal:11-114, shaders/block_select.metal:111-274).
 *
 * Precision of the operands.  16-bit storage: the QUERY is rounded to the storage format
 * before it is multiplied (FP16 rows: 11-bit mantissa, as the reference rounds its queries to
 * half, shaders/simdgroup_gemm.metal:62-69; BF16 rows: 8-bit mantissa, which is narrower than
 * the reference's half queries on that one operand, shaders/simdgroup_gemm_bf16.metal:53-58);
 * products are exact and accumulated in fp32, ||q||^2 is taken from the unrounded query.
 * Measured error on N(0,1)*0.05 data, d = 1536: 1.4e-4 relative, against the 2e-2 contract.
 * FP32 storage, tensor path: both operands are multiplied as split 16-bit planes
 * (B200F_PLANES_*): two fp16 planes of the power-of-two-scaled values, three plane products,
 * terms below 2^-22 relative dropped (measured <= 2.7e-5 on distances, contract 1e-4), or three
 * bf16 planes, six products, 2^-24 (2e-6 measured).  Queries are split to match, each row with
 * its own scale.  FP32 storage, scan path: fp32 FMA throughout for a single query; two to eight
 * queries are multiplied as tf32 pairs (x = hi + lo, three products, fp32 accumulate: terms below
 * 2^-21 relative dropped, 6.2e-6 measured on distances). */
int b200f_search(const B200FSearchArgs* args);

/* Shard-local search that allocates nothing.  It has no counterpart in the reference.
 *
 * Who needs it: code that may not call cudaMalloc at the point where it searches -- a
 * latency-critical serving loop that must never take the allocator's lock or trigger an
 * implicit device synchronisation, a plugin that runs inside somebody else's memory pool
 * and owns no device memory of its own, or a caller that sized its buffers once at
 * start-up and has none left to hand over as scratch.  Such a caller still passes the
 * queries, the stored rows and the output arrays, but no scratch: the intermediate lists
 * live in a fixed 1 MiB array inside the library image (b200f_noalloc_scratch_capacity()),
 * present on every GPU that loads the library until the process ends.
 *
 * Limits: nq <= 4 and k <= 32 (the streaming-scan path; B200F_ERR_UNSUPPORTED otherwise) and
 * a shape whose b200f_search_scratch_bytes() fits the array (B200F_ERR_SCRATCH otherwise).
 * args->scratch / scratch_bytes / path are ignored.  The first call on each device looks up
 * the array's device address (with that device current); make that first call before any
 * stream capture begins.  No cudaMalloc, cudaFree or other allocating call is made, provided
 * profiling (b200f_profile_enable) is off, which is the default.  All calls share the one
 * array, which keeps whatever the previous call left: this path initialises everything it
 * reads, so nothing has to be cleared, but two calls whose kernels overlap on the GPU
 * (different streams, or different threads) race on it -- serialise them. */
size_t b200f_noalloc_scratch_capacity(void);
int b200f_search_small_noalloc(const B200FSearchArgs* args);

/* Full nq x nb score matrix (L2: ||q||^2 + ||x||^2 - 2 q.x, IP: q.x), fp32,
 * leading dimension ld_out.  Same operands as b200f_search (k, out_*, label_base
 * ignored).  Scratch: b200f_search_scratch_bytes(nq, nb, d, 1, storage, path).
 * Replaces MetalDistance::encode / compute (src/MetalDistance.h:25-80,
 * src/MetalDistance.mm:107-128); used by the unit tests the way
 * tests/test_metal_distance.mm:98-230 uses it. */
int b200f_pairwise(const B200FSearchArgs* args, float* out_matrix, int64_t ld_out);

/* Top-k of every row of a device score matrix [nq][ncols] (leading dimension
 * ld): smallest first for L2, largest first for inner product, ties to the
 * lower column.  k <= B200F_MAX_K.  Scratch: b200f_select_scratch_bytes().
 * Replaces MetalSelect::encode / select (src/MetalSelect.mm:34-108). */
size_t b200f_select_scratch_bytes(int64_t nq, int k);
int b200f_select_rows(const float* scores, int64_t nq, int64_t ncols, int64_t ld, int metric,
                      int k, float* out_dist, int64_t* out_labels, void* scratch,
                      size_t scratch_bytes, void* stream);

/* k-way merge of P result lists per query.  dist / labels are device
 * [P][nq][k] (each list best first, padded with -1 labels); output [nq][k]
 * best first, ties to the lower label.  This is the step after the NCCL
 * allgather of per-GPU candidates; the reference is single-device and has no
 * counterpart (its closest relative is the final 4-list merge inside
 * shaders/fused_l2_topk.metal:88-131). */
int b200f_merge_lists(const float* dist, const int64_t* labels, int P, int64_t nq, int k,
                      int metric, float* out_dist, int64_t* out_labels, void* stream);

/* Same merge for lists that are not packed back to back: list p's distances start at
 * dist + p * list_stride_dist, its labels at labels + p * list_stride_labels (strides in
 * elements, each >= nq * k).  Lets the caller all-gather one buffer per rank that holds
 * [distances | labels] and merge straight out of the gathered buffer. */
int b200f_merge_lists_strided(const float* dist, const int64_t* labels, int64_t list_stride_dist,
                              int64_t list_stride_labels, int P, int64_t nq, int k, int metric,
                              float* out_dist, int64_t* out_labels, void* stream);

/* Labels of a shard-local search -> global labels when rows are placed block-cyclically over
 * nshards shards (global row g on shard (g / B) % nshards at local row (g / (B * nshards)) * B +
 * g % B): labels[i] >= 0 becomes ((l / B) * nshards + shard) * B + l % B, -1 stays.  Device
 * pointer, in place.  No counterpart in the reference (single device). */
int b200f_remap_labels_block_cyclic(int64_t* labels, int64_t count, int64_t block_rows, int nshards, int shard,
                                    void* stream);

/* Deterministic synthetic rows on the device (benchmark inputs): element
 * (row, col) depends only on (seed, row0 + row, col).
 * dist: 0 = U[0,1), 1 = N(0,1) * scale, 2 = N(0,1) then row-normalised,
 * 3 = mixture of 1,000 gaussians (centres uniform in [-1,1]^d, shared by all seeds; sigma = scale).
 * No counterpart in the reference (its bench fills host arrays with
 * std::mt19937, tests/bench_metal_flat.mm:27-33). */
int b200f_fill_synthetic(float* dst, int64_t n, int d, int64_t row0, uint64_t seed, int dist,
                         float scale, void* stream);

/* Profiling, off by default.  While enabled every launch of the dominant distance
 * kernel (tensor GEMM or streaming scan) is bracketed by CUDA events on its stream.
 * b200f_profile_read waits for the recorded events and returns the totals since the
 * last reset: kernels launched by this library, launches of the dominant kernel and
 * their summed duration in milliseconds.  The reference measures with wall clocks
 * around search() only (tests/bench_metal_flat.mm:43-54); it has no counterpart. */
int b200f_profile_enable(int on);
int b200f_profile_read(int64_t* launches, int64_t* main_launches, double* main_ms, int reset);

/* ---- index entry points (mirror of faiss_metal::MetalIndexFlat) ---------- */

typedef struct B200FResources B200FResources; /* StandardMetalResources (include/faiss-metal/StandardMetalResources.h:9-32) */
typedef struct B200FIndex B200FIndex;         /* MetalIndexFlat (include/faiss-metal/MetalIndexFlat.h:47-111)               */
typedef struct B200FToken B200FToken;         /* MetalSearchToken (include/faiss-metal/MetalIndexFlat.h:15-36)              */

/* Message of the last failed index-level call on this thread. */
const char* b200f_last_error(void);
/* Throws, inside the same exception barrier every index-level call runs behind, the exception
 * the host layer uses for `status` (-1 / -2 / -3: a bare faiss::FaissException /
 * std::runtime_error / std::bad_alloc, as foreign code could throw) and returns what the
 * barrier made of it.  Lets a test without a GPU see every error code come out of the typed
 * exceptions.  The reference throws across its C++ boundary (src/MetalIndexFlat.mm:321-326). */
int b200f_debug_raise(int status);

/* StandardMetalResources() (src/StandardMetalResources.mm:17-44): device < 0 = current device.
 *
 * Stream semantics of every index-level call: the work runs on the resources' own stream
 * (b200f_resources_stream), which does NOT synchronise with the legacy default stream or
 * any other stream.  Host pointers need no care (the calls block until the data has been
 * read / written, searchAsync until token wait).  DEVICE pointers handed to add / search /
 * search_enqueue / reconstruct_n must be complete before the call: produce them on the
 * resources' stream, or make that stream wait on an event recorded after their producer
 * (b200f_resources_wait_stream does exactly that). */
int b200f_resources_create(int device, B200FResources** out);
void b200f_resources_destroy(B200FResources* res);
int b200f_resources_device(const B200FResources* res);
void* b200f_resources_stream(const B200FResources* res);
/* Orders the resources' stream after everything queued so far on `producer_stream` (a
 * cudaStream_t of the same device; NULL = the legacy default stream): an event is recorded
 * there and the resources' stream waits for it.  No host synchronisation. */
int b200f_resources_wait_stream(B200FResources* res, void* producer_stream);
/* bytes currently held by the grow-only scratch arena (src/MetalIndexFlat.mm:102-142) */
size_t b200f_resources_scratch_bytes(const B200FResources* res);

/* MetalIndexFlat(resources, d, metric, storage) (src/MetalIndexFlat.mm:162-183). */
int b200f_index_create(B200FResources* res, int d, int metric, int storage, B200FIndex** out);
void b200f_index_destroy(B200FIndex* index);
/* add(n, x): x fp32 [n][d], host or device (src/MetalIndexFlat.mm:185-311). */
int b200f_index_add(B200FIndex* index, int64_t n, const float* x);
/* search(n, x, k, distances, labels): x host or device; outputs in the same
 * memory space as x is NOT required: each output pointer may independently be
 * host or device (src/MetalIndexFlat.mm:313-401). */
int b200f_index_search(const B200FIndex* index, int64_t n, const float* x, int64_t k,
                       float* distances, int64_t* labels);
/* Device-only, enqueue-only form of search: x / distances / labels are DEVICE pointers, the
 * work is queued on the resources' stream (b200f_resources_stream) and the call returns
 * without synchronising, so a caller can chain its own work (the multi-GPU exchange and
 * merge) on that stream.  One launch batch only (n <= 16384 for k <= 32, else n <= 1024).
 * b200f_index_synchronize waits for the stream and reports a device-side error, if any.
 * The reference's closest relative is the encode-without-wait half of searchAsync
 * (src/MetalIndexFlat.mm:478-486). */
int b200f_index_search_enqueue(const B200FIndex* index, int64_t n, const float* x, int64_t k,
                               float* distances, int64_t* labels);
int b200f_index_synchronize(const B200FIndex* index);
/* searchAsync -> token; token wait / isReady / destructor
 * (src/MetalIndexFlat.mm:403-490, :41-78). */
int b200f_index_search_async(const B200FIndex* index, int64_t n, const float* x, int64_t k,
                             float* distances, int64_t* labels, B200FToken** out);
int b200f_token_wait(B200FToken* token);
int b200f_token_is_ready(const B200FToken* token, int* ready);
void b200f_token_destroy(B200FToken* token);
/* reset() (src/MetalIndexFlat.mm:492-506), reconstruct(key, out) (:508-527). */
int b200f_index_reset(B200FIndex* index);
int b200f_index_reconstruct(const B200FIndex* index, int64_t key, float* recons);
/* Bulk form used by index_metal_to_cpu (src/MetalIndexFlat.mm:565-587):
 * rows [first, first+n) as fp32 into out (host or device). */
int b200f_index_reconstruct_n(const B200FIndex* index, int64_t first, int64_t n, float* out);
/* getters (src/MetalIndexFlat.mm:529-548) */
int64_t b200f_index_ntotal(const B200FIndex* index);
int b200f_index_d(const B200FIndex* index);
int b200f_index_metric(const B200FIndex* index);
int b200f_index_storage(const B200FIndex* index);
/* Path override for tests (setForceMPS analogue, include/faiss-metal/MetalIndexFlat.h:106). */
int b200f_index_set_path(B200FIndex* index, int path);
/* Pre-size the storage for n rows in total (avoids the x2 growth copies of
 * src/MetalIndexFlat.mm:196-208 when the final size is known). */
int b200f_index_reserve(B200FIndex* index, int64_t n);
/* How the storage grows: 0 = in place (address range reserved once, memory mapped behind the
 * rows as they are added; the default where the driver supports it), 1 = the reference's
 * allocate-copy-free (src/MetalIndexFlat.mm:196-222).  Only on an empty index.  The default
 * comes from the environment variable B200F_NO_VMM=1 (read once per process). */
int b200f_index_set_growth_mode(B200FIndex* index, int mode);
/* FP32 storage: plane format of the tensor path's operands (B200F_PLANES_*; default FP16X2, see
 * there).  The setter works on an empty index only; the getter tells what the index uses now (an
 * FP16X2 index falls back to BF16X3 by itself when a row leaves fp16's range). */
int b200f_index_set_fp32_planes(B200FIndex* index, int format);
int b200f_index_fp32_planes(const B200FIndex* index);
/* Searches of at most 8 queries whose three arrays are host memory are replayed from a CUDA
 * graph (query upload, every kernel of the search, result download in one launch), captured
 * the second time a (n, k) shape is seen and dropped whenever the index changes.  on = 0
 * switches that off.  Replaces the per-call encode of searchAsync for the single-query
 * stream (src/MetalIndexFlat.mm:403-490). */
int b200f_index_set_use_graphs(B200FIndex* index, int on);
/* Row shards: labels returned by search = local row number + base. */
int b200f_index_set_label_base(B200FIndex* index, int64_t base);
/* Device pointers to the stored rows / norms of the shard (used by the
 * multi-GPU layer and the benchmark; the reference's getVectorsData,
 * include/faiss-metal/MetalIndexFlat.h:94, returned a unified-memory pointer). */
const void* b200f_index_device_rows(const B200FIndex* index);
/* Device-side status of the most recent search (0 = fine). */
int b200f_index_last_device_status(const B200FIndex* index);
/* b200f_debug_wait_expiry on the index's stream with the index's own status word: the next
 * b200f_index_synchronize then reports B200F_ERR_DEVICE_WAIT, and the search after it runs
 * normally (every search clears the word first).  For tests of the error path. */
int b200f_index_debug_wait_expiry(B200FIndex* index, int64_t limit_cycles);

/* ---- sharded index: rows over the GPUs of one box ------------------------------------------ */
/* Mirror of faiss_b200::B200ShardedIndexFlat.  The reference is single-device
 * (src/StandardMetalResources.mm:17-23) and has no counterpart; the surface is the same
 * faiss::Index contract as above (include/faiss-metal/MetalIndexFlat.h:47-111).  Every GPU
 * searches its own rows; the per-GPU candidates are exchanged with one ncclAllGather issued by
 * the library on the resources' own stream and merged by b200f_merge_lists_strided.  NCCL is
 * loaded at run time (libnccl.so.2), only when more than one GPU takes part. */
typedef struct B200FSharded B200FSharded;

/* 128 bytes (an ncclUniqueId) that rank 0 creates and every rank of a one-process-per-GPU
 * group passes to b200f_sharded_create_rank. */
int b200f_comm_id_create(void* id128);
/* One process drives nshards GPUs (one resources handle each; several handles of ONE device
 * rehearse the same code on a single GPU with device copies in the place of NCCL).  Rows are
 * placed block-cyclically in blocks of block_rows. */
int b200f_sharded_create(B200FResources* const* res, int nshards, int d, int metric, int storage,
                         int64_t block_rows, B200FSharded** out);
/* One process per GPU: `local` holds this rank's rows (label base set by the caller) and must
 * outlive nothing: the sharded index shares its ownership.  Collective over the group when
 * world > 1 (ncclCommInitRank). */
int b200f_sharded_create_rank(B200FIndex* local, int rank, int world, const void* id128, B200FSharded** out);
void b200f_sharded_destroy(B200FSharded* index);
/* several-GPU form only (B200F_ERR_STATE otherwise) */
int b200f_sharded_add(B200FSharded* index, int64_t n, const float* x);
/* x host or device.  Host queries cross PCIe once: part i's GPU takes the i-th slice and the
 * slices are all-gathered over NVLink.  One process per GPU: collective, identical n, k, x on
 * every rank; distances = labels = NULL on ranks that do not want the result (no merge, no
 * copy back there). */
int b200f_sharded_search(const B200FSharded* index, int64_t n, const float* x, int64_t k, float* distances,
                         int64_t* labels);
/* Device pointers, one batch, no host synchronisation (see b200f_index_search_enqueue). */
int b200f_sharded_search_enqueue(const B200FSharded* index, int64_t n, const float* x, int64_t k,
                                 float* distances, int64_t* labels);
int b200f_sharded_synchronize(const B200FSharded* index);
int b200f_sharded_reset(B200FSharded* index);
int b200f_sharded_reconstruct(const B200FSharded* index, int64_t key, float* recons);
int64_t b200f_sharded_ntotal(const B200FSharded* index);   /* one process per GPU: this rank's rows */
int b200f_sharded_num_shards(const B200FSharded* index);
int b200f_sharded_set_path(B200FSharded* index, int path);
/* One process per GPU: searches of at most 8 queries with host buffers are replayed from a
 * CUDA graph holding the whole call (upload, shard search, ncclAllGather, merge, download);
 * on = 0 switches that off. */
int b200f_sharded_set_use_graphs(B200FSharded* index, int on);
/* Host-side trace of b200f_sharded_search calls (off by default; switching it on or off
 * clears the record): per call the microseconds from entry until everything was enqueued and
 * the microseconds spent waiting for the device after that.  trace_read copies up to
 * `capacity` entries and returns the number recorded (-1 on bad arguments). */
int b200f_sharded_trace(B200FSharded* index, int on);
int64_t b200f_sharded_trace_read(const B200FSharded* index, float* enqueue_us, float* wait_us, int64_t capacity);

#ifdef __cplusplus
}
#endif
#endif /* B200_FLAT_H */
