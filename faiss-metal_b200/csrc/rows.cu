// Row-wise kernels: squared norms, append-time conversion, reconstruction,
// query preparation and the synthetic-data generator.
//
// Replaces l2_norm / l2_norm_large / l2_norm_f16 / l2_norm_f16_large
// (shaders/l2_norm.metal:7-66, shaders/l2_norm_f16.metal:10-67), their dispatch
// (src/MetalL2Norm.mm:42-89) and the host conversion loops of MetalIndexFlat::add
// (src/MetalIndexFlat.mm:224-255).  One warp owns one row; lanes read 128-bit
// vectors and reduce with shuffles.  Squares are formed in fp32 (the reference's
// "f16" norm kernels square in half precision, which is not reproduced).
#include <cmath>

#include "common.cuh"

namespace b200f {

namespace {

constexpr int ROW_THREADS = 256;  // 8 warps = 8 rows per CTA pass

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) {
    return __uint_as_float((uint32_t)b << 16);
}
// fp32 -> bf16 bits, round to nearest even (src/MetalIndexFlat.mm:231-234)
__device__ __forceinline__ uint16_t float_to_bf16_bits(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ uint16_t float_to_fp16_bits(float f) {
    return __half_as_ushort(__float2half_rn(f));
}
__device__ __forceinline__ float fp16_bits_to_float(uint16_t b) {
    return __half2float(__ushort_as_half(b));
}

template <int STORAGE>
__device__ __forceinline__ float load_elem(const void* rows, int64_t off) {
    if (STORAGE == B200F_STORAGE_F32) return reinterpret_cast<const float*>(rows)[off];
    uint16_t b = reinterpret_cast<const uint16_t*>(rows)[off];
    return STORAGE == B200F_STORAGE_F16 ? fp16_bits_to_float(b) : bf16_bits_to_float(b);
}

// ---- norms -----------------------------------------------------------------------------
template <int STORAGE>
__global__ void row_norms_kernel(const void* __restrict__ rows, int64_t n, int d, int64_t pitch,
                                 float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n;
         r += warps_total) {
        float s = 0.f;
        if (STORAGE == B200F_STORAGE_F32) {
            const float* row = reinterpret_cast<const float*>(rows) + r * pitch;
            if ((pitch & 3) == 0 && ((uintptr_t)rows & 15) == 0) {
                const int d4 = d >> 2;
                const float4* row4 = reinterpret_cast<const float4*>(row);
                for (int j = lane; j < d4; j += 32) {
                    float4 v = __ldg(row4 + j);
                    s = fmaf(v.x, v.x, s);
                    s = fmaf(v.y, v.y, s);
                    s = fmaf(v.z, v.z, s);
                    s = fmaf(v.w, v.w, s);
                }
                for (int j = (d4 << 2) + lane; j < d; j += 32) s = fmaf(row[j], row[j], s);
            } else {
                for (int j = lane; j < d; j += 32) s = fmaf(row[j], row[j], s);
            }
        } else {
            const uint16_t* row = reinterpret_cast<const uint16_t*>(rows) + r * pitch;
            if ((pitch & 7) == 0 && ((uintptr_t)rows & 15) == 0) {
                const int d8 = d >> 3;
                const uint4* row8 = reinterpret_cast<const uint4*>(row);
                for (int j = lane; j < d8; j += 32) {
                    uint4 v = __ldg(row8 + j);
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int t = 0; t < 4; t++) {
                        float a, b;
                        if (STORAGE == B200F_STORAGE_F16) {
                            a = fp16_bits_to_float((uint16_t)(w[t] & 0xffffu));
                            b = fp16_bits_to_float((uint16_t)(w[t] >> 16));
                        } else {
                            a = __uint_as_float(w[t] << 16);
                            b = __uint_as_float(w[t] & 0xffff0000u);
                        }
                        s = fmaf(a, a, s);
                        s = fmaf(b, b, s);
                    }
                }
                for (int j = (d8 << 3) + lane; j < d; j += 32) {
                    float a = load_elem<STORAGE>(row, j);
                    s = fmaf(a, a, s);
                }
            } else {
                for (int j = lane; j < d; j += 32) {
                    float a = load_elem<STORAGE>(row, j);
                    s = fmaf(a, a, s);
                }
            }
        }
        s = warp_sum(s);
        if (lane == 0) out[r] = s;
    }
}

// ---- norm columns ------------------------------------------------------------------------
// The tensor path and the 16-bit scan get "||x||^2" out of the same dot product as q.x: a
// stored row carries 8 extra columns [d8, d8+8) holding -||x||^2/2 split into 16-bit pieces
// c_i, the query row carries the matching scales S_i there, so that
//     q_ext . x_ext = q.x - ||x||^2/2      (L2 key = -2 * that, + ||q||^2 at the end).
// bf16 has the exponent range of fp32: three pieces at scale 1.  fp16 does not: four
// pieces at scales 2^12, 2^1, 2^-10, 2^-21 (each an exact fp16 value) cover
// ||x||^2/2 up to 2.7e8 with at least 22 significant bits.
__device__ __forceinline__ float norm_scale(int storage, int slot) {
    if (storage == B200F_STORAGE_F16) {
        return slot == 0 ? 4096.f : slot == 1 ? 2.f : slot == 2 ? 9.765625e-4f : slot == 3 ? 4.76837158203125e-7f : 0.f;
    }
    return slot < 3 ? 1.f : 0.f;
}

// pieces of v for the 8 norm columns (16-bit patterns), format = fp16 or bf16
__device__ __forceinline__ void norm_pieces(float v, int storage, uint16_t (&out)[8]) {
    float r = v;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float S = norm_scale(storage, i);
        uint16_t bits = 0;
        if (S != 0.f) {
            const float c = r / S;
            float back;
            if (storage == B200F_STORAGE_F16) {
                bits = float_to_fp16_bits(c);
                back = fp16_bits_to_float(bits);
            } else {
                bits = float_to_bf16_bits(c);
                back = bf16_bits_to_float(bits);
            }
            r = fmaf(-S, back, r);
        }
        out[i] = bits;
    }
}

// ---- append-time conversion -----------------------------------------------------------
// One warp per row.  Writes the stored row (pad columns zeroed), the squared norm of
// the stored values, for fp32 storage the three bf16 split planes, and (norm_cols) the
// 8 norm columns after the d8 = round_up(d, 8) data columns of the 16-bit row / plane 0.
// FP32 storage keeps, beside the fp32 rows, split planes for the tensor path, in one of two formats:
//   kPlanesBf16x3  x = b0 + b1 + b2, three bf16 planes (24 bits, fp32's exponent range): six plane
//                  products reproduce the fp32 product to 2^-24
//   kPlanesFp16x2  x * s = h0 + h1, two fp16 planes (22 bits) of the row scaled by a power of two s
//                  chosen for the index (largest element near 2^6): three plane products, half
//                  the tensor work and two thirds of the plane bytes.  fp16 has a narrow exponent
//                  range, so the format only holds while every stored row fits it: an element
//                  at or beyond 2^15 after scaling, or a row whose largest element falls below
//                  2^-4 (1/1024 of the scale target: its low plane would go subnormal and lose
//                  bits), raises `range_flag`, and the index re-splits itself into bf16x3.
constexpr int kPlanesBf16x3 = 0;
constexpr int kPlanesFp16x2 = 1;

template <int STORAGE>
__global__ void store_rows_kernel(const float* __restrict__ src, int64_t src_pitch, int64_t n, int d,
                                  void* __restrict__ dst, int64_t dst_pitch,
                                  uint16_t* __restrict__ planes, int64_t plane_pitch,
                                  int64_t plane_stride, int plane_format, float plane_scale,
                                  int32_t* __restrict__ range_flag, float* __restrict__ norms, int norm_cols) {
    const int lane = threadIdx.x & 31;
    const int d8 = (d + 7) & ~7;
    const int64_t warps_total = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n;
         r += warps_total) {
        const float* row = src + r * src_pitch;
        float s = 0.f;
        if (STORAGE == B200F_STORAGE_F32) {
            float* out = reinterpret_cast<float*>(dst) + r * dst_pitch;
            if (out != row) {   // a re-split reads the stored rows themselves
                for (int j = lane; j < dst_pitch; j += 32) {
                    float v = (j < d) ? row[j] : 0.f;
                    out[j] = v;
                    s = fmaf(v, v, s);
                }
            } else {
                for (int j = lane; j < d; j += 32) s = fmaf(row[j], row[j], s);
            }
            if (planes && plane_format == kPlanesFp16x2) {
                uint16_t* p0 = planes + r * plane_pitch;
                uint16_t* p1 = p0 + plane_stride;
                float amax = 0.f;
                for (int j = lane; j < plane_pitch; j += 32) {
                    const float v = (j < d) ? row[j] * plane_scale : 0.f;
                    amax = fmaxf(amax, fabsf(v));
                    const uint16_t h0 = float_to_fp16_bits(v);
                    const float r1 = v - fp16_bits_to_float(h0);   // exact in fp32
                    p0[j] = h0;
                    p1[j] = float_to_fp16_bits(r1);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                if (lane == 0 && range_flag && (amax >= 32768.f || (amax > 0.f && amax < 0.0625f)))
                    atomicOr(range_flag, 1);
            } else if (planes) {
                uint16_t* p0 = planes + r * plane_pitch;
                uint16_t* p1 = p0 + plane_stride;
                uint16_t* p2 = p1 + plane_stride;
                for (int j = lane; j < plane_pitch; j += 32) {
                    float v = (j < d) ? row[j] : 0.f;
                    uint16_t b0 = float_to_bf16_bits(v);
                    float r1 = v - bf16_bits_to_float(b0);
                    uint16_t b1 = float_to_bf16_bits(r1);
                    float r2 = r1 - bf16_bits_to_float(b1);
                    uint16_t b2 = float_to_bf16_bits(r2);
                    p0[j] = b0;
                    p1[j] = b1;
                    p2[j] = b2;
                }
            }
        } else {
            uint16_t* out = reinterpret_cast<uint16_t*>(dst) + r * dst_pitch;
            for (int j = lane; j < dst_pitch; j += 32) {
                float v = (j < d) ? row[j] : 0.f;
                uint16_t b;
                float back;
                if (STORAGE == B200F_STORAGE_F16) {
                    b = float_to_fp16_bits(v);
                    back = fp16_bits_to_float(b);
                } else {
                    b = float_to_bf16_bits(v);
                    back = bf16_bits_to_float(b);
                }
                out[j] = b;
                s = fmaf(back, back, s);
            }
        }
        s = warp_sum(s);
        if (norms && lane == 0) norms[r] = s;
        if (norm_cols) {
            __syncwarp();
            if (lane == 0) {
                uint16_t pc[8];
                if (STORAGE == B200F_STORAGE_F32 && plane_format == kPlanesFp16x2)
                    // in the scaled units of the planes: (s x).(s x) / 2, fp16 pieces
                    norm_pieces(-0.5f * s * plane_scale * plane_scale, B200F_STORAGE_F16, pc);
                else
                    norm_pieces(-0.5f * s, STORAGE == B200F_STORAGE_F32 ? B200F_STORAGE_BF16 : STORAGE, pc);
                uint16_t* o = (STORAGE == B200F_STORAGE_F32)
                                      ? (planes ? planes + r * plane_pitch + d8 : nullptr)
                                      : reinterpret_cast<uint16_t*>(dst) + r * dst_pitch + d8;
                if (o) {
#pragma unroll
                    for (int i = 0; i < 8; i++) o[i] = pc[i];
                }
            }
        }
    }
}

// Largest |element| of a block of fp32 rows (as the bit pattern of a non-negative float, which
// orders like an unsigned integer): what the index derives the fp16x2 plane scale from.
__global__ void rows_absmax_kernel(const float* __restrict__ src, int64_t pitch, int64_t n, int d,
                                   uint32_t* __restrict__ out_max_bits) {
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = (int64_t)gridDim.x * (blockDim.x >> 5);
    float amax = 0.f;
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n; r += warps_total) {
        const float* row = src + r * pitch;
        for (int j = lane; j < d; j += 32) {
            const float v = fabsf(row[j]);
            if (v < CUDART_INF_F) amax = fmaxf(amax, v);   // NaN and INF do not set the scale
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0 && amax > 0.f) atomicMax(out_max_bits, __float_as_uint(amax));
}

template <int STORAGE>
__global__ void load_rows_kernel(const void* __restrict__ rows, int64_t n, int d, int64_t pitch,
                                 float* __restrict__ dst) {
    const int64_t total = n * (int64_t)d;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / d;
        const int j = (int)(i - r * d);
        dst[i] = load_elem<STORAGE>(rows, r * pitch + j);
    }
}

// ---- query preparation -------------------------------------------------------------------
// fp32 queries -> operand planes of the tensor path (+ exact fp32 squared norms).
// One plane in the storage format (fp16 / bf16) or three bf16 split planes (fp32 storage).
// With norm_cols the 8 columns after d8 of plane 0 receive the norm scales (see above).
__global__ void prepare_queries_kernel(const float* __restrict__ q, int64_t nq, int d, int storage,
                                       uint16_t* __restrict__ a, int64_t a_pitch,
                                       int64_t a_plane_stride, float* __restrict__ qnorm,
                                       int norm_cols, int plane_format, int x_scale_log2,
                                       float* __restrict__ rowscale) {
    const int lane = threadIdx.x & 31;
    const int d8 = (d + 7) & ~7;
    const int fmt = storage == B200F_STORAGE_F16 ? B200F_STORAGE_F16 : B200F_STORAGE_BF16;
    const bool fp16x2 = storage == B200F_STORAGE_F32 && plane_format == kPlanesFp16x2;
    const int64_t warps_total = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < nq;
         r += warps_total) {
        const float* row = q + r * (int64_t)d;
        // fp16x2 planes: every query row gets its own power-of-two scale (largest element near
        // 2^6, as the stored rows), kept at most 2^3 above the rows' scale so that the norm-column
        // scales below stay inside fp16.  The kernel's accumulator is then (sq * sx) * t, and
        // rowscale[r] = 1 / (sq * sx) brings a key back to its units.
        float sq = 1.f, ratio = 1.f;
        if (fp16x2 && a) {
            float amax = 0.f;
            for (int j = lane; j < d; j += 32) {
                const float v = fabsf(row[j]);
                if (v < CUDART_INF_F) amax = fmaxf(amax, v);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            int e = 0;
            if (amax > 0.f) (void)frexpf(amax, &e);   // amax = m * 2^e, m in [0.5, 1)
            int lq = amax > 0.f ? 7 - e : x_scale_log2;
            if (lq > x_scale_log2 + 3) lq = x_scale_log2 + 3;
            if (lq > 126) lq = 126;
            if (lq < -126) lq = -126;
            sq = ldexpf(1.f, lq);
            ratio = ldexpf(1.f, lq - x_scale_log2);            // sq / sx
            if (rowscale && lane == 0) rowscale[r] = ldexpf(1.f, -(lq + x_scale_log2));
        }
        float s = 0.f;
        for (int j = lane; j < a_pitch || j < d; j += 32) {
            float v = (j < d) ? row[j] : 0.f;
            s = fmaf(v, v, s);
            if (a && j < a_pitch) {
                uint16_t* p0 = a + r * a_pitch + j;
                const bool ncol = norm_cols && j >= d8 && j < d8 + 8;
                if (fp16x2) {
                    // norm columns: the stored side holds (sx x).(sx x) / 2 in fp16 pieces
                    const float w = ncol ? norm_scale(B200F_STORAGE_F16, j - d8) * ratio : v * sq;
                    const uint16_t h0 = float_to_fp16_bits(w);
                    p0[0] = h0;
                    p0[a_plane_stride] = ncol ? (uint16_t)0 : float_to_fp16_bits(w - fp16_bits_to_float(h0));
                    continue;
                }
                if (ncol) v = norm_scale(fmt, j - d8);
                if (storage == B200F_STORAGE_F16) {
                    *p0 = float_to_fp16_bits(v);
                } else if (storage == B200F_STORAGE_BF16) {
                    *p0 = float_to_bf16_bits(v);
                } else {
                    uint16_t b0 = float_to_bf16_bits(v);
                    float r1 = v - bf16_bits_to_float(b0);
                    uint16_t b1 = float_to_bf16_bits(r1);
                    float r2 = r1 - bf16_bits_to_float(b1);
                    p0[0] = b0;
                    p0[a_plane_stride] = b1;
                    p0[2 * a_plane_stride] = float_to_bf16_bits(r2);
                }
            }
        }
        if (qnorm) {
            s = warp_sum(s);
            if (lane == 0) qnorm[r] = s;
        }
    }
}

// ---- synthetic generator -------------------------------------------------------------------
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float synth_value(uint64_t seed, int64_t row, int col, int dist) {
    uint64_t h = mix64(seed * 0x9e3779b97f4a7c15ULL + (uint64_t)row * 0xd1342543de82ef95ULL +
                       (uint64_t)col + 1);
    h = mix64(h);
    const float u1 = ((uint32_t)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0,1)
    if (dist == 0) return ((uint32_t)(h >> 40)) * (1.0f / 16777216.0f);   // [0,1)
    const float u2 = ((uint32_t)(h & 0xffffffu)) * (1.0f / 16777216.0f);
    return sqrtf(-2.f * logf(u1)) * cospif(2.f * u2);
}

__global__ void fill_synthetic_kernel(float* __restrict__ dst, int64_t n, int d, int64_t row0,
                                      uint64_t seed, int dist, float scale) {
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n;
         r += warps_total) {
        float* row = dst + r * (int64_t)d;
        if (dist == 2) {
            float s = 0.f;
            for (int j = lane; j < d; j += 32) {
                float v = synth_value(seed, row0 + r, j, 1);
                s = fmaf(v, v, s);
            }
            s = warp_sum(s);
            const float inv = s > 0.f ? rsqrtf(s) : 0.f;
            for (int j = lane; j < d; j += 32) row[j] = synth_value(seed, row0 + r, j, 1) * inv;
        } else if (dist == 3) {
            // mixture of 1,000 gaussians: the centres (uniform in [-1,1]^d) are the same for
            // every seed, so that rows and queries of different seeds share them
            const uint64_t c = mix64(seed * 0x9e3779b97f4a7c15ULL + (uint64_t)(row0 + r) * 0xd1342543de82ef95ULL) % 1000u;
            for (int j = lane; j < d; j += 32)
                row[j] = 2.f * synth_value(0x6d697874ULL, (int64_t)c, j, 0) - 1.f +
                         scale * synth_value(seed, row0 + r, j, 1);
        } else {
            for (int j = lane; j < d; j += 32)
                row[j] = synth_value(seed, row0 + r, j, dist) * (dist == 1 ? scale : 1.f);
        }
    }
}

int grid_for_rows(int64_t n) {
    int64_t g = ceil_div64(n, ROW_THREADS / 32);
    int64_t cap = (int64_t)cached_sm_count() * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace

int device_slot() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return (dev >= 0 && dev < kMaxDevices) ? dev : kMaxDevices - 1;
}

// SM count of the CURRENT device (a process may drive several GPUs: one value per device).
int cached_sm_count() {
    static int sm[kMaxDevices] = {0};
    const int slot = device_slot();
    if (sm[slot] == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            return kNumSMsDefault;
        }
        sm[slot] = n;
    }
    return sm[slot];
}

int launch_prepare_queries(const float* q, int64_t nq, int d, int storage, uint16_t* a_planes,
                           int64_t a_pitch, int64_t a_plane_stride, float* qnorm, int norm_cols,
                           int plane_format, int x_scale_log2, float* rowscale, cudaStream_t stream) {
    if (nq <= 0) return B200F_OK;
    prepare_queries_kernel<<<grid_for_rows(nq), ROW_THREADS, 0, stream>>>(
            q, nq, d, storage, a_planes, a_pitch, a_plane_stride, qnorm, norm_cols, plane_format, x_scale_log2,
            rowscale);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

}  // namespace b200f

using namespace b200f;

extern "C" int b200f_row_norms(const void* rows, int storage, int64_t n, int d, int64_t pitch_elems,
                               float* out, void* stream) {
    if (n < 0 || d <= 0 || pitch_elems < d || (n > 0 && (!rows || !out))) return B200F_ERR_BAD_ARG;
    if (n == 0) return B200F_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int g = grid_for_rows(n);
    switch (storage) {
        case B200F_STORAGE_F32:
            row_norms_kernel<B200F_STORAGE_F32><<<g, ROW_THREADS, 0, st>>>(rows, n, d, pitch_elems, out);
            break;
        case B200F_STORAGE_F16:
            row_norms_kernel<B200F_STORAGE_F16><<<g, ROW_THREADS, 0, st>>>(rows, n, d, pitch_elems, out);
            break;
        case B200F_STORAGE_BF16:
            row_norms_kernel<B200F_STORAGE_BF16><<<g, ROW_THREADS, 0, st>>>(rows, n, d, pitch_elems, out);
            break;
        default:
            return B200F_ERR_BAD_ARG;
    }
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

namespace {
int store_rows_impl(const float* src, int64_t src_pitch, int64_t n, int d, int storage, void* dst_rows,
                    int64_t dst_pitch, uint16_t* planes, int64_t plane_pitch, int64_t plane_stride,
                    int plane_format, int plane_scale_log2, int32_t* range_flag, float* norms_or_null,
                    int norm_cols, void* stream) {
    if (n < 0 || d <= 0 || dst_pitch < d || src_pitch < d || (n > 0 && (!src || !dst_rows))) return B200F_ERR_BAD_ARG;
    if (planes && (plane_pitch < d || plane_stride < plane_pitch)) return B200F_ERR_BAD_ARG;
    if (plane_format != B200F_PLANES_BF16X3 && plane_format != B200F_PLANES_FP16X2) return B200F_ERR_BAD_ARG;
    if (plane_scale_log2 < -126 || plane_scale_log2 > 126) return B200F_ERR_BAD_ARG;
    if (norm_cols) {
        const int64_t need = ((d + 7) & ~7) + 8;
        if (storage == B200F_STORAGE_F32 ? (planes && plane_pitch < need) : dst_pitch < need)
            return B200F_ERR_BAD_ARG;
    }
    if (n == 0) return B200F_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int g = grid_for_rows(n);
    const float scale = std::ldexp(1.f, plane_scale_log2);
    switch (storage) {
        case B200F_STORAGE_F32:
            store_rows_kernel<B200F_STORAGE_F32><<<g, ROW_THREADS, 0, st>>>(
                    src, src_pitch, n, d, dst_rows, dst_pitch, planes, plane_pitch, plane_stride, plane_format, scale,
                    range_flag, norms_or_null, norm_cols);
            break;
        case B200F_STORAGE_F16:
            store_rows_kernel<B200F_STORAGE_F16><<<g, ROW_THREADS, 0, st>>>(
                    src, src_pitch, n, d, dst_rows, dst_pitch, nullptr, 0, 0, 0, 1.f, nullptr, norms_or_null, norm_cols);
            break;
        case B200F_STORAGE_BF16:
            store_rows_kernel<B200F_STORAGE_BF16><<<g, ROW_THREADS, 0, st>>>(
                    src, src_pitch, n, d, dst_rows, dst_pitch, nullptr, 0, 0, 0, 1.f, nullptr, norms_or_null, norm_cols);
            break;
        default:
            return B200F_ERR_BAD_ARG;
    }
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}
}  // namespace

extern "C" int b200f_store_rows(const float* src, int64_t n, int d, int storage, void* dst_rows,
                                int64_t dst_pitch, uint16_t* planes, int64_t plane_pitch,
                                int64_t plane_stride, float* norms_or_null, int norm_cols,
                                void* stream) {
    return store_rows_impl(src, d, n, d, storage, dst_rows, dst_pitch, planes, plane_pitch, plane_stride,
                           B200F_PLANES_BF16X3, 0, nullptr, norms_or_null, norm_cols, stream);
}

extern "C" int b200f_store_rows_fp32(const float* src, int64_t src_pitch, int64_t n, int d, float* dst_rows,
                                     int64_t dst_pitch, uint16_t* planes, int64_t plane_pitch,
                                     int64_t plane_stride, int plane_format, int plane_scale_log2,
                                     int32_t* range_flag, float* norms_or_null, int norm_cols, void* stream) {
    return store_rows_impl(src, src_pitch, n, d, B200F_STORAGE_F32, dst_rows, dst_pitch, planes, plane_pitch,
                           plane_stride, plane_format, plane_scale_log2, range_flag, norms_or_null, norm_cols, stream);
}

extern "C" int b200f_rows_absmax(const float* rows, int64_t n, int d, int64_t pitch_elems, uint32_t* max_bits,
                                 void* stream) {
    if (n < 0 || d <= 0 || pitch_elems < d || !max_bits || (n > 0 && !rows)) return B200F_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    B200F_CUDA_TRY(cudaMemsetAsync(max_bits, 0, sizeof(uint32_t), st));
    if (n == 0) return B200F_OK;
    rows_absmax_kernel<<<grid_for_rows(n), ROW_THREADS, 0, st>>>(rows, pitch_elems, n, d, max_bits);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

extern "C" int b200f_load_rows(const void* rows, int storage, int64_t n, int d, int64_t pitch_elems,
                               float* dst, void* stream) {
    if (n < 0 || d <= 0 || pitch_elems < d || (n > 0 && (!rows || !dst))) return B200F_ERR_BAD_ARG;
    if (n == 0) return B200F_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int64_t total = n * (int64_t)d;
    int64_t g = ceil_div64(total, 256);
    int64_t cap = (int64_t)cached_sm_count() * 32;
    if (g > cap) g = cap;
    switch (storage) {
        case B200F_STORAGE_F32:
            load_rows_kernel<B200F_STORAGE_F32><<<(int)g, 256, 0, st>>>(rows, n, d, pitch_elems, dst);
            break;
        case B200F_STORAGE_F16:
            load_rows_kernel<B200F_STORAGE_F16><<<(int)g, 256, 0, st>>>(rows, n, d, pitch_elems, dst);
            break;
        case B200F_STORAGE_BF16:
            load_rows_kernel<B200F_STORAGE_BF16><<<(int)g, 256, 0, st>>>(rows, n, d, pitch_elems, dst);
            break;
        default:
            return B200F_ERR_BAD_ARG;
    }
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}

extern "C" int b200f_fill_synthetic(float* dst, int64_t n, int d, int64_t row0, uint64_t seed,
                                    int dist, float scale, void* stream) {
    if (n < 0 || d <= 0 || dist < 0 || dist > 3 || (n > 0 && !dst)) return B200F_ERR_BAD_ARG;
    if (n == 0) return B200F_OK;
    fill_synthetic_kernel<<<grid_for_rows(n), ROW_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
            dst, n, d, row0, seed, dist, scale);
    count_launch();
    B200F_LAUNCH_CHECK();
    return B200F_OK;
}
