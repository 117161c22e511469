// Shared host/device helpers of the fp4t library: error reporting, number-format
// conversions and the scale-factor tile addressing used by every kernel.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "../../include/fp4t.h"

namespace fp4t {

// Thread-local error text behind fp4t_last_error().
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define FP4T_REQUIRE(cond, ...)            \
  do {                                     \
    if (!(cond)) {                         \
      ::fp4t::set_error(__VA_ARGS__);      \
      return FP4T_ERR_ARG;                 \
    }                                      \
  } while (0)

#define FP4T_CUDA(call)                                        \
  do {                                                         \
    cudaError_t e_ = (call);                                   \
    if (e_ != cudaSuccess) return ::fp4t::cuda_fail(e_, #call); \
  } while (0)

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Number of SMs the persistent kernels may fill on the current device (the device's SM count,
// or the smaller process-wide limit set with fp4t_set_sm_limit), or -1 if it is not an sm_100 part.
int sm_count();
int sm_limit();

// Dynamic tile scheduling: persistent kernels draw tile indices from a device counter so that
// CTAs that start late (their SM was busy with another stream's kernel, e.g. a collective)
// simply take fewer tiles.  Kernels on one stream never overlap, so each (device, stream)
// pair owns one counter slot; returns -1 (use the static round-robin order) when the stream
// is being captured into a graph, when the table is full or when FP4T_STATIC_TILES=1.
constexpr int kSchedSlots = 64;
int sched_slot_for(cudaStream_t stream);

// Launch attribute that lets a kernel start under the tail of its predecessor (the kernel must
// call griddepcontrol.wait before it touches global memory).  FP4T_NO_PDL=1 switches it off.
bool pdl_enabled();
inline void pdl_attribute(cudaLaunchAttribute* attr) {
  attr->id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr->val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
}
int reset_gemm_tile_counters(cudaStream_t stream);      // fp4t_gemm.cu
int set_wait_timeout_gemm(uint64_t ns);                 // fp4t_gemm.cu
int set_wait_timeout_quantize(uint64_t ns);             // fp4t_quantize.cu
int set_wait_timeout_allreduce(uint64_t ns);            // fp4t_allreduce.cu
int reset_quantize_tile_counters(cudaStream_t stream);  // fp4t_quantize.cu

// 2-D tiled tensor map over a row-major matrix [outer, inner] of `dtype` elements whose rows
// are row_pitch_bytes apart; out-of-range parts of a box read as zero.
int encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, uint64_t inner,
                         uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner, uint32_t box_outer,
                         CUtensorMapSwizzle swizzle);

// Device status word used by kernels whose entry point has no status parameter
// (set per host thread with fp4t_set_status_word, may be null).
int32_t* current_status_word();

// Device word added to the seed of in-kernel stochastic rounding when a kernel runs (null: none);
// set per device with fp4t_set_seed_offset_word.
const uint64_t* seed_offset_word();

// Byte offset of scale (outer o, k-block i) in the 128x4 tile layout with `ntx`
// tiles along the k-block axis.
__host__ __device__ __forceinline__ int64_t sf_offset(int64_t o, int64_t i, int64_t ntx) {
  return ((o >> 7) * ntx + (i >> 2)) * 512 + (o & 31) * 16 + ((o & 127) >> 5) * 4 + (i & 3);
}

// Offset inside one 512-byte tile.
__device__ __forceinline__ int sf_tile_offset(int o, int i) {
  return (o & 31) * 16 + ((o & 127) >> 5) * 4 + (i & 3);
}

#ifdef __CUDACC__

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t hi16_in_low) {
  return __uint_as_float(hi16_in_low << 16);
}

// Eight fp32 values -> eight E2M1 codes in one 32-bit word, element j in nibble j.
// Round to nearest even, saturate to +-6, sign bit kept (so -0.0f -> 0x8).
__device__ __forceinline__ uint32_t cvt_e2m1x8(float v0, float v1, float v2, float v3,
                                               float v4, float v5, float v6, float v7) {
  uint32_t out;
  asm("{\n\t"
      ".reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t"
      "}"
      : "=r"(out)
      : "f"(v0), "f"(v1), "f"(v2), "f"(v3), "f"(v4), "f"(v5), "f"(v6), "f"(v7));
  return out;
}

// Two fp32 values -> one byte of E2M1 codes (lo in bits 0..3).
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  uint32_t out;
  asm("{\n\t"
      ".reg .b8 b0;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.u32.u8 %0, b0;\n\t"
      "}"
      : "=r"(out)
      : "f"(lo), "f"(hi));
  return out;
}

// fp32 in [2^-9, 448] -> E4M3 byte, round to nearest even.
__device__ __forceinline__ uint32_t cvt_e4m3(float v) {
  return (uint32_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// NVFP4 block scale from the block's amax: clamp(amax / 6, 2^-9, 448) with a true division.
__device__ __forceinline__ float nvfp4_scale(float amax) {
  return fminf(fmaxf(__fdiv_rn(amax, 6.0f), 0x1p-9f), 448.0f);
}

// Table form of the same scale for an amax that came from bf16 (7 mantissa bits): entry m
// holds RN((1 + m/128) / 6) and its correctly rounded reciprocal; the power of two of amax
// is applied by adding to / subtracting from the exponent field.  Gives the same s as
// nvfp4_scale and r = RN(1/s) for every finite non-negative bf16 amax (checked exhaustively
// on the host), without any division.
struct ScalePair { float s, r; };
struct ScaleTable { ScalePair v[128]; };
constexpr ScaleTable make_scale_table() {
  ScaleTable t{};
  for (int m = 0; m < 128; ++m) {
    const float s = (1.0f + (float)m / 128.0f) / 6.0f;
    t.v[m].s = s;
    t.v[m].r = 1.0f / s;
  }
  return t;
}
__device__ __forceinline__ void nvfp4_scale_from_table(const float2* __restrict__ tab, float amax, float& s,
                                                       float& r) {
  // amax below 2^-102 would underflow the exponent arithmetic; it ends at the lower clamp anyway
  const uint32_t b = max(__float_as_uint(amax), 0x0C800000u);
  const float2 t = tab[(b >> 16) & 0x7Fu];
  const uint32_t e = (b & 0x7F800000u) - 0x3F800000u;
  const float sf = __uint_as_float(__float_as_uint(t.x) + e);
  const float rf = __uint_as_float(__float_as_uint(t.y) - e);
  // clamp(s, 2^-9, 448); the reciprocal is monotonic, so clamping it to [RN(1/448), 512] gives
  // RN(1/s) of the clamped scale
  s = fminf(fmaxf(sf, 0x1p-9f), 448.0f);
  r = fminf(fmaxf(rf, 1.0f / 448.0f), 512.0f);
}
// UE4M3 byte of a scale in [2^-9, 448], round to nearest even, integer / FMA pipes only.
__device__ __forceinline__ uint32_t e4m3_byte_of_scale(float s) {
  const uint32_t den = __float_as_uint(fmaf(s, 512.0f, 12582912.0f)) & 0xFu;   // multiples of 2^-9
  const uint32_t b = __float_as_uint(s);
  const uint32_t nrm = ((b + 0x7FFFFu + ((b >> 20) & 1u)) >> 20) - (120u << 3);
  return s < 0x1p-6f ? den : nrm;
}

// x / s rounded to nearest, computed as a reciprocal multiply plus one FMA correction.
// With r = RN(1/s) this returns RN(x/s) for every bf16 x and every scale derived from a
// bf16 amax (checked exhaustively on the host); -0.0f comes out as +0.0f.
__device__ __forceinline__ float div_corrected(float x, float s, float r) {
  float q = x * r;
  float rem = fmaf(-q, s, x);
  return fmaf(rem, r, q);
}

// Stochastic E2M1 rounding of y with u in [0,1):
//   e = clamp(floor(log2|y|), 0, 2), m = |y| / 2^e, r = rint(2m + (u - 0.5)),
//   q = sign(y) * 2^e * (r / 2)          (a later RNE+saturate conversion clips 8 to 6)
__device__ __forceinline__ float sr_round(float y, float u) {
  float a = fabsf(y);
  float p2 = a >= 4.0f ? 4.0f : (a >= 2.0f ? 2.0f : 1.0f);
  float inv = a >= 4.0f ? 0.25f : (a >= 2.0f ? 0.5f : 1.0f);
  float m = a * inv;
  float r = rintf(fmaf(m, 2.0f, u - 0.5f)) * 0.5f;
  float sgn = y > 0.0f ? 1.0f : (y < 0.0f ? -1.0f : 0.0f);
  return (sgn * p2) * r;
}

// ---- packed fp32 pairs (FFMA2 / FMUL2 on sm_100) --------------------------------------
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// The two bf16 halves of a 32-bit word as a packed fp32 pair (low half first).
__device__ __forceinline__ uint64_t bf16x2_to_f32x2(uint32_t w) {
  return pack2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
// Packed form of div_corrected: x / s for two lanes, rcp = RN(1/s), neg_s = -s.
__device__ __forceinline__ uint64_t div_corrected2(uint64_t x, uint64_t neg_s, uint64_t rcp) {
  const uint64_t q = mul2(x, rcp);
  const uint64_t rem = fma2(q, neg_s, x);
  return fma2(rem, rcp, q);
}

// 32-bit integer mix (two multiply-xorshift rounds).
__device__ __forceinline__ uint32_t mix32(uint32_t h) {
  h ^= h >> 16; h *= 0x7FEB352Du;
  h ^= h >> 15; h *= 0x846CA68Bu;
  h ^= h >> 16;
  return h;
}

// Stochastic rounding of y onto the E2M1 grid with 16 random bits: the grid keeps one
// mantissa bit (after lifting [0,1) to [1,2)), so adding uniform bits below that bit and
// truncating rounds up with probability equal to the discarded fraction.  Same distribution
// as sr_round, a fraction of the instructions; results above 6 are clipped by the conversion.
__device__ __forceinline__ float sr_round_bits(float y, uint32_t r16) {
  const float a = fabsf(y);
  const bool small = a < 1.0f;
  const float t = small ? a + 1.0f : a;
  const uint32_t b = (__float_as_uint(t) + (r16 << 6)) & 0xFFC00000u;
  float q = __uint_as_float(b);
  q = small ? q - 1.0f : q;
  return copysignf(q, y);
}

// MXFP8 element conversion for values that came from bf16 (at most 8 significant bits):
// setting the lowest fp32 mantissa bit moves exact ties off the tie, so the hardware's
// round-to-nearest-even conversion lands where ties-away-from-zero would.  y0 / y1 must
// already be +0 for zero inputs.
__device__ __forceinline__ uint32_t mx_e4m3x2_from_bf16(float y0, float y1) {
  const float a = __uint_as_float(__float_as_uint(y0) | 1u);
  const float b = __uint_as_float(__float_as_uint(y1) | 1u);
  uint32_t out;
  asm("{\n\t.reg .b16 h;\n\tcvt.rn.satfinite.e4m3x2.f32 h, %2, %1;\n\tcvt.u32.u16 %0, h;\n\t}"
      : "=r"(out) : "f"(a), "f"(b));
  return out;
}

// Counter-based uniform in [0,1) with 24 random bits from (seed, index).
__device__ __forceinline__ float hash_uniform(uint64_t seed, uint64_t idx) {
  uint32_t h = (uint32_t)idx * 0x9E3779B1u ^ (uint32_t)seed;
  h ^= (uint32_t)(idx >> 32) * 0x85EBCA77u + (uint32_t)(seed >> 32);
  h ^= h >> 16; h *= 0x85EBCA6Bu;
  h ^= h >> 13; h *= 0xC2B2AE35u;
  h ^= h >> 16;
  return (float)(h >> 8) * 0x1p-24f;
}

// MXFP8: E8M0 byte of a block from its amax (floor(log2 amax) - 8 + 127, clamped at 0).
__device__ __forceinline__ uint32_t mx_scale_byte(float amax) {
  int e8 = (int)(__float_as_uint(amax) >> 23) & 0xFF;
  int b = e8 - 8;
  return (uint32_t)(b < 0 ? 0 : b);
}
// Multiplier 2^-(byte-127) that maps block elements into the E4M3 range.
__device__ __forceinline__ float mx_inv_scale(uint32_t byte) {
  return __uint_as_float((254u - byte) << 23);
}

// y -> E4M3 byte. Three mantissa bits, ties away from zero, denormals kept (grid 2^-9),
// saturating at +-448.
template <bool kHalfAway>
__device__ __forceinline__ uint32_t mx_e4m3_byte(float y) {
  if (!kHalfAway) {
    return (uint32_t)__nv_cvt_float_to_fp8(y + 0.0f, __NV_SATFINITE, __NV_E4M3);
  }
  uint32_t sign = y < 0.0f ? 0x80u : 0u;  // sign(0) is 0: -0.0f encodes as +0
  float a = fabsf(y);
  bool den = a < 0x1p-6f;
  float a2 = den ? a + 0x1p-6f : a;
  uint32_t b = (__float_as_uint(a2) + 0x00080000u) >> 20;
  int v = (int)b - (den ? (121 << 3) : (120 << 3));
  v = v > 0x7E ? 0x7E : v;
  return (uint32_t)v | sign;
}

#endif  // __CUDACC__

}  // namespace fp4t
