// Fused block quantizers for NVFP4 (1x16 blocks, UE4M3 scales) and MXFP8 (1x32
// blocks, UE8M0 scales).
//
// One launch reads every 128x128 tile of the bf16 input once (TMA into shared
// memory), and writes
//   - the row-wise codes and their scales, and / or
//   - the codes and scales of the TRANSPOSED tensor (blocks along the row axis),
//     built from a shared-memory copy of the tile,
// with the scale bytes placed directly in the 128x4 tile layout the block-scaled
// MMA consumes.  The kernels are HBM-bound: algorithmic traffic per element is
// 2 B in plus 0.5 B (NVFP4) or 1 B (MXFP8) per emitted copy plus the scales.
//
// A second, generic kernel handles fp32 input and unaligned shapes with plain
// per-block loops; it is the slow but general form of the same arithmetic.
#include <mutex>

#include "fp4t_common.cuh"
#include "fp4t_ptx.cuh"

namespace fp4t {
namespace {

constexpr int kTile = 128;

struct QParams {
  const void* x;
  int64_t rows, cols, ld;
  uint8_t* codes;
  uint8_t* sf;
  uint8_t* codes_t;
  uint8_t* sf_t;
  const float* noise;
  const float* noise_t;
  float* colsum;   // optional fp32 [cols] accumulator of column sums (transposed pass only)
  uint64_t seed;
  float tscale, tscale_inv;   // per-tensor scale applied before block quantization (kPre == 2), and its reciprocal
  uint32_t rht_signs;         // generic path: bit 16 set = random Hadamard transform of each 16-block, bits 0..15 the signs
  const uint64_t* seed_dev;   // optional device word added (times an odd constant) to `seed` when the kernel runs
  int ntx_row;  // scale tiles along k for the row-wise output
  int ntx_col;  // ... for the transposed output
};

enum { kNvfp4 = 0, kMxfp8 = 1 };

// ---------------------------------------------------------------------------------------
// Fast path: bf16 input with 16-byte aligned rows.
//
// Persistent CTAs (two per SM).  Warp 8 is the producer: it streams 128x128 bf16 tiles into
// a 3-deep shared-memory ring with TMA (out-of-range parts read as zero).  Warps 0-7 wait on
// the tile's mbarrier and make two passes over it:
//   row pass   each thread owns one whole block of a row (two or four 16-byte loads);
//   column pass each thread owns two adjacent columns and 32 rows, i.e. whole blocks of the
//              transposed tensor, read from shared memory as packed bf16 pairs.
// Division by the block scale is done on packed fp32 pairs (reciprocal multiply + one FMA
// correction, exact for bf16 inputs).  Scale bytes are staged in shared memory in tile
// layout and leave as whole 512-byte tiles.
// ---------------------------------------------------------------------------------------
__constant__ ScaleTable kScaleTable = make_scale_table();

constexpr int kQStages = 3;
constexpr int kQComputeThreads = 256;
constexpr int kQThreads = kQComputeThreads + 32;
constexpr int kQTileBytes = kTile * kTile * 2;

template <int kFmt>
struct QCfg {
  static constexpr int kBlk = kFmt == kNvfp4 ? 16 : 32;
  static constexpr int kKbTile = kTile / kBlk;       // k-blocks per tile edge: 8 or 4
  static constexpr int kSfChunks = kKbTile / 4;      // 512-byte scale tiles per tile edge: 2 or 1
  static constexpr int kSfStage = kSfChunks * 512;   // bytes of one staging buffer
  static constexpr int kSmemBytes = kQStages * kQTileBytes + 4 * kSfStage + 64 + 128 + 1024 + 4096;
};

__device__ __forceinline__ void named_barrier_compute() {
  asm volatile("bar.sync 1, %0;" ::"n"(kQComputeThreads) : "memory");
}

// Four fp32 values -> four E2M1 codes (e0 in the lowest nibble) with the hardware's stochastic
// rounding; rbits supplies the random bits of all four conversions.
__device__ __forceinline__ uint32_t cvt_rs_e2m1x4(float e0, float e1, float e2, float e3, uint32_t rbits) {
  uint32_t out;
  asm("{\n\t.reg .b16 h;\n\tcvt.rs.satfinite.e2m1x4.f32 h, {%4, %3, %2, %1}, %5;\n\tcvt.u32.u16 %0, h;\n\t}"
      : "=r"(out)
      : "f"(e0), "f"(e1), "f"(e2), "f"(e3), "r"(rbits));
  return out;
}
// Random bits for eight elements (two cvt.rs words) from the index of the 8-element group:
// a Weyl step, one multiply-xorshift round for the first word and one more multiply-xorshift
// for the second.  Bit means are within 1e-3 of 1/2 and the lag-1 correlation between
// neighbouring groups is below 1e-2 (checked on the host over 4M indices).
__device__ __forceinline__ uint32_t hash_pair(uint32_t idx8, uint32_t seed_lo, uint32_t seed_hi, uint32_t& second) {
  uint32_t h = idx8 * 0x9E3779B9u + seed_lo;
  h ^= h >> 16; h *= 0x7FEB352Du; h ^= h >> 15;
  h ^= seed_hi;
  uint32_t t = h * 0x846CA68Bu;
  second = t ^ (t >> 16);
  return h;
}
__device__ __forceinline__ float amax8(const uint32_t (&w)[4]) {
  const float m0 = fmaxf(fabsf(__uint_as_float(w[0] << 16)), fabsf(__uint_as_float(w[0] & 0xFFFF0000u)));
  const float m1 = fmaxf(fabsf(__uint_as_float(w[1] << 16)), fabsf(__uint_as_float(w[1] & 0xFFFF0000u)));
  const float m2 = fmaxf(fabsf(__uint_as_float(w[2] << 16)), fabsf(__uint_as_float(w[2] & 0xFFFF0000u)));
  const float m3 = fmaxf(fabsf(__uint_as_float(w[3] << 16)), fabsf(__uint_as_float(w[3] & 0xFFFF0000u)));
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

struct TileCtx {
  const uint8_t* tile;      // 128 x 128 bf16, 256-byte rows
  uint8_t* sf_row_s;
  uint8_t* sf_col_s;
  float* colsum_s;          // [4][128] partial column sums of this tile
  const float2* scale_tab;
  int64_t row0, col0;
  uint64_t seed;            // effective seed of this launch
  int tid;
};

// ---- row-wise pass: a thread owns one whole block of a row (16 or 32 elements) ----------
// 8 (NVFP4) or 4 (MXFP8) threads cover a tile row, so the block's abs-max needs no shuffle and
// the scale work (table look-up, scale byte, packed operands) is paid once per block.
template <int kFmt, int kSr, bool kEdge, bool kTs = false>
__device__ __forceinline__ void row_pass(const QParams& p, const TileCtx& c) {
  using C = QCfg<kFmt>;
  constexpr int kTpr = kTile / C::kBlk;                // threads per tile row
  constexpr int kRowsPerIt = kQComputeThreads / kTpr;  // 32 or 64 rows per sweep
  constexpr int kIts = kTile / kRowsPerIt;             // 4 or 2 sweeps
  constexpr int kVecs = C::kBlk / 8;                   // 16-byte loads per block
  const int r_base = c.tid / kTpr, kb = c.tid % kTpr;
  const int64_t gc = c.col0 + kb * C::kBlk;
  const bool col_ok = !kEdge || gc < p.cols;
  const int64_t code_pitch = kFmt == kNvfp4 ? (p.cols >> 1) : p.cols;
  uint8_t* out = p.codes + (c.row0 + r_base) * code_pitch + (kFmt == kNvfp4 ? (gc >> 1) : gc);
  const int64_t out_step = kRowsPerIt * code_pitch;
  const uint8_t* src = c.tile + r_base * 256 + kb * (C::kBlk * 2);
  uint8_t* sf_dst = c.sf_row_s + (kb >> 2) * 512 + (kb & 3);
  const uint32_t seed_lo = (uint32_t)c.seed, seed_hi = (uint32_t)(c.seed >> 32);

  // Phase 1: every load of the thread's kIts blocks is issued before any arithmetic, and every
  // store comes after all of it.  A store into the scale staging area may alias the tile as
  // far as the compiler can tell, so loads written after it would wait for it; separating the
  // phases lets the shared-memory latency of all blocks overlap.
  uint32_t w[kIts][kVecs][4];
#pragma unroll
  for (int it = 0; it < kIts; ++it) {
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const uint4 q = *reinterpret_cast<const uint4*>(src + it * kRowsPerIt * 256 + v * 16);
      w[it][v][0] = q.x; w[it][v][1] = q.y; w[it][v][2] = q.z; w[it][v][3] = q.w;
    }
  }
  float amax[kIts];
#pragma unroll
  for (int it = 0; it < kIts; ++it) {
    amax[it] = amax8(w[it][0]);
#pragma unroll
    for (int v = 1; v < kVecs; ++v) amax[it] = fmaxf(amax[it], amax8(w[it][v]));
  }
  bool valid[kIts];
#pragma unroll
  for (int it = 0; it < kIts; ++it) valid[it] = !kEdge || (col_ok && c.row0 + it * kRowsPerIt + r_base < p.rows);

  uint32_t sf_byte[kIts];
  if (kFmt == kNvfp4) {
    float s[kIts], rcp[kIts];
#pragma unroll
    for (int it = 0; it < kIts; ++it) nvfp4_scale_from_table(c.scale_tab, kTs ? amax[it] * p.tscale : amax[it], s[it], rcp[it]);
    uint32_t packed[kIts][2];
#pragma unroll
    for (int it = 0; it < kIts; ++it) {
      const int64_t gr = c.row0 + it * kRowsPerIt + r_base;
      // with a (power of two) tensor scale t the block scale s belongs to x t: x t / s = x / (s / t)
      const float se = kTs ? s[it] * p.tscale_inv : s[it], re = kTs ? rcp[it] * p.tscale : rcp[it];
      const uint64_t rcp2 = pack2(re, re), neg2 = pack2(-se, -se);
#pragma unroll
      for (int v = 0; v < 2; ++v) {
        float y[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) unpack2(div_corrected2(bf16x2_to_f32x2(w[it][v][j]), neg2, rcp2), y[2 * j], y[2 * j + 1]);
        if (kSr == FP4T_SR_HASH) {
          uint32_t h1;
          const uint32_t h0 = hash_pair((uint32_t)((gr * p.cols + gc) >> 3) + v, seed_lo, seed_hi, h1);
          packed[it][v] = cvt_rs_e2m1x4(y[0], y[1], y[2], y[3], h0) | (cvt_rs_e2m1x4(y[4], y[5], y[6], y[7], h1) << 16);
        } else {
          if (kSr == FP4T_SR_NOISE) {
            const float4* np = reinterpret_cast<const float4*>(p.noise + gr * p.cols + gc + 8 * v);
            const float4 n0 = valid[it] ? __ldg(np) : make_float4(0.5f, 0.5f, 0.5f, 0.5f);
            const float4 n1 = valid[it] ? __ldg(np + 1) : make_float4(0.5f, 0.5f, 0.5f, 0.5f);
            y[0] = sr_round(y[0], n0.x); y[1] = sr_round(y[1], n0.y); y[2] = sr_round(y[2], n0.z); y[3] = sr_round(y[3], n0.w);
            y[4] = sr_round(y[4], n1.x); y[5] = sr_round(y[5], n1.y); y[6] = sr_round(y[6], n1.z); y[7] = sr_round(y[7], n1.w);
          }
          packed[it][v] = cvt_e2m1x8(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7]);
        }
      }
      sf_byte[it] = e4m3_byte_of_scale(s[it]);
    }
#pragma unroll
    for (int it = 0; it < kIts; ++it)
      if (valid[it]) *reinterpret_cast<uint2*>(out + it * out_step) = make_uint2(packed[it][0], packed[it][1]);
  } else {
    uint32_t o[kIts][8];
#pragma unroll
    for (int it = 0; it < kIts; ++it) {
      const uint32_t sb = mx_scale_byte(amax[it]);
      const float inv = mx_inv_scale(sb);
#pragma unroll
      for (int v = 0; v < 4; ++v) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t w0 = w[it][v][2 * h], w1 = w[it][v][2 * h + 1];
          o[it][2 * v + h] = mx_e4m3x2_from_bf16(fmaf(__uint_as_float(w0 << 16), inv, 0.0f),
                                                fmaf(__uint_as_float(w0 & 0xFFFF0000u), inv, 0.0f)) |
                             (mx_e4m3x2_from_bf16(fmaf(__uint_as_float(w1 << 16), inv, 0.0f),
                                                  fmaf(__uint_as_float(w1 & 0xFFFF0000u), inv, 0.0f)) << 16);
        }
      }
      sf_byte[it] = sb;
    }
#pragma unroll
    for (int it = 0; it < kIts; ++it) {
      if (valid[it]) {
        uint4* dst = reinterpret_cast<uint4*>(out + it * out_step);
        dst[0] = make_uint4(o[it][0], o[it][1], o[it][2], o[it][3]);
        dst[1] = make_uint4(o[it][4], o[it][5], o[it][6], o[it][7]);
      }
    }
  }
#pragma unroll
  for (int it = 0; it < kIts; ++it)
    sf_dst[sf_tile_offset(it * kRowsPerIt + r_base, 0)] = valid[it] ? (uint8_t)sf_byte[it] : (uint8_t)0;
}

// ---- transposed pass: a thread handles 2 adjacent columns x 32 rows --------------------
template <int kFmt, int kSr, bool kEdge, bool kColsum, bool kTs = false>
__device__ __forceinline__ void col_pass(const QParams& p, const TileCtx& c) {
  const int cp = c.tid & 63, q = c.tid >> 6;
  const int64_t gr0 = c.row0 + q * 32, gcA = c.col0 + 2 * cp;
  const bool rows_ok = !kEdge || gr0 < p.rows;       // rows % 32 == 0: all 32 rows in or out
  const bool okA = rows_ok && (!kEdge || gcA < p.cols), okB = rows_ok && (!kEdge || gcA + 1 < p.cols);
  const uint32_t* col_words = reinterpret_cast<const uint32_t*>(c.tile + (q * 32) * 256) + cp;
  uint64_t sum2 = 0;   // packed fp32 (0, 0)
  // all 32 words of the thread's two columns first (see row_pass on why loads precede stores)
  uint32_t w[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) w[j] = col_words[j * 64];
  if (kFmt == kNvfp4) {
    uint32_t outA[4], outB[4];
    uint32_t sfA[2], sfB[2];
    const uint32_t seed_lo = (uint32_t)c.seed ^ 0x5BD1E995u, seed_hi = (uint32_t)(c.seed >> 32);
    float sA[2], sB[2], rA[2], rB[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float mA[4], mB[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t* ww = w + h * 16 + 4 * j;
        mA[j] = fmaxf(fmaxf(fabsf(__uint_as_float(ww[0] << 16)), fabsf(__uint_as_float(ww[1] << 16))),
                      fmaxf(fabsf(__uint_as_float(ww[2] << 16)), fabsf(__uint_as_float(ww[3] << 16))));
        mB[j] = fmaxf(fmaxf(fabsf(__uint_as_float(ww[0] & 0xFFFF0000u)), fabsf(__uint_as_float(ww[1] & 0xFFFF0000u))),
                      fmaxf(fabsf(__uint_as_float(ww[2] & 0xFFFF0000u)), fabsf(__uint_as_float(ww[3] & 0xFFFF0000u))));
      }
      const float amA = fmaxf(fmaxf(mA[0], mA[1]), fmaxf(mA[2], mA[3]));
      const float amB = fmaxf(fmaxf(mB[0], mB[1]), fmaxf(mB[2], mB[3]));
      nvfp4_scale_from_table(c.scale_tab, kTs ? amA * p.tscale : amA, sA[h], rA[h]);
      nvfp4_scale_from_table(c.scale_tab, kTs ? amB * p.tscale : amB, sB[h], rB[h]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint64_t rcp2 = kTs ? pack2(rA[h] * p.tscale, rB[h] * p.tscale) : pack2(rA[h], rB[h]);
      const uint64_t neg2 = kTs ? pack2(-sA[h] * p.tscale_inv, -sB[h] * p.tscale_inv) : pack2(-sA[h], -sB[h]);
#pragma unroll
      for (int g8 = 0; g8 < 2; ++g8) {
        float yA[8], yB[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint64_t x2 = bf16x2_to_f32x2(w[h * 16 + g8 * 8 + j]);
          if (kColsum) sum2 = add2(sum2, x2);
          unpack2(div_corrected2(x2, neg2, rcp2), yA[j], yB[j]);
        }
        uint32_t a8, b8;
        if (kSr == FP4T_SR_HASH) {
          // one index per (8 rows, column) group of the transposed tensor
          const uint32_t i0 = (uint32_t)((gr0 + h * 16 + g8 * 8) >> 3) * (uint32_t)p.cols + (uint32_t)gcA;
          uint32_t a1, b1;
          const uint32_t a0 = hash_pair(i0, seed_lo, seed_hi, a1);
          const uint32_t b0 = hash_pair(i0 + 1, seed_lo, seed_hi, b1);
          a8 = cvt_rs_e2m1x4(yA[0], yA[1], yA[2], yA[3], a0) | (cvt_rs_e2m1x4(yA[4], yA[5], yA[6], yA[7], a1) << 16);
          b8 = cvt_rs_e2m1x4(yB[0], yB[1], yB[2], yB[3], b0) | (cvt_rs_e2m1x4(yB[4], yB[5], yB[6], yB[7], b1) << 16);
        } else {
          if (kSr == FP4T_SR_NOISE) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int64_t gr = gr0 + h * 16 + g8 * 8 + j;
              yA[j] = sr_round(yA[j], okA ? __ldg(p.noise_t + gcA * p.rows + gr) : 0.5f);
              yB[j] = sr_round(yB[j], okB ? __ldg(p.noise_t + (gcA + 1) * p.rows + gr) : 0.5f);
            }
          }
          a8 = cvt_e2m1x8(yA[0], yA[1], yA[2], yA[3], yA[4], yA[5], yA[6], yA[7]);
          b8 = cvt_e2m1x8(yB[0], yB[1], yB[2], yB[3], yB[4], yB[5], yB[6], yB[7]);
        }
        outA[2 * h + g8] = a8;
        outB[2 * h + g8] = b8;
      }
      sfA[h] = e4m3_byte_of_scale(sA[h]);
      sfB[h] = e4m3_byte_of_scale(sB[h]);
    }
    if (okA)
      *reinterpret_cast<uint4*>(p.codes_t + gcA * (p.rows >> 1) + (gr0 >> 1)) =
          make_uint4(outA[0], outA[1], outA[2], outA[3]);
    if (okB)
      *reinterpret_cast<uint4*>(p.codes_t + (gcA + 1) * (p.rows >> 1) + (gr0 >> 1)) =
          make_uint4(outB[0], outB[1], outB[2], outB[3]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int kb = q * 2 + h;
      c.sf_col_s[(kb >> 2) * 512 + sf_tile_offset(2 * cp, kb)] = okA ? (uint8_t)sfA[h] : (uint8_t)0;
      c.sf_col_s[(kb >> 2) * 512 + sf_tile_offset(2 * cp + 1, kb)] = okB ? (uint8_t)sfB[h] : (uint8_t)0;
    }
  } else {
    float amA = 0.0f, amB = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      amA = fmaxf(amA, fmaxf(fabsf(__uint_as_float(w[j] << 16)), fabsf(__uint_as_float(w[j + 1] << 16))));
      amB = fmaxf(amB, fmaxf(fabsf(__uint_as_float(w[j] & 0xFFFF0000u)), fabsf(__uint_as_float(w[j + 1] & 0xFFFF0000u))));
    }
    const uint32_t sbA = mx_scale_byte(amA), sbB = mx_scale_byte(amB);
    const float invA = mx_inv_scale(sbA), invB = mx_inv_scale(sbB);
    uint32_t oA[8], oB[8];
#pragma unroll
    for (int g4 = 0; g4 < 8; ++g4) {
      uint32_t a = 0, b = 0;
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const uint32_t w0 = w[g4 * 4 + j], w1 = w[g4 * 4 + j + 1];
        if (kColsum) sum2 = add2(add2(sum2, bf16x2_to_f32x2(w0)), bf16x2_to_f32x2(w1));
        a |= mx_e4m3x2_from_bf16(fmaf(__uint_as_float(w0 << 16), invA, 0.0f),
                                 fmaf(__uint_as_float(w1 << 16), invA, 0.0f)) << (8 * j);
        b |= mx_e4m3x2_from_bf16(fmaf(__uint_as_float(w0 & 0xFFFF0000u), invB, 0.0f),
                                 fmaf(__uint_as_float(w1 & 0xFFFF0000u), invB, 0.0f)) << (8 * j);
      }
      oA[g4] = a;
      oB[g4] = b;
    }
    if (okA) {
      uint4* dst = reinterpret_cast<uint4*>(p.codes_t + gcA * p.rows + gr0);
      dst[0] = make_uint4(oA[0], oA[1], oA[2], oA[3]);
      dst[1] = make_uint4(oA[4], oA[5], oA[6], oA[7]);
    }
    if (okB) {
      uint4* dst = reinterpret_cast<uint4*>(p.codes_t + (gcA + 1) * p.rows + gr0);
      dst[0] = make_uint4(oB[0], oB[1], oB[2], oB[3]);
      dst[1] = make_uint4(oB[4], oB[5], oB[6], oB[7]);
    }
    c.sf_col_s[sf_tile_offset(2 * cp, q)] = okA ? (uint8_t)sbA : (uint8_t)0;
    c.sf_col_s[sf_tile_offset(2 * cp + 1, q)] = okB ? (uint8_t)sbB : (uint8_t)0;
  }
  if (kColsum) {
    float sa, sb;
    unpack2(sum2, sa, sb);
    *reinterpret_cast<float2*>(c.colsum_s + q * kTile + 2 * cp) = make_float2(sa, sb);
  }
}

// {next tile, CTAs done} per stream slot; zero between launches (the last CTA to run dry resets them)
__device__ unsigned int g_quant_sched[2 * kSchedSlots];

// GELU of eight bf16 values, as torch's CUDA kernel computes it for bf16 tensors: in fp32,
// x * 0.5 * (1 + erf(x * sqrt(1/2))), rounded to bf16.
__device__ __forceinline__ uint32_t gelu_bf16x2(uint32_t w) {
  const float a = __uint_as_float(w << 16), b = __uint_as_float(w & 0xFFFF0000u);
  const float ga = (a * 0.5f) * (1.0f + erff(a * 0.70710678118654752440f));
  const float gb = (b * 0.5f) * (1.0f + erff(b * 0.70710678118654752440f));
  const __nv_bfloat162 h = __floats2bfloat162_rn(ga, gb);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// kPre: 0 = quantize the input as it is; 1 = quantize GELU(input) (the activation is applied to
// the tile in shared memory, so its bf16 result never travels through HBM); 2 = quantize
// input x tensor scale (a power of two, folded into the block scale's operands).
template <int kFmt, int kSr, bool kColsum, int kPre = 0>
__global__ void __launch_bounds__(kQThreads, 2)
quantize_tma_kernel(const __grid_constant__ CUtensorMap map_x, const QParams p, const int tiles_x,
                    const int num_tiles, const int sched, int32_t* status) {
  using C = QCfg<kFmt>;
  extern __shared__ uint8_t q_smem_raw[];
  const uint32_t base = (smem_u32(q_smem_raw) + 127u) & ~127u;
  uint8_t* gen = q_smem_raw + (base - smem_u32(q_smem_raw));
  uint8_t* sf_stage = gen + kQStages * kQTileBytes;            // [2 buffers][row, col][kSfStage]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sf_stage + 4 * C::kSfStage);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kQStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kQStages);
  volatile int* tile_of_stage = abort_flag + 1;   // [kQStages] tile index the producer put into each stage (-1: no more)
  float2* scale_tab = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(bars) + 64);
  float* colsum_stage = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 64 + 1024);   // [2][4][128]

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  pdl_launch_dependents();
  if (tid == kQComputeThreads) tma_prefetch_map(&map_x);   // a kernel parameter: fetched under the set-up
  if (kFmt == kNvfp4 && tid < 128) scale_tab[tid] = make_float2(kScaleTable.v[tid].s, kScaleTable.v[tid].r);
  if (tid == 0) {
    for (int s = 0; s < kQStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, kQComputeThreads / 32);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();   // the input (and the tile counter) belong to the predecessor until it is complete

  const bool want_row = p.codes != nullptr;
  const bool want_col = p.codes_t != nullptr;
  // A launch replayed from a CUDA graph carries the seed it was captured with; the optional
  // device word (bumped by the host program between replays) makes every replay draw new noise.
  const uint64_t seed = (kSr == FP4T_SR_HASH && p.seed_dev != nullptr) ? p.seed + __ldg(p.seed_dev) * 0x9E3779B97F4A7C15ull : p.seed;

  if (warp == kQComputeThreads / 32) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      // Tiles come from the stream's device counter (a CTA that starts late, because its SM was
      // busy with another stream's kernel, takes fewer) or in the static round-robin order.
      int stage = 0;
      uint32_t phase = 0;
      for (uint32_t n = 0;; ++n) {
        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, status, 11)) break;
        int t;
        if (sched >= 0) {
          const unsigned int d = atomicAdd(&g_quant_sched[2 * sched], 1u);
          t = d < (unsigned int)num_tiles ? (int)d : -1;
        } else {
          const int64_t d = (int64_t)blockIdx.x + (int64_t)n * gridDim.x;
          t = d < num_tiles ? (int)d : -1;
        }
        tile_of_stage[stage] = t;
        if (t < 0) {
          mbar_arrive(bar_full + 8 * stage);   // publishes the end marker
          if (sched >= 0) {
            const unsigned int d = atomicAdd(&g_quant_sched[2 * sched + 1], 1u);
            if (d == gridDim.x - 1u) {
              atomicExch(&g_quant_sched[2 * sched], 0u);
              atomicExch(&g_quant_sched[2 * sched + 1], 0u);
            }
          }
          break;
        }
        const int ty = t / tiles_x, tx = t - ty * tiles_x;
        mbar_expect_tx(bar_full + 8 * stage, kQTileBytes);
        tma_load_2d(base + stage * kQTileBytes, &map_x, bar_full + 8 * stage, tx * kTile, ty * kTile);
        if (++stage == kQStages) { stage = 0; phase ^= 1u; }
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
      }
    }
    __syncwarp();
    return;
  }

  // ------------------------------ compute warps ------------------------------
  int stage = 0;
  uint32_t phase = 0;
  int buf = 0;
  for (;;) {
    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, status, 12)) break;
    const int t = tile_of_stage[stage];
    if (t < 0) break;
    const int ty = t / tiles_x, tx = t - ty * tiles_x;
    TileCtx c;
    c.row0 = (int64_t)ty * kTile;
    c.col0 = (int64_t)tx * kTile;
    c.tile = gen + stage * kQTileBytes;
    c.sf_row_s = sf_stage + buf * 2 * C::kSfStage;
    c.sf_col_s = c.sf_row_s + C::kSfStage;
    c.colsum_s = colsum_stage + buf * 4 * kTile;
    c.scale_tab = scale_tab;
    c.seed = seed;
    c.tid = tid;
    if (kPre == 1) {
      // 2048 16-byte vectors per tile, eight per thread; parts of the tile outside the tensor
      // were filled with zeros and GELU(0) = 0, so they stay zeros
      uint4* tile_v = reinterpret_cast<uint4*>(gen + stage * kQTileBytes);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint4 v = tile_v[tid + i * kQComputeThreads];
        v.x = gelu_bf16x2(v.x); v.y = gelu_bf16x2(v.y); v.z = gelu_bf16x2(v.z); v.w = gelu_bf16x2(v.w);
        tile_v[tid + i * kQComputeThreads] = v;
      }
      fence_async_smem();        // these writes are ordered before the TMA refill of the stage
      named_barrier_compute();
    }
    const bool interior = c.row0 + kTile <= p.rows && c.col0 + kTile <= p.cols;
    constexpr bool kTs = kPre == 2;
    if (interior) {
      if (want_row) row_pass<kFmt, kSr, false, kTs>(p, c);
      if (want_col) col_pass<kFmt, kSr, false, kColsum, kTs>(p, c);
    } else {
      if (want_row) row_pass<kFmt, kSr, true, kTs>(p, c);
      if (want_col) col_pass<kFmt, kSr, true, kColsum, kTs>(p, c);
    }

    // the tile is consumed: hand the stage back to the producer
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
    if (++stage == kQStages) { stage = 0; phase ^= 1u; }

    // ---- scale tiles out: whole 512-byte tiles, zero padding included --------------------
    named_barrier_compute();
    constexpr int kVecs = C::kSfChunks * 32;  // 16-byte vectors per staging buffer
    if (want_row && tid < kVecs) {
      const int chunk = tid >> 5;
      const int64_t stx = (int64_t)tx * C::kSfChunks + chunk;
      if (stx < p.ntx_row) {
        uint8_t* dst = p.sf + ((int64_t)ty * p.ntx_row + stx) * 512;
        reinterpret_cast<uint4*>(dst)[tid & 31] = reinterpret_cast<const uint4*>(c.sf_row_s)[tid];
      }
    }
    if (want_col && tid >= 64 && tid < 64 + kVecs) {
      const int u = tid - 64;
      const int chunk = u >> 5;
      const int64_t stx = (int64_t)ty * C::kSfChunks + chunk;
      if (stx < p.ntx_col) {
        uint8_t* dst = p.sf_t + ((int64_t)tx * p.ntx_col + stx) * 512;
        reinterpret_cast<uint4*>(dst)[u & 31] = reinterpret_cast<const uint4*>(c.sf_col_s)[u];
      }
    }
    if (kColsum && tid >= 128) {   // column sums of the tile: 4 row quarters -> one atomic per column
      const int col = tid - 128;
      if (c.col0 + col < p.cols) {
        const float* cs = c.colsum_s + col;
        atomicAdd(p.colsum + c.col0 + col, (cs[0] + cs[kTile]) + (cs[2 * kTile] + cs[3 * kTile]));
      }
    }
    buf ^= 1;
  }
}

// ---------------------------------------------------------------------------------------
// Generic path: any input dtype / alignment, one thread per block of kBlk elements.
// `transposed` quantizes x^T (blocks run along the row axis of x).
// ---------------------------------------------------------------------------------------
template <int kFmt, typename TIn>
__global__ void quantize_generic_kernel(const QParams p, const int transposed, const int sr) {
  constexpr int kBlk = kFmt == kNvfp4 ? 16 : 32;
  // logical output matrix [outer, inner]
  const int64_t outer = transposed ? p.cols : p.rows;
  const int64_t inner = transposed ? p.rows : p.cols;
  const int64_t kblocks = inner / kBlk;
  const int64_t total = outer * kblocks;
  const TIn* __restrict__ x = static_cast<const TIn*>(p.x);
  uint8_t* codes = transposed ? p.codes_t : p.codes;
  uint8_t* sf = transposed ? p.sf_t : p.sf;
  const float* noise = transposed ? p.noise_t : p.noise;
  const int64_t ntx = transposed ? p.ntx_col : p.ntx_row;
  const uint64_t seed0 = (sr == FP4T_SR_HASH && p.seed_dev != nullptr) ? p.seed + __ldg(p.seed_dev) * 0x9E3779B97F4A7C15ull : p.seed;
  for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < total;
       b += (int64_t)gridDim.x * blockDim.x) {
    const int64_t o = b / kblocks, kb = b % kblocks;
    float f[kBlk];
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < kBlk; ++j) {
      const int64_t i = kb * kBlk + j;
      const int64_t idx = transposed ? i * p.ld + o : o * p.ld + i;
      f[j] = (float)x[idx] * p.tscale;
    }
    if (kFmt == kNvfp4 && (p.rht_signs & 0x10000u)) {
      // random Hadamard transform of the block: signs, then the 16-point fast Walsh-Hadamard
      // butterflies (strides 1, 2, 4, 8), then 1/4 -- an orthogonal map, so two operands
      // transformed with the same signs keep their dot products
#pragma unroll
      for (int j = 0; j < kBlk; ++j) f[j] = ((p.rht_signs >> (j & 15)) & 1u) ? -f[j] : f[j];
#pragma unroll
      for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if ((j & h) == 0) {
            const float a = f[j], b = f[j + h];
            f[j] = __fadd_rn(a, b);
            f[j + h] = __fsub_rn(a, b);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < kBlk; ++j) f[j] *= 0.25f;
    }
#pragma unroll
    for (int j = 0; j < kBlk; ++j) amax = fmaxf(amax, fabsf(f[j]));
    if (kFmt == kNvfp4) {
      const float s = nvfp4_scale(amax);
      uint32_t word = 0;
#pragma unroll
      for (int j = 0; j < kBlk; j += 2) {
        float y0 = __fdiv_rn(f[j], s), y1 = __fdiv_rn(f[j + 1], s);
        if (sr != FP4T_SR_NONE) {
          const int64_t e = o * inner + kb * kBlk + j;
          const uint64_t seed = transposed ? (seed0 ^ 0x5bd1e995c2b2ae35ull) : seed0;
          const float u0 = sr == FP4T_SR_NOISE ? noise[e] : hash_uniform(seed, (uint64_t)e);
          const float u1 = sr == FP4T_SR_NOISE ? noise[e + 1] : hash_uniform(seed, (uint64_t)(e + 1));
          y0 = sr_round(y0, u0);
          y1 = sr_round(y1, u1);
        } else {
          y0 = y0 == 0.0f ? 0.0f : y0;  // sign(+-0) is 0
          y1 = y1 == 0.0f ? 0.0f : y1;
        }
        const uint32_t byte = cvt_e2m1x2(y0, y1);
        codes[o * (inner >> 1) + ((kb * kBlk + j) >> 1)] = (uint8_t)byte;
        (void)word;
      }
      sf[sf_offset(o, kb, ntx)] = (uint8_t)cvt_e4m3(s);
    } else {
      const uint32_t sb = mx_scale_byte(amax);
      const float inv = mx_inv_scale(sb);
#pragma unroll
      for (int j = 0; j < kBlk; ++j) {
        codes[o * inner + kb * kBlk + j] = (uint8_t)mx_e4m3_byte<true>(f[j] * inv);
      }
      sf[sf_offset(o, kb, ntx)] = (uint8_t)sb;
    }
  }
}

template <int kFmt>
int launch_generic(const QParams& p, int x_dtype, int sr, cudaStream_t stream) {
  constexpr int kBlk = kFmt == kNvfp4 ? 16 : 32;
  for (int t = 0; t < 2; ++t) {
    uint8_t* codes = t ? p.codes_t : p.codes;
    if (!codes) continue;
    const int64_t outer = t ? p.cols : p.rows, inner = t ? p.rows : p.cols;
    uint8_t* sf = t ? p.sf_t : p.sf;
    FP4T_CUDA(cudaMemsetAsync(sf, 0, (size_t)fp4t_sf_bytes(outer, inner / kBlk), stream));
    const int64_t total = outer * (inner / kBlk);
    if (total == 0) continue;
    const int threads = 128;
    const int64_t blocks = ceil_div(total, threads);
    const int grid = (int)(blocks > 148 * 64 ? 148 * 64 : blocks);
    if (x_dtype == FP4T_DT_BF16) {
      quantize_generic_kernel<kFmt, __nv_bfloat16><<<grid, threads, 0, stream>>>(p, t, sr);
    } else {
      quantize_generic_kernel<kFmt, float><<<grid, threads, 0, stream>>>(p, t, sr);
    }
  }
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}

// Column sums of x [rows, cols] added into an fp32 accumulator: one thread per column.
template <typename TIn>
__global__ void colsum_generic_kernel(const TIn* __restrict__ x, int64_t rows, int64_t cols, int64_t ld,
                                      float* __restrict__ colsum) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float acc = 0.0f;
  for (int64_t r = 0; r < rows; ++r) acc += (float)x[r * ld + c];
  colsum[c] += acc;
}

// Zeroes the column-sum scratch.  A kernel rather than a memset so that it sits in the chain of
// dependent launches: a memset between two kernels makes the second wait for a full stream
// serialisation instead of starting under the first one's tail.
__global__ void zero_f32_kernel(float* __restrict__ p, int64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = 0.0f;
}

// fp32 accumulator -> bias gradient in the caller's dtype.
__global__ void colsum_finalize_kernel(const float* __restrict__ colsum, void* __restrict__ out, int out_f32,
                                       int64_t cols) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  if (out_f32) static_cast<float*>(out)[c] = colsum[c];
  else static_cast<__nv_bfloat16*>(out)[c] = __float2bfloat16_rn(colsum[c]);
}

// Argument checks of the quantizer entry points (no launch).  `name` is the entry point the
// caller used, so that messages name it.
template <int kFmt>
int quantize_check(const char* name, const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                   const void* codes, const void* sf, const void* codes_t, const void* sf_t, int sr_mode,
                   const float* noise, const float* noise_t) {
  constexpr int kBlk = kFmt == kNvfp4 ? 16 : 32;
  FP4T_REQUIRE(x != nullptr, "%s: x is null", name);
  FP4T_REQUIRE(x_dtype == FP4T_DT_BF16 || x_dtype == FP4T_DT_F32, "%s: x_dtype must be bf16 or f32", name);
  FP4T_REQUIRE(rows >= 0 && cols >= 0 && ld >= cols, "%s: bad shape rows=%lld cols=%lld ld=%lld", name,
               (long long)rows, (long long)cols, (long long)ld);
  FP4T_REQUIRE(codes != nullptr || codes_t != nullptr, "%s: no output requested", name);
  FP4T_REQUIRE((codes == nullptr) == (sf == nullptr), "%s: codes and sf must be given together", name);
  FP4T_REQUIRE((codes_t == nullptr) == (sf_t == nullptr), "%s: codes_t and sf_t must be given together", name);
  if (codes) FP4T_REQUIRE(cols % kBlk == 0, "%s: row-wise output needs cols %% %d == 0 (cols=%lld)", name, kBlk, (long long)cols);
  if (codes_t) FP4T_REQUIRE(rows % 32 == 0, "%s: transposed output needs rows %% 32 == 0 (rows=%lld)", name, (long long)rows);
  FP4T_REQUIRE(sr_mode >= FP4T_SR_NONE && sr_mode <= FP4T_SR_HASH, "%s: bad sr_mode %d", name, sr_mode);
  if (sr_mode == FP4T_SR_NOISE) {
    FP4T_REQUIRE((codes == nullptr || noise != nullptr) && (codes_t == nullptr || noise_t != nullptr),
                 "%s: sr_mode NOISE needs a noise tensor for every requested output", name);
  }
  return FP4T_OK;
}

template <int kFmt>
int quantize_dispatch(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                      void* codes, void* sf, void* codes_t, void* sf_t, int sr_mode,
                      const float* noise, const float* noise_t, uint64_t seed, float* colsum,
                      cudaStream_t stream, const char* name = nullptr, int pre_op = 0, float tscale = 1.0f,
                      uint32_t rht_signs = 0) {
  constexpr int kBlk = kFmt == kNvfp4 ? 16 : 32;
  if (name == nullptr) name = kFmt == kNvfp4 ? "fp4t_quantize_nvfp4" : "fp4t_quantize_mxfp8";
  {
    const int rc = quantize_check<kFmt>(name, x, x_dtype, rows, cols, ld, codes, sf, codes_t, sf_t, sr_mode, noise, noise_t);
    if (rc != FP4T_OK) return rc;
  }
  if (rows == 0 || cols == 0) return FP4T_OK;

  QParams p;
  p.x = x; p.rows = rows; p.cols = cols; p.ld = ld;
  p.codes = static_cast<uint8_t*>(codes); p.sf = static_cast<uint8_t*>(sf);
  p.codes_t = static_cast<uint8_t*>(codes_t); p.sf_t = static_cast<uint8_t*>(sf_t);
  p.noise = noise; p.noise_t = noise_t; p.seed = seed; p.seed_dev = seed_offset_word(); p.colsum = colsum;
  p.tscale = tscale; p.tscale_inv = 1.0f / tscale; p.rht_signs = rht_signs;
  const bool options = tscale != 1.0f || rht_signs != 0;
  const bool options_ok = !options || (kFmt == kNvfp4 && tscale > 0.0f && tscale < 3.0e38f);
  FP4T_REQUIRE(options_ok, "%s: tensor_scale (NVFP4 only) must be positive and finite", name);
  int mant_exp = 0;
  const bool pow2 = frexpf(tscale, &mant_exp) == 0.5f;
  p.ntx_row = (int)ceil_div(ceil_div(cols, kBlk), 4);
  p.ntx_col = (int)ceil_div(ceil_div(rows, kBlk), 4);

  // the tiled kernel's exact-division shortcut holds for bf16 inputs times a power of two; any
  // other tensor scale, and the Hadamard transform, take the general kernel
  const bool fast = x_dtype == FP4T_DT_BF16 && pow2 && rht_signs == 0 && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                    (ld % 8 == 0) && (cols % 8 == 0) &&
                    (codes == nullptr || reinterpret_cast<uintptr_t>(codes) % 16 == 0) &&
                    (codes_t == nullptr || reinterpret_cast<uintptr_t>(codes_t) % 16 == 0) &&
                    (sf == nullptr || reinterpret_cast<uintptr_t>(sf) % 16 == 0) &&
                    (sf_t == nullptr || reinterpret_cast<uintptr_t>(sf_t) % 16 == 0);
  if (pre_op != 0 && (!fast || colsum != nullptr || sr_mode != FP4T_SR_NONE)) {
    set_error("%s: the fused activation needs bf16 input with 16-byte aligned rows and outputs, round-to-nearest", name);
    return FP4T_ERR_UNSUPPORTED;
  }
  if (!fast || (colsum != nullptr && codes_t == nullptr)) {
    // column sums ride on the transposed pass of the tiled kernel; otherwise a plain kernel adds them
    if (colsum != nullptr) {
      const int threads = 256;
      const int64_t blocks = ceil_div(cols, threads);
      if (x_dtype == FP4T_DT_BF16)
        colsum_generic_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(x), rows, cols, ld, colsum);
      else
        colsum_generic_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>(static_cast<const float*>(x), rows,
                                                                                cols, ld, colsum);
      p.colsum = nullptr;
    }
    if (!fast) return launch_generic<kFmt>(p, x_dtype, sr_mode, stream);
  }

  const int sms = sm_count();
  if (sms < 0) {
    set_error("%s: the current device is not an sm_100 part", name);
    return FP4T_ERR_DEVICE;
  }
  const int64_t tiles_x = ceil_div(cols, kTile), tiles_y = ceil_div(rows, kTile);
  FP4T_REQUIRE(tiles_x * tiles_y < (1ll << 31), "%s: tensor too large for one launch", name);
  const int num_tiles = (int)(tiles_x * tiles_y);
  CUtensorMap map_x;
  const int rc = encode_tensor_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, (uint64_t)cols, (uint64_t)rows,
                                      (uint64_t)ld * 2, kTile, kTile, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != FP4T_OK) return rc;
  const int grid = num_tiles < 2 * sms ? num_tiles : 2 * sms;
  int32_t* status = current_status_word();
  const int sched = sched_slot_for(stream);
#define FP4T_LAUNCH_Q2(FMT, SR, CS) FP4T_LAUNCH_Q3(FMT, SR, CS, 0)
#define FP4T_LAUNCH_Q3(FMT, SR, CS, PRE)                                                                   \
  do {                                                                                                     \
    auto kern = quantize_tma_kernel<FMT, SR, CS, PRE>;                                                     \
    FP4T_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, QCfg<FMT>::kSmemBytes)); \
    cudaLaunchConfig_t cfg = {};                                                                           \
    cfg.gridDim = dim3((unsigned)grid, 1, 1);                                                              \
    cfg.blockDim = dim3(kQThreads, 1, 1);                                                                  \
    cfg.dynamicSmemBytes = QCfg<FMT>::kSmemBytes;                                                          \
    cfg.stream = stream;                                                                                   \
    cudaLaunchAttribute attr;                                                                              \
    pdl_attribute(&attr);                                                                                  \
    cfg.attrs = &attr;                                                                                     \
    cfg.numAttrs = 1;                                                                                      \
    FP4T_CUDA(cudaLaunchKernelEx(&cfg, kern, map_x, p, (int)tiles_x, num_tiles, sched, status));           \
  } while (0)
#define FP4T_LAUNCH_Q(FMT, SR)                  \
  do {                                          \
    if (p.colsum != nullptr) FP4T_LAUNCH_Q2(FMT, SR, true); \
    else FP4T_LAUNCH_Q2(FMT, SR, false);        \
  } while (0)
  if (pre_op == 1) {
    if (kFmt == kMxfp8) FP4T_LAUNCH_Q3(kMxfp8, FP4T_SR_NONE, false, 1);
    else FP4T_LAUNCH_Q3(kNvfp4, FP4T_SR_NONE, false, 1);
  } else if (kFmt == kNvfp4 && tscale != 1.0f) {
    if (sr_mode == FP4T_SR_NOISE) {
      set_error("%s: a tensor scale combines with round-to-nearest or in-kernel stochastic rounding", name);
      return FP4T_ERR_UNSUPPORTED;
    }
    if (sr_mode == FP4T_SR_NONE) {
      if (p.colsum != nullptr) FP4T_LAUNCH_Q3(kNvfp4, FP4T_SR_NONE, true, 2);
      else FP4T_LAUNCH_Q3(kNvfp4, FP4T_SR_NONE, false, 2);
    } else {
      if (p.colsum != nullptr) FP4T_LAUNCH_Q3(kNvfp4, FP4T_SR_HASH, true, 2);
      else FP4T_LAUNCH_Q3(kNvfp4, FP4T_SR_HASH, false, 2);
    }
  } else if (kFmt == kMxfp8) {
    FP4T_LAUNCH_Q(kMxfp8, FP4T_SR_NONE);
  } else if (sr_mode == FP4T_SR_NONE) {
    FP4T_LAUNCH_Q(kNvfp4, FP4T_SR_NONE);
  } else if (sr_mode == FP4T_SR_NOISE) {
    FP4T_LAUNCH_Q(kNvfp4, FP4T_SR_NOISE);
  } else {
    FP4T_LAUNCH_Q(kNvfp4, FP4T_SR_HASH);
  }
#undef FP4T_LAUNCH_Q
#undef FP4T_LAUNCH_Q2
#undef FP4T_LAUNCH_Q3
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}

template <int kFmt>
int quantize_bgrad(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, void* codes, void* sf,
                   void* codes_t, void* sf_t, int sr_mode, const float* noise, const float* noise_t, uint64_t seed,
                   float* colsum_scratch, void* bias_grad, int bias_grad_dtype, cudaStream_t stream,
                   const char* name = nullptr) {
  if (name == nullptr) name = kFmt == kNvfp4 ? "fp4t_quantize_nvfp4_bgrad" : "fp4t_quantize_mxfp8_bgrad";
  FP4T_REQUIRE(colsum_scratch != nullptr && bias_grad != nullptr, "%s: scratch and bias_grad must be given", name);
  FP4T_REQUIRE(reinterpret_cast<uintptr_t>(colsum_scratch) % 4 == 0, "%s: scratch must be 4-byte aligned", name);
  FP4T_REQUIRE(bias_grad_dtype == FP4T_DT_BF16 || bias_grad_dtype == FP4T_DT_F32, "%s: bad bias_grad dtype", name);
  {   // every argument is checked before the first kernel is enqueued
    const int rc = quantize_check<kFmt>(name, x, x_dtype, rows, cols, ld, codes, sf, codes_t, sf_t, sr_mode, noise, noise_t);
    if (rc != FP4T_OK) return rc;
  }
  if (cols == 0) return FP4T_OK;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ceil_div(cols, 256), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    pdl_attribute(&attr);
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    FP4T_CUDA(cudaLaunchKernelEx(&cfg, zero_f32_kernel, colsum_scratch, cols));
  }
  if (rows > 0) {
    const int rc = quantize_dispatch<kFmt>(x, x_dtype, rows, cols, ld, codes, sf, codes_t, sf_t, sr_mode, noise,
                                           noise_t, seed, colsum_scratch, stream, name);
    if (rc != FP4T_OK) return rc;
  }
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ceil_div(cols, 256), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    pdl_attribute(&attr);
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    FP4T_CUDA(cudaLaunchKernelEx(&cfg, colsum_finalize_kernel, static_cast<const float*>(colsum_scratch), bias_grad,
                                 (int)(bias_grad_dtype == FP4T_DT_F32), cols));
  }
  return FP4T_OK;
}

}  // namespace

FP4T_DEFINE_WAIT_TIMEOUT_SETTER(set_wait_timeout_quantize)

int reset_quantize_tile_counters(cudaStream_t stream) {
  void* addr = nullptr;
  FP4T_CUDA(cudaGetSymbolAddress(&addr, g_quant_sched));
  FP4T_CUDA(cudaMemsetAsync(addr, 0, sizeof(unsigned int) * 2 * kSchedSlots, stream));
  return FP4T_OK;
}
}  // namespace fp4t

extern "C" int fp4t_quantize_nvfp4_bgrad(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                         void* codes, void* sf, void* codes_t, void* sf_t, int sr_mode,
                                         const float* noise, const float* noise_t, uint64_t seed,
                                         float* colsum_scratch, void* bias_grad, int bias_grad_dtype,
                                         fp4t_stream_t stream) {
  return fp4t::quantize_bgrad<fp4t::kNvfp4>(x, x_dtype, rows, cols, ld, codes, sf, codes_t, sf_t, sr_mode, noise,
                                            noise_t, seed, colsum_scratch, bias_grad, bias_grad_dtype,
                                            reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int fp4t_quantize_mxfp8_bgrad(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                         void* codes, void* sf, void* codes_t, void* sf_t,
                                         float* colsum_scratch, void* bias_grad, int bias_grad_dtype,
                                         fp4t_stream_t stream) {
  return fp4t::quantize_bgrad<fp4t::kMxfp8>(x, x_dtype, rows, cols, ld, codes, sf, codes_t, sf_t, FP4T_SR_NONE,
                                            nullptr, nullptr, 0, colsum_scratch, bias_grad, bias_grad_dtype,
                                            reinterpret_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------
// Allocation-free variant of fp4t_quantize_nvfp4_bgrad: the fp32 column-sum scratch lives in
// this file-scope device array instead of caller memory.  Every GPU that loads the library
// carries the array (64 KiB) until the process exits.
// ---------------------------------------------------------------------------------------
static __device__ __align__(256) float g_static_colsum[FP4T_STATIC_BGRAD_MAX_COLS];

namespace fp4t {
namespace {
// In host code `g_static_colsum` is only a handle for the runtime; the address kernels and
// memsets must be given is looked up once per device, with that device current.
int static_colsum_address(float** out) {
  static std::mutex mu;
  static float* addr[64] = {nullptr};
  int dev = 0;
  FP4T_CUDA(cudaGetDevice(&dev));
  FP4T_REQUIRE(dev >= 0 && dev < 64, "fp4t_quantize_nvfp4_bgrad_static: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    FP4T_CUDA(cudaGetSymbolAddress(&p, g_static_colsum));
    addr[dev] = static_cast<float*>(p);
  }
  *out = addr[dev];
  return FP4T_OK;
}
}  // namespace
}  // namespace fp4t

extern "C" int fp4t_quantize_nvfp4_bgrad_static(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                                void* codes, void* sf, void* codes_t, void* sf_t, int sr_mode,
                                                const float* noise, const float* noise_t, uint64_t seed,
                                                void* bias_grad, int bias_grad_dtype, fp4t_stream_t stream) {
  FP4T_REQUIRE(cols <= FP4T_STATIC_BGRAD_MAX_COLS,
               "fp4t_quantize_nvfp4_bgrad_static: cols=%lld exceeds the built-in scratch of %d columns; "
               "use fp4t_quantize_nvfp4_bgrad with caller scratch",
               (long long)cols, (int)FP4T_STATIC_BGRAD_MAX_COLS);
  float* scratch = nullptr;
  const int rc = fp4t::static_colsum_address(&scratch);
  if (rc != FP4T_OK) return rc;
  return fp4t::quantize_bgrad<fp4t::kNvfp4>(x, x_dtype, rows, cols, ld, codes, sf, codes_t, sf_t, sr_mode, noise,
                                            noise_t, seed, scratch, bias_grad, bias_grad_dtype,
                                            reinterpret_cast<cudaStream_t>(stream), "fp4t_quantize_nvfp4_bgrad_static");
}

extern "C" int fp4t_quantize_nvfp4(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                   void* codes, void* sf, void* codes_t, void* sf_t, int sr_mode,
                                   const float* noise, const float* noise_t, uint64_t seed,
                                   fp4t_stream_t stream) {
  return fp4t::quantize_dispatch<fp4t::kNvfp4>(x, x_dtype, rows, cols, ld, codes, sf, codes_t, sf_t,
                                               sr_mode, noise, noise_t, seed, nullptr,
                                               reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int fp4t_quantize_mxfp8(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                   void* codes, void* sf, void* codes_t, void* sf_t,
                                   fp4t_stream_t stream) {
  return fp4t::quantize_dispatch<fp4t::kMxfp8>(x, x_dtype, rows, cols, ld, codes, sf, codes_t, sf_t,
                                               FP4T_SR_NONE, nullptr, nullptr, 0, nullptr,
                                               reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int fp4t_quantize_nvfp4_gelu(const void* x_bf16, int64_t rows, int64_t cols, int64_t ld, void* codes, void* sf,
                                        void* codes_t, void* sf_t, fp4t_stream_t stream) {
  return fp4t::quantize_dispatch<fp4t::kNvfp4>(x_bf16, FP4T_DT_BF16, rows, cols, ld, codes, sf, codes_t, sf_t, FP4T_SR_NONE,
                                               nullptr, nullptr, 0, nullptr, reinterpret_cast<cudaStream_t>(stream),
                                               "fp4t_quantize_nvfp4_gelu", 1);
}

extern "C" int fp4t_quantize_mxfp8_gelu(const void* x_bf16, int64_t rows, int64_t cols, int64_t ld, void* codes, void* sf,
                                        void* codes_t, void* sf_t, fp4t_stream_t stream) {
  return fp4t::quantize_dispatch<fp4t::kMxfp8>(x_bf16, FP4T_DT_BF16, rows, cols, ld, codes, sf, codes_t, sf_t, FP4T_SR_NONE,
                                               nullptr, nullptr, 0, nullptr, reinterpret_cast<cudaStream_t>(stream),
                                               "fp4t_quantize_mxfp8_gelu", 1);
}

extern "C" int fp4t_quantize_nvfp4_scaled(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, void* codes,
                                          void* sf, void* codes_t, void* sf_t, int sr_mode, uint64_t seed,
                                          float tensor_scale, fp4t_stream_t stream) {
  return fp4t::quantize_dispatch<fp4t::kNvfp4>(x, x_dtype, rows, cols, ld, codes, sf, codes_t, sf_t, sr_mode, nullptr,
                                               nullptr, seed, nullptr, reinterpret_cast<cudaStream_t>(stream),
                                               "fp4t_quantize_nvfp4_scaled", 0, tensor_scale, 0);
}

extern "C" int fp4t_quantize_nvfp4_rht(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, void* codes,
                                       void* sf, void* codes_t, void* sf_t, uint32_t sign_mask, float tensor_scale,
                                       fp4t_stream_t stream) {
  if (codes_t != nullptr && rows % 16 != 0) {
    fp4t::set_error("fp4t_quantize_nvfp4_rht: the transposed output needs rows %% 16 == 0");
    return FP4T_ERR_ARG;
  }
  return fp4t::quantize_dispatch<fp4t::kNvfp4>(x, x_dtype, rows, cols, ld, codes, sf, codes_t, sf_t, FP4T_SR_NONE, nullptr,
                                               nullptr, 0, nullptr, reinterpret_cast<cudaStream_t>(stream),
                                               "fp4t_quantize_nvfp4_rht", 0, tensor_scale, (sign_mask & 0xFFFFu) | 0x10000u);
}
