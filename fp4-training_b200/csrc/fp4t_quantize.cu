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
  uint64_t seed;
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
//   row pass   lane pairs (NVFP4) / quads (MXFP8) own one block of a row; amax by shuffle;
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
  static constexpr int kSmemBytes = kQStages * kQTileBytes + 4 * kSfStage + 64 + 128 + 1024;
};

__device__ __forceinline__ void named_barrier_compute() {
  asm volatile("bar.sync 1, %0;" ::"n"(kQComputeThreads) : "memory");
}

template <int kFmt, int kSr>
__global__ void __launch_bounds__(kQThreads, 2)
quantize_tma_kernel(const __grid_constant__ CUtensorMap map_x, const QParams p, const int tiles_x,
                    const int num_tiles, int32_t* status) {
  using C = QCfg<kFmt>;
  extern __shared__ uint8_t q_smem_raw[];
  const uint32_t base = (smem_u32(q_smem_raw) + 127u) & ~127u;
  uint8_t* gen = q_smem_raw + (base - smem_u32(q_smem_raw));
  uint8_t* sf_stage = gen + kQStages * kQTileBytes;            // [2 buffers][row, col][kSfStage]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sf_stage + 4 * C::kSfStage);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kQStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kQStages);
  float2* scale_tab = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(bars) + 64);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
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

  const bool want_row = p.codes != nullptr;
  const bool want_col = p.codes_t != nullptr;

  if (warp == kQComputeThreads / 32) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, status, 11)) break;
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
  for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const int ty = t / tiles_x, tx = t - ty * tiles_x;
    const int64_t row0 = (int64_t)ty * kTile, col0 = (int64_t)tx * kTile;
    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, status, 12)) break;
    const uint8_t* tile = gen + stage * kQTileBytes;
    uint8_t* sf_row_s = sf_stage + buf * 2 * C::kSfStage;
    uint8_t* sf_col_s = sf_row_s + C::kSfStage;

    // ---- row-wise pass: thread handles 8 elements of a row, 8 times -------------------
    if (want_row) {
#pragma unroll 2
      for (int it = 0; it < 8; ++it) {
        const int vi = it * kQComputeThreads + tid;
        const int r = vi >> 4, cv = vi & 15;
        const int64_t gr = row0 + r, gc = col0 + cv * 8;
        const uint4 v = *reinterpret_cast<const uint4*>(tile + r * 256 + cv * 16);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          amax = fmaxf(amax, fabsf(__uint_as_float(w[j] << 16)));
          amax = fmaxf(amax, fabsf(__uint_as_float(w[j] & 0xFFFF0000u)));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
        if (kFmt == kMxfp8) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
        const bool valid = gr < p.rows && gc < p.cols;
        const int kb = (cv * 8) / C::kBlk;
        if (kFmt == kNvfp4) {
          float s, rcp;
          nvfp4_scale_from_table(scale_tab, amax, s, rcp);
          const uint64_t rcp2 = pack2(rcp, rcp), neg2 = pack2(-s, -s);
          float y[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) unpack2(div_corrected2(bf16x2_to_f32x2(w[j]), neg2, rcp2), y[2 * j], y[2 * j + 1]);
          if (kSr == FP4T_SR_NOISE) {
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = sr_round(y[j], valid ? __ldg(p.noise + gr * p.cols + gc + j) : 0.5f);
          } else if (kSr == FP4T_SR_HASH) {
            const uint32_t e0 = (uint32_t)((gr * p.cols + gc) >> 1);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t h = mix32((e0 + j) * 0x9E3779B9u + (uint32_t)p.seed) ^ (uint32_t)(p.seed >> 32);
              y[2 * j] = sr_round_bits(y[2 * j], h & 0xFFFFu);
              y[2 * j + 1] = sr_round_bits(y[2 * j + 1], h >> 16);
            }
          }
          const uint32_t packed = cvt_e2m1x8(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7]);
          if (valid) *reinterpret_cast<uint32_t*>(p.codes + gr * (p.cols >> 1) + (gc >> 1)) = packed;
          if ((cv & 1) == 0)
            sf_row_s[(kb >> 2) * 512 + sf_tile_offset(r, kb)] = valid ? (uint8_t)e4m3_byte_of_scale(s) : (uint8_t)0;
        } else {
          const uint32_t sb = mx_scale_byte(amax);
          const float inv = mx_inv_scale(sb);
          uint32_t o[2] = {0u, 0u};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float y0 = fmaf(__uint_as_float(w[j] << 16), inv, 0.0f);
            const float y1 = fmaf(__uint_as_float(w[j] & 0xFFFF0000u), inv, 0.0f);
            o[j >> 1] |= mx_e4m3x2_from_bf16(y0, y1) << (16 * (j & 1));
          }
          if (valid) *reinterpret_cast<uint2*>(p.codes + gr * p.cols + gc) = make_uint2(o[0], o[1]);
          if ((cv & 3) == 0) sf_row_s[sf_tile_offset(r, kb)] = valid ? (uint8_t)sb : (uint8_t)0;
        }
      }
    }

    // ---- transposed pass: thread handles 2 adjacent columns x 32 rows --------------------
    if (want_col) {
      const int cp = tid & 63, q = tid >> 6;
      const int64_t gr0 = row0 + q * 32, gcA = col0 + 2 * cp;
      const bool rows_ok = gr0 < p.rows;             // rows % 32 == 0: all 32 rows in or out
      const bool okA = rows_ok && gcA < p.cols, okB = rows_ok && gcA + 1 < p.cols;
      const uint32_t* col_words = reinterpret_cast<const uint32_t*>(tile + (q * 32) * 256) + cp;
      if (kFmt == kNvfp4) {
        uint32_t outA[4], outB[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) w[j] = col_words[(h * 16 + j) * 64];
          float amA = 0.0f, amB = 0.0f;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            amA = fmaxf(amA, fabsf(__uint_as_float(w[j] << 16)));
            amB = fmaxf(amB, fabsf(__uint_as_float(w[j] & 0xFFFF0000u)));
          }
          float sA, sB, rA, rB;
          nvfp4_scale_from_table(scale_tab, amA, sA, rA);
          nvfp4_scale_from_table(scale_tab, amB, sB, rB);
          const uint64_t rcp2 = pack2(rA, rB), neg2 = pack2(-sA, -sB);
          float yA[16], yB[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) unpack2(div_corrected2(bf16x2_to_f32x2(w[j]), neg2, rcp2), yA[j], yB[j]);
          if (kSr == FP4T_SR_NOISE) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int64_t gr = gr0 + h * 16 + j;
              yA[j] = sr_round(yA[j], okA ? __ldg(p.noise_t + gcA * p.rows + gr) : 0.5f);
              yB[j] = sr_round(yB[j], okB ? __ldg(p.noise_t + (gcA + 1) * p.rows + gr) : 0.5f);
            }
          } else if (kSr == FP4T_SR_HASH) {
            const uint32_t seed_lo = (uint32_t)p.seed ^ 0x5BD1E995u, seed_hi = (uint32_t)(p.seed >> 32);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const uint32_t e = (uint32_t)((gr0 + h * 16 + j) * (p.cols >> 1) + (gcA >> 1));
              const uint32_t hsh = mix32(e * 0x9E3779B9u + seed_lo) ^ seed_hi;
              yA[j] = sr_round_bits(yA[j], hsh & 0xFFFFu);
              yB[j] = sr_round_bits(yB[j], hsh >> 16);
            }
          }
          outA[2 * h] = cvt_e2m1x8(yA[0], yA[1], yA[2], yA[3], yA[4], yA[5], yA[6], yA[7]);
          outA[2 * h + 1] = cvt_e2m1x8(yA[8], yA[9], yA[10], yA[11], yA[12], yA[13], yA[14], yA[15]);
          outB[2 * h] = cvt_e2m1x8(yB[0], yB[1], yB[2], yB[3], yB[4], yB[5], yB[6], yB[7]);
          outB[2 * h + 1] = cvt_e2m1x8(yB[8], yB[9], yB[10], yB[11], yB[12], yB[13], yB[14], yB[15]);
          const int kb = q * 2 + h;
          sf_col_s[(kb >> 2) * 512 + sf_tile_offset(2 * cp, kb)] = okA ? (uint8_t)e4m3_byte_of_scale(sA) : (uint8_t)0;
          sf_col_s[(kb >> 2) * 512 + sf_tile_offset(2 * cp + 1, kb)] = okB ? (uint8_t)e4m3_byte_of_scale(sB) : (uint8_t)0;
        }
        if (okA)
          *reinterpret_cast<uint4*>(p.codes_t + gcA * (p.rows >> 1) + (gr0 >> 1)) =
              make_uint4(outA[0], outA[1], outA[2], outA[3]);
        if (okB)
          *reinterpret_cast<uint4*>(p.codes_t + (gcA + 1) * (p.rows >> 1) + (gr0 >> 1)) =
              make_uint4(outB[0], outB[1], outB[2], outB[3]);
      } else {
        uint32_t w[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = col_words[j * 64];
        float amA = 0.0f, amB = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          amA = fmaxf(amA, fabsf(__uint_as_float(w[j] << 16)));
          amB = fmaxf(amB, fabsf(__uint_as_float(w[j] & 0xFFFF0000u)));
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
        sf_col_s[sf_tile_offset(2 * cp, q)] = okA ? (uint8_t)sbA : (uint8_t)0;
        sf_col_s[sf_tile_offset(2 * cp + 1, q)] = okB ? (uint8_t)sbB : (uint8_t)0;
      }
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
        reinterpret_cast<uint4*>(dst)[tid & 31] = reinterpret_cast<const uint4*>(sf_row_s)[tid];
      }
    }
    if (want_col && tid >= 64 && tid < 64 + kVecs) {
      const int u = tid - 64;
      const int chunk = u >> 5;
      const int64_t stx = (int64_t)ty * C::kSfChunks + chunk;
      if (stx < p.ntx_col) {
        uint8_t* dst = p.sf_t + ((int64_t)tx * p.ntx_col + stx) * 512;
        reinterpret_cast<uint4*>(dst)[u & 31] = reinterpret_cast<const uint4*>(sf_col_s)[u];
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
  for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < total;
       b += (int64_t)gridDim.x * blockDim.x) {
    const int64_t o = b / kblocks, kb = b % kblocks;
    float f[kBlk];
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < kBlk; ++j) {
      const int64_t i = kb * kBlk + j;
      const int64_t idx = transposed ? i * p.ld + o : o * p.ld + i;
      f[j] = (float)x[idx];
      amax = fmaxf(amax, fabsf(f[j]));
    }
    if (kFmt == kNvfp4) {
      const float s = nvfp4_scale(amax);
      uint32_t word = 0;
#pragma unroll
      for (int j = 0; j < kBlk; j += 2) {
        float y0 = __fdiv_rn(f[j], s), y1 = __fdiv_rn(f[j + 1], s);
        if (sr != FP4T_SR_NONE) {
          const int64_t e = o * inner + kb * kBlk + j;
          const uint64_t seed = transposed ? (p.seed ^ 0x5bd1e995c2b2ae35ull) : p.seed;
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

template <int kFmt>
int quantize_dispatch(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                      void* codes, void* sf, void* codes_t, void* sf_t, int sr_mode,
                      const float* noise, const float* noise_t, uint64_t seed, cudaStream_t stream) {
  constexpr int kBlk = kFmt == kNvfp4 ? 16 : 32;
  const char* name = kFmt == kNvfp4 ? "fp4t_quantize_nvfp4" : "fp4t_quantize_mxfp8";
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
  if (rows == 0 || cols == 0) return FP4T_OK;

  QParams p;
  p.x = x; p.rows = rows; p.cols = cols; p.ld = ld;
  p.codes = static_cast<uint8_t*>(codes); p.sf = static_cast<uint8_t*>(sf);
  p.codes_t = static_cast<uint8_t*>(codes_t); p.sf_t = static_cast<uint8_t*>(sf_t);
  p.noise = noise; p.noise_t = noise_t; p.seed = seed;
  p.ntx_row = (int)ceil_div(ceil_div(cols, kBlk), 4);
  p.ntx_col = (int)ceil_div(ceil_div(rows, kBlk), 4);

  const bool fast = x_dtype == FP4T_DT_BF16 && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                    (ld % 8 == 0) && (cols % 8 == 0) &&
                    (codes == nullptr || reinterpret_cast<uintptr_t>(codes) % 16 == 0) &&
                    (codes_t == nullptr || reinterpret_cast<uintptr_t>(codes_t) % 16 == 0) &&
                    (sf == nullptr || reinterpret_cast<uintptr_t>(sf) % 16 == 0) &&
                    (sf_t == nullptr || reinterpret_cast<uintptr_t>(sf_t) % 16 == 0);
  if (!fast) return launch_generic<kFmt>(p, x_dtype, sr_mode, stream);

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
#define FP4T_LAUNCH_Q(FMT, SR)                                                                             \
  do {                                                                                                     \
    auto kern = quantize_tma_kernel<FMT, SR>;                                                              \
    FP4T_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, QCfg<FMT>::kSmemBytes)); \
    kern<<<grid, kQThreads, QCfg<FMT>::kSmemBytes, stream>>>(map_x, p, (int)tiles_x, num_tiles, status);   \
  } while (0)
  if (kFmt == kMxfp8) {
    FP4T_LAUNCH_Q(kMxfp8, FP4T_SR_NONE);
  } else if (sr_mode == FP4T_SR_NONE) {
    FP4T_LAUNCH_Q(kNvfp4, FP4T_SR_NONE);
  } else if (sr_mode == FP4T_SR_NOISE) {
    FP4T_LAUNCH_Q(kNvfp4, FP4T_SR_NOISE);
  } else {
    FP4T_LAUNCH_Q(kNvfp4, FP4T_SR_HASH);
  }
#undef FP4T_LAUNCH_Q
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}

}  // namespace
}  // namespace fp4t

extern "C" int fp4t_quantize_nvfp4(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                   void* codes, void* sf, void* codes_t, void* sf_t, int sr_mode,
                                   const float* noise, const float* noise_t, uint64_t seed,
                                   fp4t_stream_t stream) {
  return fp4t::quantize_dispatch<fp4t::kNvfp4>(x, x_dtype, rows, cols, ld, codes, sf, codes_t, sf_t,
                                               sr_mode, noise, noise_t, seed,
                                               reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int fp4t_quantize_mxfp8(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                   void* codes, void* sf, void* codes_t, void* sf_t,
                                   fp4t_stream_t stream) {
  return fp4t::quantize_dispatch<fp4t::kMxfp8>(x, x_dtype, rows, cols, ld, codes, sf, codes_t, sf_t,
                                               FP4T_SR_NONE, nullptr, nullptr, 0,
                                               reinterpret_cast<cudaStream_t>(stream));
}
