// Fused block quantizers for NVFP4 (1x16 blocks, UE4M3 scales) and MXFP8 (1x32
// blocks, UE8M0 scales).
//
// One launch reads a 128x128 tile of the bf16 input once (16-byte coalesced
// loads), and writes
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

namespace fp4t {
namespace {

constexpr int kTile = 128;
constexpr int kThreads = 256;
constexpr int kPitchW = 68;  // 32-bit words per shared row: 64 data + 4 pad

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
// Fast path: bf16 input, 16-byte aligned rows.
// ---------------------------------------------------------------------------------------
template <int kFmt, int kSr>
__global__ void __launch_bounds__(kThreads) quantize_tile_kernel(const QParams p) {
  constexpr int kBlk = kFmt == kNvfp4 ? 16 : 32;      // elements per scale
  constexpr int kKbTile = kTile / kBlk;               // k-blocks per tile edge: 8 or 4
  constexpr int kSfChunks = kKbTile / 4;              // 512-byte scale tiles per tile edge: 2 or 1
  constexpr int kLanesPerBlk = kBlk / 8;              // lanes sharing one row-wise block: 2 or 4

  __shared__ uint32_t tile[kTile * kPitchW];
  __shared__ __align__(16) uint8_t sf_row_s[kSfChunks * 512];
  __shared__ __align__(16) uint8_t sf_col_s[kSfChunks * 512];

  const int tid = threadIdx.x;
  const int64_t row0 = (int64_t)blockIdx.y * kTile;
  const int64_t col0 = (int64_t)blockIdx.x * kTile;
  const bool want_row = p.codes != nullptr;
  const bool want_col = p.codes_t != nullptr;
  const __nv_bfloat16* __restrict__ x = static_cast<const __nv_bfloat16*>(p.x);

  for (int i = tid; i < kSfChunks * 512 / 4; i += kThreads) {
    reinterpret_cast<uint32_t*>(sf_row_s)[i] = 0u;
    reinterpret_cast<uint32_t*>(sf_col_s)[i] = 0u;
  }

  // ---- load: 8 vectors of 8 bf16 per thread, all issued before use -------------------
  uint4 v[8];
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int vi = it * kThreads + tid;
    const int r = vi >> 4, cv = vi & 15;
    const int64_t gr = row0 + r, gc = col0 + cv * 8;
    v[it] = make_uint4(0u, 0u, 0u, 0u);
    if (gr < p.rows && gc < p.cols) {
      v[it] = __ldg(reinterpret_cast<const uint4*>(x + gr * p.ld + gc));
    }
  }
  __syncthreads();  // scale staging is zeroed

  // ---- row-wise pass ----------------------------------------------------------------
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int vi = it * kThreads + tid;
    const int r = vi >> 4, cv = vi & 15;
    const int64_t gr = row0 + r, gc = col0 + cv * 8;
    const uint32_t w[4] = {v[it].x, v[it].y, v[it].z, v[it].w};
    if (want_col) {
      *reinterpret_cast<uint4*>(&tile[r * kPitchW + cv * 4]) = v[it];
    }
    if (want_row) {
      float f[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        f[2 * j] = __uint_as_float(w[j] << 16);
        f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
      }
      float amax = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
      amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
      if (kLanesPerBlk == 4) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
      const bool valid = gr < p.rows && gc < p.cols;
      const int kb = (cv * 8) / kBlk;  // k-block inside the tile
      if (kFmt == kNvfp4) {
        const float s = nvfp4_scale(amax);
        const float rcp = __fdiv_rn(1.0f, s);
        float y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = div_corrected(f[j], s, rcp);
        if (kSr != FP4T_SR_NONE) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float u;
            if (kSr == FP4T_SR_NOISE) {
              u = valid ? __ldg(p.noise + gr * p.cols + gc + j) : 0.5f;
            } else {
              u = hash_uniform(p.seed, (uint64_t)(gr * p.cols + gc + j));
            }
            y[j] = sr_round(y[j], u);
          }
        }
        const uint32_t packed = cvt_e2m1x8(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7]);
        if (valid) {
          *reinterpret_cast<uint32_t*>(p.codes + gr * (p.cols >> 1) + (gc >> 1)) = packed;
          if ((cv & 1) == 0) sf_row_s[(kb >> 2) * 512 + sf_tile_offset(r, kb)] = (uint8_t)cvt_e4m3(s);
        }
      } else {
        const uint32_t sb = mx_scale_byte(amax);
        const float inv = mx_inv_scale(sb);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          lo |= mx_e4m3_byte<true>(f[j] * inv) << (8 * j);
          hi |= mx_e4m3_byte<true>(f[4 + j] * inv) << (8 * j);
        }
        if (valid) {
          *reinterpret_cast<uint2*>(p.codes + gr * p.cols + gc) = make_uint2(lo, hi);
          if ((cv & 3) == 0) sf_row_s[sf_tile_offset(r, kb)] = (uint8_t)sb;
        }
      }
    }
  }

  // ---- transposed pass ----------------------------------------------------------------
  if (want_col) {
    __syncthreads();
    const int cp = tid & 63;       // column pair inside the tile
    const int q = tid >> 6;        // 32-row quarter of the tile
    const int64_t gr0 = row0 + q * 32;
    const int64_t gcA = col0 + 2 * cp;
    uint32_t w[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = tile[(q * 32 + j) * kPitchW + cp];

    if (kFmt == kNvfp4) {
      uint32_t outA[4], outB[4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float amA = 0.0f, amB = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          amA = fmaxf(amA, fabsf(__uint_as_float(w[h * 16 + j] << 16)));
          amB = fmaxf(amB, fabsf(__uint_as_float(w[h * 16 + j] & 0xFFFF0000u)));
        }
        const float sA = nvfp4_scale(amA), sB = nvfp4_scale(amB);
        const float rA = __fdiv_rn(1.0f, sA), rB = __fdiv_rn(1.0f, sB);
        float yA[16], yB[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          yA[j] = div_corrected(__uint_as_float(w[h * 16 + j] << 16), sA, rA);
          yB[j] = div_corrected(__uint_as_float(w[h * 16 + j] & 0xFFFF0000u), sB, rB);
        }
        if (kSr != FP4T_SR_NONE) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int64_t gr = gr0 + h * 16 + j;
            float uA, uB;
            if (kSr == FP4T_SR_NOISE) {
              const bool ok = gr < p.rows;
              uA = (ok && gcA < p.cols) ? __ldg(p.noise_t + gcA * p.rows + gr) : 0.5f;
              uB = (ok && gcA + 1 < p.cols) ? __ldg(p.noise_t + (gcA + 1) * p.rows + gr) : 0.5f;
            } else {
              uA = hash_uniform(p.seed ^ 0x5bd1e995c2b2ae35ull, (uint64_t)(gcA * p.rows + gr));
              uB = hash_uniform(p.seed ^ 0x5bd1e995c2b2ae35ull, (uint64_t)((gcA + 1) * p.rows + gr));
            }
            yA[j] = sr_round(yA[j], uA);
            yB[j] = sr_round(yB[j], uB);
          }
        }
        outA[2 * h] = cvt_e2m1x8(yA[0], yA[1], yA[2], yA[3], yA[4], yA[5], yA[6], yA[7]);
        outA[2 * h + 1] = cvt_e2m1x8(yA[8], yA[9], yA[10], yA[11], yA[12], yA[13], yA[14], yA[15]);
        outB[2 * h] = cvt_e2m1x8(yB[0], yB[1], yB[2], yB[3], yB[4], yB[5], yB[6], yB[7]);
        outB[2 * h + 1] = cvt_e2m1x8(yB[8], yB[9], yB[10], yB[11], yB[12], yB[13], yB[14], yB[15]);
        const int kb = q * 2 + h;
        if (gr0 + h * 16 < p.rows) {
          if (gcA < p.cols) sf_col_s[(kb >> 2) * 512 + sf_tile_offset(2 * cp, kb)] = (uint8_t)cvt_e4m3(sA);
          if (gcA + 1 < p.cols) sf_col_s[(kb >> 2) * 512 + sf_tile_offset(2 * cp + 1, kb)] = (uint8_t)cvt_e4m3(sB);
        }
      }
      if (gr0 < p.rows) {  // rows % 32 == 0: the quarter is entirely inside or outside
        if (gcA < p.cols)
          *reinterpret_cast<uint4*>(p.codes_t + gcA * (p.rows >> 1) + (gr0 >> 1)) =
              make_uint4(outA[0], outA[1], outA[2], outA[3]);
        if (gcA + 1 < p.cols)
          *reinterpret_cast<uint4*>(p.codes_t + (gcA + 1) * (p.rows >> 1) + (gr0 >> 1)) =
              make_uint4(outB[0], outB[1], outB[2], outB[3]);
      }
    } else {
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
      for (int g = 0; g < 8; ++g) {
        uint32_t a = 0, b = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          a |= mx_e4m3_byte<true>(__uint_as_float(w[g * 4 + j] << 16) * invA) << (8 * j);
          b |= mx_e4m3_byte<true>(__uint_as_float(w[g * 4 + j] & 0xFFFF0000u) * invB) << (8 * j);
        }
        oA[g] = a;
        oB[g] = b;
      }
      if (gr0 < p.rows) {
        if (gcA < p.cols) {
          uint4* dst = reinterpret_cast<uint4*>(p.codes_t + gcA * p.rows + gr0);
          dst[0] = make_uint4(oA[0], oA[1], oA[2], oA[3]);
          dst[1] = make_uint4(oA[4], oA[5], oA[6], oA[7]);
          sf_col_s[sf_tile_offset(2 * cp, q)] = (uint8_t)sbA;
        }
        if (gcA + 1 < p.cols) {
          uint4* dst = reinterpret_cast<uint4*>(p.codes_t + (gcA + 1) * p.rows + gr0);
          dst[0] = make_uint4(oB[0], oB[1], oB[2], oB[3]);
          dst[1] = make_uint4(oB[4], oB[5], oB[6], oB[7]);
          sf_col_s[sf_tile_offset(2 * cp + 1, q)] = (uint8_t)sbB;
        }
      }
    }
  }

  // ---- scale tiles out: whole 512-byte tiles, zero padding included --------------------
  __syncthreads();
  constexpr int kVecs = kSfChunks * 32;  // 16-byte vectors per staging buffer
  if (want_row && tid < kVecs) {
    const int chunk = tid >> 5;
    const int64_t tx = (int64_t)blockIdx.x * kSfChunks + chunk;
    if (tx < p.ntx_row) {
      uint8_t* dst = p.sf + ((int64_t)blockIdx.y * p.ntx_row + tx) * 512;
      reinterpret_cast<uint4*>(dst)[tid & 31] = reinterpret_cast<const uint4*>(sf_row_s)[tid];
    }
  }
  if (want_col && tid >= 64 && tid < 64 + kVecs) {
    const int t = tid - 64;
    const int chunk = t >> 5;
    const int64_t tx = (int64_t)blockIdx.y * kSfChunks + chunk;
    if (tx < p.ntx_col) {
      uint8_t* dst = p.sf_t + ((int64_t)blockIdx.x * p.ntx_col + tx) * 512;
      reinterpret_cast<uint4*>(dst)[t & 31] = reinterpret_cast<const uint4*>(sf_col_s)[t];
    }
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

  const dim3 grid((unsigned)ceil_div(cols, kTile), (unsigned)ceil_div(rows, kTile));
  FP4T_REQUIRE(grid.y <= 65535u, "%s: rows too large for one launch (%lld)", name, (long long)rows);
  if (kFmt == kMxfp8) {
    quantize_tile_kernel<kMxfp8, FP4T_SR_NONE><<<grid, kThreads, 0, stream>>>(p);
  } else if (sr_mode == FP4T_SR_NONE) {
    quantize_tile_kernel<kNvfp4, FP4T_SR_NONE><<<grid, kThreads, 0, stream>>>(p);
  } else if (sr_mode == FP4T_SR_NOISE) {
    quantize_tile_kernel<kNvfp4, FP4T_SR_NOISE><<<grid, kThreads, 0, stream>>>(p);
  } else {
    quantize_tile_kernel<kNvfp4, FP4T_SR_HASH><<<grid, kThreads, 0, stream>>>(p);
  }
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
