// Block-scaled GEMM on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
//   D[rows, cols] = P[rows, K] . Q[cols, K]^T (+ bias[cols]),  fp32 accumulate, bf16/fp32 out
//
// P and Q are K-major code matrices (NVFP4: E2M1 two per byte with UE4M3 scales per 16
// elements; MXFP8: E4M3 bytes with UE8M0 scales per 32 elements); their scale factors are
// in the 128x4 tile layout, which is exactly the 32-lane x 16-byte image that one
// `tcgen05.cp ... 32x128b.warpx4` drops into tensor memory for the MMA to consume.
//
// One-CTA kernel (one persistent CTA per SM, 384 threads, static tile schedule):
//   warp 0      TMA producer: per stage one 128-byte-of-K slab of P (128 rows) and of Q
//               (kBN rows) with 128-byte swizzle, plus the matching scale tiles (tensor maps
//               over the tile layout; K beyond the matrix reads as zero codes and zero
//               scales).  No multicast.
//   warp 1      MMA issuer: four tcgen05.mma per stage (K = 64 FP4 / 32 FP8 elements each)
//               into a 128 x kBN fp32 accumulator in tensor memory; tcgen05.commit releases
//               the stage and, after the last stage, publishes the accumulator.
//   warp 2      tensor-memory allocation / release.
//   warps 4-7   epilogue: tcgen05.ld 32 lanes x 32 columns at a time, + bias, convert,
//               16-byte stores.  Two accumulators alternate so the epilogue of tile i
//               overlaps the main loop of tile i+1; with kBN = 256 they overlap by 96 columns
//               (the scale factors need the rest); the epilogue pulls those columns into
//               registers first and signals the MMA warp before it converts and stores.
//   warps 8-11  scale factors: each warp copies the stage's scale tiles from shared memory
//               into its 32-lane quadrant of tensor memory with tcgen05.st (two buffers), so
//               the tensor pipe executes nothing but MMAs.  (tcgen05.cp does the same copy
//               inside the tensor pipe, in order with the MMAs; twelve of them per NVFP4
//               stage cost more pipe time than the four MMAs.)
// Two-CTA kernel: see below.
//
// Every wait on an mbarrier is bounded: if it runs out, the kernel records a code in the
// caller's status word, stops issuing work, lets copies in flight land and releases its
// tensor memory before returning.
#include <cuda.h>
#include <cstdlib>

#include "fp4t_common.cuh"
#include "fp4t_ptx.cuh"

namespace fp4t {
namespace {

enum { kNvfp4 = 0, kMxfp8 = 1 };

constexpr int kBM = 128;             // rows of P per tile (the MMA M)
constexpr int kTmemCols = 512;

constexpr int kGemm1Threads = 384;

template <int kFmt, int kBN>
struct Cfg {
  static constexpr int kSfChunks = kFmt == kNvfp4 ? 4 : 1;   // 512-byte scale tiles per 128 rows per stage
  static constexpr int kOuterB = kBN / 128;                  // 128-row scale tiles of Q per CTA tile
  static constexpr int kABytes = kBM * 128;
  static constexpr int kBBytes = kBN * 128;
  static constexpr int kSfaBytes = kSfChunks * 512;
  static constexpr int kSfbBytes = kOuterB * kSfChunks * 512;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kStages = (220 * 1024) / kStageBytes > 8 ? 8 : (220 * 1024) / kStageBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  // tensor memory: accumulators at 0 and kAccStride, two 48-column scale-factor buffers at 416 and 464
  static constexpr int kAccStride = (kBN == 256) ? 160 : 128;
  static constexpr int kChunks = kBN / 32;                     // 32-column epilogue chunks
  static constexpr int kEarlyChunks = (kBN == 256) ? 3 : 0;    // chunks the other accumulator overlaps
  static constexpr int kSfBuf0 = 416;
  static constexpr int kSfbOff = kSfChunks * 4;                // SFB columns follow the SFA columns
  static constexpr int kSfBufStride = kSfChunks * 4 + kSfChunks * kOuterB * 4;   // columns of one stage's scales
  static constexpr int kSfBufs = (96 / kSfBufStride) > 4 ? 4 : (96 / kSfBufStride);  // ring depth (2 for NVFP4)
  static constexpr int kSfBoxElems = kSfChunks * 64;           // 8-byte words per scale box row
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
  static_assert(kAccStride + kBN <= kSfBuf0, "tensor memory budget");
};

struct GemmParams {
  const uint8_t* p_sf;
  const uint8_t* q_sf;
  const __nv_bfloat16* bias;
  void* d;
  int64_t ldd;
  int rows, cols, k;
  int ntx;          // scale tiles along K (per 128 rows)
  int q_outer;      // 128-row scale tiles of Q
  int m_tiles, n_tiles, k_stages;
  int out_f32;
  int vec_ok;       // 16-byte stores allowed
  int tma_ok;       // the output can be written with tiled TMA stores
  int sched;        // tile-counter slot of the launching stream, or -1 for the static order
  int32_t* status;
};

// ------------------------------------------------------------------------------------
// tcgen05 wrappers (mbarrier / TMA wrappers live in fp4t_ptx.cuh)
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <int kFmt>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate, uint32_t sfa, uint32_t sfb) {
  if (kFmt == kNvfp4) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  }
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors. Bits: [0,14) address>>4, [16,30) leading byte offset>>4,
// [32,46) stride byte offset>>4, [46,48) version = 1, [61,64) swizzle mode.  The low word is
// just (shared address >> 4), so stepping through a stage is one 32-bit add.
constexpr uint32_t kDescHiOperand = (1024u >> 4) | (1u << 14) | (2u << 29);  // 8-row groups 1024 B apart, 128-byte swizzle
__device__ __forceinline__ uint64_t make_desc(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Instruction descriptor of the block-scaled MMA: [4,6) B scale id, [7,10) A format,
// [10,13) B format, 15/16 A/B major (0 = K), [17,23) N>>3, 23 scale format (0 UE4M3, 1 UE8M0),
// [24,29) M>>4, [29,31) A scale id.
template <int kFmt, int kBN>
__device__ __forceinline__ uint32_t make_idesc() {
  const uint32_t fmt = kFmt == kNvfp4 ? 1u /*E2M1*/ : 0u /*E4M3*/;
  const uint32_t sfmt = kFmt == kNvfp4 ? 0u : 1u;
  return (fmt << 7) | (fmt << 10) | ((uint32_t)(kBN >> 3) << 17) | (sfmt << 23) | ((uint32_t)(kBM >> 4) << 24);
}

// Epilogue of one 32-column chunk held in registers: + bias, convert, store (16-byte vectors
// when the row pitch and the chunk allow it, element-wise at ragged edges).
__device__ __forceinline__ void store_chunk(const GemmParams& g, const int row, const bool row_ok, const int col0,
                                            const uint32_t (&r)[32]) {
  if (row_ok && col0 < g.cols) {
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (g.bias != nullptr) {
      if (g.vec_ok && col0 + 32 <= g.cols) {
        const uint4* bp = reinterpret_cast<const uint4*>(g.bias + col0);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint4 b = __ldg(bp + q4);
          const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[q4 * 8 + 2 * j] += __uint_as_float(bw[j] << 16);
            v[q4 * 8 + 2 * j + 1] += __uint_as_float(bw[j] & 0xFFFF0000u);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < g.cols) v[j] += __bfloat162float(g.bias[col0 + j]);
      }
    }
    if (g.out_f32) {
      float* dp = static_cast<float*>(g.d) + (int64_t)row * g.ldd + col0;
      if (g.vec_ok && col0 + 32 <= g.cols) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          reinterpret_cast<float4*>(dp)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < g.cols) dp[j] = v[j];
      }
    } else {
      __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(g.d) + (int64_t)row * g.ldd + col0;
      if (g.vec_ok && col0 + 32 <= g.cols) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t w[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * j + 2 * t], v[8 * j + 2 * t + 1]);
            w[t] = *reinterpret_cast<uint32_t*>(&h);
          }
          reinterpret_cast<uint4*>(dp)[j] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < g.cols) dp[j] = __float2bfloat16_rn(v[j]);
      }
    }
  }
}


// Epilogue of one 32-row x 32-column chunk through shared memory and one tiled TMA store.
// Each lane holds one row of the chunk in registers; the rows go to a swizzled staging tile
// (conflict-free 16-byte writes) that the TMA store un-swizzles and clips at the matrix
// edges.  Thread-per-row stores straight to global memory scatter 16-byte pieces over 32
// rows per instruction and kept the load/store pipe busy for microseconds per tile, which
// delayed the scale-factor warps and with them the main loop.
// `buf` is this warp's staging area (4 KB, 1024-byte aligned): two 2-KB tiles for bf16 output
// that alternate, one 4-KB tile for fp32 output.
__device__ __forceinline__ void emit_chunk(const GemmParams& g, const CUtensorMap* map_d, uint8_t* buf, uint32_t& n_emit,
                                           const int lane, const int row0, const int col0, const uint32_t (&r)[32]) {
  if (row0 >= g.rows || col0 >= g.cols) return;   // warp-uniform
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  if (g.bias != nullptr) {
    if (g.vec_ok && col0 + 32 <= g.cols) {
      const uint4* bp = reinterpret_cast<const uint4*>(g.bias + col0);
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const uint4 b = __ldg(bp + q4);
        const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[q4 * 8 + 2 * j] += __uint_as_float(bw[j] << 16);
          v[q4 * 8 + 2 * j + 1] += __uint_as_float(bw[j] & 0xFFFF0000u);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < g.cols) v[j] += __bfloat162float(g.bias[col0 + j]);
    }
  }
  if (g.out_f32) {
    if (lane == 0) bulk_wait_read<0>();
    __syncwarp();
    uint8_t* rowp = buf + lane * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      *reinterpret_cast<float4*>(rowp + ((j ^ (lane & 7)) << 4)) =
          make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    fence_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(map_d, smem_u32(buf), col0, row0);
      bulk_commit();
    }
  } else {
    uint8_t* tile = buf + (n_emit & 1u) * 2048;
    if (lane == 0) bulk_wait_read<1>();
    __syncwarp();
    uint8_t* rowp = tile + lane * 64;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t w[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * j + 2 * t], v[8 * j + 2 * t + 1]);
        w[t] = *reinterpret_cast<uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(rowp + ((j ^ ((lane >> 1) & 3)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    fence_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(map_d, smem_u32(tile), col0, row0);
      bulk_commit();
    }
  }
  ++n_emit;
}

// ------------------------------------------------------------------------------------
// The kernel
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void tc_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// N consecutive 32-bit columns of this warp's lane quadrant from registers (N = 4, 8, 16 or 32).
template <int N>
__device__ __forceinline__ void tc_st_n(uint32_t taddr, const uint32_t (&v)[N]) {
  static_assert(N == 4 || N == 8 || N == 16 || N == 32, "unsupported width");
  if constexpr (N == 4) {
    tc_st4(taddr, v[0], v[1], v[2], v[3]);
  } else if constexpr (N == 8) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
                 "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
  } else if constexpr (N == 16) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
        "%15, %16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
  } else {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
        "%15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
        "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
        "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
  }
}

template <int kFmt, int kBN>
__global__ void __launch_bounds__(kGemm1Threads, 1)
gemm_blockscaled_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                        const __grid_constant__ CUtensorMap map_psf, const __grid_constant__ CUtensorMap map_qsf,
                        const GemmParams g) {
  using C = Cfg<kFmt, kBN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  // barrier block sits after the stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + C::kStages * C::kStageBytes);
  const uint32_t bar_full = smem_u32(bars);                       // [kStages] stage data landed
  const uint32_t bar_empty = bar_full + 8 * C::kStages;           // [kStages] MMAs that read the stage are done
  const uint32_t bar_sf_ready = bar_empty + 8 * C::kStages;       // [2] scale factors are in tensor memory
  const uint32_t bar_tmem_full = bar_sf_ready + 32;               // [1]
  const uint32_t bar_tmem_empty = bar_tmem_full + 8;              // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < C::kSfBufs; ++b) mbar_init(bar_sf_ready + 8 * b, 4);
    mbar_init(bar_tmem_full, 1);
    mbar_init(bar_tmem_empty, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = g.m_tiles * g.n_tiles;

  // Warps 0 and 1 work through one lane; the other lanes wait at the __syncwarp that
  // closes the branch so that each warp reaches the final block barrier converged.
  if (warp == 0) {
   if (lane == 0) {
    // ------------------------------ TMA producer ------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m_idx = tile / g.n_tiles, n_idx = tile % g.n_tiles;
      const int row_p = m_idx * kBM, row_q = n_idx * kBN;
      for (int ks = 0; ks < g.k_stages; ++ks) {
        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, g.status, 1)) { ok = false; break; }
        const uint32_t a_s = smem_base + stage * C::kStageBytes;
        const uint32_t b_s = a_s + C::kABytes;
        const uint32_t sfa_s = b_s + C::kBBytes;
        const uint32_t sfb_s = sfa_s + C::kSfaBytes;
        const uint32_t bar = bar_full + 8 * stage;
        mbar_expect_tx(bar, (uint32_t)C::kStageBytes);
        tma_load_2d(sfa_s, &map_psf, bar, ks * C::kSfBoxElems, m_idx);
#pragma unroll
        for (int o = 0; o < C::kOuterB; ++o) {
          tma_load_2d(sfb_s + o * C::kSfaBytes, &map_qsf, bar, ks * C::kSfBoxElems, n_idx * C::kOuterB + o);
        }
        tma_load_2d(a_s, &map_p, bar, ks * 128, row_p);
        tma_load_2d(b_s, &map_q, bar, ks * 128, row_q);
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (*abort_flag) {  // let copies in flight land before shared memory is given back
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {}
    }
   }
   __syncwarp();
  } else if (warp == 1) {
   if (lane == 0) {
    // ------------------------------ MMA issuer ------------------------------
    const uint32_t idesc = make_idesc<kFmt, kBN>();
    int stage = 0;
    uint32_t phase = 0;
    uint32_t k = 0;          // stages issued so far; selects the scale-factor buffer
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      if (it > 0) {
        if (!mbar_wait(bar_tmem_empty, (uint32_t)((it - 1) & 1), abort_flag, g.status, 2)) { ok = false; break; }
        tc_fence_after();
      }
      const uint32_t acc = tmem_base + (uint32_t)((it & 1) * C::kAccStride);
      for (int ks = 0; ks < g.k_stages; ++ks, ++k) {
        // scale factors in tensor memory imply the stage's data landed (the scale warps waited for it)
        if (!mbar_wait(bar_sf_ready + 8 * (k % C::kSfBufs), (k / C::kSfBufs) & 1u, abort_flag, g.status, 3)) { ok = false; break; }
        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, g.status, 7)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_lo = ((smem_base + stage * C::kStageBytes) & 0x3FFFFu) >> 4;
        const uint32_t b_lo = a_lo + (C::kABytes >> 4);
        const uint32_t sfa_t = tmem_base + C::kSfBuf0 + (k % C::kSfBufs) * C::kSfBufStride;
        const uint32_t sfb_t = sfa_t + C::kSfbOff;
        const uint32_t first = ks > 0 ? 1u : 0u;
        // K beyond the matrix is zero codes times zero scales, so every stage issues all four MMAs.
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (kFmt == kNvfp4) {
            tc_mma<kFmt>(acc, make_desc(a_lo + 2 * j, kDescHiOperand), make_desc(b_lo + 2 * j, kDescHiOperand), idesc,
                         j == 0 ? first : 1u, sfa_t + j * 4, sfb_t + j * (kBN / 32));
          } else {
            tc_mma<kFmt>(acc, make_desc(a_lo + 2 * j, kDescHiOperand), make_desc(b_lo + 2 * j, kDescHiOperand),
                         idesc | ((uint32_t)j << 29) | ((uint32_t)j << 4), j == 0 ? first : 1u, sfa_t, sfb_t);
          }
        }
        tc_commit(bar_empty + 8 * stage);   // frees the stage and its scale-factor buffer
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
      if (ok) tc_commit(bar_tmem_full);
    }
   }
   __syncwarp();
  } else if (warp >= 8) {
    // ------------------------------ scale-factor warps ------------------------------
    // Each warp owns one 32-lane quadrant of tensor memory and writes the same scale image into
    // it: lane l of a 512-byte scale tile is its 16 bytes at offset 16*l, i.e. four columns.
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t k = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      for (int ks = 0; ks < g.k_stages; ++ks, ++k) {
        const uint32_t stage = k % C::kStages, use = k / C::kStages;
        // every lane polls (no broadcast hop); the scale bytes are in registers before the wait
        // for the tensor-memory buffer, so only store + signal sit between MMA(k-2) and MMA(k)
        if (!mbar_wait(bar_full + 8 * stage, use & 1u, abort_flag, g.status, 5)) { ok = false; break; }
        const uint8_t* sfa_s = smem_gen + stage * C::kStageBytes + C::kABytes + C::kBBytes;
        const uint8_t* sfb_s = sfa_s + C::kSfaBytes;
        uint32_t va[C::kSfChunks * 4], vb[C::kSfChunks * C::kOuterB * 4];
#pragma unroll
        for (int c = 0; c < C::kSfChunks; ++c) {
          const uint4 v = *reinterpret_cast<const uint4*>(sfa_s + c * 512 + lane * 16);
          va[4 * c] = v.x; va[4 * c + 1] = v.y; va[4 * c + 2] = v.z; va[4 * c + 3] = v.w;
#pragma unroll
          for (int o = 0; o < C::kOuterB; ++o) {
            const uint4 u = *reinterpret_cast<const uint4*>(sfb_s + (o * C::kSfChunks + c) * 512 + lane * 16);
            const int j = (c * C::kOuterB + o) * 4;   // column order in tensor memory: chunk-major, then outer tile
            vb[j] = u.x; vb[j + 1] = u.y; vb[j + 2] = u.z; vb[j + 3] = u.w;
          }
        }
        if (k >= (uint32_t)C::kSfBufs) {   // the MMAs that last read this scale-factor buffer are done
          const uint32_t j = k - C::kSfBufs;
          if (!mbar_wait(bar_empty + 8 * (j % C::kStages), (j / C::kStages) & 1u, abort_flag, g.status, 6)) { ok = false; break; }
        }
        __syncwarp();   // lanes leave the polling loop at different times; tcgen05.st needs the whole warp
        tc_fence_after();
        const uint32_t sfa_t = tmem_base + lane_sel + C::kSfBuf0 + (k % C::kSfBufs) * C::kSfBufStride;
        const uint32_t sfb_t = sfa_t + C::kSfbOff;
        tc_st_n<C::kSfChunks * 4>(sfa_t, va);
        tc_st_n<C::kSfChunks * C::kOuterB * 4>(sfb_t, vb);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sf_ready + 8 * (k % C::kSfBufs));
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int m_idx = tile / g.n_tiles, n_idx = tile % g.n_tiles;
      int ok = 1;
      if (lane == 0) ok = mbar_wait(bar_tmem_full, (uint32_t)(it & 1), abort_flag, g.status, 4) ? 1 : 0;
      ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)((it & 1) * C::kAccStride);
      const int row = m_idx * kBM + quad * 32 + lane;
      const bool row_ok = row < g.rows;
      const int col_base = n_idx * kBN;
      if (kBN == 256) {
        // The columns the other accumulator overlaps (the last 96 of accumulator 0, the first 96
        // of accumulator 1) go to registers first; then the MMA warp may start the next tile.
        const int e0 = (it & 1) == 0 ? C::kChunks - C::kEarlyChunks : 0;
        uint32_t early[3][32];
#pragma unroll
        for (int e = 0; e < 3; ++e) tc_ld32(acc + (uint32_t)((e0 + e) * 32), early[e]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tmem_empty);
#pragma unroll
        for (int e = 0; e < 3; ++e) store_chunk(g, row, row_ok, col_base + (e0 + e) * 32, early[e]);
        const int r0 = (it & 1) == 0 ? 0 : C::kEarlyChunks;
#pragma unroll 1
        for (int ci = 0; ci < C::kChunks - C::kEarlyChunks; ++ci) {
          uint32_t r[32];
          tc_ld32(acc + (uint32_t)((r0 + ci) * 32), r);
          tc_wait_ld();
          store_chunk(g, row, row_ok, col_base + (r0 + ci) * 32, r);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < C::kChunks; ++c) {
          uint32_t r[32];
          tc_ld32(acc + (uint32_t)(c * 32), r);
          tc_wait_ld();
          if (c == C::kChunks - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tmem_empty);
          }
          store_chunk(g, row, row_ok, col_base + c * 32, r);
        }
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

// ------------------------------------------------------------------------------------
// Two-CTA variant: a cluster of two CTAs (two SMs) works on one 256 x kBN tile with
// cta_group::2 MMAs.  Each CTA holds its own 128 rows of P and HALF of the Q rows in shared
// memory (the MMA reads both halves across the pair), so the Q-operand traffic per SM is
// halved compared with the one-CTA kernel; the accumulator of each CTA is 128 lanes x kBN
// columns in its own tensor memory.  Every load is a plain tiled TMA load (no multicast);
// both CTAs' operand loads complete on the leader CTA's "full" barrier (armed by the leader
// alone with the bytes of both), each CTA's scale warps fill their own tensor memory and
// arrive on the leader's "scales ready" barrier, and the leader issues the MMAs for the pair
// and commits to the barriers of both CTAs.  Remote arrives are the plain form (no
// cluster-scope release): an arrive with .release.cluster from the second CTA every stage
// cost about 1 us per stage.
//   Warp roles per CTA: 0 operand producer, 1 MMA issuer (leader only), 2 tensor-memory
// allocation and then the tile scheduler (leader only: tile indices from the stream's device
// counter, or the static order, published to both CTAs through a small queue), 3 scale-tile
// producer, 4-7 epilogue, 8-11 scale factors.  Operands and scale
// tiles have separate shared-memory rings (a scale slot is free once its bytes sit in the
// scale warps' registers), and the epilogue leaves through swizzled staging tiles and tiled
// TMA stores (clipped at the matrix edges); an output whose base or pitch is not 16-byte
// aligned falls back to per-thread stores.
// ------------------------------------------------------------------------------------
constexpr int kGemm2Threads = 384;
constexpr int kSched = 4;   // depth of the in-kernel tile queue
constexpr int kSchedReaders = 21;   // roles that read each entry: 11 in the leader CTA (with the MMA issuer), 10 in the other

// {next tile, clusters done} per stream slot; both are zero between launches (the last cluster
// to run dry puts them back)
__device__ unsigned int g_gemm_sched[2 * kSchedSlots];

__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// remote arrive that publishes this thread's earlier shared::cluster stores
__device__ __forceinline__ void mbar_arrive_release_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

template <int kFmt, int kBN>
struct Cfg2 {
  static constexpr int kSfChunks = kFmt == kNvfp4 ? 4 : 1;
  static constexpr int kOuterB = kBN / 128;
  static constexpr int kABytes = kBM * 128;
  static constexpr int kBBytes = (kBN / 2) * 128;            // this CTA's half of the Q slab
  static constexpr int kSfaBytes = kSfChunks * 512;
  static constexpr int kSfbBytes = kOuterB * kSfChunks * 512;  // scales of ALL kBN columns
  // Operands and scale tiles live in separate rings.  A scale slot is free again as soon as
  // the scale warps hold its bytes in registers, long before the MMAs that use the operand
  // stage complete, so a short scale ring leaves room for one more operand stage: the main
  // loop is bound by bytes in flight (round trip x bandwidth), not by the tensor pipe.
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kSfSlotBytes = kSfaBytes + kSfbBytes;
  static constexpr int kSfSlots = 4;
  static constexpr int kEpiBytes = 4 * 4096;                   // staging tiles of the four epilogue warps
  static constexpr int kBarBytes = 512;
  // Leave a few KB of the SM's shared memory unclaimed: a small CTA of another stream's kernel
  // (the gradient all-reduce: 128 threads, 32 registers, no shared memory of its own) can then
  // be resident beside this one instead of waiting for the SM.  Five or six operand stages
  // measured the same.
  static constexpr int kLeaveFree = 4096;
  // the dynamic shared memory window is declared 1024-byte aligned (checked at run time), so no slack
  static constexpr int kBudget = 227 * 1024 - kLeaveFree - kBarBytes - kEpiBytes - kSfSlots * kSfSlotBytes;
  static constexpr int kStages = kBudget / kStageBytes > 8 ? 8 : kBudget / kStageBytes;
  static constexpr int kEpi0 = kStages * kStageBytes;          // byte offsets of the regions after the stages
  static constexpr int kSfRing0 = kEpi0 + kEpiBytes;
  static constexpr int kBar0 = kSfRing0 + kSfSlots * kSfSlotBytes;
  static constexpr int kSmemBytes = kBar0 + kBarBytes;
  // tensor memory: accumulators at 0 and kAccStride, two 48-column scale-factor buffers at 416 and 464
  static constexpr int kAccStride = (kBN == 256) ? 160 : 128;
  static constexpr int kChunks = kBN / 32;
  static constexpr int kEarlyChunks = (kBN == 256) ? 3 : 0;
  static constexpr int kSfBuf0 = 416;
  static constexpr int kSfbOff = kSfChunks * 4;
  static constexpr int kSfBufStride = kSfChunks * 4 + kSfChunks * kOuterB * 4;
  static constexpr int kSfBufs = (96 / kSfBufStride) > 4 ? 4 : (96 / kSfBufStride);
  static constexpr int kSfBoxElems = kSfChunks * 64;         // 8-byte elements per scale box row
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
  static_assert(kAccStride + kBN <= kSfBuf0, "tensor memory budget");
  static_assert((2 * kStages + 2 * kSfSlots + 4 + 2 + 2 * kSched) * 8 + 8 + 4 * kSched <= 384, "barrier block (scratch words start at byte 384)");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on an mbarrier of either CTA of the pair.  What is handed over lives in tensor memory
// (ordered by the tcgen05 fences), so no cluster-scope release of ordinary memory is requested.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// tiled TMA load of a CTA pair member: data into this CTA, completion bytes to `bar` (cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc2_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}
template <int kFmt>
__device__ __forceinline__ void tc2_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate, uint32_t sfa, uint32_t sfb) {
  if (kFmt == kNvfp4) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  }
}

template <int kFmt, int kBN>
// 136 registers (no spills) instead of the 156 the compiler takes when given the whole file:
// the 13 K registers left per SM are what the gradient all-reduce kernel lives in.
__global__ void __maxnreg__(136)
gemm2_blockscaled_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                         const __grid_constant__ CUtensorMap map_psf, const __grid_constant__ CUtensorMap map_qsf,
                         const __grid_constant__ CUtensorMap map_d, const GemmParams g) {
  using C = Cfg2<kFmt, kBN>;
  extern __shared__ __align__(1024) uint8_t smem_pair[];
  uint8_t* smem_gen = smem_pair;
  const uint32_t smem_base = smem_u32(smem_pair);
  pdl_launch_dependents();   // the next kernel in the stream may set itself up under this one's tail
  if (smem_base & 1023u) {   // the swizzled tiles need the alignment the declaration asks for
    pdl_wait();
    if (threadIdx.x == 0 && g.status) atomicCAS(g.status, 0, 29);
    return;
  }

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + C::kBar0);
  const uint32_t bar_full = smem_u32(bars);                    // [kStages] operands of both CTAs landed (leader's copy is used)
  const uint32_t bar_empty = bar_full + 8 * C::kStages;        // [kStages] MMAs that read the stage are done
  const uint32_t bar_sf_land = bar_empty + 8 * C::kStages;     // [kSfSlots] this CTA's own scale tiles landed
  const uint32_t bar_sf_free = bar_sf_land + 8 * C::kSfSlots;  // [kSfSlots] the four scale warps hold the slot's bytes
  const uint32_t bar_sf_ready = bar_sf_free + 8 * C::kSfSlots; // [<=4] scale factors are in tensor memory (leader's copy)
  const uint32_t bar_tmem_full = bar_sf_ready + 32;            // [1]
  const uint32_t bar_tmem_empty = bar_tmem_full + 8;           // [1] (leader's copy is used)
  const uint32_t bar_sched_full = bar_tmem_empty + 8;          // [kSched] a tile index was published (own copy)
  const uint32_t bar_sched_empty = bar_sched_full + 8 * kSched;  // [kSched] every role of both CTAs read it (leader's copy)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 2 * C::kSfSlots + 6 + 2 * kSched);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* sched_tile = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [kSched]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = leader
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);      // the leader's producer arms it with the bytes of BOTH CTAs
      mbar_init(bar_empty + 8 * s, 1);     // one tcgen05.commit
    }
    for (int s = 0; s < C::kSfSlots; ++s) {
      mbar_init(bar_sf_land + 8 * s, 1);
      mbar_init(bar_sf_free + 8 * s, 4);
    }
    for (int b = 0; b < C::kSfBufs; ++b) mbar_init(bar_sf_ready + 8 * b, 8);   // four scale warps in each CTA
    mbar_init(bar_tmem_full, 1);
    mbar_init(bar_tmem_empty, 8);          // four epilogue warps in each CTA
    for (int q = 0; q < kSched; ++q) {
      mbar_init(bar_sched_full + 8 * q, 1);
      mbar_init(bar_sched_empty + 8 * q, kSchedReaders);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();       // barriers of both CTAs are initialised before any remote arrive
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched only this CTA pair's shared and tensor memory; from here on the
  // kernel reads its operands and the tile counter, so the predecessor has to be complete.
  pdl_wait();

  // pair tile = 256 rows x kBN columns
  const int pair_m_tiles = (g.m_tiles + 1) >> 1;
  const int num_tiles = pair_m_tiles * g.n_tiles;
  const uint32_t leader_full = mapa_u32(bar_full, 0);
  const uint32_t leader_tmem_empty = mapa_u32(bar_tmem_empty, 0);
  const uint32_t leader_sf_ready = mapa_u32(bar_sf_ready, 0);
  const uint32_t leader_sched_empty = mapa_u32(bar_sched_empty, 0);

  // Next tile of this CTA pair, for the n-th iteration of a role's tile loop (one thread per
  // role calls it): wait for the queue entry, read it, hand the entry back.  The arrive is
  // made to depend on the value read so that the entry cannot be reused before the load returned.
  auto sched_next = [&](uint32_t n, int code) -> int {
    const uint32_t q = n % kSched;
    if (!mbar_try_cluster(bar_sched_full + 8 * q, (n / kSched) & 1u) &&
        !mbar_wait_cluster(bar_sched_full + 8 * q, (n / kSched) & 1u, abort_flag, g.status, code))
      return -1;
    const int tile = sched_tile[q];
    if (tile >= -1) mbar_arrive_cluster(leader_sched_empty + 8 * q);
    return tile;
  };

  if (warp == 2) {
   if (lane == 0 && leader) {
    // ------------------------------ tile scheduler (leader CTA) ------------------------------
    // Publishes tile indices to both CTAs, a few tiles ahead of the roles that consume them:
    // drawn from the stream's device counter (clusters that start late take fewer tiles), or
    // the static round-robin order when no counter slot is given.
    const uint32_t peer_sched_full = mapa_u32(bar_sched_full, 1);
    const uint32_t peer_sched_tile = mapa_u32(smem_u32(const_cast<int*>(sched_tile)), 1);
    for (uint32_t n = 0;; ++n) {
      const uint32_t q = n % kSched;
      if (n >= (uint32_t)kSched &&
          !mbar_wait(bar_sched_empty + 8 * q, ((n / kSched) - 1u) & 1u, abort_flag, g.status, 30))
        break;
      int tile;
      if (g.sched >= 0) {
        const unsigned int t = atomicAdd(&g_gemm_sched[2 * g.sched], 1u);
        tile = t < (unsigned int)num_tiles ? (int)t : -1;
      } else {
        const int t = cluster_id + (int)n * num_clusters;
        tile = t < num_tiles ? t : -1;
      }
      sched_tile[q] = tile;
      st_shared_cluster_u32(peer_sched_tile + 4 * q, (uint32_t)tile);
      mbar_arrive(bar_sched_full + 8 * q);
      mbar_arrive_release_cluster(peer_sched_full + 8 * q);
      if (tile < 0) {
        if (g.sched >= 0) {   // the last cluster to run dry zeroes the counters for the next launch
          const unsigned int d = atomicAdd(&g_gemm_sched[2 * g.sched + 1], 1u);
          if (d == (unsigned int)num_clusters - 1u) {
            atomicExch(&g_gemm_sched[2 * g.sched], 0u);
            atomicExch(&g_gemm_sched[2 * g.sched + 1], 0u);
          }
        }
        break;
      }
    }
   }
   __syncwarp();
  } else if (warp == 0) {
   if (lane == 0) {
    // ------------------------------ operand producer (both CTAs) ------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (uint32_t tn = 0; ok; ++tn) {
      const int tile = sched_next(tn, 31);
      if (tile < 0) break;
      const int pm = tile / g.n_tiles, n_idx = tile % g.n_tiles;
      const int row_p = (pm * 2 + (int)rank) * kBM;           // this CTA's 128-row tile of P
      const int row_q = n_idx * kBN + (int)rank * (kBN / 2);  // this CTA's half of the Q rows
      for (int ks = 0; ks < g.k_stages; ++ks) {
        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, g.status, 21)) { ok = false; break; }
        const uint32_t a_s = smem_base + stage * C::kStageBytes;
        const uint32_t b_s = a_s + C::kABytes;
        const uint32_t bar = leader_full + 8 * stage;
        // Only the leader arms the barrier, with the bytes both CTAs are about to load; the
        // other CTA's copies simply complete on it (its arrival count keeps the phase open).
        if (leader) mbar_expect_tx(bar_full + 8 * stage, 2u * (uint32_t)C::kStageBytes);
        tma_load_2d_pair(a_s, &map_p, bar, ks * 128, row_p);
        tma_load_2d_pair(b_s, &map_q, bar, ks * 128, row_q);
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (*abort_flag) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {}
    }
   }
   __syncwarp();
  } else if (warp == 3) {
   if (lane == 0) {
    // ------------------------------ scale-tile producer (both CTAs) ------------------------------
    int slot = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (uint32_t tn = 0; ok; ++tn) {
      const int tile = sched_next(tn, 32);
      if (tile < 0) break;
      const int pm = tile / g.n_tiles, n_idx = tile % g.n_tiles;
      const int m_tile = pm * 2 + (int)rank;
      for (int ks = 0; ks < g.k_stages; ++ks) {
        if (!mbar_wait(bar_sf_free + 8 * slot, phase ^ 1u, abort_flag, g.status, 28)) { ok = false; break; }
        const uint32_t sfa_s = smem_base + C::kSfRing0 + slot * C::kSfSlotBytes;
        const uint32_t sfb_s = sfa_s + C::kSfaBytes;
        const uint32_t sbar = bar_sf_land + 8 * slot;
        mbar_expect_tx(sbar, (uint32_t)C::kSfSlotBytes);
        tma_load_2d(sfa_s, &map_psf, sbar, ks * C::kSfBoxElems, m_tile);
#pragma unroll
        for (int o = 0; o < C::kOuterB; ++o) {
          tma_load_2d(sfb_s + o * C::kSfaBytes, &map_qsf, sbar, ks * C::kSfBoxElems, n_idx * C::kOuterB + o);
        }
        if (++slot == C::kSfSlots) { slot = 0; phase ^= 1u; }
      }
    }
    if (*abort_flag) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {}
    }
   }
   __syncwarp();
  } else if (warp == 1) {
   if (lane == 0 && leader) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    const uint32_t idesc = (make_idesc<kFmt, kBN>() & ~(0x1Fu << 24)) | ((uint32_t)(256 >> 4) << 24);  // M = 256
    const uint32_t peer_empty = mapa_u32(bar_empty, 1), peer_tmem_full = mapa_u32(bar_tmem_full, 1);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t k = 0;          // stages issued so far; selects the scale-factor buffer
    int it = 0;
    bool ok = true;
    for (; ok; ++it) {
      if (sched_next((uint32_t)it, 33) < 0) break;
      if (it > 0) {
        if (!mbar_wait(bar_tmem_empty, (uint32_t)((it - 1) & 1), abort_flag, g.status, 22)) { ok = false; break; }
        tc_fence_after();
      }
      const uint32_t acc = tmem_base + (uint32_t)((it & 1) * C::kAccStride);
      for (int ks = 0; ks < g.k_stages; ++ks, ++k) {
        if (!mbar_wait(bar_sf_ready + 8 * (k % C::kSfBufs), (k / C::kSfBufs) & 1u, abort_flag, g.status, 25)) { ok = false; break; }
        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, g.status, 23)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_lo = ((smem_base + stage * C::kStageBytes) & 0x3FFFFu) >> 4;
        const uint32_t b_lo = a_lo + (C::kABytes >> 4);
        const uint32_t sfa_t = tmem_base + C::kSfBuf0 + (k % C::kSfBufs) * C::kSfBufStride;
        const uint32_t sfb_t = sfa_t + C::kSfbOff;
        const uint32_t first = ks > 0 ? 1u : 0u;
        // K beyond the matrix is zero codes times zero scales, so every stage issues all four MMAs.
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (kFmt == kNvfp4) {
            tc2_mma<kFmt>(acc, make_desc(a_lo + 2 * j, kDescHiOperand), make_desc(b_lo + 2 * j, kDescHiOperand), idesc,
                          j == 0 ? first : 1u, sfa_t + j * 4, sfb_t + j * (kBN / 32));
          } else {
            tc2_mma<kFmt>(acc, make_desc(a_lo + 2 * j, kDescHiOperand), make_desc(b_lo + 2 * j, kDescHiOperand),
                          idesc | ((uint32_t)j << 29) | ((uint32_t)j << 4), j == 0 ? first : 1u, sfa_t, sfb_t);
          }
        }
        tc2_commit(bar_empty + 8 * stage);     // frees the stage (and its scale-factor buffer) in this CTA ...
        tc2_commit(peer_empty + 8 * stage);    // ... and in the other one
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
      if (ok) {
        tc2_commit(bar_tmem_full);
        tc2_commit(peer_tmem_full);
      }
    }
   }
   __syncwarp();
  } else if (warp >= 8) {
    // ------------------------------ scale-factor warps (both CTAs) ------------------------------
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t sf_scratch = bar_full + 384 + 4 * (warp & 3);   // unused tail of the barrier block
    uint32_t k = 0;
    bool ok = true;
    for (uint32_t tn = 0; ok; ++tn) {
      int tile = 0;
      if (lane == 0) tile = sched_next(tn, 34);
      tile = __shfl_sync(0xFFFFFFFFu, tile, 0);
      if (tile < 0) break;
      for (int ks = 0; ks < g.k_stages; ++ks, ++k) {
        const uint32_t slot = k % C::kSfSlots, use = k / C::kSfSlots;
        if (!mbar_wait(bar_sf_land + 8 * slot, use & 1u, abort_flag, g.status, 26)) { ok = false; break; }
        const uint8_t* sfa_s = smem_gen + C::kSfRing0 + slot * C::kSfSlotBytes;
        const uint8_t* sfb_s = sfa_s + C::kSfaBytes;
        uint32_t va[C::kSfChunks * 4], vb[C::kSfChunks * C::kOuterB * 4];
#pragma unroll
        for (int c = 0; c < C::kSfChunks; ++c) {
          const uint4 v = *reinterpret_cast<const uint4*>(sfa_s + c * 512 + lane * 16);
          va[4 * c] = v.x; va[4 * c + 1] = v.y; va[4 * c + 2] = v.z; va[4 * c + 3] = v.w;
#pragma unroll
          for (int o = 0; o < C::kOuterB; ++o) {
            const uint4 u = *reinterpret_cast<const uint4*>(sfb_s + (o * C::kSfChunks + c) * 512 + lane * 16);
            const int j = (c * C::kOuterB + o) * 4;
            vb[j] = u.x; vb[j + 1] = u.y; vb[j + 2] = u.z; vb[j + 3] = u.w;
          }
        }
        // The slot is handed back before the registers are used, so "the loads have returned" has
        // to be made explicit: every lane stores a word that depends on each of its loads, and
        // the arrive (a release, after the warp barrier) cannot pass those stores.  Without this
        // the refill of the slot raced with loads still in flight.
        {
          uint32_t dep = 0;
#pragma unroll
          for (int c = 0; c < C::kSfChunks; ++c) dep ^= va[4 * c + 3];
#pragma unroll
          for (int j = 0; j < C::kSfChunks * C::kOuterB; ++j) dep ^= vb[4 * j + 3];
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(sf_scratch), "r"(dep) : "memory");
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sf_free + 8 * slot);   // the slot may be refilled
        if (k >= (uint32_t)C::kSfBufs) {   // the MMAs that last read this scale-factor buffer are done
          const uint32_t j = k - C::kSfBufs;
          if (!mbar_wait(bar_empty + 8 * (j % C::kStages), (j / C::kStages) & 1u, abort_flag, g.status, 27)) { ok = false; break; }
        }
        __syncwarp();   // lanes leave the polling loop at different times; tcgen05.st needs the whole warp
        tc_fence_after();
        const uint32_t sfa_t = tmem_base + lane_sel + C::kSfBuf0 + (k % C::kSfBufs) * C::kSfBufStride;
        const uint32_t sfb_t = sfa_t + C::kSfbOff;
        tc_st_n<C::kSfChunks * 4>(sfa_t, va);
        tc_st_n<C::kSfChunks * C::kOuterB * 4>(sfb_t, vb);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_sf_ready + 8 * (k % C::kSfBufs));
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int quad = warp & 3;
    uint8_t* epi_buf = smem_gen + C::kEpi0 + quad * 4096;
    uint32_t n_emit = 0;
    int it = 0;
    for (;; ++it) {
      int tile = 0;
      if (lane == 0) tile = sched_next((uint32_t)it, 35);
      tile = __shfl_sync(0xFFFFFFFFu, tile, 0);
      if (tile < 0) break;
      const int pm = tile / g.n_tiles, n_idx = tile % g.n_tiles;
      int ok = 1;
      if (lane == 0) ok = mbar_wait(bar_tmem_full, (uint32_t)(it & 1), abort_flag, g.status, 24) ? 1 : 0;
      ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)((it & 1) * C::kAccStride);
      const int row0 = (pm * 2 + (int)rank) * kBM + quad * 32;
      const int row = row0 + lane;
      const bool row_ok = row < g.rows;
      const int col_base = n_idx * kBN;
      auto put = [&](int col0, const uint32_t (&r)[32]) {
        if (g.tma_ok) emit_chunk(g, &map_d, epi_buf, n_emit, lane, row0, col0, r);
        else store_chunk(g, row, row_ok, col0, r);
      };
      if (kBN == 256) {
        // The columns the other accumulator overlaps go to registers first; then the MMA warp
        // may start the next tile.
        const int e0 = (it & 1) == 0 ? C::kChunks - C::kEarlyChunks : 0;
        uint32_t early[3][32];
#pragma unroll
        for (int e = 0; e < 3; ++e) tc_ld32(acc + (uint32_t)((e0 + e) * 32), early[e]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_tmem_empty);
#pragma unroll
        for (int e = 0; e < 3; ++e) put(col_base + (e0 + e) * 32, early[e]);
        const int r0 = (it & 1) == 0 ? 0 : C::kEarlyChunks;
#pragma unroll 1
        for (int ci = 0; ci < C::kChunks - C::kEarlyChunks; ++ci) {
          uint32_t r[32];
          tc_ld32(acc + (uint32_t)((r0 + ci) * 32), r);
          tc_wait_ld();
          put(col_base + (r0 + ci) * 32, r);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < C::kChunks; ++c) {
          uint32_t r[32];
          tc_ld32(acc + (uint32_t)(c * 32), r);
          tc_wait_ld();
          if (c == C::kChunks - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_tmem_empty);
          }
          put(col_base + c * 32, r);
        }
      }
    }
    if (lane == 0) bulk_wait_all<0>();   // staged tiles are read and written out before shared memory goes away
    __syncwarp();
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // the other CTA no longer signals into this one's shared memory
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

// ------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------
// K-major byte matrix [outer, kbytes] -> tensor map with a {128 bytes, box_rows} box, 128-byte swizzle.
int make_operand_map(CUtensorMap* map, const void* base, int64_t outer, int64_t kbytes, int box_rows) {
  return encode_tensor_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, base, (uint64_t)kbytes, (uint64_t)outer,
                              (uint64_t)kbytes, 128u, (uint32_t)box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
}

// Scale buffer (128x4 tile layout) as a 2-D matrix of 8-byte words: one row per 128-row band,
// 64 words per 512-byte tile.  A box of `box_words` words is the scale data of one K stage.
int make_sf_map(CUtensorMap* map, const void* base, int64_t outer, int64_t ntx, int box_words) {
  return encode_tensor_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, base, (uint64_t)ntx * 64,
                              (uint64_t)ceil_div(outer, 128), (uint64_t)ntx * 512, (uint32_t)box_words, 1u,
                              CU_TENSOR_MAP_SWIZZLE_NONE);
}

template <int kFmt, int kBN>
int launch_gemm(const void* p_codes, const void* q_codes, const GemmParams& g0, int64_t kbytes, cudaStream_t stream) {
  using C = Cfg<kFmt, kBN>;
  GemmParams g = g0;
  g.n_tiles = (int)ceil_div(g.cols, kBN);
  CUtensorMap map_p, map_q, map_psf, map_qsf;
  int rc = make_operand_map(&map_p, p_codes, g.rows, kbytes, kBM);
  if (rc != FP4T_OK) return rc;
  rc = make_operand_map(&map_q, q_codes, g.cols, kbytes, kBN);
  if (rc != FP4T_OK) return rc;
  rc = make_sf_map(&map_psf, g.p_sf, g.rows, g.ntx, C::kSfBoxElems);
  if (rc != FP4T_OK) return rc;
  rc = make_sf_map(&map_qsf, g.q_sf, g.cols, g.ntx, C::kSfBoxElems);
  if (rc != FP4T_OK) return rc;
  auto kern = gemm_blockscaled_kernel<kFmt, kBN>;
  FP4T_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
  const int sms = sm_count();
  const int tiles = g.m_tiles * g.n_tiles;
  const int grid = tiles < sms ? tiles : sms;
  kern<<<grid, kGemm1Threads, C::kSmemBytes, stream>>>(map_p, map_q, map_psf, map_qsf, g);
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}

template <int kFmt, int kBN>
int max_clusters() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    using C = Cfg2<kFmt, kBN>;
    auto kern = gemm2_blockscaled_kernel<kFmt, kBN>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess) {
      cached[dev] = -1;
      return -1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 148, 1, 1);
    cfg.blockDim = dim3(kGemm2Threads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = -1;
    }
    cached[dev] = n;
  }
  return cached[dev];
}

template <int kFmt, int kBN>
int launch_gemm2(const void* p_codes, const void* q_codes, const GemmParams& g0, int64_t kbytes, int clusters,
                 cudaStream_t stream) {
  using C = Cfg2<kFmt, kBN>;
  GemmParams g = g0;
  g.n_tiles = (int)ceil_div(g.cols, kBN);
  CUtensorMap map_p, map_q, map_psf, map_qsf;
  int rc = make_operand_map(&map_p, p_codes, g.rows, kbytes, kBM);
  if (rc != FP4T_OK) return rc;
  rc = make_operand_map(&map_q, q_codes, g.cols, kbytes, kBN / 2);
  if (rc != FP4T_OK) return rc;
  rc = make_sf_map(&map_psf, g.p_sf, g.rows, g.ntx, C::kSfBoxElems);
  if (rc != FP4T_OK) return rc;
  rc = make_sf_map(&map_qsf, g.q_sf, g.cols, g.ntx, C::kSfBoxElems);
  if (rc != FP4T_OK) return rc;
  CUtensorMap map_d = {};
  if (g.tma_ok) {   // 32 x 32 element boxes; the swizzle width equals the box row (64 B bf16, 128 B fp32)
    rc = encode_tensor_map_2d(&map_d, g.out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                              g.d, (uint64_t)g.cols, (uint64_t)g.rows, (uint64_t)g.ldd * (g.out_f32 ? 4 : 2), 32u, 32u,
                              g.out_f32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc != FP4T_OK) return rc;
  }
  const int pair_tiles = ((g.m_tiles + 1) / 2) * g.n_tiles;
  const int lim = sm_limit();
  if (lim > 0 && lim / 2 < clusters) clusters = lim / 2 > 0 ? lim / 2 : 1;
  const int nclusters = pair_tiles < clusters ? pair_tiles : clusters;
  auto kern = gemm2_blockscaled_kernel<kFmt, kBN>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * nclusters, 1, 1);
  cfg.blockDim = dim3(kGemm2Threads, 1, 1);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  pdl_attribute(&attr[1]);
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  FP4T_CUDA(cudaLaunchKernelEx(&cfg, kern, map_p, map_q, map_psf, map_qsf, map_d, g));
  return FP4T_OK;
}

template <int kFmt>
int gemm_dispatch(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf, const void* bias,
                  void* d, int d_dtype, int64_t ldd, int64_t rows, int64_t cols, int64_t k, int32_t* status,
                  cudaStream_t stream) {
  const char* name = kFmt == kNvfp4 ? "fp4t_gemm_nvfp4" : "fp4t_gemm_mxfp8";
  constexpr int kBlk = kFmt == kNvfp4 ? 16 : 32;
  FP4T_REQUIRE(p_codes && p_sf && q_codes && q_sf && d, "%s: null pointer", name);
  FP4T_REQUIRE(d_dtype == FP4T_DT_BF16 || d_dtype == FP4T_DT_F32, "%s: output dtype must be bf16 or f32", name);
  FP4T_REQUIRE(rows >= 0 && cols >= 0 && k > 0, "%s: bad shape rows=%lld cols=%lld k=%lld", name, (long long)rows,
               (long long)cols, (long long)k);
  FP4T_REQUIRE(rows < (1ll << 31) && cols < (1ll << 31) && k < (1ll << 31), "%s: dimension exceeds 2^31", name);
  FP4T_REQUIRE(ldd >= cols, "%s: ldd (%lld) < cols (%lld)", name, (long long)ldd, (long long)cols);
  if (kFmt == kNvfp4) FP4T_REQUIRE(k % 32 == 0, "%s: K must be a multiple of 32 (K=%lld)", name, (long long)k);
  else FP4T_REQUIRE(k % 16 == 0, "%s: K must be a multiple of 16 (K=%lld)", name, (long long)k);
  FP4T_REQUIRE(reinterpret_cast<uintptr_t>(p_codes) % 16 == 0 && reinterpret_cast<uintptr_t>(q_codes) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(p_sf) % 16 == 0 && reinterpret_cast<uintptr_t>(q_sf) % 16 == 0,
               "%s: code and scale pointers must be 16-byte aligned", name);
  if (rows == 0 || cols == 0) return FP4T_OK;
  const int sms = sm_count();
  if (sms < 0) {
    set_error("%s: the current device is not an sm_100 part", name);
    return FP4T_ERR_DEVICE;
  }

  GemmParams g;
  g.p_sf = static_cast<const uint8_t*>(p_sf);
  g.q_sf = static_cast<const uint8_t*>(q_sf);
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.d = d;
  g.ldd = ldd;
  g.rows = (int)rows; g.cols = (int)cols; g.k = (int)k;
  const int64_t kblocks = ceil_div(k, kBlk);
  g.ntx = (int)ceil_div(kblocks, 4);
  g.q_outer = (int)ceil_div(cols, 128);
  g.m_tiles = (int)ceil_div(rows, kBM);
  const int64_t kbytes = kFmt == kNvfp4 ? k / 2 : k;
  g.k_stages = (int)ceil_div(kbytes, 128);
  g.out_f32 = d_dtype == FP4T_DT_F32;
  const int esz = g.out_f32 ? 4 : 2;
  g.vec_ok = (reinterpret_cast<uintptr_t>(d) % 16 == 0) && ((ldd * esz) % 16 == 0) &&
             (bias == nullptr || reinterpret_cast<uintptr_t>(bias) % 16 == 0);
  g.tma_ok = (reinterpret_cast<uintptr_t>(d) % 16 == 0) && ((ldd * esz) % 16 == 0);
  g.sched = sched_slot_for(stream);
  g.status = status;
  g.n_tiles = 0;

  // Two-CTA kernel whenever there are at least two 128-row tiles (FP4T_GEMM_1CTA=1 keeps the
  // one-CTA kernel, for comparisons).
  static const bool force_1cta = [] { const char* e = getenv("FP4T_GEMM_1CTA"); return e && e[0] == '1'; }();
  if (g.m_tiles >= 2 && !force_1cta) {
    const int c256 = max_clusters<kFmt, 256>(), c128 = max_clusters<kFmt, 128>();
    if (c256 > 0 && c128 > 0) {
      const int64_t pm = (g.m_tiles + 1) / 2;
      // time of a tile is set by the bytes it pulls in per K slab: 128 rows of P plus BN rows of Q
      const double k256 = (double)ceil_div(pm * ceil_div(cols, 256), c256) * (128.0 + 256.0);
      const double k128 = (double)ceil_div(pm * ceil_div(cols, 128), c128) * (128.0 + 128.0);
      if (k256 <= k128) return launch_gemm2<kFmt, 256>(p_codes, q_codes, g, kbytes, c256, stream);
      return launch_gemm2<kFmt, 128>(p_codes, q_codes, g, kbytes, c128, stream);
    }
  }
  // Tile width: fewer, wider tiles unless narrow ones fill the machine better.
  const int64_t t256 = (int64_t)g.m_tiles * ceil_div(cols, 256), t128 = (int64_t)g.m_tiles * ceil_div(cols, 128);
  const double cost256 = (double)ceil_div(t256, sms) * (128.0 + 256.0);
  const double cost128 = (double)ceil_div(t128, sms) * (128.0 + 128.0);
  if (cost256 <= cost128) return launch_gemm<kFmt, 256>(p_codes, q_codes, g, kbytes, stream);
  return launch_gemm<kFmt, 128>(p_codes, q_codes, g, kbytes, stream);
}

}  // namespace

FP4T_DEFINE_WAIT_TIMEOUT_SETTER(set_wait_timeout_gemm)

int reset_gemm_tile_counters(cudaStream_t stream) {
  void* addr = nullptr;
  FP4T_CUDA(cudaGetSymbolAddress(&addr, g_gemm_sched));
  FP4T_CUDA(cudaMemsetAsync(addr, 0, sizeof(unsigned int) * 2 * kSchedSlots, stream));
  return FP4T_OK;
}
}  // namespace fp4t

extern "C" int fp4t_gemm_nvfp4(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                               const void* bias_bf16, void* d, int d_dtype, int64_t ldd, int64_t rows,
                               int64_t cols, int64_t k, int32_t* status, fp4t_stream_t stream) {
  return fp4t::gemm_dispatch<fp4t::kNvfp4>(p_codes, p_sf, q_codes, q_sf, bias_bf16, d, d_dtype, ldd, rows, cols, k,
                                           status, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int fp4t_gemm_mxfp8(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                               const void* bias_bf16, void* d, int d_dtype, int64_t ldd, int64_t rows,
                               int64_t cols, int64_t k, int32_t* status, fp4t_stream_t stream) {
  return fp4t::gemm_dispatch<fp4t::kMxfp8>(p_codes, p_sf, q_codes, q_sf, bias_bf16, d, d_dtype, ldd, rows, cols, k,
                                           status, reinterpret_cast<cudaStream_t>(stream));
}
