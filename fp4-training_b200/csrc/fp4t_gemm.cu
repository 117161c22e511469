// Block-scaled GEMM on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
//   D[rows, cols] = P[rows, K] . Q[cols, K]^T (+ bias[cols]),  fp32 accumulate, bf16/fp32 out
//
// P and Q are K-major code matrices (NVFP4: E2M1 two per byte with UE4M3 scales per 16
// elements; MXFP8: E4M3 bytes with UE8M0 scales per 32 elements); their scale factors are
// in the 128x4 tile layout, which is exactly the 32-lane x 16-byte image that one
// `tcgen05.cp ... 32x128b.warpx4` drops into tensor memory for the MMA to consume.
//
// One persistent kernel, 256 or 384 threads, in two forms selected at compile time:
//   kCtas == 2  a cluster of two CTAs (two SMs) works on one 256 x kBN tile with cta_group::2
//               MMAs.  Each CTA holds its own 128 rows of P and HALF of the Q rows in shared
//               memory (the MMA reads both halves across the pair), so the Q traffic per SM is
//               half of what two independent CTAs would pull; the accumulator of each CTA is
//               128 lanes x kBN columns of its own tensor memory.  Used whenever the output has
//               more than 128 rows.
//   kCtas == 1  one CTA per 128 x kBN tile (outputs of at most 128 rows: the skinny shapes).
//
// Warp roles (per CTA):
//   warp 0   producer: per stage one 128-byte-of-K slab of P (128 rows) and of Q (this CTA's
//            rows) with 128-byte swizzle, plus the scale tiles of that slab (tensor maps over
//            the tile layout; K beyond the matrix reads as zero codes and zero scales, so every
//            stage is whole).  Plain tiled TMA loads, no multicast; in the pair form the loads
//            of both CTAs complete on the leader CTA's barrier, which the leader alone arms
//            with the pair's byte count.
//   warp 1   MMA issuer (leader CTA only).  The WHOLE warp runs the loop and waits on the
//            barriers; one elected lane issues, per stage, the copies of the stage's scale tiles
//            from shared memory into tensor memory (tcgen05.cp, executed by the tensor pipe in
//            order with the MMAs, so no hand-shake is needed for the scale factors), the four
//            tcgen05.mma (K = 64 FP4 / 32 FP8 elements each) and ONE tcgen05.commit that
//            releases the stage in both CTAs (multicast arrive).  Measured on B200: with the
//            loop run by a converged warp the issue keeps the tensor pipe full (512 cycles per
//            256x256x256 stage, twelve copies included); a single lane inside a divergent
//            branch, two commits and two waits per stage needs about 880 cycles.
//   warp 2   tensor-memory allocation, then the tile scheduler (leader): tile indices from the
//            stream's device counter (or the static order), published to both CTAs through a
//            small queue in shared memory.
//   warps 4-7 (4-11 for short K loops: two per lane quadrant, half of the tile's columns each)
//            epilogue: tcgen05.ld 32 lanes x 32 columns at a time, + bias, convert, swizzled
//            staging tiles in shared memory, one tiled TMA store per chunk (clipped at the
//            matrix edges; per-thread stores when base or pitch are not 16-byte aligned).  Two
//            accumulators alternate so the epilogue of tile i overlaps the main loop of tile
//            i+1; with kBN = 256 they overlap by some columns (the scale factors need the
//            rest of tensor memory), which the epilogue pulls into registers first and then
//            releases the MMA warp.
//
// Options of the same kernel: alpha on the accumulator (per-tensor operand scales), a
// block-quantizing epilogue (the output leaves as the next GEMM's row-wise operand), and a split
// of the K loop over otherwise idle clusters with fp32 partials in a workspace that a small
// kernel sums (outputs of a few tiles over a long K).
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

constexpr int kBM = 128;             // rows of P per CTA tile (the MMA M per CTA)
constexpr int kTmemCols = 512;
// Epilogue warps per CTA (a template parameter of the kernel): 4, one per tensor-memory lane
// quadrant, or 8, two per quadrant with half of a tile's columns each.  A tile with a long K loop
// hides the four-warp epilogue under the next tile's MMAs and runs 2-3 % faster without the extra
// warps resident (measured at K = 4096); a tile whose MMAs take less time than draining it (K up
// to kWideEpilogueStages stages) is bound by the epilogue and gets eight.
constexpr int kWideEpilogueStages = 8;
constexpr int gemm_threads(int epi_warps) { return 128 + 32 * epi_warps; }   // producer, MMA issuer, scheduler, an idle warp, epilogue
constexpr int kSched = 4;            // depth of the in-kernel tile queue

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
  int splits;       // > 1: split-K, split s of a tile accumulates K stages [s ks_per_split, ...) into slice s of a fp32 workspace
  int ks_per_split;
  int slice_rows;   // rows of one workspace slice (a multiple of the cluster tile height)
  int out_q;        // 0: bf16 / fp32 output; FP4T_QOUT_MXFP8 / FP4T_QOUT_NVFP4: block-quantized output
  uint8_t* d_sf;    // scale bytes of the quantized output (128x4 tile layout of logical [rows, cols / block])
  int d_ntx;        // scale tiles along the columns of the quantized output
  float alpha;      // the accumulator is multiplied by alpha before the bias (undoes per-tensor operand scales)
  int32_t* status;
};

// {next tile, clusters done} per stream slot; both are zero between launches (the last cluster
// to run dry puts them back)
__device__ unsigned int g_gemm_sched[2 * kSchedSlots];

// ------------------------------------------------------------------------------------
// tcgen05 / cluster wrappers (mbarrier / TMA wrappers live in fp4t_ptx.cuh)
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
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

// One lane of a converged warp, the same one on every call with all 32 lanes active.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t e;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(e));
  return e;
}

// Shared-memory matrix descriptors. Bits: [0,14) address>>4, [16,30) leading byte offset>>4,
// [32,46) stride byte offset>>4, [46,48) version = 1, [61,64) swizzle mode.  The low word is
// just (shared address >> 4), so stepping through a stage is one 32-bit add.
constexpr uint32_t kDescHiOperand = (1024u >> 4) | (1u << 14) | (2u << 29);  // 8-row groups 1024 B apart, 128-byte swizzle
constexpr uint32_t kDescHiScale = (128u >> 4) | (1u << 14);                  // 8-row groups 128 B apart, no swizzle
__device__ __forceinline__ uint64_t make_desc(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Instruction descriptor of the block-scaled MMA: [4,6) B scale id, [7,10) A format,
// [10,13) B format, 15/16 A/B major (0 = K), [17,23) N>>3, 23 scale format (0 UE4M3, 1 UE8M0),
// [24,29) M>>4, [29,31) A scale id.
template <int kFmt, int kBN, int kM>
__device__ __forceinline__ uint32_t make_idesc() {
  const uint32_t fmt = kFmt == kNvfp4 ? 1u /*E2M1*/ : 0u /*E4M3*/;
  const uint32_t sfmt = kFmt == kNvfp4 ? 0u : 1u;
  return (fmt << 7) | (fmt << 10) | ((uint32_t)(kBN >> 3) << 17) | (sfmt << 23) | ((uint32_t)(kM >> 4) << 24);
}

template <int kCtas>
__device__ __forceinline__ void tc_commit_all(uint32_t bar) {
  // arrives on `bar` once every tcgen05 operation this thread issued so far has completed;
  // in the pair form the same barrier offset is signalled in both CTAs with one instruction
  if (kCtas == 2) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3)
                 : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  }
}
// one 512-byte scale tile (32 lanes x 16 bytes), broadcast to the four lane quadrants of tensor memory
template <int kCtas>
__device__ __forceinline__ void tc_cp_scale_tile(uint32_t taddr, uint64_t desc) {
  if (kCtas == 2) asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
  else asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
template <int kFmt, int kCtas>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate, uint32_t sfa, uint32_t sfb) {
  if (kFmt == kNvfp4) {
    if (kCtas == 2)
      asm volatile(
          "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
          "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
          ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
          : "memory");
    else
      asm volatile(
          "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
          "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
          ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
          : "memory");
  } else {
    if (kCtas == 2)
      asm volatile(
          "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
          "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
          ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
          : "memory");
    else
      asm volatile(
          "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
          "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
          ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
          : "memory");
  }
}

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
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// remote arrive that publishes this thread's earlier shared::cluster stores
__device__ __forceinline__ void mbar_arrive_release_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
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

// Epilogue of one 32-column chunk held in registers: + bias, convert, store (16-byte vectors
// when the row pitch and the chunk allow it, element-wise at ragged edges).
__device__ __forceinline__ void store_chunk(const GemmParams& g, const int row, const bool row_ok, const int col0,
                                            const uint32_t (&r)[32]) {
  if (row_ok && col0 < g.cols) {
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (g.alpha != 1.0f) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= g.alpha;
    }
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
                                           const int lane, const int row0, const int row_store, const int col0,
                                           const uint32_t (&r)[32]) {
  // row0: first row of the chunk in the logical output (bounds); row_store: its row in the
  // tensor map (the same, or shifted into the split's workspace slice)
  if (row0 >= g.rows || col0 >= g.cols) return;   // warp-uniform
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  if (g.alpha != 1.0f) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= g.alpha;
  }
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
      tma_store_2d(map_d, smem_u32(buf), col0, row_store);
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
      tma_store_2d(map_d, smem_u32(tile), col0, row_store);
      bulk_commit();
    }
  }
  ++n_emit;
}

// Epilogue of one 32-column chunk as a block-quantized operand: the lane's 32 accumulators
// (+ bias) become one MXFP8 block (E4M3 codes, UE8M0 scale) or two NVFP4 blocks (E2M1 codes,
// UE4M3 scales), written row-major with the scales in the tile layout -- the row-wise operand
// form the next GEMM reads.  Same arithmetic as the quantizers' general (fp32-input) path:
// true divisions, E4M3 elements rounded half away from zero, E2M1 round-to-nearest-even.
__device__ __forceinline__ void quant_chunk(const GemmParams& g, const int row, const bool row_ok, const int col0,
                                            const uint32_t (&r)[32]) {
  if (!row_ok || col0 >= g.cols) return;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  if (g.alpha != 1.0f) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= g.alpha;
  }
  if (g.bias != nullptr) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] += __bfloat162float(g.bias[col0 + j]);
  }
  if (g.out_q == FP4T_QOUT_MXFP8) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
    const uint32_t sb = mx_scale_byte(amax);
    const float inv = mx_inv_scale(sb);
    uint32_t w[8];
#pragma unroll
    for (int q4 = 0; q4 < 8; ++q4) {
      w[q4] = mx_e4m3_byte<true>(v[4 * q4] * inv) | (mx_e4m3_byte<true>(v[4 * q4 + 1] * inv) << 8) |
              (mx_e4m3_byte<true>(v[4 * q4 + 2] * inv) << 16) | (mx_e4m3_byte<true>(v[4 * q4 + 3] * inv) << 24);
    }
    uint8_t* dp = static_cast<uint8_t*>(g.d) + (int64_t)row * g.ldd + col0;
    reinterpret_cast<uint4*>(dp)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(dp)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    g.d_sf[sf_offset(row, col0 >> 5, g.d_ntx)] = (uint8_t)sb;
  } else {
    uint32_t w[4];
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      float amax = 0.0f;
#pragma unroll
      for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[16 * b + j]));
      const float s = nvfp4_scale(amax);
      float y[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float t = __fdiv_rn(v[16 * b + j], s);
        y[j] = t == 0.0f ? 0.0f : t;     // sign(+-0) is 0
      }
      w[2 * b] = cvt_e2m1x8(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7]);
      w[2 * b + 1] = cvt_e2m1x8(y[8], y[9], y[10], y[11], y[12], y[13], y[14], y[15]);
      g.d_sf[sf_offset(row, (col0 >> 4) + b, g.d_ntx)] = (uint8_t)cvt_e4m3(s);
    }
    uint8_t* dp = static_cast<uint8_t*>(g.d) + (int64_t)row * g.ldd + (col0 >> 1);
    *reinterpret_cast<uint4*>(dp) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ------------------------------------------------------------------------------------
// The kernel
// ------------------------------------------------------------------------------------
template <int kFmt, int kBN, int kCtas, int kEpiWarps = 4>
struct Cfg {
  static constexpr int kSfChunks = kFmt == kNvfp4 ? 4 : 1;   // 512-byte scale tiles per 128 rows per stage
  static constexpr int kOuterB = (kBN + 127) / 128;          // 128-row scale tiles of Q per tile (a 64-column tile uses half of one)
  static constexpr int kABytes = kBM * 128;
  static constexpr int kBRows = kBN / kCtas;                 // Q rows this CTA loads
  static constexpr int kBBytes = kBRows * 128;
  static constexpr int kSfaBytes = kSfChunks * 512;
  static constexpr int kSfbBytes = kOuterB * kSfChunks * 512;  // scales of ALL kBN columns (each CTA's MMA half needs them)
  static constexpr int kLoadBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;   // bytes one CTA loads per stage
  static constexpr int kStageBytes = (kLoadBytes + 1023) / 1024 * 1024;          // operand tiles start 1024-byte aligned
  static constexpr int kSfaOff = kABytes + kBBytes;
  static constexpr int kSfbOff = kSfaOff + kSfaBytes;
  static constexpr int kEpiBytes = kEpiWarps * 4096;         // staging tiles of the epilogue warps
  static constexpr int kBarBytes = 512;
  // the dynamic shared memory window is declared 1024-byte aligned (checked at run time), so no slack
  static constexpr int kBudget = 227 * 1024 - kBarBytes - kEpiBytes;
  static constexpr int kStages = kBudget / kStageBytes > 8 ? 8 : kBudget / kStageBytes;
  static constexpr int kEpi0 = kStages * kStageBytes;        // byte offsets of the regions after the stages
  static constexpr int kBar0 = kEpi0 + kEpiBytes;
  static constexpr int kSmemBytes = kBar0 + kBarBytes;
  // Tensor memory.  The scale factors of ONE MMA take 4 columns for the 128 rows of P and 4 per
  // 128 rows of Q; the tensor pipe executes the copies into them in order with the MMAs that
  // read them, so two such sets, used alternately (per MMA for NVFP4, whose four MMAs of a stage
  // each have their own scale tile; per stage for MXFP8, whose four MMAs pick bytes of one tile),
  // are all that is needed.  They sit at the top; the accumulators at 0 and kAccStride below.
  static constexpr int kSfSetCols = 4 + 4 * kOuterB;
  static constexpr int kSfSets = 2;
  static constexpr int kSfBuf0 = kTmemCols - kSfSets * kSfSetCols;
  static constexpr int kChunks = kBN / 32;                   // 32-column epilogue chunks
  // chunks of one accumulator that the other one overlaps (drained to registers first)
  static constexpr int kEarlyChunks = (2 * kBN <= kSfBuf0) ? 0 : (2 * kBN - kSfBuf0 + 31) / 32;
  static constexpr int kAccStride = kBN - 32 * kEarlyChunks;
  static constexpr int kSfBoxElems = kSfChunks * 64;         // 8-byte elements per scale box row
  static constexpr int kSchedReaders = kCtas * (1 + kEpiWarps) + 1;  // roles that read each queue entry: per CTA the producer and the epilogue warps, + the MMA issuer in the leader
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
  static_assert(kStages >= 3, "too few stages");
  static_assert(kAccStride + kBN <= kSfBuf0, "tensor memory budget");
  static_assert(kEarlyChunks <= 3, "the early drain holds at most three chunks in registers");
  static_assert((2 * kStages + 2 + 2 * kSched) * 8 + 8 + 4 * kSched <= kBarBytes, "barrier block");
};

template <int kFmt, int kBN, int kCtas, int kEpiWarps>
__global__ void __launch_bounds__(gemm_threads(kEpiWarps), 1)
gemm_blockscaled_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                        const __grid_constant__ CUtensorMap map_psf, const __grid_constant__ CUtensorMap map_qsf,
                        const __grid_constant__ CUtensorMap map_d, const GemmParams g) {
  using C = Cfg<kFmt, kBN, kCtas, kEpiWarps>;
  constexpr bool kPair = kCtas == 2;
  extern __shared__ __align__(1024) uint8_t smem_dyn[];
  uint8_t* smem_gen = smem_dyn;
  const uint32_t smem_base = smem_u32(smem_dyn);
  pdl_launch_dependents();   // the next kernel in the stream may set itself up under this one's tail
  if (smem_base & 1023u) {   // the swizzled tiles need the alignment the declaration asks for
    pdl_wait();
    if (threadIdx.x == 0 && g.status) atomicCAS(g.status, 0, 29);
    return;
  }

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + C::kBar0);
  const uint32_t bar_full = smem_u32(bars);                    // [kStages] the stage's tiles of all CTAs landed (leader's copy is used)
  const uint32_t bar_empty = bar_full + 8 * C::kStages;        // [kStages] the MMAs that read the stage are done (own copy)
  const uint32_t bar_tmem_full = bar_empty + 8 * C::kStages;   // [1] accumulator complete (own copy)
  const uint32_t bar_tmem_empty = bar_tmem_full + 8;           // [1] accumulator drained (leader's copy is used)
  const uint32_t bar_sched_full = bar_tmem_empty + 8;          // [kSched] a tile index was published (own copy)
  const uint32_t bar_sched_empty = bar_sched_full + 8 * kSched;  // [kSched] every role read it (leader's copy)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 2 + 2 * kSched);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* sched_tile = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [kSched]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = kPair ? cluster_ctarank() : 0u;       // 0 = leader
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x / kCtas;
  const int num_clusters = gridDim.x / kCtas;

  if (threadIdx.x == 32) {   // the descriptors are kernel parameters: their fetch can run under the set-up below
    tma_prefetch_map(&map_p);
    tma_prefetch_map(&map_q);
    tma_prefetch_map(&map_psf);
    tma_prefetch_map(&map_qsf);
    if (g.tma_ok) tma_prefetch_map(&map_d);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);      // the leader's producer arms it with the bytes of ALL CTAs
      mbar_init(bar_empty + 8 * s, 1);     // one tcgen05.commit
    }
    mbar_init(bar_tmem_full, 1);
    mbar_init(bar_tmem_empty, kEpiWarps * kCtas);  // every epilogue warp of every CTA
    for (int q = 0; q < kSched; ++q) {
      mbar_init(bar_sched_full + 8 * q, 1);
      mbar_init(bar_sched_empty + 8 * q, C::kSchedReaders);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    if (kPair) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"((uint32_t)kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"((uint32_t)kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (kPair) cluster_sync_all();       // barriers of both CTAs are initialised before any remote arrive
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched only this cluster's shared and tensor memory; from here on the
  // kernel reads its operands and the tile counter, so the predecessor has to be complete.
  pdl_wait();

  // cluster tile = (128 * kCtas) rows x kBN columns
  const int pair_m_tiles = (g.m_tiles + kCtas - 1) / kCtas;
  const int num_tiles = pair_m_tiles * g.n_tiles * g.splits;   // work units: (tile, K split)
  const uint32_t leader_full = kPair ? mapa_u32(bar_full, 0) : bar_full;
  const uint32_t leader_tmem_empty = kPair ? mapa_u32(bar_tmem_empty, 0) : bar_tmem_empty;
  const uint32_t leader_sched_empty = kPair ? mapa_u32(bar_sched_empty, 0) : bar_sched_empty;

  // Next tile of this cluster, for the n-th iteration of a role's tile loop (one thread per
  // role calls it): wait for the queue entry, read it, hand the entry back.  The arrive is
  // made to depend on the value read so that the entry cannot be reused before the load returned.
  auto sched_next = [&](uint32_t n, int code) -> int {
    const uint32_t q = n % kSched;
    if (!mbar_try_cluster(bar_sched_full + 8 * q, (n / kSched) & 1u) &&
        !mbar_wait_cluster(bar_sched_full + 8 * q, (n / kSched) & 1u, abort_flag, g.status, code))
      return -1;
    const int tile = sched_tile[q];
    if (tile >= -1) {
      if (kPair) mbar_arrive_cluster(leader_sched_empty + 8 * q);
      else mbar_arrive(bar_sched_empty + 8 * q);
    }
    return tile;
  };

  if (warp == 2) {
   if (lane == 0 && leader) {
    // ------------------------------ tile scheduler (leader CTA) ------------------------------
    // Publishes tile indices a few tiles ahead of the roles that consume them: drawn from the
    // stream's device counter (clusters that start late take fewer tiles), or the static
    // round-robin order when no counter slot is given.
    const uint32_t peer_sched_full = kPair ? mapa_u32(bar_sched_full, 1) : 0u;
    const uint32_t peer_sched_tile = kPair ? mapa_u32(smem_u32(const_cast<int*>(sched_tile)), 1) : 0u;
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
      if (kPair) {
        st_shared_cluster_u32(peer_sched_tile + 4 * q, (uint32_t)tile);
        mbar_arrive(bar_sched_full + 8 * q);
        mbar_arrive_release_cluster(peer_sched_full + 8 * q);
      } else {
        mbar_arrive(bar_sched_full + 8 * q);
      }
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
    // ------------------------------ producer (every CTA) ------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (uint32_t tn = 0; ok; ++tn) {
      const int unit = sched_next(tn, 31);
      if (unit < 0) break;
      const int tile = unit / g.splits, split = unit - tile * g.splits;
      const int ks0 = split * g.ks_per_split, ks1 = min(ks0 + g.ks_per_split, g.k_stages);
      const int pm = tile / g.n_tiles, n_idx = tile % g.n_tiles;
      const int m_tile = pm * kCtas + (int)rank;              // this CTA's 128-row tile of P
      const int row_p = m_tile * kBM;
      const int row_q = n_idx * kBN + (int)rank * C::kBRows;  // this CTA's share of the Q rows
      for (int ks = ks0; ks < ks1; ++ks) {
        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, g.status, 21)) { ok = false; break; }
        const uint32_t a_s = smem_base + stage * C::kStageBytes;
        const uint32_t b_s = a_s + C::kABytes;
        const uint32_t sfa_s = a_s + C::kSfaOff;
        const uint32_t sfb_s = a_s + C::kSfbOff;
        const uint32_t bar = leader_full + 8 * stage;
        // Only the leader arms the barrier, with the bytes all CTAs are about to load; the
        // other CTA's copies simply complete on it (its arrival count keeps the phase open).
        if (leader) mbar_expect_tx(bar_full + 8 * stage, (uint32_t)(kCtas * C::kLoadBytes));
        if (kPair) {
          tma_load_2d_pair(sfa_s, &map_psf, bar, ks * C::kSfBoxElems, m_tile);
#pragma unroll
          for (int o = 0; o < C::kOuterB; ++o)
            tma_load_2d_pair(sfb_s + o * C::kSfaBytes, &map_qsf, bar, ks * C::kSfBoxElems, (n_idx * kBN) / 128 + o);
          tma_load_2d_pair(a_s, &map_p, bar, ks * 128, row_p);
          tma_load_2d_pair(b_s, &map_q, bar, ks * 128, row_q);
        } else {
          tma_load_2d(sfa_s, &map_psf, bar, ks * C::kSfBoxElems, m_tile);
#pragma unroll
          for (int o = 0; o < C::kOuterB; ++o)
            tma_load_2d(sfb_s + o * C::kSfaBytes, &map_qsf, bar, ks * C::kSfBoxElems, (n_idx * kBN) / 128 + o);
          tma_load_2d(a_s, &map_p, bar, ks * 128, row_p);
          tma_load_2d(b_s, &map_q, bar, ks * 128, row_q);
        }
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (*abort_flag) {   // let copies in flight land before shared memory is given back
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {}
    }
   }
   __syncwarp();
  } else if (warp == 1) {
   if (leader) {
    // ------------------------------ MMA issuer (leader CTA, whole warp) ------------------------------
    const uint32_t elected = elect_one();
    const uint32_t idesc = make_idesc<kFmt, kBN, kBM * kCtas>();
    int stage = 0;
    uint32_t phase = 0;
    uint32_t k = 0;          // stages issued so far
    bool ok = true;
    for (int it = 0; ok; ++it) {
      int unit = 0;
      if (lane == 0) unit = sched_next((uint32_t)it, 33);
      unit = __shfl_sync(0xFFFFFFFFu, unit, 0);
      if (unit < 0) break;
      const int tile = unit / g.splits, split = unit - tile * g.splits;
      const int ks0 = split * g.ks_per_split, ks1 = min(ks0 + g.ks_per_split, g.k_stages);
      if (it > 0) {
        ok = mbar_wait(bar_tmem_empty, (uint32_t)((it - 1) & 1), abort_flag, g.status, 22);
        if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
        tc_fence_after();
      }
      const uint32_t acc = tmem_base + (uint32_t)((it & 1) * C::kAccStride);
      // a 64-column tile starts in the middle of a 128-row scale tile of Q every other time:
      // its 32-row groups are columns 2.. of the copied tile
      const uint32_t sfb_shift = kBN < 128 ? (uint32_t)((((tile % g.n_tiles) * kBN) & 127) >> 5) : 0u;
      for (int ks = ks0; ks < ks1; ++ks, ++k) {
        ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, g.status, 23);
        if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
        tc_fence_after();
        if (elected) {
          const uint32_t a_lo = ((smem_base + stage * C::kStageBytes) & 0x3FFFFu) >> 4;
          const uint32_t b_lo = a_lo + (C::kABytes >> 4);
          const uint32_t sfa_lo = a_lo + (C::kSfaOff >> 4);
          const uint32_t sfb_lo = a_lo + (C::kSfbOff >> 4);
          const uint32_t first = ks > ks0 ? 1u : 0u;
          // Scale tile c of P's rows and tiles (o, c) of Q's rows go to the set the MMA reads.  K
          // beyond the matrix is zero codes times zero scales, so every stage issues all four MMAs.
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t set = kFmt == kNvfp4 ? (uint32_t)(j & 1) : (k & 1u);
            const uint32_t sfa_t = tmem_base + C::kSfBuf0 + set * C::kSfSetCols;
            const uint32_t sfb_t = sfa_t + 4;
            if (kFmt == kNvfp4 || j == 0) {
              const int c = kFmt == kNvfp4 ? j : 0;
              tc_cp_scale_tile<kCtas>(sfa_t, make_desc(sfa_lo + c * (512 >> 4), kDescHiScale));
#pragma unroll
              for (int o = 0; o < C::kOuterB; ++o)
                tc_cp_scale_tile<kCtas>(sfb_t + 4 * o, make_desc(sfb_lo + (o * C::kSfChunks + c) * (512 >> 4), kDescHiScale));
            }
            const uint32_t id = kFmt == kNvfp4 ? idesc : (idesc | ((uint32_t)j << 29) | ((uint32_t)j << 4));
            tc_mma<kFmt, kCtas>(acc, make_desc(a_lo + 2 * j, kDescHiOperand), make_desc(b_lo + 2 * j, kDescHiOperand), id,
                                j == 0 ? first : 1u, sfa_t, sfb_t + sfb_shift);
          }
          tc_commit_all<kCtas>(bar_empty + 8 * stage);   // frees the stage in every CTA of the cluster
        }
        __syncwarp();
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
      if (ok) {
        if (elected) tc_commit_all<kCtas>(bar_tmem_full);
        __syncwarp();
      }
    }
   }
   __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------ epilogue (every CTA) ------------------------------
    // A warp reads the 32 tensor-memory lanes of its quadrant (warp & 3); with eight warps the two
    // of a quadrant take half of the tile's 32-column chunks each.
    const int quad = warp & 3;
    constexpr int kParts = kEpiWarps / 4;
    const int half = (warp - 4) >> 2;
    constexpr int kHalf = C::kChunks / kParts;
    static_assert(kEpiWarps == 4 || kEpiWarps == 8, "one or two epilogue warps per lane quadrant");
    static_assert(C::kChunks % kParts == 0 && C::kEarlyChunks <= kHalf, "chunks split evenly over the warps of a quadrant");
    uint8_t* epi_buf = smem_gen + C::kEpi0 + (warp - 4) * 4096;
    uint32_t n_emit = 0;
    int it = 0;
    for (;; ++it) {
      int unit = 0;
      if (lane == 0) unit = sched_next((uint32_t)it, 35);
      unit = __shfl_sync(0xFFFFFFFFu, unit, 0);
      if (unit < 0) break;
      const int tile = unit / g.splits, split = unit - tile * g.splits;
      const int pm = tile / g.n_tiles, n_idx = tile % g.n_tiles;
      int ok = 1;
      if (lane == 0) ok = mbar_wait(bar_tmem_full, (uint32_t)(it & 1), abort_flag, g.status, 24) ? 1 : 0;
      ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)((it & 1) * C::kAccStride);
      const int row0 = (pm * kCtas + (int)rank) * kBM + quad * 32;
      const int row = row0 + lane;
      const bool row_ok = row < g.rows;
      const int col_base = n_idx * kBN;
      auto put = [&](int col0, const uint32_t (&r)[32]) {
        if (g.out_q) quant_chunk(g, row, row_ok, col0, r);
        else if (g.tma_ok) emit_chunk(g, &map_d, epi_buf, n_emit, lane, row0, row0 + split * g.slice_rows, col0, r);
        else store_chunk(g, row, row_ok, col0, r);
      };
      auto release = [&]() {     // the other accumulator's columns are free: the MMA warp may start the next tile
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (kPair) mbar_arrive_cluster(leader_tmem_empty);
          else mbar_arrive(bar_tmem_empty);
        }
      };
      if (C::kEarlyChunks > 0) {
        // The columns the other accumulator overlaps (the last ones of accumulator 0, the first
        // ones of accumulator 1) go to registers first, in the warps whose part holds them.  With
        // two warps per quadrant the other one signals at once: it is done with the previous tile,
        // which is all the MMA warp needs to know from it before that tile's accumulator is reused.
        constexpr int kE = C::kEarlyChunks > 0 ? C::kEarlyChunks : 1;
        const bool acc0 = (it & 1) == 0;
        const bool owner = acc0 ? half == kParts - 1 : half == 0;
        if (owner) {
          const int e0 = acc0 ? C::kChunks - kE : 0;
          uint32_t early[kE][32];
#pragma unroll
          for (int e = 0; e < kE; ++e) tc_ld32(acc + (uint32_t)((e0 + e) * 32), early[e]);
          tc_wait_ld();
          release();
#pragma unroll
          for (int e = 0; e < kE; ++e) put(col_base + (e0 + e) * 32, early[e]);
          const int r0 = acc0 ? (kParts - 1) * kHalf : kE;
#pragma unroll 1
          for (int ci = 0; ci < kHalf - kE; ++ci) {
            uint32_t r[32];
            tc_ld32(acc + (uint32_t)((r0 + ci) * 32), r);
            tc_wait_ld();
            put(col_base + (r0 + ci) * 32, r);
          }
        } else {
          release();
          const int r0 = half * kHalf;
#pragma unroll 1
          for (int ci = 0; ci < kHalf; ++ci) {
            uint32_t r[32];
            tc_ld32(acc + (uint32_t)((r0 + ci) * 32), r);
            tc_wait_ld();
            put(col_base + (r0 + ci) * 32, r);
          }
        }
      } else {
#pragma unroll 1
        for (int ci = 0; ci < kHalf; ++ci) {
          const int c = half * kHalf + ci;
          uint32_t r[32];
          tc_ld32(acc + (uint32_t)(c * 32), r);
          tc_wait_ld();
          if (ci == kHalf - 1) release();
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
  if (kPair) cluster_sync_all();      // the other CTA no longer signals into this one's shared memory
  if (warp == 2) {
    tc_fence_after();
    if (kPair)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                   : "memory");
  }
}

// Split-K finish: out[r, c] = sum over the splits' fp32 slices (+ bias[c]), in the output dtype.
__global__ void splitk_finalize_kernel(const float* __restrict__ ws, int splits, int64_t slice_elems, void* __restrict__ d,
                                       int out_f32, int64_t ldd, int rows, int cols,
                                       const __nv_bfloat16* __restrict__ bias) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = (int64_t)rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / cols), c = (int)(i - (int64_t)r * cols);
    float acc = 0.0f;
    for (int s = 0; s < splits; ++s) acc += ws[s * slice_elems + i];
    if (bias != nullptr) acc += __bfloat162float(bias[c]);
    if (out_f32) static_cast<float*>(d)[(int64_t)r * ldd + c] = acc;
    else static_cast<__nv_bfloat16*>(d)[(int64_t)r * ldd + c] = __float2bfloat16_rn(acc);
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

// Clusters of kCtas CTAs that can be resident at once (one CTA per SM), per device.
template <int kFmt, int kBN, int kCtas, int kEpiWarps = 4>
int max_clusters() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    using C = Cfg<kFmt, kBN, kCtas, kEpiWarps>;
    auto kern = gemm_blockscaled_kernel<kFmt, kBN, kCtas, kEpiWarps>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      cached[dev] = -1;
      return -1;
    }
    int n = 0;
    if (kCtas == 1) {
      n = sm_count();
    } else {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(kCtas * 148, 1, 1);
      cfg.blockDim = dim3(gemm_threads(kEpiWarps), 1, 1);
      cfg.dynamicSmemBytes = C::kSmemBytes;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = kCtas;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = -1;
      }
    }
    cached[dev] = n > 0 ? n : -1;
  }
  return cached[dev];
}

template <int kFmt, int kBN, int kCtas, int kEpiWarps>
int launch_gemm(const void* p_codes, const void* q_codes, const GemmParams& g0, int64_t kbytes, int clusters,
                cudaStream_t stream) {
  using C = Cfg<kFmt, kBN, kCtas, kEpiWarps>;
  GemmParams g = g0;
  g.n_tiles = (int)ceil_div(g.cols, kBN);
  CUtensorMap map_p, map_q, map_psf, map_qsf;
  int rc = make_operand_map(&map_p, p_codes, g.rows, kbytes, kBM);
  if (rc != FP4T_OK) return rc;
  rc = make_operand_map(&map_q, q_codes, g.cols, kbytes, C::kBRows);
  if (rc != FP4T_OK) return rc;
  rc = make_sf_map(&map_psf, g.p_sf, g.rows, g.ntx, C::kSfBoxElems);
  if (rc != FP4T_OK) return rc;
  rc = make_sf_map(&map_qsf, g.q_sf, g.cols, g.ntx, C::kSfBoxElems);
  if (rc != FP4T_OK) return rc;
  CUtensorMap map_d = {};
  if (g.tma_ok) {   // 32 x 32 element boxes; the swizzle width equals the box row (64 B bf16, 128 B fp32)
    const uint64_t d_rows = g.splits > 1 ? (uint64_t)g.splits * g.slice_rows : (uint64_t)g.rows;
    rc = encode_tensor_map_2d(&map_d, g.out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                              g.d, (uint64_t)g.cols, d_rows, (uint64_t)g.ldd * (g.out_f32 ? 4 : 2), 32u, 32u,
                              g.out_f32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc != FP4T_OK) return rc;
  }
  const int cluster_tiles = (int)ceil_div(g.m_tiles, kCtas) * g.n_tiles * g.splits;
  const int lim = sm_limit();
  if (lim > 0 && lim / kCtas < clusters) clusters = lim / kCtas > 0 ? lim / kCtas : 1;
  const int nclusters = cluster_tiles < clusters ? cluster_tiles : clusters;
  if (max_clusters<kFmt, kBN, kCtas, kEpiWarps>() <= 0) {   // also raises the kernel's shared-memory limit, once
    set_error("gemm: the kernel cannot be resident on this device");
    return FP4T_ERR_DEVICE;
  }
  auto kern = gemm_blockscaled_kernel<kFmt, kBN, kCtas, kEpiWarps>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kCtas * nclusters, 1, 1);
  cfg.blockDim = dim3(gemm_threads(kEpiWarps), 1, 1);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCtas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  pdl_attribute(&attr[1]);
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  FP4T_CUDA(cudaLaunchKernelEx(&cfg, kern, map_p, map_q, map_psf, map_qsf, map_d, g));
  return FP4T_OK;
}

// Optional split-K resources of a call: a caller-owned fp32 workspace.
struct SplitK {
  void* ws = nullptr;
  int64_t ws_bytes = 0;
};

// Launches the kernel of width kBN; with a workspace, and when the output has so few tiles that
// most SMs would idle (the wgrad of a small layer over a long batch: 192 x 192 x 25600 is ONE
// tile), the K loop is split over the idle clusters: split s of a tile writes its fp32 partial
// to slice s of the workspace and a small kernel adds the slices (+ bias) into the output.
template <int kFmt, int kBN, int kCtas>
int launch_maybe_split(const void* p_codes, const void* q_codes, const GemmParams& g, int64_t kbytes, int clusters,
                       const SplitK& sk, cudaStream_t stream) {
  const int64_t cm = ceil_div(g.m_tiles, kCtas);
  const int64_t tiles = cm * ceil_div(g.cols, kBN);
  int splits = 1;
  const int64_t slice_rows = cm * kCtas * kBM;
  if (sk.ws != nullptr && !g.out_q && tiles * 2 <= clusters && g.k_stages >= 4) {
    int64_t s = clusters / tiles;
    if (s > g.k_stages / 2) s = g.k_stages / 2;
    const int64_t slice_bytes = slice_rows * g.cols * 4;
    if (s * slice_bytes > sk.ws_bytes) s = sk.ws_bytes / slice_bytes;
    if (s >= 2) splits = (int)s;
  }
  if (splits == 1) {
    if (g.k_stages <= kWideEpilogueStages) return launch_gemm<kFmt, kBN, kCtas, 8>(p_codes, q_codes, g, kbytes, clusters, stream);
    return launch_gemm<kFmt, kBN, kCtas, 4>(p_codes, q_codes, g, kbytes, clusters, stream);
  }
  GemmParams gs = g;
  gs.ks_per_split = (int)ceil_div(g.k_stages, splits);
  gs.splits = (int)ceil_div(g.k_stages, gs.ks_per_split);     // no empty split
  gs.slice_rows = (int)slice_rows;
  gs.d = sk.ws;
  gs.ldd = g.cols;
  gs.out_f32 = 1;
  gs.bias = nullptr;
  gs.vec_ok = gs.tma_ok = (reinterpret_cast<uintptr_t>(sk.ws) % 16 == 0) && ((g.cols * 4) % 16 == 0);
  int rc = gs.ks_per_split <= kWideEpilogueStages
               ? launch_gemm<kFmt, kBN, kCtas, 8>(p_codes, q_codes, gs, kbytes, clusters, stream)
               : launch_gemm<kFmt, kBN, kCtas, 4>(p_codes, q_codes, gs, kbytes, clusters, stream);
  if (rc != FP4T_OK) return rc;
  const int64_t total = (int64_t)g.rows * g.cols;
  cudaLaunchConfig_t cfg = {};
  const int64_t blocks = ceil_div(total, 256);
  cfg.gridDim = dim3((unsigned)(blocks > 148 * 8 ? 148 * 8 : blocks), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  pdl_attribute(&attr);
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  FP4T_CUDA(cudaLaunchKernelEx(&cfg, splitk_finalize_kernel, static_cast<const float*>(sk.ws), gs.splits,
                               slice_rows * (int64_t)g.cols, g.d, g.out_f32, g.ldd, g.rows, g.cols, g.bias));
  return FP4T_OK;
}

template <int kFmt, int kCtas>
int launch_best_width(const void* p_codes, const void* q_codes, const GemmParams& g, int64_t kbytes, int64_t cols,
                      const SplitK& sk, cudaStream_t stream, const char* name) {
  const int c256 = max_clusters<kFmt, 256, kCtas>(), c128 = max_clusters<kFmt, 128, kCtas>();
  if (c256 <= 0 || c128 <= 0) {
    set_error("%s: the kernel cannot be resident on this device", name);
    return FP4T_ERR_DEVICE;
  }
  // Tile width: fewer, wider tiles unless narrow ones fill the machine better.  Relative time of
  // a tile per K slab, measured on long-K products (16384 x 128 x 8192 against 16384 x 256 x 8192,
  // one wave each: 17.2 against 19.3 us): a 128-column tile costs 0.89 of a 256-column one, not
  // the 0.67 its operand bytes suggest (the 128 rows of P and the scale tiles do not shrink).
  const int64_t cm = ceil_div(g.m_tiles, kCtas);
  const double k256 = (double)ceil_div(cm * ceil_div(cols, 256), c256) * 384.0;
  const double k128 = (double)ceil_div(cm * ceil_div(cols, 128), c128) * 342.0;
  if (kCtas == 1) {
    // skinny outputs (at most 128 rows): the whole job is streaming Q once, so what matters is
    // that every SM pulls; 64-column tiles double the number of CTAs at work
    const int c64 = max_clusters<kFmt, 64, 1>();
    const double k64 = c64 > 0 ? (double)ceil_div(cm * ceil_div(cols, 64), c64) * (128.0 + 64.0) : 1e30;
    if (k64 < k128 && k64 < k256) return launch_maybe_split<kFmt, 64, 1>(p_codes, q_codes, g, kbytes, c64, sk, stream);
  }
  if (k256 <= k128) return launch_maybe_split<kFmt, 256, kCtas>(p_codes, q_codes, g, kbytes, c256, sk, stream);
  return launch_maybe_split<kFmt, 128, kCtas>(p_codes, q_codes, g, kbytes, c128, sk, stream);
}

template <int kFmt>
int gemm_dispatch(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf, const void* bias,
                  void* d, int d_dtype, int64_t ldd, int64_t rows, int64_t cols, int64_t k, int32_t* status,
                  cudaStream_t stream, int out_q = 0, void* d_sf = nullptr, void* workspace = nullptr,
                  int64_t workspace_bytes = 0, float alpha = 1.0f, const char* name_override = nullptr) {
  const char* name = name_override ? name_override : out_q ? (kFmt == kNvfp4 ? "fp4t_gemm_nvfp4_qout" : "fp4t_gemm_mxfp8_qout")
                           : (kFmt == kNvfp4 ? "fp4t_gemm_nvfp4" : "fp4t_gemm_mxfp8");
  constexpr int kBlk = kFmt == kNvfp4 ? 16 : 32;
  FP4T_REQUIRE(p_codes && p_sf && q_codes && q_sf && d, "%s: null pointer", name);
  FP4T_REQUIRE(alpha == alpha && alpha - alpha == 0.0f, "%s: alpha must be finite", name);
  if (out_q) {
    FP4T_REQUIRE(out_q == FP4T_QOUT_MXFP8 || out_q == FP4T_QOUT_NVFP4, "%s: out_fmt must be FP4T_QOUT_MXFP8 or FP4T_QOUT_NVFP4", name);
    FP4T_REQUIRE(d_sf != nullptr, "%s: d_sf is null", name);
    FP4T_REQUIRE(cols % 32 == 0, "%s: a quantized output needs cols %% 32 == 0 (cols=%lld)", name, (long long)cols);
    FP4T_REQUIRE(reinterpret_cast<uintptr_t>(d) % 16 == 0 && ldd % 16 == 0,
                 "%s: quantized output rows must be 16-byte aligned (ldd is in bytes of codes)", name);
    d_dtype = FP4T_DT_BF16;   // unused by the quantizing epilogue
  }
  FP4T_REQUIRE(d_dtype == FP4T_DT_BF16 || d_dtype == FP4T_DT_F32, "%s: output dtype must be bf16 or f32", name);
  FP4T_REQUIRE(rows >= 0 && cols >= 0 && k > 0, "%s: bad shape rows=%lld cols=%lld k=%lld", name, (long long)rows,
               (long long)cols, (long long)k);
  FP4T_REQUIRE(rows < (1ll << 31) && cols < (1ll << 31) && k < (1ll << 31), "%s: dimension exceeds 2^31", name);
  FP4T_REQUIRE(ldd >= (out_q == FP4T_QOUT_NVFP4 ? cols / 2 : cols), "%s: ldd (%lld) too small for cols (%lld)", name,
               (long long)ldd, (long long)cols);
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
  g.splits = 1;
  g.ks_per_split = g.k_stages;
  g.slice_rows = 0;
  g.out_q = out_q;
  g.alpha = alpha;
  g.d_sf = static_cast<uint8_t*>(d_sf);
  g.d_ntx = out_q ? (int)ceil_div(cols / (out_q == FP4T_QOUT_NVFP4 ? 16 : 32), 4) : 0;
  if (out_q) {
    g.tma_ok = 0;   // the quantizing epilogue stores from registers
    // rows and column blocks that pad the scale buffer to whole tiles must read as zero
    FP4T_CUDA(cudaMemsetAsync(d_sf, 0, (size_t)fp4t_sf_bytes(rows, cols / (out_q == FP4T_QOUT_NVFP4 ? 16 : 32)), stream));
  }

  // CTA pairs whenever there are at least two 128-row tiles (FP4T_GEMM_1CTA=1 keeps the
  // single-CTA form, for comparisons).
  static const bool force_1cta = [] { const char* e = getenv("FP4T_GEMM_1CTA"); return e && e[0] == '1'; }();
  SplitK sk;
  if (workspace != nullptr && workspace_bytes > 0) {
    FP4T_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, "%s: the workspace must be 16-byte aligned", name);
    sk.ws = workspace;
    sk.ws_bytes = workspace_bytes;
  }
  if (g.m_tiles >= 2 && !force_1cta) return launch_best_width<kFmt, 2>(p_codes, q_codes, g, kbytes, cols, sk, stream, name);
  return launch_best_width<kFmt, 1>(p_codes, q_codes, g, kbytes, cols, sk, stream, name);
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

extern "C" int fp4t_gemm_nvfp4_qout(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                                    const void* bias_bf16, void* d_codes, void* d_sf, int out_fmt, int64_t ldd,
                                    int64_t rows, int64_t cols, int64_t k, int32_t* status, fp4t_stream_t stream) {
  return fp4t::gemm_dispatch<fp4t::kNvfp4>(p_codes, p_sf, q_codes, q_sf, bias_bf16, d_codes, FP4T_DT_BF16, ldd, rows, cols,
                                           k, status, reinterpret_cast<cudaStream_t>(stream), out_fmt, d_sf);
}

extern "C" int fp4t_gemm_mxfp8_qout(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                                    const void* bias_bf16, void* d_codes, void* d_sf, int out_fmt, int64_t ldd,
                                    int64_t rows, int64_t cols, int64_t k, int32_t* status, fp4t_stream_t stream) {
  return fp4t::gemm_dispatch<fp4t::kMxfp8>(p_codes, p_sf, q_codes, q_sf, bias_bf16, d_codes, FP4T_DT_BF16, ldd, rows, cols,
                                           k, status, reinterpret_cast<cudaStream_t>(stream), out_fmt, d_sf);
}

// Largest output (elements) for which a split-K workspace is worth having: beyond it the
// output's own tiles fill the machine.
static const int64_t kSplitKMaxOutput = 1ll << 21;

extern "C" int64_t fp4t_gemm_splitk_workspace_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0 || rows * cols > kSplitKMaxOutput) return 0;
  const int64_t slice = (rows + 255) / 256 * 256 * cols * 4;
  int64_t splits = (64ll << 20) / slice;          // at most 64 MiB
  if (splits > 74) splits = 74;
  return splits >= 2 ? splits * slice : 0;
}

extern "C" int fp4t_gemm_nvfp4_splitk(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                                      const void* bias_bf16, void* d, int d_dtype, int64_t ldd, int64_t rows,
                                      int64_t cols, int64_t k, void* workspace, int64_t workspace_bytes,
                                      int32_t* status, fp4t_stream_t stream) {
  return fp4t::gemm_dispatch<fp4t::kNvfp4>(p_codes, p_sf, q_codes, q_sf, bias_bf16, d, d_dtype, ldd, rows, cols, k,
                                           status, reinterpret_cast<cudaStream_t>(stream), 0, nullptr, workspace,
                                           workspace_bytes);
}

extern "C" int fp4t_gemm_mxfp8_splitk(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                                      const void* bias_bf16, void* d, int d_dtype, int64_t ldd, int64_t rows,
                                      int64_t cols, int64_t k, void* workspace, int64_t workspace_bytes,
                                      int32_t* status, fp4t_stream_t stream) {
  return fp4t::gemm_dispatch<fp4t::kMxfp8>(p_codes, p_sf, q_codes, q_sf, bias_bf16, d, d_dtype, ldd, rows, cols, k,
                                           status, reinterpret_cast<cudaStream_t>(stream), 0, nullptr, workspace,
                                           workspace_bytes);
}

extern "C" int fp4t_gemm_nvfp4_scaled(const void* p_codes, const void* p_sf, const void* q_codes, const void* q_sf,
                                      const void* bias_bf16, void* d, int d_dtype, int64_t ldd, int64_t rows,
                                      int64_t cols, int64_t k, float alpha, void* workspace, int64_t workspace_bytes,
                                      int32_t* status, fp4t_stream_t stream) {
  return fp4t::gemm_dispatch<fp4t::kNvfp4>(p_codes, p_sf, q_codes, q_sf, bias_bf16, d, d_dtype, ldd, rows, cols, k,
                                           status, reinterpret_cast<cudaStream_t>(stream), 0, nullptr, workspace,
                                           workspace_bytes, alpha, "fp4t_gemm_nvfp4_scaled");
}
