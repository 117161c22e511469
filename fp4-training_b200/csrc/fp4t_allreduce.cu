// Sum all-reduce of the weight-gradient buffer over the GPUs of one NVSwitch domain, in place,
// with the reduction done inside the switch (multimem.ld_reduce / multimem.st on the buffer's
// multicast address).  This is the data-parallel exchange step of the linear layer: in the
// reference it is torch DDP's NCCL all-reduce of `weight.grad` / `bias.grad`.
//
// The collective runs on a side stream under the next layer's (or step's) quantizers and GEMMs,
// which are persistent kernels that fill every SM.  A library all-reduce brings 16+ CTAs of
// 512-640 threads that cannot share an SM with them, so while it runs those SMs are lost to the
// compute kernels.  This kernel is built to be resident BESIDE them: 256 threads, 40 registers,
// no shared memory beyond a word, one CTA per SM, and the same shared-memory carve-out preference
// (an SM keeps one L1 / shared split while CTAs are resident; without the preference the kernel
// waited for the SM to drain).  The compute kernels leave that much of each SM unclaimed (the
// GEMM is held to 136 registers, the quantizers use 96).
//
// Two-shot: every rank owns 1/world of the buffer.  After a cross-GPU barrier (all ranks'
// gradients are complete) each rank pulls its slice through the multicast address -- the
// switch adds the `world` copies in fp32 -- and pushes the sums back through the same address,
// which writes them into every rank's buffer; a second barrier makes the sums visible
// everywhere before the kernel ends.  The barriers are per CTA (CTA b of every rank meets CTA b
// of the others), flags live in a symmetric buffer of each rank and carry an increasing epoch,
// so nothing has to be reset between calls.  Every wait is bounded (half of the library's wait
// limit: 2 s by default) and reports through the status word.
#include "fp4t_common.cuh"
#include "fp4t_ptx.cuh"

namespace fp4t {
namespace {

constexpr int kArThreads = 256;
constexpr int kArMaxWorld = 8;
constexpr int kArUnroll = 4;

struct ArParams {
  uint8_t* mc;                    // multicast address of the gradient buffer
  uint32_t* flags[kArMaxWorld];   // flag array of every rank (peer-mapped), [ctas][world] words
  int64_t n16;                    // 16-byte units in the buffer
  int rank, world;
  uint32_t epoch;
  int32_t* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const uint8_t* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_bf16x8(uint8_t* mc_addr, const uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__global__ void __launch_bounds__(kArThreads, 6)
allreduce_multimem_kernel(const ArParams p) {
  __shared__ int s_abort;
  const int b = blockIdx.x, t = threadIdx.x;
  if (t == 0) s_abort = 0;
  __syncthreads();

  // CTA b of this rank meets CTA b of every other rank: thread t announces to rank t and waits
  // for rank t's announcement.  `target` grows with every call, so stale values never match.
  auto meet = [&](uint32_t target, int code) -> bool {
    if (t < p.world) {
      st_release_sys(p.flags[t] + (size_t)b * p.world + p.rank, target);
      const uint32_t* mine = p.flags[p.rank] + (size_t)b * p.world + t;
      const uint64_t t0 = globaltimer_ns();
      const uint64_t limit = g_wait_timeout_ns >> 1;
      uint32_t spins = 0;
      while ((int32_t)(ld_acquire_sys(mine) - target) < 0) {
        __nanosleep(400);   // a warp that polls flat out takes issue slots from the compute kernel beside it
        if ((++spins & 255u) == 0u && globaltimer_ns() - t0 > limit) {
          if (p.status) atomicCAS(p.status, 0, code);
          s_abort = 1;
          break;
        }
      }
    }
    __syncthreads();
    return s_abort == 0;
  };

  if (!meet(2u * p.epoch + 1u, 41)) return;   // every rank's gradients are complete

  const int64_t per = (p.n16 + p.world - 1) / p.world;
  const int64_t lo = (int64_t)p.rank * per;
  const int64_t hi = lo + per < p.n16 ? lo + per : p.n16;
  const int64_t stride = (int64_t)gridDim.x * kArThreads;
  for (int64_t i = lo + (int64_t)b * kArThreads + t; i < hi; i += kArUnroll * stride) {
    uint4 v[kArUnroll];
#pragma unroll
    for (int u = 0; u < kArUnroll; ++u)
      if (i + u * stride < hi) v[u] = multimem_ld_reduce_bf16x8(p.mc + (i + u * stride) * 16);
#pragma unroll
    for (int u = 0; u < kArUnroll; ++u)
      if (i + u * stride < hi) multimem_st_bf16x8(p.mc + (i + u * stride) * 16, v[u]);
  }

  __threadfence_system();                     // this thread's sums are out before the CTA announces
  __syncthreads();
  meet(2u * p.epoch + 2u, 42);                // every rank's slice has reached every buffer
}

// ------------------------------------------------------------------------------------
// Pieces of the copy-engine exchange: the bulk bytes of a reduce-scatter + all-gather travel as
// peer copies on the GPU's copy engines, which take no SM from the persistent compute kernels;
// what is left for the SMs is a one-warp rendezvous between the ranks and the sum of the
// `world` partial shards (a few MB).
// ------------------------------------------------------------------------------------
constexpr int kMeetSlots = 16;
constexpr int kMeetCounterBase = 1024;   // word index of the per-slot local call counters

struct MeetParams {
  uint32_t* flags[kArMaxWorld];   // flag words of every rank (peer-mapped): [slot][world], counters from word 1024
  int rank, world, slot;
  int32_t* status;
};

// One warp.  Call k of a slot (counted in a device word, so a launch replayed from a CUDA graph
// counts on) writes k into this rank's word at every peer and waits until every peer's word
// here has reached k.  Work that precedes the launch in stream order on each rank is complete,
// and visible through peer reads, on every rank after it.
__global__ void __launch_bounds__(32, 1) rank_meet_kernel(const MeetParams p) {
  const int t = threadIdx.x;
  uint32_t target = 0;
  if (t == 0) {
    uint32_t* counter = p.flags[p.rank] + kMeetCounterBase + p.slot;
    target = *counter + 1u;
    *counter = target;
  }
  target = __shfl_sync(0xffffffffu, target, 0);
  if (t < p.world) {
    __threadfence_system();
    st_release_sys(p.flags[t] + (size_t)p.slot * kArMaxWorld + p.rank, target);
    const uint32_t* mine = p.flags[p.rank] + (size_t)p.slot * kArMaxWorld + t;
    const uint64_t t0 = globaltimer_ns();
    const uint64_t limit = g_wait_timeout_ns >> 1;
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - target) < 0) {
      __nanosleep(200);
      if ((++spins & 255u) == 0u && globaltimer_ns() - t0 > limit) {
        if (p.status) atomicCAS(p.status, 0, 43);
        break;
      }
    }
  }
}

struct SumParams {
  const uint4* src[kArMaxWorld];
  uint4* dst;
  int64_t n16;
  int n_src;
};

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    acc[2 * j] += __uint_as_float(w[j] << 16);
    acc[2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
  }
}

// dst = bf16(sum over sources in the order given, accumulated in fp32).  Four 16-byte items per
// thread and source are in flight at once: the kernel is a stream of independent loads and lives
// on memory-level parallelism.
constexpr int kSumUnroll = 4;
__global__ void __launch_bounds__(kArThreads, 4) sum_shards_kernel(const SumParams p) {
  const int64_t stride = (int64_t)gridDim.x * kArThreads;
  for (int64_t i0 = (int64_t)blockIdx.x * kArThreads + threadIdx.x; i0 < p.n16; i0 += kSumUnroll * stride) {
    float acc[kSumUnroll][8];
#pragma unroll
    for (int u = 0; u < kSumUnroll; ++u)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
#pragma unroll 2
    for (int r = 0; r < p.n_src; ++r) {
      uint4 v[kSumUnroll];
#pragma unroll
      for (int u = 0; u < kSumUnroll; ++u)
        v[u] = (i0 + u * stride < p.n16) ? __ldg(p.src[r] + i0 + u * stride) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < kSumUnroll; ++u) add_bf16x8(acc[u], v[u]);
    }
#pragma unroll
    for (int u = 0; u < kSumUnroll; ++u) {
      if (i0 + u * stride < p.n16) {
        uint4 o;
        uint32_t* ow = &o.x;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(acc[u][2 * j], acc[u][2 * j + 1]);
          ow[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        p.dst[i0 + u * stride] = o;
      }
    }
  }
}

// dst[i] = sum over the ranks of their copies of 16-byte item i of a symmetric buffer, added by
// the switch in fp32 (multimem.ld_reduce on the buffer's multicast address) and written to local
// memory: the reduce-scatter half of the exchange with 1/world of the bytes passing through SMs.
__global__ void __launch_bounds__(kArThreads, 6)
reduce_shard_multimem_kernel(const uint8_t* __restrict__ mc, uint4* __restrict__ dst, const int64_t n16) {
  const int64_t stride = (int64_t)gridDim.x * kArThreads;
  for (int64_t i = (int64_t)blockIdx.x * kArThreads + threadIdx.x; i < n16; i += kArUnroll * stride) {
    uint4 v[kArUnroll];
#pragma unroll
    for (int u = 0; u < kArUnroll; ++u)
      if (i + u * stride < n16) v[u] = multimem_ld_reduce_bf16x8(mc + (i + u * stride) * 16);
#pragma unroll
    for (int u = 0; u < kArUnroll; ++u)
      if (i + u * stride < n16) dst[i + u * stride] = v[u];
  }
}

}  // namespace

FP4T_DEFINE_WAIT_TIMEOUT_SETTER(set_wait_timeout_allreduce)
}  // namespace fp4t

extern "C" int fp4t_allreduce_sum_bf16_multimem(void* multicast_ptr, const void* const* flag_ptrs, int rank, int world,
                                                int64_t numel, uint32_t epoch, int ctas, int32_t* status,
                                                fp4t_stream_t stream) {
  using namespace fp4t;
  const char* name = "fp4t_allreduce_sum_bf16_multimem";
  FP4T_REQUIRE(multicast_ptr != nullptr && flag_ptrs != nullptr, "%s: null pointer", name);
  FP4T_REQUIRE(world >= 1 && world <= kArMaxWorld, "%s: world size %d not in 1..%d", name, world, kArMaxWorld);
  FP4T_REQUIRE(rank >= 0 && rank < world, "%s: rank %d out of range", name, rank);
  FP4T_REQUIRE(numel >= 0 && numel % 8 == 0, "%s: numel (%lld) must be a multiple of 8", name, (long long)numel);
  FP4T_REQUIRE(reinterpret_cast<uintptr_t>(multicast_ptr) % 16 == 0, "%s: buffer must be 16-byte aligned", name);
  FP4T_REQUIRE(epoch >= 1u, "%s: epoch starts at 1", name);
  FP4T_REQUIRE(ctas >= 1 && ctas <= FP4T_ALLREDUCE_MAX_CTAS, "%s: ctas %d not in 1..%d", name, ctas,
               FP4T_ALLREDUCE_MAX_CTAS);
  if (numel == 0) return FP4T_OK;
  ArParams p;
  p.mc = static_cast<uint8_t*>(multicast_ptr);
  for (int r = 0; r < kArMaxWorld; ++r) {
    p.flags[r] = r < world ? static_cast<uint32_t*>(const_cast<void*>(flag_ptrs[r])) : nullptr;
    FP4T_REQUIRE(r >= world || p.flags[r] != nullptr, "%s: flag pointer of rank %d is null", name, r);
  }
  p.n16 = numel / 8;
  p.rank = rank;
  p.world = world;
  p.epoch = epoch;
  p.status = status;
  // the same grid on every rank (CTA b meets CTA b): a function of the sizes only
  const int64_t per = (p.n16 + world - 1) / world;
  int64_t grid = (per + (int64_t)kArThreads * kArUnroll - 1) / ((int64_t)kArThreads * kArUnroll);
  if (grid > ctas) grid = ctas;
  if (grid < 1) grid = 1;
  // An SM keeps one split of its L1 / shared-memory array while it has resident CTAs.  The
  // compute kernels ask for (almost) all of it as shared memory; a kernel that preferred L1 could
  // only start on an SM after they drained, so ask for the same split.
  static const cudaError_t carve = cudaFuncSetAttribute(allreduce_multimem_kernel,
                                                        cudaFuncAttributePreferredSharedMemoryCarveout,
                                                        cudaSharedmemCarveoutMaxShared);
  FP4T_CUDA(carve);
  allreduce_multimem_kernel<<<(unsigned)grid, kArThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}

extern "C" int fp4t_rank_meet(const void* const* flag_ptrs, int rank, int world, int slot, int32_t* status,
                              fp4t_stream_t stream) {
  using namespace fp4t;
  const char* name = "fp4t_rank_meet";
  FP4T_REQUIRE(flag_ptrs != nullptr, "%s: null pointer", name);
  FP4T_REQUIRE(world >= 1 && world <= kArMaxWorld, "%s: world size %d not in 1..%d", name, world, kArMaxWorld);
  FP4T_REQUIRE(rank >= 0 && rank < world, "%s: rank %d out of range", name, rank);
  FP4T_REQUIRE(slot >= 0 && slot < kMeetSlots, "%s: slot %d not in 0..%d", name, slot, kMeetSlots - 1);
  MeetParams p;
  for (int r = 0; r < kArMaxWorld; ++r) {
    p.flags[r] = r < world ? static_cast<uint32_t*>(const_cast<void*>(flag_ptrs[r])) : nullptr;
    FP4T_REQUIRE(r >= world || p.flags[r] != nullptr, "%s: flag pointer of rank %d is null", name, r);
  }
  p.rank = rank; p.world = world; p.slot = slot; p.status = status;
  static const cudaError_t carve = cudaFuncSetAttribute(rank_meet_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                                        cudaSharedmemCarveoutMaxShared);
  FP4T_CUDA(carve);
  rank_meet_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}

extern "C" int fp4t_sum_bf16_shards(void* dst, const void* const* srcs, int n_src, int64_t numel, int ctas,
                                    fp4t_stream_t stream) {
  using namespace fp4t;
  const char* name = "fp4t_sum_bf16_shards";
  FP4T_REQUIRE(dst != nullptr && srcs != nullptr, "%s: null pointer", name);
  FP4T_REQUIRE(n_src >= 1 && n_src <= kArMaxWorld, "%s: n_src %d not in 1..%d", name, n_src, kArMaxWorld);
  FP4T_REQUIRE(numel >= 0 && numel % 8 == 0, "%s: numel (%lld) must be a multiple of 8", name, (long long)numel);
  FP4T_REQUIRE(ctas >= 1 && ctas <= FP4T_ALLREDUCE_MAX_CTAS, "%s: ctas %d not in 1..%d", name, ctas,
               FP4T_ALLREDUCE_MAX_CTAS);
  FP4T_REQUIRE(reinterpret_cast<uintptr_t>(dst) % 16 == 0, "%s: buffers must be 16-byte aligned", name);
  SumParams p;
  for (int r = 0; r < kArMaxWorld; ++r) {
    p.src[r] = r < n_src ? static_cast<const uint4*>(srcs[r]) : nullptr;
    FP4T_REQUIRE(r >= n_src || (p.src[r] != nullptr && reinterpret_cast<uintptr_t>(p.src[r]) % 16 == 0),
                 "%s: source %d is null or not 16-byte aligned", name, r);
  }
  if (numel == 0) return FP4T_OK;
  p.dst = static_cast<uint4*>(dst);
  p.n16 = numel / 8;
  p.n_src = n_src;
  int64_t grid = (p.n16 + (int64_t)kArThreads * kSumUnroll - 1) / ((int64_t)kArThreads * kSumUnroll);
  if (grid > ctas) grid = ctas;
  static const cudaError_t carve = cudaFuncSetAttribute(sum_shards_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                                        cudaSharedmemCarveoutMaxShared);
  FP4T_CUDA(carve);
  sum_shards_kernel<<<(unsigned)grid, kArThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}

extern "C" int fp4t_reduce_shard_bf16_multimem(const void* multicast_shard_ptr, void* dst, int64_t numel, int ctas,
                                               fp4t_stream_t stream) {
  using namespace fp4t;
  const char* name = "fp4t_reduce_shard_bf16_multimem";
  FP4T_REQUIRE(multicast_shard_ptr != nullptr && dst != nullptr, "%s: null pointer", name);
  FP4T_REQUIRE(numel >= 0 && numel % 8 == 0, "%s: numel (%lld) must be a multiple of 8", name, (long long)numel);
  FP4T_REQUIRE(reinterpret_cast<uintptr_t>(multicast_shard_ptr) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0,
               "%s: buffers must be 16-byte aligned", name);
  FP4T_REQUIRE(ctas >= 1 && ctas <= FP4T_ALLREDUCE_MAX_CTAS, "%s: ctas %d not in 1..%d", name, ctas,
               FP4T_ALLREDUCE_MAX_CTAS);
  if (numel == 0) return FP4T_OK;
  const int64_t n16 = numel / 8;
  int64_t grid = (n16 + (int64_t)kArThreads * kArUnroll - 1) / ((int64_t)kArThreads * kArUnroll);
  if (grid > ctas) grid = ctas;
  static const cudaError_t carve = cudaFuncSetAttribute(reduce_shard_multimem_kernel,
                                                        cudaFuncAttributePreferredSharedMemoryCarveout,
                                                        cudaSharedmemCarveoutMaxShared);
  FP4T_CUDA(carve);
  reduce_shard_multimem_kernel<<<(unsigned)grid, kArThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(multicast_shard_ptr), static_cast<uint4*>(dst), n16);
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}
