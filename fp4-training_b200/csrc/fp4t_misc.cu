// Error reporting and the small byte-level operators of the C ABI: FP4 pack / unpack,
// scale-matrix re-layouts and a byte transpose.  All are HBM-bound copies with index
// arithmetic; they exist for operand forms the reference's op signatures accept and the
// fused quantizers do not already produce.
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <cstdarg>
#include <cstdio>

#include "fp4t_common.cuh"

namespace fp4t {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return FP4T_ERR_CUDA;
}

static thread_local int32_t* g_status_word = nullptr;
int32_t* current_status_word() { return g_status_word; }

static std::atomic<const uint64_t*> g_seed_word[64];
const uint64_t* seed_offset_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  return g_seed_word[dev].load(std::memory_order_relaxed);
}

static std::atomic<int> g_sm_limit{0};
int sm_limit() { return g_sm_limit.load(std::memory_order_relaxed); }

bool pdl_enabled() {
  static const bool off = [] { const char* e = getenv("FP4T_NO_PDL"); return e && e[0] == '1'; }();
  return !off;
}

int sched_slot_for(cudaStream_t stream) {
  static const bool force_static = [] { const char* e = getenv("FP4T_STATIC_TILES"); return e && e[0] == '1'; }();
  if (force_static) return -1;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return -1;
  }
  // cudaStreamPerThread is ONE handle value that stands for a different stream in every host
  // thread: grids launched through it from two threads may run at the same time and must not
  // share a counter.  (The legacy default stream, handle 0 or cudaStreamLegacy, is one stream.)
  if (stream == cudaStreamPerThread) return -1;
  if (stream == cudaStreamLegacy) stream = nullptr;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  struct Key { int dev; cudaStream_t stream; };
  static std::mutex mu;
  static Key keys[kSchedSlots];
  static int used = 0;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < used; ++i)
    if (keys[i].dev == dev && keys[i].stream == stream) return i;
  if (used == kSchedSlots) return -1;
  keys[used] = Key{dev, stream};
  return used++;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0, major = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cached[dev] = (major == 10 && n > 0) ? n : -1;
  }
  const int lim = sm_limit();
  if (cached[dev] > 0 && lim > 0 && lim < cached[dev]) return lim;
  return cached[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  }
  return fn;
}

int encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, uint64_t inner,
                         uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner, uint32_t box_outer,
                         CUtensorMapSwizzle swizzle) {
  // The encode call goes to the driver directly and needs a current context.  A thread that
  // has made no runtime call yet (e.g. an autograd worker on device 0) has none bound;
  // selecting the device it already has binds that device's primary context.
  int cur_dev = 0;
  FP4T_CUDA(cudaGetDevice(&cur_dev));
  FP4T_CUDA(cudaSetDevice(cur_dev));
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return FP4T_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  const cuuint64_t strides[1] = {(cuuint64_t)row_pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (inner=%llu outer=%llu pitch=%llu box=%ux%u)", (int)r,
              (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)row_pitch_bytes, box_inner,
              box_outer);
    return FP4T_ERR_CUDA;
  }
  return FP4T_OK;
}

namespace {

inline int grid_for(int64_t items, int threads) {
  const int64_t b = ceil_div(items, threads);
  return (int)(b > 148 * 32 ? 148 * 32 : (b < 1 ? 1 : b));
}

template <typename TIn>
__global__ void pack_e2m1_kernel(const TIn* __restrict__ v, uint8_t* __restrict__ codes, int64_t nbytes) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nbytes;
       i += (int64_t)gridDim.x * blockDim.x) {
    codes[i] = (uint8_t)cvt_e2m1x2((float)v[2 * i], (float)v[2 * i + 1]);
  }
}

__global__ void unpack_e2m1_kernel(const uint8_t* __restrict__ codes, float* __restrict__ v, int64_t nbytes) {
  const float grid[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nbytes;
       i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t b = codes[i];
    const float lo = grid[b & 7], hi = grid[(b >> 4) & 7];
    v[2 * i] = (b & 8) ? -lo : lo;
    v[2 * i + 1] = (b & 0x80) ? -hi : hi;
  }
}

// mode 0: logical [outer, inner]      -> canonical tiles
// mode 1: logical [inner, outer]      -> reference column-wise layout
// mode 2: reference column-wise bytes -> canonical tiles of the transpose
__global__ void sf_relayout_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                   int64_t outer, int64_t inner, int mode) {
  const int64_t ntx_k = (inner + 3) / 4;        // tiles along k-blocks
  const int64_t nt_o = (outer + 127) / 128;     // tiles along outer
  const int64_t total = outer * inner;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    int64_t o, i;
    if (mode == 0) { o = e / inner; i = e % inner; } else { i = e / outer; o = e % outer; }
    const int64_t canon = sf_offset(o, i, ntx_k);
    const int64_t refcol = ((i >> 2) * 32 + (o & 31)) * (nt_o * 16) + (o >> 7) * 16 + ((o & 127) >> 5) * 4 + (i & 3);
    if (mode == 0) dst[canon] = src[e];
    else if (mode == 1) dst[refcol] = src[e];
    else dst[canon] = src[refcol];
  }
}

__global__ void transpose_bytes_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                       int64_t rows, int64_t cols) {
  __shared__ uint8_t t[64][65];
  const int64_t r0 = (int64_t)blockIdx.y * 64, c0 = (int64_t)blockIdx.x * 64;
  for (int j = threadIdx.y; j < 64; j += blockDim.y) {
    const int64_t r = r0 + j, c = c0 + threadIdx.x;
    t[j][threadIdx.x] = (r < rows && c < cols) ? src[r * cols + c] : (uint8_t)0;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 64; j += blockDim.y) {
    const int64_t c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[c * rows + r] = t[threadIdx.x][j];
  }
}

int sf_relayout(const void* src, void* dst, int64_t outer, int64_t inner, int mode, cudaStream_t stream,
                const char* name) {
  FP4T_REQUIRE(src && dst, "%s: null pointer", name);
  FP4T_REQUIRE(outer >= 0 && inner >= 0, "%s: negative size", name);
  if (outer == 0 || inner == 0) return FP4T_OK;
  FP4T_CUDA(cudaMemsetAsync(dst, 0, (size_t)fp4t_sf_bytes(outer, inner), stream));
  sf_relayout_kernel<<<grid_for(outer * inner, 256), 256, 0, stream>>>(
      static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), outer, inner, mode);
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}

}  // namespace
}  // namespace fp4t

using namespace fp4t;

extern "C" const char* fp4t_last_error(void) { return fp4t::g_error; }
extern "C" int fp4t_version(void) { return 101; }

extern "C" int fp4t_reset_tile_counters(fp4t_stream_t stream) {
  int rc = fp4t::reset_gemm_tile_counters(reinterpret_cast<cudaStream_t>(stream));
  if (rc != FP4T_OK) return rc;
  return fp4t::reset_quantize_tile_counters(reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int fp4t_set_wait_timeout_ns(uint64_t ns) {
  FP4T_REQUIRE(ns >= 1000ull, "fp4t_set_wait_timeout_ns: the limit must be at least 1000 ns");
  int rc = fp4t::set_wait_timeout_gemm(ns);
  if (rc == FP4T_OK) rc = fp4t::set_wait_timeout_quantize(ns);
  if (rc == FP4T_OK) rc = fp4t::set_wait_timeout_allreduce(ns);
  return rc;
}

extern "C" int fp4t_set_sm_limit(int sms) {
  FP4T_REQUIRE(sms >= 0, "fp4t_set_sm_limit: negative limit");
  fp4t::g_sm_limit.store(sms, std::memory_order_relaxed);
  return FP4T_OK;
}

extern "C" int fp4t_set_seed_offset_word(const uint64_t* device_word) {
  int dev = 0;
  FP4T_CUDA(cudaGetDevice(&dev));
  FP4T_REQUIRE(dev >= 0 && dev < 64, "fp4t_set_seed_offset_word: device ordinal %d out of range", dev);
  FP4T_REQUIRE(reinterpret_cast<uintptr_t>(device_word) % 8 == 0, "fp4t_set_seed_offset_word: the word must be 8-byte aligned");
  fp4t::g_seed_word[dev].store(device_word, std::memory_order_relaxed);
  return FP4T_OK;
}

extern "C" int fp4t_set_status_word(int32_t* device_word) {
  fp4t::g_status_word = device_word;
  return FP4T_OK;
}

extern "C" int64_t fp4t_sf_bytes(int64_t outer, int64_t kblocks) {
  if (outer <= 0 || kblocks <= 0) return 0;
  return ceil_div(outer, 128) * ceil_div(kblocks, 4) * 512;
}

extern "C" int fp4t_pack_e2m1(const void* values, int in_dtype, void* codes, int64_t rows, int64_t cols,
                              fp4t_stream_t stream) {
  FP4T_REQUIRE(values && codes, "fp4t_pack_e2m1: null pointer");
  FP4T_REQUIRE(rows >= 0 && cols >= 0 && cols % 2 == 0, "fp4t_pack_e2m1: cols must be even (cols=%lld)", (long long)cols);
  FP4T_REQUIRE(in_dtype == FP4T_DT_F32 || in_dtype == FP4T_DT_BF16, "fp4t_pack_e2m1: bad dtype");
  const int64_t nbytes = rows * cols / 2;
  if (nbytes == 0) return FP4T_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (in_dtype == FP4T_DT_F32)
    pack_e2m1_kernel<float><<<grid_for(nbytes, 256), 256, 0, s>>>(static_cast<const float*>(values), static_cast<uint8_t*>(codes), nbytes);
  else
    pack_e2m1_kernel<__nv_bfloat16><<<grid_for(nbytes, 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(values), static_cast<uint8_t*>(codes), nbytes);
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}

extern "C" int fp4t_unpack_e2m1(const void* codes, float* values, int64_t rows, int64_t cols,
                                fp4t_stream_t stream) {
  FP4T_REQUIRE(values && codes, "fp4t_unpack_e2m1: null pointer");
  FP4T_REQUIRE(rows >= 0 && cols >= 0 && cols % 2 == 0, "fp4t_unpack_e2m1: cols must be even");
  const int64_t nbytes = rows * cols / 2;
  if (nbytes == 0) return FP4T_OK;
  unpack_e2m1_kernel<<<grid_for(nbytes, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(codes), values, nbytes);
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}

extern "C" int fp4t_swizzle_rowwise(const void* logical, void* dst, int64_t outer, int64_t inner,
                                    fp4t_stream_t stream) {
  return sf_relayout(logical, dst, outer, inner, 0, reinterpret_cast<cudaStream_t>(stream), "fp4t_swizzle_rowwise");
}
extern "C" int fp4t_swizzle_colwise(const void* logical, void* dst, int64_t inner, int64_t outer,
                                    fp4t_stream_t stream) {
  return sf_relayout(logical, dst, outer, inner, 1, reinterpret_cast<cudaStream_t>(stream), "fp4t_swizzle_colwise");
}
extern "C" int fp4t_unswizzle_colwise_to_rowwise(const void* src, void* dst, int64_t inner, int64_t outer,
                                                 fp4t_stream_t stream) {
  return sf_relayout(src, dst, outer, inner, 2, reinterpret_cast<cudaStream_t>(stream), "fp4t_unswizzle_colwise_to_rowwise");
}

extern "C" int fp4t_transpose_bytes(const void* src, void* dst, int64_t rows, int64_t cols,
                                    fp4t_stream_t stream) {
  FP4T_REQUIRE(src && dst, "fp4t_transpose_bytes: null pointer");
  FP4T_REQUIRE(rows >= 0 && cols >= 0, "fp4t_transpose_bytes: negative size");
  if (rows == 0 || cols == 0) return FP4T_OK;
  const dim3 grid((unsigned)ceil_div(cols, 64), (unsigned)ceil_div(rows, 64));
  FP4T_REQUIRE(grid.y <= 65535u, "fp4t_transpose_bytes: rows too large");
  transpose_bytes_kernel<<<grid, dim3(64, 4), 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows, cols);
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}
