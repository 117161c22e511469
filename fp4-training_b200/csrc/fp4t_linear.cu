// One-call forward and backward of a quantized linear layer on top of the quantizer and GEMM
// entry points: the host crosses the C ABI twice per layer and step instead of six times, and
// every intermediate (codes, scales, column-sum scratch) lives in one caller-owned workspace.
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "fp4t_common.cuh"

namespace fp4t {
namespace {

inline int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

struct Sections {
  int64_t xc, xsf, wc, wsf, xtc, xtsf, wtc, wtsf, total;      // forward workspace
};
struct BwdSections {
  int64_t gc, gsf, gtc, gtsf, colsum, splitk, splitk_bytes, total;   // backward workspace
};

inline int64_t code_bytes(int fmt, int64_t outer, int64_t k) { return fmt == 0 ? outer * (k / 2) : outer * k; }
inline int64_t sf_bytes(int fmt, int64_t outer, int64_t k) { return fp4t_sf_bytes(outer, k / (fmt == 0 ? 16 : 32)); }

Sections fwd_sections(int fmt, int64_t n, int64_t ic, int64_t oc) {
  Sections s;
  int64_t o = 0;
  s.xc = o;   o += align256(code_bytes(fmt, n, ic));
  s.xsf = o;  o += align256(sf_bytes(fmt, n, ic));
  s.wc = o;   o += align256(code_bytes(fmt, oc, ic));
  s.wsf = o;  o += align256(sf_bytes(fmt, oc, ic));
  s.xtc = o;  o += align256(code_bytes(fmt, ic, n));
  s.xtsf = o; o += align256(sf_bytes(fmt, ic, n));
  s.wtc = o;  o += align256(code_bytes(fmt, ic, oc));
  s.wtsf = o; o += align256(sf_bytes(fmt, ic, oc));
  s.total = o;
  return s;
}
BwdSections bwd_sections(int fmt, int64_t n, int64_t oc, int64_t ic) {
  BwdSections s;
  int64_t o = 0;
  s.gc = o;     o += align256(code_bytes(fmt, n, oc));
  s.gsf = o;    o += align256(sf_bytes(fmt, n, oc));
  s.gtc = o;    o += align256(code_bytes(fmt, oc, n));
  s.gtsf = o;   o += align256(sf_bytes(fmt, oc, n));
  s.colsum = o; o += align256(oc * 4);
  // fp32 slices for a split-K wgrad: dW [oc, ic] of a small layer has too few tiles for the
  // machine while its K (the batch) is long
  s.splitk_bytes = fp4t_gemm_splitk_workspace_bytes(oc, ic);
  s.splitk = o; o += align256(s.splitk_bytes);
  s.total = o;
  return s;
}

// Whether large layers run the independent halves of a call on two streams (below).  Off unless
// asked for (fp4t_set_layer_concurrency, or FP4T_CONCURRENT_LAYER=1 in the environment): it pays
// when the caller's stream has the GPU to itself (0.2470 -> 0.2432 ms per step at 8192 x 4096 x
// 4096), and it must stay off next to kernels that wait for another GPU -- the rendezvous of the
// gradient exchange: streams share a small number of hardware queues, a kernel that waits holds
// its queue, and work of the helper stream queued behind it waits with it (measured on two GPUs:
// 0.258 -> 0.300 ms per step, and runs that did not finish in time).
std::atomic<int> g_layer_concurrency{-1};
bool layer_concurrency() {
  int v = g_layer_concurrency.load(std::memory_order_relaxed);
  if (v < 0) {
    const char* e = getenv("FP4T_CONCURRENT_LAYER");
    v = (e && e[0] == '1') ? 1 : 0;
    g_layer_concurrency.store(v, std::memory_order_relaxed);
  }
  return v == 1;
}

// A helper stream and two events per (device, caller stream): dgrad runs beside wgrad (below).
struct SideLane {
  int dev;
  cudaStream_t owner;
  cudaStream_t side;
  cudaEvent_t fork, join;
};
SideLane* side_lane_for(cudaStream_t stream) {
  static std::mutex mu;
  static SideLane lanes[kSchedSlots];
  static int used = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  if (stream == cudaStreamPerThread) return nullptr;    // one handle, a different stream per host thread
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < used; ++i)
    if (lanes[i].dev == dev && lanes[i].owner == stream) return &lanes[i];
  if (used == kSchedSlots) return nullptr;
  SideLane l{dev, stream, nullptr, nullptr, nullptr};
  if (cudaStreamCreateWithFlags(&l.side, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&l.fork, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&l.join, cudaEventDisableTiming) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  lanes[used] = l;
  return &lanes[used++];
}

}  // namespace
}  // namespace fp4t

using namespace fp4t;

extern "C" int64_t fp4t_linear_workspace_bytes(int fmt, int64_t n, int64_t ic, int64_t oc) {
  if (fmt < 0 || fmt > 1 || n < 0 || ic < 0 || oc < 0) return -1;
  return fwd_sections(fmt, n, ic, oc).total;
}

extern "C" int64_t fp4t_linear_backward_workspace_bytes(int fmt, int64_t n, int64_t oc, int64_t ic) {
  if (fmt < 0 || fmt > 1 || n < 0 || oc < 0 || ic < 0) return -1;
  return bwd_sections(fmt, n, oc, ic).total;
}

extern "C" int fp4t_linear_forward(int fmt, const void* x, int x_dtype, int64_t n, int64_t ic, int64_t ldx,
                                   const void* w, int w_dtype, int64_t oc, int64_t ldw, const void* bias_bf16,
                                   void* y, int y_dtype, int64_t ldy, void* workspace, int keep, int32_t* status,
                                   fp4t_stream_t stream) {
  FP4T_REQUIRE(fmt == 0 || fmt == 1, "fp4t_linear_forward: fmt must be 0 (NVFP4) or 1 (MXFP8)");
  FP4T_REQUIRE(x && w && y && workspace, "fp4t_linear_forward: null pointer");
  FP4T_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "fp4t_linear_forward: workspace must be 256-byte aligned");
  FP4T_REQUIRE((keep & ~3) == 0, "fp4t_linear_forward: keep is a 2-bit mask");
  const Sections s = fwd_sections(fmt, n, ic, oc);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const bool keep_wt = keep & 1, keep_xt = keep & 2;
  int rc;
  // The two quantizers are independent persistent grids, and W's ends in a partly filled wave of
  // tiles (4096 x 4096: 3.46 waves); for large layers, and with layer concurrency switched on, X's
  // runs on the helper stream beside it and takes the SMs that wave leaves idle.  The GEMM, on the
  // caller's stream, waits for both.
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  SideLane* lane = (layer_concurrency() && (double)n * (double)ic >= 1.6e7 && (double)oc * (double)ic >= 4.0e6) ? side_lane_for(cs) : nullptr;
  fp4t_stream_t xstream = stream;
  if (lane != nullptr) {
    FP4T_CUDA(cudaEventRecord(lane->fork, cs));
    FP4T_CUDA(cudaStreamWaitEvent(lane->side, lane->fork, 0));
    xstream = reinterpret_cast<fp4t_stream_t>(lane->side);
  }
  auto join = [&]() -> int {
    if (lane == nullptr) return FP4T_OK;
    FP4T_CUDA(cudaEventRecord(lane->join, lane->side));
    FP4T_CUDA(cudaStreamWaitEvent(cs, lane->join, 0));
    return FP4T_OK;
  };
  if (fmt == 0) {
    rc = fp4t_quantize_nvfp4(w, w_dtype, oc, ic, ldw, ws + s.wc, ws + s.wsf, keep_wt ? ws + s.wtc : nullptr,
                             keep_wt ? ws + s.wtsf : nullptr, FP4T_SR_NONE, nullptr, nullptr, 0, stream);
    const int rc2 = fp4t_quantize_nvfp4(x, x_dtype, n, ic, ldx, ws + s.xc, ws + s.xsf, keep_xt ? ws + s.xtc : nullptr,
                                        keep_xt ? ws + s.xtsf : nullptr, FP4T_SR_NONE, nullptr, nullptr, 0, xstream);
    const int rc3 = join();
    if (rc != FP4T_OK) return rc;
    if (rc2 != FP4T_OK) return rc2;
    if (rc3 != FP4T_OK) return rc3;
    return fp4t_gemm_nvfp4(ws + s.xc, ws + s.xsf, ws + s.wc, ws + s.wsf, bias_bf16, y, y_dtype, ldy, n, oc, ic, status,
                           stream);
  }
  rc = fp4t_quantize_mxfp8(w, w_dtype, oc, ic, ldw, ws + s.wc, ws + s.wsf, keep_wt ? ws + s.wtc : nullptr,
                           keep_wt ? ws + s.wtsf : nullptr, stream);
  const int rc2 = fp4t_quantize_mxfp8(x, x_dtype, n, ic, ldx, ws + s.xc, ws + s.xsf, keep_xt ? ws + s.xtc : nullptr,
                                      keep_xt ? ws + s.xtsf : nullptr, xstream);
  const int rc3 = join();
  if (rc != FP4T_OK) return rc;
  if (rc2 != FP4T_OK) return rc2;
  if (rc3 != FP4T_OK) return rc3;
  return fp4t_gemm_mxfp8(ws + s.xc, ws + s.xsf, ws + s.wc, ws + s.wsf, bias_bf16, y, y_dtype, ldy, n, oc, ic, status,
                         stream);
}

extern "C" int fp4t_linear_backward(int fmt, const void* g, int g_dtype, int64_t n, int64_t oc, int64_t ldg,
                                    int64_t ic, const void* fwd_workspace, void* bwd_workspace, void* dx, int64_t lddx,
                                    void* dw, int64_t lddw, void* db, int out_dtype, int sr_mode, const float* noise,
                                    const float* noise_t, uint64_t seed, int32_t* status, fp4t_stream_t stream) {
  FP4T_REQUIRE(fmt == 0 || fmt == 1, "fp4t_linear_backward: fmt must be 0 (NVFP4) or 1 (MXFP8)");
  FP4T_REQUIRE(g && fwd_workspace && bwd_workspace, "fp4t_linear_backward: null pointer");
  FP4T_REQUIRE(dx || dw || db, "fp4t_linear_backward: no output requested");
  FP4T_REQUIRE(reinterpret_cast<uintptr_t>(bwd_workspace) % 256 == 0 &&
                   reinterpret_cast<uintptr_t>(fwd_workspace) % 256 == 0,
               "fp4t_linear_backward: workspaces must be 256-byte aligned");
  const Sections f = fwd_sections(fmt, n, ic, oc);
  const BwdSections b = bwd_sections(fmt, n, oc, ic);
  const uint8_t* fw = static_cast<const uint8_t*>(fwd_workspace);
  uint8_t* bw = static_cast<uint8_t*>(bwd_workspace);
  void* gc = dx ? bw + b.gc : nullptr;
  void* gsf = dx ? bw + b.gsf : nullptr;
  void* gtc = dw ? bw + b.gtc : nullptr;
  void* gtsf = dw ? bw + b.gtsf : nullptr;
  int rc = FP4T_OK;
  if (dx || dw) {
    if (fmt == 0) {
      rc = db ? fp4t_quantize_nvfp4_bgrad(g, g_dtype, n, oc, ldg, gc, gsf, gtc, gtsf, sr_mode, noise, noise_t, seed,
                                          reinterpret_cast<float*>(bw + b.colsum), db, out_dtype, stream)
              : fp4t_quantize_nvfp4(g, g_dtype, n, oc, ldg, gc, gsf, gtc, gtsf, sr_mode, noise, noise_t, seed, stream);
    } else {
      rc = db ? fp4t_quantize_mxfp8_bgrad(g, g_dtype, n, oc, ldg, gc, gsf, gtc, gtsf,
                                          reinterpret_cast<float*>(bw + b.colsum), db, out_dtype, stream)
              : fp4t_quantize_mxfp8(g, g_dtype, n, oc, ldg, gc, gsf, gtc, gtsf, stream);
    }
    if (rc != FP4T_OK) return rc;
  } else {
    set_error("fp4t_linear_backward: a bias gradient alone is a plain column sum; request dx or dw as well");
    return FP4T_ERR_UNSUPPORTED;
  }
  auto gemm = fmt == 0 ? fp4t_gemm_nvfp4 : fp4t_gemm_mxfp8;
  auto gemm_splitk = fmt == 0 ? fp4t_gemm_nvfp4_splitk : fp4t_gemm_mxfp8_splitk;
  // dgrad and wgrad depend on the quantized dY only, not on each other.  Both are persistent
  // grids that end in a partly filled wave of tiles (wgrad of a square layer over a long batch:
  // 3.46 waves of 74 clusters), so they are put on two streams: wgrad stays on the caller's
  // stream -- its CTAs are resident first -- and dgrad's clusters take the SMs that wgrad's last
  // wave leaves idle instead of waiting for the whole grid to end.  The caller's stream waits
  // for both.  Only when layer concurrency is switched on (see layer_concurrency above).
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // small layers gain nothing from it: the fork and join cost about as much as their tails
  const bool big = (double)n * (double)oc * (double)ic >= 1.0e10;
  SideLane* lane = (dx && dw && layer_concurrency() && big) ? side_lane_for(s) : nullptr;
  if (lane != nullptr) {
    FP4T_CUDA(cudaEventRecord(lane->fork, s));
    FP4T_CUDA(cudaStreamWaitEvent(lane->side, lane->fork, 0));
    rc = gemm_splitk(gtc, gtsf, fw + f.xtc, fw + f.xtsf, nullptr, dw, out_dtype, lddw, oc, ic, n,
                     b.splitk_bytes ? bw + b.splitk : nullptr, b.splitk_bytes, status, stream);
    int rc2 = gemm(gc, gsf, fw + f.wtc, fw + f.wtsf, nullptr, dx, out_dtype, lddx, n, ic, oc, status,
                   reinterpret_cast<fp4t_stream_t>(lane->side));
    // the join is made whatever the launches returned, so that the side stream never outlives the call
    FP4T_CUDA(cudaEventRecord(lane->join, lane->side));
    FP4T_CUDA(cudaStreamWaitEvent(s, lane->join, 0));
    return rc != FP4T_OK ? rc : rc2;
  }
  if (dx) {   // dX[n, ic] = dY[n, oc] . (W^T)[ic, oc]^T
    rc = gemm(gc, gsf, fw + f.wtc, fw + f.wtsf, nullptr, dx, out_dtype, lddx, n, ic, oc, status, stream);
    if (rc != FP4T_OK) return rc;
  }
  if (dw) {   // dW[oc, ic] = (dY^T)[oc, n] . (X^T)[ic, n]^T
    rc = gemm_splitk(gtc, gtsf, fw + f.xtc, fw + f.xtsf, nullptr, dw, out_dtype, lddw, oc, ic, n,
                     b.splitk_bytes ? bw + b.splitk : nullptr, b.splitk_bytes, status, stream);
    if (rc != FP4T_OK) return rc;
  }
  return FP4T_OK;
}

extern "C" int fp4t_set_layer_concurrency(int on) {
  g_layer_concurrency.store(on ? 1 : 0, std::memory_order_relaxed);
  return FP4T_OK;
}
