// LayerNorm in front of the quantized projections (the `preln` of the reference's attention and
// MLP blocks, models/transformer_block.py:45-52,89-93): forward with the cast to the projections'
// input dtype fused in, and a backward that produces the input gradient and the gamma / beta
// gradients in one pass over the rows.
//
// The rows are short (the embedding width, a few hundred to a thousand elements) and there are
// very many of them (batch x tokens), so both kernels give one warp to a row: the row lives in
// registers, the statistics are warp-shuffle reductions, every global access is a 16-byte
// vector, and nothing goes through shared memory except the per-CTA reduction of the parameter
// gradients.  HBM-bound by design: forward reads the row once and writes it once (fp32 -> bf16:
// 6 bytes per element), backward reads x and dy and writes dx (10-12 bytes per element).
//
// The parameter gradients are column sums over all rows.  Each warp keeps its columns' partial
// sums in registers across the rows it walks, a CTA adds its warps' partials in shared memory
// and writes one row of a [CTAs, 2, cols] workspace; a second small kernel adds those rows in a
// fixed order, so the result does not depend on scheduling.
#include "fp4t_common.cuh"

namespace fp4t {
namespace {

constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;
constexpr int kNormMaxCols = 1024;      // 8 float4 per lane

struct NormFwd {
  const void* x; int x_dtype; int64_t ldx;
  const float* gamma; const float* beta; float eps;
  void* y; int y_dtype; int64_t ldy;
  float* mean; float* rstd;
  int64_t rows; int cols;
};

struct NormBwd {
  const void* dy; int dy_dtype; int64_t lddy;
  const void* x; int x_dtype; int64_t ldx;
  const float* mean; const float* rstd; const float* gamma;
  void* dx; int64_t lddx;
  float* partial;        // [gridDim.x][2][cols]
  int64_t rows; int cols;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// four consecutive elements starting at element index e of a row
__device__ __forceinline__ float4 load4(const void* row, int dtype, int e) {
  if (dtype == FP4T_DT_F32) return __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(row) + e));
  const uint2 u = __ldg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(row) + e));
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u), __uint_as_float(u.y << 16),
                     __uint_as_float(u.y & 0xFFFF0000u));
}
__device__ __forceinline__ void store4(void* row, int dtype, int e, const float4 v) {
  if (dtype == FP4T_DT_F32) {
    *reinterpret_cast<float4*>(static_cast<float*>(row) + e) = v;
  } else {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&a);
    u.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(row) + e) = u;
  }
}

// kV: float4 chunks per lane (cols <= 128 kV)
template <int kV>
__global__ void __launch_bounds__(kNormThreads) layernorm_fwd_kernel(const NormFwd p) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kNormWarps + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kNormWarps;
  const int chunks = p.cols >> 2;
  const size_t xes = p.x_dtype == FP4T_DT_F32 ? 4 : 2, yes = p.y_dtype == FP4T_DT_F32 ? 4 : 2;
  float4 gm[kV], bt[kV];
#pragma unroll
  for (int v = 0; v < kV; ++v) {
    const int c = lane + 32 * v;
    gm[v] = c < chunks ? __ldg(reinterpret_cast<const float4*>(p.gamma) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    bt[v] = c < chunks ? __ldg(reinterpret_cast<const float4*>(p.beta) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float inv_n = 1.0f / (float)p.cols;
  for (int64_t r = warp0; r < p.rows; r += nwarps) {
    const void* xrow = static_cast<const uint8_t*>(p.x) + (size_t)r * p.ldx * xes;
    float4 x[kV];
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < kV; ++v) {
      const int c = lane + 32 * v;
      x[v] = c < chunks ? load4(xrow, p.x_dtype, 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
      s += (x[v].x + x[v].y) + (x[v].z + x[v].w);
    }
    const float mean = warp_sum(s) * inv_n;
    float q = 0.f;
#pragma unroll
    for (int v = 0; v < kV; ++v) {
      if (lane + 32 * v < chunks) {
        const float a = x[v].x - mean, b = x[v].y - mean, c = x[v].z - mean, d = x[v].w - mean;
        q += (a * a + b * b) + (c * c + d * d);
      }
    }
    const float rstd = rsqrtf(warp_sum(q) * inv_n + p.eps);
    void* yrow = static_cast<uint8_t*>(p.y) + (size_t)r * p.ldy * yes;
#pragma unroll
    for (int v = 0; v < kV; ++v) {
      const int c = lane + 32 * v;
      if (c < chunks) {
        float4 o;
        o.x = (x[v].x - mean) * rstd * gm[v].x + bt[v].x;
        o.y = (x[v].y - mean) * rstd * gm[v].y + bt[v].y;
        o.z = (x[v].z - mean) * rstd * gm[v].z + bt[v].z;
        o.w = (x[v].w - mean) * rstd * gm[v].w + bt[v].w;
        store4(yrow, p.y_dtype, 4 * c, o);
      }
    }
    if (lane == 0) {
      p.mean[r] = mean;
      p.rstd[r] = rstd;
    }
  }
}

template <int kV>
__global__ void __launch_bounds__(kNormThreads) layernorm_bwd_kernel(const NormBwd p) {
  __shared__ float red[2][128 * kV];      // the CTA's dgamma / dbeta, added warp by warp in warp order
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t warp0 = (int64_t)blockIdx.x * kNormWarps + warp;
  const int64_t nwarps = (int64_t)gridDim.x * kNormWarps;
  const int chunks = p.cols >> 2;
  const size_t xes = p.x_dtype == FP4T_DT_F32 ? 4 : 2, ges = p.dy_dtype == FP4T_DT_F32 ? 4 : 2;
  float4 gm[kV], dg[kV], db[kV];
#pragma unroll
  for (int v = 0; v < kV; ++v) {
    const int c = lane + 32 * v;
    gm[v] = c < chunks ? __ldg(reinterpret_cast<const float4*>(p.gamma) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    dg[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    db[v] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float inv_n = 1.0f / (float)p.cols;
  for (int64_t r = warp0; r < p.rows; r += nwarps) {
    const void* xrow = static_cast<const uint8_t*>(p.x) + (size_t)r * p.ldx * xes;
    const void* grow = static_cast<const uint8_t*>(p.dy) + (size_t)r * p.lddy * ges;
    const float mean = __ldg(p.mean + r), rstd = __ldg(p.rstd + r);
    float4 xh[kV], g[kV];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int v = 0; v < kV; ++v) {
      const int c = lane + 32 * v;
      if (c < chunks) {
        const float4 x = load4(xrow, p.x_dtype, 4 * c), dy = load4(grow, p.dy_dtype, 4 * c);
        xh[v] = make_float4((x.x - mean) * rstd, (x.y - mean) * rstd, (x.z - mean) * rstd, (x.w - mean) * rstd);
        g[v] = make_float4(dy.x * gm[v].x, dy.y * gm[v].y, dy.z * gm[v].z, dy.w * gm[v].w);
        s1 += (g[v].x + g[v].y) + (g[v].z + g[v].w);
        s2 += (g[v].x * xh[v].x + g[v].y * xh[v].y) + (g[v].z * xh[v].z + g[v].w * xh[v].w);
        dg[v].x += dy.x * xh[v].x; dg[v].y += dy.y * xh[v].y; dg[v].z += dy.z * xh[v].z; dg[v].w += dy.w * xh[v].w;
        db[v].x += dy.x; db[v].y += dy.y; db[v].z += dy.z; db[v].w += dy.w;
      } else {
        xh[v] = make_float4(0.f, 0.f, 0.f, 0.f);
        g[v] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    const float c1 = warp_sum(s1) * inv_n, c2 = warp_sum(s2) * inv_n;
    void* drow = static_cast<uint8_t*>(p.dx) + (size_t)r * p.lddx * xes;
#pragma unroll
    for (int v = 0; v < kV; ++v) {
      const int c = lane + 32 * v;
      if (c < chunks) {
        float4 o;
        o.x = rstd * (g[v].x - c1 - xh[v].x * c2);
        o.y = rstd * (g[v].y - c1 - xh[v].y * c2);
        o.z = rstd * (g[v].z - c1 - xh[v].z * c2);
        o.w = rstd * (g[v].w - c1 - xh[v].w * c2);
        store4(drow, p.x_dtype, 4 * c, o);
      }
    }
  }
  // this CTA's column sums: the warps add into shared memory one after the other (a fixed order),
  // then one row of the workspace is written
  for (int w = 0; w < kNormWarps; ++w) {
    if (warp == w) {
#pragma unroll
      for (int v = 0; v < kV; ++v) {
        const int c = lane + 32 * v;
        if (c < chunks) {
          float4* a = reinterpret_cast<float4*>(&red[0][4 * c]);
          float4* b = reinterpret_cast<float4*>(&red[1][4 * c]);
          if (w == 0) {
            *a = dg[v];
            *b = db[v];
          } else {
            float4 t = *a;
            t.x += dg[v].x; t.y += dg[v].y; t.z += dg[v].z; t.w += dg[v].w;
            *a = t;
            t = *b;
            t.x += db[v].x; t.y += db[v].y; t.z += db[v].z; t.w += db[v].w;
            *b = t;
          }
        }
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < 2 * p.cols; i += kNormThreads) {
    const int which = i / p.cols, c = i - which * p.cols;
    p.partial[(size_t)blockIdx.x * 2 * p.cols + i] = red[which][c];
  }
}

// dgamma[c] / dbeta[c] = sum over the CTAs' partial rows.  One CTA per 32 columns of the
// [2 cols] row; warp w adds rows w, w + 32, ... (four independent chains), then the 32 warps'
// sums are added in warp order: a fixed association, whatever the scheduling.
constexpr int kParamWarps = 32;
__global__ void __launch_bounds__(32 * kParamWarps) layernorm_param_grad_kernel(const float* __restrict__ partial, int nparts,
                                                                                int cols, float* __restrict__ dgamma,
                                                                                float* __restrict__ dbeta) {
  __shared__ float red[kParamWarps][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + lane;
  const size_t pitch = (size_t)2 * cols;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (i < 2 * cols) {
    int k = warp;
    for (; k + 3 * kParamWarps < nparts; k += 4 * kParamWarps) {
      s0 += partial[(size_t)k * pitch + i];
      s1 += partial[(size_t)(k + kParamWarps) * pitch + i];
      s2 += partial[(size_t)(k + 2 * kParamWarps) * pitch + i];
      s3 += partial[(size_t)(k + 3 * kParamWarps) * pitch + i];
    }
    for (; k < nparts; k += kParamWarps) s0 += partial[(size_t)k * pitch + i];
  }
  red[warp][lane] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (warp == 0 && i < 2 * cols) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kParamWarps; ++w) s += red[w][lane];
    if (i < cols) dgamma[i] = s;
    else dbeta[i - cols] = s;
  }
}

// One wave of CTAs: as many as are resident at once (all warps walk the rows with the same
// stride, so a second, partial wave would run at a fraction of the machine), at most 4 per SM
// to keep the number of partial parameter-gradient rows small.
template <typename Kernel>
int norm_grid(Kernel kern, int64_t rows) {
  const int sms = sm_count();
  if (sms <= 0) return -1;
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kNormThreads, 0) != cudaSuccess || occ <= 0) {
    cudaGetLastError();
    occ = 1;
  }
  if (occ > 4) occ = 4;
  const int64_t want = ceil_div(rows, kNormWarps);
  const int64_t cap = (int64_t)sms * occ;
  return (int)(want < cap ? want : cap);
}
int max_norm_grid() {
  const int sms = sm_count();
  return sms > 0 ? sms * 4 : -1;
}

int check_common(const char* name, int64_t rows, int64_t cols) {
  FP4T_REQUIRE(rows >= 0 && cols > 0, "%s: bad shape rows=%lld cols=%lld", name, (long long)rows, (long long)cols);
  FP4T_REQUIRE(cols % 4 == 0 && cols <= kNormMaxCols, "%s: cols (%lld) must be a multiple of 4, at most %d", name,
               (long long)cols, kNormMaxCols);
  return FP4T_OK;
}
bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace
}  // namespace fp4t

using namespace fp4t;

extern "C" int fp4t_layernorm_forward(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ldx, const float* gamma,
                                      const float* beta, float eps, void* y, int y_dtype, int64_t ldy, float* mean,
                                      float* rstd, fp4t_stream_t stream) {
  const char* name = "fp4t_layernorm_forward";
  int rc = check_common(name, rows, cols);
  if (rc != FP4T_OK) return rc;
  FP4T_REQUIRE(x && gamma && beta && y && mean && rstd, "%s: null pointer", name);
  FP4T_REQUIRE((x_dtype == FP4T_DT_F32 || x_dtype == FP4T_DT_BF16) && (y_dtype == FP4T_DT_F32 || y_dtype == FP4T_DT_BF16),
               "%s: dtypes must be f32 or bf16", name);
  FP4T_REQUIRE(ldx >= cols && ldy >= cols && ldx % 4 == 0 && ldy % 4 == 0, "%s: row pitches must be multiples of 4, at least cols", name);
  FP4T_REQUIRE(aligned16(x) && aligned16(y) && aligned16(gamma) && aligned16(beta), "%s: pointers must be 16-byte aligned", name);
  FP4T_REQUIRE(eps >= 0.0f, "%s: eps must not be negative", name);
  if (rows == 0) return FP4T_OK;
  const int grid = cols <= 256 ? norm_grid(layernorm_fwd_kernel<2>, rows)
                   : cols <= 512 ? norm_grid(layernorm_fwd_kernel<4>, rows) : norm_grid(layernorm_fwd_kernel<8>, rows);
  if (grid <= 0) {
    set_error("%s: the current device is not an sm_100 part", name);
    return FP4T_ERR_DEVICE;
  }
  NormFwd p{x, x_dtype, ldx, gamma, beta, eps, y, y_dtype, ldy, mean, rstd, rows, (int)cols};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (cols <= 256) layernorm_fwd_kernel<2><<<grid, kNormThreads, 0, s>>>(p);
  else if (cols <= 512) layernorm_fwd_kernel<4><<<grid, kNormThreads, 0, s>>>(p);
  else layernorm_fwd_kernel<8><<<grid, kNormThreads, 0, s>>>(p);
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}

extern "C" int64_t fp4t_layernorm_backward_workspace_bytes(int64_t rows, int64_t cols) {
  if (rows < 0 || cols <= 0 || cols > kNormMaxCols) return -1;
  const int grid = max_norm_grid();     // an upper bound of the backward kernel's grid
  if (grid <= 0) return -1;
  return (int64_t)grid * 2 * cols * (int64_t)sizeof(float);
}

extern "C" int fp4t_layernorm_backward(const void* dy, int dy_dtype, int64_t lddy, const void* x, int x_dtype, int64_t ldx,
                                       const float* mean, const float* rstd, const float* gamma, int64_t rows, int64_t cols,
                                       void* dx, int64_t lddx, float* dgamma, float* dbeta, void* workspace,
                                       fp4t_stream_t stream) {
  const char* name = "fp4t_layernorm_backward";
  int rc = check_common(name, rows, cols);
  if (rc != FP4T_OK) return rc;
  FP4T_REQUIRE(dy && x && mean && rstd && gamma && dx && dgamma && dbeta && workspace, "%s: null pointer", name);
  FP4T_REQUIRE((x_dtype == FP4T_DT_F32 || x_dtype == FP4T_DT_BF16) && (dy_dtype == FP4T_DT_F32 || dy_dtype == FP4T_DT_BF16),
               "%s: dtypes must be f32 or bf16", name);
  FP4T_REQUIRE(ldx >= cols && lddy >= cols && lddx >= cols && ldx % 4 == 0 && lddy % 4 == 0 && lddx % 4 == 0,
               "%s: row pitches must be multiples of 4, at least cols", name);
  FP4T_REQUIRE(aligned16(x) && aligned16(dy) && aligned16(dx) && aligned16(gamma) && aligned16(workspace),
               "%s: pointers must be 16-byte aligned", name);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (rows == 0) {
    FP4T_CUDA(cudaMemsetAsync(dgamma, 0, (size_t)cols * sizeof(float), s));
    FP4T_CUDA(cudaMemsetAsync(dbeta, 0, (size_t)cols * sizeof(float), s));
    return FP4T_OK;
  }
  const int grid = cols <= 256 ? norm_grid(layernorm_bwd_kernel<2>, rows)
                   : cols <= 512 ? norm_grid(layernorm_bwd_kernel<4>, rows) : norm_grid(layernorm_bwd_kernel<8>, rows);
  if (grid <= 0) {
    set_error("%s: the current device is not an sm_100 part", name);
    return FP4T_ERR_DEVICE;
  }
  NormBwd p{dy, dy_dtype, lddy, x, x_dtype, ldx, mean, rstd, gamma, dx, lddx, static_cast<float*>(workspace), rows, (int)cols};
  if (cols <= 256) layernorm_bwd_kernel<2><<<grid, kNormThreads, 0, s>>>(p);
  else if (cols <= 512) layernorm_bwd_kernel<4><<<grid, kNormThreads, 0, s>>>(p);
  else layernorm_bwd_kernel<8><<<grid, kNormThreads, 0, s>>>(p);
  FP4T_CUDA(cudaGetLastError());
  layernorm_param_grad_kernel<<<(unsigned)ceil_div(2 * cols, 32), 32 * kParamWarps, 0, s>>>(
      static_cast<const float*>(workspace), grid, (int)cols, dgamma, dbeta);
  FP4T_CUDA(cudaGetLastError());
  return FP4T_OK;
}
