// LayerNorm forward/backward, GELU forward/backward, and microbatch BatchNorm (channels-last) kernels, sm_100a.
//
// Reference call sites: ViT / BERT blocks (`benchmarks/moco-v3/vits.py:132`, `benchmarks/distilbert/bert.py`),
// GELU inside their MLPs, and the microbatch-aware BatchNorm (`tspipe/batchnorm.py:45-120`), all plain ATen calls
// there.  Under bf16 autocast ATen's layer_norm up-casts to fp32 and writes fp32; these kernels read and write
// the activation dtype directly and keep statistics in fp32.
#include "common.cuh"
#include "tspipe_kernels.h"

namespace {

constexpr int kLnMaxVec = 4;   // per-lane register tile: 4 x 8 elements -> rows up to 1024 wide stay in registers

// ---------------------------------------------------------------------------------------------
// LayerNorm forward: one warp per row.  D % 8 == 0 and D <= 1024 -> single pass from registers.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) ln_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                                     const float* __restrict__ b, T* __restrict__ y,
                                                     float* __restrict__ mean, float* __restrict__ rstd, int rows,
                                                     int d, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + warp;
  if (row >= rows) return;
  const T* xr = x + (int64_t)row * d;
  T* yr = y + (int64_t)row * d;
  float v[kLnMaxVec][8];
  float s = 0.f;
  const int nvec = d >> 3;
#pragma unroll
  for (int k = 0; k < kLnMaxVec; ++k) {
    const int vi = lane + 32 * k;
    if (vi < nvec) {
      tsp::ld8(xr, (int64_t)vi * 8, v[k]);
#pragma unroll
      for (int e = 0; e < 8; ++e) s += v[k][e];
    }
  }
  const float mu = tsp::warp_sum(s) / d;
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < kLnMaxVec; ++k) {
    const int vi = lane + 32 * k;
    if (vi < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) { const float c = v[k][e] - mu; q += c * c; }
    }
  }
  const float rs = rsqrtf(tsp::warp_sum(q) / d + eps);
  if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
#pragma unroll
  for (int k = 0; k < kLnMaxVec; ++k) {
    const int vi = lane + 32 * k;
    if (vi < nvec) {
      float wv[8], bv[8], o[8];
      tsp::ld8(w, (int64_t)vi * 8, wv);
      tsp::ld8(b, (int64_t)vi * 8, bv);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[k][e] - mu) * rs * wv[e] + bv[e];
      tsp::st8(yr, (int64_t)vi * 8, o);
    }
  }
}

// LayerNorm backward, part 1: dx per row (one warp per row) + per-block partial dw/db over the block's rows.
// partial layout: [gridDim.x][2][d] fp32 (scratch memory owned by the caller).
template <typename T>
__global__ void __launch_bounds__(128) ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                     const float* __restrict__ w, const float* __restrict__ mean,
                                                     const float* __restrict__ rstd, T* __restrict__ dx,
                                                     float* __restrict__ partial, int rows, int d,
                                                     int rows_per_block) {
  extern __shared__ float sm[];            // [2][d] accumulators for the block
  float* sdw = sm;
  float* sdb = sm + d;
  for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) sm[i] = 0.f;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = d >> 3;
  const int row0 = blockIdx.x * rows_per_block;
  const int row1 = min(rows, row0 + rows_per_block);
  float adw[kLnMaxVec][8], adb[kLnMaxVec][8];
#pragma unroll
  for (int k = 0; k < kLnMaxVec; ++k)
#pragma unroll
    for (int e = 0; e < 8; ++e) { adw[k][e] = 0.f; adb[k][e] = 0.f; }
  for (int row = row0 + warp; row < row1; row += 4) {
    const T* xr = x + (int64_t)row * d;
    const T* gr = dy + (int64_t)row * d;
    T* dr = dx + (int64_t)row * d;
    const float mu = mean[row], rs = rstd[row];
    float xh[kLnMaxVec][8], gw[kLnMaxVec][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < kLnMaxVec; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        float xv[8], gv[8], wv[8];
        tsp::ld8(xr, (int64_t)vi * 8, xv);
        tsp::ld8(gr, (int64_t)vi * 8, gv);
        tsp::ld8(w, (int64_t)vi * 8, wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[k][e] = (xv[e] - mu) * rs;
          gw[k][e] = gv[e] * wv[e];
          s1 += gw[k][e];
          s2 += gw[k][e] * xh[k][e];
          adw[k][e] += gv[e] * xh[k][e];
          adb[k][e] += gv[e];
        }
      }
    }
    s1 = tsp::warp_sum(s1) / d;
    s2 = tsp::warp_sum(s2) / d;
#pragma unroll
    for (int k = 0; k < kLnMaxVec; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rs * (gw[k][e] - s1 - xh[k][e] * s2);
        tsp::st8(dr, (int64_t)vi * 8, o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < kLnMaxVec; ++k) {
    const int vi = lane + 32 * k;
    if (vi < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        atomicAdd(sdw + vi * 8 + e, adw[k][e]);
        atomicAdd(sdb + vi * 8 + e, adb[k][e]);
      }
    }
  }
  __syncthreads();
  float* out = partial + (int64_t)blockIdx.x * 2 * d;
  for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) out[i] = sm[i];
}

// LayerNorm backward, split form: (a) dx only - one warp per row, no cross-row state, high occupancy;
// (b) dw/db as a column reduction over rows: thread = 8 columns, block = a contiguous range of rows, per-block
// partial sums to `partial` ([gridDim.x][2][d]), reduced by ln_bwd_reduce_kernel.
template <typename T>
__global__ void __launch_bounds__(128) ln_bwd_dx_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                        const float* __restrict__ w, const float* __restrict__ mean,
                                                        const float* __restrict__ rstd, T* __restrict__ dx, int rows,
                                                        int d) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + warp;
  if (row >= rows) return;
  const int nvec = d >> 3;
  const T* xr = x + (int64_t)row * d;
  const T* gr = dy + (int64_t)row * d;
  T* dr = dx + (int64_t)row * d;
  const float mu = mean[row], rs = rstd[row];
  float xh[kLnMaxVec][8], gw[kLnMaxVec][8];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int k = 0; k < kLnMaxVec; ++k) {
    const int vi = lane + 32 * k;
    if (vi < nvec) {
      float xv[8], gv[8], wv[8];
      tsp::ld8(xr, (int64_t)vi * 8, xv);
      tsp::ld8(gr, (int64_t)vi * 8, gv);
      tsp::ld8(w, (int64_t)vi * 8, wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        xh[k][e] = (xv[e] - mu) * rs;
        gw[k][e] = gv[e] * wv[e];
        s1 += gw[k][e];
        s2 += gw[k][e] * xh[k][e];
      }
    }
  }
  s1 = tsp::warp_sum(s1) / d;
  s2 = tsp::warp_sum(s2) / d;
#pragma unroll
  for (int k = 0; k < kLnMaxVec; ++k) {
    const int vi = lane + 32 * k;
    if (vi < nvec) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = rs * (gw[k][e] - s1 - xh[k][e] * s2);
      tsp::st8(dr, (int64_t)vi * 8, o);
    }
  }
}

// block = (d/8 column vectors) x (256 / (d/8) rows in parallel); dynamic smem = threads * 16 floats
template <typename T>
__global__ void __launch_bounds__(256) ln_bwd_colsum_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                            const float* __restrict__ mean,
                                                            const float* __restrict__ rstd,
                                                            float* __restrict__ partial, int rows, int d) {
  extern __shared__ float sm[];
  const int nvec = d >> 3;
  const int tx_n = nvec < 256 ? nvec : 256;
  const int ty_n = 256 / tx_n;
  const int tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
  const bool active = ty < ty_n && tx < nvec;
  float a[8], b[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { a[e] = 0.f; b[e] = 0.f; }
  if (active) {
    const int rows_per_block = (rows + gridDim.x - 1) / gridDim.x;
    const int r0 = blockIdx.x * rows_per_block;
    const int r1 = min(rows, r0 + rows_per_block);
    for (int r = r0 + ty; r < r1; r += ty_n) {
      float gv[8], xv[8];
      tsp::ld8(dy, (int64_t)r * d + tx * 8, gv);
      tsp::ld8(x, (int64_t)r * d + tx * 8, xv);
      const float mu = mean[r], rs = rstd[r];
#pragma unroll
      for (int e = 0; e < 8; ++e) { a[e] += gv[e] * (xv[e] - mu) * rs; b[e] += gv[e]; }
    }
  }
  float* mine = sm + (int64_t)threadIdx.x * 16;
#pragma unroll
  for (int e = 0; e < 8; ++e) { mine[e] = a[e]; mine[8 + e] = b[e]; }
  __syncthreads();
  if (ty == 0 && tx < nvec) {
    for (int k = 1; k < ty_n; ++k) {
      const float* o = sm + (int64_t)(k * tx_n + tx) * 16;
#pragma unroll
      for (int e = 0; e < 8; ++e) { a[e] += o[e]; b[e] += o[8 + e]; }
    }
    float* out = partial + (int64_t)blockIdx.x * 2 * d;
#pragma unroll
    for (int e = 0; e < 8; ++e) { out[tx * 8 + e] = a[e]; out[d + tx * 8 + e] = b[e]; }
  }
}

// part 2: dw[j] = sum_blocks partial[b][0][j], db likewise.
__global__ void __launch_bounds__(256) ln_bwd_reduce_kernel(const float* __restrict__ partial, int nblocks, int d,
                                                            float* __restrict__ dw, float* __restrict__ db) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= 2 * d) return;
  float acc = 0.f;
  for (int b = 0; b < nblocks; ++b) acc += partial[(int64_t)b * 2 * d + j];
  if (j < d) dw[j] = acc; else db[j - d] = acc;
}

// ---------------------------------------------------------------------------------------------
// GELU (erf form), optionally with the bias add in front: y = gelu(x + bias)
// ---------------------------------------------------------------------------------------------
// erf through the rational form of Abramowitz & Stegun 7.1.26 (|error| <= 1.5e-7, below fp32 resolution of the
// products it enters): one reciprocal, one exponential and six FMAs instead of the two-branch library routine -
// these kernels are bound by instruction issue, not by memory.  E = exp(-z^2) is returned for the backward.
__device__ __forceinline__ float erf_fast(float z, float& e_out) {
  const float az = fabsf(z);
  const float t = __frcp_rn(fmaf(0.3275911f, az, 1.f));
  float p = fmaf(1.061405429f, t, -1.453152027f);
  p = fmaf(p, t, 1.421413741f);
  p = fmaf(p, t, -0.284496736f);
  p = fmaf(p, t, 0.254829592f);
  p *= t;
  const float e = exp2f(-1.4426950408889634f * az * az);
  e_out = e;
  return copysignf(fmaf(-p, e, 1.f), z);
}
__device__ __forceinline__ float gelu_f(float x) {
  float e;
  return 0.5f * x * (1.f + erf_fast(x * 0.70710678118654752f, e));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  float e;                                        // e = exp(-x^2 / 2): the Gaussian density needs it too
  const float cdf = 0.5f * (1.f + erf_fast(x * 0.70710678118654752f, e));
  return fmaf(x * 0.3989422804014327f, e, cdf);
}

// Column (in 8-element vectors) of vector i in a matrix with cpv vectors per row.  A 64-bit remainder by a run-time
// value costs about a hundred instructions; vector counts fit 32 bits in practice.
__device__ __forceinline__ uint32_t bias_col(int64_t i, uint32_t cpv) {
  return i < (int64_t)0xffffffffu ? (uint32_t)i % cpv : (uint32_t)(i % (int64_t)cpv);
}

// Four independent 8-element vectors per thread and trip: all loads are issued before the first use (a single
// load in flight per thread left these kernels at 3 TB/s).
template <typename T>
__global__ void __launch_bounds__(256) gelu_fwd_kernel(const T* __restrict__ x, const float* __restrict__ bias,
                                                       T* __restrict__ y, int64_t n, int d) {
  const int64_t nv = n >> 3;
  const uint32_t cpv = (uint32_t)(d >> 3);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < nv; i += 4 * stride) {
    tsp::Raw8<T> raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) tsp::ldraw(x, (i + u * stride) * 8, raw[u]);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float v[8], o[8];
      tsp::cvt8(raw[u], v);
      if (bias) {
        float b[8];
        tsp::ld8(bias, (int64_t)bias_col(i + u * stride, cpv) * 8, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += b[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = gelu_f(v[e]);
      tsp::st8(y, (i + u * stride) * 8, o);
    }
  }
  for (; i < nv; i += stride) {
    float v[8], o[8];
    tsp::ld8(x, i * 8, v);
    if (bias) {
      float b[8];
      tsp::ld8(bias, (int64_t)bias_col(i, cpv) * 8, b);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += b[e];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = gelu_f(v[e]);
    tsp::st8(y, i * 8, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) gelu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                       const float* __restrict__ bias, T* __restrict__ dx, int64_t n,
                                                       int d) {
  const int64_t nv = n >> 3;
  const uint32_t cpv = (uint32_t)(d >> 3);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + stride < nv; i += 2 * stride) {
    tsp::Raw8<T> xr[2], gr[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) { tsp::ldraw(x, (i + u * stride) * 8, xr[u]); tsp::ldraw(dy, (i + u * stride) * 8, gr[u]); }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float v[8], g[8], o[8];
      tsp::cvt8(xr[u], v);
      tsp::cvt8(gr[u], g);
      if (bias) {
        float b[8];
        tsp::ld8(bias, (int64_t)bias_col(i + u * stride, cpv) * 8, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += b[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = g[e] * gelu_grad_f(v[e]);
      tsp::st8(dx, (i + u * stride) * 8, o);
    }
  }
  for (; i < nv; i += stride) {
    float v[8], g[8], o[8];
    tsp::ld8(x, i * 8, v);
    tsp::ld8(dy, i * 8, g);
    if (bias) {
      float b[8];
      tsp::ld8(bias, (int64_t)bias_col(i, cpv) * 8, b);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += b[e];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = g[e] * gelu_grad_f(v[e]);
    tsp::st8(dx, i * 8, o);
  }
}

}  // namespace

extern "C" {

int tsp_layernorm_fwd(const void* x, const float* w, const float* b, void* y, float* mean, float* rstd, int rows, int d,
                      float eps, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (d % 8 != 0 || d > 8 * 32 * kLnMaxVec) return -3;
  const int grid = (rows + 3) / 4;
  if (dtype == TSP_DTYPE_BF16)
    ln_fwd_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)x, w, b, (__nv_bfloat16*)y, mean, rstd,
                                                           rows, d, eps);
  else
    ln_fwd_kernel<float><<<grid, 128, 0, stream>>>((const float*)x, w, b, (float*)y, mean, rstd, rows, d, eps);
  return TSP_LAUNCH_CHECK();
}

int tsp_layernorm_bwd_blocks(int rows) {
  int nb = (rows + 63) / 64;
  const int cap = 148 * 4;
  return nb > cap ? cap : (nb < 1 ? 1 : nb);
}

// `partial` is scratch of tsp_layernorm_bwd_blocks(rows) * 2 * d floats.
int tsp_layernorm_bwd(const void* dy, const void* x, const float* w, const float* mean, const float* rstd, void* dx,
                      float* dw, float* db, float* partial, int rows, int d, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (d % 8 != 0 || d > 8 * 32 * kLnMaxVec) return -3;
  const int nb = tsp_layernorm_bwd_blocks(rows);
  const int grid_dx = (rows + 3) / 4;
  const size_t smem = sizeof(float) * 16 * 256;
  if (dtype == TSP_DTYPE_BF16) {
    ln_bwd_dx_kernel<__nv_bfloat16><<<grid_dx, 128, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, w,
                                                                 mean, rstd, (__nv_bfloat16*)dx, rows, d);
    ln_bwd_colsum_kernel<__nv_bfloat16><<<nb, 256, smem, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                                   mean, rstd, partial, rows, d);
  } else {
    ln_bwd_dx_kernel<float><<<grid_dx, 128, 0, stream>>>((const float*)dy, (const float*)x, w, mean, rstd, (float*)dx,
                                                         rows, d);
    ln_bwd_colsum_kernel<float><<<nb, 256, smem, stream>>>((const float*)dy, (const float*)x, mean, rstd, partial, rows,
                                                           d);
  }
  ln_bwd_reduce_kernel<<<(2 * d + 255) / 256, 256, 0, stream>>>(partial, nb, d, dw, db);
  return TSP_LAUNCH_CHECK();
}

int tsp_gelu_fwd(const void* x, const float* bias, void* y, int64_t n, int d, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 8 != 0 || (bias && d % 8 != 0)) return -3;
  int64_t blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == TSP_DTYPE_BF16)
    gelu_fwd_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, bias, (__nv_bfloat16*)y, n, d);
  else
    gelu_fwd_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)x, bias, (float*)y, n, d);
  return TSP_LAUNCH_CHECK();
}

int tsp_gelu_bwd(const void* dy, const void* x, const float* bias, void* dx, int64_t n, int d, int dtype,
                 cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 8 != 0 || (bias && d % 8 != 0)) return -3;
  int64_t blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == TSP_DTYPE_BF16)
    gelu_bwd_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, bias,
                                                                    (__nv_bfloat16*)dx, n, d);
  else
    gelu_bwd_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)dy, (const float*)x, bias, (float*)dx, n, d);
  return TSP_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// LayerNorm backward for callers that must not allocate (see tspipe_noalloc.h).
// The per-block dw/db partial sums go to this fixed array instead of a caller-provided buffer.
// Every GPU that loads the library holds these 1.16 MiB until the process exits.
// ---------------------------------------------------------------------------------------------
#include "tspipe_noalloc.h"

static __device__ __align__(256) float g_ln_bwd_scratch[TSP_NOALLOC_LN_MAX_BLOCKS * 2 * TSP_NOALLOC_LN_MAX_D];

int tsp_layernorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* mean, const float* rstd,
                              void* dx, float* dw, float* db, int rows, int d, int dtype, cudaStream_t stream) {
  // In host code `g_ln_bwd_scratch` is only a handle for the runtime, not an address a kernel can use: the
  // device address has to be looked up, once per device, with that device current.
  static float* scratch_of_device[TSP_NOALLOC_MAX_DEVICES] = {nullptr};
  if (rows < 0 || d <= 0) return -3;
  if (rows == 0) return 0;
  if (d % 8 != 0) return -3;
  if (d > TSP_NOALLOC_LN_MAX_D) return TSP_NOALLOC_ERR_TOO_LARGE;
  if (dtype != TSP_DTYPE_F32 && dtype != TSP_DTYPE_BF16) return -3;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= TSP_NOALLOC_MAX_DEVICES) return TSP_NOALLOC_ERR_TOO_LARGE;
  float* scratch = scratch_of_device[dev];
  if (scratch == nullptr) {
    e = cudaGetSymbolAddress((void**)&scratch, g_ln_bwd_scratch);
    if (e != cudaSuccess) return (int)e;
    scratch_of_device[dev] = scratch;
  }
  int nb = tsp_layernorm_bwd_blocks(rows);
  if (nb > TSP_NOALLOC_LN_MAX_BLOCKS) nb = TSP_NOALLOC_LN_MAX_BLOCKS;
  const int rpb = (rows + nb - 1) / nb;
  const size_t smem = sizeof(float) * 2 * (size_t)d;
  // Nothing in the scratch has to start at zero: each of the nb blocks overwrites its whole 2*d slice and the
  // reduction reads exactly those nb slices, so what an earlier call left behind is never read.
  if (dtype == TSP_DTYPE_BF16)
    ln_bwd_kernel<__nv_bfloat16><<<nb, 128, smem, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, w, mean,
                                                            rstd, (__nv_bfloat16*)dx, scratch, rows, d, rpb);
  else
    ln_bwd_kernel<float><<<nb, 128, smem, stream>>>((const float*)dy, (const float*)x, w, mean, rstd, (float*)dx,
                                                    scratch, rows, d, rpb);
  ln_bwd_reduce_kernel<<<(2 * d + 255) / 256, 256, 0, stream>>>(scratch, nb, d, dw, db);
  return TSP_LAUNCH_CHECK();
}

}  // extern "C"
