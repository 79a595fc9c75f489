// 3x3 / stride 2 / pad 1 max pooling and global average pooling for channels-last activations, forward and backward
// (sm_100a).
//
// ResNet stem (`benchmarks/byol/models/resnet_base_network.py` via torchvision's `maxpool`).  The library's NHWC
// kernels take ~0.4 ms forward / ~0.9 ms backward on a [128, 64, 112, 112] bf16 activation; both are pure
// streaming problems (read 205 MB, write 51 MB and the reverse).  Forward stores the winning tap (0..8) per output
// element in one byte; backward is a gather: every input element looks at the <= 4 windows that contain it and sums
// the gradients of those whose winner it is - no atomics, deterministic.
#include "common.cuh"
#include "tspipe_kernels.h"

namespace {

template <typename T>
__global__ void __launch_bounds__(256) maxpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                          uint8_t* __restrict__ idx, int n, int h, int w, int c,
                                                          int ho, int wo) {
  const int cpv = c >> 3;
  const int64_t total = (int64_t)n * ho * wo * cpv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int cg = (int)(i % cpv);
    int64_t p = i / cpv;
    const int ox = (int)(p % wo); p /= wo;
    const int oy = (int)(p % ho);
    const int b = (int)(p / ho);
    float best[8];
    int arg[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { best[e] = -INFINITY; arg[e] = 0; }
#pragma unroll
    for (int ky = 0; ky < 3; ++ky) {
      const int iy = oy * 2 - 1 + ky;
      if (iy < 0 || iy >= h) continue;
#pragma unroll
      for (int kx = 0; kx < 3; ++kx) {
        const int ix = ox * 2 - 1 + kx;
        if (ix < 0 || ix >= w) continue;
        float v[8];
        tsp::ld8(x, (((int64_t)b * h + iy) * w + ix) * c + cg * 8, v);
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (v[e] > best[e]) { best[e] = v[e]; arg[e] = ky * 3 + kx; }
      }
    }
    const int64_t o = (((int64_t)b * ho + oy) * wo + ox) * c + cg * 8;
    tsp::st8(y, o, best);
    if (idx != nullptr) {
      uint2 packed;
      packed.x = (uint32_t)arg[0] | ((uint32_t)arg[1] << 8) | ((uint32_t)arg[2] << 16) | ((uint32_t)arg[3] << 24);
      packed.y = (uint32_t)arg[4] | ((uint32_t)arg[5] << 8) | ((uint32_t)arg[6] << 16) | ((uint32_t)arg[7] << 24);
      *reinterpret_cast<uint2*>(idx + o) = packed;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(const T* __restrict__ dy, const uint8_t* __restrict__ idx,
                                                          T* __restrict__ dx, int n, int h, int w, int c, int ho,
                                                          int wo) {
  const int cpv = c >> 3;
  const int64_t total = (int64_t)n * h * w * cpv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int cg = (int)(i % cpv);
    int64_t p = i / cpv;
    const int ix = (int)(p % w); p /= w;
    const int iy = (int)(p % h);
    const int b = (int)(p / h);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    // windows (oy, ox) with oy*2-1 <= iy <= oy*2+1  <=>  oy in [ceil((iy-1)/2), floor((iy+1)/2)]
    const int oy0 = iy >> 1, oy1 = (iy + 1) >> 1;
    const int ox0 = ix >> 1, ox1 = (ix + 1) >> 1;
    for (int oy = oy0; oy <= oy1; ++oy) {
      if (oy >= ho) continue;
      const int ky = iy - (oy * 2 - 1);
      for (int ox = ox0; ox <= ox1; ++ox) {
        if (ox >= wo) continue;
        const int kx = ix - (ox * 2 - 1);
        const int tap = ky * 3 + kx;
        const int64_t o = (((int64_t)b * ho + oy) * wo + ox) * c + cg * 8;
        const uint2 packed = *reinterpret_cast<const uint2*>(idx + o);
        float g[8];
        tsp::ld8(dy, o, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t word = e < 4 ? packed.x : packed.y;
          const int a = (int)((word >> (8 * (e & 3))) & 0xFF);
          if (a == tap) acc[e] += g[e];
        }
      }
    }
    tsp::st8(dx, i * 8, acc);
  }
}

// Global average pool of a channels-last activation: y[b, c] = mean over the hw positions of x[b, :, c].  One thread
// per (image, 8 channels): consecutive threads read consecutive 16-byte groups of a pixel's channel vector.
template <typename T>
__global__ void __launch_bounds__(256) avgpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int n, int hw,
                                                          int c) {
  const int cpv = c >> 3;
  const int64_t total = (int64_t)n * cpv;
  const float inv = 1.f / (float)hw;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int cg = (int)(i % cpv);
    const int64_t b = i / cpv;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int p = 0; p < hw; ++p) {
      float v[8];
      tsp::ld8(x, (b * hw + p) * c + cg * 8, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[e];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] *= inv;
    tsp::st8(y, b * c + cg * 8, acc);
  }
}

// dx[b, p, c] = dy[b, c] / hw
template <typename T>
__global__ void __launch_bounds__(256) avgpool_bwd_kernel(const T* __restrict__ dy, T* __restrict__ dx, int n, int hw,
                                                          int c) {
  const int cpv = c >> 3;
  const int64_t total = (int64_t)n * hw * cpv;
  const float inv = 1.f / (float)hw;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int cg = (int)(i % cpv);
    const int64_t b = i / cpv / hw;
    float v[8];
    tsp::ld8(dy, b * c + cg * 8, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] *= inv;
    tsp::st8(dx, i * 8, v);
  }
}

inline int blocks_for(int64_t n) {
  int64_t b = (n + 255) / 256;
  if (b > 148 * 16) b = 148 * 16;
  return (int)(b < 1 ? 1 : b);
}

}  // namespace

extern "C" {

// x [n, h, w, c] -> y [n, ho, wo, c], ho = (h + 1) / 2, wo = (w + 1) / 2 ; idx (optional) [n, ho, wo, c] bytes.
int tsp_maxpool3x3s2_fwd(const void* x, void* y, uint8_t* idx, int n, int h, int w, int c, int dtype,
                         cudaStream_t stream) {
  if (n <= 0) return 0;
  if (c % 8 != 0) return -3;
  const int ho = (h + 1) / 2, wo = (w + 1) / 2;
  const int grid = blocks_for((int64_t)n * ho * wo * (c / 8));
  if (dtype == TSP_DTYPE_BF16)
    maxpool_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, idx, n, h, w,
                                                                c, ho, wo);
  else
    maxpool_fwd_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (float*)y, idx, n, h, w, c, ho, wo);
  return TSP_LAUNCH_CHECK();
}

int tsp_maxpool3x3s2_bwd(const void* dy, const uint8_t* idx, void* dx, int n, int h, int w, int c, int dtype,
                         cudaStream_t stream) {
  if (n <= 0) return 0;
  if (c % 8 != 0) return -3;
  const int ho = (h + 1) / 2, wo = (w + 1) / 2;
  const int grid = blocks_for((int64_t)n * h * w * (c / 8));
  if (dtype == TSP_DTYPE_BF16)
    maxpool_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dy, idx, (__nv_bfloat16*)dx, n, h,
                                                                w, c, ho, wo);
  else
    maxpool_bwd_kernel<float><<<grid, 256, 0, stream>>>((const float*)dy, idx, (float*)dx, n, h, w, c, ho, wo);
  return TSP_LAUNCH_CHECK();
}

// x [n, h*w, c] channels-last -> y [n, c] (mean over the positions); c a multiple of 8.
int tsp_avgpool_fwd(const void* x, void* y, int n, int hw, int c, int dtype, cudaStream_t stream) {
  if (n <= 0 || hw <= 0) return 0;
  if (c % 8 != 0) return -3;
  const int grid = blocks_for((int64_t)n * (c / 8));
  if (dtype == TSP_DTYPE_BF16)
    avgpool_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, hw, c);
  else
    avgpool_fwd_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (float*)y, n, hw, c);
  return TSP_LAUNCH_CHECK();
}

int tsp_avgpool_bwd(const void* dy, void* dx, int n, int hw, int c, int dtype, cudaStream_t stream) {
  if (n <= 0 || hw <= 0) return 0;
  if (c % 8 != 0) return -3;
  const int grid = blocks_for((int64_t)n * hw * (c / 8));
  if (dtype == TSP_DTYPE_BF16)
    avgpool_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, n, hw, c);
  else
    avgpool_bwd_kernel<float><<<grid, 256, 0, stream>>>((const float*)dy, (float*)dx, n, hw, c);
  return TSP_LAUNCH_CHECK();
}

}  // extern "C"
