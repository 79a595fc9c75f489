// Fused loss kernels (forward value + gradient in one launch), sm_100a.
//
// Reference math: BYOL regression `benchmarks/byol/trainer.py:51-55,192-196`; soft-target KD
// `benchmarks/soft_target/kd_losses/st.py:18-23` + CE `benchmarks/soft_target/train_kd.py:448-453`;
// DistilBERT KL/MLM-CE terms `benchmarks/distilbert/distiller.py:711-772`.  The reference evaluates each with
// 5-10 library ops (normalize, softmax, log_softmax, kl_div, cross_entropy, masked_select copies) and a
// second sweep in autograd; the loss GPU holds the whole mini-batch, so these are latency- and
// bandwidth-bound row kernels: one read of the rows (teacher rows may sit behind a peer pointer), one write of
// the student gradient.
#include "common.cuh"
#include "tspipe_kernels.h"

namespace {

// ---------------------------------------------------------------------------------------------
// BYOL: loss += scale * sum_rows (2 - 2 cos(x_r, y_r)) ; gx = scale * d/dx
// one warp per row
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) byol_kernel(const T* __restrict__ x, const T* __restrict__ y, int n, int d,
                                                   float scale, float* __restrict__ loss, T* __restrict__ gx) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + warp;
  float contrib = 0.f;
  if (row < n) {
    const T* xr = x + (int64_t)row * d;
    const T* yr = y + (int64_t)row * d;
    float xx = 0.f, yy = 0.f, xy = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float a = tsp::ld(xr, i), b = tsp::ld(yr, i);
      xx += a * a; yy += b * b; xy += a * b;
    }
    xx = tsp::warp_sum(xx); yy = tsp::warp_sum(yy); xy = tsp::warp_sum(xy);
    const float nx = fmaxf(sqrtf(xx), 1e-12f), ny = fmaxf(sqrtf(yy), 1e-12f);
    const float cosv = xy / (nx * ny);
    contrib = 2.f - 2.f * cosv;
    if (gx != nullptr) {
      T* gr = gx + (int64_t)row * d;
      const float c1 = -2.f * scale / (nx * ny), c2 = 2.f * scale * cosv / (nx * nx);
      for (int i = lane; i < d; i += 32) tsp::st(gr, i, c1 * tsp::ld(yr, i) + c2 * tsp::ld(xr, i));
    }
  }
  __shared__ float part[4];
  if (lane == 0) part[warp] = contrib;
  __syncthreads();
  if (threadIdx.x == 0) atomicAdd(loss, scale * (part[0] + part[1] + part[2] + part[3]));
}

// ---------------------------------------------------------------------------------------------
// Soft-target KD + CE, one block per row:
//   loss += w_ce * CE(s, label) [label >= 0] + w_kd * T^2 * KL(softmax(t/T) || softmax(s/T))
//   gs    = w_ce * (softmax(s) - onehot) + w_kd * T * (softmax(s/T) - softmax(t/T))
// rows with row_mask == 0 are skipped (gradient zero).  `t` may be null when w_kd == 0.
// ---------------------------------------------------------------------------------------------
template <typename TS, typename TT>
__global__ void __launch_bounds__(256) kd_ce_kernel(const TS* __restrict__ s, const TT* __restrict__ t,
                                                    const int64_t* __restrict__ labels,
                                                    const uint8_t* __restrict__ row_mask, int n, int c, float temp,
                                                    float w_ce, float w_kd, float* __restrict__ loss,
                                                    TS* __restrict__ gs) {
  __shared__ float scratch[33];
  const int row = blockIdx.x;
  if (row >= n) return;
  const TS* sr = s + (int64_t)row * c;
  const TT* tr = t ? t + (int64_t)row * c : nullptr;
  TS* gr = gs ? gs + (int64_t)row * c : nullptr;
  if (row_mask != nullptr && row_mask[row] == 0) {
    if (gr) for (int i = threadIdx.x; i < c; i += blockDim.x) tsp::st(gr, i, 0.f);
    return;
  }
  const bool kd = (w_kd != 0.f) && tr != nullptr;
  const float inv_t = 1.f / temp;
  float ms = -INFINITY, mt = -INFINITY;
  for (int i = threadIdx.x; i < c; i += blockDim.x) {
    ms = fmaxf(ms, tsp::ld(sr, i));
    if (kd) mt = fmaxf(mt, tsp::ld(tr, i));
  }
  ms = tsp::block_max(ms, scratch);
  if (kd) mt = tsp::block_max(mt, scratch);
  float z1 = 0.f, zs = 0.f, zt = 0.f;
  for (int i = threadIdx.x; i < c; i += blockDim.x) {
    const float a = tsp::ld(sr, i) - ms;
    z1 += __expf(a);
    if (kd) { zs += __expf(a * inv_t); zt += __expf((tsp::ld(tr, i) - mt) * inv_t); }
  }
  z1 = tsp::block_sum(z1, scratch);
  if (kd) { zs = tsp::block_sum(zs, scratch); zt = tsp::block_sum(zt, scratch); }
  const float l1 = logf(z1), lsT = kd ? logf(zs) : 0.f, ltT = kd ? logf(zt) : 0.f;
  const int64_t label = labels ? labels[row] : -1;
  const bool has_ce = (w_ce != 0.f) && label >= 0 && label < c;
  float kl = 0.f;
  for (int i = threadIdx.x; i < c; i += blockDim.x) {
    const float a = tsp::ld(sr, i) - ms;
    float g = 0.f;
    if (has_ce) g = w_ce * (__expf(a - l1) - (i == label ? 1.f : 0.f));
    if (kd) {
      const float lps = a * inv_t - lsT;
      const float lpt = (tsp::ld(tr, i) - mt) * inv_t - ltT;
      const float pt = __expf(lpt);
      kl += pt * (lpt - lps);
      g += w_kd * temp * (__expf(lps) - pt);
    }
    if (gr) tsp::st(gr, i, g);
  }
  if (kd) kl = tsp::block_sum(kl, scratch);
  if (threadIdx.x == 0) {
    float v = 0.f;
    if (has_ce) v += w_ce * (l1 - (tsp::ld(sr, label) - ms));
    if (kd) v += w_kd * temp * temp * kl;
    atomicAdd(loss, v);
  }
}

// ---------------------------------------------------------------------------------------------
// Cosine-embedding term of the DistilBERT loss (target +1): loss += scale * sum_rows (1 - cos) over selected rows
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) cosine_kernel(const T* __restrict__ x, const T* __restrict__ y,
                                                     const uint8_t* __restrict__ row_mask, int n, int d, float scale,
                                                     float* __restrict__ loss, T* __restrict__ gx) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + warp;
  float contrib = 0.f;
  if (row < n) {
    const T* xr = x + (int64_t)row * d;
    const T* yr = y + (int64_t)row * d;
    T* gr = gx ? gx + (int64_t)row * d : nullptr;
    const bool on = row_mask == nullptr || row_mask[row] != 0;
    if (on) {
      float xx = 0.f, yy = 0.f, xy = 0.f;
      for (int i = lane; i < d; i += 32) {
        const float a = tsp::ld(xr, i), b = tsp::ld(yr, i);
        xx += a * a; yy += b * b; xy += a * b;
      }
      xx = tsp::warp_sum(xx) + 1e-8f; yy = tsp::warp_sum(yy) + 1e-8f; xy = tsp::warp_sum(xy);
      const float inv = rsqrtf(xx * yy);
      const float cosv = xy * inv;
      contrib = 1.f - cosv;
      if (gr) {
        const float c1 = -scale * inv, c2 = scale * cosv / xx;
        for (int i = lane; i < d; i += 32) tsp::st(gr, i, c1 * tsp::ld(yr, i) + c2 * tsp::ld(xr, i));
      }
    } else if (gr) {
      for (int i = lane; i < d; i += 32) tsp::st(gr, i, 0.f);
    }
  }
  __shared__ float part[4];
  if (lane == 0) part[warp] = contrib;
  __syncthreads();
  if (threadIdx.x == 0) atomicAdd(loss, scale * (part[0] + part[1] + part[2] + part[3]));
}

}  // namespace

extern "C" {

int tsp_byol_loss(const void* x, const void* y, int n, int d, int dtype, float scale, float* loss, void* gx,
                  cudaStream_t stream) {
  if (n <= 0) return 0;
  const int grid = (n + 3) / 4;
  if (dtype == TSP_DTYPE_BF16)
    byol_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)y, n, d, scale,
                                                         loss, (__nv_bfloat16*)gx);
  else
    byol_kernel<float><<<grid, 128, 0, stream>>>((const float*)x, (const float*)y, n, d, scale, loss, (float*)gx);
  return TSP_LAUNCH_CHECK();
}

int tsp_cosine_loss(const void* x, const void* y, const uint8_t* row_mask, int n, int d, int dtype, float scale,
                    float* loss, void* gx, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int grid = (n + 3) / 4;
  if (dtype == TSP_DTYPE_BF16)
    cosine_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)y, row_mask,
                                                           n, d, scale, loss, (__nv_bfloat16*)gx);
  else
    cosine_kernel<float><<<grid, 128, 0, stream>>>((const float*)x, (const float*)y, row_mask, n, d, scale, loss,
                                                   (float*)gx);
  return TSP_LAUNCH_CHECK();
}

int tsp_kd_ce_loss(const void* s, const void* t, const int64_t* labels, const uint8_t* row_mask, int n, int c,
                   int s_dtype, int t_dtype, float temp, float w_ce, float w_kd, float* loss, void* gs,
                   cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = c >= 2048 ? 256 : (c >= 512 ? 128 : 64);
#define TSP_KD(TS, TT)                                                                                             \
  kd_ce_kernel<TS, TT><<<n, threads, 0, stream>>>((const TS*)s, (const TT*)t, labels, row_mask, n, c, temp, w_ce, \
                                                  w_kd, loss, (TS*)gs)
  if (s_dtype == TSP_DTYPE_BF16 && t_dtype == TSP_DTYPE_BF16) TSP_KD(__nv_bfloat16, __nv_bfloat16);
  else if (s_dtype == TSP_DTYPE_BF16) TSP_KD(__nv_bfloat16, float);
  else if (t_dtype == TSP_DTYPE_BF16) TSP_KD(float, __nv_bfloat16);
  else TSP_KD(float, float);
#undef TSP_KD
  return TSP_LAUNCH_CHECK();
}

}  // extern "C"
