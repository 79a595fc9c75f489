// Optimizer and momentum-teacher kernels over flat parameter buffers (sm_100a).
//
// Reference behaviour: LARS `benchmarks/byol/main.py:13-46` (= `benchmarks/moco-v3/moco/optimizer.py`),
// AdamW / SGD from torch.optim as used by `benchmarks/distilbert/distiller.py:150` and
// `benchmarks/soft_target/train_kd.py:209-213`, momentum update `benchmarks/byol/trainer.py:198-212`.
// The reference runs 6-10 elementwise launches and two norm reductions PER TENSOR; here a whole
// partition is one flat fp32 buffer cut into fixed-size chunks that never straddle a tensor, so a step
// is two launches (LARS: norms, apply) or one (AdamW, SGD, EMA), bound by HBM (or NVLink for a peer source).
#include "common.cuh"
#include "tspipe_kernels.h"

namespace {

constexpr int kThreads = 256;

// ---------------------------------------------------------------------------------------------
// EMA: t = m*t + (1-m)*s ; `s` may point into a peer GPU's memory (plain loads over NVLink).
// Optionally writes a bf16 shadow of the new teacher for bf16 compute copies.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) ema_kernel(float* __restrict__ t, const float* __restrict__ s, int64_t n,
                                                       float m, __nv_bfloat16* __restrict__ shadow) {
  const float om = 1.f - m;
  const int64_t n4 = n >> 2;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  float4* t4 = reinterpret_cast<float4*>(t);
  const float4* s4 = reinterpret_cast<const float4*>(s);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 a = t4[i];
    const float4 b = __ldg(s4 + i);
    a.x = m * a.x + om * b.x; a.y = m * a.y + om * b.y; a.z = m * a.z + om * b.z; a.w = m * a.w + om * b.w;
    t4[i] = a;
    if (shadow) {
      __nv_bfloat162* sh = reinterpret_cast<__nv_bfloat162*>(shadow) + 2 * i;
      sh[0] = __floats2bfloat162_rn(a.x, a.y);
      sh[1] = __floats2bfloat162_rn(a.z, a.w);
    }
  }
  for (int64_t i = (n4 << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float a = m * t[i] + om * s[i];
    t[i] = a;
    if (shadow) shadow[i] = __float2bfloat16(a);
  }
}

// ---------------------------------------------------------------------------------------------
// chunked multi-tensor kernels.  chunk = (segment id, first element, length); segment = one tensor.
// ---------------------------------------------------------------------------------------------
struct ChunkView {
  int seg;
  int64_t begin;
  int len;
};

__device__ __forceinline__ ChunkView load_chunk(const int64_t* __restrict__ chunks, int c) {
  ChunkView v;
  v.seg = (int)chunks[3 * (int64_t)c];
  v.begin = chunks[3 * (int64_t)c + 1];
  v.len = (int)chunks[3 * (int64_t)c + 2];
  return v;
}

// norms[2*seg] += sum p^2 ; norms[2*seg+1] += sum (grad_scale*g + wd*p)^2   (only segments with adapt != 0)
__global__ void __launch_bounds__(kThreads) lars_norms_kernel(const float* __restrict__ p, const float* __restrict__ g,
                                                              const int64_t* __restrict__ chunks,
                                                              const float* __restrict__ seg_hp, float grad_scale,
                                                              float* __restrict__ norms) {
  __shared__ float scratch[33];
  const ChunkView c = load_chunk(chunks, blockIdx.x);
  const float* hp = seg_hp + 5 * (int64_t)c.seg;      // lr, wd, momentum, trust, adapt
  if (hp[4] == 0.f) return;
  const float wd = hp[1];
  float sp = 0.f, su = 0.f;
  const bool vec = ((c.begin & 3) == 0);
  if (vec) {
    const float4* p4 = reinterpret_cast<const float4*>(p + c.begin);
    const float4* g4 = reinterpret_cast<const float4*>(g + c.begin);
    const int n4 = c.len >> 2;
    for (int i = threadIdx.x; i < n4; i += kThreads) {
      const float4 a = p4[i], b = g4[i];
      float u;
      sp += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
      u = grad_scale * b.x + wd * a.x; su += u * u;
      u = grad_scale * b.y + wd * a.y; su += u * u;
      u = grad_scale * b.z + wd * a.z; su += u * u;
      u = grad_scale * b.w + wd * a.w; su += u * u;
    }
    for (int i = (n4 << 2) + threadIdx.x; i < c.len; i += kThreads) {
      const float a = p[c.begin + i], u = grad_scale * g[c.begin + i] + wd * a;
      sp += a * a; su += u * u;
    }
  } else {
    for (int i = threadIdx.x; i < c.len; i += kThreads) {
      const float a = p[c.begin + i], u = grad_scale * g[c.begin + i] + wd * a;
      sp += a * a; su += u * u;
    }
  }
  sp = tsp::block_sum(sp, scratch);
  su = tsp::block_sum(su, scratch);
  if (threadIdx.x == 0) {
    atomicAdd(norms + 2 * c.seg, sp);
    atomicAdd(norms + 2 * c.seg + 1, su);
  }
}

// LARS apply (+ optional fused momentum-teacher update for segments that have a local teacher copy):
//   dp = adapt ? q*(gs*g + wd*p) : gs*g ; mu = mom*mu + dp ; p -= lr*mu ; [t = m*t + (1-m)*p]
__global__ void __launch_bounds__(kThreads) lars_apply_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                              float* __restrict__ mu,
                                                              const int64_t* __restrict__ chunks,
                                                              const float* __restrict__ seg_hp, float grad_scale,
                                                              const float* __restrict__ norms,
                                                              float* __restrict__ teacher, int64_t teacher_n,
                                                              float ema_m) {
  const ChunkView c = load_chunk(chunks, blockIdx.x);
  const float* hp = seg_hp + 5 * (int64_t)c.seg;
  const float lr = hp[0], wd = hp[1], mom = hp[2], trust = hp[3];
  const bool adapt = hp[4] != 0.f;
  float q = 1.f;
  if (adapt) {
    const float pn = sqrtf(norms[2 * c.seg]), un = sqrtf(norms[2 * c.seg + 1]);
    q = (pn > 0.f && un > 0.f) ? trust * pn / un : 1.f;
  }
  const float wd_eff = adapt ? wd : 0.f;
  const float om = 1.f - ema_m;
  const bool has_t = teacher != nullptr;
  // 16-byte vectors over the aligned body (segments start on 256-byte boundaries), scalars for the tail
  const int n4 = ((c.begin & 3) == 0) ? (c.len >> 2) : 0;
  float4* p4 = reinterpret_cast<float4*>(p + c.begin);
  const float4* g4 = reinterpret_cast<const float4*>(g + c.begin);
  float4* m4 = reinterpret_cast<float4*>(mu + c.begin);
  float4* t4 = has_t ? reinterpret_cast<float4*>(teacher + c.begin) : nullptr;
  for (int i = threadIdx.x; i < n4; i += kThreads) {
    float4 pv = p4[i], mv = m4[i];
    const float4 gv = g4[i];
    const bool t_ok = has_t && (c.begin + 4 * (int64_t)i + 3 < teacher_n);
    float4 tv = t_ok ? t4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
#define TSP_LARS1(X)                                                   \
    {                                                                  \
      const float dp = q * (grad_scale * gv.X + wd_eff * pv.X);        \
      mv.X = mom * mv.X + dp;                                          \
      pv.X -= lr * mv.X;                                               \
      tv.X = ema_m * tv.X + om * pv.X;                                 \
    }
    TSP_LARS1(x) TSP_LARS1(y) TSP_LARS1(z) TSP_LARS1(w)
#undef TSP_LARS1
    p4[i] = pv;
    m4[i] = mv;
    if (t_ok) t4[i] = tv;
  }
  for (int i = (n4 << 2) + threadIdx.x; i < c.len; i += kThreads) {
    const int64_t k = c.begin + i;
    const float pv = p[k];
    const float dp = q * (grad_scale * g[k] + wd_eff * pv);
    const float m2 = mom * mu[k] + dp;
    mu[k] = m2;
    const float np = pv - lr * m2;
    p[k] = np;
    if (has_t && k < teacher_n) teacher[k] = ema_m * teacher[k] + om * np;
  }
}

// AdamW (decoupled weight decay), per-segment hyper-parameters: lr, beta1, beta2, eps, wd, bias1, bias2
__global__ void __launch_bounds__(kThreads) adamw_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                         float* __restrict__ m, float* __restrict__ v,
                                                         const int64_t* __restrict__ chunks,
                                                         const float* __restrict__ seg_hp, float grad_scale,
                                                         float* __restrict__ teacher, int64_t teacher_n, float ema_m) {
  const ChunkView c = load_chunk(chunks, blockIdx.x);
  const float* hp = seg_hp + 7 * (int64_t)c.seg;
  const float lr = hp[0], b1 = hp[1], b2 = hp[2], eps = hp[3], wd = hp[4], bc1 = hp[5], bc2 = hp[6];
  const float om = 1.f - ema_m;
  const float step = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  for (int i = threadIdx.x; i < c.len; i += kThreads) {
    const int64_t k = c.begin + i;
    const float gv = grad_scale * g[k];
    float pv = p[k] * (1.f - lr * wd);
    const float mv = b1 * m[k] + (1.f - b1) * gv;
    const float vv = b2 * v[k] + (1.f - b2) * gv * gv;
    m[k] = mv; v[k] = vv;
    pv -= step * mv / (sqrtf(vv) * inv_sqrt_bc2 + eps);
    p[k] = pv;
    if (teacher != nullptr && k < teacher_n) teacher[k] = ema_m * teacher[k] + om * pv;
  }
}

// SGD with momentum / nesterov / L2 weight decay; per-segment: lr, momentum, dampening, wd, nesterov, first_step
__global__ void __launch_bounds__(kThreads) sgd_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                       float* __restrict__ buf, const int64_t* __restrict__ chunks,
                                                       const float* __restrict__ seg_hp, float grad_scale,
                                                       float* __restrict__ teacher, int64_t teacher_n, float ema_m) {
  const ChunkView c = load_chunk(chunks, blockIdx.x);
  const float* hp = seg_hp + 6 * (int64_t)c.seg;
  const float lr = hp[0], mom = hp[1], damp = hp[2], wd = hp[3];
  const bool nesterov = hp[4] != 0.f, first = hp[5] != 0.f;
  const float om = 1.f - ema_m;
  for (int i = threadIdx.x; i < c.len; i += kThreads) {
    const int64_t k = c.begin + i;
    const float pv = p[k];
    float d = grad_scale * g[k] + wd * pv;
    if (mom != 0.f) {
      const float b = first ? d : mom * buf[k] + (1.f - damp) * d;
      buf[k] = b;
      d = nesterov ? d + mom * b : b;
    }
    const float np = pv - lr * d;
    p[k] = np;
    if (teacher != nullptr && k < teacher_n) teacher[k] = ema_m * teacher[k] + om * np;
  }
}

inline int ema_grid(int64_t n) {
  int64_t blocks = (n / 4 + kThreads - 1) / kThreads;
  const int64_t cap = 148 * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace

extern "C" {

int tsp_ema_update(float* teacher, const float* student, int64_t n, float momentum, void* bf16_shadow,
                   cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(teacher) | reinterpret_cast<uintptr_t>(student)) & 15) return -2;
  ema_kernel<<<ema_grid(n), kThreads, 0, stream>>>(teacher, student, n, momentum,
                                                  reinterpret_cast<__nv_bfloat16*>(bf16_shadow));
  return TSP_LAUNCH_CHECK();
}

int tsp_lars_step(float* p, const float* g, float* mu, const int64_t* chunks, int n_chunks, const float* seg_hp,
                  float grad_scale, float* norms, int n_seg, float* teacher, int64_t teacher_n, float ema_m,
                  cudaStream_t stream) {
  if (n_chunks <= 0) return 0;
  cudaError_t e = cudaMemsetAsync(norms, 0, sizeof(float) * 2 * (size_t)n_seg, stream);
  if (e != cudaSuccess) return (int)e;
  lars_norms_kernel<<<n_chunks, kThreads, 0, stream>>>(p, g, chunks, seg_hp, grad_scale, norms);
  lars_apply_kernel<<<n_chunks, kThreads, 0, stream>>>(p, g, mu, chunks, seg_hp, grad_scale, norms, teacher,
                                                       teacher_n, ema_m);
  return TSP_LAUNCH_CHECK();
}

int tsp_lars_norms(const float* p, const float* g, const int64_t* chunks, int n_chunks, const float* seg_hp,
                   float grad_scale, float* norms, int n_seg, cudaStream_t stream) {
  if (n_chunks <= 0) return 0;
  cudaError_t e = cudaMemsetAsync(norms, 0, sizeof(float) * 2 * (size_t)n_seg, stream);
  if (e != cudaSuccess) return (int)e;
  lars_norms_kernel<<<n_chunks, kThreads, 0, stream>>>(p, g, chunks, seg_hp, grad_scale, norms);
  return TSP_LAUNCH_CHECK();
}

int tsp_lars_apply(float* p, const float* g, float* mu, const int64_t* chunks, int n_chunks, const float* seg_hp,
                   float grad_scale, const float* norms, float* teacher, int64_t teacher_n, float ema_m,
                   cudaStream_t stream) {
  if (n_chunks <= 0) return 0;
  lars_apply_kernel<<<n_chunks, kThreads, 0, stream>>>(p, g, mu, chunks, seg_hp, grad_scale, norms, teacher,
                                                       teacher_n, ema_m);
  return TSP_LAUNCH_CHECK();
}

int tsp_adamw_step(float* p, const float* g, float* m, float* v, const int64_t* chunks, int n_chunks,
                   const float* seg_hp, float grad_scale, float* teacher, int64_t teacher_n, float ema_m,
                   cudaStream_t stream) {
  if (n_chunks <= 0) return 0;
  adamw_kernel<<<n_chunks, kThreads, 0, stream>>>(p, g, m, v, chunks, seg_hp, grad_scale, teacher, teacher_n, ema_m);
  return TSP_LAUNCH_CHECK();
}

int tsp_sgd_step(float* p, const float* g, float* buf, const int64_t* chunks, int n_chunks, const float* seg_hp,
                 float grad_scale, float* teacher, int64_t teacher_n, float ema_m, cudaStream_t stream) {
  if (n_chunks <= 0) return 0;
  sgd_kernel<<<n_chunks, kThreads, 0, stream>>>(p, g, buf, chunks, seg_hp, grad_scale, teacher, teacher_n, ema_m);
  return TSP_LAUNCH_CHECK();
}

}  // extern "C"
