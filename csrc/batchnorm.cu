// Microbatch BatchNorm for channels-last activations, fused with ReLU and the residual add (sm_100a).
//
// Reference: `tspipe/batchnorm.py:45-120` - F.batch_norm on the microbatch plus two extra full reductions
// (`input.sum`, `(input**2).sum`) for the deferred running statistics, followed by separate ReLU and
// residual-add kernels in the ResNet blocks (`benchmarks/byol/models/resnet_base_network.py`).  On B200 those
// memory-bound passes take more time than the convolutions.  Here:
//   forward  = statistics pass (per-channel sum / sum of squares; these ARE the deferred accumulators)
//              + one pass y = relu(scale*x + shift [+ residual]);
//   backward = reduction pass (sum dy', sum dy'*xhat with dy' = dy masked by y > 0; writes dy' as the residual
//              gradient when there is a residual) + one pass for dx.
// x is viewed as [M, C] with C contiguous (NHWC or [N, C]); C % 8 == 0; statistics in fp32.
#include "common.cuh"
#include "tspipe_kernels.h"

namespace {

constexpr int kBlock = 256;

struct Tile {
  int tx_n;   // threads along the channel-vector axis
  int ty_n;   // rows processed in parallel by a block
};

__host__ __device__ inline Tile make_tile(int cpv) {
  Tile t;
  t.tx_n = cpv < kBlock ? cpv : kBlock;
  t.ty_n = kBlock / t.tx_n;
  if (t.ty_n < 1) t.ty_n = 1;
  return t;
}

// ---------------------------------------------------------------------------------------------
// per-channel sums:  out[c] += sum_rows a(r,c),  out[C + c] += sum_rows b(r,c)
//   MODE 0 (forward statistics): a = x, b = x*x
//   MODE 1 (backward reduction): a = dy', b = dy' * (x - mean) * rstd with dy' = dy masked by the ReLU:
//          mask from y > 0 when `y` is given (residual case), else recomputed as scale*x + shift > 0 when
//          `relu` is set (no extra tensor read); optionally stores dy' to dres.
// grid = (row blocks, channel slabs); block = tx_n * ty_n threads; smem = ty_n * tx_n * 16 floats.
// ---------------------------------------------------------------------------------------------
template <typename T, int MODE>
__global__ void __launch_bounds__(kBlock, MODE == 0 ? 5 : 2) bn_colsum_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                           const T* __restrict__ y, T* __restrict__ dres,
                                                           const float* __restrict__ mean_rstd,
                                                           const float* __restrict__ w, const float* __restrict__ bias,
                                                           int relu, int64_t m, int c, float* __restrict__ out) {
  extern __shared__ float sm[];
  {   // blockIdx.z = segment: an independent group of m rows with its own statistics
    const int64_t so = (int64_t)blockIdx.z * m * c;
    x += so;
    if (dy != nullptr) dy += so;
    if (y != nullptr) y += so;
    if (dres != nullptr) dres += so;
    if (mean_rstd != nullptr) mean_rstd += (int64_t)blockIdx.z * 2 * c;
    out += (int64_t)blockIdx.z * 2 * c;
  }
  const int cpv = c >> 3;
  const Tile tl = make_tile(cpv);
  const int tx = threadIdx.x % tl.tx_n, ty = threadIdx.x / tl.tx_n;
  const int cg = blockIdx.y * tl.tx_n + tx;
  const bool active = (ty < tl.ty_n) && (cg < cpv);
  float a[8], b[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { a[e] = 0.f; b[e] = 0.f; }
  float mu[8], rs[8], sc[8], sh[8];
  const bool recompute_mask = (MODE == 1) && relu && (y == nullptr);
  if (MODE == 1 && active) {
    tsp::ld8(mean_rstd, (int64_t)cg * 8, mu);
    tsp::ld8(mean_rstd + c, (int64_t)cg * 8, rs);
    if (recompute_mask) {
      float wv[8], bv[8];
      tsp::ld8(w, (int64_t)cg * 8, wv);
      tsp::ld8(bias, (int64_t)cg * 8, bv);
#pragma unroll
      for (int e = 0; e < 8; ++e) { sc[e] = wv[e] * rs[e]; sh[e] = bv[e] - mu[e] * sc[e]; }
    }
  }
  if (active) {
    // each block owns one contiguous range of rows: consecutive iterations stream consecutive memory
    const int64_t rows_per_block = (m + gridDim.x - 1) / gridDim.x;
    const int64_t r_begin = (int64_t)blockIdx.x * rows_per_block;
    const int64_t r_end = r_begin + rows_per_block < m ? r_begin + rows_per_block : m;
    const int64_t step = tl.ty_n;
    const int64_t col = (int64_t)cg * 8;
    int64_t r = r_begin + ty;
    if (MODE == 0) {
      // eight independent 16/32-byte loads in flight per thread before any arithmetic (raw registers)
      for (; r + 7 * step < r_end; r += 8 * step) {
        tsp::Raw8<T> raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) tsp::ldraw(x, (r + u * step) * c + col, raw[u]);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          float v[8];
          tsp::cvt8(raw[u], v);
#pragma unroll
          for (int e = 0; e < 8; ++e) { a[e] += v[e]; b[e] += v[e] * v[e]; }
        }
      }
      for (; r < r_end; r += step) {
        float v0[8];
        tsp::ld8(x, r * c + col, v0);
#pragma unroll
        for (int e = 0; e < 8; ++e) { a[e] += v0[e]; b[e] += v0[e] * v0[e]; }
      }
    } else {
      for (; r < r_end; r += 2 * step) {
        const bool two = r + step < r_end;
        const int64_t off0 = r * c + col, off1 = (r + step) * c + col;
        float x0[8], x1[8], g0[8], g1[8], y0[8], y1[8];
        tsp::ld8(x, off0, x0);
        tsp::ld8(dy, off0, g0);
        if (y != nullptr) tsp::ld8(y, off0, y0);
        if (two) {
          tsp::ld8(x, off1, x1);
          tsp::ld8(dy, off1, g1);
          if (y != nullptr) tsp::ld8(y, off1, y1);
        }
        if (y != nullptr) {
#pragma unroll
          for (int e = 0; e < 8; ++e) { g0[e] = y0[e] > 0.f ? g0[e] : 0.f; if (two) g1[e] = y1[e] > 0.f ? g1[e] : 0.f; }
        } else if (recompute_mask) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            g0[e] = (x0[e] * sc[e] + sh[e]) > 0.f ? g0[e] : 0.f;
            if (two) g1[e] = (x1[e] * sc[e] + sh[e]) > 0.f ? g1[e] : 0.f;
          }
        }
        if (dres != nullptr) { tsp::st8(dres, off0, g0); if (two) tsp::st8(dres, off1, g1); }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          a[e] += g0[e]; b[e] += g0[e] * (x0[e] - mu[e]) * rs[e];
          if (two) { a[e] += g1[e]; b[e] += g1[e] * (x1[e] - mu[e]) * rs[e]; }
        }
      }
    }
  }
  // reduce over ty through shared memory, then one atomic per channel per block
  float* mine = sm + ((int64_t)ty * tl.tx_n + tx) * 16;
  if (ty < tl.ty_n) {
#pragma unroll
    for (int e = 0; e < 8; ++e) { mine[e] = a[e]; mine[8 + e] = b[e]; }
  }
  __syncthreads();
  if (ty == 0 && cg < cpv) {
    for (int k = 1; k < tl.ty_n; ++k) {
      const float* o = sm + ((int64_t)k * tl.tx_n + tx) * 16;
#pragma unroll
      for (int e = 0; e < 8; ++e) { a[e] += o[e]; b[e] += o[8 + e]; }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      atomicAdd(out + cg * 8 + e, a[e]);
      atomicAdd(out + c + cg * 8 + e, b[e]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Streaming version of the per-channel sums for bf16 (same MODEs and results as bn_colsum_kernel).
//
// A read-only pass is bound by how many bytes an SM keeps in flight, not by arithmetic.  Instead of raising
// occupancy, one producer thread per CTA streams the CTA's contiguous row range through a ring of shared-memory
// buffers with bulk asynchronous copies (cp.async.bulk, completion on an mbarrier; 64 - 192 KB in flight per SM
// with no registers tied up), and 8 consumer warps read the buffers with conflict-free 16-byte loads.  With
// c/8 a power of two <= 256, consumer thread t always meets the channels 8 * (t % (c/8)) .. +7, so its partial
// sums stay in registers; one shared-memory reduction and one atomic per channel per CTA finish the job.
// Measured on [256*56*56, 256] bf16 (411 MB): 84 us = 4.9 TB/s, the same as a kernel that only reads.
//
// Waits are bounded (kStreamSpin polls); a wait that runs out sets g_bn_status and every role leaves its loop.
// ---------------------------------------------------------------------------------------------
constexpr int kStreamConsumers = 256;
constexpr int kStreamThreads = kStreamConsumers + 32;
constexpr int kStreamStages = 4;
constexpr uint32_t kStreamSpin = 1u << 22;
__device__ int g_bn_status = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool stream_wait(uint64_t* bar, uint32_t parity, int code) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < kStreamSpin; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    // The error word lives in global memory: the round trip to L2 per failed poll is the back-off of this loop
    // (polling flat out slowed the statistics pass from 38 us to 77 us on a 205 MB activation: the 8 waiting
    // warps took issue slots from the producer thread).
    if (*((volatile int*)&g_bn_status) != 0) return false;
  }
  atomicCAS(&g_bn_status, 0, code);
  return false;
}
__device__ __forceinline__ void stream_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) { const float2 f = __bfloat1622float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
}

// NARR = number of streamed arrays: MODE 0: x; MODE 1: x, dy (, y).  `chunk` bytes per array and stage.
template <int MODE>
__global__ void __launch_bounds__(kStreamThreads, 1)
bn_colsum_stream_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                        const __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ dres,
                        const float* __restrict__ mean_rstd, const float* __restrict__ w,
                        const float* __restrict__ bias, int relu, int64_t m, int c, int chunk,
                        float* __restrict__ out) {
  extern __shared__ __align__(128) uint8_t stream_smem[];
  {   // blockIdx.y = segment: an independent group of m rows with its own statistics
    const int64_t so = (int64_t)blockIdx.y * m * c;
    x += so;
    if (dy != nullptr) dy += so;
    if (y != nullptr) y += so;
    if (dres != nullptr) dres += so;
    if (mean_rstd != nullptr) mean_rstd += (int64_t)blockIdx.y * 2 * c;
    out += (int64_t)blockIdx.y * 2 * c;
  }
  const int narr = MODE == 0 ? 1 : (y != nullptr ? 3 : 2);
  const int stage_bytes = narr * chunk;
  uint8_t* bufs = stream_smem;
  uint64_t* full = (uint64_t*)(stream_smem + kStreamStages * stage_bytes);
  uint64_t* empty = full + kStreamStages;
  float* red = (float*)(empty + kStreamStages);            // [kStreamConsumers][16]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row_bytes = c * 2, cpv = c >> 3;
  const int rows_per_chunk = chunk / row_bytes;
  const int64_t rows_per_block = (m + gridDim.x - 1) / gridDim.x;
  const int64_t r_begin = (int64_t)blockIdx.x * rows_per_block;
  const int64_t r_end = r_begin + rows_per_block < m ? r_begin + rows_per_block : m;
  const int64_t nrows = r_end > r_begin ? r_end - r_begin : 0;
  const int n_chunks = (int)((nrows + rows_per_chunk - 1) / rows_per_chunk);
  if (tid == 0) {
    for (int s = 0; s < kStreamStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(full + s)), "r"(1));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(empty + s)), "r"(kStreamConsumers / 32));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  float a[8], b[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { a[e] = 0.f; b[e] = 0.f; }
  if (warp == kStreamConsumers / 32) {
    // ---------------- producer ----------------
    if (lane == 0) {
      for (int i = 0; i < n_chunks; ++i) {
        const int s = i % kStreamStages;
        const uint32_t round = i / kStreamStages;
        if (round > 0 && !stream_wait(empty + s, (round - 1) & 1, 1)) break;
        const int64_t r0 = r_begin + (int64_t)i * rows_per_chunk;
        const int64_t rows = r_end - r0 < rows_per_chunk ? r_end - r0 : rows_per_chunk;
        const uint32_t bytes = (uint32_t)(rows * row_bytes);
        const int64_t off = r0 * row_bytes;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(full + s)),
                     "r"(bytes * (uint32_t)narr)
                     : "memory");
        uint8_t* dst = bufs + s * stage_bytes;
        stream_load(dst, (const uint8_t*)x + off, bytes, full + s);
        if (MODE == 1) {
          stream_load(dst + chunk, (const uint8_t*)dy + off, bytes, full + s);
          if (narr == 3) stream_load(dst + 2 * chunk, (const uint8_t*)y + off, bytes, full + s);
        }
      }
    }
  } else {
    // ---------------- consumers ----------------
    const int cv = tid % cpv;                               // this thread's channel vector, fixed for all chunks
    float mu[8], rs[8], sc[8], sh[8];
    const bool recompute_mask = (MODE == 1) && relu && (y == nullptr);
    if (MODE == 1) {
      tsp::ld8(mean_rstd, (int64_t)cv * 8, mu);
      tsp::ld8(mean_rstd + c, (int64_t)cv * 8, rs);
      if (recompute_mask) {
        float wv[8], bv[8];
        tsp::ld8(w, (int64_t)cv * 8, wv);
        tsp::ld8(bias, (int64_t)cv * 8, bv);
#pragma unroll
        for (int e = 0; e < 8; ++e) { sc[e] = wv[e] * rs[e]; sh[e] = bv[e] - mu[e] * sc[e]; }
      }
    }
    for (int i = 0; i < n_chunks; ++i) {
      const int s = i % kStreamStages;
      const uint32_t round = i / kStreamStages;
      if (!stream_wait(full + s, round & 1, 2)) break;
      const int64_t r0 = r_begin + (int64_t)i * rows_per_chunk;
      const int64_t rows = r_end - r0 < rows_per_chunk ? r_end - r0 : rows_per_chunk;
      const int nvec = (int)(rows * cpv);
      const uint4* sx = (const uint4*)(bufs + s * stage_bytes);
      if (MODE == 0) {
        int v = tid;
        for (; v + 3 * kStreamConsumers < nvec; v += 4 * kStreamConsumers) {
          const uint4 q0 = sx[v], q1 = sx[v + kStreamConsumers], q2 = sx[v + 2 * kStreamConsumers],
                      q3 = sx[v + 3 * kStreamConsumers];
          float f[8];
          unpack8(q0, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) { a[e] += f[e]; b[e] += f[e] * f[e]; }
          unpack8(q1, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) { a[e] += f[e]; b[e] += f[e] * f[e]; }
          unpack8(q2, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) { a[e] += f[e]; b[e] += f[e] * f[e]; }
          unpack8(q3, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) { a[e] += f[e]; b[e] += f[e] * f[e]; }
        }
        for (; v < nvec; v += kStreamConsumers) {
          float f[8];
          unpack8(sx[v], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) { a[e] += f[e]; b[e] += f[e] * f[e]; }
        }
      } else {
        const uint4* sg = (const uint4*)(bufs + s * stage_bytes + chunk);
        const uint4* sy = (const uint4*)(bufs + s * stage_bytes + 2 * chunk);
        uint4* gres = dres == nullptr ? nullptr : (uint4*)((uint8_t*)dres + r0 * row_bytes);
#pragma unroll 2
        for (int v = tid; v < nvec; v += kStreamConsumers) {
          float xv[8], g[8];
          unpack8(sx[v], xv);
          unpack8(sg[v], g);
          if (narr == 3) {
            float yv[8];
            unpack8(sy[v], yv);
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] = yv[e] > 0.f ? g[e] : 0.f;
          } else if (recompute_mask) {
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] = (xv[e] * sc[e] + sh[e]) > 0.f ? g[e] : 0.f;
          }
          if (gres != nullptr) {
            uint4 raw;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(g[2 * k], g[2 * k + 1]);
            gres[v] = raw;
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) { a[e] += g[e]; b[e] += g[e] * (xv[e] - mu[e]) * rs[e]; }
        }
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(empty + s)) : "memory");
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) { red[tid * 16 + e] = a[e]; red[tid * 16 + 8 + e] = b[e]; }
  }
  if (*((volatile int*)&g_bn_status) != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);        // let copies that are still in flight land
  }
  __syncthreads();
  // threads with equal tid % cpv hold the same channels: sum the groups, one atomic per channel and CTA
  const int groups = kStreamConsumers / cpv;
  for (int p = tid; p < 16 * cpv; p += kStreamThreads) {
    const int cv = p >> 4, e = p & 15;
    float acc = 0.f;
    for (int g = 0; g < groups; ++g) acc += red[(g * cpv + cv) * 16 + e];
    atomicAdd(out + (e < 8 ? 0 : c) + cv * 8 + (e & 7), acc);
  }
}

// ---------------------------------------------------------------------------------------------
// forward apply: y = act(scale*x + shift [+ res]).
//   training: mean/var from `sums` (sum, sum of squares over m rows); block 0 saves mean / rstd and folds the
//             sums into the deferred accumulators (acc_sum, acc_sumsq) when given.
//   eval:     mean/var from `fixed` ([mean | var]).
// dynamic smem: 2*c floats (scale | shift).  A thread's channel group is loop-invariant whenever the grid
// stride is a multiple of c/8 (all power-of-two widths), so scale/shift then stay in registers.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kBlock) bn_apply_kernel(const T* __restrict__ x, const T* __restrict__ res,
                                                          T* __restrict__ y, const float* __restrict__ sums,
                                                          const float* __restrict__ fixed,
                                                          const float* __restrict__ w, const float* __restrict__ b,
                                                          float* __restrict__ save_mean_rstd,
                                                          float* __restrict__ acc_sum, float* __restrict__ acc_sumsq,
                                                          float* __restrict__ acc_count, int64_t acc_seg_stride,
                                                          int64_t m, int c, float eps, int relu) {
  extern __shared__ float sm[];
  {   // blockIdx.y = segment: m rows with their own statistics (and their own set of accumulators)
    const int64_t so = (int64_t)blockIdx.y * m * c;
    x += so;
    y += so;
    if (res != nullptr) res += so;
    if (sums != nullptr) sums += (int64_t)blockIdx.y * 2 * c;
    if (save_mean_rstd != nullptr) save_mean_rstd += (int64_t)blockIdx.y * 2 * c;
    if (acc_sum != nullptr) { acc_sum += blockIdx.y * acc_seg_stride; acc_sumsq += blockIdx.y * acc_seg_stride; }
    if (acc_count != nullptr) acc_count += blockIdx.y * acc_seg_stride;
  }
  float* scale = sm;
  float* shift = sm + c;
  const float inv_m = 1.f / (float)m;
  for (int i = threadIdx.x; i < c; i += blockDim.x) {
    float mean, var;
    if (fixed != nullptr) {
      mean = fixed[i]; var = fixed[c + i];
    } else {
      const float s = sums[i], q = sums[c + i];
      mean = s * inv_m;
      var = fmaxf(q * inv_m - mean * mean, 0.f);
      if (blockIdx.x == 0) {
        if (acc_sum != nullptr) { acc_sum[i] += s; acc_sumsq[i] += q; }
        if (acc_count != nullptr) acc_count[i] += (float)m;
      }
    }
    const float rstd = rsqrtf(var + eps);
    if (blockIdx.x == 0 && save_mean_rstd != nullptr) { save_mean_rstd[i] = mean; save_mean_rstd[c + i] = rstd; }
    const float sc = (w ? w[i] : 1.f) * rstd;
    scale[i] = sc;
    shift[i] = (b ? b[i] : 0.f) - mean * sc;
  }
  __syncthreads();
  const int cpv = c >> 3;
  const int64_t nvec = m * cpv;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  int cg = (int)(i % cpv);
  const int dcg = (int)(stride % cpv);
  float sc[8], sh[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { sc[e] = scale[cg * 8 + e]; sh[e] = shift[cg * 8 + e]; }
  if (dcg == 0) {
    // four independent vectors per thread and trip: all loads are issued before the first use
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      tsp::Raw8<T> xr[4], rr[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) tsp::ldraw(x, (i + u * stride) * 8, xr[u]);
      if (res != nullptr) {
#pragma unroll
        for (int u = 0; u < 4; ++u) tsp::ldraw(res, (i + u * stride) * 8, rr[u]);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float v[8], o[8];
        tsp::cvt8(xr[u], v);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[e] * sc[e] + sh[e];
        if (res != nullptr) {
          float r[8];
          tsp::cvt8(rr[u], r);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += r[e];
        }
        if (relu) {
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = fmaxf(o[e], 0.f);
        }
        tsp::st8(y, (i + u * stride) * 8, o);
      }
    }
  }
  for (; i < nvec; i += stride) {
    float v[8], o[8];
    tsp::ld8(x, i * 8, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = v[e] * sc[e] + sh[e];
    if (res != nullptr) {
      float r[8];
      tsp::ld8(res, i * 8, r);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] += r[e];
    }
    if (relu) {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = fmaxf(o[e], 0.f);
    }
    tsp::st8(y, i * 8, o);
    if (dcg != 0) {
      cg += dcg;
      if (cg >= cpv) cg -= cpv;
#pragma unroll
      for (int e = 0; e < 8; ++e) { sc[e] = scale[cg * 8 + e]; sh[e] = shift[cg * 8 + e]; }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// backward apply: dx = w*rstd * (dy' - sum(dy')/m - xhat * sum(dy'*xhat)/m), dy' masked as in the reduction
// (by y > 0 when `y` is given, by scale*x + shift > 0 when `relu` is set and y is null).
// Per element: dx = A*dy' + B*x + D with A = w*rstd, B = -A*rstd*k2, D = -A*k1 - B*mean.
// dynamic smem: 5*c floats (A | B | D | scale | shift)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kBlock) bn_bwd_apply_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                              const T* __restrict__ y,
                                                              const float* __restrict__ mean_rstd,
                                                              const float* __restrict__ w,
                                                              const float* __restrict__ bias, int relu,
                                                              const float* __restrict__ sums, T* __restrict__ dx,
                                                              int64_t m, int c) {
  extern __shared__ float sm[];
  {   // blockIdx.y = segment
    const int64_t so = (int64_t)blockIdx.y * m * c;
    dy += so;
    x += so;
    dx += so;
    if (y != nullptr) y += so;
    mean_rstd += (int64_t)blockIdx.y * 2 * c;
    sums += (int64_t)blockIdx.y * 2 * c;
  }
  float* s_a = sm;
  float* s_b = sm + c;
  float* s_d = sm + 2 * c;
  float* s_sc = sm + 3 * c;
  float* s_sh = sm + 4 * c;
  const float inv_m = 1.f / (float)m;
  const bool recompute_mask = relu && (y == nullptr);
  for (int i = threadIdx.x; i < c; i += blockDim.x) {
    const float mean = mean_rstd[i], rs = mean_rstd[c + i];
    const float k1 = sums[i] * inv_m, k2 = sums[c + i] * inv_m;
    const float wv = w ? w[i] : 1.f;
    const float A = wv * rs;
    const float B = -A * rs * k2;
    s_a[i] = A;
    s_b[i] = B;
    s_d[i] = -A * k1 - B * mean;
    s_sc[i] = A;
    s_sh[i] = (bias ? bias[i] : 0.f) - mean * A;
  }
  __syncthreads();
  const int cpv = c >> 3;
  const int64_t nvec = m * cpv;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  int cg = (int)(i % cpv);
  const int dcg = (int)(stride % cpv);
  float A[8], B[8], D[8], sh[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { A[e] = s_a[cg * 8 + e]; B[e] = s_b[cg * 8 + e]; D[e] = s_d[cg * 8 + e]; sh[e] = s_sh[cg * 8 + e]; }
  if (dcg == 0) {
    // two independent vectors per thread and trip (4 - 6 loads in flight)
    for (; i + stride < nvec; i += 2 * stride) {
      tsp::Raw8<T> gr[2], xr[2], yr[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) { tsp::ldraw(dy, (i + u * stride) * 8, gr[u]); tsp::ldraw(x, (i + u * stride) * 8, xr[u]); }
      if (y != nullptr) {
#pragma unroll
        for (int u = 0; u < 2; ++u) tsp::ldraw(y, (i + u * stride) * 8, yr[u]);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        float g[8], xv[8], o[8];
        tsp::cvt8(gr[u], g);
        tsp::cvt8(xr[u], xv);
        if (y != nullptr) {
          float yv[8];
          tsp::cvt8(yr[u], yv);
#pragma unroll
          for (int e = 0; e < 8; ++e) g[e] = yv[e] > 0.f ? g[e] : 0.f;
        } else if (recompute_mask) {
#pragma unroll
          for (int e = 0; e < 8; ++e) g[e] = (xv[e] * A[e] + sh[e]) > 0.f ? g[e] : 0.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = A[e] * g[e] + B[e] * xv[e] + D[e];
        tsp::st8(dx, (i + u * stride) * 8, o);
      }
    }
  }
  for (; i < nvec; i += stride) {
    float g[8], xv[8], o[8];
    tsp::ld8(dy, i * 8, g);
    tsp::ld8(x, i * 8, xv);
    if (y != nullptr) {
      float yv[8];
      tsp::ld8(y, i * 8, yv);
#pragma unroll
      for (int e = 0; e < 8; ++e) g[e] = yv[e] > 0.f ? g[e] : 0.f;
    } else if (recompute_mask) {
#pragma unroll
      for (int e = 0; e < 8; ++e) g[e] = (xv[e] * A[e] + sh[e]) > 0.f ? g[e] : 0.f;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = A[e] * g[e] + B[e] * xv[e] + D[e];
    tsp::st8(dx, i * 8, o);
    if (dcg != 0) {
      cg += dcg;
      if (cg >= cpv) cg -= cpv;
#pragma unroll
      for (int e = 0; e < 8; ++e) { A[e] = s_a[cg * 8 + e]; B[e] = s_b[cg * 8 + e]; D[e] = s_d[cg * 8 + e]; sh[e] = s_sh[cg * 8 + e]; }
    }
  }
}

inline int row_blocks(int64_t m, int ty_n, int slabs) {
  int64_t want = (m + ty_n - 1) / ty_n;
  int64_t cap = (148 * 8) / (slabs > 0 ? slabs : 1);
  if (cap < 1) cap = 1;
  // keep at least ~32 rows per thread-row so that the atomics stay a small part of the work
  int64_t by_work = (m + (int64_t)ty_n * 32 - 1) / ((int64_t)ty_n * 32);
  if (by_work < 1) by_work = 1;
  int64_t g = want < cap ? want : cap;
  if (g > by_work) g = by_work;
  return (int)(g < 1 ? 1 : g);
}

inline int elem_blocks(int64_t nvec) {
  int64_t b = (nvec + kBlock - 1) / kBlock;
  if (b > 148 * 16) b = 148 * 16;
  return (int)(b < 1 ? 1 : b);
}

// Streaming kernel eligibility: bf16, c/8 a power of two in [8, 256], enough rows to give every CTA work.
inline bool stream_ok(int64_t m, int c, int dtype) {
  const int cpv = c / 8;
  return dtype == TSP_DTYPE_BF16 && cpv >= 8 && cpv <= kStreamConsumers && (cpv & (cpv - 1)) == 0 &&
         m * (int64_t)c * 2 >= (1 << 20);
}

template <int MODE>
int launch_stream(const void* x, const void* dy, const void* y, void* dres, const float* mean_rstd, const float* w,
                  const float* bias, int relu, int64_t m, int c, int segs, float* sums, cudaStream_t stream) {
  const int narr = MODE == 0 ? 1 : (y != nullptr ? 3 : 2);
  const int64_t row_bytes = (int64_t)c * 2;
  // bytes per array and stage: 32 KB for one streamed array, 16 KB for two or three (at most 192 KB of ring);
  // smaller for small tensors so that every CTA still gets a few chunks to overlap
  int chunk = narr == 1 ? 32768 : 16384;
  while (chunk > 8192 && m * row_bytes < (int64_t)148 * 4 * chunk) chunk >>= 1;
  if (chunk < row_bytes) chunk = (int)row_bytes;
  const int64_t rows_per_chunk = chunk / row_bytes;
  int64_t grid = 148 / segs;                     // CTAs per segment: one CTA per SM over all segments
  if (grid < 1) grid = 1;
  const int64_t want = (m + 2 * rows_per_chunk - 1) / (2 * rows_per_chunk);
  if (want < grid) grid = want < 1 ? 1 : want;
  const size_t smem = (size_t)kStreamStages * narr * chunk + 2 * kStreamStages * 8 + kStreamConsumers * 16 * 4;
  auto kern = bn_colsum_stream_kernel<MODE>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  kern<<<dim3((unsigned)grid, (unsigned)segs), kStreamThreads, smem, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                    (const __nv_bfloat16*)y, (__nv_bfloat16*)dres, mean_rstd, w, bias,
                                                    relu, m, c, chunk, sums);
  return TSP_LAUNCH_CHECK();
}

}  // namespace

extern "C" {

// 0 while no bounded wait of the streaming statistics kernels has run out on the current device; the first
// failing role otherwise (1 producer, 2 consumer).  Synchronises the device.  `reset` != 0 clears it.
int tsp_bn_stream_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_bn_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_bn_status, &zero, sizeof(int));
  }
  return v;
}

// sums [2*c] fp32 is zeroed here, then receives per-channel sum(x) and sum(x^2).
// All four entry points take the activation as `segs` consecutive groups of m / segs rows; every group is
// normalised with its own statistics (two augmented views stacked along the batch axis).  Per-group arrays are
// laid out group-major: sums [segs][2c], save_mean_rstd [segs][2c].
int tsp_bn_stats(const void* x, int64_t m, int c, int dtype, float* sums, int segs, cudaStream_t stream) {
  if (m <= 0) return 0;
  if (c % 8 != 0 || c > 8192 || segs < 1 || m % segs != 0) return -3;
  cudaError_t e = cudaMemsetAsync(sums, 0, sizeof(float) * 2 * (size_t)c * segs, stream);
  if (e != cudaSuccess) return (int)e;
  m /= segs;
  if (stream_ok(m, c, dtype))
    return launch_stream<0>(x, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, m, c, segs, sums, stream);
  const int cpv = c / 8;
  const Tile tl = make_tile(cpv);
  const int slabs = (cpv + tl.tx_n - 1) / tl.tx_n;
  dim3 grid(row_blocks(m, tl.ty_n, slabs), slabs, segs);
  const size_t smem = sizeof(float) * 16 * (size_t)tl.tx_n * tl.ty_n;
  if (dtype == TSP_DTYPE_BF16)
    bn_colsum_kernel<__nv_bfloat16, 0><<<grid, kBlock, smem, stream>>>((const __nv_bfloat16*)x, nullptr, nullptr, nullptr,
                                                                       nullptr, nullptr, nullptr, 0, m, c, sums);
  else
    bn_colsum_kernel<float, 0><<<grid, kBlock, smem, stream>>>((const float*)x, nullptr, nullptr, nullptr, nullptr, nullptr,
                                                               nullptr, 0, m, c, sums);
  return TSP_LAUNCH_CHECK();
}

// acc_sum / acc_sumsq / acc_count (optional): accumulators of the deferred running statistics; group g adds into
// acc + g * acc_seg_stride, so that each group's mini-batch can be committed on its own.
int tsp_bn_apply(const void* x, const void* res, void* y, const float* sums, const float* fixed_mean_var,
                 const float* w, const float* b, float* save_mean_rstd, float* acc_sum, float* acc_sumsq,
                 float* acc_count, int64_t acc_seg_stride, int64_t m, int c, float eps, int relu, int dtype, int segs,
                 cudaStream_t stream) {
  if (m <= 0) return 0;
  if (c % 8 != 0 || c > 4096 || segs < 1 || m % segs != 0) return -3;
  m /= segs;
  const size_t smem = sizeof(float) * 2 * (size_t)c;
  int gx = elem_blocks(m * (c / 8));
  if (segs > 1 && gx > (148 * 16) / segs) gx = (148 * 16) / segs;
  const dim3 grid(gx, segs);
  if (dtype == TSP_DTYPE_BF16)
    bn_apply_kernel<__nv_bfloat16><<<grid, kBlock, smem, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res,
                                                                   (__nv_bfloat16*)y, sums, fixed_mean_var, w, b,
                                                                   save_mean_rstd, acc_sum, acc_sumsq, acc_count,
                                                                   acc_seg_stride, m, c, eps, relu);
  else
    bn_apply_kernel<float><<<grid, kBlock, smem, stream>>>((const float*)x, (const float*)res, (float*)y, sums,
                                                           fixed_mean_var, w, b, save_mean_rstd, acc_sum, acc_sumsq,
                                                           acc_count, acc_seg_stride, m, c, eps, relu);
  return TSP_LAUNCH_CHECK();
}

// sums [segs][2*c] is zeroed, then receives per group sum(dy') and sum(dy' * xhat) (db and dw are their sums over
// the groups).  `y` non-null applies the ReLU mask; `dres` non-null receives dy'.
int tsp_bn_bwd_reduce(const void* dy, const void* x, const void* y, void* dres, const float* mean_rstd, const float* w,
                      const float* bias, int relu, int64_t m, int c, int dtype, float* sums, int segs,
                      cudaStream_t stream) {
  if (m <= 0) return 0;
  if (c % 8 != 0 || c > 8192 || segs < 1 || m % segs != 0) return -3;
  cudaError_t e = cudaMemsetAsync(sums, 0, sizeof(float) * 2 * (size_t)c * segs, stream);
  if (e != cudaSuccess) return (int)e;
  m /= segs;
  if (stream_ok(m, c, dtype))
    return launch_stream<1>(x, dy, y, dres, mean_rstd, w, bias, relu, m, c, segs, sums, stream);
  const int cpv = c / 8;
  const Tile tl = make_tile(cpv);
  const int slabs = (cpv + tl.tx_n - 1) / tl.tx_n;
  dim3 grid(row_blocks(m, tl.ty_n, slabs), slabs, segs);
  const size_t smem = sizeof(float) * 16 * (size_t)tl.tx_n * tl.ty_n;
  if (dtype == TSP_DTYPE_BF16)
    bn_colsum_kernel<__nv_bfloat16, 1><<<grid, kBlock, smem, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                                       (const __nv_bfloat16*)y, (__nv_bfloat16*)dres,
                                                                       mean_rstd, w, bias, relu, m, c, sums);
  else
    bn_colsum_kernel<float, 1><<<grid, kBlock, smem, stream>>>((const float*)x, (const float*)dy, (const float*)y,
                                                               (float*)dres, mean_rstd, w, bias, relu, m, c, sums);
  return TSP_LAUNCH_CHECK();
}

int tsp_bn_bwd_apply(const void* dy, const void* x, const void* y, const float* mean_rstd, const float* w,
                     const float* bias, int relu, const float* sums, void* dx, int64_t m, int c, int dtype, int segs,
                     cudaStream_t stream) {
  if (m <= 0) return 0;
  if (c % 8 != 0 || c > 4096 || segs < 1 || m % segs != 0) return -3;
  m /= segs;
  const size_t smem = sizeof(float) * 5 * (size_t)c;
  if (smem > 48 * 1024) {      // opt in to more than the default dynamic shared memory
    cudaFuncSetAttribute(bn_bwd_apply_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    cudaFuncSetAttribute(bn_bwd_apply_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
  }
  int gx = elem_blocks(m * (c / 8));
  if (segs > 1 && gx > (148 * 16) / segs) gx = (148 * 16) / segs;
  const dim3 grid(gx, segs);
  if (dtype == TSP_DTYPE_BF16)
    bn_bwd_apply_kernel<__nv_bfloat16><<<grid, kBlock, smem, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                                       (const __nv_bfloat16*)y, mean_rstd, w, bias, relu,
                                                                       sums, (__nv_bfloat16*)dx, m, c);
  else
    bn_bwd_apply_kernel<float><<<grid, kBlock, smem, stream>>>((const float*)dy, (const float*)x, (const float*)y,
                                                               mean_rstd, w, bias, relu, sums, (float*)dx, m, c);
  return TSP_LAUNCH_CHECK();
}

}  // extern "C"
