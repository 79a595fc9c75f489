// Kernels that read or write other GPUs' memory through peer-mapped pointers (NVLink 5 / NVSwitch), sm_100a.
//
// The reference has no data parallelism in its runtime; its baselines use DDP's bucketed NCCL all-reduce followed
// by a per-tensor optimizer (`benchmarks/moco-v3/main.py:249-254`, `benchmarks/byol/main.py:13-46`).  Here, with R
// pipeline replicas, the gradient reduce-scatter, the cast/scale, the sharded LARS / AdamW step and the all-gather of
// the updated parameters are two launches (LARS: the trust ratio needs whole-tensor norms in between) or one (AdamW):
//   * each rank owns the flat range [lo, hi) of its stage's parameter buffer;
//   * it sums that range of every replica's gradient buffer with plain peer loads (the reduce-scatter),
//   * updates parameter and optimizer state of the range,
//   * and stores the new parameters into every replica's parameter buffer with peer stores (the all-gather).
// Ordering between the ranks (peers' backward passes done -> gradient reads; reads done -> parameter stores; stores
// done -> next forward) goes through signal words in peer-mapped memory: a rank announces a phase by storing an
// increasing counter into slot [its index] of every peer's pad (tsp_signal_arrive), and waits for a phase by spinning,
// with a time limit, until every slot of its own pad has reached the counter (tsp_signal_wait).  A wait that runs out
// records a code in a status word and the kernel returns: nothing traps, nothing hangs.  Every rank runs on its own
// GPU, so a waiting kernel never shares a GPU with the kernel it waits for.
#include "common.cuh"
#include "tspipe_kernels.h"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxPeers = 8;

struct PeerPtrs {
  float* p[kMaxPeers];
};

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

// g_out[k] = scale * sum_r grads[r][k] over the chunk; LARS norms accumulated for adaptive segments.
__global__ void __launch_bounds__(kThreads) dp_reduce_norms_kernel(PeerPtrs grads, int n_peers, float scale,
                                                                   float* __restrict__ g_out,
                                                                   const float* __restrict__ p,
                                                                   const int64_t* __restrict__ chunks,
                                                                   const float* __restrict__ seg_hp,
                                                                   float* __restrict__ norms) {
  __shared__ float scratch[33];
  const ChunkView c = load_chunk(chunks, blockIdx.x);
  const float* hp = seg_hp + 5 * (int64_t)c.seg;
  const bool adapt = norms != nullptr && hp[4] != 0.f;
  const float wd = hp[1];
  float sp = 0.f, su = 0.f;
  // 16-byte peer loads where the chunk starts on a 4-element boundary (flat segments and replica shards do): a
  // quarter of the round trips over NVLink; the last len % 4 elements (and unaligned chunks) go one by one.
  const int n4 = (c.begin & 3) == 0 ? c.len >> 2 : 0;
  for (int i = threadIdx.x; i < n4; i += kThreads) {
    const int64_t k = c.begin + 4 * (int64_t)i;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < n_peers) {
        const float4 t = *reinterpret_cast<const float4*>(grads.p[r] + k);
        s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
      }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    *reinterpret_cast<float4*>(g_out + k) = s;
    if (adapt) {
      const float4 a = *reinterpret_cast<const float4*>(p + k);
      const float ux = s.x + wd * a.x, uy = s.y + wd * a.y, uz = s.z + wd * a.z, uw = s.w + wd * a.w;
      sp += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
      su += ux * ux + uy * uy + uz * uz + uw * uw;
    }
  }
  for (int i = 4 * n4 + threadIdx.x; i < c.len; i += kThreads) {
    const int64_t k = c.begin + i;
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < n_peers) s += grads.p[r][k];
    s *= scale;
    g_out[k] = s;
    if (adapt) {
      const float a = p[k], u = s + wd * a;
      sp += a * a;
      su += u * u;
    }
  }
  if (adapt) {
    sp = tsp::block_sum(sp, scratch);
    su = tsp::block_sum(su, scratch);
    if (threadIdx.x == 0) {
      atomicAdd(norms + 2 * c.seg, sp);
      atomicAdd(norms + 2 * c.seg + 1, su);
    }
  }
}

// LARS apply on the owned range (gradient already reduced into g), new parameters stored to every replica.
__global__ void __launch_bounds__(kThreads) dp_lars_apply_kernel(PeerPtrs params, int n_peers, int self,
                                                                 const float* __restrict__ g, float* __restrict__ mu,
                                                                 const int64_t* __restrict__ chunks,
                                                                 const float* __restrict__ seg_hp,
                                                                 const float* __restrict__ norms) {
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
  const float* p_self = params.p[self];
  const int n4 = (c.begin & 3) == 0 ? c.len >> 2 : 0;
  for (int i = threadIdx.x; i < n4; i += kThreads) {
    const int64_t k = c.begin + 4 * (int64_t)i;
    const float4 pv = *reinterpret_cast<const float4*>(p_self + k);
    const float4 gv = *reinterpret_cast<const float4*>(g + k);
    float4 mv = *reinterpret_cast<const float4*>(mu + k);
    mv.x = mom * mv.x + q * (gv.x + wd_eff * pv.x);
    mv.y = mom * mv.y + q * (gv.y + wd_eff * pv.y);
    mv.z = mom * mv.z + q * (gv.z + wd_eff * pv.z);
    mv.w = mom * mv.w + q * (gv.w + wd_eff * pv.w);
    *reinterpret_cast<float4*>(mu + k) = mv;
    const float4 np = make_float4(pv.x - lr * mv.x, pv.y - lr * mv.y, pv.z - lr * mv.z, pv.w - lr * mv.w);
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < n_peers) *reinterpret_cast<float4*>(params.p[r] + k) = np;
  }
  for (int i = 4 * n4 + threadIdx.x; i < c.len; i += kThreads) {
    const int64_t k = c.begin + i;
    const float pv = p_self[k];
    const float dp = q * (g[k] + wd_eff * pv);
    const float m2 = mom * mu[k] + dp;
    mu[k] = m2;
    const float np = pv - lr * m2;
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < n_peers) params.p[r][k] = np;
  }
}

// AdamW: reduce + update + store to all replicas in one pass.
__global__ void __launch_bounds__(kThreads) dp_adamw_kernel(PeerPtrs grads, PeerPtrs params, int n_peers, int self,
                                                            float scale, float* __restrict__ m, float* __restrict__ v,
                                                            const int64_t* __restrict__ chunks,
                                                            const float* __restrict__ seg_hp) {
  const ChunkView c = load_chunk(chunks, blockIdx.x);
  const float* hp = seg_hp + 7 * (int64_t)c.seg;
  const float lr = hp[0], b1 = hp[1], b2 = hp[2], eps = hp[3], wd = hp[4], bc1 = hp[5], bc2 = hp[6];
  const float step = lr / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  const float* p_self = params.p[self];
  auto update = [&](float gv, float pv, float& mv, float& vv) -> float {
    pv *= (1.f - lr * wd);
    mv = b1 * mv + (1.f - b1) * gv;
    vv = b2 * vv + (1.f - b2) * gv * gv;
    return pv - step * mv / (sqrtf(vv) * inv_sqrt_bc2 + eps);
  };
  const int n4 = (c.begin & 3) == 0 ? c.len >> 2 : 0;
  for (int i = threadIdx.x; i < n4; i += kThreads) {
    const int64_t k = c.begin + 4 * (int64_t)i;
    float4 gv = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < n_peers) {
        const float4 t = *reinterpret_cast<const float4*>(grads.p[r] + k);
        gv.x += t.x; gv.y += t.y; gv.z += t.z; gv.w += t.w;
      }
    const float4 pv = *reinterpret_cast<const float4*>(p_self + k);
    float4 mv = *reinterpret_cast<const float4*>(m + k), vv = *reinterpret_cast<const float4*>(v + k);
    float4 np;
    np.x = update(gv.x * scale, pv.x, mv.x, vv.x);
    np.y = update(gv.y * scale, pv.y, mv.y, vv.y);
    np.z = update(gv.z * scale, pv.z, mv.z, vv.z);
    np.w = update(gv.w * scale, pv.w, mv.w, vv.w);
    *reinterpret_cast<float4*>(m + k) = mv;
    *reinterpret_cast<float4*>(v + k) = vv;
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < n_peers) *reinterpret_cast<float4*>(params.p[r] + k) = np;
  }
  for (int i = 4 * n4 + threadIdx.x; i < c.len; i += kThreads) {
    const int64_t k = c.begin + i;
    float gv = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < n_peers) gv += grads.p[r][k];
    float mv = m[k], vv = v[k];
    const float pv = update(gv * scale, p_self[k], mv, vv);
    m[k] = mv;
    v[k] = vv;
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < n_peers) params.p[r][k] = pv;
  }
}

// ---- signal words ------------------------------------------------------------------------------------------------
struct PadPtrs {
  int* p[kMaxPeers];
};

// everything this stream did before is visible to the peers before they can see the counter
__global__ void signal_arrive_kernel(PadPtrs pads, int n_peers, int self, int value) {
  const int r = threadIdx.x;
  if (r < n_peers) {
    __threadfence_system();
    asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(pads.p[r] + self), "r"(value) : "memory");
  }
}

__device__ __forceinline__ unsigned long long timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// thread r waits until slot r of this rank's pad has reached `value`; gives up after limit_ns
__global__ void signal_wait_kernel(const int* __restrict__ pad, int n_peers, int value, unsigned long long limit_ns,
                                   int* __restrict__ status, int code) {
  const int r = threadIdx.x;
  if (r >= n_peers) return;
  const unsigned long long t0 = timer_ns();
  for (;;) {
    int seen;
    asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(seen) : "l"(pad + r) : "memory");
    if (seen - value >= 0) break;                    // counters only grow (wrap-safe comparison)
    if (timer_ns() - t0 > limit_ns) {
      atomicCAS(status, 0, code);
      break;
    }
    __nanosleep(200);
  }
  __threadfence_system();
}

// each rank's partial LARS norms go to slot [self] of every peer's table: dst_r[self * n + i] = norms[i]
__global__ void __launch_bounds__(kThreads) publish_norms_kernel(PeerPtrs tables, int n_peers, int self,
                                                                 const float* __restrict__ norms, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n * n_peers; i += gridDim.x * blockDim.x) {
    const int r = i / n, k = i - r * n;
    tables.p[r][(int64_t)self * n + k] = norms[k];
  }
}

// norms[i] = sum over ranks of table[r * n + i]
__global__ void __launch_bounds__(kThreads) sum_norms_kernel(const float* __restrict__ table, int n_peers, int n,
                                                             float* __restrict__ norms) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int r = 0; r < n_peers; ++r) s += table[(int64_t)r * n + i];
    norms[i] = s;
  }
}

// dst[r * n + i] = src_r[i]: concatenate one equally sized block per peer (16-byte units) into local memory.
__global__ void __launch_bounds__(kThreads) gather_blocks_kernel(PeerPtrs srcs, int n_peers, int64_t n16,
                                                                 uint4* __restrict__ dst) {
  const int64_t total = n16 * n_peers;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / n16);
    const int64_t j = i - (int64_t)r * n16;
    dst[i] = reinterpret_cast<const uint4*>(srcs.p[r])[j];
  }
}

inline bool fill(PeerPtrs& dst, void* const* src, int n) {
  if (n < 1 || n > kMaxPeers) return false;
  for (int i = 0; i < kMaxPeers; ++i) dst.p[i] = i < n ? (float*)src[i] : nullptr;
  return true;
}

}  // namespace

// SMs that the persistent tensor-core kernels leave free (see tsp_set_sm_reserve)
int g_tsp_sm_reserve = 0;

extern "C" {

// The persistent tcgen05 kernels (convolutions, GEMMs) launch one CTA per SM with almost all of its shared memory; a
// communication kernel that becomes ready while one of them runs (an NCCL send / receive of a stage link, a peer
// reduction on a side stream) finds no SM until a CTA retires, i.e. until the whole persistent kernel ends.  With a
// reserve of n, those kernels launch on (SM count - n) SMs and the rest stay available.  Set by the runtime when a
// job has stage links; 0 for single-stage jobs.
void tsp_set_sm_reserve(int n) { g_tsp_sm_reserve = n < 0 ? 0 : (n > 64 ? 64 : n); }
int tsp_get_sm_reserve(void) { return g_tsp_sm_reserve; }

// Make `peer_device`'s memory addressable from kernels of the current device.  0 = ok / already enabled,
// -5 = the two devices have no peer path.
int tsp_enable_peer_access(int peer_device) {
  int cur = -1;
  cudaError_t e = cudaGetDevice(&cur);
  if (e != cudaSuccess) return (int)e;
  if (cur == peer_device) return 0;
  int can = 0;
  e = cudaDeviceCanAccessPeer(&can, cur, peer_device);
  if (e != cudaSuccess) return (int)e;
  if (!can) return -5;
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return (int)e;
}

// Map a buffer exported by another process (64-byte CUDA IPC handle of its allocation) into the CURRENT device's
// address space; peer access to the owning device is enabled by the runtime as part of the mapping.  The handle
// must come from a different process.  `*base` receives the mapped allocation base (add the exporter's offset).
int tsp_ipc_import(const unsigned char* handle64, void** base) {
  cudaIpcMemHandle_t h;
  for (int i = 0; i < 64; ++i) reinterpret_cast<unsigned char*>(&h)[i] = handle64[i];
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return (int)e;
  }
  *base = p;
  return 0;
}

int tsp_ipc_close(void* base) { return (int)cudaIpcCloseMemHandle(base); }

// Capability query only: 1 when `device` can take part in NVLink multicast objects (the in-switch reduction path that
// `multimem` instructions address), 0 when it cannot, negative when the driver cannot be asked.  Nothing is created or
// bound here: a rank that dies while its memory is bound to a multicast object disturbs the other GPUs, so the
// kernels of this library move data with plain peer loads / stores and copy engines and only report the capability.
int tsp_multicast_supported(int device) {
  typedef int (*GetAttrFn)(int*, int, int);
  static GetAttrFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuDeviceGetAttribute", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess && p != nullptr) {
      fn = (GetAttrFn)p;
    } else {
      (void)cudaGetLastError();
      return -1;
    }
  }
  int value = 0;
  const int kMulticastSupported = 132;          // CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED
  if (fn(&value, kMulticastSupported, device) != 0) return -2;
  return value ? 1 : 0;
}

// Stream-ordered copy between any two device addresses this process can reach (own memory or a mapped peer
// buffer).  The driver moves the bytes with a copy engine over NVLink: no SM is involved, so a transfer never
// competes with the persistent compute kernels for a place on the GPU.
int tsp_copy_async(void* dst, const void* src, int64_t bytes, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  return (int)cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, stream);
}

// All-gather by peer loads: block r of `dst` receives `bytes_each` bytes read from srcs[r] (own or peer memory).
int tsp_gather_blocks(void* const* srcs, int n_peers, int64_t bytes_each, void* dst, cudaStream_t stream) {
  if (bytes_each <= 0) return 0;
  if (bytes_each % 16) return -3;
  PeerPtrs sp;
  if (!fill(sp, srcs, n_peers)) return -3;
  const int64_t n16 = bytes_each / 16;
  int64_t blocks = (n16 * n_peers + kThreads - 1) / kThreads;
  if (blocks > 148 * 8) blocks = 148 * 8;
  gather_blocks_kernel<<<(int)blocks, kThreads, 0, stream>>>(sp, n_peers, n16, (uint4*)dst);
  return TSP_LAUNCH_CHECK();
}

// Store `value` into slot [self] of every rank's signal pad (pads[r] = rank r's pad of >= n_peers ints, own pad
// included).  Stream-ordered: everything enqueued before on `stream` is visible to a peer that sees the value.
int tsp_signal_arrive(void* const* pads, int n_peers, int self, int value, cudaStream_t stream) {
  if (n_peers < 1 || n_peers > kMaxPeers || self < 0 || self >= n_peers) return -3;
  PadPtrs pp;
  for (int i = 0; i < kMaxPeers; ++i) pp.p[i] = i < n_peers ? (int*)pads[i] : nullptr;
  signal_arrive_kernel<<<1, 32, 0, stream>>>(pp, n_peers, self, value);
  return TSP_LAUNCH_CHECK();
}

// Wait on `stream` until every one of the n_peers slots of this rank's pad has reached `value`, at most limit_ms
// milliseconds.  When the limit runs out, *status (one zeroed int in device memory) becomes `code` and the kernel
// returns normally; the caller reads the status word.
int tsp_signal_wait(const void* pad, int n_peers, int value, int limit_ms, int* status, int code, cudaStream_t stream) {
  if (n_peers < 1 || n_peers > kMaxPeers || limit_ms < 1) return -3;
  signal_wait_kernel<<<1, 32, 0, stream>>>((const int*)pad, n_peers, value, (unsigned long long)limit_ms * 1000000ull,
                                           status, code);
  return TSP_LAUNCH_CHECK();
}

// All-gather of the per-rank partial LARS norms through peer stores: tables[r] = rank r's [n_peers][n] table.
int tsp_publish_norms(void* const* tables, int n_peers, int self, const float* norms, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  PeerPtrs tp;
  if (!fill(tp, tables, n_peers) || self < 0 || self >= n_peers) return -3;
  publish_norms_kernel<<<(n * n_peers + kThreads - 1) / kThreads, kThreads, 0, stream>>>(tp, n_peers, self, norms, n);
  return TSP_LAUNCH_CHECK();
}

int tsp_sum_norms(const float* table, int n_peers, int n, float* norms, cudaStream_t stream) {
  if (n <= 0) return 0;
  sum_norms_kernel<<<(n + kThreads - 1) / kThreads, kThreads, 0, stream>>>(table, n_peers, n, norms);
  return TSP_LAUNCH_CHECK();
}

int tsp_dp_reduce_norms(void* const* grads, int n_peers, float scale, float* g_out, const float* p,
                        const int64_t* chunks, int n_chunks, const float* seg_hp, float* norms, int n_seg,
                        cudaStream_t stream) {
  if (n_chunks <= 0) return 0;
  PeerPtrs gp;
  if (!fill(gp, grads, n_peers)) return -3;
  if (norms != nullptr) {
    cudaError_t e = cudaMemsetAsync(norms, 0, sizeof(float) * 2 * (size_t)n_seg, stream);
    if (e != cudaSuccess) return (int)e;
  }
  dp_reduce_norms_kernel<<<n_chunks, kThreads, 0, stream>>>(gp, n_peers, scale, g_out, p, chunks, seg_hp, norms);
  return TSP_LAUNCH_CHECK();
}

int tsp_dp_lars_apply(void* const* params, int n_peers, int self, const float* g, float* mu, const int64_t* chunks,
                      int n_chunks, const float* seg_hp, const float* norms, cudaStream_t stream) {
  if (n_chunks <= 0) return 0;
  PeerPtrs pp;
  if (!fill(pp, params, n_peers) || self < 0 || self >= n_peers) return -3;
  dp_lars_apply_kernel<<<n_chunks, kThreads, 0, stream>>>(pp, n_peers, self, g, mu, chunks, seg_hp, norms);
  return TSP_LAUNCH_CHECK();
}

int tsp_dp_adamw_step(void* const* grads, void* const* params, int n_peers, int self, float scale, float* m, float* v,
                      const int64_t* chunks, int n_chunks, const float* seg_hp, cudaStream_t stream) {
  if (n_chunks <= 0) return 0;
  PeerPtrs gp, pp;
  if (!fill(gp, grads, n_peers) || !fill(pp, params, n_peers) || self < 0 || self >= n_peers) return -3;
  dp_adamw_kernel<<<n_chunks, kThreads, 0, stream>>>(gp, pp, n_peers, self, scale, m, v, chunks, seg_hp);
  return TSP_LAUNCH_CHECK();
}

}  // extern "C"
