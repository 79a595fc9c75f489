// ResNet stem convolution on the 5th-generation tensor cores: y = conv2d(x, w), 7 x 7, stride 2, padding 3,
// 3 -> 64 channels, channels-last bf16, with the per-channel sum / sum of squares of y (the statistics of the
// BatchNorm that follows) accumulated in the epilogue.
//
// Reference call site: the first layer of torchvision's ResNet used by `benchmarks/byol/models/resnet_base_network.py`
// and `benchmarks/soft_target/models/resnet.py` (library convolution there).  The library's kernel for this
// shape pads 3 input channels to 8 and runs at a few percent of the machine; as an implicit GEMM the layer is
// M = N*OH*OW output pixels, N = 64, K = 7*7*3 = 147 (160 after padding to the MMA's k = 16) and is bound by
// writing y.
//
// One persistent CTA per SM walks a contiguous range of output rows (n, oh); one output row (OW <= 128 pixels)
// is one 128 x 64 accumulator tile.
//   warps 0-3  im2col: the input rows 2*oh-3 .. 2*oh+3 live in a 16-slot ring in shared memory (cp.async, two
//              new rows per output row, prefetched one tile ahead); each thread owns one output pixel and writes
//              its 160 patch values (k = kh*21 + kw*3 + c) as 16-byte pieces into the 128-byte-swizzled K-major
//              operand layout that tcgen05.mma reads;
//   warp  4    one thread issues 10 x tcgen05.mma (128 x 64 x 16) per tile, accumulators in tensor memory
//              (two buffers), weights [64][192] resident in shared memory (loaded once by TMA);
//   warps 5-8  epilogue: tcgen05.ld -> bf16 -> swizzled staging -> TMA store (3-d map, rows >= OW clipped),
//              and column sums of the staged tile for the BatchNorm statistics.
// Every mbarrier wait is bounded; a wait that runs out sets *status and all roles leave their loops.
#include <cuda.h>

#include "common.cuh"
#include "tspipe_kernels.h"

extern int g_tsp_sm_reserve;          // defined in peer.cu

namespace {

constexpr int kCout = 64;
constexpr int kK = 160;                   // 147 rounded up to a multiple of 16
constexpr int kKPad = 192;                // weight matrix row length: three 64-wide k blocks
constexpr int kAStages = 3;
constexpr int kABlockBytes = 128 * 128;   // one k block of A: 128 rows x 128 bytes
constexpr int kAStageBytes = 3 * kABlockBytes;
constexpr int kBBlockBytes = kCout * 128;
constexpr int kBBytes = 3 * kBBlockBytes;
constexpr int kRingSlots = 16;
constexpr int kAhead = 3;                 // output rows between the fetch of an input row pair and its use (7 + 2 * kAhead <= 16)
constexpr int kRowElems = 704;            // 16 leading pad + up to 672 data + trailing zeros
constexpr int kRowBytes = kRowElems * 2;
constexpr int kRingBytes = kRingSlots * kRowBytes;
constexpr int kStoreBufBytes = 32 * 128;
constexpr int kStoreBytes = 4 * 2 * kStoreBufBytes;
constexpr int kSmemBytes = kAStages * kAStageBytes + kBBytes + kStoreBytes + kRingBytes + 1024 + 256;
constexpr int kThreads = 9 * 32;
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    // The error word lives in global memory, so this check costs a round trip to L2 per failed poll.  That is
    // deliberate: it is the back-off of the spin loop.  Polling the barrier flat out, or backing off with a short
    // nanosleep instead, were both measured slower (fused contrastive loss: 481 us with this loop, 607 us polling
    // flat out, 740 us with __nanosleep(32)).
    if (*((volatile int*)status) != 0) return false;
  }
  atomicCAS(status, 0, code);
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32_issue(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ void producer_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Barrier over the 128 im2col threads that also ANDs a flag, so that all of them take the same way out.
__device__ __forceinline__ bool producer_barrier_and(bool ok) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, 128, q;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"((uint32_t)ok)
      : "memory");
  return out != 0;
}

// Rows [ih_lo, ih_hi] of image n into their ring slots: cp.async for rows inside the image, zeros outside.
__device__ __forceinline__ void ring_load(uint8_t* ring, const __nv_bfloat16* x, int n, int ih_lo, int ih_hi, int h, int w,
                                          int tid) {
  const int vec_per_row = (w * 3 * 2) / 16;
  const int total = (ih_hi - ih_lo + 1) * vec_per_row;
  for (int v = tid; v < total; v += 128) {
    const int r = v / vec_per_row, col = v - r * vec_per_row;
    const int ih = ih_lo + r;
    uint8_t* dst = ring + ((ih + 16) & (kRingSlots - 1)) * kRowBytes + 32 + col * 16;
    if (ih >= 0 && ih < h) {
      const uint8_t* src = (const uint8_t*)x + ((int64_t)(n * h + ih) * w * 3) * 2 + col * 16;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
conv_stem_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_y,
                 const __nv_bfloat16* __restrict__ x, int n_img, int h, int w, int oh_n, int ow_n, int imgs_per_seg,
                 float* __restrict__ sums, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* a_tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* b_tile = a_tiles + kAStages * kAStageBytes;
  uint8_t* store_bufs = b_tile + kBBytes;
  uint8_t* ring = store_bufs + kStoreBytes;
  uint64_t* bars = (uint64_t*)(ring + kRingBytes);
  uint64_t* full_bar = bars;                     // [kAStages]  im2col -> MMA (4 arrivals: one per producer warp)
  uint64_t* empty_bar = bars + kAStages;         // [kAStages]  MMA -> im2col
  uint64_t* tmem_full_bar = bars + 2 * kAStages;        // [2]
  uint64_t* tmem_empty_bar = bars + 2 * kAStages + 2;   // [2]  4 arrivals
  uint64_t* w_bar = bars + 2 * kAStages + 4;
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kAStages + 5);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int num_tiles = n_img * oh_n;
  const int per_cta = (num_tiles + gridDim.x - 1) / gridDim.x;
  const int t_begin = blockIdx.x * per_cta;
  const int t_end = t_begin + per_cta < num_tiles ? t_begin + per_cta : num_tiles;

  if (tid == 0) {
    for (int s = 0; s < kAStages; ++s) { mbar_init(full_bar + s, 4); mbar_init(empty_bar + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tmem_full_bar + a, 1); mbar_init(tmem_empty_bar + a, 4); }
    mbar_init(w_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_y) : "memory");
  }
  // the ring's padding (and everything else) starts as zeros; data columns are rewritten per row
  for (int i = tid; i < kRingBytes / 16; i += kThreads) reinterpret_cast<uint4*>(ring)[i] = make_uint4(0u, 0u, 0u, 0u);
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(128u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
    // ---------------- im2col producers: thread = output pixel ----------------
    const int p = tid;
    bool ok = true;
    int have_n = -1, have_oh = -2;                 // image / output row whose 7 input rows are resident
    uint32_t it = 0;
    for (int t = t_begin; t < t_end && ok; ++t, ++it) {
      const int n = t / oh_n, oh = t - n * oh_n;
      const int ih0 = 2 * oh - 3;
      // Input rows are fetched kAhead output rows ahead of their use (global latency is a few tile times): at
      // tile t the copies of tile t + kAhead are issued and all but the kAhead - 1 most recent groups are awaited.
      if (n != have_n || oh != have_oh + 1) {      // start of a run of consecutive output rows of one image
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        producer_barrier();                        // nobody still reads rows of the previous run
        ring_load(ring, x, n, ih0, ih0 + 6, h, w, tid);
#pragma unroll
        for (int d = 1; d < kAhead; ++d) {
          if (t + d < t_end && oh + d < oh_n) ring_load(ring, x, n, ih0 + 5 + 2 * d, ih0 + 6 + 2 * d, h, w, tid);
          else asm volatile("cp.async.commit_group;" ::: "memory");
        }
      }
      const int s = it % kAStages;
      const uint32_t round = it / kAStages;
      bool mine = true;
      if (round > 0) mine = mbar_wait(empty_bar + s, (round - 1) & 1, status, 1);
      asm volatile("cp.async.wait_group %0;" ::"n"(kAhead - 1) : "memory");
      ok = producer_barrier_and(mine);             // this tile's rows are in the ring, for every thread
      if (!ok) break;
      have_n = n; have_oh = oh;
      if (t + kAhead < t_end && oh + kAhead < oh_n)
        ring_load(ring, x, n, ih0 + 5 + 2 * kAhead, ih0 + 6 + 2 * kAhead, h, w, tid);
      else
        asm volatile("cp.async.commit_group;" ::: "memory");
      if (p < ow_n) {
        uint8_t* a_stage = a_tiles + s * kAStageBytes;
        const uint32_t row_off = (uint32_t)(p >> 3) * 1024u + (uint32_t)(p & 7) * 128u;
        // Patch row kh of this pixel = 21 bf16 starting at byte 12 p + 14 of the ring row: always 2 bytes past a
        // 4-byte boundary.  Read the 11 aligned words that cover it (lanes 12 bytes apart: conflict-free) and
        // recombine halves: the k stream (kh * 21 + i) is cut into 32-bit output words with compile-time shuffles.
        const uint8_t* rows[7];
#pragma unroll
        for (int kh = 0; kh < 7; ++kh)
          rows[kh] = ring + ((ih0 + kh + 16) & (kRingSlots - 1)) * kRowBytes + 12 * p + 12;
        auto ldw = [&](int kh, int c) -> uint32_t { return *reinterpret_cast<const uint32_t*>(rows[kh] + 4 * c); };
#pragma unroll
        for (int q = 0; q < kK / 8; ++q) {          // 16-byte piece q: k = 8q .. 8q+7
          uint32_t wd[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int s0 = 8 * q + 2 * e, s1 = s0 + 1;        // stream positions of the two halves
            uint32_t out = 0;
            if (s0 < 147) {
              const int kh0 = s0 / 21, h0 = s0 % 21 + 1;       // halfword index inside the 22-halfword window
              if (s1 >= 147) {
                out = ldw(kh0, h0 >> 1) >> 16;                // last element of the patch, zero above
              } else if (s1 / 21 == kh0) {
                out = (h0 & 1) ? __funnelshift_r(ldw(kh0, h0 >> 1), ldw(kh0, (h0 >> 1) + 1), 16) : ldw(kh0, h0 >> 1);
              } else {                                         // last element of row kh0, first of row kh0 + 1
                out = __byte_perm(ldw(kh0, 10), ldw(kh0 + 1, 0), 0x7632);
              }
            }
            wd[e] = out;
          }
          const int kb = q >> 3, piece = q & 7;
          *reinterpret_cast<uint4*>(a_stage + kb * kABlockBytes + row_off + ((piece ^ (p & 7)) << 4)) =
              make_uint4(wd[0], wd[1], wd[2], wd[3]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(full_bar + s);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (warp == 4) {
    // ---------------- weights + MMA issuer ----------------
    if (lane == 0) {
      mbar_expect_tx(w_bar, (uint32_t)kBBytes);
      for (int kb = 0; kb < 3; ++kb) tma_load_2d(b_tile + kb * kBBlockBytes, &tmap_w, w_bar, kb * 64, 0);
      bool ok = mbar_wait(w_bar, 0, status, 5);
      constexpr uint32_t idesc = make_idesc(128, kCout);
      uint32_t it = 0;
      for (int t = t_begin; t < t_end && ok; ++t, ++it) {
        const uint32_t acc = it & 1, use = it >> 1;
        if (use > 0) {
          ok = mbar_wait(tmem_empty_bar + acc, (use - 1) & 1, status, 4);
          if (!ok) break;
        }
        const int s = it % kAStages;
        ok = mbar_wait(full_bar + s, (it / kAStages) & 1, status, 2);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(a_tiles + s * kAStageBytes), b_addr = smem_u32(b_tile);
#pragma unroll
        for (int kk = 0; kk < kK / 16; ++kk) {
          const int kb = kk >> 2, in = kk & 3;
          umma_bf16(tmem_base + acc * kCout, make_smem_desc(a_addr + kb * kABlockBytes) + (uint64_t)(2 * in),
                    make_smem_desc(b_addr + kb * kBBlockBytes) + (uint64_t)(2 * in), idesc, kk > 0 ? 1u : 0u);
        }
        umma_commit(empty_bar + s);
        umma_commit(tmem_full_bar + acc);
      }
    }
  } else {
    // ---------------- epilogue: warps 5..8, TMEM lanes 32*(warp%4) .. +31 ----------------
    const int quarter = warp & 3;
    uint8_t* my_bufs = store_bufs + quarter * 2 * kStoreBufBytes;
    float s0 = 0.f, s1 = 0.f, q0 = 0.f, q1 = 0.f;          // channels 2*lane, 2*lane+1
    int cur_seg = t_begin < t_end ? (t_begin / oh_n) / imgs_per_seg : 0;
    auto flush_sums = [&](int seg) {
      if (sums != nullptr) {
        float* dst = sums + seg * 2 * kCout;
        atomicAdd(dst + 2 * lane, s0);
        atomicAdd(dst + 2 * lane + 1, s1);
        atomicAdd(dst + kCout + 2 * lane, q0);
        atomicAdd(dst + kCout + 2 * lane + 1, q1);
      }
      s0 = s1 = q0 = q1 = 0.f;
    };
    uint32_t it = 0;
    bool ok = true;
    for (int t = t_begin; t < t_end && ok; ++t, ++it) {
      const int seg = (t / oh_n) / imgs_per_seg;           // statistics are kept per group of images
      if (seg != cur_seg) { flush_sums(cur_seg); cur_seg = seg; }
      const uint32_t acc = it & 1, use = it >> 1;
      ok = __all_sync(0xffffffffu, mbar_wait(tmem_full_bar + acc, use & 1, status, 3));   // one way out per warp
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t r[64];
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kCout;
      tmem_ld_32x32_issue(taddr, r);
      tmem_ld_32x32_issue(taddr + 32, r + 32);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar + acc);      // the accumulator is in registers now
      uint8_t* buf = my_bufs + (it & 1) * kStoreBufBytes;
      if (it >= 2) {
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        __syncwarp();
      }
      uint8_t* my_row = buf + lane * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
        v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
        v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
        v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
        *reinterpret_cast<uint4*>(my_row + ((j ^ (lane & 7)) << 4)) = v;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      const int row0 = quarter * 32;
      if (lane == 0) {
        if (row0 < ow_n) tma_store_3d(&tmap_y, buf, 0, row0, t);
        else asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
      // statistics of the rounded outputs: lane owns channels 2*lane, 2*lane+1 of the warp's valid rows
      const int valid = ow_n - row0 < 32 ? ow_n - row0 : 32;
#pragma unroll 8
      for (int rr = 0; rr < 32; ++rr) {              // fixed trip count: the loads of a group are issued together
        const uint32_t wv = *reinterpret_cast<const uint32_t*>(buf + rr * 128 + (((lane >> 2) ^ (rr & 7)) << 4) + (lane & 3) * 4);
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv));
        if (rr < valid) { s0 += f.x; q0 += f.x * f.x; s1 += f.y; q1 += f.y * f.y; }
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __syncwarp();
    flush_sums(cur_seg);
  }
  if (*((volatile int*)status) != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);        // let copies and MMAs that are still in flight land
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128u) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

}  // namespace

extern "C" {

// y[n, oh, ow, 64] = conv7x7/2 pad 3 of x[n, h, w, 3] (both bf16, channels-last memory) with wmat[64][192] bf16:
// wmat[oc][kh*21 + kw*3 + c] = weight[oc][c][kh][kw], zero beyond k = 146.  h even, w % 8 == 0, 8 <= w <= 224.
// `sums` (optional, [segs][128] floats, zeroed by the caller) receives per-channel sum and sum of squares of y for
// each of the `segs` consecutive groups of n / segs images.
// `status`: one zeroed int in device memory; non-zero afterwards = a bounded wait ran out and y is not valid.
int tsp_conv_stem_fwd(const void* x, const void* wmat, void* y, float* sums, int n, int h, int w, int segs,
                      int* status, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (segs < 1 || n % segs != 0) return -3;
  if ((h & 1) || (w & 7) || w > 224 || h < 8 || w < 8) return -3;
  if ((((uintptr_t)x | (uintptr_t)wmat | (uintptr_t)y) & 15) != 0) return -2;
  const int oh = h / 2, ow = w / 2;
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -6;
  CUtensorMap tw, ty;
  {
    cuuint64_t dims[2] = {(cuuint64_t)kKPad, (cuuint64_t)kCout};
    cuuint64_t strides[1] = {(cuuint64_t)kKPad * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)kCout};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&tw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(wmat), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return -6;
  }
  {
    cuuint64_t dims[3] = {(cuuint64_t)kCout, (cuuint64_t)ow, (cuuint64_t)n * oh};
    cuuint64_t strides[2] = {(cuuint64_t)kCout * 2, (cuuint64_t)ow * kCout * 2};
    cuuint32_t box[3] = {(cuuint32_t)kCout, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (enc(&ty, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) !=
        CUDA_SUCCESS)
      return -6;
  }
  static bool attr_set[64] = {};
  static int n_sm[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(conv_stem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    cudaDeviceGetAttribute(&n_sm[dev], cudaDevAttrMultiProcessorCount, dev);
    if (n_sm[dev] <= 0) n_sm[dev] = 148;
    attr_set[dev] = true;
  }
  const int tiles = n * oh;
  const int usable = n_sm[dev] - g_tsp_sm_reserve > 8 ? n_sm[dev] - g_tsp_sm_reserve : 8;
  const int grid = tiles < usable ? tiles : usable;
  conv_stem_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tw, ty, (const __nv_bfloat16*)x, n, h, w, oh, ow, n / segs, sums, status);
  return TSP_LAUNCH_CHECK();
}

}  // extern "C"
