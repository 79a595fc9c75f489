// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * B[N,K]^T (+ bias) (-> GELU), fp32 accumulation.
//
//   * operands staged by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, each CTA loads its own tiles) into a 4-stage
//     shared-memory ring, one elected producer thread;
//   * tcgen05.mma.cta_group::1.kind::f16 (UMMA 128 x BN x 16) issued by one elected thread, accumulators in
//     tensor memory (TMEM), smem slots released with tcgen05.commit -> mbarrier;
//   * four epilogue warps read the accumulator with tcgen05.ld, fuse bias / GELU, convert, stage 32-row x 128-byte
//     blocks in swizzled shared memory and write them with TMA stores (direct stores when C is not 16-byte aligned).
// Reference call sites: every nn.Linear of the ViT / BERT blocks and heads (library GEMMs there:
// `benchmarks/moco-v3/vits.py`, `benchmarks/distilbert/bert.py`, `benchmarks/byol/models/mlp_head.py`).
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiting role records an error code in
// `status[0]`, stops issuing work and the CTA runs to its normal end (TMEM is released, nothing traps).
#include <cuda.h>

#include "common.cuh"
#include "tspipe_kernels.h"

namespace {

constexpr int BM = 128;          // CTA tile rows  (UMMA M)
constexpr int BK = 64;           // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kThreads = 192;    // warp 0: TMA, warp 1: MMA + TMEM alloc, warps 2..5: epilogue
constexpr uint32_t kSpinLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait.  Returns false (and leaves an error code) when the phase did not complete within the limit.
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
    // deliberate: it is the back-off of the spin loop.  Polling the barrier flat out was measured slower (the
    // waiting warps take issue slots from the one thread that feeds the pipeline).
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

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);          // start address, 16-byte units
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                              // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16: D = f32, A = B = bf16, both K-major, dense.
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
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// TMA store of one 32-row x 128-byte block (128-byte swizzle) from shared memory; rows / columns beyond the
// tensor's extent are clipped by the hardware.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

constexpr int kStoreBufBytes = 32 * 128;             // 32 rows x 128 bytes of C = one TMA store
constexpr int kStoreBytes = 4 * 2 * kStoreBufBytes;  // two staging buffers per epilogue warp

template <int BN>
struct Cfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;             // two accumulator buffers; power of two, <= 512
  static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// epilogue modes
constexpr int EPI_NONE = 0, EPI_BIAS_GELU = 2;   // 1 = bias only

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

constexpr int kMaxBSources = 8;
struct BMaps {
  CUtensorMap m[kMaxBSources];
};

// Persistent kernel: one CTA per SM walks tiles t = blockIdx.x, blockIdx.x + gridDim.x, ...  Two accumulator
// buffers in TMEM let the epilogue of tile i run while the MMAs of tile i+1 are issued; the smem ring keeps
// streaming across tile boundaries.
template <int BN, typename OutT, bool STATS>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ BMaps bmaps,
                    const __grid_constant__ CUtensorMap tmap_c, int tma_store, int rows_per_b, OutT* __restrict__ c, const float* __restrict__ bias, int m, int n, int k, int ldc,
                    int epi, float* __restrict__ col_sums, int seg_rows, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  using C = Cfg<BN>;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* store_bufs = tiles + kStages * C::kStageBytes;   // 1024-aligned: the swizzle follows address bits
  uint64_t* bars = (uint64_t*)(store_bufs + kStoreBytes);
  uint64_t* full_bar = bars;                         // [kStages]  TMA -> MMA
  uint64_t* empty_bar = bars + kStages;              // [kStages]  MMA -> TMA
  uint64_t* tmem_full_bar = bars + 2 * kStages;      // [2]        MMA -> epilogue
  uint64_t* tmem_empty_bar = bars + 2 * kStages + 2; // [2]        epilogue -> MMA
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kStages + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (m + BM - 1) / BM, tiles_n = (n + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar + a, 1);
      mbar_init(tmem_empty_bar + a, 4);              // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&bmaps.m[0]) : "memory");
  }
  if (warp == 1) {        // one full warp allocates both accumulator buffers
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)C::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t round = it / kStages;
          if (round > 0 && !mbar_wait(empty_bar + s, (round - 1) & 1, status, 1)) { ok = false; break; }
          uint8_t* a_dst = tiles + s * C::kStageBytes;
          uint8_t* b_dst = a_dst + C::kABytes;
          mbar_expect_tx(full_bar + s, (uint32_t)C::kStageBytes);
          tma_load_2d(a_dst, &tmap_a, full_bar + s, kb * BK, m0);
          // B may be the row-wise concatenation of several buffers (one per GPU): tile rows n0.. live in
          // source n0 / rows_per_b, which this CTA reads with its own TMA load (local or peer memory alike)
          const int src = n0 / rows_per_b;
          tma_load_2d(b_dst, &bmaps.m[src], full_bar + s, kb * BK, n0 - src * rows_per_b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++lt) {
        const uint32_t acc = lt & 1, use = lt >> 1;
        if (use > 0) {
          ok = mbar_wait(tmem_empty_bar + acc, (use - 1) & 1, status, 4);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t round = it / kStages;
          ok = mbar_wait(full_bar + s, round & 1, status, 2);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(tiles + s * C::kStageBytes);
          const uint32_t b_addr = a_addr + C::kABytes;
          const uint64_t a_desc = make_smem_desc(a_addr), b_desc = make_smem_desc(b_addr);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
            umma_bf16(d_tmem, a_desc + (uint64_t)(2 * kk), b_desc + (uint64_t)(2 * kk), idesc,
                      (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar + s);          // smem slot is free once these MMAs have read it
        }
        umma_commit(tmem_full_bar + acc);      // accumulator complete (or: nothing more will be issued)
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5, TMEM lanes 32*(warp%4) .. +31 ----------------
    // Blocks of 128 output bytes per row (64 bf16 or 32 fp32 columns) go TMEM -> registers -> (bias, GELU,
    // convert) -> swizzled shared memory -> one TMA store of 32 rows; two staging buffers per warp, so the
    // store of block i overlaps the conversion of block i + 1.  Without a usable tensor map for C (unaligned
    // base or row pitch) every thread stores its own row directly.
    constexpr int kCols = 128 / (int)sizeof(OutT);
    const int quarter = warp & 3;
    uint8_t* my_bufs = store_bufs + quarter * 2 * kStoreBufBytes;
    uint32_t lt = 0, nstore = 0;
    bool ok = true;
    // STATS: per-column sum and sum of squares of the rounded outputs (the statistics of a BatchNorm that
    // follows a 1x1 convolution), kept in registers while this warp stays in the same column block and row
    // group: cs[i] = {sum, sumsq of column 2*lane, sum, sumsq of column 2*lane+1} of 64-column block i.
    constexpr int kStatBlocks = BN / 64;
    float cs[kStatBlocks][4];
#pragma unroll
    for (int i = 0; i < kStatBlocks; ++i) { cs[i][0] = cs[i][1] = cs[i][2] = cs[i][3] = 0.f; }
    int cur_n0 = -1, cur_seg = 0;
    auto flush_stats = [&]() {
      if (cur_n0 >= 0) {
        float* dst = col_sums + (int64_t)cur_seg * 2 * n;
#pragma unroll
        for (int i = 0; i < kStatBlocks; ++i) {
          const int col = cur_n0 + 64 * i + 2 * lane;
          if (col < n) { atomicAdd(dst + col, cs[i][0]); atomicAdd(dst + n + col, cs[i][1]); }
          if (col + 1 < n) { atomicAdd(dst + col + 1, cs[i][2]); atomicAdd(dst + n + col + 1, cs[i][3]); }
          cs[i][0] = cs[i][1] = cs[i][2] = cs[i][3] = 0.f;
        }
      }
    };
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++lt) {
      const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
      const uint32_t acc = lt & 1, use = lt >> 1;
      if (STATS) {
        const int seg = m0 / seg_rows;
        if (n0 != cur_n0 || seg != cur_seg) { flush_stats(); cur_n0 = n0; cur_seg = seg; }
      }
      ok = __all_sync(0xffffffffu, mbar_wait(tmem_full_bar + acc, use & 1, status, 3));   // one way out per warp
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row0 = m0 + quarter * 32, row = row0 + lane;
      // one block of kCols columns; returns false past the matrix edge
      auto chunk = [&](int c0, float* st) -> bool {
        if (n0 + c0 >= n) return false;            // columns past the matrix edge: nothing to convert or store
        float v[kCols];
        {
          uint32_t r[kCols];
          const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + (uint32_t)c0;
          tmem_ld_32x32_issue(taddr, r);
          if constexpr (kCols == 64) tmem_ld_32x32_issue(taddr + 32, r + 32);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < kCols; ++j) v[j] = __uint_as_float(r[j]);
        }
        const int col = n0 + c0;
        if (epi != EPI_NONE && col < n) {
#pragma unroll
          for (int j = 0; j < kCols; ++j) {
            v[j] += (col + j < n) ? bias[col + j] : 0.f;
            if (epi == EPI_BIAS_GELU) v[j] = gelu_erf(v[j]);
          }
        }
        if (tma_store) {
          uint8_t* buf = my_bufs + (nstore & 1) * kStoreBufBytes;
          if (nstore >= 2) {         // the store issued two blocks ago has finished reading this buffer
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
          }
          uint8_t* my_row = buf + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {   // 16-byte piece j of this row sits at piece (j ^ (row & 7))
            uint4 q;
            if constexpr (kCols == 64) {
              q.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
              q.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
              q.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
              q.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
            } else {
              q.x = __float_as_uint(v[4 * j + 0]);
              q.y = __float_as_uint(v[4 * j + 1]);
              q.z = __float_as_uint(v[4 * j + 2]);
              q.w = __float_as_uint(v[4 * j + 3]);
            }
            *reinterpret_cast<uint4*>(my_row + ((j ^ (lane & 7)) << 4)) = q;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if (row0 < m && col < n) tma_store_2d(&tmap_c, buf, col, row0);
            else asm volatile("cp.async.bulk.commit_group;" ::: "memory");     // keep the group count in step
          }
          ++nstore;
          if (STATS && st != nullptr) {
            // column sums of the staged (rounded) block: lane owns columns 2*lane, 2*lane+1; rows past the
            // matrix edge hold exact zeros (their A rows were zero-filled)
#pragma unroll 8
            for (int rr = 0; rr < 32; ++rr) {
              const uint32_t wv = *reinterpret_cast<const uint32_t*>(buf + rr * 128 + (((lane >> 2) ^ (rr & 7)) << 4) +
                                                                     (lane & 3) * 4);
              const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv));
              st[0] += f.x; st[1] += f.x * f.x; st[2] += f.y; st[3] += f.y * f.y;
            }
          }
        } else if (row < m && col < n) {
          OutT* dst = c + (int64_t)row * ldc + col;
#pragma unroll
          for (int j = 0; j < kCols; ++j)       // constant indices only: v stays in registers
            if (col + j < n) tsp::st(dst, j, v[j]);
        }
        return true;
      };
      if constexpr (STATS) {
        static_assert(!STATS || kCols == 64, "column statistics are kept for bf16 outputs");
        bool more = true;
#pragma unroll
        for (int i = 0; i < kStatBlocks; ++i)
          if (more) more = chunk(64 * i, cs[i]);
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += kCols)
          if (!chunk(c0, nullptr)) break;
      }
      // this warp has drained its quarter of the accumulator: hand the buffer back to the MMA issuer
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar + acc);
    }
    if (STATS) flush_stats();
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // staging buffers are free again
    __syncwarp();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// host side: tensor maps through the driver entry point (no link-time dependency on libcuda)
// ---------------------------------------------------------------------------------------------
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

// 2-D bf16 row-major [rows, cols] tensor, box = [box_rows, 64 columns], 128-byte swizzle, zero fill out of bounds
bool make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int ld, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_store_map(CUtensorMap* map, void* ptr, int rows, int cols, int ld, bool bf16) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return false;
  const int esz = bf16 ? 2 : 4;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * esz};
  cuuint32_t box[2] = {(cuuint32_t)(128 / esz), 32};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ptr, dims, strides, box,
             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, typename OutT, bool STATS = false>
int launch(const void* a, void* const* b_srcs, int n_src, int rows_per_b, void* c, const float* bias, int m, int n,
           int k, int lda, int ldb, int ldc, int epi, int* status, cudaStream_t stream, float* col_sums = nullptr,
           int seg_rows = 1) {
  CUtensorMap ta;
  BMaps tb;
  if (!make_map(&ta, a, m, k, lda, BM)) return -6;
  for (int i = 0; i < kMaxBSources; ++i) {
    const int src = i < n_src ? i : 0;
    const int rows = n_src == 1 ? n : rows_per_b;
    if (!make_map(&tb.m[i], b_srcs[src], rows, k, ldb, BN)) return -6;
  }
  CUtensorMap tc = ta;          // placeholder when C cannot be described (the kernel then stores directly)
  const bool aligned_c = (((uintptr_t)c & 15) == 0) && ((ldc * (int)sizeof(OutT)) % 16 == 0);
  const int tma_store = aligned_c && make_store_map(&tc, c, m, n, ldc, sizeof(OutT) == 2) ? 1 : 0;
  if (STATS && !tma_store) return -3;           // the statistics are taken from the staged blocks
  auto kern = gemm_tcgen05_kernel<BN, OutT, STATS>;
  static bool attr_set[64] = {};
  static int n_sm[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    cudaDeviceGetAttribute(&n_sm[dev], cudaDevAttrMultiProcessorCount, dev);
    if (n_sm[dev] <= 0) n_sm[dev] = 148;
    attr_set[dev] = true;
  }
  const int num_tiles = ((n + BN - 1) / BN) * ((m + BM - 1) / BM);
  const int grid = num_tiles < n_sm[dev] ? num_tiles : n_sm[dev];
  kern<<<grid, kThreads, Cfg<BN>::kSmemBytes, stream>>>(ta, tb, tc, tma_store, n_src == 1 ? n + BN : rows_per_b,
                                                        (OutT*)c, bias, m, n, k, ldc, epi, col_sums, seg_rows, status);
  return TSP_LAUNCH_CHECK();
}

}  // namespace

extern "C" {

// C[m,n] = A[m,k] * B[n,k]^T (+ bias[n]) (-> GELU).  A, B bf16 row-major with leading dimensions lda / ldb
// (elements; multiples of 8, base pointers 16-byte aligned); C bf16 (out_dtype 1) or fp32 (0), leading dim ldc.
// epi: 0 none, 1 bias, 2 bias + GELU.  `status` is one int in device memory, zeroed by the caller; a non-zero
// value after the kernel means a bounded wait ran out (1 producer, 2 MMA on operands, 3 epilogue, 4 MMA on a free
// accumulator) and C is not valid.
int tsp_gemm_bf16_tn(const void* a, const void* b, void* c, const float* bias, int m, int n, int k, int lda, int ldb,
                     int ldc, int out_dtype, int epi, int* status, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (k % 8)) return -3;
  if (((uintptr_t)a | (uintptr_t)b) & 15) return -2;
  if (epi != 0 && bias == nullptr) return -3;
  void* srcs[1] = {const_cast<void*>(b)};
  const bool wide = n >= 256;
  if (out_dtype == TSP_DTYPE_BF16)
    return wide ? launch<256, __nv_bfloat16>(a, srcs, 1, n, c, bias, m, n, k, lda, ldb, ldc, epi, status, stream)
                : launch<128, __nv_bfloat16>(a, srcs, 1, n, c, bias, m, n, k, lda, ldb, ldc, epi, status, stream);
  return wide ? launch<256, float>(a, srcs, 1, n, c, bias, m, n, k, lda, ldb, ldc, epi, status, stream)
              : launch<128, float>(a, srcs, 1, n, c, bias, m, n, k, lda, ldb, ldc, epi, status, stream);
}

// Same product with B given as `n_src` equally sized row blocks [rows_per_b, k] that may live on different GPUs
// (peer-mapped pointers): C[:, r*rows_per_b : (r+1)*rows_per_b] = A * B_r^T.  This is the all-gather of the
// MoCo keys folded into the contrastive-logit GEMM: every CTA pulls the key tile it needs straight from the owning
// GPU with an ordinary (single-destination) TMA load.  rows_per_b must be a multiple of the N tile (256, or 128
// when the total is below 256).
int tsp_gemm_bf16_tn_gathered_b(const void* a, void* const* b_srcs, int n_src, int rows_per_b, void* c, int m, int k,
                                int lda, int ldb, int ldc, int out_dtype, int* status, cudaStream_t stream) {
  if (m <= 0 || n_src <= 0 || rows_per_b <= 0 || k <= 0) return 0;
  if (n_src > kMaxBSources) return -3;
  if ((lda % 8) || (ldb % 8) || (k % 8)) return -3;
  const int n = n_src * rows_per_b;
  const bool wide = n >= 256 && rows_per_b % 256 == 0;
  if (!wide && rows_per_b % 128 != 0) return -3;
  for (int i = 0; i < n_src; ++i)
    if ((uintptr_t)b_srcs[i] & 15) return -2;
  if (out_dtype == TSP_DTYPE_BF16)
    return wide ? launch<256, __nv_bfloat16>(a, b_srcs, n_src, rows_per_b, c, nullptr, m, n, k, lda, ldb, ldc, 0, status, stream)
                : launch<128, __nv_bfloat16>(a, b_srcs, n_src, rows_per_b, c, nullptr, m, n, k, lda, ldb, ldc, 0, status, stream);
  return wide ? launch<256, float>(a, b_srcs, n_src, rows_per_b, c, nullptr, m, n, k, lda, ldb, ldc, 0, status, stream)
              : launch<128, float>(a, b_srcs, n_src, rows_per_b, c, nullptr, m, n, k, lda, ldb, ldc, 0, status, stream);
}

// C (bf16) = A B^T plus per-column statistics of the rounded result for a BatchNorm that follows: col_sums
// [segs][2n] fp32 (zeroed by the caller) receives, for each of the `segs` consecutive groups of m / segs rows, the
// column sums and the column sums of squares.  m / segs must be a multiple of 128; C 16-byte aligned with a row
// pitch that is a multiple of 16 bytes.
int tsp_gemm_bf16_tn_stats(const void* a, const void* b, void* c, int m, int n, int k, int lda, int ldb, int ldc,
                           float* col_sums, int segs, int* status, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (k % 8) || segs < 1 || m % segs != 0 || (m / segs) % 128 != 0) return -3;
  if (((uintptr_t)a | (uintptr_t)b) & 15) return -2;
  void* const srcs[1] = {const_cast<void*>(b)};
  if (n > 128)
    return launch<256, __nv_bfloat16, true>(a, srcs, 1, n, c, nullptr, m, n, k, lda, ldb, ldc, 0, status, stream, col_sums,
                                            m / segs);
  return launch<128, __nv_bfloat16, true>(a, srcs, 1, n, c, nullptr, m, n, k, lda, ldb, ldc, 0, status, stream, col_sums,
                                          m / segs);
}

}  // extern "C"
