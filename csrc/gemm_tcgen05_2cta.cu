// bf16 GEMM with two SMs per output tile: C[M,N] = A[M,K] * B[N,K]^T, fp32 accumulation, 256 x 256 tiles.
//
// A cluster of two CTAs owns one 256 x 256 tile.  CTA r of the pair loads rows [128 r, 128 r + 128) of the A tile and
// rows [128 r, 128 r + 128) of the B tile (half of N) with its own TMA loads; the leader CTA (rank 0) issues
// tcgen05.mma.cta_group::2, which reads A from both CTAs' shared memory and the two halves of B, and writes each
// CTA's 128 x 256 accumulator slice into that CTA's tensor memory.  Compared with the one-CTA kernel
// (gemm_tcgen05.cu: 48 KB of operands per 128 x 256 x 64 step) each SM moves 32 KB per step for the same FLOPs.
//
// Synchronisation (all mbarriers; every wait bounded in time, see tc5::mbar_wait):
//   full[s]        in the leader: armed by the leader's producer with the bytes of BOTH CTAs; every TMA load of the
//                  pair completes its bytes on the leader's barrier (cp.async.bulk.tensor ... .cta_group::2);
//   empty[g]       in each CTA, one per GROUP of two slots: after the MMAs of a group's second slot the leader issues
//                  ONE tcgen05.commit that arrives on the barrier of both CTAs (a commit costs the issuing thread as
//                  much as eight MMA issues; two per k-block made the issuing thread, not the tensor core, the limit);
//   tmem_full[a]   in each CTA: committed by the leader (to both CTAs at once) after the last MMA of a tile;
//   tmem_empty[a]  in the leader: 8 arrivals, one per epilogue warp of the pair (the peer's arrive remotely).
// Epilogue: TMEM -> registers -> swizzled shared memory -> TMA store (32 rows x 128 bytes per store, two buffers
// per warp); direct per-thread stores when C has no 16-byte-aligned base and row pitch.
// The cluster is synchronised once after barrier initialisation and once before exit, so no CTA leaves while its
// partner can still touch its shared memory.
#include <cuda.h>

#include "tcgen05.cuh"
#include "tspipe_kernels.h"

extern int g_tsp_sm_reserve;          // defined in peer.cu

namespace {

constexpr int BM = 128;          // rows per CTA (pair tile: 256)
constexpr int BN = 256;          // tile columns; each CTA stages BN / 2 rows of B
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kStages = 6;
constexpr int kThreads = 192;
constexpr uint64_t kWaitNs = 2000000000ull;   // every mbarrier wait gives up after two seconds
constexpr int kGroup = 2;                       // stages released per tcgen05.commit
constexpr int kGroups = kStages / kGroup;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = (BN / 2) * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;                  // per CTA
constexpr int kTmemCols = 2 * BN;                               // two accumulator buffers
constexpr int kStoreBufBytes = 32 * 128;                        // 32 rows x 128 bytes of C, one TMA store
constexpr int kStoreBytes = 4 * 2 * kStoreBufBytes;             // two buffers per epilogue warp
constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 + 256;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(local_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory whose byte count completes on a barrier of the pair's leader.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t leader_bar, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(map), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}

__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// one commit that arrives on the barrier at the same shared-memory offset in BOTH CTAs of the pair (a commit costs
// the issuing thread about as much as eight MMA issues, so the pair is signalled with one instruction, not two)
__device__ __forceinline__ void umma_commit_pair_both(uint32_t local_bar_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(local_bar_addr), "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ void umma_bf16_pair_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(tc5::kDescHi), "r"(idesc), "r"(accumulate)
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

template <typename OutT, bool STATS>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_c, int tma_store, OutT* __restrict__ c,
                         const float* __restrict__ bias, int m, int n, int k, int ldc, int epi,
                         float* __restrict__ col_sums, int seg_rows, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* store_bufs = tiles + kStages * kStageBytes; // 1024-aligned: the swizzle pattern follows address bits
  uint64_t* bars = (uint64_t*)(store_bufs + kStoreBytes);
  uint64_t* full_bar = bars;                           // [kStages]  used in the leader only
  uint64_t* empty_bar = bars + kStages;                // [kStages]  in each CTA
  uint64_t* tmem_full_bar = bars + 2 * kStages;        // [2]        in each CTA
  uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;   // [2]        used in the leader only
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kStages + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (m + 2 * BM - 1) / (2 * BM), tiles_n = (n + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar + a, 1);
      mbar_init(tmem_empty_bar + a, 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
  }
  if (warp == 1) {        // warp 1 of BOTH CTAs: paired allocation of both accumulator buffers
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                                   // both CTAs' barriers exist before anyone signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (one thread per CTA) ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        // N tiles fastest: the pairs that run together share rows of A (read from DRAM once, then from L2) and sweep
        // the weights, which stay in L2; walking all of M per N tile would stream A from DRAM once per N tile
        const int m0 = (t / tiles_n) * 2 * BM + (int)rank * BM;
        const int n0 = (t % tiles_n) * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          if (it % kGroup == 0) {                 // first stage of a group: the whole group must have been released
            const uint32_t grp = (it / kGroup) % kGroups, round = (it / kGroup) / kGroups;
            if (round > 0 && !tc5::mbar_wait_parked(empty_bar + grp, (round - 1) & 1, status, 1, kWaitNs)) { ok = false; break; }
          }
          uint8_t* a_dst = tiles + s * kStageBytes;
          uint8_t* b_dst = a_dst + kABytes;
          if (leader) mbar_expect_tx(full_bar + s, 2u * (uint32_t)kStageBytes);
          const uint32_t lbar = map_to_cta(smem_u32(full_bar + s), 0);
          tma_load_2d_pair(a_dst, &tmap_a, lbar, kb * BK, m0);
          tma_load_2d_pair(b_dst, &tmap_b, lbar, kb * BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc(2 * BM, BN);
      const uint32_t tiles_addr = smem_u32(tiles);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs, ++lt) {
        const uint32_t acc = lt & 1, use = lt >> 1;
        if (use > 0) {
          ok = tc5::mbar_wait(tmem_empty_bar + acc, (use - 1) & 1, status, 4, kWaitNs);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t d_tmem = tmem_base + acc * BN;
        uint32_t accum = 0u;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t round = it / kStages;
          ok = tc5::mbar_wait(full_bar + s, round & 1, status, 2, kWaitNs);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = tiles_addr + s * kStageBytes;
          const uint32_t a_lo = tc5::desc_lo_k_major(a_addr), b_lo = tc5::desc_lo_k_major(a_addr + kABytes);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            umma_bf16_pair_lo(d_tmem, a_lo + 2 * kk, b_lo + 2 * kk, idesc, accum);
            accum = 1u;
          }
          // the group's slots are free again in both CTAs once these MMAs have read them
          if (it % kGroup == kGroup - 1) umma_commit_pair_both(smem_u32(empty_bar + (it / kGroup) % kGroups));
        }
        umma_commit_pair_both(smem_u32(tmem_full_bar + acc));
      }
    }
  } else {
    // ---------------- epilogue (both CTAs): this CTA's 128 rows, all BN columns ----------------
    // Per warp: 32 accumulator rows.  Blocks of 128 output bytes per row (64 bf16 or 32 fp32 columns) go
    // TMEM -> registers -> (bias, GELU, convert) -> swizzled shared memory -> one TMA store; two staging
    // buffers per warp, so the store of block i overlaps the conversion of block i + 1.  Without a usable
    // tensor map for C (unaligned base or row pitch) every thread stores its own row directly.
    constexpr int kCols = 128 / (int)sizeof(OutT);
    const int quarter = warp & 3;
    uint8_t* my_bufs = store_bufs + quarter * 2 * kStoreBufBytes;
    uint32_t lt = 0, nstore = 0;
    bool ok = true;
    // STATS: per-column sum and sum of squares of the rounded outputs (the statistics of a BatchNorm that
    // follows a 1x1 convolution), kept in registers while this warp stays in the same column block and row
    // group: cs[i] = {sum, sumsq of column 2*lane, sum, sumsq of column 2*lane+1} of 64-column block i.
    float cs[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { cs[i][0] = cs[i][1] = cs[i][2] = cs[i][3] = 0.f; }
    int cur_n0 = -1, cur_seg = 0;
    auto flush_stats = [&]() {
      if (cur_n0 >= 0) {
        float* dst = col_sums + (int64_t)cur_seg * 2 * n;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = cur_n0 + 64 * i + 2 * lane;
          if (col < n) { atomicAdd(dst + col, cs[i][0]); atomicAdd(dst + n + col, cs[i][1]); }
          if (col + 1 < n) { atomicAdd(dst + col + 1, cs[i][2]); atomicAdd(dst + n + col + 1, cs[i][3]); }
          cs[i][0] = cs[i][1] = cs[i][2] = cs[i][3] = 0.f;
        }
      }
    };
    for (int t = pair; t < num_tiles && ok; t += num_pairs, ++lt) {
      const int m0 = (t / tiles_n) * 2 * BM + (int)rank * BM, n0 = (t % tiles_n) * BN;
      const uint32_t acc = lt & 1, use = lt >> 1;
      if (STATS) {
        const int seg = m0 / seg_rows;
        if (n0 != cur_n0 || seg != cur_seg) { flush_stats(); cur_n0 = n0; cur_seg = seg; }
      }
      ok = tc5::mbar_wait_warp(tmem_full_bar + acc, use & 1, status, 3, kWaitNs, lane);   // one way out per warp
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
        if (epi != 0 && col < n) {
          if (col + kCols <= n && (((uintptr_t)(bias + col)) & 15) == 0) {
            // whole block inside the matrix: the block's bias values as 16-byte loads (every lane reads the same
            // addresses, one broadcast transaction each) instead of one scalar load per element
            const float4* bp = reinterpret_cast<const float4*>(bias + col);
#pragma unroll
            for (int j = 0; j < kCols / 4; ++j) {
              const float4 b4 = __ldg(bp + j);
              v[4 * j + 0] += b4.x; v[4 * j + 1] += b4.y; v[4 * j + 2] += b4.z; v[4 * j + 3] += b4.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < kCols; ++j) v[j] += (col + j < n) ? bias[col + j] : 0.f;
          }
          if (epi == 2) {
#pragma unroll
            for (int j = 0; j < kCols; ++j) v[j] = gelu_erf(v[j]);
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
        if (chunk(0, cs[0]) && chunk(64, cs[1]) && chunk(128, cs[2])) chunk(192, cs[3]);
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += kCols)
          if (!chunk(c0, nullptr)) break;
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(tmem_empty_bar + acc), 0));
    }
    if (STATS) flush_stats();
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // staging buffers are free again
    __syncwarp();
  }
  if (*((volatile int*)status) != 0) {
    // a wait ran out somewhere: give TMA loads and MMAs that are still in flight time to land before the pair's
    // shared memory and tensor memory are released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                                   // nobody touches the partner's memory after this point
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                 : "memory");
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

template <typename OutT, bool STATS>
int launch(const void* a, const void* b, void* c, const float* bias, int m, int n, int k, int lda, int ldb, int ldc,
           int epi, float* col_sums, int seg_rows, int* status, cudaStream_t stream) {
  CUtensorMap ta, tb;
  if (!make_map(&ta, a, m, k, lda, BM) || !make_map(&tb, b, n, k, ldb, BN / 2)) return -6;
  CUtensorMap tc = ta;          // placeholder when C cannot be described (the kernel then stores directly)
  const bool aligned_c = (((uintptr_t)c & 15) == 0) && ((ldc * (int)sizeof(OutT)) % 16 == 0);
  const int tma_store = aligned_c && make_store_map(&tc, c, m, n, ldc, sizeof(OutT) == 2) ? 1 : 0;
  if (STATS && !tma_store) return -3;           // the statistics are taken from the staged blocks
  auto kern = gemm_tcgen05_2cta_kernel<OutT, STATS>;
  static bool attr_set[64] = {};
  static int n_sm[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    cudaDeviceGetAttribute(&n_sm[dev], cudaDevAttrMultiProcessorCount, dev);
    if (n_sm[dev] <= 0) n_sm[dev] = 148;
    attr_set[dev] = true;
  }
  const int num_tiles = ((n + BN - 1) / BN) * ((m + 2 * BM - 1) / (2 * BM));
  int pairs = (n_sm[dev] - g_tsp_sm_reserve) / 2;      // SMs left to communication kernels stay free
  if (pairs < 4) pairs = 4;
  if (pairs > num_tiles) pairs = num_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, tma_store, (OutT*)c, bias, m, n, k, ldc, epi, col_sums, seg_rows, status);
  return (int)e;
}

}  // namespace

extern "C" {

// Two-SM variant of tsp_gemm_bf16_tn, same arguments: C[m,n] = A[m,k] * B[n,k]^T (+ bias[n]) (-> GELU), bf16
// operands, C bf16 or fp32; epi 0 none, 1 bias, 2 bias + GELU.
// `status`: one zeroed int in device memory; non-zero afterwards = a bounded wait ran out (1 producer, 2 MMA on
// operands, 3 epilogue, 4 MMA on a free accumulator) and C is not valid.
int tsp_gemm_bf16_tn_2cta(const void* a, const void* b, void* c, const float* bias, int m, int n, int k, int lda,
                          int ldb, int ldc, int out_dtype, int epi, int* status, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  if (epi != 0 && bias == nullptr) return -3;
  if ((lda % 8) || (ldb % 8) || (k % 8)) return -3;
  if (((uintptr_t)a | (uintptr_t)b) & 15) return -2;
  if (out_dtype == TSP_DTYPE_BF16) return launch<__nv_bfloat16, false>(a, b, c, bias, m, n, k, lda, ldb, ldc, epi, nullptr, 1, status, stream);
  return launch<float, false>(a, b, c, bias, m, n, k, lda, ldb, ldc, epi, nullptr, 1, status, stream);
}

// C (bf16) = A B^T as above, plus per-column statistics of the rounded result for a BatchNorm that follows:
// col_sums [segs][2n] fp32 (zeroed by the caller) receives, for each of the `segs` consecutive groups of
// m / segs rows, the column sums and the column sums of squares.  m / segs must be a multiple of 128; C must be
// 16-byte aligned with a row pitch that is a multiple of 16 bytes.
int tsp_gemm_bf16_tn_2cta_stats(const void* a, const void* b, void* c, int m, int n, int k, int lda, int ldb, int ldc,
                                float* col_sums, int segs, int* status, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (k % 8) || segs < 1 || m % segs != 0 || (m / segs) % 128 != 0) return -3;
  if (((uintptr_t)a | (uintptr_t)b) & 15) return -2;
  return launch<__nv_bfloat16, true>(a, b, c, nullptr, m, n, k, lda, ldb, ldc, 0, col_sums, m / segs, status, stream);
}

}  // extern "C"
