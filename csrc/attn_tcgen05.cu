// Fused softmax(Q K^T * scale) V forward on the 5th-generation tensor cores (flash-attention style: the
// score matrix never leaves the SM).  O[b, i, :] = sum_j p_ij V[b, j, :], lse[b, i] = log sum_j exp(scale * s_ij).
//
// Two users:
//   * attention of the ViT / BERT blocks when no gradient is needed (teacher / momentum-encoder forward):
//     head dim 64, a few hundred keys (`benchmarks/moco-v3/vits.py` via timm's Attention in the reference:
//     two batched GEMMs + softmax kernels);
//   * the MoCo-v3 contrastive loss (`benchmarks/moco-v3/main.py:149-160`): with V = K = normalised keys and
//     scale = 1/T, lse gives the cross-entropy and O the gradient w.r.t. the queries
//     (dL/dq_i = 2/N * (O_i - k_i)), so loss forward and backward are this one kernel and the N x N logits
//     are never written to memory.
//
// One CTA per (128-query tile, batch*head).  Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 softmax
// (thread = query row) and epilogue.
//   S = Q K^T      tcgen05.mma, A = Q [128 x D] and B = K tile [BN x D], both K-major (128-byte swizzle), S in TMEM
//                  (two buffers, so the scores of tile j+1 are computed while tile j is in the softmax);
//   P              exp2 of the scaled scores, written as bf16 into shared memory in the K-major operand layout;
//   O += P V       tcgen05.mma, A = P [128 x BN] K-major, B = V tile [BN x DV] as loaded (MN-major descriptor:
//                  64-column blocks LBO apart, 8-key groups 1024 bytes apart), O accumulates in TMEM.
// Running maximum: O is rescaled in TMEM (tcgen05.ld / tcgen05.st) only when some row's maximum grew; with a
// known bound on the scores (`fixed_max`, e.g. 1/T for cosine logits) no rescaling is ever needed.
// Every mbarrier wait is bounded; a wait that runs out sets *status and all roles leave their loops.
#include <cuda.h>
#include <math.h>

#include "common.cuh"
#include "tspipe_kernels.h"

namespace {

constexpr int BM = 128;
constexpr int kThreads = 192;
constexpr int kStages = 2;
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr float kLog2e = 1.4426950408889634f;

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
// coordinates: (column, row, head, batch)
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z,
                                            int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// K-major operand tile, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// MN-major operand tile as TMA leaves a [k rows][64 contiguous mn elements] box: 128-byte swizzle, the next 64
// mn elements `lbo` bytes further on, the next 8 k rows 1024 bytes further on.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t smem_addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16, D = f32, A = B = bf16, A K-major; B K-major or MN-major (bit 16).
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
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
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

// SAME: V is the very tensor K (contrastive loss): one tile in shared memory serves both products.
template <int D, int DV, int BN, bool SAME>
struct Cfg {
  static constexpr int kQBytes = BM * D * 2;                  // D/64 blocks of [128 rows x 128 bytes]
  static constexpr int kKBytes = BN * D * 2;                  // D/64 blocks of [BN rows x 128 bytes]
  static constexpr int kVBytes = SAME ? 0 : BN * DV * 2;      // DV/64 blocks of [BN rows x 128 bytes]
  static constexpr int kPBytes = BM * BN * 2;                 // BN/64 blocks of [128 rows x 128 bytes]
  static constexpr int kOutBytes = 4 * 32 * 128;              // one 32-row x 128-byte staging block per warp
  static constexpr int kSmemBytes = kQBytes + kStages * (kKBytes + kVBytes) + 2 * kPBytes + kOutBytes + 1024 + 256;
  static constexpr int kTmemCols = 512;
  static constexpr int kOCol = 2 * BN;                        // S buffers at columns 0 and BN, O behind them
};

// K may be the row-wise concatenation of several equally sized buffers (one per GPU): key tile j then comes from
// source (j * BN) / rows_per_src, which this CTA reads with its own TMA load (local or peer memory alike).
constexpr int kMaxKSources = 8;
struct KMaps {
  CUtensorMap m[kMaxKSources];
};

template <int D, int DV, int BN, bool SAME, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ KMaps kmaps, int rows_per_src,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                float* __restrict__ lse, int nq, int nk, int heads, float scale, float fixed_max, int use_fixed_max,
                int* __restrict__ status) {
  using C = Cfg<D, DV, BN, SAME>;
  static_assert(!SAME || D == DV, "one tile can only serve both products when the widths agree");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* q_s = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* kv_s = q_s + C::kQBytes;
  uint8_t* p_s = kv_s + kStages * (C::kKBytes + C::kVBytes);
  uint8_t* out_s = p_s + 2 * C::kPBytes;
  uint64_t* bars = (uint64_t*)(out_s + C::kOutBytes);
  uint64_t* q_full = bars;                 // 1
  uint64_t* kv_full = bars + 1;            // [kStages]
  uint64_t* kv_empty = kv_full + kStages;  // [kStages]
  uint64_t* s_full = kv_empty + kStages;   // [2]  MMA -> softmax
  uint64_t* s_empty = s_full + 2;          // [2]  softmax -> MMA (4 arrivals)
  uint64_t* p_full = s_empty + 2;          // [2]  softmax -> MMA (4 arrivals)
  uint64_t* p_empty = p_full + 2;          // [2]  MMA -> softmax
  uint64_t* o_done = p_empty + 2;          // 1    MMA -> softmax: O holds tiles 0..j (one phase per tile)
  uint64_t* o_final = o_done + 1;          // 1    MMA -> epilogue: every product has completed
  uint32_t* tmem_slot = (uint32_t*)(o_final + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BM, bh = blockIdx.y, head = bh % heads, bat = bh / heads;
  const int n_tiles = (nk + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) { mbar_init(kv_full + s, 1); mbar_init(kv_empty + s, 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full + b, 1);
      mbar_init(s_empty + b, 4);
      mbar_init(p_full + b, 4);
      mbar_init(p_empty + b, 1);
    }
    mbar_init(o_done, 1);
    mbar_init(o_final, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&kmaps.m[0]) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_v) : "memory");
  }
  if (warp == 1) {
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
      mbar_expect_tx(q_full, (uint32_t)C::kQBytes);
      for (int kb = 0; kb < D / 64; ++kb) tma_load_4d(q_s + kb * (BM * 128), &tmap_q, q_full, kb * 64, q0, head, bat);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kStages;
        const uint32_t round = j / kStages;
        if (round > 0 && !mbar_wait(kv_empty + s, (round - 1) & 1, status, 1)) break;
        uint8_t* k_dst = kv_s + s * (C::kKBytes + C::kVBytes);
        uint8_t* v_dst = k_dst + C::kKBytes;
        mbar_expect_tx(kv_full + s, (uint32_t)(C::kKBytes + C::kVBytes));
        const int src = (j * BN) / rows_per_src, row_in_src = j * BN - src * rows_per_src;
        for (int kb = 0; kb < D / 64; ++kb)
          tma_load_4d(k_dst + kb * (BN * 128), &kmaps.m[src], kv_full + s, kb * 64, row_in_src, head, bat);
        if (!SAME) {
          for (int cb = 0; cb < DV / 64; ++cb)
            tma_load_4d(v_dst + cb * (BN * 128), &tmap_v, kv_full + s, cb * 64, j * BN, head, bat);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(BM, BN, false);
      constexpr uint32_t idesc_o = make_idesc(BM, DV, true);
      bool ok = mbar_wait(q_full, 0, status, 2);
      auto issue_s = [&](int j) -> bool {              // S[j & 1] = Q K_j^T
        const int s = j % kStages;
        if (!mbar_wait(kv_full + s, (j / kStages) & 1, status, 2)) return false;
        if (j >= 2 && !mbar_wait(s_empty + (j & 1), ((j >> 1) - 1) & 1, status, 4)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t q_addr = smem_u32(q_s), k_addr = smem_u32(kv_s + s * (C::kKBytes + C::kVBytes));
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int kb = kk >> 2, in = kk & 3;
          umma_bf16(tmem_base + (uint32_t)((j & 1) * BN), desc_k_major(q_addr + kb * (BM * 128)) + (uint64_t)(2 * in),
                    desc_k_major(k_addr + kb * (BN * 128)) + (uint64_t)(2 * in), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(s_full + (j & 1));
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        ok = mbar_wait(p_full + (j & 1), (j >> 1) & 1, status, 5);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int s = j % kStages;
        const uint32_t p_addr = smem_u32(p_s + (j & 1) * C::kPBytes);
        const uint32_t v_addr = smem_u32(kv_s + s * (C::kKBytes + C::kVBytes) + (SAME ? 0 : C::kKBytes));
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {           // 16 keys per MMA
          const int kb = ks >> 2, in = ks & 3;
          umma_bf16(tmem_base + (uint32_t)C::kOCol, desc_k_major(p_addr + kb * (BM * 128)) + (uint64_t)(2 * in),
                    desc_mn_major(v_addr + ks * (16 * 128), BN * 128), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(kv_empty + s);
        umma_commit(p_empty + (j & 1));
        umma_commit(o_done);
      }
      if (ok) umma_commit(o_final);
    }
  } else {
    // ---------------- softmax + epilogue: thread = query row ----------------
    const int quarter = warp & 3;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int r = quarter * 32 + lane;                  // row inside the tile
    const float sc2 = scale * kLog2e;
    float m_run = use_fixed_max ? fixed_max * kLog2e : -INFINITY;   // running maximum, log2 domain
    float l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int b = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(s_full + b, (j >> 1) & 1, status, 3));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float x[BN];
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 32) tmem_ld32(tmem_base + lane_addr + (uint32_t)(b * BN + c0), reinterpret_cast<uint32_t*>(x) + c0);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty + b);          // the scores are in registers
      const int n_valid = nk - j * BN;                  // keys beyond nk were zero-filled by TMA: mask them
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < BN; ++c) {
        x[c] = c < n_valid ? x[c] * sc2 : -INFINITY;
        mx = fmaxf(mx, x[c]);
      }
      float alpha = 1.f;
      if (!use_fixed_max) {
        const float m_new = fmaxf(m_run, mx);
        alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
        m_run = m_new;
      }
      float sum = 0.f;
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
#pragma unroll
      for (int c = 0; c < BN; ++c) {
        x[c] = exp2f(x[c] - m_use);
        sum += x[c];
      }
      l_run = l_run * alpha + sum;
      if (j > 0 && !use_fixed_max) {
        // O (tiles 0..j-1) must be complete before it is rescaled or added to
        ok = __all_sync(0xffffffffu, mbar_wait(o_done, (j - 1) & 1, status, 6));
        if (!ok) break;
        if (!__all_sync(0xffffffffu, alpha == 1.f)) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
          for (int c0 = 0; c0 < DV; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tmem_base + lane_addr + (uint32_t)(C::kOCol + c0), o);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st32(tmem_base + lane_addr + (uint32_t)(C::kOCol + c0), o);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
      }
      if (j >= 2) {                                     // P[b] was last read by the MMAs of tile j - 2
        ok = __all_sync(0xffffffffu, mbar_wait(p_empty + b, ((j >> 1) - 1) & 1, status, 7));
        if (!ok) break;
      }
      uint8_t* p_row = p_s + b * C::kPBytes + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
      for (int q = 0; q < BN / 8; ++q) {                // 16-byte piece q of the row: keys 8q .. 8q+7
        uint4 v;
        v.x = pack_bf16x2(x[8 * q + 0], x[8 * q + 1]);
        v.y = pack_bf16x2(x[8 * q + 2], x[8 * q + 3]);
        v.z = pack_bf16x2(x[8 * q + 4], x[8 * q + 5]);
        v.w = pack_bf16x2(x[8 * q + 6], x[8 * q + 7]);
        *reinterpret_cast<uint4*>(p_row + (q >> 3) * (BM * 128) + (((q & 7) ^ (r & 7)) << 4)) = v;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + b);
    }
    // ---------------- epilogue: O / l -> global, lse ----------------
    if (ok && n_tiles > 0) ok = __all_sync(0xffffffffu, mbar_wait(o_final, 0, status, 8));
    if (ok && n_tiles > 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      constexpr int kCols = 128 / (int)sizeof(OutT);    // columns per 128-byte staging row
      uint8_t* buf = out_s + quarter * (32 * 128);
      const int row0 = q0 + quarter * 32;
#pragma unroll 1
      for (int c0 = 0; c0 < DV; c0 += kCols) {
        uint32_t o[kCols];
        tmem_ld32(tmem_base + lane_addr + (uint32_t)(C::kOCol + c0), o);
        if constexpr (kCols == 64) tmem_ld32(tmem_base + lane_addr + (uint32_t)(C::kOCol + c0 + 32), o + 32);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (c0 > 0) {                                    // the previous block's store has read the buffer
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
        }
        uint8_t* my_row = buf + lane * 128;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          uint4 v;
          if constexpr (kCols == 64) {
            v.x = pack_bf16x2(__uint_as_float(o[8 * q + 0]) * inv_l, __uint_as_float(o[8 * q + 1]) * inv_l);
            v.y = pack_bf16x2(__uint_as_float(o[8 * q + 2]) * inv_l, __uint_as_float(o[8 * q + 3]) * inv_l);
            v.z = pack_bf16x2(__uint_as_float(o[8 * q + 4]) * inv_l, __uint_as_float(o[8 * q + 5]) * inv_l);
            v.w = pack_bf16x2(__uint_as_float(o[8 * q + 6]) * inv_l, __uint_as_float(o[8 * q + 7]) * inv_l);
          } else {
            v.x = __float_as_uint(__uint_as_float(o[4 * q + 0]) * inv_l);
            v.y = __float_as_uint(__uint_as_float(o[4 * q + 1]) * inv_l);
            v.z = __float_as_uint(__uint_as_float(o[4 * q + 2]) * inv_l);
            v.w = __float_as_uint(__uint_as_float(o[4 * q + 3]) * inv_l);
          }
          *reinterpret_cast<uint4*>(my_row + ((q ^ (lane & 7)) << 4)) = v;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          if (row0 < nq) tma_store_4d(&tmap_o, buf, c0, row0, head, bat);
          else asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      __syncwarp();
      if (lse != nullptr && q0 + r < nq)
        lse[(int64_t)bh * nq + q0 + r] = l_run > 0.f ? (m_run + log2f(l_run)) / kLog2e : -INFINITY;
    }
  }
  if (*((volatile int*)status) != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);      // let copies and MMAs that are still in flight land
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols)
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

// [batch][head][rows][cols] view: `ld` elements between rows, `hs` between heads, `bs` between batches.
bool make_map4(CUtensorMap* map, const void* ptr, int batch, int heads, int rows, int cols, int64_t ld, int64_t hs,
               int64_t bs, int box_cols, int box_rows, bool fp32) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return false;
  const int esz = fp32 ? 4 : 2;
  cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)heads, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)ld * esz, (cuuint64_t)hs * esz, (cuuint64_t)bs * esz};
  cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr),
             dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Strides { int64_t ld, hs, bs; };

template <int D, int DV, int BN, bool SAME, typename OutT>
int launch(const void* q, void* const* k_srcs, int n_src, const void* v, void* o, float* lse, int batch, int heads, int nq,
           int nk, Strides sq, Strides sk, Strides sv, Strides so, float scale, float fixed_max, int use_fixed_max,
           int* status, cudaStream_t stream) {
  using C = Cfg<D, DV, BN, SAME>;
  CUtensorMap tq, tv, to;
  KMaps tk;
  constexpr bool f32 = sizeof(OutT) == 4;
  const int rows_per_src = n_src == 1 ? nk : nk / n_src;
  for (int i = 0; i < kMaxKSources; ++i)
    if (!make_map4(&tk.m[i], k_srcs[i < n_src ? i : 0], batch, heads, rows_per_src, D, sk.ld, sk.hs, sk.bs, 64, BN, false))
      return -6;
  if (!make_map4(&tq, q, batch, heads, nq, D, sq.ld, sq.hs, sq.bs, 64, BM, false) ||
      !make_map4(&tv, v, batch, heads, SAME ? rows_per_src : nk, DV, sv.ld, sv.hs, sv.bs, 64, BN, false) ||
      !make_map4(&to, o, batch, heads, nq, DV, so.ld, so.hs, so.bs, f32 ? 32 : 64, 32, f32))
    return -6;
  auto kern = attn_fwd_kernel<D, DV, BN, SAME, OutT>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  dim3 grid((nq + BM - 1) / BM, batch * heads);
  kern<<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, n_src == 1 ? nk + BN : rows_per_src, tv, to, lse, nq, nk, heads,
                                                  scale, fixed_max, use_fixed_max, status);
  return TSP_LAUNCH_CHECK();
}

}  // namespace

extern "C" {

// O[b, h, i, :] = softmax_j(scale * Q[b, h, i, :] . K[b, h, j, :]) V[b, h, j, :].
// Q, K, V bf16; element (b, h, row, col) of X lives at X + b * X_strides[2] + h * X_strides[1] + row * X_strides[0]
// + col (strides in elements, multiples of 8; base pointers 16-byte aligned), so heads that are interleaved in
// memory (the qkv projection's output) need no copy.  O bf16 (out_dtype 1) or fp32 (0).  lse (optional)
// [batch * heads][nq] fp32.  (d, dv) = (64, 64), or (256, 256) with V the same tensor as K (contrastive loss).
// use_fixed_max: scale * s <= fixed_max is known to hold for every score (p = exp(scale * s - fixed_max) cannot
// overflow), which removes all rescaling.
// `status`: one zeroed int in device memory; non-zero afterwards = a bounded wait ran out and O is not valid.
int tsp_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int heads, int nq, int nk,
                 int d, int dv, const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                 const int64_t* o_strides, float scale, float fixed_max, int use_fixed_max, int out_dtype, int* status,
                 cudaStream_t stream) {
  if (batch <= 0 || heads <= 0 || nq <= 0 || nk <= 0) return 0;
  if ((int64_t)batch * heads > 65535) return -3;
  if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15) != 0) return -2;
  const Strides sq = {q_strides[0], q_strides[1], q_strides[2]}, sk = {k_strides[0], k_strides[1], k_strides[2]},
                sv = {v_strides[0], v_strides[1], v_strides[2]}, so = {o_strides[0], o_strides[1], o_strides[2]};
  if ((sq.ld | sq.hs | sq.bs | sk.ld | sk.hs | sk.bs | sv.ld | sv.hs | sv.bs) & 7) return -3;
  const bool bf16 = out_dtype == TSP_DTYPE_BF16;
  const int oesz = bf16 ? 2 : 4;
  if ((so.ld * oesz) % 16 != 0 || (so.hs * oesz) % 16 != 0 || (so.bs * oesz) % 16 != 0) return -3;
  void* const srcs[1] = {const_cast<void*>(k)};
#define TSP_ATTN_ARGS q, srcs, 1, v, o, lse, batch, heads, nq, nk, sq, sk, sv, so, scale, fixed_max, use_fixed_max, status, stream
  if (d == 64 && dv == 64)
    return bf16 ? launch<64, 64, 128, false, __nv_bfloat16>(TSP_ATTN_ARGS) : launch<64, 64, 128, false, float>(TSP_ATTN_ARGS);
  if (d == 256 && dv == 256 && k == v && sk.ld == sv.ld && sk.hs == sv.hs && sk.bs == sv.bs)
    return bf16 ? launch<256, 256, 64, true, __nv_bfloat16>(TSP_ATTN_ARGS) : launch<256, 256, 64, true, float>(TSP_ATTN_ARGS);
#undef TSP_ATTN_ARGS
  return -3;
}

// Contrastive-loss form with the keys of `n_src` replicas read in place: Q [nq][256] bf16 (pitch 256), K = V = the
// row-wise concatenation of k_srcs[0..n_src) (each [rows_per_src][256] bf16, pitch 256; pointers may be peer
// memory - every CTA fetches its own tiles with plain TMA loads).  O [nq][256] fp32, lse [nq].  rows_per_src % 64 == 0.
int tsp_attn_nce_gathered(const void* q, void* const* k_srcs, int n_src, int rows_per_src, void* o, float* lse, int nq,
                          float scale, float fixed_max, int* status, cudaStream_t stream) {
  if (nq <= 0 || n_src <= 0 || rows_per_src <= 0) return 0;
  if (n_src > kMaxKSources || rows_per_src % 64 != 0) return -3;
  if ((((uintptr_t)q | (uintptr_t)o) & 15) != 0) return -2;
  for (int i = 0; i < n_src; ++i)
    if (((uintptr_t)k_srcs[i] & 15) != 0) return -2;
  const int nk = n_src * rows_per_src;
  const Strides sq = {256, (int64_t)nq * 256, (int64_t)nq * 256};
  const Strides sk = {256, (int64_t)rows_per_src * 256, (int64_t)rows_per_src * 256};
  return launch<256, 256, 64, true, float>(q, k_srcs, n_src, k_srcs[0], o, lse, 1, 1, nq, nk, sq, sk, sk, sq, scale,
                                           fixed_max, 1, status, stream);
}

}  // extern "C"
