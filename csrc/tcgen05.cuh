// Device and host helpers shared by the tcgen05 / TMEM / TMA kernels: mbarriers with bounded waits, TMA tile
// loads, shared-memory matrix descriptors (K-major and MN-major, 128-byte swizzle), the kind::f16 instruction
// descriptor, MMA issue / commit, TMEM loads, and tensor-map encoding through the driver entry point.
#pragma once
#include <cuda.h>
#include <dlfcn.h>

#include "common.cuh"

namespace tc5 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t addr, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(addr), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait.  Returns false (and leaves `code` in *status unless another role got there first) when the phase
// did not complete within `limit_ns` nanoseconds.  mbarrier.try_wait suspends the thread for a short,
// hardware-chosen time per attempt, so the loop does not fight the issuing threads for slots; every 32 failed
// attempts it looks at the error word in global memory (so that all roles leave once one of them gave up) and at
// the clock.  A stage of these kernels is 0.1 - 0.4 us of tensor-core work: checking the error word after every
// attempt (an L2 round trip of about that length) would make every hand-over late.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code, uint64_t limit_ns) {
  const uint32_t addr = smem_u32(bar);
  uint64_t t0 = 0;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(addr, parity)) return true;
    if (*((volatile int*)status) != 0) return false;
    const uint64_t now = global_timer_ns();
    if (t0 == 0) t0 = now;
    else if (now - t0 > limit_ns) break;
  }
  atomicCAS(status, 0, code);
  return false;
}

// Wait of a role that is not on the critical path (epilogue warps, the TMA producer): mbarrier.try_wait with a long
// suspend-time hint parks the thread until the phase completes or the hint expires, so a waiting warp issues a few
// instructions per microsecond instead of competing with the MMA-issuing thread on its scheduler.
__device__ __forceinline__ bool mbar_wait_parked(uint64_t* bar, uint32_t parity, int* status, int code,
                                                 uint64_t limit_ns) {
  const uint32_t addr = smem_u32(bar);
  uint64_t t0 = 0;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 8; ++i) {
      uint32_t done;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
          "selp.b32 %0, 1, 0, p;\n\t}"
          : "=r"(done)
          : "r"(addr), "r"(parity), "r"(2000u)
          : "memory");
      if (done) return true;
    }
    if (*((volatile int*)status) != 0) return false;
    const uint64_t now = global_timer_ns();
    if (t0 == 0) t0 = now;
    else if (now - t0 > limit_ns) break;
  }
  atomicCAS(status, 0, code);
  return false;
}
// The same for a whole warp: lane 0 waits, the others park at the warp barrier; every lane gets the result.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, int* status, int code, uint64_t limit_ns,
                                               int lane) {
  int ok = 0;
  if (lane == 0) ok = mbar_wait_parked(bar, parity, status, code, limit_ns) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// The MMA-issuing thread is the one serial resource of these kernels (an issue costs it about 50 cycles), so its loop
// works on 32-bit halves of the matrix descriptors: the high word (stride byte offset 1024, version, 128-byte swizzle)
// is the same constant for K-major and MN-major tiles, the low word is (address >> 4) plus the leading-byte-offset
// field, and stepping through a tile only ever adds to the low word (shared-memory addresses stay below 2^18, so the
// 14-bit address field cannot carry).
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo_k_major(uint32_t smem_addr) { return (smem_addr >> 4) | (1u << 16); }
__device__ __forceinline__ uint32_t desc_lo_mn_major(uint32_t smem_addr, uint32_t lbo) {
  return (smem_addr >> 4) | ((lbo >> 4) << 16);
}
__device__ __forceinline__ void umma_bf16_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z,
                                            int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// TMA store of one 32-row x 128-byte block (128-byte swizzle) from shared memory; rows / columns beyond the
// tensor's extent are clipped by the hardware.  x must be a multiple of 8 elements (16 bytes).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// K-major operand tile [rows][64 bf16 = 128 bytes], 128-byte swizzle, 8-row groups 1024 bytes apart.  Advancing 16
// elements along K inside the swizzled row = +2 in the (16-byte) address field.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;                              // leading byte offset: unused for swizzled K-major
  d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                              // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
  return d;
}
// MN-major operand tile as TMA leaves a [k rows][64 contiguous mn elements] box: 128-byte swizzle, the next 64 mn
// elements `lbo` bytes further on, the next 8 k rows 1024 bytes further on.  Advancing 16 along K = +2048 bytes.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t smem_addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16 instruction descriptor: D = f32, A = B = bf16, dense; either operand K-major or MN-major.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (a_mn_major ? (1u << 15) : 0u) | (b_mn_major ? (1u << 16) : 0u) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
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
// arrive on `bar` once every MMA issued so far by this thread has completed
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

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

// ---------------------------------------------------------------------------------------------------------------
// host side: tensor maps through the driver entry point (no link-time dependency on libcuda)
// ---------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess && p != nullptr) {
      fn = (EncodeTiledFn)p;
    } else {
      (void)cudaGetLastError();               // the query failed (seen on a thread's first runtime call): ask the
      void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);      // driver library itself
      if (h != nullptr) fn = (EncodeTiledFn)dlsym(h, "cuTensorMapEncodeTiled");
    }
  }
  return fn;
}

// bf16 tensor of up to 4 dimensions, innermost first: dims[i] elements, strides[i] BYTES for i >= 1 (the innermost
// dimension is contiguous), box[i] elements.  128-byte swizzle: box[0] must be 64.  Out-of-range elements read as 0.
inline bool make_bf16_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                          const uint32_t* box) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return false;
  cuuint64_t d[4], s[3];
  cuuint32_t b[4], e[4];
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; e[i] = 1; }
  for (int i = 1; i < rank; ++i) s[i - 1] = strides[i];
  CUresult r = CUDA_ERROR_UNKNOWN;
  for (int attempt = 0; attempt < 2 && r != CUDA_SUCCESS; ++attempt) {
    // The encoder is a driver call and wants a current context.  A thread that has not made a runtime call yet (an
    // autograd worker calling straight into this library) has none: bind the device's primary context and retry.
    if (attempt == 1) (void)cudaFree(nullptr);
    r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS;
}

}  // namespace tc5
