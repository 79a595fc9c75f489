// Implicit-GEMM convolutions (and the matching products of linear layers) on the 5th-generation tensor cores.
//
// Activations are channels-last bf16 ([N, H, W, C], C a multiple of 64), weights bf16 [Cout][kh][kw][Cin], square
// kernels of size 1 or 3, stride 1 or 2, padding (k - 1) / 2.  Three products, all with fp32 accumulation in TMEM:
//
//   forward    Y[p, co]  = sum_{tap, ci} X[p + tap, ci] * W[co, tap, ci]            (tsp_conv_fprop)
//   data grad  dX[p, ci] = sum_{tap, co} dY[p - tap, co] * W[co, tap, ci]           (tsp_conv_dgrad)
//   weight grad dW[co, tap, ci] += sum_p X[p + tap, ci] * dY[p, co]                 (tsp_conv_wgrad)
//
// No im2col buffer exists anywhere: an M tile is a BOX of output pixels (w x h x n, at most 128 of them) and the
// operand tile for one filter tap is that same box shifted by the tap's offset, fetched by ONE 4-D TMA tile load
// (cp.async.bulk.tensor.4d, 128-byte swizzle); rows that fall into the padding are zero-filled by the TMA unit.
// Stride 2 needs no strided traversal either: the input is addressed through four tensor maps, one per (row, column)
// parity, each an ordinary dense view with doubled pitches, and every tap reads exactly one of them.  A 1x1 stride-1
// convolution degenerates to a plain GEMM over the flattened pixels (box = 128 consecutive pixels).
//
// A 3x3 stride-1 convolution of an image at most 61 pixels wide does not fetch nine shifted boxes per channel block
// (nine trips through L2 for the same pixels): conv_halo_kernel loads the box ONCE with a one-pixel border
// ((w + 2) x (h + 2) pixels, border zero-filled by TMA), enumerates the accumulator rows in that bordered pitch, and
// the operand of tap (kh, kw) is the same shared-memory tile read from row kh * (w + 2) + kw on - a shifted start
// address in the matrix descriptor (whose base-offset field carries the swizzle phase of the shifted start).  The
// rows that correspond to border columns are computed and thrown away.
//
//   forward / data grad (conv_fwd_kernel): A = shifted pixel box [pixels x 64 channels], K-major; B = weight tile,
//     K-major for the forward ([co][tap, ci] rows) and MN-major for the data gradient (the same weight matrix read
//     as [co rows (K)][ci (N)] boxes, so no transposed copy of the weights is ever made).  The data gradient of a
//     stride-2 convolution runs once per output parity class with the taps that reach that class.  Epilogue: TMEM ->
//     registers -> bf16 -> shared memory -> 16-byte coalesced stores to the pixel addresses; optionally per-channel
//     sum / sum of squares of the rounded outputs (the statistics of the BatchNorm that follows), per view segment.
//   weight grad (conv_wgrad_kernel): both operands are pixel boxes as loaded, i.e. MN-major: M = (tap, ci) (two
//     64-channel boxes of the shifted input), N = co (BN / 64 boxes of dY), K = the box's pixels.  The pixel range is
//     split over CTAs and every CTA adds its partial tile into the fp32 gradient with red.global.add.f32 (coalesced
//     along ci), which is also what accumulates micro-batches.
//
// Roles per CTA (192 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-5 epilogue.  Persistent
// over tiles, shared-memory ring of 3-6 stages, two accumulator buffers in TMEM so the epilogue of tile i overlaps
// the MMAs of tile i + 1.  Every mbarrier wait is bounded: a wait that runs out writes a code into *status (1 producer,
// 2 MMA on operands, 3 epilogue, 4 MMA on a free accumulator), all roles leave their loops, TMEM is released.
//
// Reference call sites: every nn.Conv2d of the torchvision ResNets (`benchmarks/byol/models/resnet_base_network.py:60-77`,
// `benchmarks/soft_target/models/resnet.py`) and every nn.Linear backward of the ViT / BERT blocks and MLP heads
// (`benchmarks/moco-v3/vits.py`, `benchmarks/distilbert/bert.py:104-266`, `benchmarks/byol/models/mlp_head.py:4-26`),
// all library (cuDNN / cuBLAS) calls there.
#include <cuda.h>
#include <stdlib.h>

#include "tcgen05.cuh"
#include "tspipe_kernels.h"

namespace {

using namespace tc5;

constexpr int kThreads = 320;           // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue (two per TMEM lane quarter)
constexpr int kWgThreads = 192;         // weight gradient: warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int kBoxBytes = 128 * 128;        // shared memory reserved per pixel box: 128 rows x 64 bf16
constexpr int kMaxTaps = 9;

struct Geom {
  int out_w, out_h, out_n;                  // extent of the pixel grid the tiles walk
  int box_w, box_h, box_n;                  // pixel box of one tile
  int tiles_w, tiles_h, tiles_n;
  int row_pitch;                            // accumulator rows per box row: box_w, or box_w + 2 in the halo kernel
  int pix;                                  // row_pitch * box_h * box_n  (<= 128): accumulator rows in use
  int halo_rows;                            // halo kernel: (box_w + 2) * (box_h + 2) rows fetched per channel block
  int b_resident;                           // halo kernel: the nine weight tiles are loaded once and stay
  int tma_store;                            // forward kernel, flat pixel grid: the epilogue writes with TMA stores
  int n_fastest;                            // tile index = m_tile * tiles_n + n_tile (else n_tile * tiles_m + m_tile)
  unsigned long long wait_ns;               // give-up time of every mbarrier wait
  int n_taps;
  int kc;                                   // channels per tap on the contraction side (forward) / on the M side (wgrad)
  int nc;                                   // channels on the N side
  int rows_per_seg;                         // statistics: pixels per segment, in walk order (n, h, w)
  int out_sn, out_sh, out_sw;               // output pitches of the pixel grid, in units of 8 elements
  int ldw;                                  // wgrad: row pitch of dW in elements
  int splits;                               // wgrad: pieces of the pixel range
  int tap_dw[kMaxTaps], tap_dh[kMaxTaps], tap_map[kMaxTaps], tap_col[kMaxTaps];
  int tap_off[kMaxTaps];                    // halo kernel: first shared-memory row of the tap's operand
};
struct ActMaps {
  CUtensorMap m[4];
};

template <int BN>
struct FwdCfg {
  static constexpr int kABytes = kBoxBytes;
  static constexpr int kBBytes = BN * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kGroup = 2;                          // stages released per tcgen05.commit (a commit costs the
  static constexpr int kGroups = kStages / kGroup;          // issuing thread about as much as eight MMAs)
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kStoreBytes = 8 * 32 * 128;          // one 32-row x 128-byte staging block per epilogue warp
  static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 + 256;
};

// Tiles are dealt to the CTAs in contiguous ranges (tile index = n_tile * tiles_m + m_tile): a CTA then stays on one
// block of output channels - one set of weights, one set of statistics accumulators - for nearly all of its tiles,
// and consecutive tiles are neighbouring pixel boxes.
__device__ __forceinline__ int tile_begin(int num_tiles, unsigned cta) {
  return (int)((long long)num_tiles * cta / gridDim.x);
}

// Split a tile index into (pixel tile, channel tile).  With statistics a CTA should stay on one channel block (one set
// of accumulators, few flushes): channel-major.  Without, channel tiles run fastest: the CTAs that run together share
// a pixel tile's input (fetched from DRAM once, then from L2) and sweep the weights, which stay in L2.
__device__ __forceinline__ void split_tile(const Geom& g, int t, int tiles_m, int tiles_nn, int& tm, int& tn) {
  if (g.n_fastest) { tm = t / tiles_nn; tn = t % tiles_nn; }
  else { tm = t % tiles_m; tn = t / tiles_m; }
}

__device__ __forceinline__ void tile_origin(const Geom& g, int tm, int& w0, int& h0, int& n0) {
  const int wb = tm % g.tiles_w, r = tm / g.tiles_w;
  w0 = wb * g.box_w;
  h0 = (r % g.tiles_h) * g.box_h;
  n0 = (r / g.tiles_h) * g.box_n;
}

// Epilogue warps (2..9) of the forward / data-gradient kernels.  A tile has `n_sub` accumulators of 128 rows (SUBS
// reserved per TMEM buffer); accumulator row p of the tile (p = 128 * sub + TMEM lane) is pixel
// (p % row_pitch, (p / row_pitch) % box_h, p / (row_pitch * box_h)) of the tile's box; rows in border columns, past
// the box or outside the image are not stored.  Warp w owns TMEM lanes 32 * (w % 4) .. + 31; the two warps that share
// a lane quarter split the (accumulator, 64-channel block) units between them.  Per unit: TMEM -> registers -> bf16
// -> swizzled shared memory (rows that are not stored are written as zeros) -> per-channel sums from shared memory
// (STATS) and coalesced 16-byte stores, 8 lanes per pixel.
template <int BN, int SUBS, int ACC_BUFS, bool STATS>
__device__ __forceinline__ void fwd_epilogue(const Geom& g, int num_tiles, int tiles_m, int n_sub, uint32_t tmem_base,
                                             uint64_t* tmem_full_bar, uint64_t* tmem_empty_bar, uint8_t* store_bufs,
                                             __nv_bfloat16* __restrict__ out, float* __restrict__ col_sums,
                                             int* __restrict__ status, int warp, int lane,
                                             const CUtensorMap* __restrict__ omap = nullptr) {
  const int quarter = warp & 3, group = (warp - 2) >> 2;
  const bool tma_out = omap != nullptr && g.tma_store != 0;       // flat pixel grid: 32-row blocks go out as TMA stores
  uint8_t* buf = store_bufs + (warp - 2) * (32 * 128);
  uint32_t lt = 0;
  bool ok = true;
  constexpr int kStatBlocks = BN / 64;
  float cs[kStatBlocks][4];
#pragma unroll
  for (int i = 0; i < kStatBlocks; ++i) { cs[i][0] = cs[i][1] = cs[i][2] = cs[i][3] = 0.f; }
  int cur_c0 = -1, cur_seg = 0;
  auto flush_stats = [&]() {
    if (cur_c0 >= 0) {
      float* dst = col_sums + (int64_t)cur_seg * 2 * g.nc;
#pragma unroll
      for (int i = 0; i < kStatBlocks; ++i) {
        const int col = cur_c0 + 64 * i + 2 * lane;
        // (the blocks of the other warp of this lane quarter hold zeros here; nc is even: col and col + 1 exist together)
        if (col < g.nc && (cs[i][1] != 0.f || cs[i][3] != 0.f)) {
          atomicAdd(dst + col, cs[i][0]); atomicAdd(dst + g.nc + col, cs[i][1]);
          atomicAdd(dst + col + 1, cs[i][2]); atomicAdd(dst + g.nc + col + 1, cs[i][3]);
        }
        cs[i][0] = cs[i][1] = cs[i][2] = cs[i][3] = 0.f;
      }
    }
  };
  const int t_begin = tile_begin(num_tiles, blockIdx.x), t_end = tile_begin(num_tiles, blockIdx.x + 1);
  for (int t = t_begin; t < t_end && ok; ++t, ++lt) {
    int w0, h0, n0, tm, tn;
    split_tile(g, t, tiles_m, (g.nc + BN - 1) / BN, tm, tn);
    tile_origin(g, tm, w0, h0, n0);
    const int c0 = tn * BN;
    const uint32_t acc = lt % ACC_BUFS, use = lt / ACC_BUFS;
    if (STATS) {
      const int seg = (int)((((int64_t)n0 * g.out_h + h0) * g.out_w + w0) / g.rows_per_seg);
      if (c0 != cur_c0 || seg != cur_seg) { flush_stats(); cur_c0 = c0; cur_seg = seg; }
    }
    ok = mbar_wait_warp(tmem_full_bar + acc, use & 1, status, 3, g.wait_ns, lane);
    if (!ok) break;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
    for (int sub = 0; sub < SUBS; ++sub) {
      if (sub < n_sub) {
        // this lane's pixel and where it is stored (units of 8 elements), -1 for rows that are not stored
        int row_off = -1;
        {
          const int p = sub * 128 + quarter * 32 + lane;
          const int bw = p % g.row_pitch, r2 = p / g.row_pitch;
          const int w = w0 + bw, h = h0 + r2 % g.box_h, n = n0 + r2 / g.box_h;
          if (p < g.pix && bw < g.box_w && w < g.out_w && h < g.out_h && n < g.out_n)
            row_off = n * g.out_sn + h * g.out_sh + w * g.out_sw;
        }
#pragma unroll
        for (int i = 0; i < kStatBlocks; ++i) {
          const int col = c0 + 64 * i;
          constexpr int kUnits = SUBS * kStatBlocks;
          const bool mine = kUnits == 1 ? group == 0 : ((sub * kStatBlocks + i) & 1) == group;
          if (mine && col < g.nc) {
            uint32_t r[64];
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (acc * SUBS + sub) * BN + (uint32_t)(64 * i);
            tmem_ld_32x32_issue(taddr, r);
            tmem_ld_32x32_issue(taddr + 32, r + 32);
            tmem_ld_wait();
            uint8_t* my_row = buf + lane * 128;
            const bool keep = row_off >= 0;
            if (tma_out) {             // the previous block's store has finished reading the staging buffer
              if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
              __syncwarp();
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {         // 16-byte piece j of this row sits at piece (j ^ (row & 7))
              uint4 q = make_uint4(0u, 0u, 0u, 0u);
              if (keep) {
                q.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                q.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                q.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                q.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
              }
              *reinterpret_cast<uint4*>(my_row + ((j ^ (lane & 7)) << 4)) = q;
            }
            __syncwarp();
            if (tma_out) {
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) tma_store_2d(omap, buf, col, w0 + sub * 128 + quarter * 32);   // rows past the end are clipped
            } else {
              // coalesced stores: 8 lanes write the 128 bytes of one pixel's channel block, 4 pixels per instruction
              const int pc = lane & 7;
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const int rr = 4 * k + (lane >> 3);
                const int off = __shfl_sync(0xffffffffu, row_off, rr);
                const uint4 q = *reinterpret_cast<const uint4*>(buf + rr * 128 + ((pc ^ (rr & 7)) << 4));
                if (off >= 0) *reinterpret_cast<uint4*>(out + ((int64_t)off << 3) + col + pc * 8) = q;
              }
              __syncwarp();
            }
            // (the block's stores are on their way: the sums overlap them)
            if (STATS) {
              // column sums of the rounded block (rows that are not stored hold zeros): this lane owns columns
              // 2 * lane and 2 * lane + 1
#pragma unroll 8
              for (int rr = 0; rr < 32; ++rr) {
                const uint32_t wv = *reinterpret_cast<const uint32_t*>(buf + rr * 128 + (((lane >> 2) ^ (rr & 7)) << 4) +
                                                                       (lane & 3) * 4);
                const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv));
                cs[i][0] += f.x; cs[i][1] = fmaf(f.x, f.x, cs[i][1]); cs[i][2] += f.y; cs[i][3] = fmaf(f.y, f.y, cs[i][3]);
              }
            }
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive(tmem_empty_bar + acc);
  }
  if (STATS) flush_stats();
  if (tma_out) {
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");     // staging buffer free, stores complete
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------------------------------
// forward / data gradient
// ---------------------------------------------------------------------------------------------------------------
template <int BN, bool B_MN, bool STATS>
__global__ void __launch_bounds__(kThreads, 1)
conv_fwd_kernel(const __grid_constant__ ActMaps amaps, const __grid_constant__ CUtensorMap wmap,
                const __grid_constant__ CUtensorMap omap, const __grid_constant__ Geom g, __nv_bfloat16* __restrict__ out,
                float* __restrict__ col_sums, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  using C = FwdCfg<BN>;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* store_bufs = tiles + C::kStages * C::kStageBytes;
  uint64_t* bars = (uint64_t*)(store_bufs + C::kStoreBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* tmem_full_bar = bars + 2 * C::kStages;
  uint64_t* tmem_empty_bar = bars + 2 * C::kStages + 2;
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * C::kStages + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = g.tiles_w * g.tiles_h * g.tiles_n, tiles_nn = (g.nc + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_nn;
  const int kcb = g.kc >> 6;
  const int num_kb = g.n_taps * kcb;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar + a, 1);
      mbar_init(tmem_empty_bar + a, 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&amaps.m[0]) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
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
      uint32_t it = 0;
      bool ok = true;
      const uint32_t tx = (uint32_t)(g.pix * 128 + C::kBBytes);     // a box is written in full, zero fill included
      for (int t = tile_begin(num_tiles, blockIdx.x); t < tile_begin(num_tiles, blockIdx.x + 1) && ok; ++t) {
        int w0, h0, n0, tm, tn;
        split_tile(g, t, tiles_m, tiles_nn, tm, tn);
        tile_origin(g, tm, w0, h0, n0);
        const int c0 = tn * BN;
        for (int tap = 0; tap < g.n_taps && ok; ++tap) {
          const CUtensorMap* am = &amaps.m[g.tap_map[tap]];
          const int xw = w0 + g.tap_dw[tap], xh = h0 + g.tap_dh[tap], wcol = g.tap_col[tap];
          for (int cb = 0; cb < kcb; ++cb, ++it) {
            const int s = it % C::kStages;
            if (it % C::kGroup == 0) {              // first stage of a group: the whole group must have been released
              const uint32_t grp = (it / C::kGroup) % C::kGroups, round = (it / C::kGroup) / C::kGroups;
              if (round > 0 && !mbar_wait_parked(empty_bar + grp, (round - 1) & 1, status, 1, g.wait_ns)) { ok = false; break; }
            }
            uint8_t* a_dst = tiles + s * C::kStageBytes;
            uint8_t* b_dst = a_dst + C::kABytes;
            mbar_expect_tx(full_bar + s, tx);
            tma_load_4d(a_dst, am, full_bar + s, cb * 64, xw, xh, n0);
            if constexpr (!B_MN) {
              tma_load_2d(b_dst, &wmap, full_bar + s, wcol + cb * 64, c0);       // [BN rows (co)][64 (tap, ci)]
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)                                  // [64 rows (co)][64 (tap, ci)] each
                tma_load_2d(b_dst + j * 8192, &wmap, full_bar + s, wcol + c0 + j * 64, cb * 64);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(128, BN, false, B_MN);
      const uint32_t tiles_addr = smem_u32(tiles);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = tile_begin(num_tiles, blockIdx.x); t < tile_begin(num_tiles, blockIdx.x + 1) && ok; ++t, ++lt) {
        const uint32_t acc = lt & 1, use = lt >> 1;
        if (use > 0) {
          ok = mbar_wait(tmem_empty_bar + acc, (use - 1) & 1, status, 4, g.wait_ns);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t d_tmem = tmem_base + acc * BN;
        uint32_t accum = 0u;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % C::kStages;
          const uint32_t round = it / C::kStages;
          ok = mbar_wait(full_bar + s, round & 1, status, 2, g.wait_ns);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = tiles_addr + s * C::kStageBytes;
          const uint32_t a_lo = desc_lo_k_major(a_addr);
          const uint32_t b_lo = B_MN ? desc_lo_mn_major(a_addr + C::kABytes, 8192) : desc_lo_k_major(a_addr + C::kABytes);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {          // 16 along K: +32 bytes in a K-major row, +2048 bytes (16 rows) MN-major
            umma_bf16_lo(d_tmem, a_lo + 2 * kk, b_lo + (B_MN ? 128 * kk : 2 * kk), idesc, accum);
            accum = 1u;
          }
          if (it % C::kGroup == C::kGroup - 1) umma_commit(empty_bar + (it / C::kGroup) % C::kGroups);
        }
        umma_commit(tmem_full_bar + acc);
      }
    }
  } else {
    fwd_epilogue<BN, 1, 2, STATS>(g, num_tiles, tiles_m, 1, tmem_base, tmem_full_bar, tmem_empty_bar, store_bufs, out,
                                  col_sums, status, warp, lane, &omap);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------------
// 3x3, stride 1: forward / data gradient with the bordered pixel box resident in shared memory
// ---------------------------------------------------------------------------------------------------------------
template <int BN>
struct HaloCfg {
  static constexpr int kARows = 384;                          // bordered box: up to 256 accumulator rows + 2 rows + 2
  static constexpr int kABytes = kARows * 128;
  static constexpr int kAStages = 2;
  static constexpr int kBBytes = BN * 128;                    // weights of one tap and one 64-channel block
  static constexpr int kBStages = BN == 64 ? 9 : (BN == 128 ? 6 : 3);
  static constexpr int kBGroup = BN == 256 ? 1 : 3;           // weight stages released per tcgen05.commit
  static constexpr int kBGroups = kBStages / kBGroup;
  static constexpr int kAccBufs = BN == 256 ? 1 : 2;          // TMEM: kAccBufs x 2 accumulators x BN columns <= 512
  static constexpr int kTmemCols = kAccBufs * 2 * BN;
  static constexpr int kStoreBytes = 8 * 32 * 128;
  static constexpr int kSmemBytes = kAStages * kABytes + kBStages * kBBytes + kStoreBytes + 1024 + 512;
};

// The operand of tap (kh, kw) is the bordered box read from row tap_off = kh * pitch + kw on: a start address that is
// not 1024-byte aligned.  The tensor core applies the 128-byte swizzle to the bits of the absolute shared-memory
// address, as TMA did when it wrote the tile, so the shifted start needs nothing beyond its address (the descriptor's
// base-offset field stays 0; setting it to the start's phase gives wrong products - measured).
// One tile = a bordered box of up to 256 accumulator rows (two 128-row accumulators that share every weight tile).
// g.b_resident: all weight tiles of the problem (9 taps, one channel block, one N tile) fit the weight ring; they are
// loaded once and stay.
template <int BN, bool B_MN, bool STATS>
__global__ void __launch_bounds__(kThreads, 1)
conv_halo_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap wmap,
                 const __grid_constant__ Geom g, __nv_bfloat16* __restrict__ out, float* __restrict__ col_sums,
                 int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  using C = HaloCfg<BN>;
  uint8_t* a_tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* b_tiles = a_tiles + C::kAStages * C::kABytes;
  uint8_t* store_bufs = b_tiles + C::kBStages * C::kBBytes;
  uint64_t* bars = (uint64_t*)(store_bufs + C::kStoreBytes);
  uint64_t* a_full = bars;
  uint64_t* a_empty = a_full + C::kAStages;
  uint64_t* b_full = a_empty + C::kAStages;
  uint64_t* b_empty = b_full + C::kBStages;
  uint64_t* tmem_full_bar = b_empty + C::kBStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_slot = (uint32_t*)(tmem_empty_bar + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = g.tiles_w * g.tiles_h * g.tiles_n, tiles_nn = (g.nc + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_nn;
  const int kcb = g.kc >> 6;
  const int n_sub = (g.pix + 127) >> 7;
  const bool resident = g.b_resident != 0;

  // Rows of an A stage past the bordered box are never written by TMA but are read for accumulator rows that are
  // thrown away; they are zeroed once so that those rows stay finite.
  {
    uint4* p = reinterpret_cast<uint4*>(a_tiles);
    for (int i = threadIdx.x; i < C::kAStages * C::kABytes / 16; i += kThreads) p[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kAStages; ++s) { mbar_init(a_full + s, 1); mbar_init(a_empty + s, 1); }
    for (int s = 0; s < C::kBStages; ++s) { mbar_init(b_full + s, 1); mbar_init(b_empty + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tmem_full_bar + a, 1); mbar_init(tmem_empty_bar + a, 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&amap) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
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
  const int t_first = tile_begin(num_tiles, blockIdx.x), my_tiles = tile_begin(num_tiles, blockIdx.x + 1) - t_first;

  if (warp == 0) {
    // ---------------- TMA producer: one bordered box per (tile, channel block), nine weight tiles after it; the box
    // of the NEXT channel block is requested before the weight tiles of the current one ----------------
    if (lane == 0) {
      const int units = my_tiles * kcb;
      uint32_t ib = 0;
      bool ok = true;
      auto load_a = [&](int u) -> bool {
        const int t = t_first + u / kcb, cb = u % kcb;
        int w0, h0, n0, tm, tn;
        split_tile(g, t, tiles_m, tiles_nn, tm, tn);
        tile_origin(g, tm, w0, h0, n0);
        const int s = u % C::kAStages;
        const uint32_t round = (uint32_t)u / C::kAStages;
        if (round > 0 && !mbar_wait_parked(a_empty + s, (round - 1) & 1, status, 1, g.wait_ns)) return false;
        mbar_expect_tx(a_full + s, (uint32_t)g.halo_rows * 128u);
        tma_load_4d(a_tiles + s * C::kABytes, &amap, a_full + s, cb * 64, w0 - 1, h0 - 1, n0);
        return true;
      };
      if (units > 0) ok = load_a(0);
      for (int u = 0; u < units && ok; ++u) {
        if (u + 1 < units && !load_a(u + 1)) { ok = false; break; }
        if (resident && u > 0) continue;
        const int t = t_first + u / kcb, cb = u % kcb;
        int tm, tn;
        split_tile(g, t, tiles_m, tiles_nn, tm, tn);
        const int c0 = tn * BN;
        for (int tap = 0; tap < 9; ++tap, ++ib) {
          const int s = ib % C::kBStages;
          if (ib % C::kBGroup == 0) {
            const uint32_t grp = (ib / C::kBGroup) % C::kBGroups, round = (ib / C::kBGroup) / C::kBGroups;
            if (round > 0 && !mbar_wait_parked(b_empty + grp, (round - 1) & 1, status, 1, g.wait_ns)) { ok = false; break; }
          }
          uint8_t* b_dst = b_tiles + s * C::kBBytes;
          mbar_expect_tx(b_full + s, (uint32_t)C::kBBytes);
          if constexpr (!B_MN) {
            tma_load_2d(b_dst, &wmap, b_full + s, g.tap_col[tap] + cb * 64, c0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * 8192, &wmap, b_full + s, g.tap_col[tap] + c0 + j * 64, cb * 64);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(128, BN, false, B_MN);
      const uint32_t a_addr0 = smem_u32(a_tiles), b_addr0 = smem_u32(b_tiles);
      uint32_t ia = 0, ib = 0;
      bool ok = true;
      for (int lt = 0; lt < my_tiles && ok; ++lt) {
        const uint32_t acc = (uint32_t)lt % C::kAccBufs, use = (uint32_t)lt / C::kAccBufs;
        if (use > 0) {
          ok = mbar_wait(tmem_empty_bar + acc, (use - 1) & 1, status, 4, g.wait_ns);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t d_tmem = tmem_base + acc * 2 * BN;
        uint32_t accum = 0u;
        for (int cb = 0; cb < kcb && ok; ++cb, ++ia) {
          const int sa = ia % C::kAStages;
          ok = mbar_wait(a_full + sa, (ia / C::kAStages) & 1, status, 2, g.wait_ns);
          if (!ok) break;
          const uint32_t a_lo0 = desc_lo_k_major(a_addr0 + sa * C::kABytes);
          for (int tap = 0; tap < 9; ++tap, ++ib) {
            const int sb = resident ? tap : (int)(ib % C::kBStages);
            if (!resident || ia == 0) {
              ok = mbar_wait(b_full + sb, resident ? 0u : ((ib / C::kBStages) & 1), status, 2, g.wait_ns);
              if (!ok) break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t b_addr = b_addr0 + sb * C::kBBytes;
            const uint32_t b_lo = B_MN ? desc_lo_mn_major(b_addr, 8192) : desc_lo_k_major(b_addr);
            const uint32_t a_lo = a_lo0 + 8 * g.tap_off[tap];        // one row = 128 bytes = 8 address units
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_bf16_lo(d_tmem, a_lo + 2 * kk, b_lo + (B_MN ? 128 * kk : 2 * kk), idesc, kk == 0 ? accum : 1u);
            if (n_sub > 1) {
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)                         // second accumulator: 128 rows further on
                umma_bf16_lo(d_tmem + BN, a_lo + 1024 + 2 * kk, b_lo + (B_MN ? 128 * kk : 2 * kk), idesc,
                             kk == 0 ? accum : 1u);
            }
            accum = 1u;
            if (!resident && ib % C::kBGroup == C::kBGroup - 1) umma_commit(b_empty + (ib / C::kBGroup) % C::kBGroups);
          }
          if (ok) umma_commit(a_empty + sa);
        }
        umma_commit(tmem_full_bar + acc);
      }
    }
  } else {
    fwd_epilogue<BN, 2, C::kAccBufs, STATS>(g, num_tiles, tiles_m, n_sub, tmem_base, tmem_full_bar, tmem_empty_bar,
                                            store_bufs, out, col_sums, status, warp, lane);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------------
// weight gradient
// ---------------------------------------------------------------------------------------------------------------
template <int BN>
struct WgCfg {
  static constexpr int kBoxRows = BN == 256 ? 64 : 128;         // pixels per box (the K extent of one stage)
  static constexpr int kBox = kBoxRows * 128;                   // bytes reserved per box
  static constexpr int kABytes = 2 * kBox;                      // two 64-channel boxes of the shifted input (M = 128)
  static constexpr int kBBytes = (BN / 64) * kBox;              // BN / 64 boxes of dY
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = BN == 128 ? 3 : 4;
  static constexpr int kGroup = BN == 128 ? 1 : 2;              // stages released per tcgen05.commit
  static constexpr int kGroups = kStages / kGroup;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

template <int BN>
__global__ void __launch_bounds__(kWgThreads, 1)
conv_wgrad_kernel(const __grid_constant__ ActMaps xmaps, const __grid_constant__ CUtensorMap dymap,
                  const __grid_constant__ Geom g, float* __restrict__ dw, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  using C = WgCfg<BN>;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(tiles + C::kStages * C::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* tmem_full_bar = bars + 2 * C::kStages;
  uint64_t* tmem_empty_bar = bars + 2 * C::kStages + 2;
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * C::kStages + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kcb = g.kc >> 6;
  const int m_blocks = g.n_taps * kcb;                       // 64-wide blocks of the (tap, ci) index
  const int m_tiles = (m_blocks + 1) >> 1, n_tiles = (g.nc + BN - 1) / BN;
  const int boxes = g.tiles_w * g.tiles_h * g.tiles_n;
  const int num_items = m_tiles * n_tiles * g.splits;
  const int ksteps = (g.pix + 15) >> 4;                      // MMAs (K = 16 pixels) per box

  // Rows of a stage buffer beyond the box's pixel count are never written by TMA; the last MMA of a box whose pixel
  // count is not a multiple of 16 reads up to 15 of them.  They are zeroed once here and stay zero.
  {
    uint4* p = reinterpret_cast<uint4*>(tiles);
    const int n16 = C::kStages * C::kStageBytes / 16;
    for (int i = threadIdx.x; i < n16; i += kWgThreads) p[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar + a, 1);
      mbar_init(tmem_empty_bar + a, 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&xmaps.m[0]) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&dymap) : "memory");
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
      uint32_t it = 0;
      bool ok = true;
      const uint32_t tx = (uint32_t)((2 + BN / 64) * g.pix * 128);
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int mt = item % m_tiles, nt = (item / m_tiles) % n_tiles, sp = item / (m_tiles * n_tiles);
        const int b_lo = (int)((int64_t)boxes * sp / g.splits), b_hi = (int)((int64_t)boxes * (sp + 1) / g.splits);
        int mb[2] = {2 * mt, 2 * mt + 1};
        if (mb[1] >= m_blocks) mb[1] = mb[0];                 // odd block count: the last tile's upper half is a copy
        for (int bx = b_lo; bx < b_hi; ++bx, ++it) {
          int w0, h0, n0;
          tile_origin(g, bx, w0, h0, n0);
          const int s = it % C::kStages;
          if (it % C::kGroup == 0) {
            const uint32_t grp = (it / C::kGroup) % C::kGroups, round = (it / C::kGroup) / C::kGroups;
            if (round > 0 && !mbar_wait_parked(empty_bar + grp, (round - 1) & 1, status, 1, g.wait_ns)) { ok = false; break; }
          }
          uint8_t* a_dst = tiles + s * C::kStageBytes;
          uint8_t* b_dst = a_dst + C::kABytes;
          mbar_expect_tx(full_bar + s, tx);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int tap = mb[h] / kcb, cb = mb[h] % kcb;
            tma_load_4d(a_dst + h * C::kBox, &xmaps.m[g.tap_map[tap]], full_bar + s, cb * 64, w0 + g.tap_dw[tap],
                        h0 + g.tap_dh[tap], n0);
          }
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)                    // channel blocks past nc read as zeros
            tma_load_4d(b_dst + j * C::kBox, &dymap, full_bar + s, nt * BN + j * 64, w0, h0, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(128, BN, true, true);
      const uint32_t tiles_addr = smem_u32(tiles);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++lt) {
        const int sp = item / (m_tiles * n_tiles);
        const int b_lo = (int)((int64_t)boxes * sp / g.splits), b_hi = (int)((int64_t)boxes * (sp + 1) / g.splits);
        const uint32_t acc = lt & 1, use = lt >> 1;
        if (use > 0) {
          ok = mbar_wait(tmem_empty_bar + acc, (use - 1) & 1, status, 4, g.wait_ns);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t d_tmem = tmem_base + acc * BN;
        uint32_t accum = 0u;
        for (int bx = b_lo; bx < b_hi; ++bx, ++it) {
          const int s = it % C::kStages;
          const uint32_t round = it / C::kStages;
          ok = mbar_wait(full_bar + s, round & 1, status, 2, g.wait_ns);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = tiles_addr + s * C::kStageBytes;
          const uint32_t a_dlo = desc_lo_mn_major(a_addr, C::kBox), b_dlo = desc_lo_mn_major(a_addr + C::kABytes, C::kBox);
          for (int ks = 0; ks < ksteps; ++ks) {                     // 16 pixels further on: +2048 bytes
            umma_bf16_lo(d_tmem, a_dlo + 128 * ks, b_dlo + 128 * ks, idesc, accum);
            accum = 1u;
          }
          if (it % C::kGroup == C::kGroup - 1) umma_commit(empty_bar + (it / C::kGroup) % C::kGroups);
        }
        umma_commit(tmem_full_bar + acc);
      }
    }
  } else {
    // ---------------- epilogue: add the partial tile into dW[co][(tap, ci)] ----------------
    const int quarter = warp & 3;
    uint32_t lt = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++lt) {
      const int mt = item % m_tiles, nt = (item / m_tiles) % n_tiles, sp = item / (m_tiles * n_tiles);
      const int b_lo = (int)((int64_t)boxes * sp / g.splits), b_hi = (int)((int64_t)boxes * (sp + 1) / g.splits);
      const uint32_t acc = lt & 1, use = lt >> 1;
      ok = mbar_wait_warp(tmem_full_bar + acc, use & 1, status, 3, g.wait_ns, lane);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int m = mt * 128 + quarter * 32 + lane;             // index into the (tap, ci) axis
      const bool row_ok = m < m_blocks * 64 && b_hi > b_lo;     // (an empty pixel range leaves the accumulator unset)
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int co0 = nt * BN + c0;
        if (co0 >= g.nc) break;
        uint32_t r[32];
        tmem_ld_32x32_issue(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + (uint32_t)c0, r);
        tmem_ld_wait();
        if (row_ok) {
          float* dst = dw + (int64_t)co0 * g.ldw + m;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (co0 + j < g.nc) atomicAdd(dst + (int64_t)j * g.ldw, __uint_as_float(r[j]));
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar + acc);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols)
                 : "memory");
  }
}

// One barrier that nothing ever completes, waited on with the same bounded wait the kernels above use: the wait gives
// up after `limit_ns`, leaves `code` in *status and the kernel returns normally.
__global__ void bounded_wait_probe_kernel(unsigned long long limit_ns, int code, int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait(&bar, 0, status, code, limit_ns);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
unsigned long long g_wait_ns = 2000000000ull;     // give-up time of the kernels' mbarrier waits (2 s)

}  // namespace
extern int g_tsp_sm_reserve;          // defined in peer.cu
namespace {

int sm_count() {
  static int n_sm[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (n_sm[dev] == 0) {
    cudaDeviceGetAttribute(&n_sm[dev], cudaDevAttrMultiProcessorCount, dev);
    if (n_sm[dev] <= 0) n_sm[dev] = 148;
  }
  const int n = n_sm[dev] - g_tsp_sm_reserve;       // SMs left to communication kernels stay free
  return n > 8 ? n : 8;
}

// Pixel box for a w x h x n grid: at most max_pix pixels, as few tiles as possible, tiles of equal size where it
// divides.
void choose_box(int w, int h, int n, int max_pix, int& bw, int& bh, int& bn) {
  bw = w < max_pix ? w : max_pix;
  const int hmax = max_pix / bw;
  bh = 1;
  if (hmax > 1) {
    const int th = (h + hmax - 1) / hmax;           // tiles along h
    bh = (h + th - 1) / th;
  }
  const int nmax = max_pix / (bw * bh);
  bn = 1;
  if (nmax > 1 && bh >= h) {
    const int tn = (n + nmax - 1) / nmax;
    bn = (n + tn - 1) / tn;
  }
}

// Tensor map of a dense channels-last view: base + (c, w, h, n) with pitches pw / ph / pn ELEMENTS, box as given.
bool act_map(CUtensorMap* map, const void* base, int c, int w, int h, int n, int64_t pw, int64_t ph, int64_t pn, int bw,
             int bh, int bn) {
  const uint64_t dims[4] = {(uint64_t)c, (uint64_t)w, (uint64_t)h, (uint64_t)n};
  const uint64_t strides[4] = {2, (uint64_t)pw * 2, (uint64_t)ph * 2, (uint64_t)pn * 2};
  const uint32_t box[4] = {64, (uint32_t)bw, (uint32_t)bh, (uint32_t)bn};
  return make_bf16_map(map, base, 4, dims, strides, box);
}

// A convolution problem seen from its OUTPUT pixel grid: where the shifted input boxes come from.
struct Plan {
  Geom g;
  ActMaps maps;
  bool ok;
};

// Shifted-input side of the forward product (and of the weight gradient): input x [n, h, w, cin], kernel k, stride s.
// `flat` = 1x1 stride 1: all pixels as one row of n*h*w.
Plan plan_input(const void* x, int n, int h, int w, int cin, int k, int s, int max_pix = 128) {
  Plan p = {};
  Geom& g = p.g;
  const int pad = (k - 1) / 2;
  const bool flat = k == 1 && s == 1;
  const int ho = (h + 2 * pad - k) / s + 1, wo = (w + 2 * pad - k) / s + 1;
  if (flat) {
    g.out_w = n * h * w; g.out_h = 1; g.out_n = 1;
  } else {
    g.out_w = wo; g.out_h = ho; g.out_n = n;
  }
  choose_box(g.out_w, g.out_h, g.out_n, max_pix, g.box_w, g.box_h, g.box_n);
  g.tiles_w = (g.out_w + g.box_w - 1) / g.box_w;
  g.tiles_h = (g.out_h + g.box_h - 1) / g.box_h;
  g.tiles_n = (g.out_n + g.box_n - 1) / g.box_n;
  g.row_pitch = g.box_w;
  g.pix = g.box_w * g.box_h * g.box_n;
  g.wait_ns = g_wait_ns;
  g.n_taps = k * k;
  g.kc = cin;
  p.ok = true;
  if (flat) {
    p.ok = act_map(&p.maps.m[0], x, cin, g.out_w, 1, 1, cin, (int64_t)cin * g.out_w, (int64_t)cin * g.out_w, g.box_w, 1, 1);
    for (int i = 1; i < 4; ++i) p.maps.m[i] = p.maps.m[0];
    g.tap_dw[0] = g.tap_dh[0] = g.tap_map[0] = g.tap_col[0] = 0;
    return p;
  }
  if (s == 1) {
    p.ok = act_map(&p.maps.m[0], x, cin, w, h, n, cin, (int64_t)w * cin, (int64_t)h * w * cin, g.box_w, g.box_h, g.box_n);
    for (int i = 1; i < 4; ++i) p.maps.m[i] = p.maps.m[0];
  } else {
    // one dense view per (row parity, column parity): x[n, 2a + ph, 2b + pw, :]
    for (int ph = 0; ph < 2 && p.ok; ++ph)
      for (int pw = 0; pw < 2 && p.ok; ++pw) {
        const __nv_bfloat16* base = (const __nv_bfloat16*)x + ((int64_t)ph * w + pw) * cin;
        p.ok = act_map(&p.maps.m[ph * 2 + pw], base, cin, w / 2, h / 2, n, 2 * (int64_t)cin, 2 * (int64_t)w * cin,
                       (int64_t)h * w * cin, g.box_w, g.box_h, g.box_n);
      }
  }
  for (int kh = 0; kh < k; ++kh)
    for (int kw = 0; kw < k; ++kw) {
      const int t = kh * k + kw;
      const int dh = kh - pad, dw_ = kw - pad;            // input row = s * ho + dh
      if (s == 1) {
        g.tap_dh[t] = dh; g.tap_dw[t] = dw_; g.tap_map[t] = 0;
      } else {
        const int ph = dh & 1, pw = dw_ & 1;              // parity of the input row / column (two's complement: -1 -> 1)
        g.tap_dh[t] = (dh - ph) / 2; g.tap_dw[t] = (dw_ - pw) / 2; g.tap_map[t] = ph * 2 + pw;
      }
      g.tap_col[t] = t * cin;
    }
  return p;
}

template <int BN, bool B_MN, bool STATS>
int launch_fwd(const Plan& p, const CUtensorMap& wmap, void* out, float* col_sums, int* status, cudaStream_t stream) {
  auto kern = conv_fwd_kernel<BN, B_MN, STATS>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  Geom g = p.g;
  const int num_tiles = g.tiles_w * g.tiles_h * g.tiles_n * ((g.nc + BN - 1) / BN);
  const int n_sm = sm_count();
  const int grid = num_tiles < n_sm ? num_tiles : n_sm;
  // flat pixel grid (1x1 stride 1, dense output rows): [pixels, nc] matrix written in 32-row x 64-channel TMA stores
  CUtensorMap omap = wmap;
  g.tma_store = 0;
  g.n_fastest = STATS ? 0 : 1;
  if (g.out_h == 1 && g.out_n == 1 && g.out_sw * 8 == g.nc && g.box_w == 128) {
    const uint64_t dims[2] = {(uint64_t)g.nc, (uint64_t)g.out_w};
    const uint64_t strides[2] = {2, (uint64_t)g.nc * 2};
    const uint32_t box[2] = {64, 32};
    if (make_bf16_map(&omap, out, 2, dims, strides, box)) g.tma_store = 1;
  }
  kern<<<grid, kThreads, FwdCfg<BN>::kSmemBytes, stream>>>(p.maps, wmap, omap, g, (__nv_bfloat16*)out, col_sums, status);
  return TSP_LAUNCH_CHECK();
}

template <bool B_MN, bool STATS>
int dispatch_fwd(int bn, const Plan& p, const CUtensorMap& wmap, void* out, float* col_sums, int* status,
                 cudaStream_t stream) {
  if (bn == 256) return launch_fwd<256, B_MN, STATS>(p, wmap, out, col_sums, status, stream);
  if (bn == 128) return launch_fwd<128, B_MN, STATS>(p, wmap, out, col_sums, status, stream);
  return launch_fwd<64, B_MN, STATS>(p, wmap, out, col_sums, status, stream);
}

// 3x3 stride-1 walk over an image grid with the bordered box kept in shared memory (conv_halo_kernel): applies when
// a bordered row fits (w <= 61) and the image is large enough that one box per image does not waste the tile.
bool halo_applies(int k, int s, int w, int h) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("TSP_CONV_HALO");
    enabled = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return enabled && k == 3 && s == 1 && w <= 61 && h * (w + 2) > 64;
}

// Geometry of the halo kernel over src[n, h, w, c] (the forward's input, or dy for the data gradient).
bool plan_halo(Geom& g, CUtensorMap* amap, const void* src, int n, int h, int w, int c) {
  g = Geom{};
  const int pitch = w + 2, hmax = 256 / pitch;        // up to 256 accumulator rows (two accumulators) per tile
  const int th = (h + hmax - 1) / hmax;
  g.out_w = w; g.out_h = h; g.out_n = n;
  g.box_w = w; g.box_h = (h + th - 1) / th; g.box_n = 1;
  g.tiles_w = 1; g.tiles_h = th; g.tiles_n = n;
  g.row_pitch = pitch;
  g.pix = pitch * g.box_h;
  g.halo_rows = pitch * (g.box_h + 2);
  g.n_taps = 9;
  g.kc = c;
  g.rows_per_seg = 1 << 30;
  g.wait_ns = g_wait_ns;
  return act_map(amap, src, c, w, h, n, c, (int64_t)w * c, (int64_t)h * w * c, pitch, g.box_h + 2, 1);
}

template <int BN, bool B_MN, bool STATS>
int launch_halo(Geom& g, const CUtensorMap& amap, const CUtensorMap& wmap, void* out, float* col_sums, int* status,
                cudaStream_t stream) {
  g.n_fastest = STATS ? 0 : 1;
  auto kern = conv_halo_kernel<BN, B_MN, STATS>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, HaloCfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  const int num_tiles = g.tiles_w * g.tiles_h * g.tiles_n * ((g.nc + BN - 1) / BN);
  const int n_sm = sm_count();
  const int grid = num_tiles < n_sm ? num_tiles : n_sm;
  kern<<<grid, kThreads, HaloCfg<BN>::kSmemBytes, stream>>>(amap, wmap, g, (__nv_bfloat16*)out, col_sums, status);
  return TSP_LAUNCH_CHECK();
}

template <bool B_MN, bool STATS>
int dispatch_halo(int bn, Geom& g, const CUtensorMap& amap, const CUtensorMap& wmap, void* out, float* col_sums,
                  int* status, cudaStream_t stream) {
  g.b_resident = (bn == 64 && g.kc == 64 && g.nc == 64) ? 1 : 0;      // 9 weight tiles = the 9 ring slots
  if (bn == 256) return launch_halo<256, B_MN, STATS>(g, amap, wmap, out, col_sums, status, stream);
  if (bn == 128) return launch_halo<128, B_MN, STATS>(g, amap, wmap, out, col_sums, status, stream);
  return launch_halo<64, B_MN, STATS>(g, amap, wmap, out, col_sums, status, stream);
}

int pick_bn(int nc) { return nc % 256 == 0 ? 256 : (nc % 128 == 0 ? 128 : 64); }

template <int BN>
int launch_wgrad(const Plan& p, const CUtensorMap& dymap, float* dw, int* status, cudaStream_t stream) {
  auto kern = conv_wgrad_kernel<BN>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WgCfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  const Geom& g = p.g;
  const int m_tiles = (g.n_taps * (g.kc / 64) + 1) / 2, n_tiles = (g.nc + BN - 1) / BN;
  const int items = m_tiles * n_tiles * g.splits;
  const int n_sm = sm_count();
  const int grid = items < n_sm ? items : n_sm;
  kern<<<grid, kWgThreads, WgCfg<BN>::kSmemBytes, stream>>>(p.maps, dymap, g, dw, status);
  return TSP_LAUNCH_CHECK();
}

bool shape_ok(int n, int h, int w, int cin, int cout, int k, int s) {
  if (n <= 0 || h <= 0 || w <= 0) return false;
  if (cin % 64 || cout % 64 || cin <= 0 || cout <= 0) return false;
  if (!(k == 1 || k == 3) || !(s == 1 || s == 2)) return false;
  if (s == 2 && ((h | w) & 1)) return false;
  return true;
}

}  // namespace

extern "C" {

// Give-up time (milliseconds, default 2000) of every mbarrier wait in the kernels of this file launched afterwards.
void tsp_conv_set_wait_limit_ms(int ms) { g_wait_ns = (unsigned long long)(ms > 0 ? ms : 1) * 1000000ull; }

// Failure-detection self-test: runs the kernels' bounded mbarrier wait on a barrier that is never completed.  After
// about `limit_ms` milliseconds the wait gives up, *status (one zeroed int in device memory) becomes `code`, and the
// kernel ends normally: nothing traps, the context stays usable.
int tsp_bounded_wait_probe(int limit_ms, int code, int* status, cudaStream_t stream) {
  if (limit_ms < 1 || limit_ms > 2000) return -3;
  bounded_wait_probe_kernel<<<1, 32, 0, stream>>>((unsigned long long)limit_ms * 1000000ull, code, status);
  return TSP_LAUNCH_CHECK();
}

// y[n, ho, wo, cout] = conv(x[n, h, w, cin], wgt[cout][k][k][cin]), stride s, padding (k - 1) / 2; all bf16,
// channels-last, 16-byte aligned, cin and cout multiples of 64.  col_sums (optional, zeroed by the caller):
// [segs][2 * cout] fp32 receives per-channel sum and sum of squares of y over each of `segs` equal groups of
// consecutive images (n divisible by segs; for a 1x1 stride-1 convolution the pixels per group must be a multiple of
// 128).  `status`: one zeroed int in device memory; non-zero afterwards = a bounded wait ran out, y is not valid.
int tsp_conv_fprop(const void* x, const void* wgt, void* y, float* col_sums, int segs, int n, int h, int w, int cin,
                   int cout, int k, int s, int* status, cudaStream_t stream) {
  if (!shape_ok(n, h, w, cin, cout, k, s)) return -3;
  if (((uintptr_t)x | (uintptr_t)wgt | (uintptr_t)y) & 15) return -2;
  const int pad = (k - 1) / 2, ho = (h + 2 * pad - k) / s + 1, wo = (w + 2 * pad - k) / s + 1;
  if ((int64_t)n * ho * wo * cout / 8 >= (int64_t)1 << 31) return -3;
  if (halo_applies(k, s, w, h)) {
    Geom g;
    CUtensorMap amap, wmap;
    if (!plan_halo(g, &amap, x, n, h, w, cin)) return -6;
    g.nc = cout;
    for (int t = 0; t < 9; ++t) { g.tap_off[t] = (t / 3) * g.row_pitch + t % 3; g.tap_col[t] = t * cin; }
    g.out_sw = cout / 8; g.out_sh = w * (cout / 8); g.out_sn = h * w * (cout / 8);
    if (col_sums != nullptr) {
      if (segs < 1 || n % segs) return -3;
      g.rows_per_seg = (int)((int64_t)n * h * w / segs);
    }
    const int bn = pick_bn(cout);
    const uint64_t dims[2] = {(uint64_t)9 * cin, (uint64_t)cout};
    const uint64_t strides[2] = {2, (uint64_t)9 * cin * 2};
    const uint32_t box[2] = {64, (uint32_t)bn};
    if (!make_bf16_map(&wmap, wgt, 2, dims, strides, box)) return -6;
    if (col_sums != nullptr) return dispatch_halo<false, true>(bn, g, amap, wmap, y, col_sums, status, stream);
    return dispatch_halo<false, false>(bn, g, amap, wmap, y, nullptr, status, stream);
  }
  Plan p = plan_input(x, n, h, w, cin, k, s);
  if (!p.ok) return -6;
  Geom& g = p.g;
  g.nc = cout;
  const bool flat = k == 1 && s == 1;
  g.out_sw = cout / 8;
  g.out_sh = flat ? 0 : wo * (cout / 8);
  g.out_sn = flat ? 0 : ho * wo * (cout / 8);
  g.rows_per_seg = 1 << 30;
  if (col_sums != nullptr) {
    if (segs < 1 || n % segs) return -3;
    const int64_t rows = (int64_t)n * ho * wo / segs;
    if (flat && rows % 128) return -3;
    if (!flat && g.box_n > 1 && (n / segs) % g.box_n) return -3;
    g.rows_per_seg = (int)rows;
  }
  const int bn = pick_bn(cout);
  CUtensorMap wmap;
  const uint64_t dims[2] = {(uint64_t)k * k * cin, (uint64_t)cout};
  const uint64_t strides[2] = {2, (uint64_t)k * k * cin * 2};
  const uint32_t box[2] = {64, (uint32_t)bn};
  if (!make_bf16_map(&wmap, wgt, 2, dims, strides, box)) return -6;
  if (col_sums != nullptr) return dispatch_fwd<false, true>(bn, p, wmap, y, col_sums, status, stream);
  return dispatch_fwd<false, false>(bn, p, wmap, y, nullptr, status, stream);
}

// dx[n, h, w, cin] = gradient of tsp_conv_fprop's input given dy[n, ho, wo, cout] and the same weights
// wgt[cout][k][k][cin] (read in place through MN-major operand tiles).  Every element of dx is written.
int tsp_conv_dgrad(const void* dy, const void* wgt, void* dx, int n, int h, int w, int cin, int cout, int k, int s,
                   int* status, cudaStream_t stream) {
  if (!shape_ok(n, h, w, cin, cout, k, s)) return -3;
  if (((uintptr_t)dy | (uintptr_t)wgt | (uintptr_t)dx) & 15) return -2;
  const int pad = (k - 1) / 2, ho = (h + 2 * pad - k) / s + 1, wo = (w + 2 * pad - k) / s + 1;
  if ((int64_t)n * h * w * cin / 8 >= (int64_t)1 << 31) return -3;
  const int bn = pick_bn(cin);
  CUtensorMap wmap;                       // rows = co (contraction), columns = (tap, ci): boxes of 64 x 64
  const uint64_t dims[2] = {(uint64_t)k * k * cin, (uint64_t)cout};
  const uint64_t strides[2] = {2, (uint64_t)k * k * cin * 2};
  const uint32_t box[2] = {64, 64};
  if (!make_bf16_map(&wmap, wgt, 2, dims, strides, box)) return -6;
  if (halo_applies(k, s, wo, ho)) {
    Geom g;
    CUtensorMap amap;
    if (!plan_halo(g, &amap, dy, n, ho, wo, cout)) return -6;
    g.nc = cin;
    for (int t = 0; t < 9; ++t) {              // dx[p] takes tap (kh, kw) from dy[p + (1 - kh, 1 - kw)]
      g.tap_off[t] = (2 - t / 3) * g.row_pitch + (2 - t % 3);
      g.tap_col[t] = t * cin;
    }
    g.out_sw = cin / 8; g.out_sh = w * (cin / 8); g.out_sn = h * w * (cin / 8);
    return dispatch_halo<true, false>(bn, g, amap, wmap, dx, nullptr, status, stream);
  }
  if (s == 1) {
    // dx[p] = sum_tap dy[p + (pad - kh, pad - kw)] w[:, kh, kw, :]: the forward kernel over dy with mirrored offsets
    Plan p = plan_input(dy, n, ho, wo, cout, k, 1);
    if (!p.ok) return -6;
    Geom& g = p.g;
    g.nc = cin;
    for (int kh = 0; kh < k; ++kh)
      for (int kw = 0; kw < k; ++kw) {
        const int t = kh * k + kw;
        g.tap_dh[t] = pad - kh; g.tap_dw[t] = pad - kw; g.tap_map[t] = 0; g.tap_col[t] = t * cin;
      }
    const bool flat = k == 1;
    g.out_sw = cin / 8;
    g.out_sh = flat ? 0 : w * (cin / 8);
    g.out_sn = flat ? 0 : h * w * (cin / 8);
    g.rows_per_seg = 1 << 30;
    return dispatch_fwd<true, false>(bn, p, wmap, dx, nullptr, status, stream);
  }
  // stride 2: dx[n, 2a + ph, 2b + pw] gets the taps with kh = ph + pad (mod 2), from dy[a + (ph + pad - kh) / 2, ...].
  // One launch per parity class over the (h / 2) x (w / 2) grid of that class; a class no tap reaches is zero
  // (1x1 stride 2: only the even / even class receives anything).
  if (k == 1) {
    cudaError_t e = cudaMemsetAsync(dx, 0, (size_t)n * h * w * cin * 2, stream);
    if (e != cudaSuccess) return (int)e;
  }
  for (int ph = 0; ph < 2; ++ph)
    for (int pw = 0; pw < 2; ++pw) {
      Plan p = plan_input(dy, n, ho, wo, cout, 3, 1);       // geometry of a dense walk over dy's grid (taps set below)
      if (!p.ok) return -6;
      Geom& g = p.g;
      g.nc = cin;
      int nt = 0;
      for (int kh = 0; kh < k; ++kh)
        for (int kw = 0; kw < k; ++kw) {
          if (((ph + pad - kh) & 1) || ((pw + pad - kw) & 1)) continue;
          g.tap_dh[nt] = (ph + pad - kh) / 2; g.tap_dw[nt] = (pw + pad - kw) / 2; g.tap_map[nt] = 0;
          g.tap_col[nt] = (kh * k + kw) * cin;
          ++nt;
        }
      g.n_taps = nt;
      __nv_bfloat16* base = (__nv_bfloat16*)dx + ((int64_t)ph * w + pw) * cin;
      if (nt == 0) continue;                                 // zero, written by the memset above
      g.out_sw = 2 * cin / 8;
      g.out_sh = 2 * w * (cin / 8);
      g.out_sn = h * w * (cin / 8);
      g.rows_per_seg = 1 << 30;
      const int rc = dispatch_fwd<true, false>(bn, p, wmap, base, nullptr, status, stream);
      if (rc != 0) return rc;
    }
  return 0;
}

// dw[cout][k][k][cin] (fp32) += gradient of tsp_conv_fprop's weights given its input x and dy.  The caller zeroes dw
// (or keeps a running sum in it: micro-batches accumulate).
int tsp_conv_wgrad(const void* x, const void* dy, float* dw, int n, int h, int w, int cin, int cout, int k, int s,
                   int* status, cudaStream_t stream) {
  if (!shape_ok(n, h, w, cin, cout, k, s)) return -3;
  if (((uintptr_t)x | (uintptr_t)dy) & 15) return -2;
  const int bn = cout % 256 == 0 ? 256 : (cout % 128 == 0 ? 128 : 64);
  Plan p = plan_input(x, n, h, w, cin, k, s, bn == 256 ? 64 : 128);
  if (!p.ok) return -6;
  Geom& g = p.g;
  const int pad = (k - 1) / 2, ho = (h + 2 * pad - k) / s + 1, wo = (w + 2 * pad - k) / s + 1;
  g.nc = cout;
  g.ldw = k * k * cin;
  const bool flat = k == 1 && s == 1;
  CUtensorMap dymap;
  const bool ok = flat ? act_map(&dymap, dy, cout, g.out_w, 1, 1, cout, (int64_t)cout * g.out_w, (int64_t)cout * g.out_w,
                                 g.box_w, 1, 1)
                       : act_map(&dymap, dy, cout, wo, ho, n, cout, (int64_t)wo * cout, (int64_t)ho * wo * cout, g.box_w,
                                 g.box_h, g.box_n);
  if (!ok) return -6;
  // Work items = output tiles x pieces of the pixel range; about two items per SM and never a handful more than a
  // multiple of the SM count (those would cost a whole extra round).
  const int m_tiles = (g.n_taps * (cin / 64) + 1) / 2, n_tiles = (cout + bn - 1) / bn;
  const int tiles = m_tiles * n_tiles, boxes = g.tiles_w * g.tiles_h * g.tiles_n;
  int splits = 2 * sm_count() / tiles;
  if (splits > boxes) splits = boxes;
  if (splits < 1) splits = 1;
  g.splits = splits;
  if (bn == 256) return launch_wgrad<256>(p, dymap, dw, status, stream);
  if (bn == 128) return launch_wgrad<128>(p, dymap, dw, status, stream);
  return launch_wgrad<64>(p, dymap, dw, status, stream);
}

}  // extern "C"
