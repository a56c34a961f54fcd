// Second-generation tensor-core kernel of the deformable-convolution forward (16-bit
// operands: bf16 or fp16) for sm_100a.
//
// Same contraction as dcn_fwd_tc (out[p, co] = sum_k A[p, k] * Wt[co, k], A never written to
// global memory; it replaces the gather kernel, the per-sample GEMM loop and the bias pass of
// mmcv/ops/csrc/common/cuda/modulated_deform_conv_cuda_kernel.cuh:186-245 and
// mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:108-137), with the producer side split into
// two decoupled roles:
//
//   * table builders (2 warps; a warp takes every other (tap, deform group) block of 128
//     entries, four rows per thread, all loads of a block in flight together) turn offsets and
//     masks into tap-table entries -- four 16-bit corner weights with the modulation folded
//     in, and the byte offset of the top-left corner -- and publish them through a ring of
//     table segments in shared memory.  They run ahead of the gather, which therefore never
//     waits for an offset or a mask.
//   * gather warps (16) read an entry, fetch the four corners, blend them on packed 16-bit
//     FMAs and write the 128-byte-swizzled operand tile tcgen05.mma reads.  The input is a
//     channels-last copy with a one-pixel zero border around every sample: a corner outside
//     the image reads zeros, a sample outside the sampling gate points at an all-zero
//     neighbourhood with zero weights, so the loads carry no predicates and a corner inside
//     the image is always read (0 * Inf = NaN as in the reference,
//     modulated_deform_conv_cuda_kernel.cuh:100-107).  Two rows per thread are in flight and
//     the rotation runs across k-stage boundaries.
//   * K is walked in units of (32-channel half-chunk, tap); a k-stage is two consecutive units.
//     The 32-channel slice of the tile's input neighbourhood (its undeformed footprint plus a
//     margin) is brought into shared memory by one tensor-map copy (cp.async.bulk.tensor, zero
//     fill outside the tensor) per half-chunk, double-buffered; entries whose 2x2 neighbourhood
//     lies inside that window are read from shared memory (64 bytes per pixel; the two units of
//     a row read their left/right corners in opposite order when needed, so that the eight
//     lanes of a row never meet in a bank), the others from global memory, through the same
//     generic loads.
//
// MMA issue, weight loader (cp.async.bulk + mbarrier complete_tx) and the accumulator
// double-buffering in tensor memory are as in dcn_fwd_tc.  Every mbarrier wait is bounded.
#include <atomic>
#include <climits>
#include <cstring>

#include <cuda.h>

#include "dcn_internal.cuh"
#include "dcn_ptx.cuh"

namespace dcn {

namespace {

constexpr int kEpiWarps = 4;
constexpr int kMmaWarp2 = 4;
constexpr int kLoadWarp2 = 5;
constexpr int kFirstBuildWarp = 6;
constexpr int kBuildWarps = 2;
constexpr int kFirstGatherWarp = kFirstBuildWarp + kBuildWarps;
constexpr int kGatherWarps = 16;
constexpr int kThreads2 = (kFirstGatherWarp + kGatherWarps) * 32;  // 768: six warps per scheduler, 80 registers per thread
constexpr int kPasses2 = (kBM * 8) / (kGatherWarps * 32);          // rows of a stage per gather thread
constexpr int kRowsPerPass = kGatherWarps * 4;
constexpr int kTabStride2 = kBM + 4;  // entries of one (tap, deform group) block, skewed
constexpr uint32_t kWinFlag = 0x80000000u;  // table entry: the neighbourhood is read from global memory

struct alignas(64) Tc2Args {
  CUtensorMap win_map;       // padded channels-last input as a 4-D tensor (window copies)
  CUtensorMap out_map;       // output as a 4-D tensor (epilogue stores through the copy engine)
  Geom g;
  TcPlan tp;
  const void *xpad;          // channels-last input with a zero border, [N][H+2][W+2][C] + one zero row
  const uint8_t *wtiles;     // pre-swizzled weight stages
  const void *offset, *mask, *bias;
  void *output;
  int *status;
  unsigned long long *counters;  // optional phase timers (block 0 only), or nullptr
  unsigned long long wait_limit_ns;
  int debug_flags;
};

// Non-blocking test of a barrier phase (mbar_try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// 16-byte loads.  `tok` is passed through untouched; code that must come after a load's issue
// takes `tok` as an input.
__device__ __forceinline__ uint4 ld16_global(const void *p, uint32_t &tok) {
  uint4 r;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p), "r"(tok));
  asm volatile("" : "+r"(tok));
  return r;
}
__device__ __forceinline__ uint4 lds16(uint32_t addr, uint32_t &tok) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "r"(addr), "r"(tok));
  asm volatile("" : "+r"(tok));
  return r;
}
// One lane reads global memory, another the shared-memory window: the same 16-byte load, in
// the lane's own state space.
__device__ __forceinline__ uint4 ld16_either(bool from_global, const void *gp, uint32_t sp, uint32_t &tok) {
  uint4 r;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.u32 p, %6, 0;\n\t"
      "@p ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];\n\t"
      "@!p ld.shared.v4.u32 {%0, %1, %2, %3}, [%5];\n\t}"
      : "=&r"(r.x), "=&r"(r.y), "=&r"(r.z), "=&r"(r.w)
      : "l"(gp), "r"(sp), "r"((uint32_t)from_global), "r"(tok));
  asm volatile("" : "+r"(tok));
  return r;
}
__device__ __forceinline__ void sts16(uint32_t addr, const uint4 &v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}


// Shared memory: a 1 KiB control block first (barriers, tensor-memory slot, abort flag, the
// wait limit and the status pointer: at fixed offsets, so that the out-of-line slow path of a
// wait finds them without arguments), then the rings.
constexpr uint32_t kCtrlBytes = 1024;
constexpr uint32_t kCtrlTmemSlot = 512, kCtrlAbort = 520, kCtrlLimit = 528, kCtrlStatus = 536;

struct Smem2 {
  uint8_t *a, *b, *win;
  uint8_t *epi;        // staging of the epilogue's tensor stores
  uint8_t *tab_w;      // four 16-bit corner weights per entry (8 bytes)
  uint8_t *tab_off;    // byte offset of the top-left corner (bit 31: from global memory)
  uint8_t *bias_s;
};

__host__ __device__ inline size_t win_bytes(const TcPlan &tp) { return (size_t)tp.win_h * tp.win_w * 64; }  // 32 channels per pixel
__host__ __device__ inline size_t epi_bytes(const TcPlan &tp) {
  return tp.epi_tma ? (size_t)kEpiWarps * 2 * 32 * 32 * tp.io_bytes : 0;  // per warp: two slabs of 32 channels x 32 pixels
}

__device__ __forceinline__ uint8_t *smem_aligned() {
  extern __shared__ uint8_t smem_raw[];
  return (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
}

__device__ __forceinline__ Smem2 carve2(uint8_t *base, const TcPlan &tp) {
  Smem2 L;
  uint8_t *p = base + kCtrlBytes;
  L.a = p; p += (size_t)tp.a_stages * kTileBytes;
  L.b = p; p += (size_t)tp.b_stages * tp.BN * 128;
  L.win = p; p += 2 * win_bytes(tp);
  L.epi = p; p += epi_bytes(tp);
  const size_t ents = (size_t)tp.tab_slots * tp.tab_slot_blocks * kTabStride2;
  L.tab_w = p; p += ents * 8;
  L.tab_off = p; p += ents * 4;
  L.bias_s = (uint8_t *)(((uintptr_t)p + 15) & ~(uintptr_t)15);
  return L;
}

// Out-of-line continuation of a wait: polls until the phase completes, the block aborts or the
// time limit passes (then it raises the abort flag and records `code` in the status word).
__device__ __noinline__ bool mbar_wait_slow2(uint32_t bar, uint32_t parity, int code, int backoff) {
  uint8_t *ctrl = smem_aligned();
  volatile int *abort_s = (volatile int *)(ctrl + kCtrlAbort);
  const unsigned long long limit = *(const unsigned long long *)(ctrl + kCtrlLimit);
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (backoff) __nanosleep(200);
    if ((it & 15u) == 0u) {
      if (*abort_s) return false;
      if (globaltimer_ns() - t0 > limit) {
        *abort_s = 1;
        atomicCAS(*(int **)(ctrl + kCtrlStatus), 0, code);
        return false;
      }
    }
  }
}
// Bounded wait.  Returns false when the block is aborting.
__device__ __forceinline__ bool mbar_wait2(uint32_t bar, uint32_t parity, int code, int backoff = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow2(bar, parity, code, backoff);
}

__device__ __forceinline__ uint2 lds8(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds4(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts8(uint32_t addr, uint32_t x, uint32_t y) {
  asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void sts4(uint32_t addr, uint32_t x) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(x) : "memory");
}

struct TileId2 {
  int n, ho0, wo0, grp, nt;
};
__device__ __forceinline__ TileId2 decode_item2(uint32_t item, const Geom &g, const TcPlan &tp) {
  const uint32_t per_mt = (uint32_t)(g.groups * tp.NT);
  const uint32_t mt = item / per_mt;
  const uint32_t rem = item - mt * per_mt;
  const uint32_t tiles_img = (uint32_t)(tp.tiles_x * tp.tiles_y);
  TileId2 t;
  t.n = (int)(mt / tiles_img);
  const uint32_t ti = mt - (uint32_t)t.n * tiles_img;
  const uint32_t ty = ti / (uint32_t)tp.tiles_x;
  t.ho0 = (int)ty * (kBM >> tp.tw_log2);
  t.wo0 = (int)(ti - ty * (uint32_t)tp.tiles_x) << tp.tw_log2;
  t.grp = (int)(rem / (uint32_t)tp.NT);
  t.nt = (int)rem - t.grp * tp.NT;
  return t;
}

// First input row / column of the window of the tile at (ho0, wo0), in image coordinates.
__device__ __forceinline__ int win_y0(const Geom &g, const TcPlan &tp, int ho0) {
  return ho0 * g.stride_h - g.pad_h - tp.win_my;
}
__device__ __forceinline__ int win_x0(const Geom &g, const TcPlan &tp, int wo0) {
  return wo0 * g.stride_w - g.pad_w - tp.win_mx;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, int c0, int c1,
                                            int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, uint32_t src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

template <int MODE>
__device__ __forceinline__ uint32_t pack_weights2(float a, float b) {
  if constexpr (MODE == kModeBf16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
  } else {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
  }
}

}  // namespace

size_t tc2_smem_bytes(const TcPlan &tp) {
  size_t s = 1024 + kCtrlBytes;  // slack for manual 1024-byte alignment, control block
  s += (size_t)tp.a_stages * kTileBytes + (size_t)tp.b_stages * tp.BN * 128;
  s += 2 * win_bytes(tp) + epi_bytes(tp);
  s += (size_t)tp.tab_slots * tp.tab_slot_blocks * kTabStride2 * 12;
  s += (size_t)2 * tp.BN * tp.io_bytes + 32;  // bias staging, one copy per accumulator buffer
  return s;
}

template <typename TIO, int MODE, bool kWin, bool kSegStage>
__global__ void __launch_bounds__(kThreads2, 1) dcn_fwd_tc2(const __grid_constant__ Tc2Args a) {
  uint8_t *smem = smem_aligned();
  const Geom &g = a.g;
  const TcPlan &tp = a.tp;
  const Smem2 L = carve2(smem, tp);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int A = tp.a_stages, B = tp.b_stages, RS = tp.tab_slots;
  const uint32_t bar0 = smem_u32(smem);
  // barrier i lives at bar0 + 8*i
  const uint32_t full_a = bar0, empty_a = full_a + 8 * A, full_b = empty_a + 8 * A,
                 empty_b = full_b + 8 * B, tmem_full = empty_b + 8 * B, tmem_empty = tmem_full + 16,
                 tab_full = tmem_empty + 16, tab_empty = tab_full + 8 * RS,
                 win_full = tab_empty + 8 * RS, win_empty = win_full + 16;
  volatile int *abort_s = (volatile int *)(smem + kCtrlAbort);
  const uint32_t b_stage_bytes = (uint32_t)tp.BN * 128u;

  if (threadIdx.x == 0) {
    for (int i = 0; i < A; ++i) {
      mbar_init(full_a + 8 * i, kGatherWarps);
      mbar_init(empty_a + 8 * i, 1);
    }
    for (int i = 0; i < B; ++i) {
      mbar_init(full_b + 8 * i, 1);
      mbar_init(empty_b + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tmem_full + 8 * i, 1);
      mbar_init(tmem_empty + 8 * i, kEpiWarps);
      mbar_init(win_full + 8 * i, 1);
      mbar_init(win_empty + 8 * i, kGatherWarps);
    }
    for (int i = 0; i < RS; ++i) {
      mbar_init(tab_full + 8 * i, kBuildWarps);
      mbar_init(tab_empty + 8 * i, kGatherWarps);
    }
    *abort_s = 0;
    *(unsigned long long *)(smem + kCtrlLimit) = a.wait_limit_ns;
    *(int **)(smem + kCtrlStatus) = a.status;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp2) {
    tmem_alloc(smem_u32(smem + kCtrlTmemSlot), (uint32_t)tp.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *(const uint32_t *)(smem + kCtrlTmemSlot);

  const uint32_t items = (uint32_t)tp.items;
  const long long plane = (long long)g.Ho * g.Wo;
  const int tw_mask = (1 << tp.tw_log2) - 1;
  const int T = g.T;
  // K is walked in units of (32-channel half-chunk, tap), half-chunk-major; a k-stage holds two
  // consecutive units (64 bytes each of the operand row).
  // table segments: one per k-stage (tab_span == 0: two units, ndu deform groups each), or one
  // per run of tab_span half-chunks that share their single deform group (one block per tap)
  constexpr bool seg_per_stage = kSegStage;
  const uint32_t slot_entries = (uint32_t)tp.tab_slot_blocks * kTabStride2;
  const uint32_t Wp = (uint32_t)g.W + 2u;
  const uint32_t Cb = (uint32_t)g.C * 2u;       // bytes of one padded pixel
  const uint32_t Rb = Wp * Cb;                  // bytes of one padded row

  if (warp < kEpiWarps) {
    // ------------------------------ epilogue ------------------------------
    // Thread = one pixel (accumulator row); per 32 output channels one tcgen05.ld, then bias,
    // activation, rounding.  Stores: through the tensor-copy engine when the output's rows are
    // 16-byte multiples (a warp stages 32 channels x its 32 pixels in shared memory and one lane
    // issues a 4-D tensor store of that box, which also clips tiles that overhang the image),
    // else one element per lane and channel.
    TIO *out = (TIO *)a.output;
    const TIO *bias = (const TIO *)a.bias;
    const int row = warp * 32 + lane;
    const int ty = row >> tp.tw_log2, tx = row & tw_mask;
    const bool act_any = g.act == DCN_ACT_SIGMOID && g.act_hi > g.act_lo;
    PhaseTimer pt(a.counters, blockIdx.x == 0 && threadIdx.x == 0);
    uint32_t li = 0;
    int staged_co0[2] = {-1, -1};
    uint32_t slab = 0;  // tensor-store staging buffer in use (two per warp)
    constexpr uint32_t kSlabBytes = 32u * 32u * (uint32_t)sizeof(TIO);
    const uint32_t epi_base = smem_u32(L.epi) + (uint32_t)warp * 2u * kSlabBytes;
    for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, ++li) {
      const TileId2 t = decode_item2(item, g, tp);
      const int buf = (int)(li & 1);
      const uint32_t par = (li >> 1) & 1u;
      const int ncols = min(tp.BN, g.Cog - t.nt * tp.BN);
      const int co0 = t.grp * g.Cog + t.nt * tp.BN;
      const bool act_tile = act_any && co0 < g.act_hi && co0 + ncols > g.act_lo;
      pt.lap(13);
      bool ok = mbar_wait2(tmem_full + 8 * buf, par, 3, 1);
      ok = __all_sync(0xffffffffu, ok);  // the tcgen05 instructions below need the whole warp
      if (!ok) break;
      pt.lap(12);
      tc_fence_after();
      // Bias copy of this accumulator buffer (rewritten when its channels change; every warp
      // writes the same values, after the wait above so that no warp still reads the old ones).
      TIO *bias_w = reinterpret_cast<TIO *>(L.bias_s) + buf * tp.BN;
      if (co0 != staged_co0[buf]) {
        __syncwarp();
        for (int i = lane; i < tp.BN; i += 32)
          st_from_float(bias_w, i, (bias && i < ncols) ? ld_as_float(bias, co0 + i) : 0.f);
        __syncwarp();
        staged_co0[buf] = co0;
      }
      const uint32_t taddr = tmem_base + (uint32_t)(buf * tp.BN) + ((uint32_t)(warp * 32) << 16);
      if (tp.epi_tma) {
        for (int c0 = 0; c0 < ncols; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + (uint32_t)c0, r);
          tmem_ld_wait();
          const TIO *bs = bias_w + c0;
          // the slab about to be overwritten must have been read by the store issued from it
          bulk_wait_read<1>();
          __syncwarp();
          const uint32_t sbase = epi_base + slab * kSlabBytes + (uint32_t)lane * (uint32_t)sizeof(TIO);
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            float b4[4];
            load4_as_float(bs + 4 * j4, b4);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int j = 4 * j4 + k;
              float v = __uint_as_float(r[j]) + b4[k];
              if (act_tile) v = apply_act(g, co0 + c0 + j, v);
              if constexpr (sizeof(TIO) == 2) {
                TIO o;
                st_from_float(&o, 0, v);
                const unsigned short bits = *reinterpret_cast<const unsigned short *>(&o);
                asm volatile("st.shared.u16 [%0], %1;" ::"r"(sbase + (uint32_t)j * 64u), "h"(bits) : "memory");
              } else {
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(sbase + (uint32_t)j * 128u), "f"(v) : "memory");
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            // box: the warp's 32 pixels (rows of the tile) x 32 channels of one sample; pixels
            // beyond the image and channels beyond the tensor are clipped by the copy engine
            tma_store_4d(&a.out_map, epi_base + slab * kSlabBytes, t.wo0 + ((warp * 32) & tw_mask),
                         t.ho0 + ((warp * 32) >> tp.tw_log2), co0 + c0, t.n);
            bulk_commit();
          }
          slab ^= 1u;
        }
      } else {
        const int ho = t.ho0 + ty, wo = t.wo0 + tx;
        const bool valid = ho < g.Ho && wo < g.Wo;
        TIO *orow = out + (long long)t.n * g.out_sn + (long long)co0 * plane + (long long)ho * g.Wo + wo;
        for (int c0 = 0; c0 < ncols; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + (uint32_t)c0, r);
          tmem_ld_wait();
          const TIO *bs = bias_w + c0;
          TIO *oc = orow + (long long)c0 * plane;
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            float b4[4];
            load4_as_float(bs + 4 * j4, b4);
            float v[4] = {__uint_as_float(r[4 * j4]) + b4[0], __uint_as_float(r[4 * j4 + 1]) + b4[1],
                          __uint_as_float(r[4 * j4 + 2]) + b4[2], __uint_as_float(r[4 * j4 + 3]) + b4[3]};
#pragma unroll
            for (int k = 0; k < 4; ++k)
              if (act_tile) v[k] = apply_act(g, co0 + c0 + 4 * j4 + k, v[k]);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int j = 4 * j4 + k;
              if (valid && c0 + j < ncols) st_from_float(oc, (long long)j * plane, v[k]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty + 8 * buf);
    }
    if (tp.epi_tma) bulk_wait_all();  // the stores read shared memory until they complete
  } else if (warp == kMmaWarp2) {
    // ------------------------------ MMA issuer ------------------------------
    // The whole warp walks the loop (warp-uniform barrier addresses and descriptors); one
    // elected lane issues the tensor-core instructions.
    constexpr uint32_t kFmt = MODE == kModeBf16 ? 1u : 0u;
    const uint32_t idesc = (1u << 4) | (kFmt << 7) | (kFmt << 10) | ((uint32_t)(tp.BN >> 3) << 17) |
                           ((uint32_t)(kBM >> 4) << 24);
    uint32_t sa = 0, pa = 0, sb = 0, pb = 0, li = 0;
    bool ok = true;
    PhaseTimer pt(a.counters, blockIdx.x == 0 && lane == 0);
    for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x, ++li) {
      const int buf = (int)(li & 1);
      const uint32_t par = (li >> 1) & 1u;
      pt.lap(11);
      ok = __all_sync(0xffffffffu, mbar_wait2(tmem_empty + 8 * buf, par ^ 1u, 4));
      if (!ok) break;
      pt.lap(10);
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)(buf * tp.BN);
      for (int ks = 0; ks < tp.S; ++ks) {
        ok = __all_sync(0xffffffffu, mbar_wait2(full_b + 8 * sb, pb, 5));
        if (!ok) break;
        pt.lap(8);
        ok = __all_sync(0xffffffffu, mbar_wait2(full_a + 8 * sa, pa, 6));
        if (!ok) break;
        pt.lap(9);
        tc_fence_after();
        const uint64_t adesc = smem_desc_sw128(smem_u32(L.a) + sa * (uint32_t)kTileBytes);
        const uint64_t bdesc = smem_desc_sw128(smem_u32(L.b) + sb * b_stage_bytes);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                      (ks | k) != 0 ? 1u : 0u);
          umma_commit(empty_a + 8 * sa);
          umma_commit(empty_b + 8 * sb);
          if (ks == tp.S - 1) umma_commit(tmem_full + 8 * buf);
        }
        __syncwarp();
        if (++sa == (uint32_t)A) { sa = 0; pa ^= 1u; }
        if (++sb == (uint32_t)B) { sb = 0; pb ^= 1u; }
        pt.lap(11);
      }
    }
    __syncwarp();
  } else if (warp == kLoadWarp2) {
    // ------------------ weight loader (+ input windows) ------------------
    if (lane == 0) {
      const uint32_t per_mt = (uint32_t)(g.groups * tp.NT);
      uint32_t sb = 0, pb = 0;
      bool ok = true;
      // window copies: one per (tile, 32-channel half-chunk), issued as soon as its buffer is free; `wq` counts
      // them; the loop below polls for the next one between weight copies
      uint32_t w_item = blockIdx.x, wq = 0;
      int w_cc = 0;
      const uint32_t wbytes = (uint32_t)win_bytes(tp);
      auto try_window = [&]() {
        // buffer wq & 1 was last used by window wq - 2
        if (kWin && w_item < items && mbar_test(win_empty + 8 * (wq & 1u), ((wq >> 1) & 1u) ^ 1u)) {
          const TileId2 t = decode_item2(w_item, g, tp);
          const uint32_t wb = wq & 1u;
          mbar_arrive_expect_tx(win_full + 8 * wb, wbytes);
          // coordinates in the padded tensor: (channel, column + 1, row + 1, sample)
          tma_load_4d(smem_u32(L.win) + wb * wbytes, &a.win_map, t.grp * g.Cg + w_cc * 32,
                      win_x0(g, tp, t.wo0) + 1, win_y0(g, tp, t.ho0) + 1, t.n, win_full + 8 * wb);
          ++wq;
          if (++w_cc == tp.KH) { w_cc = 0; w_item += gridDim.x; }
        }
      };
      PhaseTimer pt(a.counters, blockIdx.x == 0);
      for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const uint32_t rem = item % per_mt;
        const uint8_t *src = a.wtiles + (size_t)rem * tp.S * b_stage_bytes;
        for (int ks = 0; ks < tp.S; ++ks) {
          pt.lap(15);
          if (kWin) {
            // while waiting for a free weight stage keep serving the windows
            const unsigned long long t0 = globaltimer_ns();
            uint32_t it = 0;
            try_window();
            while (!mbar_test(empty_b + 8 * sb, pb ^ 1u)) {
              try_window();
              if ((++it & 63u) == 0u) {
                if (*abort_s) { ok = false; break; }
                if (globaltimer_ns() - t0 > a.wait_limit_ns) {
                  *abort_s = 1;
                  atomicCAS(a.status, 0, 7);
                  ok = false;
                  break;
                }
              }
            }
          } else {
            ok = mbar_wait2(empty_b + 8 * sb, pb ^ 1u, 7);
          }
          if (!ok) break;
          pt.lap(14);
          const bool withhold = (a.debug_flags & 1) && item + gridDim.x >= items && ks == tp.S - 1;
          if (!withhold) {
            mbar_arrive_expect_tx(full_b + 8 * sb, b_stage_bytes);
            bulk_copy_g2s(smem_u32(L.b) + sb * b_stage_bytes, src + (size_t)ks * b_stage_bytes,
                          b_stage_bytes, full_b + 8 * sb);
          }
          if (++sb == (uint32_t)B) { sb = 0; pb ^= 1u; }
        }
      }
      if (kWin) {
        // windows still owed (the gather of the last tile waits for them)
        const unsigned long long t0 = globaltimer_ns();
        uint32_t it = 0;
        while (ok && w_item < items) {
          try_window();
          if ((++it & 63u) == 0u) {
            if (*abort_s) break;
            if (globaltimer_ns() - t0 > a.wait_limit_ns) {
              *abort_s = 1;
              atomicCAS(a.status, 0, 11);
              break;
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp < kFirstGatherWarp) {
    // ------------------------------ table builders ------------------------------
    // The (unit, deform group) blocks of all segments form one stream; builder warp b computes
    // blocks b, b + 2, ...: four rows per thread.  The twelve loads of a block are in flight
    // together, and a block is computed only after the loads of the warp's next block have
    // been issued.
    const int bw = warp - kFirstBuildWarp;
    const TIO *off = (const TIO *)a.offset;
    const TIO *msk = (const TIO *)a.mask;
    const uint32_t dead_off = ((uint32_t)(g.H + 1) * Rb) | kWinFlag;  // an all-zero 2x2 neighbourhood
    const bool dense_planes = g.off_ps == 1 && g.msk_ps == 1 && g.off_cs == plane && g.msk_cs == plane;
    const int wh = tp.win_h, ww = tp.win_w;
    const uint32_t tabw_addr = smem_u32(L.tab_w) + (uint32_t)lane * 8u;
    const uint32_t tabo_addr = smem_u32(L.tab_off) + (uint32_t)lane * 4u;
    uint32_t q = 0, turn = 0;
    bool ok = true;
    PhaseTimer pt(a.counters, blockIdx.x == 0 && bw == 0 && lane == 0);

    // Ask L2 for the offset and mask planes of tile `nitem` (dense planes only).
    auto prefetch_tile = [&](uint32_t nitem) {
      if (!dense_planes || nitem >= items) return;
      const TileId2 nt_ = decode_item2(nitem, g, tp);
      const int lr_log2 = max(0, tp.tw_log2 + (sizeof(TIO) == 4 ? 2 : 1) - 7);
      const int pp_log2 = (7 - tp.tw_log2) + lr_log2;  // 128-byte lines per plane of the tile
      const int planes_off = off ? g.dg * 2 * T : 0;
      const int planes = planes_off + (msk ? g.dg * T : 0);
      const TIO *obase = off ? off + (long long)nt_.n * g.off_sn : nullptr;
      const TIO *mbase = msk ? msk + (long long)nt_.n * g.msk_sn : nullptr;
      for (int idx = bw * 32 + lane; idx < (planes << pp_log2); idx += kBuildWarps * 32) {
        const int pl = idx >> pp_log2, r = idx & ((1 << pp_log2) - 1);
        const int ry = r >> lr_log2, rl = r & ((1 << lr_log2) - 1);
        const int ho = nt_.ho0 + ry;
        if (ho >= g.Ho) continue;
        const long long pixel = (long long)ho * g.Wo + nt_.wo0;
        const TIO *ptr = pl < planes_off ? obase + (long long)pl * plane + pixel
                                         : mbase + (long long)(pl - planes_off) * plane + pixel;
        if (nt_.wo0 + rl * (int)(128 / sizeof(TIO)) < g.Wo)
          prefetch_l2(reinterpret_cast<const char *>(ptr) + rl * 128);
      }
    };

    // the block whose loads are in flight (always one of the current tile)
    uint32_t roh[4], row_[4], rmm[4];
    bool pend = false, pend_first = false, pend_last = false;
    uint32_t pend_e = 0, pend_slot = 0, pend_par = 0;
    int pend_ti = 0, pend_tj = 0;
    int ho0 = 0, wo0 = 0, wy0 = 0, wx0 = 0;   // current tile
    // entries of the pending block, then its segment's hand-over if it was this warp's last
    // block there
    auto flush = [&]() -> bool {
      if (!pend) return true;
      pend = false;
      if (pend_first) {
        pt.lap(1);
        const bool r = mbar_wait2(tab_empty + 8 * pend_slot, pend_par, 9);
        pt.lap(6);
        if (!r) return false;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float4 wt = make_float4(0.f, 0.f, 0.f, 0.f);
        uint32_t eo = dead_off;
        // this thread's rows: lane, lane + 32, lane + 64, lane + 96
        const int r = lane + 32 * j;
        const int ho = ho0 + (r >> tp.tw_log2), wo = wo0 + (r & tw_mask);
        const float h_im = (float)(ho * g.stride_h - g.pad_h + pend_ti * g.dil_h) + RawOf<TIO>::to_float(roh[j]);
        const float w_im = (float)(wo * g.stride_w - g.pad_w + pend_tj * g.dil_w) + RawOf<TIO>::to_float(row_[j]);
        if (ho < g.Ho && wo < g.Wo && h_im > -1.f && w_im > -1.f && h_im < (float)g.H && w_im < (float)g.W) {
          const float m = msk ? mask_value(g, RawOf<TIO>::to_float(rmm[j])) : 1.f;
          const float hf = floorf(h_im), wf = floorf(w_im);
          const float lh = h_im - hf, lw = w_im - wf;
          const float hh = 1.f - lh, hw = 1.f - lw;
          wt.x = hh * hw * m; wt.y = hh * lw * m; wt.z = lh * hw * m; wt.w = lh * lw * m;
          const int hl = (int)hf, wl = (int)wf;
          // inside the shared-memory window: offset within the window (64 bytes per pixel);
          // else (flagged) the offset within the padded sample
          const int wy = hl - wy0, wx = wl - wx0;
          if (kWin && wy >= 0 && wx >= 0 && wy + 1 < wh && wx + 1 < ww)
            eo = (uint32_t)(wy * ww + wx) * 64u;
          else
            eo = (((uint32_t)(hl + 1) * Wp + (uint32_t)(wl + 1)) * Cb) | kWinFlag;
        }
        const uint32_t e = pend_e + 32u * (uint32_t)j;
        sts8(tabw_addr + e * 8u, pack_weights2<MODE>(wt.x, wt.y), pack_weights2<MODE>(wt.z, wt.w));
        sts4(tabo_addr + e * 4u, eo);
      }
      if (pend_last) {
        __syncwarp();
        if (lane == 0) mbar_arrive(tab_full + 8 * pend_slot);
      }
      return true;
    };

    prefetch_tile(blockIdx.x);
    for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
      ok = flush();   // (a pending block belongs to the previous tile)
      if (!ok) break;
      const TileId2 t = decode_item2(item, g, tp);
      prefetch_tile(item + gridDim.x);
      ho0 = t.ho0; wo0 = t.wo0;
      wy0 = win_y0(g, tp, t.ho0); wx0 = win_x0(g, tp, t.wo0);
      // pixel of each of this thread's rows (a row beyond the image reads pixel 0; its entry
      // fails the test above)
      int pix[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = lane + 32 * j;
        const int ho = t.ho0 + (r >> tp.tw_log2), wo = t.wo0 + (r & tw_mask);
        pix[j] = (ho < g.Ho && wo < g.Wo) ? ho * g.Wo + wo : 0;
      }
      const TIO *offn = off ? off + (long long)t.n * g.off_sn : nullptr;
      const TIO *mskn = msk ? msk + (long long)t.n * g.msk_sn : nullptr;
      const int nseg = seg_per_stage ? tp.S : tp.KH / tp.tab_span;
      // running unit (stage segments): half-chunk, tap and the tap's row / column
      int u_hc = 0, u_tap = 0, u_ti = 0, u_tj = 0;
      int c_hc = -1, dg_lo = 0, nd = 1;   // deform groups of half-chunk c_hc
      for (int sg = 0; sg < nseg && ok; ++sg, ++q) {
        const uint32_t slot = q % (uint32_t)RS;
        const uint32_t spar = ((q / (uint32_t)RS) & 1u) ^ 1u;
        // the segment's units: two consecutive (half-chunk, tap) units, or the taps of one run
        const int n_u = seg_per_stage ? min(2, tp.U - 2 * sg) : T;
        if (!seg_per_stage) { u_hc = sg * tp.tab_span; u_tap = 0; u_ti = 0; u_tj = 0; }
        bool first_mine = true;
        for (int ui = 0; ui < n_u && ok; ++ui) {
          const int hc = u_hc, tap = u_tap, ti = u_ti, tj = u_tj;
          // next unit
          if (++u_tj == g.kw) { u_tj = 0; ++u_ti; }
          if (++u_tap == T) { u_tap = 0; u_ti = 0; u_tj = 0; ++u_hc; }
          if (hc != c_hc) {
            c_hc = hc;
            const int c0 = t.grp * g.Cg + hc * 32;
            dg_lo = c0 / g.cpdg;
            nd = seg_per_stage ? (min(c0 + 32, (t.grp + 1) * g.Cg) - 1) / g.cpdg - dg_lo + 1 : 1;
          }
          for (int d = 0; d < nd && ok; ++d) {
            const bool mine = (int)turn == bw;
            if (++turn == (uint32_t)kBuildWarps) turn = 0;
            if (!mine) continue;
            // loads of this block, issued before the pending block is computed
            uint32_t noh[4], now_[4], nmm[4];
            const TIO *ob = off ? offn + ((long long)(dg_lo + d) * 2 * T + 2 * tap) * g.off_cs : nullptr;
            const TIO *mb = msk ? mskn + ((long long)(dg_lo + d) * T + tap) * g.msk_cs : nullptr;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              noh[j] = 0; now_[j] = 0; nmm[j] = 0;
              if (off) {
                const TIO *pp = ob + (long long)pix[j] * g.off_ps;
                noh[j] = ldg_raw_ordered(pp);
                now_[j] = ldg_raw_ordered(pp + g.off_cs);
              }
              if (msk) nmm[j] = ldg_raw_ordered(mb + (long long)pix[j] * g.msk_ps);
            }
            ok = flush();
            if (!ok) break;
#pragma unroll
            for (int j = 0; j < 4; ++j) { roh[j] = noh[j]; row_[j] = now_[j]; rmm[j] = nmm[j]; }
            pend = true;
            pend_first = first_mine;
            pend_last = false;
            first_mine = false;
            pend_slot = slot;
            pend_par = spar;
            pend_ti = ti;
            pend_tj = tj;
            pend_e = slot * slot_entries +
                     (seg_per_stage ? (uint32_t)(ui * tp.ndu + d) : (uint32_t)tap) * kTabStride2;
          }
        }
        if (!ok) break;
        if (first_mine) {
          // none of the segment's blocks was this warp's: it still waits for the slot and
          // arrives, so that no arrival is counted for the slot's previous use
          ok = mbar_wait2(tab_empty + 8 * slot, spar, 9);
          if (!ok) break;
          __syncwarp();
          if (lane == 0) mbar_arrive(tab_full + 8 * slot);
        } else {
          pend_last = true;  // the pending block is this warp's last one of the segment
        }
      }
    }
    if (ok) ok = flush();
    if (!ok) *abort_s = 1;
  } else {
    // ------------------------------ gather ------------------------------
    const int gw = warp - kFirstGatherWarp;
    const int sub = lane >> 3;  // row within the warp's group of four
    const int v = lane & 7;     // 16-byte vector of the 128-byte row
    const int usel = v >> 2;    // which of the stage's two units this lane gathers
    const int cv = v & 3;       // 8-channel vector within the unit
    const int row0 = gw * 4 + sub;
    const uint32_t a_base = smem_u32(L.a) + (uint32_t)(row0 * 128 + ((v ^ (row0 & 7)) << 4));
    const char *xpad = reinterpret_cast<const char *>(a.xpad);
    const uint32_t wbytes = (uint32_t)win_bytes(tp);
    const uint32_t win_rb = (uint32_t)tp.win_w * 64u;
    const uint32_t win_s = smem_u32(L.win) + (uint32_t)cv * 16u;
    const uint32_t tabw_addr = smem_u32(L.tab_w) + (uint32_t)row0 * 8u;
    const uint32_t tabo_addr = smem_u32(L.tab_off) + (uint32_t)row0 * 4u;
    const int KH = tp.KH;
    const int nseg = seg_per_stage ? tp.S : KH / tp.tab_span;   // table segments per tile

    const uint32_t span = seg_per_stage ? 1u : (uint32_t)tp.tab_span;
    // position: the k-stage (item, s) whose loads are issued next; its unit A = 2 s is
    // (half-chunk hcA, tap tapA); in run mode hcA is half-chunk inrunA of run runA
    uint32_t item = blockIdx.x;
    int s = 0, hcA = 0, tapA = 0;
    uint32_t runA = 0, inrunA = 0;
    uint32_t sa = 0, pa = 0;
    // running counts over the tiles of this block: window of (tile, half-chunk 0), table
    // segment of (tile, run 0); table ring position of the current stage (stage segments)
    uint32_t win_base = 0, seg_base = 0, slotS = 0, phS = 0;
    // windows / run segments: next one to wait for, next one to hand back
    uint32_t win_acq = 0, win_rel = 0, seg_acq = 0, seg_rel = 0;
    // this lane's unit of the stage; the values below change with its half-chunk only
    int my_hc = -2;
    const char *gbase = nullptr;   // sample + channel bytes of this lane's vector (global)
    uint32_t wbase = 0;            // window buffer of the half-chunk + this lane's 16 bytes (shared address)
    uint32_t e_fixed = 0;          // table entry of row0 without the stage's (or tap's) part
    uint32_t e0 = 0;               // table entry of pass 0
    bool zero_vec = false;
    int grp = 0;
    const char *sbase = nullptr;
    auto enter_item = [&]() {
      const TileId2 t = decode_item2(item, g, tp);
      grp = t.grp;
      sbase = xpad + (unsigned long long)t.n * ((unsigned long long)(g.H + 2) * Rb);
      my_hc = -2;
    };
    // Per-lane values of the stage at the current position.
    auto enter_stage = [&]() {
      int hc = hcA, tap = tapA;
      uint32_t run = runA;
      if (usel) {
        if (++tap == T) {
          tap = 0; ++hc;
          if (inrunA + 1u == span) ++run;
        }
      }
      const int key = 2 * s + usel < tp.U ? hc : -1;
      if (key != my_hc) {
        my_hc = key;
        const int cg = hc * 32 + cv * 8;           // channel within the conv group
        zero_vec = key < 0 || cg >= g.Cg;
        const int c0 = grp * g.Cg + hc * 32;
        const int c = zero_vec ? grp * g.Cg : c0 + cv * 8;
        gbase = sbase + (unsigned long long)c * 2ull;
        wbase = win_s + ((win_base + (uint32_t)hc) & 1u) * wbytes;
        if (seg_per_stage)
          e_fixed = ((uint32_t)(usel * tp.ndu) + (zero_vec ? 0u : (uint32_t)(c / g.cpdg - c0 / g.cpdg))) * kTabStride2;
        else
          e_fixed = ((seg_base + run) & 1u) * slot_entries;
      }
      e0 = seg_per_stage ? slotS * slot_entries + e_fixed : e_fixed + (uint32_t)tap * kTabStride2;
    };

    uint4 qd[2][4];
    uint2 wq2[2];
    uint32_t tok = 0;
    bool ok = true;
    PhaseTimer pt(a.counters, blockIdx.x == 0 && gw == 0 && lane == 0);
    // loads of pass p of the k-stage at the current position into register set p
    auto issue = [&](int p) {
      uint2 w = make_uint2(0u, 0u);
      uint32_t o = ((uint32_t)(g.H + 1) * Rb) | kWinFlag;   // an all-zero neighbourhood
      if (!zero_vec) {
        const uint32_t e = e0 + (uint32_t)(p * kRowsPerPass);
        w = lds8(tabw_addr + e * 8u);
        o = lds4(tabo_addr + e * 4u);
      }
      const uint32_t ob = o & ~kWinFlag;
      if constexpr (kWin) {
        // The two units of a row read 64-byte slots; the lanes of unit 0 start with the
        // even slot of their left/right pair and those of unit 1 with the odd one, so the
        // eight lanes of a row always cover all 32 banks.  (The window's row pitch is an even
        // number of slots: the bottom corners repeat the top ones' parity.)
        const bool from_global = (o & kWinFlag) != 0u;
        const bool swap = (((ob >> 6) & 1u) != (uint32_t)usel) && !from_global;
        if (swap) w = make_uint2(__byte_perm(w.x, 0u, 0x1032), __byte_perm(w.y, 0u, 0x1032));
        const uint32_t sp = wbase + ob;
        const uint32_t s1 = swap ? sp + 64u : sp, s2 = swap ? sp : sp + 64u;
        if (!__any_sync(0xffffffffu, from_global)) {
          // the usual case: every lane of the warp reads the window
          qd[p][0] = lds16(s1, tok);
          qd[p][1] = lds16(s2, tok);
          qd[p][2] = lds16(s1 + win_rb, tok);
          qd[p][3] = lds16(s2 + win_rb, tok);
        } else {
          const char *base = gbase + ob;
          qd[p][0] = ld16_either(from_global, base, s1, tok);
          qd[p][1] = ld16_either(from_global, base + Cb, s2, tok);
          qd[p][2] = ld16_either(from_global, base + Rb, s1 + win_rb, tok);
          qd[p][3] = ld16_either(from_global, base + Rb + Cb, s2 + win_rb, tok);
        }
      } else {
        const char *base = gbase + ob;
        qd[p][0] = ld16_global(base, tok);
        qd[p][1] = ld16_global(base + Cb, tok);
        qd[p][2] = ld16_global(base + Rb, tok);
        qd[p][3] = ld16_global(base + Rb + Cb, tok);
      }
      wq2[p] = w;
    };
    auto blend_store = [&](uint32_t stage_addr, int p) {
      uint4 w = table_weights<MODE>(wq2[p]);
      w.x |= tok;  // tok is 0: pins the blend behind the loads issued before it
      uint4 r;
      if constexpr (MODE == kModeBf16) r = blend8_bf16(w, qd[p][0], qd[p][1], qd[p][2], qd[p][3]);
      else r = blend8_f16(w, qd[p][0], qd[p][1], qd[p][2], qd[p][3]);
      sts16(stage_addr + (uint32_t)(p * kRowsPerPass * 128), r);
    };
    // What the loads of the k-stage at the current position need: its table segment(s) and
    // the windows of both its units (unit B's are the later ones).
    auto acquire = [&]() -> bool {
      uint32_t hcB = (uint32_t)hcA, runB = runA;
      if (tapA + 1 == T && 2 * s + 1 < tp.U) {
        ++hcB;
        if (inrunA + 1u == span) ++runB;
      }
      if (seg_per_stage) {
        if (!mbar_wait2(tab_full + 8 * slotS, phS, 12)) return false;
      } else {
        while (seg_acq <= seg_base + runB) {
          if (!mbar_wait2(tab_full + 8 * (seg_acq & 1u), (seg_acq >> 1) & 1u, 12)) return false;
          ++seg_acq;
        }
      }
      if (kWin) {
        while (win_acq <= win_base + hcB) {
          if (!mbar_wait2(win_full + 8 * (win_acq & 1u), (win_acq >> 1) & 1u, 13)) return false;
          ++win_acq;
        }
      }
      return true;
    };

    bool valid = item < items;
    if (valid) {
      enter_item();
      ok = acquire();
      pt.lap(2);
      if (ok) { enter_stage(); issue(0); }
    }
    while (valid && ok) {
#pragma unroll
      for (int p = 1; p < kPasses2; ++p) issue(p);
      // Every read of the finishing stage's table entries has been issued.
      const uint32_t cur_sa = sa | (pa << 8);   // ring slot and phase of the finishing stage
      if (seg_per_stage) {
        // its segment goes back to the builders
        __syncwarp();
        if (lane == 0) mbar_arrive(tab_empty + 8 * slotS);
        if (++slotS == (uint32_t)RS) { slotS = 0; phS ^= 1u; }
      }
      // move the position to the next stage
      if (++sa == (uint32_t)A) { sa = 0; pa ^= 1u; }
      tapA += 2;
      while (tapA >= T) {
        tapA -= T; ++hcA;
        if (++inrunA == span) { inrunA = 0; ++runA; }
      }
      if (++s == tp.S) {
        s = 0; hcA = 0; tapA = 0; runA = 0; inrunA = 0;
        win_base += (uint32_t)KH;
        seg_base += (uint32_t)nseg;
        item += gridDim.x;
        valid = item < items;
        if (valid) enter_item();
      }
      if (!seg_per_stage) {
        // run segments before the next stage's first unit go back to the builders
        const uint32_t seg_keep = valid ? seg_base + runA : seg_acq;
        if (seg_rel < seg_keep) {
          __syncwarp();
          if (lane == 0)
            for (uint32_t i = seg_rel; i < seg_keep; ++i) mbar_arrive(tab_empty + 8 * (i & 1u));
          seg_rel = seg_keep;
        }
      }
      pt.lap(4);
      ok = mbar_wait2(empty_a + 8 * (cur_sa & 0xffu), (cur_sa >> 8) ^ 1u, 8);
      pt.lap(3);
      if (!ok) break;
      const uint32_t cur_addr = a_base + (cur_sa & 0xffu) * (uint32_t)kTileBytes;
      blend_store(cur_addr, 0);
      if (valid) {
        pt.lap(4);
        ok = acquire();
        pt.lap(2);
        if (!ok) break;
        enter_stage();
        issue(0);
      }
#pragma unroll
      for (int p = 1; p < kPasses2; ++p) blend_store(cur_addr, p);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(full_a + 8 * (cur_sa & 0xffu));
      if (kWin) {
        // all loads from the windows before the next stage's first unit have returned (their
        // values were consumed above): those windows go back to the loader
        const uint32_t win_keep = valid ? win_base + (uint32_t)hcA : win_acq;
        if (win_rel < win_keep) {
          if (lane == 0)
            for (uint32_t i = win_rel; i < win_keep; ++i) mbar_arrive(win_empty + 8 * (i & 1u));
          win_rel = win_keep;
        }
      }
    }
    if (!ok) *abort_s = 1;
  }

  // ------------------------------ teardown ------------------------------
  if (*abort_s) {
    // give copies and MMAs already in flight time to land before memory is released
    for (int i = 0; i < 20; ++i) __nanosleep(50000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)tp.tmem_cols);
  }
}

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime (the library does not link
// against the driver library).
EncodeTiledFn encode_fn() {
  static std::atomic<EncodeTiledFn> fn{nullptr};
  EncodeTiledFn f = fn.load(std::memory_order_acquire);
  if (f) return f;
  void *p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || !p) {
    cudaGetLastError();
    return nullptr;
  }
  f = (EncodeTiledFn)p;
  fn.store(f, std::memory_order_release);
  return f;
}

template <typename TIO, int MODE, bool kWin, bool kSegStage>
cudaError_t launch_one2(const Tc2Args &a, const TcPlan &tp, cudaStream_t s) {
  auto kern = dcn_fwd_tc2<TIO, MODE, kWin, kSegStage>;
  static std::atomic<unsigned long long> done_mask{0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const unsigned long long bit = 1ull << (dev & 63);
  if (!(done_mask.load(std::memory_order_acquire) & bit)) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return e;
    done_mask.fetch_or(bit, std::memory_order_release);
  }
  // leave what the kernel does not need of the SM's 256 KB to L1 (the global part of the
  // gather lives on it): the smallest shared-memory configuration that holds the block
  static std::atomic<int> carve_pct[64];
  int pct = 100;
  {
    const size_t need = tp.smem + 1024;
    const size_t configs_kb[] = {8, 16, 32, 64, 100, 132, 164, 196, 228};
    for (size_t kb : configs_kb)
      if (kb * 1024 >= need) { pct = (int)(kb * 1024 * 100 / 233472); break; }
  }
  if (carve_pct[dev & 63].load(std::memory_order_acquire) != pct) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, pct > 100 ? 100 : pct);
    if (e != cudaSuccess) return e;
    carve_pct[dev & 63].store(pct, std::memory_order_release);
  }
  kern<<<tp.grid, kThreads2, tp.smem, s>>>(a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_tc2(const Geom &g, const TcPlan &tp, const Ptrs &p, int dtype, const void *xpad,
                       const void *wtiles, int *status, unsigned long long *counters,
                       unsigned long long wait_limit_ns, int debug_flags, cudaStream_t s) {
  if (tp.items == 0) return cudaSuccess;
  Tc2Args a;
  memset(&a, 0, sizeof(a));
  a.g = g;
  a.tp = tp;
  a.xpad = xpad;
  a.wtiles = (const uint8_t *)wtiles;
  a.offset = p.offset;
  a.mask = p.mask;
  a.bias = p.bias;
  a.output = p.output;
  a.status = status;
  a.counters = counters;
  a.wait_limit_ns = wait_limit_ns ? wait_limit_ns : kWaitLimitNs;
  a.debug_flags = debug_flags;
  const CUtensorMapDataType in_type =
      tp.op_format == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (tp.win_h > 0) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    const cuuint64_t dims[4] = {(cuuint64_t)g.C, (cuuint64_t)g.W + 2, (cuuint64_t)g.H + 2, (cuuint64_t)g.N};
    const cuuint64_t strides[3] = {(cuuint64_t)g.C * 2, (cuuint64_t)(g.W + 2) * g.C * 2,
                                   (cuuint64_t)(g.H + 2) * (g.W + 2) * g.C * 2};
    const cuuint32_t box[4] = {32, (cuuint32_t)tp.win_w, (cuuint32_t)tp.win_h, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&a.win_map, in_type, 4, const_cast<void *>(xpad), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  if (tp.epi_tma) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    const CUtensorMapDataType out_type =
        dtype == DCN_DTYPE_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                               : (dtype == DCN_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                         : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
    const cuuint64_t es = (cuuint64_t)tp.io_bytes;
    const cuuint64_t dims[4] = {(cuuint64_t)g.Wo, (cuuint64_t)g.Ho, (cuuint64_t)g.Co, (cuuint64_t)g.N};
    const cuuint64_t strides[3] = {(cuuint64_t)g.Wo * es, (cuuint64_t)g.Ho * g.Wo * es,
                                   (cuuint64_t)g.out_sn * es};
    const cuuint32_t tw = 1u << tp.tw_log2;
    const cuuint32_t box[4] = {tw, 32u / tw, 32, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&a.out_map, out_type, 4, p.output, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  const bool win = tp.win_h > 0, seg_stage = tp.tab_span == 0;
#define DCN_TC2_LAUNCH(TIO, MODE)                                                              \
  (win ? (seg_stage ? launch_one2<TIO, MODE, true, true>(a, tp, s)                             \
                    : launch_one2<TIO, MODE, true, false>(a, tp, s))                           \
       : (seg_stage ? launch_one2<TIO, MODE, false, true>(a, tp, s)                            \
                    : launch_one2<TIO, MODE, false, false>(a, tp, s)))
  if (dtype == DCN_DTYPE_F32) return DCN_TC2_LAUNCH(float, kModeBf16);
  if (dtype == DCN_DTYPE_F16) return DCN_TC2_LAUNCH(__half, kModeF16);
  return DCN_TC2_LAUNCH(__nv_bfloat16, kModeBf16);
#undef DCN_TC2_LAUNCH
}

}  // namespace dcn
