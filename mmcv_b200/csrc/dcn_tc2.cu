// Second-generation tensor-core kernel of the deformable-convolution forward (16-bit
// operands: bf16 or fp16) for sm_100a.
//
// Same contraction as dcn_fwd_tc (out[p, co] = sum_k A[p, k] * Wt[co, k], A never written to
// global memory; it replaces the gather kernel, the per-sample GEMM loop and the bias pass of
// mmcv/ops/csrc/common/cuda/modulated_deform_conv_cuda_kernel.cuh:186-245 and
// mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:108-137), with the producer side split into
// two decoupled roles:
//
//   * table builders (4 warps; a warp owns every fourth table segment and fills its blocks of
//     128 entries, four rows per thread) turn offsets and
//     masks into tap-table entries -- four 16-bit corner weights with the modulation folded
//     in, and the byte offset of the top-left corner -- and publish them through a ring of
//     table segments in shared memory.  They run ahead of the gather, which therefore never
//     waits for an offset or a mask.
//   * gather warps (16, in two groups that fill alternate k-stages) read an entry, fetch the
//     four corners, blend them on packed 16-bit FMAs and write the 128-byte-swizzled operand
//     tile tcgen05.mma reads; a thread blends 16 channels of one (row, unit).  The input is a
//     channels-last copy with a one-pixel zero border around every sample: a corner outside
//     the image reads zeros, a sample outside the sampling gate points at an all-zero
//     neighbourhood with zero weights, so the loads carry no predicates and a corner inside
//     the image is always read (0 * Inf = NaN as in the reference,
//     modulated_deform_conv_cuda_kernel.cuh:100-107).
//   * K is walked in units of (32-channel half-chunk, tap); a k-stage is two consecutive units.
//     The 32-channel slice of the tile's input neighbourhood (its undeformed footprint plus a
//     margin) is brought into shared memory by one tensor-map copy (cp.async.bulk.tensor, zero
//     fill outside the tensor) per half-chunk, double-buffered; entries whose 2x2 neighbourhood
//     lies inside that window are read from shared memory (64 bytes per pixel; which of the
//     left/right corners and which of its two 16-byte vectors a lane reads first depends on
//     the slot's and the row's parity, so that the eight lanes of a quarter warp never meet in
//     a bank), the others from global memory.
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
constexpr int kWinWarp = 6;   // (warp 7 idles: the builders are a warpgroup of their own)
constexpr int kFirstBuildWarp = 8;
constexpr int kBuildWarps = 4;
constexpr int kFirstGatherWarp = kFirstBuildWarp + kBuildWarps;
constexpr int kGatherWarps = 16;
constexpr int kThreads2 = (kFirstGatherWarp + kGatherWarps) * 32;  // 896 = 7 warpgroups: epilogue | MMA, weight loader, window loader, - | 4 builders | 4 x gather
constexpr int kGroups2 = 2;                              // gather groups; group i fills k-stages i, i + 2, ...
constexpr int kWarpsPerGroup = kGatherWarps / kGroups2;  // 8 warps: 64 rows per pass, two passes per stage
constexpr int kTabStride2 = kBM + 8;  // entries of one (unit / tap, deform group) block; the skew puts the
                                      // blocks of a stage's two units into different bank halves
constexpr uint32_t kWinFlag = 0x80000000u;  // table entry: the neighbourhood is read from global memory

// Register budget per role (setmaxnreg works on warpgroups of four consecutive warps; the
// block starts with 72 registers per thread): the two warpgroups that hold the epilogue and the
// MMA / loader warps give registers back, the four gather warpgroups take them, the builders
// keep theirs.
constexpr int kRegsLight = 56, kRegsGather = 80;
template <int N>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

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

// Continuation of a wait (kept out of the fast path): polls until the phase completes, the block aborts or the
// time limit passes (then it raises the abort flag and records `code` in the status word).
__device__ __forceinline__ bool mbar_wait_slow2(uint32_t bar, uint32_t parity, int code, int backoff) {
  uint8_t *ctrl = smem_aligned();
  volatile int *abort_s = (volatile int *)(ctrl + kCtrlAbort);
  const unsigned long long limit = *(const unsigned long long *)(ctrl + kCtrlLimit);
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (backoff) __nanosleep((unsigned)backoff);
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
__device__ __forceinline__ bool mbar_wait2(uint32_t bar, uint32_t parity, int code, int backoff = 100) {
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

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr)
      : "memory");
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
      mbar_init(full_a + 8 * i, kWarpsPerGroup);
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
      mbar_init(tab_full + 8 * i, kSegStage ? 1 : kBuildWarps);   // the segment's owner, or all builders
      mbar_init(tab_empty + 8 * i, kSegStage ? kWarpsPerGroup : kGatherWarps);
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

  if (warp < kFirstBuildWarp) {
  reg_dec<kRegsLight>();
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
      bool ok = mbar_wait2(tmem_full + 8 * buf, par, 3, 200);
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
          // the slab about to be overwritten must have been read by the store issued from it
          bulk_wait_read<1>();
          __syncwarp();
          const uint32_t sbase = epi_base + slab * kSlabBytes + (uint32_t)lane * (uint32_t)sizeof(TIO);
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            uint32_t r[16];
            tmem_ld16(taddr + (uint32_t)(c0 + 16 * h), r);
            tmem_ld_wait();
            const TIO *bs = bias_w + c0 + 16 * h;
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              float b4[4];
              load4_as_float(bs + 4 * j4, b4);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int j = 4 * j4 + k;
                float v = __uint_as_float(r[j]) + b4[k];
                if (act_tile) v = apply_act(g, co0 + c0 + 16 * h + j, v);
                const uint32_t sa_ = sbase + (uint32_t)(16 * h + j) * 32u * (uint32_t)sizeof(TIO);
                if constexpr (sizeof(TIO) == 2) {
                  TIO o;
                  st_from_float(&o, 0, v);
                  const unsigned short bits = *reinterpret_cast<const unsigned short *>(&o);
                  asm volatile("st.shared.u16 [%0], %1;" ::"r"(sa_), "h"(bits) : "memory");
                } else {
                  asm volatile("st.shared.f32 [%0], %1;" ::"r"(sa_), "f"(v) : "memory");
                }
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
#pragma unroll 1
        for (int c0 = 0; c0 < ncols; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(taddr + (uint32_t)c0, r);
          tmem_ld_wait();
          const TIO *bs = bias_w + c0;
          TIO *oc = orow + (long long)c0 * plane;
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
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
      ok = __all_sync(0xffffffffu, mbar_wait2(tmem_empty + 8 * buf, par ^ 1u, 4, 0));
      if (!ok) break;
      pt.lap(10);
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)(buf * tp.BN);
      for (int ks = 0; ks < tp.S; ++ks) {
        ok = __all_sync(0xffffffffu, mbar_wait2(full_b + 8 * sb, pb, 5, 0));
        if (!ok) break;
        pt.lap(8);
        ok = __all_sync(0xffffffffu, mbar_wait2(full_a + 8 * sa, pa, 6, 0));
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
    // ------------------------------ weight loader ------------------------------
    if (lane == 0) {
      const uint32_t per_mt = (uint32_t)(g.groups * tp.NT);
      uint32_t sb = 0, pb = 0;
      bool ok = true;
      PhaseTimer pt(a.counters, blockIdx.x == 0);
      for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const uint32_t rem = item % per_mt;
        const uint8_t *src = a.wtiles + (size_t)rem * tp.S * b_stage_bytes;
        for (int ks = 0; ks < tp.S; ++ks) {
          pt.lap(15);
          ok = mbar_wait2(empty_b + 8 * sb, pb ^ 1u, 7);
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
    }
    __syncwarp();
  } else if (warp == kWinWarp) {
    // ------------------------------ window loader ------------------------------
    // One tensor-map copy per (tile, 32-channel half-chunk), in the order the gather uses
    // them, into the two window buffers in turn.
    if (kWin && lane == 0) {
      const uint32_t wbytes = (uint32_t)win_bytes(tp);
      uint32_t wq = 0;
      bool ok = true;
      for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const TileId2 t = decode_item2(item, g, tp);
        for (int hc = 0; hc < tp.KH; ++hc, ++wq) {
          const uint32_t wb = wq & 1u;
          // buffer wb was last used by window wq - 2
          ok = mbar_wait2(win_empty + 8 * wb, ((wq >> 1) & 1u) ^ 1u, 11);
          if (!ok) break;
          mbar_arrive_expect_tx(win_full + 8 * wb, wbytes);
          // coordinates in the padded tensor: (channel, column + 1, row + 1, sample)
          tma_load_4d(smem_u32(L.win) + wb * wbytes, &a.win_map, t.grp * g.Cg + hc * 32,
                      win_x0(g, tp, t.wo0) + 1, win_y0(g, tp, t.ho0) + 1, t.n, win_full + 8 * wb);
        }
      }
    }
    __syncwarp();
  }
  } else if (warp < kFirstGatherWarp) {
    // ------------------------------ table builders ------------------------------
    // A block = the 128 entries of one (unit or tap, deform group): four rows per thread.
    const int bw = warp - kFirstBuildWarp;
    const TIO *off = (const TIO *)a.offset;
    const TIO *msk = (const TIO *)a.mask;
    const uint32_t dead_off = ((uint32_t)(g.H + 1) * Rb) | kWinFlag;  // an all-zero 2x2 neighbourhood
    const bool dense_planes = g.off_ps == 1 && g.msk_ps == 1 && g.off_cs == plane && g.msk_cs == plane;
    const int wh = tp.win_h, ww = tp.win_w;
    const uint32_t tabw_addr = smem_u32(L.tab_w) + (uint32_t)lane * 8u;
    const uint32_t tabo_addr = smem_u32(L.tab_off) + (uint32_t)lane * 4u;
    bool ok = true;
    PhaseTimer pt(a.counters, blockIdx.x == 0 && bw == 0 && lane == 0);
    const uint32_t nseg = seg_per_stage ? (uint32_t)tp.S : (uint32_t)(tp.KH / tp.tab_span);  // segments per tile

    // Ask L2 for a quarter (this warp's) of the offset and mask planes of tile `nitem` (dense
    // planes only).
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

    uint32_t cur_item = 0xffffffffu;
    TileId2 t = {0, 0, 0, 0, 0};
    int wy0 = 0, wx0 = 0;
    const TIO *offn = nullptr, *mskn = nullptr;
    auto enter_tile = [&](uint32_t item) {
      if (item == cur_item) return;
      cur_item = item;
      t = decode_item2(item, g, tp);
      prefetch_tile(item + gridDim.x);
      wy0 = win_y0(g, tp, t.ho0); wx0 = win_x0(g, tp, t.wo0);
      offn = off ? off + (long long)t.n * g.off_sn : nullptr;
      mskn = msk ? msk + (long long)t.n * g.msk_sn : nullptr;
    };
    // The 128 entries of table block `blk` of slot `slot`: tap (ti, tj) = `tap`, deform group dgi.
    auto do_block = [&](uint32_t slot, uint32_t blk, int tap, int ti, int tj, int dgi) {
      const float tif = (float)(ti * g.dil_h), tjf = (float)(tj * g.dil_w);
      const TIO *ob = off ? offn + ((long long)dgi * 2 * T + 2 * tap) * g.off_cs : nullptr;
      const TIO *mb = msk ? mskn + ((long long)dgi * T + tap) * g.msk_cs : nullptr;
      const uint32_t e0 = slot * slot_entries + blk * kTabStride2;
      // this thread's rows: lane, lane + 32, lane + 64, lane + 96, two at a time (the six loads
      // of a pair in flight together)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t roh[2], row_[2], rmm[2];
        float hbf[2], wbf[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int r = lane + 64 * half + 32 * j;
          const int ho = t.ho0 + (r >> tp.tw_log2), wo = t.wo0 + (r & tw_mask);
          const bool rv = ho < g.Ho && wo < g.Wo;
          // a row beyond the image reads pixel 0 and gets a position that fails the gate
          const long long pix = rv ? (long long)ho * g.Wo + wo : 0;
          hbf[j] = rv ? (float)(ho * g.stride_h - g.pad_h) + tif : -1.0e9f;
          wbf[j] = (float)(wo * g.stride_w - g.pad_w) + tjf;
          roh[j] = 0; row_[j] = 0; rmm[j] = 0;
          if (off) {
            const TIO *pp = ob + pix * g.off_ps;
            roh[j] = ldg_raw_ordered(pp);
            row_[j] = ldg_raw_ordered(pp + g.off_cs);
          }
          if (msk) rmm[j] = ldg_raw_ordered(mb + pix * g.msk_ps);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float4 wt = make_float4(0.f, 0.f, 0.f, 0.f);
          uint32_t eo = dead_off;
          const float h_im = hbf[j] + RawOf<TIO>::to_float(roh[j]);
          const float w_im = wbf[j] + RawOf<TIO>::to_float(row_[j]);
          if (h_im > -1.f && w_im > -1.f && h_im < (float)g.H && w_im < (float)g.W) {
            const float m = msk ? mask_value(g, RawOf<TIO>::to_float(rmm[j])) : 1.f;
            const float hf = floorf(h_im), wf = floorf(w_im);
            const float lh = h_im - hf, lw = w_im - wf;
            const float hh = 1.f - lh, hw = 1.f - lw;
            wt.x = hh * hw * m; wt.y = hh * lw * m; wt.z = lh * hw * m; wt.w = lh * lw * m;
            const int hl = (int)hf, wl = (int)wf;
            // inside the shared-memory window: offset within the window (64 bytes per pixel);
            // else (flagged) the offset within the padded sample
            const uint32_t wy = (uint32_t)(hl - wy0), wx = (uint32_t)(wl - wx0);
            if (kWin && wy < (uint32_t)(wh - 1) && wx < (uint32_t)(ww - 1))
              eo = (wy * (uint32_t)ww + wx) * 64u;
            else
              eo = (((uint32_t)(hl + 1) * Wp + (uint32_t)(wl + 1)) * Cb) | kWinFlag;
          }
          const uint32_t e = e0 + 64u * (uint32_t)half + 32u * (uint32_t)j;
          sts8(tabw_addr + e * 8u, pack_weights2<MODE>(wt.x, wt.y), pack_weights2<MODE>(wt.z, wt.w));
          sts4(tabo_addr + e * 4u, eo);
        }
      }
    };
    prefetch_tile(blockIdx.x);
    if constexpr (kSegStage) {
      // Stage segments: builder warp b owns the segments b, b + 4, ... (counted over all tiles
      // of this block): it alone fills them and hands them over.  (The ring is deeper than the
      // builders are many, so a warp never meets a slot two uses ahead of its last visit.)
      uint32_t item = blockIdx.x, sg = (uint32_t)bw, q = (uint32_t)bw;
      for (;; sg += (uint32_t)kBuildWarps, q += (uint32_t)kBuildWarps) {
        while (item < items && sg >= nseg) { sg -= nseg; item += gridDim.x; }
        if (item >= items || !ok) break;
        enter_tile(item);
        const uint32_t slot = q % (uint32_t)RS;
        pt.lap(1);
        ok = mbar_wait2(tab_empty + 8 * slot, ((q / (uint32_t)RS) & 1u) ^ 1u, 9);
        pt.lap(6);
        if (!ok) break;
        // the segment's two consecutive (half-chunk, tap) units
        const int n_u = min(2, tp.U - 2 * (int)sg);
        int u_hc = (2 * (int)sg) / T, u_tap = 2 * (int)sg - u_hc * T;
        for (int ui = 0; ui < n_u; ++ui) {
          const int c0 = t.grp * g.Cg + u_hc * 32;
          const int dg_lo = c0 / g.cpdg;
          const int nd = (min(c0 + 32, (t.grp + 1) * g.Cg) - 1) / g.cpdg - dg_lo + 1;
          const int ti = u_tap / g.kw;
          for (int d = 0; d < nd; ++d)
            do_block(slot, (uint32_t)(ui * tp.ndu + d), u_tap, ti, u_tap - ti * g.kw, dg_lo + d);
          if (++u_tap == T) { u_tap = 0; ++u_hc; }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(tab_full + 8 * slot);
      }
    } else {
      // Run segments (one block per tap, two slots): every builder warp visits every segment
      // and fills every fourth block of it; all of them hand it over.
      uint32_t q = 0;
      for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
        enter_tile(item);
        for (uint32_t sg = 0; sg < nseg && ok; ++sg, ++q) {
          const uint32_t slot = q & 1u;
          pt.lap(1);
          ok = mbar_wait2(tab_empty + 8 * slot, ((q >> 1) & 1u) ^ 1u, 9);
          pt.lap(6);
          if (!ok) break;
          const int c0 = t.grp * g.Cg + (int)sg * tp.tab_span * 32;
          const int dgi = c0 / g.cpdg;
          for (int tap = bw; tap < T; tap += kBuildWarps) {
            const int ti = tap / g.kw;
            do_block(slot, (uint32_t)tap, tap, ti, tap - ti * g.kw, dgi);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(tab_full + 8 * slot);
        }
      }
    }
    if (!ok) *abort_s = 1;
  } else {
    // ------------------------------ gather ------------------------------
    reg_inc<kRegsGather>();
    // Group gi fills the k-stages gi, gi + 2, ... (counted over all tiles of this block).  A
    // stage is two passes of 64 rows; in a pass a warp covers eight rows and a lane blends the
    // 16 channels {q1, q2} x 8 of one (row, unit): lane = 4 * row + 2 * unit + p.
    const int gw = warp - kFirstGatherWarp;
    const int gi = gw / kWarpsPerGroup, gwl = gw % kWarpsPerGroup;
    const int rr = lane >> 2;          // row within the warp's eight
    const int usel = (lane >> 1) & 1;  // which of the stage's two units
    const int row0 = gwl * 8 + rr;     // pass p: row0 + 64 p
    // Odd rows take their second vector first: the rows of a quarter warp then read (and
    // write) different bank quarters.
    const uint32_t q1 = (uint32_t)(lane & 1) ^ (uint32_t)((rr & 1) << 1), q2 = q1 ^ 2u;
    // operand tile: 16-byte chunk (4 * unit + q) of row r lives at chunk index ^ (r & 7)
    const uint32_t a_row = smem_u32(L.a) + (uint32_t)row0 * 128u;
    const uint32_t a_c1 = ((uint32_t)(4 * usel) + q1) ^ (uint32_t)(row0 & 7);
    const uint32_t a_c2 = ((uint32_t)(4 * usel) + q2) ^ (uint32_t)(row0 & 7);
    const char *xpad = reinterpret_cast<const char *>(a.xpad);
    const uint32_t wbytes = (uint32_t)win_bytes(tp);
    const uint32_t win_rb = (uint32_t)tp.win_w * 64u;
    const uint32_t win_s = smem_u32(L.win);
    const uint32_t tabw_addr = smem_u32(L.tab_w) + (uint32_t)row0 * 8u;
    const uint32_t tabo_addr = smem_u32(L.tab_off) + (uint32_t)row0 * 4u;
    const int KH = tp.KH;
    const uint32_t span = seg_per_stage ? 1u : (uint32_t)tp.tab_span;
    const uint32_t nseg = seg_per_stage ? (uint32_t)tp.S : (uint32_t)KH / span;   // table segments per tile
    const uint32_t dead_o = ((uint32_t)(g.H + 1) * Rb) | kWinFlag;   // an all-zero neighbourhood

    // position: the k-stage (item, s) this group fills next; its unit A = 2 s is (half-chunk
    // hcA, tap tapA); with run segments hcA is half-chunk inrunA of run runA
    uint32_t item = blockIdx.x;
    int s = gi, hcA = 0, tapA = 0;
    uint32_t runA = 0, inrunA = 0;
    uint32_t sa = (uint32_t)gi % (uint32_t)A, pa = ((uint32_t)gi / (uint32_t)A) & 1u;
    // running counts over the tiles of this block: window of (tile, half-chunk 0), table
    // segment of (tile, run 0); table ring position of the current stage (stage segments)
    uint32_t win_base = 0, seg_base = 0;
    uint32_t slotS = (uint32_t)gi % (uint32_t)RS, phS = ((uint32_t)gi / (uint32_t)RS) & 1u;
    // windows / run segments: next one to wait for, next one to hand back
    uint32_t win_acq = 0, win_rel = 0, seg_acq = 0, seg_rel = 0;
    bool ok = true;
    PhaseTimer pt(a.counters, blockIdx.x == 0 && gw == 0 && lane == 0);

    // unit A of stage s of a tile: (hcA, tapA) = divmod(2 s, T), and its run
    auto locate = [&]() {
      hcA = 0; tapA = 2 * s; runA = 0; inrunA = 0;
      while (tapA >= T) {
        tapA -= T; ++hcA;
        if (++inrunA == span) { inrunA = 0; ++runA; }
      }
    };
    // tiles are skipped while the stage index runs past their end
    auto normalise = [&]() {
      while (item < items && s >= tp.S) {
        s -= tp.S;
        item += gridDim.x;
        win_base += (uint32_t)KH;
        seg_base += nseg;
      }
      locate();
    };
    normalise();
    int my_hc = -2;
    uint32_t my_item = 0xffffffffu;
    const char *gbase = nullptr;   // sample + channel bytes of this lane's unit (global)
    uint32_t wbase = 0;            // window buffer of the unit's half-chunk (shared address)
    uint32_t e_fixed = 0;          // table entry of row0 without the stage's (or tap's) part
    bool zero_vec = false;
    const char *sbase = nullptr;
    int grp = 0;

    while (item < items && ok) {
      // ---- what the stage needs: table segment(s), the windows of both its units
      uint32_t hcB = (uint32_t)hcA, runB = runA;
      if (tapA + 1 == T && 2 * s + 1 < tp.U) {
        ++hcB;
        if (inrunA + 1u == span) ++runB;
      }
      if (seg_per_stage) {
        ok = mbar_wait2(tab_full + 8 * slotS, phS, 12);
      } else {
        while (ok && seg_acq <= seg_base + runB) {
          ok = mbar_wait2(tab_full + 8 * (seg_acq & 1u), (seg_acq >> 1) & 1u, 12);
          ++seg_acq;
        }
      }
      if (kWin) {
        while (ok && win_acq <= win_base + hcB) {
          ok = mbar_wait2(win_full + 8 * (win_acq & 1u), (win_acq >> 1) & 1u, 13);
          ++win_acq;
        }
      }
      pt.lap(2);
      if (!ok) break;
      // ---- this lane's unit
      if (item != my_item) {
        my_item = item;
        my_hc = -2;
        const TileId2 t = decode_item2(item, g, tp);
        grp = t.grp;
        sbase = xpad + (unsigned long long)t.n * ((unsigned long long)(g.H + 2) * Rb);
      }
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
        // a unit beyond the tile's last one, or channels beyond the group: zero vectors
        const int c0 = grp * g.Cg + hc * 32;
        zero_vec = key < 0 || hc * 32 + 16 * (int)(lane & 1) >= g.Cg;   // (Cg is a multiple of 8; see issue)
        gbase = sbase + (unsigned long long)(key < 0 ? grp * g.Cg : c0) * 2ull;
        wbase = win_s + ((win_base + (uint32_t)hc) & 1u) * wbytes;
        if (seg_per_stage) e_fixed = (uint32_t)(usel * tp.ndu) * kTabStride2;
        else e_fixed = ((seg_base + run) & 1u) * slot_entries;
      }
      const uint32_t e0 = seg_per_stage ? slotS * slot_entries + e_fixed : e_fixed + (uint32_t)tap * kTabStride2;
      // deform group of each of the two vectors within the unit's set (stage segments; a unit
      // spans several deform groups only when a deform group has fewer than 32 channels)
      uint32_t eq1 = 0, eq2 = 0;
      if (seg_per_stage && tp.ndu > 1 && key >= 0) {
        const int c0 = grp * g.Cg + hc * 32;
        eq1 = (uint32_t)((c0 + 8 * (int)q1) / g.cpdg - c0 / g.cpdg) * kTabStride2;
        eq2 = (uint32_t)((c0 + 8 * (int)q2) / g.cpdg - c0 / g.cpdg) * kTabStride2;
      }
      const bool v1_dead = key < 0 || hc * 32 + 8 * (int)q1 >= g.Cg;
      const bool v2_dead = key < 0 || hc * 32 + 8 * (int)q2 >= g.Cg;
      pt.lap(0);
      ok = mbar_wait2(empty_a + 8 * sa, pa ^ 1u, 8);
      pt.lap(3);
      if (!ok) break;
      const uint32_t stage_row = a_row + sa * (uint32_t)kTileBytes;
#pragma unroll 1
      for (int p = 0; p < 2; ++p) {
        // the vector's entry: weights and offset (both vectors share it unless their deform
        // groups differ)
        const uint32_t e = e0 + (uint32_t)(p * 64);
        const uint32_t dst = stage_row + (uint32_t)(p * 64 * 128);
        // the lane's two vectors, one after the other (they share the entry unless their deform
        // groups differ)
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const uint32_t q = k ? q2 : q1, eq = k ? eq2 : eq1;
          const bool dead = k ? v2_dead : v1_dead;
          uint32_t tok = 0;
          uint4 X[4];
          uint2 w = make_uint2(0u, 0u);
          uint32_t o = dead_o;
          if (!dead) { w = lds8(tabw_addr + (e + eq) * 8u); o = lds4(tabo_addr + (e + eq) * 4u); }
          const bool fg = (o & kWinFlag) != 0u;
          const uint32_t ob = (o & ~kWinFlag) + 16u * q;
          if constexpr (kWin) {
            // The lanes of unit 0 start with the even 64-byte slot of their left/right pair
            // and those of unit 1 with the odd one (the window's row pitch is an even number
            // of slots, so the bottom corners repeat the parity): with the rows' vector order,
            // the eight lanes of a quarter warp cover all 32 banks.
            const bool sw = (((o >> 6) & 1u) != (uint32_t)usel) && !fg;
            if (sw) w = make_uint2(__byte_perm(w.x, 0u, 0x1032), __byte_perm(w.y, 0u, 0x1032));
            const uint32_t sp = wbase + ob;
            const uint32_t sa_ = sw ? sp + 64u : sp, sb_ = sw ? sp : sp + 64u;
            if (!__any_sync(0xffffffffu, fg)) {
              // the usual case: every lane of the warp reads the window
              X[0] = lds16(sa_, tok); X[1] = lds16(sb_, tok);
              X[2] = lds16(sa_ + win_rb, tok); X[3] = lds16(sb_ + win_rb, tok);
            } else {
              const char *b = gbase + ob;
              X[0] = ld16_either(fg, b, sa_, tok); X[1] = ld16_either(fg, b + Cb, sb_, tok);
              X[2] = ld16_either(fg, b + Rb, sa_ + win_rb, tok);
              X[3] = ld16_either(fg, b + Rb + Cb, sb_ + win_rb, tok);
            }
          } else {
            const char *b = gbase + ob;
            X[0] = ld16_global(b, tok); X[1] = ld16_global(b + Cb, tok);
            X[2] = ld16_global(b + Rb, tok); X[3] = ld16_global(b + Rb + Cb, tok);
          }
          uint4 wa = table_weights<MODE>(w);
          wa.x |= tok;  // tok is 0: keeps the blend behind the loads
          uint4 r;
          if constexpr (MODE == kModeBf16) r = blend8_bf16(wa, X[0], X[1], X[2], X[3]);
          else r = blend8_f16(wa, X[0], X[1], X[2], X[3]);
          sts16(dst + ((k ? a_c2 : a_c1) << 4), r);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(full_a + 8 * sa);
      pt.lap(4);
      // ---- hand back what the group is done with, move on by kGroups2 stages
      if (seg_per_stage) {
        if (lane == 0) mbar_arrive(tab_empty + 8 * slotS);
        slotS += (uint32_t)kGroups2;
        while (slotS >= (uint32_t)RS) { slotS -= (uint32_t)RS; phS ^= 1u; }
      }
      sa += (uint32_t)kGroups2;
      while (sa >= (uint32_t)A) { sa -= (uint32_t)A; pa ^= 1u; }
      s += kGroups2;
      if (s < tp.S) {
        tapA += 2 * kGroups2;
        while (tapA >= T) {
          tapA -= T; ++hcA;
          if (++inrunA == span) { inrunA = 0; ++runA; }
        }
      } else {
        normalise();
      }
      const bool more = item < items;
      if (!seg_per_stage) {
        // run segments before the next stage's first unit go back to the builders
        const uint32_t seg_keep = more ? seg_base + runA : seg_acq;
        if (seg_rel < seg_keep) {
          if (lane == 0)
            for (uint32_t i = seg_rel; i < seg_keep; ++i) mbar_arrive(tab_empty + 8 * (i & 1u));
          seg_rel = seg_keep;
        }
      }
      if (kWin) {
        // windows before the next stage's first unit go back to the loader (the loads from
        // them have returned: their values were consumed above)
        const uint32_t win_keep = more ? win_base + (uint32_t)hcA : win_acq;
        if (win_rel < win_keep) {
          if (lane == 0)
            for (uint32_t i = win_rel; i < win_keep; ++i) mbar_arrive(win_empty + 8 * (i & 1u));
          win_rel = win_keep;
        }
      }
    }
    (void)zero_vec;
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
