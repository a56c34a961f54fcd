// Second-generation tensor-core kernel of the deformable-convolution forward (16-bit
// operands: bf16 or fp16) for sm_100a.
//
// Same contraction as dcn_fwd_tc (out[p, co] = sum_k A[p, k] * Wt[co, k], A never written to
// global memory; it replaces the gather kernel, the per-sample GEMM loop and the bias pass of
// mmcv/ops/csrc/common/cuda/modulated_deform_conv_cuda_kernel.cuh:186-245 and
// mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:108-137), with a different producer side:
//
//   * gather warps (16, in two groups that fill alternate k-stages): a warp covers 16 rows of
//     a stage, i.e. 32 (row, unit) pairs, and each of its lanes owns ONE of them: it turns the
//     pair's offsets and mask into a tap entry -- four 16-bit corner weights with the
//     modulation folded in, and the byte offset of the top-left corner -- one own stage ahead,
//     from loads issued another stage earlier, and then fetches the four corners of the unit's
//     four 16-byte vectors, blends them on packed 16-bit FMAs and writes the 128-byte-swizzled
//     operand tile tcgen05.mma reads.  An entry never leaves its lane and no tap table exists
//     in memory.  Everything else a unit needs comes from a small lookup table built once per
//     block (tap displacement, offset / mask channel, half-chunk, channel byte offset).  The input is a
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
//     left/right corners a lane reads first depends on the slot's parity and the order of its
//     four vectors on the row number, so that the eight lanes of a quarter warp never meet in
//     a bank, neither reading the window nor writing the swizzled operand rows), the others
//     from the padded copy in global memory, whose lines the lane requested when it built the
//     entry.
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
constexpr int kWinWarp = 6;   // (warp 7 idles)
constexpr int kFirstGatherWarp = 8;
constexpr int kGatherWarps = 16;
constexpr int kThreads2 = (kFirstGatherWarp + kGatherWarps) * 32;  // 768: six warps per scheduler, 80 registers per thread
constexpr int kGroups2 = 2;                              // gather groups; group i fills k-stages i, i + 2, ...
constexpr int kWarpsPerGroup = kGatherWarps / kGroups2;  // 8 warps x 16 rows: the 128 rows of a stage

// Register budget per role (setmaxnreg works on warpgroups of four consecutive warps; the
// block starts with 80 registers per thread): the two warpgroups that hold the epilogue and the
// MMA / loader warps give registers back, the four gather warpgroups take them.
constexpr int kRegsLight = 64, kRegsGather = 88;
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

// Offsets and mask elements are read once: they bypass L1, which is left to the prefetched
// corner runs of the samples outside the window.
__device__ __forceinline__ uint32_t ldg_raw_stream(const float *p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.b32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_raw_stream(const __nv_bfloat16 *p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_raw_stream(const __half *p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ void prefetch_l1(const void *p) {
  asm volatile("prefetch.global.L1 [%0];" ::"l"(p));
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
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
  return r;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t r;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r) : "r"(addr));
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
__device__ __forceinline__ void sts16(uint32_t addr, const uint4 &v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}


// Shared memory: a control block first (barriers, tensor-memory slot, abort flag, the
// wait limit and the status pointer: at fixed offsets, so that the out-of-line slow path of a
// wait finds them without arguments), then the rings.
constexpr uint32_t kCtrlBytes = 4096;   // 1 KiB of fixed fields and barriers, then the two lookup tables
constexpr uint32_t kCtrlTmemSlot = 512, kCtrlAbort = 520, kCtrlLimit = 528, kCtrlStatus = 536;
// lookup tables (built once per block): tap -> sampling displacement (dy, dx) as floats, and
// (conv group, half-chunk) -> deform group
constexpr uint32_t kLutBytes = 3072;   // the K-unit table: 16 bytes x 2 S entries x conv groups

struct Smem2 {
  uint8_t *a, *b, *win;
  uint8_t *epi;        // staging of the epilogue's tensor stores
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
  L.bias_s = (uint8_t *)(((uintptr_t)p + 15) & ~(uintptr_t)15);
  return L;
}

// Continuation of a wait (kept out of the fast path): polls until the phase completes, the block aborts or the
// time limit passes (then it raises the abort flag and records `code` in the status word).
__device__ __forceinline__ bool mbar_wait_slow2(uint32_t bar, uint32_t parity, int code, int backoff) {
  uint8_t *ctrl = smem_aligned();
  volatile int *abort_s = (volatile int *)(ctrl + kCtrlAbort);
  // The tensor-core issuer sits in the middle of every dependency chain (codes 4-6): its waits
  // run out after the limit, everybody else's after twice the limit, so that the recorded code
  // names the hand-over nearest to the producer that went missing.
  // (the timer is first read at the sixteenth poll: short waits, the usual case, never pay for it)
  unsigned long long t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (backoff) __nanosleep((unsigned)backoff);
    if ((it & 15u) == 0u) {
      if (*abort_s) return false;
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      unsigned long long limit = *(const unsigned long long *)(ctrl + kCtrlLimit);
      if (code < 4 || code > 6) limit *= 2;
      if (now - t0 > limit) {
        *abort_s = 1;
        atomicCAS(*(int **)(ctrl + kCtrlStatus), 0, code);
        return false;
      }
    }
  }
}
// Bounded wait.  Returns false when the block is aborting.
// Sleep between the polls of a wait, in ns, by role (0: poll back to back).  try_wait already
// suspends the thread in hardware for a while; the sleep keeps the waiting roles from taking issue
// slots from the gather warps.
#ifndef DCN_TC2_BACKOFF
#define DCN_TC2_BACKOFF 100
#endif
#ifndef TC2_BO_EPI
#define TC2_BO_EPI 200
#endif
#ifndef TC2_BO_MMA
#define TC2_BO_MMA 0
#endif
#ifndef TC2_BO_LOAD
#define TC2_BO_LOAD DCN_TC2_BACKOFF
#endif
#ifndef TC2_BO_GATHER
#define TC2_BO_GATHER DCN_TC2_BACKOFF
#endif
__device__ __forceinline__ bool mbar_wait2(uint32_t bar, uint32_t parity, int code, int backoff = DCN_TC2_BACKOFF) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow2(bar, parity, code, backoff);
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
  s += (size_t)2 * tp.BN * tp.io_bytes + 32;  // bias staging, one copy per accumulator buffer
  return s;
}

template <typename TIO, int MODE, bool kWin>
__global__ void __launch_bounds__(kThreads2, 1) dcn_fwd_tc2(const __grid_constant__ Tc2Args a) {
  uint8_t *smem = smem_aligned();
  const Geom &g = a.g;
  const TcPlan &tp = a.tp;
  const Smem2 L = carve2(smem, tp);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int A = tp.a_stages, B = tp.b_stages;
  const uint32_t bar0 = smem_u32(smem);
  // barrier i lives at bar0 + 8*i
  const uint32_t full_a = bar0, empty_a = full_a + 8 * A, full_b = empty_a + 8 * A,
                 empty_b = full_b + 8 * B, tmem_full = empty_b + 8 * B, tmem_empty = tmem_full + 16,
                 win_full = tmem_empty + 16, win_empty = win_full + 16;
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
    *abort_s = 0;
    *(unsigned long long *)(smem + kCtrlLimit) = a.wait_limit_ns;
    *(int **)(smem + kCtrlStatus) = a.status;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  {
    // One 16-byte entry per (conv group, K unit u = half-chunk * T + tap), 2 S entries per group:
    // tap displacement (dy, dx) as floats; channel of the unit's y-offset plane | channel of its
    // mask plane << 16; half-chunk | exists << 8 | byte offset of the unit's first channel
    // inside a pixel << 9.
    uint4 *lut = reinterpret_cast<uint4 *>(smem + 1024);
    const int per_grp = 2 * tp.S;
    for (int i = threadIdx.x; i < g.groups * per_grp; i += blockDim.x) {
      const int grp = i / per_grp, u = i - grp * per_grp;
      const bool exists = u < tp.U;
      const int hc = exists ? u / g.T : 0, tap = exists ? u - hc * g.T : 0;
      const int ti = tap / g.kw, tj = tap - ti * g.kw;
      const int c0 = grp * g.Cg + hc * 32;
      const int dgi = c0 / g.cpdg;
      uint4 e;
      e.x = __float_as_uint((float)(ti * g.dil_h));
      e.y = __float_as_uint((float)(tj * g.dil_w));
      e.z = (uint32_t)(dgi * 2 * g.T + 2 * tap) | ((uint32_t)(dgi * g.T + tap) << 16);
      e.w = (uint32_t)hc | (exists ? 256u : 0u) | ((uint32_t)(c0 * 2) << 9);
      lut[i] = e;
    }
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
  // consecutive units (64 bytes each of the operand row).  A unit lies inside one deform group.
  const uint32_t Wp = (uint32_t)g.W + 2u;
  const uint32_t Cb = (uint32_t)g.C * 2u;       // bytes of one padded pixel
  const uint32_t Rb = Wp * Cb;                  // bytes of one padded row

  if (warp < kFirstGatherWarp) {
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
    StageTimer pt(a.counters, blockIdx.x == 0 && threadIdx.x == 0);
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
      bool ok = mbar_wait2(tmem_full + 8 * buf, par, 3, TC2_BO_EPI);
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
#ifdef DCN_TC2_ABLATE
      if (a.debug_flags & 32) {
        uint32_t r[16];
        tmem_ld16(taddr, r);
        tmem_ld_wait();
      } else
#endif
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
    StageTimer pt(a.counters, blockIdx.x == 0 && lane == 0);
    for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x, ++li) {
      const int buf = (int)(li & 1);
      const uint32_t par = (li >> 1) & 1u;
      pt.lap(11);
      ok = __all_sync(0xffffffffu, mbar_wait2(tmem_empty + 8 * buf, par ^ 1u, 4, TC2_BO_MMA));
      if (!ok) break;
      pt.lap(10);
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)(buf * tp.BN);
      for (int ks = 0; ks < tp.S; ++ks) {
        ok = __all_sync(0xffffffffu, mbar_wait2(full_b + 8 * sb, pb, 5, TC2_BO_MMA));
        if (!ok) break;
        pt.lap(8);
        ok = __all_sync(0xffffffffu, mbar_wait2(full_a + 8 * sa, pa, 6, TC2_BO_MMA));
        if (!ok) break;
        pt.lap(9);
        tc_fence_after();
        const uint64_t adesc = smem_desc_sw128(smem_u32(L.a) + sa * (uint32_t)kTileBytes);
        const uint64_t bdesc = smem_desc_sw128(smem_u32(L.b) + sb * b_stage_bytes);
        if (elect_one()) {
#ifdef DCN_TC2_ABLATE
          if (!(a.debug_flags & 64))
#endif
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
      StageTimer pt(a.counters, blockIdx.x == 0);
      for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const uint32_t rem = item % per_mt;
        const uint8_t *src = a.wtiles + (size_t)rem * tp.S * b_stage_bytes;
        for (int ks = 0; ks < tp.S; ++ks) {
          pt.lap(15);
          ok = mbar_wait2(empty_b + 8 * sb, pb ^ 1u, 7, TC2_BO_LOAD);
          if (!ok) break;
          pt.lap(14);
          const bool withhold = (a.debug_flags & 1) && item + gridDim.x >= items && ks == tp.S - 1;
#ifdef DCN_TC2_ABLATE
          if (a.debug_flags & 512) {
            mbar_arrive(full_b + 8 * sb);
          } else
#endif
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
          ok = mbar_wait2(win_empty + 8 * wb, ((wq >> 1) & 1u) ^ 1u, 11, TC2_BO_LOAD);
          if (!ok) break;
#ifdef DCN_TC2_ABLATE
          if (a.debug_flags & 1024) { mbar_arrive(win_full + 8 * wb); continue; }
#endif
          mbar_arrive_expect_tx(win_full + 8 * wb, wbytes);
          // coordinates in the padded tensor: (channel, column + 1, row + 1, sample)
          tma_load_4d(smem_u32(L.win) + wb * wbytes, &a.win_map, t.grp * g.Cg + hc * 32,
                      win_x0(g, tp, t.wo0) + 1, win_y0(g, tp, t.ho0) + 1, t.n, win_full + 8 * wb);
        }
      }
    }
    __syncwarp();
  }
  } else {
    // ------------------------------ gather ------------------------------
    reg_inc<kRegsGather>();
    // Group gi fills the k-stages gi, gi + 2, ... (counted over all tiles of this block).  In a
    // stage a warp covers sixteen rows and a lane owns one (row, unit): lane = 2 * row + unit.
    // It computes that pair's tap entry a stage ahead (from offset / mask elements loaded a stage
    // before that) and then blends the unit's 32 channels, four 16-byte vectors, itself: no
    // entry ever leaves its lane.
    const int gw = warp - kFirstGatherWarp;
    const int gi = gw / kWarpsPerGroup, gwl = gw % kWarpsPerGroup;
    const int rr = lane >> 1;          // row within the warp's sixteen
    const int usel = lane & 1;         // which of the stage's two units
    const int row0 = gwl * 16 + rr;    // this lane's row of the tile
    const int brow = row0;             // (the row whose entry this lane builds: its own)
    // Vector order.  A lane walks the unit's four 16-byte vectors in the order q0 ^ k, k = 0..3,
    // with q0 = sigma(row & 3), sigma = (0, 3, 1, 2).  Both r -> sigma(r) and r -> sigma(r) ^ r
    // are permutations of 0..3, so among the four rows of a quarter warp the vectors read in one
    // instruction differ (window reads: bank quarter = slot parity * 4 + vector) and so do the
    // swizzled chunks written (chunk = (4 * unit + vector) ^ (row & 7)): no bank conflicts on
    // either side.
    const uint32_t q0 = (0x9cu >> (2 * (rr & 3))) & 3u;   // sigma packed two bits per entry: 0, 3, 1, 2
    // operand tile: 16-byte chunk (4 * unit + q) of row r lives at chunk index ^ (r & 7)
    const uint32_t a_row = smem_u32(L.a) + (uint32_t)row0 * 128u;
    const uint32_t a_c0 = (((uint32_t)(4 * usel) + q0) ^ (uint32_t)(row0 & 7)) << 4;   // vector k: a_c0 ^ (k << 4)
    const char *xpad = reinterpret_cast<const char *>(a.xpad);
    const TIO *off = (const TIO *)a.offset;
    const TIO *msk = (const TIO *)a.mask;
    const uint32_t wbytes = (uint32_t)win_bytes(tp);
    const uint32_t win_rb = (uint32_t)tp.win_w * 64u;
    const uint32_t win_s = smem_u32(L.win);
    const int KH = tp.KH;

    const uint32_t lut_s = smem_u32(smem + 1024);
    const uint32_t lut_grp_bytes = (uint32_t)(2 * tp.S) * 16u;
    const uint32_t off_cs = (uint32_t)g.off_cs, msk_cs = (uint32_t)g.msk_cs;   // (a sample's planes hold < 2^31 elements)
    // ---- position of a k-stage: tile and stage in the tile (its units are 2 s and 2 s + 1)
    struct Pos {
      uint32_t item;
      int s;
    };
    uint32_t tiles_done = 0;   // tiles the position `nxt` has left behind
    auto locate = [&](Pos &p) {
      while (p.item < items && p.s >= tp.S) {
        p.s -= tp.S;
        p.item += gridDim.x;
        ++tiles_done;
      }
    };
    auto advance = [&](Pos &p) {   // to the group's next stage
      p.s += kGroups2;
      locate(p);
    };
    // ---- the tile of position `nxt`, decoded when it changes: what the entry of this lane's
    // (row, unit) needs, and what the gather of that tile needs later
    uint32_t t_item = 0xffffffffu;
    uint32_t t_lut = lut_s;                 // the tile's conv group in the unit table
    int t_wy0 = 0, t_wx0 = 0;
    const char *t_sbase = nullptr;          // the tile's sample in the padded copy
    const TIO *t_off = nullptr, *t_msk = nullptr;   // the sample's offsets / masks at this lane's pixel
    float t_hb = -1.0e9f, t_wb = 0.f;       // this lane's row: sampling position without tap and offset
    auto enter_tile = [&](uint32_t item) {
      t_item = item;
      const TileId2 t = decode_item2(item, g, tp);
      t_lut = lut_s + (uint32_t)t.grp * lut_grp_bytes;
      t_wy0 = win_y0(g, tp, t.ho0); t_wx0 = win_x0(g, tp, t.wo0);
      t_sbase = xpad + (unsigned long long)t.n * ((unsigned long long)(g.H + 2) * Rb);
      const int ho = t.ho0 + (brow >> tp.tw_log2), wo = t.wo0 + (brow & tw_mask);
      const bool rv = ho < g.Ho && wo < g.Wo;
      // a row beyond the image gets a position that fails the sampling gate, and reads pixel 0
      const long long pix = rv ? (long long)ho * g.Wo + wo : 0;
      t_hb = rv ? (float)(ho * g.stride_h - g.pad_h) : -1.0e9f;
      t_wb = (float)(wo * g.stride_w - g.pad_w);
      t_off = off ? off + (long long)t.n * g.off_sn + pix * g.off_ps : nullptr;
      t_msk = msk ? msk + (long long)t.n * g.msk_sn + pix * g.msk_ps : nullptr;
    };
    // ---- the entry this lane builds for the stage at position p: loads issued by entry_loads,
    // consumed by entry_build one own stage later
    uint32_t roh = 0, row_ = 0, rmm = 0;   // raw offset (y, x) and mask elements
    float bh = -1.0e9f, bw_ = 0.f;          // sampling position without the offset
    uint32_t n_misc = 0;                    // the unit's table word 3 (half-chunk, exists, channel byte offset)
    uint32_t n_hcA = 0, n_hcB = 0;          // half-chunks of the stage's first and last existing unit
    auto entry_loads = [&](const Pos &p) {
      roh = 0; row_ = 0; rmm = 0; bh = -1.0e9f; bw_ = 0.f; n_misc = 0;
      if (p.item >= items) return;
      if (p.item != t_item) enter_tile(p.item);
      const uint32_t ea = t_lut + (uint32_t)p.s * 32u;     // unit 2 s; unit 2 s + 1 follows
      const uint4 e = lds128(ea + (uint32_t)usel * 16u);
      const uint32_t mA = lds32(ea + 12u), mB = lds32(ea + 28u);
      n_hcA = mA & 255u;
      n_hcB = (mB & 256u) ? (mB & 255u) : n_hcA;
      n_misc = e.w;
      if (!(e.w & 256u)) return;            // no such unit: a dead entry
#ifdef DCN_TC2_ABLATE
      if (a.debug_flags & 4) return;        // (timing experiment: bookkeeping only, no element loads)
#endif
      bh = t_hb + __uint_as_float(e.x);
      bw_ = t_wb + __uint_as_float(e.y);
      if (off) {
        const TIO *pp = t_off + (e.z & 0xffffu) * off_cs;
        roh = ldg_raw_stream(pp);
        row_ = ldg_raw_stream(pp + off_cs);
      }
      if (msk) rmm = ldg_raw_stream(t_msk + (e.z >> 16) * msk_cs);
    };
    // the entry: weights (w00 w01 | w10 w11), offset of the top-left corner within the padded
    // sample, and within the shared-memory window (kNoWin: the neighbourhood is not inside it)
    // (kDeadWin: the sample contributes nothing -- its position fails the sampling gate, or the
    // unit does not exist; the gather then stores zeros without reading anything)
    constexpr uint32_t kNoWin = 0xffffffffu, kDeadWin = 0xfffffffeu;
    const uint32_t dead_g = (uint32_t)(g.H + 1) * Rb;   // an all-zero neighbourhood
    uint32_t ew0 = 0, ew1 = 0, eog = dead_g, eow = kDeadWin;
    auto entry_build = [&]() {
      // (runs before the loads of the stage after it: t_wy0 / t_wx0 / t_sbase still belong to this entry's tile)
      ew0 = 0; ew1 = 0; eog = dead_g; eow = kDeadWin;
      const float h_im = bh + RawOf<TIO>::to_float(roh);
      const float w_im = bw_ + RawOf<TIO>::to_float(row_);
      if (h_im > -1.f && w_im > -1.f && h_im < (float)g.H && w_im < (float)g.W) {
        const float m = msk ? mask_value(g, RawOf<TIO>::to_float(rmm)) : 1.f;
        const float hf = floorf(h_im), wf = floorf(w_im);
        const float lh = h_im - hf, lw = w_im - wf;
        const float hh = 1.f - lh, hw = 1.f - lw;
        ew0 = pack_weights2<MODE>(hh * hw * m, hh * lw * m);
        ew1 = pack_weights2<MODE>(lh * hw * m, lh * lw * m);
        const int hl = (int)hf, wl = (int)wf;
        eog = ((uint32_t)(hl + 1) * Wp + (uint32_t)(wl + 1)) * Cb;
        eow = kNoWin;
        if (kWin) {
          const uint32_t wy = (uint32_t)(hl - t_wy0), wx = (uint32_t)(wl - t_wx0);
          if (wy < (uint32_t)(tp.win_h - 1) && wx < (uint32_t)(tp.win_w - 1)) {
            eow = (wy * (uint32_t)tp.win_w + wx) * 64u;
          } else {
            // outside the window (rare): this lane will read the
            // padded copy a stage from now; ask for its four 64-byte corner runs now
            const char *b = t_sbase + (n_misc >> 9) + eog;
            prefetch_l1(b); prefetch_l1(b + 32); prefetch_l1(b + Cb); prefetch_l1(b + Cb + 32);
            prefetch_l1(b + Rb); prefetch_l1(b + Rb + 32); prefetch_l1(b + Rb + Cb); prefetch_l1(b + Rb + Cb + 32);
          }
        }
      }
    };

    Pos cur;
    cur.item = blockIdx.x; cur.s = gi;
    locate(cur);
    uint32_t sa = (uint32_t)gi % (uint32_t)A, pa = ((uint32_t)gi / (uint32_t)A) & 1u;
    uint32_t win_acq = 0, win_rel = 0;   // windows: next one to wait for, next one to hand back
    bool ok = true;
    StageTimer pt(a.counters, blockIdx.x == 0 && gw == 0 && lane == 0);
    // the first stage's entry
    entry_loads(cur);
    entry_build();
    // what the gather of the current stage needs: its tile (copied from the decoded tile when
    // `cur` enters it) and its units' table words (loaded with the entry a stage earlier)
    uint32_t c_item = cur.item, c_win_base = tiles_done * (uint32_t)KH;
    const char *c_sbase = t_sbase;
    uint32_t c_misc = n_misc, c_hcA = n_hcA, c_hcB = n_hcB;
    const bool ragged = (g.Cg & 31) != 0;   // the last half-chunk of a group is partly beyond its channels
    Pos nxt = cur;
    if (cur.item < items) advance(nxt);
    entry_loads(nxt);

    while (cur.item < items && ok) {
      // ---- this lane's unit of the stage
      const uint32_t hc = c_misc & 255u;
      const char *gbase = c_sbase + (c_misc >> 9);
      const uint32_t wbase = win_s + ((c_win_base + hc) & 1u) * wbytes;
      // vectors beyond the unit's channels (a group whose size is not a multiple of 32) are zero;
      // a unit that does not exist has a dead entry and needs nothing here
      const int cg_left = ragged ? g.Cg - (int)hc * 32 : 32;   // channels of the unit inside the group
      // ---- the windows of both units of the stage (unit B's is the later one)
      if (kWin) {
        while (ok && win_acq <= c_win_base + c_hcB) {
          ok = mbar_wait2(win_full + 8 * (win_acq & 1u), (win_acq >> 1) & 1u, 13, TC2_BO_GATHER);
          ++win_acq;
        }
      }
      pt.lap(2);
      if (!ok) break;
      ok = mbar_wait2(empty_a + 8 * sa, pa ^ 1u, 8, TC2_BO_GATHER);
      pt.lap(3);
      if (!ok) break;
      const uint32_t stage_row = a_row + sa * (uint32_t)kTileBytes;
#ifdef DCN_TC2_ABLATE
      const int abl = a.debug_flags;
#else
      constexpr int abl = 0;
#endif
      if (!(abl & 16)) {
        const uint32_t dst = stage_row;
        const uint32_t w0 = ew0, w1 = ew1;
        if constexpr (kWin) {
          // The four corner vectors come from the window; a lane whose neighbourhood lies outside
          // it (rare; it asked for those lines when it built the entry) reads the padded copy
          // instead, and a dead sample reads the window's first pixel and stores zeros.  The lanes
          // of unit 0 start with the even 64-byte slot of their left/right pair and those of unit
          // 1 with the odd one (the window's row pitch is an even number of slots, so the bottom
          // corners repeat the parity).
          uint32_t ow = eow;
          bool miss = ow == kNoWin;
          if (abl & 256) miss = false;
          const bool dead = ow == kDeadWin;
          if (ow >= kDeadWin) ow = 0;
          const bool sw = !miss && ((ow >> 6) & 1u) != (uint32_t)usel;
          const uint32_t v0 = sw ? __byte_perm(w0, 0u, 0x1032) : w0;
          const uint32_t v1 = sw ? __byte_perm(w1, 0u, 0x1032) : w1;
          const uint32_t sp = wbase + ow;
          const uint32_t s1 = sw ? sp + 64u : sp, s2 = sw ? sp : sp + 64u;
          const char *gb = gbase + eog;
          const uint4 wa0 = table_weights<MODE>(make_uint2(v0, v1));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t q = q0 ^ (uint32_t)k;
            const uint32_t q16 = 16u * q;
            uint32_t tok = 0;
            uint4 X[4];
            if (abl & 2) {
              X[0] = X[1] = X[2] = X[3] = make_uint4(w0, w1, ow, q16);
            } else if (miss) {
              const char *b = gb + q16;
              X[0] = ld16_global(b, tok); X[1] = ld16_global(b + Cb, tok);
              X[2] = ld16_global(b + Rb, tok); X[3] = ld16_global(b + Rb + Cb, tok);
            } else {
              X[0] = lds16(s1 + q16, tok); X[1] = lds16(s2 + q16, tok);
              X[2] = lds16(s1 + win_rb + q16, tok); X[3] = lds16(s2 + win_rb + q16, tok);
            }
            uint4 wa = wa0;
            wa.x |= tok;  // tok is 0: keeps the blend behind the loads
            uint4 r;
            if (abl & 8) r = X[0];
            else if constexpr (MODE == kModeBf16) r = blend8_bf16(wa, X[0], X[1], X[2], X[3]);
            else r = blend8_f16(wa, X[0], X[1], X[2], X[3]);
            if (dead || 8 * (int)q >= cg_left) r = make_uint4(0u, 0u, 0u, 0u);
            if (!(abl & 128)) sts16(dst + (a_c0 ^ ((uint32_t)k << 4)), r);
          }
        } else {
          // no window: every lane reads the padded copy in global memory (a dead sample reads the
          // all-zero neighbourhood with zero weights)
          const char *gb = gbase + eog;
          const uint4 wa0 = table_weights<MODE>(make_uint2(w0, w1));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t q = q0 ^ (uint32_t)k;
            const char *b = gb + 16u * q;
            uint32_t tok = 0;
            uint4 X[4];
            X[0] = ld16_global(b, tok); X[1] = ld16_global(b + Cb, tok);
            X[2] = ld16_global(b + Rb, tok); X[3] = ld16_global(b + Rb + Cb, tok);
            uint4 wa = wa0;
            wa.x |= tok;
            uint4 r;
            if constexpr (MODE == kModeBf16) r = blend8_bf16(wa, X[0], X[1], X[2], X[3]);
            else r = blend8_f16(wa, X[0], X[1], X[2], X[3]);
            if (8 * (int)q >= cg_left) r = make_uint4(0u, 0u, 0u, 0u);
            sts16(dst + (a_c0 ^ ((uint32_t)k << 4)), r);
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(full_a + 8 * sa);
      pt.lap(4);
      // ---- the next stage: its entry from the loads issued a stage ago, then the loads of the
      // stage after it
      if (!(abl & 4)) entry_build();
      sa += (uint32_t)kGroups2;
      while (sa >= (uint32_t)A) { sa -= (uint32_t)A; pa ^= 1u; }
      cur = nxt;
      c_misc = n_misc; c_hcA = n_hcA; c_hcB = n_hcB;
      if (cur.item != c_item && cur.item < items) {
        // (`nxt` entered this tile a stage ago: the decoded tile is this one)
        c_item = cur.item;
        c_win_base = tiles_done * (uint32_t)KH;
        c_sbase = t_sbase;
      }
      if (nxt.item < items) advance(nxt);
      entry_loads(nxt);
      if (kWin) {
        // windows before the next stage's first unit go back to the loader (the loads from
        // them have returned: their values were consumed above)
        const uint32_t win_keep = cur.item < items ? c_win_base + c_hcA : win_acq;
        if (win_rel < win_keep) {
          if (lane == 0)
            for (uint32_t i = win_rel; i < win_keep; ++i) mbar_arrive(win_empty + 8 * (i & 1u));
          win_rel = win_keep;
        }
      }
      pt.lap(0);
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

template <typename TIO, int MODE, bool kWin>
cudaError_t launch_one2(const Tc2Args &a, const TcPlan &tp, cudaStream_t s) {
  auto kern = dcn_fwd_tc2<TIO, MODE, kWin>;
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
  const bool win = tp.win_h > 0;
  if (dtype == DCN_DTYPE_F32)
    return win ? launch_one2<float, kModeBf16, true>(a, tp, s) : launch_one2<float, kModeBf16, false>(a, tp, s);
  if (dtype == DCN_DTYPE_F16)
    return win ? launch_one2<__half, kModeF16, true>(a, tp, s) : launch_one2<__half, kModeF16, false>(a, tp, s);
  return win ? launch_one2<__nv_bfloat16, kModeBf16, true>(a, tp, s)
             : launch_one2<__nv_bfloat16, kModeBf16, false>(a, tp, s);
}

}  // namespace dcn
