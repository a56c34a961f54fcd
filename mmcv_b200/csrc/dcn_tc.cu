// Tensor-core path of the deformable-convolution forward for sm_100a.
//
// One persistent kernel computes out[p, co] = sum_k A[p, k] * Wt[co, k] as an implicit
// GEMM whose A operand (the reference's "columns",
// mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:101-112) is never written to global
// memory: producer warps sample the input with the learned offsets (bilinear, four
// corners, modulation mask folded into the corner weights), write bf16 operand tiles
// straight into shared memory in the 128-byte-swizzled K-major layout tcgen05.mma reads,
// and one thread issues tcgen05.mma (kind::f16, fp32 accumulation in tensor memory).
// Weight tiles arrive through the bulk-copy engine (cp.async.bulk + mbarrier
// complete_tx) from a pre-swizzled image; four epilogue warps read the accumulator with
// tcgen05.ld, add the bias and store NCHW rows.  It replaces the gather kernel, the
// per-sample cuBLAS GEMM loop and the bias pass of the reference
// (mmcv/ops/csrc/common/cuda/modulated_deform_conv_cuda_kernel.cuh:186-245,
//  mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:108-137).
//
// K is ordered (64-channel chunk, tap, channel-in-chunk); the weight image is permuted
// to match, so the order is invisible outside this file.
//
// Every wait on an mbarrier is bounded: after kWaitLimitNs the waiting thread raises a
// block-wide abort flag, records a code in the status word and every role leaves its
// loop; tensor memory is released on every exit path.
#include <atomic>
#include <climits>

#include "dcn_internal.cuh"
#include "dcn_ptx.cuh"

namespace dcn {

namespace {

constexpr int kEpilogueWarps = 4;
constexpr int kMmaWarp = 4;
constexpr int kLoadWarp = 5;
constexpr int kFirstProducerWarp = 6;

// Arithmetic modes of the contraction.
//  kModeBf16:   bf16 operands, one operand tile per stage, 64 channels per stage;
//  kModeF16:    the same with fp16 operands;
//  kModeTf32x3: fp32 data split into a TF32 high part and a remainder (a = hi + lo, both
//               held as fp32 bit patterns; the tensor core reads their top 19 bits), two
//               operand tiles per stage, 32 channels per stage, three MMAs per k-step:
//               hi*hi + lo*hi + hi*lo with fp32 accumulation.
template <int MODE> struct ModeTraits;
template <> struct ModeTraits<kModeBf16> {
  using TabW = uint2;  // table entry: four 16-bit corner weights
  static constexpr int kCh = 64, kCpv = 8, kEsz = 2, kTiles = 1;
};
template <> struct ModeTraits<kModeF16> {
  using TabW = uint2;
  static constexpr int kCh = 64, kCpv = 8, kEsz = 2, kTiles = 1;
};
template <> struct ModeTraits<kModeTf32x3> {
  using TabW = uint4;  // table entry: four fp32 corner weights
  static constexpr int kCh = 32, kCpv = 4, kEsz = 4, kTiles = 2;
};

struct TcArgs {
  Geom g;
  TcPlan tp;
  const void *xcl;           // channels-last input [N, H, W, C], bf16 or fp32 by mode
  const uint8_t *wtiles;     // pre-swizzled weight stages
  const void *offset, *mask, *bias;
  void *output;
  int *status;
  unsigned long long *counters;  // optional phase timers (block 0 only), or nullptr
};

constexpr int kRowInvalid = INT_MIN;
// Entries of one (tap, deform group) block of the tap table: the rows plus a skew of four, so
// that the blocks of two deform groups read by one warp fall into different banks.
constexpr int kTabStride = kBM + 4;
// (tap, deform group) blocks of the tap table: all taps, or, when every producer group keeps a
// table of its own taps (producer_cfg thousands digit & 2), groups x ceil(taps / groups).
// bytes of a table entry's corner weights: four 16-bit values, or four fp32 for TF32x3
__host__ __device__ inline size_t tab_weight_bytes(const TcPlan &tp) { return tp.op_format == 2 ? 16 : 8; }
__host__ __device__ inline int tab_blocks(const TcPlan &tp, int T) {
  const int G = (tp.producer_cfg / 100) % 10;
  const bool own = ((tp.producer_cfg / 1000) & 2) != 0;
  return (own ? G * ((T + G - 1) / G) : T) * tp.ndgc;
}

struct SmemLayout {
  uint8_t *a, *b;
  uint8_t *tab_w;      // four corner weights per (tap, deform group, row): 8 or 16 bytes each
  uint32_t *tab_off;   // byte offset of the top-left corner from the sample's base
  int *row_h, *row_w, *row_pix;
  uint64_t *bars;
  uint32_t *tmem_slot;
  int *abort_flag;
  uint8_t *bias_s;     // bias of the tile's output channels in the tensors' type, two copies (tile parity)
};

__device__ __forceinline__ SmemLayout carve(uint8_t *base, const TcPlan &tp, int T) {
  SmemLayout L;
  uint8_t *p = base;
  L.a = p; p += (size_t)tp.a_stages * tp.tiles_per_stage * kTileBytes;
  L.b = p; p += (size_t)tp.b_stages * tp.tiles_per_stage * tp.BN * 128;
  L.tab_w = p; p += (size_t)tab_blocks(tp, T) * kTabStride * tab_weight_bytes(tp);
  L.tab_off = (uint32_t *)p; p += (size_t)tab_blocks(tp, T) * kTabStride * sizeof(uint32_t);
  L.row_h = (int *)p; p += kBM * sizeof(int);
  L.row_w = (int *)p; p += kBM * sizeof(int);
  L.row_pix = (int *)p; p += kBM * sizeof(int);
  L.bars = (uint64_t *)p; p += (size_t)(2 * tp.a_stages + 2 * tp.b_stages + 8) * sizeof(uint64_t);
  L.tmem_slot = (uint32_t *)p; p += 8;
  L.abort_flag = (int *)p; p += 8;
  L.bias_s = (uint8_t *)(((uintptr_t)p + 15) & ~(uintptr_t)15);
  return L;
}

}  // namespace

size_t tc_smem_bytes(const TcPlan &tp, int T) {
  size_t s = 1024;  // slack for manual 1024-byte alignment
  s += (size_t)tp.tiles_per_stage * ((size_t)tp.a_stages * kTileBytes + (size_t)tp.b_stages * tp.BN * 128);
  s += (size_t)tab_blocks(tp, T) * kTabStride * (tab_weight_bytes(tp) + sizeof(uint32_t));
  s += 3 * kBM * sizeof(int);
  s += (size_t)(2 * tp.a_stages + 2 * tp.b_stages + 8) * sizeof(uint64_t) + 16;
  s += (size_t)2 * tp.BN * tp.io_bytes + 16;  // bias staging, one copy per accumulator buffer
  return s;
}

// Tile geometry: a tile is TH x TW output pixels of ONE sample (TH*TW = 128, TW a power of
// two); tile row r is pixel (r / TW, r % TW) of the tile.
struct TileId {
  int n, ho0, wo0, grp, nt;
};
__device__ __forceinline__ TileId decode_item(long long item, const Geom &g, const TcPlan &tp) {
  const int per_mt = g.groups * tp.NT;
  const long long mt = item / per_mt;
  const int rem = (int)(item - mt * per_mt);
  const int tiles_img = tp.tiles_x * tp.tiles_y;
  TileId t;
  t.n = (int)(mt / tiles_img);
  const int ti = (int)(mt - (long long)t.n * tiles_img);
  const int ty = ti / tp.tiles_x;
  t.ho0 = ty * (kBM >> tp.tw_log2);
  t.wo0 = (ti - ty * tp.tiles_x) << tp.tw_log2;
  t.grp = rem / tp.NT;
  t.nt = rem - t.grp * tp.NT;
  return t;
}

// PCFG encodes the producer layout as [1]*1000 + groups*100 + warps_per_group*10 + rows_in_flight:
// `groups` groups of `warps_per_group` warps fill alternate stages, and every thread keeps
// `rows_in_flight` rows (four 16-byte loads each) in flight; with the leading 1 the rows of a
// stage are software-pipelined (the next row's loads are issued before a row is blended),
// without it they are loaded and blended in batches.
template <typename TIO, int MODE, int PCFG>
__global__ void __launch_bounds__((kFirstProducerWarp + ((PCFG / 100) % 10) * ((PCFG / 10) % 10)) * 32, 1)
dcn_fwd_tc(const __grid_constant__ TcArgs a) {
  constexpr int kGroups = (PCFG / 100) % 10;  // group i fills k-stages i, i+G, ...
  constexpr bool kPipe = ((PCFG / 1000) & 1) != 0;  // gather software-pipelined over the passes
  constexpr bool kOwn = ((PCFG / 1000) & 2) != 0;   // every group keeps a table of its own taps (below)
  constexpr int kWpg = (PCFG / 10) % 10;    // warps per group
  constexpr int kBatch = PCFG % 10;         // rows of a thread in flight at a time
  constexpr int NPW = kGroups * kWpg;
  constexpr int kPasses = 32 / kWpg;        // rows of a stage per thread
  constexpr int kRowStep = 4 * kWpg;        // distance between them
  using MT = ModeTraits<MODE>;
  constexpr int kAStageBytes = MT::kTiles * kTileBytes;
  constexpr int kProdThreads = NPW * 32;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const Geom &g = a.g;
  const TcPlan &tp = a.tp;
  const SmemLayout L = carve(smem, tp, g.T);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int A = tp.a_stages, B = tp.b_stages;
  const uint32_t bar0 = smem_u32(L.bars);
  // barrier i lives at bar0 + 8*i
  const uint32_t full_a = bar0, empty_a = bar0 + 8 * A, full_b = bar0 + 16 * A,
                 empty_b = bar0 + 16 * A + 8 * B, tmem_full = bar0 + 16 * A + 16 * B,
                 tmem_empty = tmem_full + 16, prod_bar = tmem_full + 32;
  volatile int *abort_s = L.abort_flag;
  const uint32_t b_tile_bytes = (uint32_t)tp.BN * 128u;
  const uint32_t b_stage_bytes = b_tile_bytes * MT::kTiles;

  if (threadIdx.x == 0) {
    for (int i = 0; i < A; ++i) {
      mbar_init(full_a + 8 * i, kWpg);  // the warps of one producer group
      mbar_init(empty_a + 8 * i, 1);
    }
    for (int i = 0; i < B; ++i) {
      mbar_init(full_b + 8 * i, 1);
      mbar_init(empty_b + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tmem_full + 8 * i, 1);
      mbar_init(tmem_empty + 8 * i, kEpilogueWarps);
    }
    mbar_init(prod_bar, kProdThreads);
    for (int i = 0; i < 3; ++i) mbar_init(prod_bar + 8 * (1 + i), kWpg * 32);  // one per producer group
    *L.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(L.tmem_slot), (uint32_t)tp.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *L.tmem_slot;

  const long long items = tp.items;
  const long long plane = (long long)g.Ho * g.Wo;
  const int tw_mask = (1 << tp.tw_log2) - 1;

  if (warp < kEpilogueWarps) {
    // ------------------------------ epilogue ------------------------------
    // Thread = one pixel (accumulator row); per 32 output channels one tcgen05.ld, then bias,
    // activation, rounding and a store per channel (NCHW: a warp's 32 pixels of one channel
    // are one or two contiguous runs).  The tile's bias is staged in shared memory as fp32 so
    // that the inner loop has no global loads in front of its stores.
    TIO *out = (TIO *)a.output;
    const TIO *bias = (const TIO *)a.bias;
    const int row = warp * 32 + lane;
    const int ty = row >> tp.tw_log2, tx = row & tw_mask;
    const bool act_any = g.act == DCN_ACT_SIGMOID && g.act_hi > g.act_lo;
    StageTimer pt(a.counters, blockIdx.x == 0 && threadIdx.x == 0);
    long long li = 0;
    int staged_co0[2] = {-1, -1};
    for (long long item = blockIdx.x; item < items; item += gridDim.x, ++li) {
      const TileId t = decode_item(item, g, tp);
      const int buf = (int)(li & 1);
      const uint32_t par = (uint32_t)((li >> 1) & 1);
      const int ho = t.ho0 + ty, wo = t.wo0 + tx;
      const bool valid = ho < g.Ho && wo < g.Wo;
      const int ncols = min(tp.BN, g.Cog - t.nt * tp.BN);
      const int co0 = t.grp * g.Cog + t.nt * tp.BN;
      TIO *orow = out + (long long)t.n * g.out_sn + (long long)co0 * plane + (long long)ho * g.Wo + wo;
      const bool act_tile = act_any && co0 < g.act_hi && co0 + ncols > g.act_lo;
      pt.lap(13);
      if (!mbar_wait<true>(tmem_full + 8 * buf, par, abort_s, a.status, 3)) break;
      pt.lap(12);
      tc_fence_after();
      // Bias copy of this accumulator buffer.  When its channels change, every epilogue warp
      // writes the whole copy (the same values: no rendezvous between the warps is needed).
      // This comes after the wait above on purpose: the accumulator buffer is only filled
      // again once all four warps have released it, so no warp still reads the copy's
      // previous contents.
      TIO *bias_w = reinterpret_cast<TIO *>(L.bias_s) + buf * tp.BN;
      if (co0 != staged_co0[buf]) {
        __syncwarp();
        for (int i = lane; i < tp.BN; i += 32)
          st_from_float(bias_w, i, (bias && i < ncols) ? ld_as_float(bias, co0 + i) : 0.f);
        __syncwarp();
        staged_co0[buf] = co0;
      }
      const uint32_t taddr = tmem_base + (uint32_t)(buf * tp.BN) + ((uint32_t)(warp * 32) << 16);
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty + 8 * buf);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer ------------------------------
    // The whole warp walks the loop (so that barrier addresses, descriptors and counters are
    // warp-uniform values) and one elected lane issues the tensor-core instructions.
    {
      // fp32 accumulate, both operands K-major, M = 128 pixels, N = BN channels;
      // operand format 0 = fp16, 1 = bf16, 2 = tf32
      constexpr uint32_t kFmt = MODE == kModeBf16 ? 1u : (MODE == kModeF16 ? 0u : 2u);
      const uint32_t idesc = (1u << 4) | (kFmt << 7) | (kFmt << 10) |
                             ((uint32_t)(tp.BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      uint32_t sa = 0, pa = 0, sb = 0, pb = 0;
      long long li = 0;
      bool ok = true;
      StageTimer pt(a.counters, blockIdx.x == 0 && lane == 0);
      for (long long item = blockIdx.x; item < items && ok; item += gridDim.x, ++li) {
        const int buf = (int)(li & 1);
        const uint32_t par = (uint32_t)((li >> 1) & 1);
        pt.lap(11);
        ok = mbar_wait(tmem_empty + 8 * buf, par ^ 1u, abort_s, a.status, 4);
        if (!ok) break;
        pt.lap(10);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * tp.BN);
        for (int ks = 0; ks < tp.S; ++ks) {
          pt.lap(11);
          ok = mbar_wait(full_b + 8 * sb, pb, abort_s, a.status, 5);
          if (!ok) break;
          pt.lap(8);
          ok = mbar_wait(full_a + 8 * sa, pa, abort_s, a.status, 6);
          if (!ok) break;
          pt.lap(9);
          tc_fence_after();
          const uint64_t adesc = smem_desc_sw128(smem_u32(L.a + (size_t)sa * kAStageBytes));
          const uint64_t bdesc = smem_desc_sw128(smem_u32(L.b + (size_t)sb * b_stage_bytes));
          if (elect_one()) {
            // four k-steps of 32 bytes per 128-byte row: 16 bf16 or 8 tf32 elements each
            if constexpr (MODE != kModeTf32x3) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_bf16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                          (ks | k) != 0 ? 1u : 0u);
            } else {
              // operand tiles of a stage: [hi][lo]; products hi*hi + lo*hi + hi*lo
              const uint64_t adesc_lo = adesc + (uint64_t)(kTileBytes >> 4);
              const uint64_t bdesc_lo = bdesc + (uint64_t)(b_tile_bytes >> 4);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                umma_tf32(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                          (ks | k) != 0 ? 1u : 0u);
                umma_tf32(d_tmem, adesc_lo + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, 1u);
                umma_tf32(d_tmem, adesc + (uint64_t)(2 * k), bdesc_lo + (uint64_t)(2 * k), idesc, 1u);
              }
            }
            umma_commit(empty_a + 8 * sa);
            umma_commit(empty_b + 8 * sb);
            if (ks == tp.S - 1) umma_commit(tmem_full + 8 * buf);
          }
          __syncwarp();
          if (++sa == (uint32_t)A) { sa = 0; pa ^= 1u; }
          if (++sb == (uint32_t)B) { sb = 0; pb ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == kLoadWarp) {
    // ------------------------------ weight loader ------------------------------
    if (lane == 0) {
      const int per_mt = g.groups * tp.NT;
      uint32_t sb = 0, pb = 0;
      bool ok = true;
      StageTimer pt(a.counters, blockIdx.x == 0);
      for (long long item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int rem = (int)(item % per_mt);
        const uint8_t *src = a.wtiles + (size_t)rem * tp.S * b_stage_bytes;
        for (int ks = 0; ks < tp.S; ++ks) {
          pt.lap(15);
          ok = mbar_wait(empty_b + 8 * sb, pb ^ 1u, abort_s, a.status, 7);
          if (!ok) break;
          pt.lap(14);
          mbar_arrive_expect_tx(full_b + 8 * sb, b_stage_bytes);
          bulk_copy_g2s(smem_u32(L.b + (size_t)sb * b_stage_bytes),
                        src + (size_t)ks * b_stage_bytes, b_stage_bytes, full_b + 8 * sb);
          if (++sb == (uint32_t)B) { sb = 0; pb ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ producers ------------------------------
    const int ptid = threadIdx.x - kFirstProducerWarp * 32;
    const int pw = ptid >> 5;
    const int gi = pw / kWpg;    // producer group
    const int pwl = pw % kWpg;   // warp within the group
    const int sub = lane >> 3;   // row within the warp's group of four
    const int v = lane & 7;      // 16-byte vector (8 bf16 / 4 fp32 channels) of the 128-byte row
    const TIO *off = (const TIO *)a.offset;
    const TIO *msk = (const TIO *)a.mask;
    const uint32_t Wp = (uint32_t)(g.W + 2 * tp.in_pad);   // row pitch of the copy, in pixels
    const uint32_t cW2 = (uint32_t)g.C * MT::kEsz, cH2 = Wp * (uint32_t)g.C * MT::kEsz;
    const uint32_t cHW2 = cH2 + cW2;
    // this thread's first row of a stage and where its 16 bytes go (128-byte swizzle); its
    // other rows are kRowStep rows further, which keeps the swizzle phase
    const int row0 = pwl * 4 + sub;
    const uint32_t soff0 = (uint32_t)(row0 * 128 + ((v ^ (row0 & 7)) << 4));
    // rows whose tap entries this thread computes when a table is rebuilt
    // (with per-group tables: the threads of a group share out the group's own entries)
    const int btid = kOwn ? ptid - gi * kWpg * 32 : ptid;
    const int trow = btid & (kBM - 1);
    const int tpart = btid >> 7, tparts = (kOwn ? kWpg * 32 : kProdThreads) >> 7;
    typename MT::TabW *const tabw = reinterpret_cast<typename MT::TabW *>(L.tab_w);
    // first (tap, deform group) block of this group's table
    const int tab0 = kOwn ? gi * ((g.T + kGroups - 1) / kGroups) * tp.ndgc : 0;
    uint32_t sa = (uint32_t)gi % (uint32_t)A, pa = 0, pp = 0;
    bool ok = true;
    // Producer-only rendezvous on an mbarrier, so that it is bounded like every other wait.
    const uint32_t my_bar = kOwn ? prod_bar + 8 * (1 + gi) : prod_bar;  // the group's, or everybody's
    auto psync = [&]() -> bool {
      mbar_arrive(my_bar);
      const bool r = mbar_wait(my_bar, pp, abort_s, a.status, 9);
      pp ^= 1u;
      return r;
    };
    uint32_t tcount = 0;  // global k-stage counter of this CTA (same in every producer)
    bool built = false;   // (per-group tables) this group has a table that may still be read
    StageTimer pt(a.counters, blockIdx.x == 0 && ptid == 0);
    for (long long item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const TileId t = decode_item(item, g, tp);
      pt.lap(0);
      if constexpr (!kOwn) {
        // all producers are done with the previous tile's tables before they are rebuilt
        if (!(ok = psync())) break;
        pt.lap(2);
        if (ptid < kBM) {
          const int ho = t.ho0 + (ptid >> tp.tw_log2), wo = t.wo0 + (ptid & tw_mask);
          const bool valid = ho < g.Ho && wo < g.Wo;
          L.row_h[ptid] = valid ? ho * g.stride_h - g.pad_h : kRowInvalid;
          L.row_w[ptid] = wo * g.stride_w - g.pad_w;
          L.row_pix[ptid] = valid ? ho * g.Wo + wo : 0;
        }
        pt.lap(0);
        if (!(ok = psync())) break;
        pt.lap(2);
      }
      // Ask L2 for the offsets and masks of the tile after this one (of this one too, the
      // first time): the tap tables are built from them and would otherwise wait on DRAM.
      const bool dense_planes = g.off_ps == 1 && g.msk_ps == 1 && g.off_cs == plane && g.msk_cs == plane;
      for (long long nitem = (item == (long long)blockIdx.x ? item : item + gridDim.x);
           dense_planes && nitem <= item + gridDim.x && nitem < items; nitem += gridDim.x) {
        const TileId nt_ = decode_item(nitem, g, tp);
        // 128-byte lines per tile row, rows per tile: both powers of two, so the index of a
        // line splits into (plane, row, line) with shifts
        const int lr_log2 = max(0, tp.tw_log2 + (sizeof(TIO) == 4 ? 2 : 1) - 7);
        const int pp_log2 = (7 - tp.tw_log2) + lr_log2;  // lines per plane
        const int planes_off = off ? g.dg * 2 * g.T : 0;
        const int planes = planes_off + (msk ? g.dg * g.T : 0);
        const TIO *obase = off ? off + (long long)nt_.n * g.off_sn : nullptr;
        const TIO *mbase = msk ? msk + (long long)nt_.n * g.msk_sn : nullptr;
        for (int idx = ptid; idx < (planes << pp_log2); idx += kProdThreads) {
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
      }
      pt.lap(17);
      const char *xb = reinterpret_cast<const char *>(a.xcl) +
                       (long long)t.n * (g.H + 2 * tp.in_pad) * Wp * g.C * MT::kEsz;
      int cur_lo = -1, cur_nd = 0;
      for (int cc = 0; cc < tp.KC && ok; ++cc) {
        const int c0 = t.grp * g.Cg + cc * MT::kCh;
        const int dg_lo = c0 / g.cpdg;
        const int dg_hi = (min(c0 + MT::kCh, (t.grp + 1) * g.Cg) - 1) / g.cpdg;
        const int nd = dg_hi - dg_lo + 1;
        // Shared table: rebuilt when the chunk's deform groups differ from the previous
        // chunk's.  Per-group tables hold only the group's own taps of one chunk (the taps of
        // the stages it fills), so they are rebuilt every chunk, by the group alone: while one
        // group rebuilds, the other keeps gathering.  (Chosen by the plan when every chunk has
        // deform groups of its own anyway.)
        const int own_t0 = kOwn ? (gi + kGroups - (int)(tcount % kGroups)) % kGroups : 0;
        if (kOwn || dg_lo != cur_lo || nd != cur_nd) {
          pt.lap(0);
          if ((kOwn ? built : cur_lo >= 0) && !(ok = psync())) break;
          built = true;
          pt.lap(2);
          pt.count(6);
          {
            // Each thread fills the entries e = tpart, tpart + tparts, ... of its row.  The
            // offset/mask loads of a batch of entries are all issued before any is used, so
            // their DRAM latency overlaps.
            int hb, wb, pix;
            bool rvalid;
            if constexpr (kOwn) {
              const int ho = t.ho0 + (trow >> tp.tw_log2), wo = t.wo0 + (trow & tw_mask);
              rvalid = ho < g.Ho && wo < g.Wo;
              hb = ho * g.stride_h - g.pad_h;
              wb = wo * g.stride_w - g.pad_w;
              pix = rvalid ? ho * g.Wo + wo : 0;
            } else {
              hb = L.row_h[trow]; wb = L.row_w[trow]; pix = L.row_pix[trow];
              rvalid = hb != kRowInvalid;
            }
            const TIO *offp = off ? off + (long long)t.n * g.off_sn + (long long)pix * g.off_ps : nullptr;
            const TIO *mskp = msk ? msk + (long long)t.n * g.msk_sn + (long long)pix * g.msk_ps : nullptr;
            constexpr int kTapStep = kOwn ? kGroups : 1;  // taps of consecutive table blocks
            const int n_taps = kOwn ? (own_t0 < g.T ? (g.T - own_t0 + kGroups - 1) / kGroups : 0) : g.T;
            const int total = n_taps * nd;
            constexpr int kEnt = NPW <= 8 ? 9 : (NPW <= 12 ? 6 : 5);  // entries in flight per thread
            // entry e <-> (table block j, dgl); block j is tap own_t0 + j * kTapStep <-> (ti, tj)
            int j = 0, tap = own_t0, dgl = tpart, ti = own_t0 / g.kw, tj = own_t0 - (own_t0 / g.kw) * g.kw;
            auto normalise = [&]() {
              while (dgl >= nd) {
                dgl -= nd;
                ++j;
                tap += kTapStep;
#pragma unroll
                for (int q = 0; q < kTapStep; ++q)
                  if (++tj == g.kw) { tj = 0; ++ti; }
              }
            };
            normalise();
            for (int e0 = tpart; e0 < total; e0 += tparts * kEnt) {
              typename RawOf<TIO>::type oh[kEnt], ow[kEnt], mm[kEnt];  // raw element bits
              int where[kEnt];
#pragma unroll
              for (int k = 0; k < kEnt; ++k) {
                oh[k] = 0; ow[k] = 0; mm[k] = 0;
                where[k] = -1;
                if (e0 + k * tparts < total) {
                  where[k] = j | (dgl << 12) | (ti << 16) | (tj << 24);
                  const int tap_k = tap;
                  if (rvalid) {
                    if (offp) {
                      const long long ch = ((long long)(dg_lo + dgl) * 2 * g.T + 2 * tap_k) * g.off_cs;
                      oh[k] = ldg_raw_ordered(offp + ch);
                      ow[k] = ldg_raw_ordered(offp + ch + g.off_cs);
                    }
                    if (mskp)
                      mm[k] = ldg_raw_ordered(mskp + ((long long)(dg_lo + dgl) * g.T + tap_k) * g.msk_cs);
                  }
                  dgl += tparts;
                  normalise();
                }
              }
              asm volatile("" ::: "memory");  // every load of the batch is issued before this
              pt.lap(16);
#pragma unroll
              for (int k = 0; k < kEnt; ++k) {
                if (where[k] < 0) continue;
                const int etap = where[k] & 0xfff, edgl = (where[k] >> 12) & 0xf;
                const int ei = (where[k] >> 16) & 0xff, ej = (where[k] >> 24) & 0xff;
                float4 wt = make_float4(0.f, 0.f, 0.f, 0.f);
                int h_low = 0, w_low = 0;
                if (rvalid)
                  tap_weights(RawOf<TIO>::to_float(oh[k]), RawOf<TIO>::to_float(ow[k]),
                              mskp ? mask_value(g, RawOf<TIO>::to_float(mm[k])) : 1.f, hb + ei * g.dil_h,
                              wb + ej * g.dil_w, g.H, g.W, wt, h_low, w_low);
                // a corner the reference does not read has the integer 0 as its weight and is not
                // read here either; a corner it reads with a weight that is (or rounds to) zero
                // keeps a signed zero, so that a non-finite sample under it gives NaN as it does
                // in the reference
                typename MT::TabW wq;
                if constexpr (MODE == kModeTf32x3) {
                  wq.x = __float_as_uint(wt.x);
                  wq.y = __float_as_uint(wt.y);
                  wq.z = __float_as_uint(wt.z);
                  wq.w = __float_as_uint(wt.w);
                } else {
                  uint32_t b0, b1, b2, b3;
                  if constexpr (MODE == kModeBf16) {
                    b0 = __bfloat16_as_ushort(__float2bfloat16_rn(wt.x));
                    b1 = __bfloat16_as_ushort(__float2bfloat16_rn(wt.y));
                    b2 = __bfloat16_as_ushort(__float2bfloat16_rn(wt.z));
                    b3 = __bfloat16_as_ushort(__float2bfloat16_rn(wt.w));
                  } else {
                    b0 = __half_as_ushort(__float2half_rn(wt.x));
                    b1 = __half_as_ushort(__float2half_rn(wt.y));
                    b2 = __half_as_ushort(__float2half_rn(wt.z));
                    b3 = __half_as_ushort(__float2half_rn(wt.w));
                  }
                  b0 = (b0 & 0x7fffu) ? b0 : (corner_is_read(wt.x) ? 0x8000u : 0u);
                  b1 = (b1 & 0x7fffu) ? b1 : (corner_is_read(wt.y) ? 0x8000u : 0u);
                  b2 = (b2 & 0x7fffu) ? b2 : (corner_is_read(wt.z) ? 0x8000u : 0u);
                  b3 = (b3 & 0x7fffu) ? b3 : (corner_is_read(wt.w) ? 0x8000u : 0u);
                  wq.x = b0 | (b1 << 16);
                  wq.y = b2 | (b3 << 16);
                }
                const int slot = (tab0 + etap * tp.ndgc + edgl) * kTabStride + trow;
                tabw[slot] = wq;
                L.tab_off[slot] = (uint32_t)(((h_low + tp.in_pad) * (int)Wp + w_low + tp.in_pad) * g.C * MT::kEsz);
              }
            }
          }
          pt.lap(1);
          if (!(ok = psync())) break;
          pt.lap(2);
          cur_lo = dg_lo;
          cur_nd = nd;
        }
        // the last chunk of a group may be partly beyond its channels: those vectors are zero
        const bool vvalid = cc * MT::kCh + v * MT::kCpv < g.Cg;
        const int c = vvalid ? c0 + v * MT::kCpv : c0;
        const int dgl = c / g.cpdg - dg_lo;
        const uint32_t c2 = (uint32_t)c * MT::kEsz;
        int own_j = 0;  // this group's stages of the chunk so far
        for (int tap = 0; tap < g.T; ++tap, ++tcount) {
          if (kGroups > 1 && (int)(tcount % kGroups) != gi) continue;
          pt.lap(0);
          pt.count(5);
          uint8_t *stage = L.a + (size_t)sa * kAStageBytes + soff0;
          const int slot0 = (tab0 + (kOwn ? own_j : tap) * tp.ndgc + dgl) * kTabStride + row0;
          ++own_j;
          const uint4 z = make_uint4(0u, 0u, 0u, 0u);
          if constexpr (kPipe) {
            // kBatch register sets rotate over the passes: the loads of pass p + kBatch - 1 are
            // issued before pass p is blended, so that a pass's loads fly during the blends of
            // the passes before it.  (Carrying the rotation across stage boundaries as well
            // measured slower.)
            uint4 q[kBatch][4], wq[kBatch];
            uint32_t tok = 0;
            auto issue = [&](int p) {
              const int sl = p % kBatch;
              wq[sl] = vvalid ? table_weights<MODE>(tabw[slot0 + p * kRowStep]) : z;
              const uint32_t o = L.tab_off[slot0 + p * kRowStep] + c2;
              q[sl][0] = ldg16_pinned(xb + o, wq[sl].x, tok);
              q[sl][1] = ldg16_pinned(xb + (uint32_t)(o + cW2), wq[sl].y, tok);
              q[sl][2] = ldg16_pinned(xb + (uint32_t)(o + cH2), wq[sl].z, tok);
              q[sl][3] = ldg16_pinned(xb + (uint32_t)(o + cHW2), wq[sl].w, tok);
            };
#pragma unroll
            for (int p = 0; p < kBatch - 1; ++p) issue(p);
#pragma unroll
            for (int p = 0; p < kPasses; ++p) {
              if (p + kBatch - 1 < kPasses) issue(p + kBatch - 1);
              if (p == 0) {
                // the stage must be free only now, with the first loads already in flight
                pt.lap(4);
                ok = mbar_wait(empty_a + 8 * sa, pa ^ 1u, abort_s, a.status, 8);
                pt.lap(3);
              }
              const int sl = p % kBatch;
              uint4 w = wq[sl];
              w.x |= tok;   // tok is 0: pins the blend behind the issue above
              uint8_t *dst = stage + p * kRowStep * 128;
              if constexpr (MODE == kModeBf16) {
                *reinterpret_cast<uint4 *>(dst) = blend8_bf16(w, q[sl][0], q[sl][1], q[sl][2], q[sl][3]);
              } else if constexpr (MODE == kModeF16) {
                *reinterpret_cast<uint4 *>(dst) = blend8_f16(w, q[sl][0], q[sl][1], q[sl][2], q[sl][3]);
              } else {
                uint4 hi, lo;
                blend4_tf32(w, q[sl][0], q[sl][1], q[sl][2], q[sl][3], hi, lo);
                *reinterpret_cast<uint4 *>(dst) = hi;
                *reinterpret_cast<uint4 *>(dst + kTileBytes) = lo;
              }
            }
          } else {
#pragma unroll
          for (int p0 = 0; p0 < kPasses; p0 += kBatch) {
            uint4 q[kBatch][4], wq[kBatch];
#pragma unroll
            for (int ps = 0; ps < kBatch; ++ps) {
              wq[ps] = vvalid ? table_weights<MODE>(tabw[slot0 + (p0 + ps) * kRowStep]) : z;
              const uint32_t o = L.tab_off[slot0 + (p0 + ps) * kRowStep] + c2;
              q[ps][0] = wq[ps].x ? __ldg((const uint4 *)(xb + o)) : z;
              q[ps][1] = wq[ps].y ? __ldg((const uint4 *)(xb + (uint32_t)(o + cW2))) : z;
              q[ps][2] = wq[ps].z ? __ldg((const uint4 *)(xb + (uint32_t)(o + cH2))) : z;
              q[ps][3] = wq[ps].w ? __ldg((const uint4 *)(xb + (uint32_t)(o + cHW2))) : z;
            }
            if (p0 == 0) {
              // the stage must be free only now, with this batch's loads already in flight
              pt.lap(4);
              ok = mbar_wait(empty_a + 8 * sa, pa ^ 1u, abort_s, a.status, 8);
              pt.lap(3);
            }
#pragma unroll
            for (int ps = 0; ps < kBatch; ++ps) {
              uint8_t *dst = stage + (p0 + ps) * kRowStep * 128;
              if constexpr (MODE == kModeBf16) {
                *reinterpret_cast<uint4 *>(dst) =
                    blend8_bf16(wq[ps], q[ps][0], q[ps][1], q[ps][2], q[ps][3]);
              } else if constexpr (MODE == kModeF16) {
                *reinterpret_cast<uint4 *>(dst) =
                    blend8_f16(wq[ps], q[ps][0], q[ps][1], q[ps][2], q[ps][3]);
              } else {
                uint4 hi, lo;
                blend4_tf32(wq[ps], q[ps][0], q[ps][1], q[ps][2], q[ps][3], hi, lo);
                *reinterpret_cast<uint4 *>(dst) = hi;
                *reinterpret_cast<uint4 *>(dst + kTileBytes) = lo;
              }
            }
          }
          }
          if (!ok) break;
          pt.lap(4);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(full_a + 8 * sa);
          pt.lap(7);
          sa += (uint32_t)kGroups;
          if (sa >= (uint32_t)A) { sa -= (uint32_t)A; pa ^= 1u; }
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
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)tp.tmem_cols);
  }
}

// ---------------------------------------------------------------------------------
// Preparation kernels
// ---------------------------------------------------------------------------------

// Input [N,C,H,W] (any element strides) -> channels-last [N,H,W,C] in bf16 or fp32.
template <typename T, typename TO>
__global__ void __launch_bounds__(256)
dcn_stage_input_cl(const T *__restrict__ x, TO *__restrict__ y, int C, int H, int W,
                   long long sn, long long sc, long long sh, long long sw, int pad) {
  __shared__ float tile[32][33];
  const int n = blockIdx.z;
  const int q0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int HW = H * W;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  {
    const int q = q0 + tx;
    const int h = q / W, w = q - h * W;
    const long long src = (long long)n * sn + (long long)h * sh + (long long)w * sw;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = c0 + ty + 8 * k;
      tile[ty + 8 * k][tx] = (q < HW && c < C) ? ld_as_float(x, src + (long long)c * sc) : 0.f;
    }
  }
  __syncthreads();
  {
    const int c = c0 + tx;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int q = q0 + ty + 8 * k;
      if (q < HW && c < C) {
        // with a border, pixel (h, w) goes to (h + pad, w + pad) of an (H + 2 pad) x (W + 2 pad) image
        const long long dq = pad ? (long long)n * (H + 2 * pad) * (W + 2 * pad) +
                                       (long long)(q / W + pad) * (W + 2 * pad) + (q % W + pad)
                                 : (long long)n * HW + q;
        st_from_float(y, dq * C + c, tile[tx][ty + 8 * k]);
      }
    }
  }
}

// The same for 16-bit tensors whose planes are contiguous and whose pixel count is a multiple
// of eight: 64 channels x 64 pixels per block through an 8 KiB shared-memory tile.  A lane
// loads eight pixels of two neighbouring channels (two 16-byte loads), interleaves them into
// eight (channel pair) words and writes those to the pixels' rows; the rows are then read and
// stored as 16-byte vectors, 128 contiguous bytes per quarter warp.  16-byte chunks of a row
// are XORed with (pixel & 7), which keeps both shared-memory phases free of bank conflicts.
__global__ void __launch_bounds__(256)
dcn_stage_input_cl_16bit(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, int C,
                         long long HW, long long sn, long long sc, int W, int pad) {
  __shared__ __align__(16) uint32_t tile[64][32];
  const int n = blockIdx.z;
  const long long q0 = (long long)blockIdx.x * 64;
  const int c0 = blockIdx.y * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    const long long q = q0 + warp * 8;
    const int ch = c0 + 2 * lane;
    uint4 va = make_uint4(0u, 0u, 0u, 0u), vb = va;
    if (q < HW && ch < C) {
      const uint8_t *src = x + ((long long)n * sn + (long long)ch * sc + q) * 2;
      va = __ldg(reinterpret_cast<const uint4 *>(src));
      vb = __ldg(reinterpret_cast<const uint4 *>(src + sc * 2));
    }
    const uint32_t a[4] = {va.x, va.y, va.z, va.w}, b[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int p = warp * 8 + i;
      tile[p][(((lane >> 2) ^ (p & 7)) << 2) | (lane & 3)] =
          __byte_perm(a[i >> 1], b[i >> 1], (i & 1) ? 0x7632 : 0x5410);
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int vec = threadIdx.x + k * 256;
    const int p = vec >> 3, o = vec & 7;
    const uint4 d = *reinterpret_cast<const uint4 *>(&tile[p][(o ^ (p & 7)) << 2]);
    if (q0 + p < HW && c0 + o * 8 < C) {
      const long long q = q0 + p;
      // (a sample has fewer than 2^31 pixels: 32-bit divisions)
      const int qi = (int)q, H = (int)HW / W;
      const int row = qi / W, col = qi - row * W;
      const long long dq = pad ? (long long)n * (H + 2 * pad) * (W + 2 * pad) +
                                     (long long)(row + pad) * (W + 2 * pad) + (col + pad)
                               : (long long)n * HW + q;
      *reinterpret_cast<uint4 *>(y + (dq * C + c0 + o * 8) * 2) = d;
    }
  }
}

// Zeroes the border of a padded channels-last copy [N][H+2][W+2][C] and the extra row that
// follows the last sample; 16 bytes per thread and step (C * esize is a multiple of 16).
__global__ void __launch_bounds__(256)
dcn_zero_border(uint8_t *__restrict__ y, int N, int H, int W, int vec_per_px) {
  const int Wp = W + 2, Hp = H + 2;
  const long long per_sample = 2LL * Wp + 2LL * H;  // border pixels of one sample
  const long long total = ((long long)N * per_sample + Wp) * vec_per_px;
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long bp = i / vec_per_px;
    const int vv = (int)(i - bp * vec_per_px);
    long long pix;  // pixel index in the padded buffer
    if (bp >= (long long)N * per_sample) {
      pix = (long long)N * Hp * Wp + (bp - (long long)N * per_sample);
    } else {
      const long long n = bp / per_sample;
      const long long r = bp - n * per_sample;
      long long hh, ww;
      if (r < Wp) { hh = 0; ww = r; }
      else if (r < 2LL * Wp) { hh = Hp - 1; ww = r - Wp; }
      else { const long long k = r - 2LL * Wp; hh = 1 + (k >> 1); ww = (k & 1) ? Wp - 1 : 0; }
      pix = (n * Hp + hh) * Wp + ww;
    }
    *reinterpret_cast<uint4 *>(y + (pix * vec_per_px + vv) * 16) = z;
  }
}

// Channels-last input (dense, the copy's own 16-bit type) -> the same with a zero border.
__global__ void __launch_bounds__(256)
dcn_pad_cl_copy(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, long long n_px, int H, int W,
                int vec_per_px) {
  const long long total = n_px * vec_per_px;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long px = i / vec_per_px;
    const int vv = (int)(i - px * vec_per_px);
    const long long n = px / ((long long)H * W);
    const long long q = px - n * (long long)H * W;
    const long long dq = (n * (H + 2) + q / W + 1) * (W + 2) + q % W + 1;
    *reinterpret_cast<uint4 *>(y + (dq * vec_per_px + vv) * 16) =
        __ldg(reinterpret_cast<const uint4 *>(x + i * 16));
  }
}

// The fp32 counterpart (TF32x3 keeps fp32 data): 32 channels x 64 pixels per block; a lane loads
// four pixels of one channel per 16-byte load and writes one word per pixel row.
__global__ void __launch_bounds__(256)
dcn_stage_input_cl_32bit(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, int C,
                         long long HW, long long sn, long long sc) {
  __shared__ __align__(16) uint32_t tile[64][32];
  const int n = blockIdx.z;
  const long long q0 = (long long)blockIdx.x * 64;
  const int c0 = blockIdx.y * 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int pl = warp * 8 + h * 4;  // first of four pixels
    const int ch = c0 + lane;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (q0 + pl < HW && ch < C)
      v = __ldg(reinterpret_cast<const uint4 *>(x + ((long long)n * sn + (long long)ch * sc + q0 + pl) * 4));
    const uint32_t e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int p = pl + i;
      tile[p][(((lane >> 2) ^ (p & 7)) << 2) | (lane & 3)] = e[i];
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int vec = threadIdx.x + k * 256;
    const int p = vec >> 3, o = vec & 7;
    const uint4 d = *reinterpret_cast<const uint4 *>(&tile[p][(o ^ (p & 7)) << 2]);
    if (q0 + p < HW && c0 + o * 4 < C)
      *reinterpret_cast<uint4 *>(y + (((long long)n * HW + q0 + p) * C + c0 + o * 4) * 4) = d;
  }
}

namespace {
template <typename T, typename TO>
void stage_launch(const Geom &g, const void *input, void *xcl, dim3 grid, int pad, cudaStream_t s) {
  dcn_stage_input_cl<T, TO><<<grid, 256, 0, s>>>((const T *)input, (TO *)xcl, g.C, g.H, g.W,
                                                  g.in_sn, g.in_sc, g.in_sh, g.in_sw, pad);
}
template <typename TO>
void stage_from(const Geom &g, const void *input, int dtype, void *xcl, dim3 grid, int pad,
                cudaStream_t s) {
  if (dtype == DCN_DTYPE_F32) stage_launch<float, TO>(g, input, xcl, grid, pad, s);
  else if (dtype == DCN_DTYPE_F16) stage_launch<__half, TO>(g, input, xcl, grid, pad, s);
  else stage_launch<__nv_bfloat16, TO>(g, input, xcl, grid, pad, s);
}
}  // namespace

// op_format: element type of the channels-last copy (0 fp16, 1 bf16, 2 fp32 for TF32x3)
cudaError_t launch_stage_input_cl(const Geom &g, const void *input, int dtype, void *xcl,
                                  int op_format, int pad, cudaStream_t s) {
  if (g.N == 0) return cudaSuccess;
  if (pad) {
    // the border (and the all-zero row after the last sample) first; the copies below fill
    // the interior
    const int vpp = g.C * (op_format == 2 ? 4 : 2) / 16;
    const long long total = ((long long)g.N * (2LL * (g.W + 2) + 2LL * g.H) + g.W + 2) * vpp;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    dcn_zero_border<<<blocks, 256, 0, s>>>((uint8_t *)xcl, g.N, g.H, g.W, vpp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    // dense channels-last input in the copy's type: a plain vector copy
    const bool same16 = dtype != DCN_DTYPE_F32 && op_format != 2 &&
                        (op_format == 0) == (dtype == DCN_DTYPE_F16);
    if (same16 && g.in_sc == 1 && g.in_sw == g.C && g.in_sh == (long long)g.W * g.C &&
        g.in_sn == (long long)g.H * g.W * g.C && ((uintptr_t)input & 15) == 0) {
      const long long n_px = (long long)g.N * g.H * g.W;
      const long long tv = n_px * vpp;
      const unsigned cb = (unsigned)((tv + 255) / 256 < 148 * 64 ? (tv + 255) / 256 : 148 * 64);
      dcn_pad_cl_copy<<<cb, 256, 0, s>>>((const uint8_t *)input, (uint8_t *)xcl, n_px, g.H, g.W, vpp);
      return cudaGetLastError();
    }
  }
  {
    // 16-bit in, the same 16-bit type out, contiguous planes
    const bool same16 = dtype != DCN_DTYPE_F32 && op_format != 2 &&
                        (op_format == 0) == (dtype == DCN_DTYPE_F16);
    const long long HW = (long long)g.H * g.W;
    if (same16 && g.in_sw == 1 && g.in_sh == g.W && HW % 8 == 0 && g.C % 8 == 0 &&
        g.in_sn % 8 == 0 && g.in_sc % 8 == 0 && ((uintptr_t)input & 15) == 0 && g.N <= 65535 &&
        (g.C + 63) / 64 <= 65535) {
      dim3 grid((unsigned)((HW + 63) / 64), (unsigned)((g.C + 63) / 64), (unsigned)g.N);
      dcn_stage_input_cl_16bit<<<grid, 256, 0, s>>>((const uint8_t *)input, (uint8_t *)xcl, g.C, HW,
                                                    g.in_sn, g.in_sc, g.W, pad);
      return cudaGetLastError();
    }
    // fp32 in, fp32 out
    if (!pad && dtype == DCN_DTYPE_F32 && op_format == 2 && g.in_sw == 1 && g.in_sh == g.W && HW % 4 == 0 &&
        g.C % 4 == 0 && g.in_sn % 4 == 0 && g.in_sc % 4 == 0 && ((uintptr_t)input & 15) == 0 &&
        g.N <= 65535 && (g.C + 31) / 32 <= 65535) {
      dim3 grid((unsigned)((HW + 63) / 64), (unsigned)((g.C + 31) / 32), (unsigned)g.N);
      dcn_stage_input_cl_32bit<<<grid, 256, 0, s>>>((const uint8_t *)input, (uint8_t *)xcl, g.C, HW,
                                                    g.in_sn, g.in_sc);
      return cudaGetLastError();
    }
  }
  dim3 grid((g.H * g.W + 31) / 32, (g.C + 31) / 32, g.N);
  if (op_format == 2) stage_from<float>(g, input, dtype, xcl, grid, pad, s);
  else if (op_format == 0) stage_from<__half>(g, input, dtype, xcl, grid, pad, s);
  else stage_from<__nv_bfloat16>(g, input, dtype, xcl, grid, pad, s);
  return cudaGetLastError();
}

// Weight [Co, Cg, kh, kw] -> one pre-swizzled shared-memory image per
// (group, n-tile, k-stage): BN rows of 128 bytes, 16-byte chunk index XORed with (row & 7).
// k-stage = chunk*T + tap.  bf16 mode: 64 channels per row.  TF32x3 mode: 32 fp32 channels
// per row and two images per stage, the TF32 high parts (low 13 mantissa bits cleared)
// followed by the exact remainders.
template <typename T>
__global__ void __launch_bounds__(256)
dcn_weight_tiles(const T *__restrict__ w, uint8_t *__restrict__ dst, int Cg, int Cog, int Tt,
                 int BN, int NT, int S, int op_format) {
  const int tf32 = op_format == 2;
  const int blk = blockIdx.x;  // (grp*NT + nt)*S + ks
  const int ks = blk % S;
  const int gn = blk / S;
  const int nt = gn % NT, grp = gn / NT;
  const int cc = ks / Tt, tap = ks - cc * Tt;
  const int ch = tf32 ? 32 : 64;  // channels per row
  uint8_t *out = dst + (size_t)blk * BN * 128 * (tf32 ? 2 : 1);
  // blockIdx.y: which sixteen rows of the image (many small blocks: the strided reads of the
  // weights are latency-bound, so parallelism is what makes this pass short)
  const int e_end = min(BN, ((int)blockIdx.y + 1) * 16) * ch;
#pragma unroll 4
  for (int e = (int)blockIdx.y * 16 * ch + threadIdx.x; e < e_end; e += blockDim.x) {
    const int r = e / ch, j = e - r * ch;
    const int col = nt * BN + r;
    float val = 0.f;
    if (col < Cog && cc * ch + j < Cg) {
      const long long co = (long long)grp * Cog + col;
      val = ld_as_float(w, (co * Cg + (cc * ch + j)) * Tt + tap);
    }
    if (tf32) {
      const int byte = r * 128 + (((j >> 2) ^ (r & 7)) << 4) + (j & 3) * 4;
      const uint32_t hb = __float_as_uint(val) & 0xffffe000u;
      *reinterpret_cast<uint32_t *>(out + byte) = hb;
      *reinterpret_cast<float *>(out + (size_t)BN * 128 + byte) = val - __uint_as_float(hb);
    } else {
      const int byte = r * 128 + (((j >> 3) ^ (r & 7)) << 4) + (j & 7) * 2;
      if (op_format == 0)
        *reinterpret_cast<__half *>(out + byte) = __float2half_rn(val);
      else
        *reinterpret_cast<__nv_bfloat16 *>(out + byte) = __float2bfloat16_rn(val);
    }
  }
}

// The same for the second-generation kernel, whose k-stage holds two (32-channel half-chunk,
// tap) units, half-chunk-major: unit u = hc*T + tap, stage s = units 2s and 2s+1, 64 bytes
// each of a row.  A unit beyond the last one, and channels beyond the group, are zero.
template <typename T>
__global__ void __launch_bounds__(256)
dcn_weight_tiles2(const T *__restrict__ w, uint8_t *__restrict__ dst, int Cg, int Cog, int Tt,
                  int BN, int NT, int S, int U, int op_format) {
  const int blk = blockIdx.x;  // (grp*NT + nt)*S + ks
  const int ks = blk % S;
  const int gn = blk / S;
  const int nt = gn % NT, grp = gn / NT;
  uint8_t *out = dst + (size_t)blk * BN * 128;
  const int e_end = min(BN, ((int)blockIdx.y + 1) * 16) * 64;
#pragma unroll 4
  for (int e = (int)blockIdx.y * 16 * 64 + threadIdx.x; e < e_end; e += blockDim.x) {
    const int r = e >> 6, j = e & 63;
    const int col = nt * BN + r;
    const int unit = 2 * ks + (j >> 5);
    const int hc = unit / Tt, tap = unit - hc * Tt;
    const int ch = hc * 32 + (j & 31);
    float val = 0.f;
    if (col < Cog && unit < U && ch < Cg) {
      const long long co = (long long)grp * Cog + col;
      val = ld_as_float(w, (co * Cg + ch) * Tt + tap);
    }
    const int byte = r * 128 + (((j >> 3) ^ (r & 7)) << 4) + (j & 7) * 2;
    if (op_format == 0)
      *reinterpret_cast<__half *>(out + byte) = __float2half_rn(val);
    else
      *reinterpret_cast<__nv_bfloat16 *>(out + byte) = __float2bfloat16_rn(val);
  }
}

cudaError_t launch_weight_tiles(const Geom &g, const TcPlan &tp, const void *weight, int dtype,
                                void *wtiles, cudaStream_t s) {
  const dim3 blocks((unsigned)(g.groups * tp.NT * tp.S), (unsigned)((tp.BN + 15) / 16));
  if (tp.version == 2) {
    if (dtype == DCN_DTYPE_F32)
      dcn_weight_tiles2<float><<<blocks, 256, 0, s>>>((const float *)weight, (uint8_t *)wtiles, g.Cg,
                                                      g.Cog, g.T, tp.BN, tp.NT, tp.S, tp.U, tp.op_format);
    else if (dtype == DCN_DTYPE_F16)
      dcn_weight_tiles2<__half><<<blocks, 256, 0, s>>>((const __half *)weight, (uint8_t *)wtiles, g.Cg,
                                                       g.Cog, g.T, tp.BN, tp.NT, tp.S, tp.U, tp.op_format);
    else
      dcn_weight_tiles2<__nv_bfloat16><<<blocks, 256, 0, s>>>(
          (const __nv_bfloat16 *)weight, (uint8_t *)wtiles, g.Cg, g.Cog, g.T, tp.BN, tp.NT, tp.S, tp.U,
          tp.op_format);
    return cudaGetLastError();
  }
  if (dtype == DCN_DTYPE_F32)
    dcn_weight_tiles<float><<<blocks, 256, 0, s>>>((const float *)weight, (uint8_t *)wtiles, g.Cg,
                                                   g.Cog, g.T, tp.BN, tp.NT, tp.S, tp.op_format);
  else if (dtype == DCN_DTYPE_F16)
    dcn_weight_tiles<__half><<<blocks, 256, 0, s>>>((const __half *)weight, (uint8_t *)wtiles, g.Cg,
                                                    g.Cog, g.T, tp.BN, tp.NT, tp.S, tp.op_format);
  else
    dcn_weight_tiles<__nv_bfloat16><<<blocks, 256, 0, s>>>(
        (const __nv_bfloat16 *)weight, (uint8_t *)wtiles, g.Cg, g.Cog, g.T, tp.BN, tp.NT, tp.S,
        tp.op_format);
  return cudaGetLastError();
}

__global__ void dcn_clear_status(int *status) {
  // the whole 256-byte workspace header: status word and the optional phase counters
  status[threadIdx.x] = 0;
}

cudaError_t launch_clear_status(int *status, cudaStream_t s) {
  dcn_clear_status<<<1, 64, 0, s>>>(status);
  return cudaGetLastError();
}

namespace {
template <typename TIO, int MODE, int PCFG>
cudaError_t launch_one(const TcArgs &a, const TcPlan &tp, cudaStream_t s) {
  auto kern = dcn_fwd_tc<TIO, MODE, PCFG>;
  constexpr int kThreads = (kFirstProducerWarp + ((PCFG / 100) % 10) * ((PCFG / 10) % 10)) * 32;
  // opt in to large dynamic shared memory once per device and instantiation
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
  // leave what the kernel does not need of the SM's 256 KB to L1: the gather lives on it
  static std::atomic<int> carve_pct[64];
  // (the smallest shared-memory configuration that holds the block and its 1 KB system
  // reserve; the percentage is rounded down so that the driver lands on that configuration)
  int pct = 100;
  {
    const size_t need = tp.smem + 1024;
    const size_t configs_kb[] = {8, 16, 32, 64, 100, 132, 164, 196, 228};
    for (size_t kb : configs_kb)
      if (kb * 1024 >= need) { pct = (int)(kb * 1024 * 100 / 233472); break; }
  }
  if (carve_pct[dev & 63].load(std::memory_order_acquire) != pct) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                             pct > 100 ? 100 : pct);
    if (e != cudaSuccess) return e;
    carve_pct[dev & 63].store(pct, std::memory_order_release);
  }
  kern<<<tp.grid, kThreads, tp.smem, s>>>(a);
  return cudaGetLastError();
}
template <typename TIO, int MODE>
cudaError_t launch_mode(const TcArgs &a, const TcPlan &tp, cudaStream_t s) {
  switch (tp.producer_cfg) {
    case 342: return launch_one<TIO, MODE, 342>(a, tp, s);
    case 1282: return launch_one<TIO, MODE, 1282>(a, tp, s);
    case 3282: return launch_one<TIO, MODE, 3282>(a, tp, s);
    case 282: return launch_one<TIO, MODE, 282>(a, tp, s);
    default: return launch_one<TIO, MODE, 1282>(a, tp, s);
  }
}
template <typename TIO>
cudaError_t launch_io(const TcArgs &a, const TcPlan &tp, cudaStream_t s) {
  if (tp.op_format == 2) return launch_mode<TIO, kModeTf32x3>(a, tp, s);
  if (tp.op_format == 0) return launch_mode<TIO, kModeF16>(a, tp, s);
  return launch_mode<TIO, kModeBf16>(a, tp, s);
}
}  // namespace

int tc_threads(const TcPlan &tp) {
  if (tp.version == 2) return 768;  // dcn_fwd_tc2: 4 epilogue, MMA, 2 loaders, 1 idle and 16 gather warps
  return (kFirstProducerWarp + ((tp.producer_cfg / 100) % 10) * ((tp.producer_cfg / 10) % 10)) * 32;
}

cudaError_t launch_tc(const Geom &g, const TcPlan &tp, const Ptrs &p, int dtype, const void *xcl,
                      const void *wtiles, int *status, unsigned long long *counters,
                      cudaStream_t s) {
  if (tp.items == 0) return cudaSuccess;
  TcArgs a;
  a.g = g;
  a.tp = tp;
  a.xcl = xcl;
  a.wtiles = (const uint8_t *)wtiles;
  a.offset = p.offset;
  a.mask = p.mask;
  a.bias = p.bias;
  a.output = p.output;
  a.status = status;
  a.counters = counters;
  if (dtype == DCN_DTYPE_F32) return launch_io<float>(a, tp, s);
  if (dtype == DCN_DTYPE_F16) return launch_io<__half>(a, tp, s);
  return launch_io<__nv_bfloat16>(a, tp, s);
}

}  // namespace dcn
