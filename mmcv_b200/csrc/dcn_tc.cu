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
#include "dcn_internal.cuh"

namespace dcn {

namespace {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s per wait
constexpr int kEpilogueWarps = 4;
constexpr int kMmaWarp = 4;
constexpr int kLoadWarp = 5;
constexpr int kFirstProducerWarp = 6;
constexpr int kProducerThreads = kTcProducerWarps * 32;
constexpr int kAStageBytes = kBM * kBK * 2;  // 16 KiB

struct TcArgs {
  Geom g;
  TcPlan tp;
  const __nv_bfloat16 *xcl;  // channels-last bf16 input [N, H, W, C]
  const uint8_t *wtiles;     // pre-swizzled weight stages
  const void *offset, *mask, *bias;
  void *output;
  int *status;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the block is aborting.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_s,
                                          int *status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 31u) == 0u) {
      if (*abort_s) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) {
        *abort_s = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes,
                                              uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes
// (64 elements) with the 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)1 << 16;            // leading byte offset (unused with swizzle), 16 B
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;            // descriptor version of this architecture
  d |= (uint64_t)2 << 61;            // 128-byte swizzle
  return d;
}

__device__ __forceinline__ void unpack_fma(float (&acc)[8], float w, const uint4 &q) {
  const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] = fmaf(w, f.x, acc[2 * i]);
    acc[2 * i + 1] = fmaf(w, f.y, acc[2 * i + 1]);
  }
}

struct SmemLayout {
  uint8_t *a, *b;
  float4 *tab_w;
  int *tab_base;
  int *row_n, *row_h, *row_w, *row_pix;
  uint64_t *bars;
  uint32_t *tmem_slot;
  int *abort_flag;
};

__device__ __forceinline__ SmemLayout carve(uint8_t *base, const TcPlan &tp, int T) {
  SmemLayout L;
  uint8_t *p = base;
  L.a = p; p += (size_t)tp.a_stages * kAStageBytes;
  L.b = p; p += (size_t)tp.b_stages * tp.BN * 128;
  L.tab_w = (float4 *)p; p += (size_t)T * tp.ndgc * kBM * sizeof(float4);
  L.tab_base = (int *)p; p += (size_t)T * tp.ndgc * kBM * sizeof(int);
  L.row_n = (int *)p; p += kBM * sizeof(int);
  L.row_h = (int *)p; p += kBM * sizeof(int);
  L.row_w = (int *)p; p += kBM * sizeof(int);
  L.row_pix = (int *)p; p += kBM * sizeof(int);
  L.bars = (uint64_t *)p; p += (size_t)(2 * tp.a_stages + 2 * tp.b_stages + 5) * sizeof(uint64_t);
  L.tmem_slot = (uint32_t *)p; p += 8;
  L.abort_flag = (int *)p;
  return L;
}

}  // namespace

size_t tc_smem_bytes(const TcPlan &tp, int T) {
  size_t s = 1024;  // slack for manual 1024-byte alignment
  s += (size_t)tp.a_stages * kAStageBytes + (size_t)tp.b_stages * tp.BN * 128;
  s += (size_t)T * tp.ndgc * kBM * (sizeof(float4) + sizeof(int));
  s += 4 * kBM * sizeof(int);
  s += (size_t)(2 * tp.a_stages + 2 * tp.b_stages + 5) * sizeof(uint64_t) + 16;
  return s;
}

template <typename TIO>
__global__ void __launch_bounds__(kTcThreads, 1)
dcn_fwd_tc_bf16(const __grid_constant__ TcArgs a) {
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
  const uint32_t b_stage_bytes = (uint32_t)tp.BN * 128u;

  if (threadIdx.x == 0) {
    for (int i = 0; i < A; ++i) {
      mbar_init(full_a + 8 * i, kTcProducerWarps);
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
    mbar_init(prod_bar, kProducerThreads);
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
  const int per_mt = g.groups * tp.NT;
  const long long plane = (long long)g.Ho * g.Wo;

  if (warp < kEpilogueWarps) {
    // ------------------------------ epilogue ------------------------------
    TIO *out = (TIO *)a.output;
    const TIO *bias = (const TIO *)a.bias;
    const int row = warp * 32 + lane;
    long long li = 0;
    for (long long item = blockIdx.x; item < items; item += gridDim.x, ++li) {
      const long long mt = item / per_mt;
      const int rem = (int)(item % per_mt);
      const int grp = rem / tp.NT, nt = rem % tp.NT;
      const int buf = (int)(li & 1);
      const uint32_t par = (uint32_t)((li >> 1) & 1);
      const long long p = mt * kBM + row;
      const bool valid = p < g.P;
      long long obase = 0;
      if (valid) {
        const long long n = p / plane;
        obase = n * g.out_sn + (p - n * plane);
      }
      const int ncols = min(tp.BN, g.Cog - nt * tp.BN);
      const int co0 = grp * g.Cog + nt * tp.BN;
      if (!mbar_wait(tmem_full + 8 * buf, par, abort_s, a.status, 3)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t)(buf * tp.BN) + ((uint32_t)(warp * 32) << 16);
      for (int c0 = 0; c0 < ncols; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + (uint32_t)c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (c0 + j < ncols) {
            const int co = co0 + c0 + j;
            float v = __uint_as_float(r[j]);
            if (bias) v += ld_as_float(bias, co);
            v = apply_act(g, co, v);
            if (valid) st_from_float(out, obase + (long long)co * plane, v);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty + 8 * buf);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                             ((uint32_t)(tp.BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      uint32_t sa = 0, pa = 0, sb = 0, pb = 0;
      long long li = 0;
      bool ok = true;
      for (long long item = blockIdx.x; item < items && ok; item += gridDim.x, ++li) {
        const int buf = (int)(li & 1);
        const uint32_t par = (uint32_t)((li >> 1) & 1);
        ok = mbar_wait(tmem_empty + 8 * buf, par ^ 1u, abort_s, a.status, 4);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * tp.BN);
        for (int ks = 0; ks < tp.S; ++ks) {
          ok = mbar_wait(full_b + 8 * sb, pb, abort_s, a.status, 5);
          if (!ok) break;
          ok = mbar_wait(full_a + 8 * sa, pa, abort_s, a.status, 6);
          if (!ok) break;
          tc_fence_after();
          const uint64_t adesc = smem_desc_sw128(smem_u32(L.a + (size_t)sa * kAStageBytes));
          const uint64_t bdesc = smem_desc_sw128(smem_u32(L.b + (size_t)sb * b_stage_bytes));
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            umma_bf16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                      (ks | k) != 0 ? 1u : 0u);
          umma_commit(empty_a + 8 * sa);
          umma_commit(empty_b + 8 * sb);
          if (++sa == (uint32_t)A) { sa = 0; pa ^= 1u; }
          if (++sb == (uint32_t)B) { sb = 0; pb ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tmem_full + 8 * buf);
      }
    }
    __syncwarp();
  } else if (warp == kLoadWarp) {
    // ------------------------------ weight loader ------------------------------
    if (lane == 0) {
      uint32_t sb = 0, pb = 0;
      bool ok = true;
      for (long long item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int rem = (int)(item % per_mt);
        const uint8_t *src = a.wtiles + (size_t)rem * tp.S * b_stage_bytes;
        for (int ks = 0; ks < tp.S; ++ks) {
          ok = mbar_wait(empty_b + 8 * sb, pb ^ 1u, abort_s, a.status, 7);
          if (!ok) break;
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
    const int sub = lane >> 3;  // row within the warp's group of four
    const int v = lane & 7;     // 16-byte vector (8 channels) within the 128-byte row
    const TIO *off = (const TIO *)a.offset;
    const TIO *msk = (const TIO *)a.mask;
    const long long img = (long long)g.H * g.W;
    const long long cW = (long long)g.C, cH = (long long)g.W * g.C;
    uint32_t sa = 0, pa = 0, pp = 0;
    bool ok = true;
    // Producer-only rendezvous on an mbarrier, so that it is bounded like every other wait.
    auto psync = [&]() -> bool {
      mbar_arrive(prod_bar);
      const bool r = mbar_wait(prod_bar, pp, abort_s, a.status, 9);
      pp ^= 1u;
      return r;
    };
    for (long long item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const long long mt = item / per_mt;
      const int grp = (int)(item % per_mt) / tp.NT;
      // all producers are done with the previous tile's tables before they are rebuilt
      if (!(ok = psync())) break;
      if (ptid < kBM) {
        const long long p = mt * kBM + ptid;
        int n = -1, hb = 0, wb = 0, pix = 0;
        if (p < g.P) {
          n = (int)(p / plane);
          pix = (int)(p - (long long)n * plane);
          const int ho = pix / g.Wo, wo = pix - ho * g.Wo;
          hb = ho * g.stride_h - g.pad_h;
          wb = wo * g.stride_w - g.pad_w;
        }
        L.row_n[ptid] = n;
        L.row_h[ptid] = hb;
        L.row_w[ptid] = wb;
        L.row_pix[ptid] = pix;
      }
      if (!(ok = psync())) break;
      int cur_lo = -1, cur_nd = 0;
      for (int cc = 0; cc < tp.KC && ok; ++cc) {
        const int c0 = grp * g.Cg + cc * kBK;
        const int dg_lo = c0 / g.cpdg;
        const int dg_hi = min(g.dg - 1, (c0 + kBK - 1) / g.cpdg);
        const int nd = dg_hi - dg_lo + 1;
        if (dg_lo != cur_lo || nd != cur_nd) {
          if (cur_lo >= 0 && !(ok = psync())) break;
          const int entries = g.T * nd * kBM;
          for (int e = ptid; e < entries; e += kProducerThreads) {
            const int row = e & (kBM - 1);
            const int q = e >> 7;
            const int dgl = q % nd, tap = q / nd;
            const int n = L.row_n[row];
            float4 wt = make_float4(0.f, 0.f, 0.f, 0.f);
            int base = 0;
            if (n >= 0) {
              const int pix = L.row_pix[row];
              const int i = tap / g.kw, j = tap - i * g.kw;
              float oh = 0.f, ow = 0.f, m = 1.f;
              if (off) {
                const TIO *o = off + (long long)n * g.off_sn +
                               ((long long)(dg_lo + dgl) * 2 * g.T + 2 * tap) * plane + pix;
                oh = ld_as_float(o, 0);
                ow = ld_as_float(o, plane);
              }
              if (msk)
                m = ld_as_float(msk, (long long)n * g.msk_sn +
                                         ((long long)(dg_lo + dgl) * g.T + tap) * plane + pix);
              int h_low, w_low;
              tap_weights(oh, ow, m, L.row_h[row] + i * g.dil_h, L.row_w[row] + j * g.dil_w,
                          g.H, g.W, wt, h_low, w_low);
              base = (int)((long long)n * img) + h_low * g.W + w_low;
            }
            const int slot = (tap * tp.ndgc + dgl) * kBM + row;
            L.tab_w[slot] = wt;
            L.tab_base[slot] = base;
          }
          if (!(ok = psync())) break;
          cur_lo = dg_lo;
          cur_nd = nd;
        }
        const int c = c0 + v * 8;
        const int dgl = c / g.cpdg - dg_lo;
        const __nv_bfloat16 *xc = a.xcl + c;
        for (int tap = 0; tap < g.T; ++tap) {
          ok = mbar_wait(empty_a + 8 * sa, pa ^ 1u, abort_s, a.status, 8);
          if (!ok) break;
          uint8_t *stage = L.a + (size_t)sa * kAStageBytes;
          const int slot0 = (tap * tp.ndgc + dgl) * kBM;
          uint4 q[4][4];
          float4 wts[4];
#pragma unroll
          for (int ps = 0; ps < 4; ++ps) {
            const int row = ps * 32 + pw * 4 + sub;
            const float4 wt = L.tab_w[slot0 + row];
            const long long e0 = (long long)L.tab_base[slot0 + row] * cW;
            const uint4 z = make_uint4(0u, 0u, 0u, 0u);
            q[ps][0] = wt.x != 0.f ? __ldg((const uint4 *)(xc + e0)) : z;
            q[ps][1] = wt.y != 0.f ? __ldg((const uint4 *)(xc + e0 + cW)) : z;
            q[ps][2] = wt.z != 0.f ? __ldg((const uint4 *)(xc + e0 + cH)) : z;
            q[ps][3] = wt.w != 0.f ? __ldg((const uint4 *)(xc + e0 + cH + cW)) : z;
            wts[ps] = wt;
          }
#pragma unroll
          for (int ps = 0; ps < 4; ++ps) {
            const int row = ps * 32 + pw * 4 + sub;
            float acc[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.f;
            unpack_fma(acc, wts[ps].x, q[ps][0]);
            unpack_fma(acc, wts[ps].y, q[ps][1]);
            unpack_fma(acc, wts[ps].z, q[ps][2]);
            unpack_fma(acc, wts[ps].w, q[ps][3]);
            uint4 o;
            __nv_bfloat162 *oh2 = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) oh2[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            *reinterpret_cast<uint4 *>(stage + row * 128 + ((v ^ (row & 7)) << 4)) = o;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(full_a + 8 * sa);
          if (++sa == (uint32_t)A) { sa = 0; pa ^= 1u; }
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

// Input [N,C,H,W] (any element strides) -> channels-last bf16 [N,H,W,C].
template <typename T>
__global__ void __launch_bounds__(256)
dcn_stage_input_cl(const T *__restrict__ x, __nv_bfloat16 *__restrict__ y, int C, int H, int W,
                   long long sn, long long sc, long long sh, long long sw) {
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
      if (q < HW && c < C)
        y[((long long)n * HW + q) * C + c] = __float2bfloat16_rn(tile[tx][ty + 8 * k]);
    }
  }
}

cudaError_t launch_stage_input_cl(const Geom &g, const void *input, int dtype,
                                  __nv_bfloat16 *xcl, cudaStream_t s) {
  if (g.N == 0) return cudaSuccess;
  dim3 grid((g.H * g.W + 31) / 32, (g.C + 31) / 32, g.N);
  if (dtype == DCN_DTYPE_F32)
    dcn_stage_input_cl<float><<<grid, 256, 0, s>>>((const float *)input, xcl, g.C, g.H, g.W,
                                                    g.in_sn, g.in_sc, g.in_sh, g.in_sw);
  else
    dcn_stage_input_cl<__nv_bfloat16><<<grid, 256, 0, s>>>(
        (const __nv_bfloat16 *)input, xcl, g.C, g.H, g.W, g.in_sn, g.in_sc, g.in_sh, g.in_sw);
  return cudaGetLastError();
}

// Weight [Co, Cg, kh, kw] -> one pre-swizzled shared-memory image per
// (group, n-tile, k-stage): BN rows of 64 bf16 (128 bytes), 16-byte chunk index XORed
// with (row & 7).  k-stage = chunk*T + tap; column = channel within the 64-chunk.
template <typename T>
__global__ void __launch_bounds__(256)
dcn_weight_tiles(const T *__restrict__ w, uint8_t *__restrict__ dst, int Cg, int Cog, int Tt,
                 int BN, int NT, int S) {
  const int blk = blockIdx.x;  // (grp*NT + nt)*S + ks
  const int ks = blk % S;
  const int gn = blk / S;
  const int nt = gn % NT, grp = gn / NT;
  const int cc = ks / Tt, tap = ks - cc * Tt;
  uint8_t *out = dst + (size_t)blk * BN * 128;
  for (int e = threadIdx.x; e < BN * 64; e += blockDim.x) {
    const int r = e >> 6, j = e & 63;
    const int col = nt * BN + r;
    float val = 0.f;
    if (col < Cog) {
      const long long co = (long long)grp * Cog + col;
      val = ld_as_float(w, (co * Cg + (cc * 64 + j)) * Tt + tap);
    }
    const int byte = r * 128 + (((j >> 3) ^ (r & 7)) << 4) + (j & 7) * 2;
    *reinterpret_cast<__nv_bfloat16 *>(out + byte) = __float2bfloat16_rn(val);
  }
}

cudaError_t launch_weight_tiles(const Geom &g, const TcPlan &tp, const void *weight, int dtype,
                                void *wtiles, cudaStream_t s) {
  const int blocks = g.groups * tp.NT * tp.S;
  if (dtype == DCN_DTYPE_F32)
    dcn_weight_tiles<float><<<blocks, 256, 0, s>>>((const float *)weight, (uint8_t *)wtiles, g.Cg,
                                                   g.Cog, g.T, tp.BN, tp.NT, tp.S);
  else
    dcn_weight_tiles<__nv_bfloat16><<<blocks, 256, 0, s>>>(
        (const __nv_bfloat16 *)weight, (uint8_t *)wtiles, g.Cg, g.Cog, g.T, tp.BN, tp.NT, tp.S);
  return cudaGetLastError();
}

__global__ void dcn_clear_status(int *status) { *status = 0; }

cudaError_t launch_clear_status(int *status, cudaStream_t s) {
  dcn_clear_status<<<1, 1, 0, s>>>(status);
  return cudaGetLastError();
}

cudaError_t tc_set_attributes(size_t smem) {
  cudaError_t e = cudaFuncSetAttribute(dcn_fwd_tc_bf16<float>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(dcn_fwd_tc_bf16<__nv_bfloat16>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

cudaError_t launch_tc_bf16(const Geom &g, const TcPlan &tp, const Ptrs &p, int dtype,
                           const __nv_bfloat16 *xcl, const void *wtiles, int *status,
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
  if (dtype == DCN_DTYPE_F32)
    dcn_fwd_tc_bf16<float><<<tp.grid, kTcThreads, tp.smem, s>>>(a);
  else
    dcn_fwd_tc_bf16<__nv_bfloat16><<<tp.grid, kTcThreads, tp.smem, s>>>(a);
  return cudaGetLastError();
}

}  // namespace dcn
