// Ordinary convolution on the tensor cores for sm_100a: the offset / mask branch of the Pack
// layers (mmcv/ops/modulated_deform_conv.py:311-335, mmcv/ops/deform_conv.py:397-415), which the
// reference gives to a library convolution.
//
// Same implicit GEMM as the deformable kernels, out[p, co] = sum_k A[p, k] * Wt[co, k], with
// k = (64-channel chunk, tap, channel).  With all offsets zero the A tile of a tap is the
// input shifted by the tap's displacement, so no thread computes anything for it: one lane
// issues, per k-stage, a 4-D tensor-map box load (cp.async.bulk.tensor) of [64 channels x tile
// width x tile height] from the channels-last copy of the input that carries a one-pixel zero
// border (the same copy the deformable kernel reads), with the convolution's stride as the
// box's element stride, its dilation in the start coordinate, and zero fill outside the tensor
// as the rest of the padding.  The copy engine writes the 128-byte-swizzled layout tcgen05.mma
// reads.  The weight stage arrives by a bulk copy on the same barrier.  One warp issues the
// MMAs (fp32 accumulators double-buffered in tensor memory), four warps run the epilogue
// (bias, optional sigmoid on a channel range, NCHW stores).  Every wait is bounded.
#include <atomic>
#include <cstring>

#include <cuda.h>

#include "dcn_internal.cuh"
#include "dcn_ptx.cuh"

namespace dcn {

namespace {

constexpr int kConvThreads = 6 * 32;   // 4 epilogue warps, MMA warp, loader warp

struct alignas(64) ConvArgs {
  CUtensorMap in_map;   // padded channels-last input [N][H+2][W+2][C], box [64][TW][TH][1]
  Geom g;
  TcPlan tp;
  const uint8_t *wtiles;
  const void *bias;
  void *output;
  int *status;
  unsigned long long wait_limit_ns;
  int stages;
};

__device__ __forceinline__ bool conv_wait(uint32_t bar, uint32_t parity, volatile int *abort_s, int *status,
                                          int code, unsigned long long limit, unsigned backoff) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (backoff) __nanosleep(backoff);
    if ((it & 15u) == 0u) {
      if (*abort_s) return false;
      if (globaltimer_ns() - t0 > limit) {
        *abort_s = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void conv_tma_load_4d(uint32_t dst, const CUtensorMap *map, int c0, int c1,
                                                 int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void conv_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

struct ConvTile {
  int n, ho0, wo0, grp, nt;
};
__device__ __forceinline__ ConvTile conv_decode(uint32_t item, const Geom &g, const TcPlan &tp) {
  const uint32_t per_mt = (uint32_t)(g.groups * tp.NT);
  const uint32_t mt = item / per_mt;
  const uint32_t rem = item - mt * per_mt;
  const uint32_t tiles_img = (uint32_t)(tp.tiles_x * tp.tiles_y);
  ConvTile t;
  t.n = (int)(mt / tiles_img);
  const uint32_t ti = mt - (uint32_t)t.n * tiles_img;
  const uint32_t ty = ti / (uint32_t)tp.tiles_x;
  t.ho0 = (int)ty * (kBM >> tp.tw_log2);
  t.wo0 = (int)(ti - ty * (uint32_t)tp.tiles_x) << tp.tw_log2;
  t.grp = (int)(rem / (uint32_t)tp.NT);
  t.nt = (int)rem - t.grp * tp.NT;
  return t;
}

}  // namespace

size_t conv_smem_bytes(const TcPlan &tp, int stages) {
  return 1024 + 1024 + (size_t)stages * (kTileBytes + (size_t)tp.BN * 128) + (size_t)2 * tp.BN * tp.io_bytes + 32;
}

template <typename TIO, int MODE>
__global__ void __launch_bounds__(kConvThreads, 1) dcn_conv_tma(const __grid_constant__ ConvArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const Geom &g = a.g;
  const TcPlan &tp = a.tp;
  const int ST = a.stages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // control block: barriers, tensor-memory slot, abort flag; then the operand and weight rings
  const uint32_t bar0 = smem_u32(smem);
  const uint32_t full = bar0, empty = full + 8 * ST, tmem_full = empty + 8 * ST, tmem_empty = tmem_full + 16;
  uint32_t *tmem_slot = (uint32_t *)(smem + 896);
  volatile int *abort_s = (volatile int *)(smem + 904);
  uint8_t *ring_a = smem + 1024;
  const uint32_t b_stage_bytes = (uint32_t)tp.BN * 128u;
  uint8_t *ring_b = ring_a + (size_t)ST * kTileBytes;
  uint8_t *bias_s = ring_b + (size_t)ST * b_stage_bytes;
  const unsigned long long limit = a.wait_limit_ns;

  if (threadIdx.x == 0) {
    for (int i = 0; i < ST; ++i) {
      mbar_init(full + 8 * i, 1);
      mbar_init(empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tmem_full + 8 * i, 1);
      mbar_init(tmem_empty + 8 * i, 4);
    }
    *abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(tmem_slot), (uint32_t)tp.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t items = (uint32_t)tp.items;
  const long long plane = (long long)g.Ho * g.Wo;
  const int tw_mask = (1 << tp.tw_log2) - 1;

  if (warp < 4) {
    // ------------------------------ epilogue ------------------------------
    TIO *out = (TIO *)a.output;
    const TIO *bias = (const TIO *)a.bias;
    const int row = warp * 32 + lane;
    const int ty = row >> tp.tw_log2, tx = row & tw_mask;
    const bool act_any = g.act == DCN_ACT_SIGMOID && g.act_hi > g.act_lo;
    uint32_t li = 0;
    int staged_co0[2] = {-1, -1};
    for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, ++li) {
      const ConvTile t = conv_decode(item, g, tp);
      const int buf = (int)(li & 1);
      const int ncols = min(tp.BN, g.Cog - t.nt * tp.BN);
      const int co0 = t.grp * g.Cog + t.nt * tp.BN;
      const bool act_tile = act_any && co0 < g.act_hi && co0 + ncols > g.act_lo;
      bool ok = conv_wait(tmem_full + 8 * buf, (li >> 1) & 1u, abort_s, a.status, 3, limit, 200);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      TIO *bias_w = reinterpret_cast<TIO *>(bias_s) + buf * tp.BN;
      if (co0 != staged_co0[buf]) {
        __syncwarp();
        for (int i = lane; i < tp.BN; i += 32)
          st_from_float(bias_w, i, (bias && i < ncols) ? ld_as_float(bias, co0 + i) : 0.f);
        __syncwarp();
        staged_co0[buf] = co0;
      }
      const uint32_t taddr = tmem_base + (uint32_t)(buf * tp.BN) + ((uint32_t)(warp * 32) << 16);
      const int ho = t.ho0 + ty, wo = t.wo0 + tx;
      const bool valid = ho < g.Ho && wo < g.Wo;
      TIO *orow = out + (long long)t.n * g.out_sn + (long long)co0 * plane + (long long)ho * g.Wo + wo;
#pragma unroll 1
      for (int c0 = 0; c0 < ncols; c0 += 16) {
        uint32_t r[16];
        conv_tmem_ld16(taddr + (uint32_t)c0, r);
        tmem_ld_wait();
        const TIO *bs = bias_w + c0;
        TIO *oc = orow + (long long)c0 * plane;
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          float b4[4];
          load4_as_float(bs + 4 * j4, b4);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int j = 4 * j4 + k;
            float v = __uint_as_float(r[j]) + b4[k];
            if (act_tile) v = apply_act(g, co0 + c0 + j, v);
            if (valid && c0 + j < ncols) st_from_float(oc, (long long)j * plane, v);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty + 8 * buf);
    }
  } else if (warp == 4) {
    // ------------------------------ MMA issuer ------------------------------
    constexpr uint32_t kFmt = MODE == kModeBf16 ? 1u : 0u;
    const uint32_t idesc = (1u << 4) | (kFmt << 7) | (kFmt << 10) | ((uint32_t)(tp.BN >> 3) << 17) |
                           ((uint32_t)(kBM >> 4) << 24);
    uint32_t st = 0, ph = 0, li = 0;
    bool ok = true;
    for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x, ++li) {
      const int buf = (int)(li & 1);
      ok = __all_sync(0xffffffffu, conv_wait(tmem_empty + 8 * buf, ((li >> 1) & 1u) ^ 1u, abort_s, a.status, 4, limit, 0));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)(buf * tp.BN);
      for (int ks = 0; ks < tp.S; ++ks) {
        ok = __all_sync(0xffffffffu, conv_wait(full + 8 * st, ph, abort_s, a.status, 5, limit, 0));
        if (!ok) break;
        tc_fence_after();
        const uint64_t adesc = smem_desc_sw128(smem_u32(ring_a) + st * (uint32_t)kTileBytes);
        const uint64_t bdesc = smem_desc_sw128(smem_u32(ring_b) + st * b_stage_bytes);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (ks | k) != 0 ? 1u : 0u);
          umma_commit(empty + 8 * st);
          if (ks == tp.S - 1) umma_commit(tmem_full + 8 * buf);
        }
        __syncwarp();
        if (++st == (uint32_t)ST) { st = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ loader ------------------------------
    if (lane == 0) {
      const uint32_t per_mt = (uint32_t)(g.groups * tp.NT);
      uint32_t st = 0, ph = 0;
      bool ok = true;
      for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const ConvTile t = conv_decode(item, g, tp);
        const uint8_t *src = a.wtiles + (size_t)(item % per_mt) * tp.S * b_stage_bytes;
        int ks = 0;
        for (int cc = 0; cc < tp.KC && ok; ++cc) {
          const int c0 = t.grp * g.Cg + cc * 64;
          for (int i = 0; i < g.kh && ok; ++i)
            for (int j = 0; j < g.kw; ++j, ++ks) {
              ok = conv_wait(empty + 8 * st, ph ^ 1u, abort_s, a.status, 7, limit, 50);
              if (!ok) break;
              mbar_arrive_expect_tx(full + 8 * st, (uint32_t)kTileBytes + b_stage_bytes);
              // start of the box in the padded tensor: (channel, column + 1, row + 1, sample)
              conv_tma_load_4d(smem_u32(ring_a) + st * (uint32_t)kTileBytes, &a.in_map, c0,
                               t.wo0 * g.stride_w - g.pad_w + j * g.dil_w + 1,
                               t.ho0 * g.stride_h - g.pad_h + i * g.dil_h + 1, t.n, full + 8 * st);
              bulk_copy_g2s(smem_u32(ring_b) + st * b_stage_bytes, src + (size_t)ks * b_stage_bytes,
                            b_stage_bytes, full + 8 * st);
              if (++st == (uint32_t)ST) { st = 0; ph ^= 1u; }
            }
        }
      }
    }
    __syncwarp();
  }

  if (*abort_s) {
    for (int i = 0; i < 20; ++i) __nanosleep(50000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)tp.tmem_cols);
  }
}

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn conv_encode_fn() {
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

template <typename TIO, int MODE>
cudaError_t conv_launch_one(const ConvArgs &a, const TcPlan &tp, size_t smem, cudaStream_t s) {
  auto kern = dcn_conv_tma<TIO, MODE>;
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
  kern<<<tp.grid, kConvThreads, smem, s>>>(a);
  return cudaGetLastError();
}

}  // namespace

// The convolution takes: 16-bit operands, channels per group a multiple of 64 or a single group
// (a 64-channel box must not reach into another group's channels), box dimensions <= 256.
bool conv_tma_supported(const Geom &g, const TcPlan &tp) {
  if (tp.op_format == 2) return false;
  if (!(g.Cg % 64 == 0 || g.groups == 1)) return false;
  if (g.C % 8 != 0) return false;
  if (g.stride_h > 8 || g.stride_w > 8) return false;
  return true;
}

cudaError_t launch_conv_tma(const Geom &g, const TcPlan &tp, const Ptrs &p, int dtype, const void *xpad,
                            const void *wtiles, int *status, unsigned long long wait_limit_ns,
                            cudaStream_t s) {
  if (tp.items == 0) return cudaSuccess;
  ConvArgs a;
  memset(&a, 0, sizeof(a));
  a.g = g;
  a.tp = tp;
  a.wtiles = (const uint8_t *)wtiles;
  a.bias = p.bias;
  a.output = p.output;
  a.status = status;
  a.wait_limit_ns = wait_limit_ns ? wait_limit_ns : kWaitLimitNs;
  // as many stages as fit (at most eight)
  int stages = 8;
  while (stages > 2 && conv_smem_bytes(tp, stages) > 200 * 1024) --stages;
  a.stages = stages;
  EncodeTiledFn enc = conv_encode_fn();
  if (!enc) return cudaErrorNotSupported;
  const cuuint32_t tw = 1u << tp.tw_log2, th = (cuuint32_t)kBM >> tp.tw_log2;
  const cuuint64_t dims[4] = {(cuuint64_t)g.C, (cuuint64_t)g.W + 2, (cuuint64_t)g.H + 2, (cuuint64_t)g.N};
  const cuuint64_t strides[3] = {(cuuint64_t)g.C * 2, (cuuint64_t)(g.W + 2) * g.C * 2,
                                 (cuuint64_t)(g.H + 2) * (g.W + 2) * g.C * 2};
  // the box spans the traversed extent; with a stride only every stride-th element is copied
  const cuuint32_t box[4] = {64, (tw - 1) * (cuuint32_t)g.stride_w + 1, (th - 1) * (cuuint32_t)g.stride_h + 1, 1};
  const cuuint32_t estr[4] = {1, (cuuint32_t)g.stride_w, (cuuint32_t)g.stride_h, 1};
  if (box[1] > 256 || box[2] > 256) return cudaErrorInvalidValue;
  if (enc(&a.in_map, tp.op_format == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
          const_cast<void *>(xpad), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  const size_t smem = conv_smem_bytes(tp, stages);
  if (dtype == DCN_DTYPE_F32) return conv_launch_one<float, kModeBf16>(a, tp, smem, s);
  if (dtype == DCN_DTYPE_F16) return conv_launch_one<__half, kModeF16>(a, tp, smem, s);
  return conv_launch_one<__nv_bfloat16, kModeBf16>(a, tp, smem, s);
}

}  // namespace dcn
