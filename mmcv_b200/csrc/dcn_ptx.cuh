// PTX wrappers and small device helpers shared by the tensor-core kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "dcn_internal.cuh"

namespace dcn {
namespace {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s per wait
// How long one mbarrier.try_wait may keep the thread suspended in hardware (it wakes at once
// when the phase completes): waiting warps then take no issue slots from the producers.
constexpr uint32_t kSuspendHintNs = 20000u;
enum { kModeBf16 = 0, kModeTf32x3 = 1, kModeF16 = 2 };  // arithmetic modes of the contraction
constexpr int kTileBytes = kBM * 128;  // one operand tile: 128 rows of 128 bytes (16 KiB)

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
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the block is aborting.  kBackoff: sleep between polls;
// used by the roles that wait long and are not on the critical path (epilogue, loader), so
// that their polling does not take issue slots from the producer warps.
template <bool kBackoff = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_s,
                                          int *status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (kBackoff) __nanosleep(200);
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
// Phase timer for the optional counters: adds the clock cycles since `t0` to slot `i` and
// restarts `t0`.
struct PhaseTimer {
  unsigned long long *c;
  long long t0;
  __device__ __forceinline__ PhaseTimer(unsigned long long *counters, bool elected)
      : c(elected ? counters : nullptr), t0(0) {
    if (c) t0 = clock64();
  }
  __device__ __forceinline__ void lap(int i) {
    if (c) {
      // fire-and-forget reductions: a read-modify-write here would put a memory round
      // trip into the phase that follows
      const long long t1 = clock64();
      atomicAdd(c + i, (unsigned long long)(t1 - t0));
      t0 = t1;
    }
  }
  __device__ __forceinline__ void count(int i) {
    if (c) atomicAdd(c + i, 1ull);
  }
};

// The kernels use PhaseTimer only when built with -DDCN_B200_PHASE_COUNTERS (the timers cost
// the gather / producer warps four registers and a dozen instructions per stage); otherwise
// this stand-in, whose calls vanish.
struct NoTimer {
  __device__ __forceinline__ NoTimer(unsigned long long *, bool) {}
  __device__ __forceinline__ void lap(int) {}
  __device__ __forceinline__ void count(int) {}
};
#ifdef DCN_B200_PHASE_COUNTERS
using StageTimer = PhaseTimer;
#else
using StageTimer = NoTimer;
#endif

__device__ __forceinline__ void prefetch_l2(const void *p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
// Loads whose issue order the compiler must keep (volatile): a batch of them is issued
// back to back so that their latencies overlap, and only then is the first one consumed.
// The value is returned raw; converting it (raw_to_float) is a use and waits for the load.
__device__ __forceinline__ uint32_t ldg_raw_ordered(const float *p) {
  uint32_t v;
  asm volatile("ld.global.nc.b32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_raw_ordered(const __nv_bfloat16 *p) {
  uint32_t v;  // a 32-bit register: two 16-bit results packed into one would be a use
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_raw_ordered(const __half *p) {
  uint32_t v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
template <typename T> struct RawOf {
  using type = uint32_t;
  static __device__ __forceinline__ float to_float(uint32_t v) { return __uint_as_float(v); }
};
template <> struct RawOf<__nv_bfloat16> {
  using type = uint32_t;
  static __device__ __forceinline__ float to_float(uint32_t v) { return __uint_as_float(v << 16); }
};
template <> struct RawOf<__half> {
  using type = uint32_t;
  static __device__ __forceinline__ float to_float(uint32_t v) {
    return __half2float(__ushort_as_half((unsigned short)v));
  }
};
// 16-byte read-only load, zero when `take` is 0.  `tok` is passed through untouched; code that
// must come after this load's issue takes `tok` as an input.
__device__ __forceinline__ uint4 ldg16_pinned(const void *p, uint32_t take, uint32_t &tok) {
  uint4 r;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.u32 p, %5, 0;\n\t"
      "mov.u32 %0, 0;\n\tmov.u32 %1, 0;\n\tmov.u32 %2, 0;\n\tmov.u32 %3, 0;\n\t"
      "@p ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];\n\t}"
      : "=&r"(r.x), "=&r"(r.y), "=&r"(r.z), "=&r"(r.w)
      : "l"(p), "r"(take), "r"(tok));
  asm volatile("" : "+r"(tok));
  return r;
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
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// True in exactly one lane of the (fully converged) warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
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

__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t u) {
  return *reinterpret_cast<const __nv_bfloat162 *>(&u);
}
__device__ __forceinline__ uint32_t bf162_bits(__nv_bfloat162 h) {
  return *reinterpret_cast<const uint32_t *>(&h);
}

// A table entry's corner weights in the form the blends take: each 16-bit weight twice (a
// pair), or the four fp32 weights as they are.
template <int MODE>
__device__ __forceinline__ uint4 table_weights(const uint2 &w) {
  return make_uint4(__byte_perm(w.x, 0u, 0x1010), __byte_perm(w.x, 0u, 0x3232),
                    __byte_perm(w.y, 0u, 0x1010), __byte_perm(w.y, 0u, 0x3232));
}
template <int MODE>
__device__ __forceinline__ uint4 table_weights(const uint4 &w) { return w; }

// Four consecutive elements (8- or 16-byte aligned) as floats, with one load.
__device__ __forceinline__ void load4_as_float(const float *p, float (&o)[4]) {
  const float4 v = *reinterpret_cast<const float4 *>(p);
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
__device__ __forceinline__ void load4_as_float(const __nv_bfloat16 *p, float (&o)[4]) {
  const uint2 v = *reinterpret_cast<const uint2 *>(p);
  o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
  o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
}
__device__ __forceinline__ void load4_as_float(const __half *p, float (&o)[4]) {
  const uint2 v = *reinterpret_cast<const uint2 *>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}

// The modulation value of a tap: the mask element, or its sigmoid when the tensor holds logits.
__device__ __forceinline__ float mask_value(const Geom &g, float m) {
  return g.mask_act == DCN_ACT_SIGMOID ? 1.f / (1.f + __expf(-m)) : m;
}

// Bilinear blend of four 8-channel bf16 corner vectors on packed bf16 FMAs: one multiply
// and three fused multiply-adds per channel pair, each rounding to bf16.  `w` holds each
// corner weight twice (a bf16 pair).
__device__ __forceinline__ uint4 blend8_bf16(const uint4 &w, const uint4 &q0, const uint4 &q1,
                                             const uint4 &q2, const uint4 &q3) {
  uint4 o;
  const __nv_bfloat162 w0 = as_bf162(w.x), w1 = as_bf162(w.y), w2 = as_bf162(w.z),
                       w3 = as_bf162(w.w);
  const uint32_t *a0 = reinterpret_cast<const uint32_t *>(&q0);
  const uint32_t *a1 = reinterpret_cast<const uint32_t *>(&q1);
  const uint32_t *a2 = reinterpret_cast<const uint32_t *>(&q2);
  const uint32_t *a3 = reinterpret_cast<const uint32_t *>(&q3);
  uint32_t *r = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 t = __hmul2(w0, as_bf162(a0[i]));
    t = __hfma2(w1, as_bf162(a1[i]), t);
    t = __hfma2(w2, as_bf162(a2[i]), t);
    t = __hfma2(w3, as_bf162(a3[i]), t);
    r[i] = bf162_bits(t);
  }
  return o;
}

// The same blend on packed fp16 FMAs (fp16 tensors).
__device__ __forceinline__ uint4 blend8_f16(const uint4 &w, const uint4 &q0, const uint4 &q1,
                                            const uint4 &q2, const uint4 &q3) {
  uint4 o;
  const __half2 *wh = reinterpret_cast<const __half2 *>(&w);
  const __half2 *a0 = reinterpret_cast<const __half2 *>(&q0);
  const __half2 *a1 = reinterpret_cast<const __half2 *>(&q1);
  const __half2 *a2 = reinterpret_cast<const __half2 *>(&q2);
  const __half2 *a3 = reinterpret_cast<const __half2 *>(&q3);
  __half2 *r = reinterpret_cast<__half2 *>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 t = __hmul2(wh[0], a0[i]);
    t = __hfma2(wh[1], a1[i], t);
    t = __hfma2(wh[2], a2[i], t);
    t = __hfma2(wh[3], a3[i], t);
    r[i] = t;
  }
  return o;
}

// Bilinear blend of four 4-channel fp32 corner vectors in fp32 (weights are fp32 bits),
// split into the TF32 high part (low 13 mantissa bits cleared) and the exact remainder.
__device__ __forceinline__ void blend4_tf32(const uint4 &w, const uint4 &q0, const uint4 &q1,
                                            const uint4 &q2, const uint4 &q3, uint4 &hi,
                                            uint4 &lo) {
  const float w0 = __uint_as_float(w.x), w1 = __uint_as_float(w.y), w2 = __uint_as_float(w.z),
              w3 = __uint_as_float(w.w);
  const uint32_t *a0 = reinterpret_cast<const uint32_t *>(&q0);
  const uint32_t *a1 = reinterpret_cast<const uint32_t *>(&q1);
  const uint32_t *a2 = reinterpret_cast<const uint32_t *>(&q2);
  const uint32_t *a3 = reinterpret_cast<const uint32_t *>(&q3);
  uint32_t *h = reinterpret_cast<uint32_t *>(&hi);
  uint32_t *l = reinterpret_cast<uint32_t *>(&lo);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float t = w0 * __uint_as_float(a0[i]);
    t = fmaf(w1, __uint_as_float(a1[i]), t);
    t = fmaf(w2, __uint_as_float(a2[i]), t);
    t = fmaf(w3, __uint_as_float(a3[i]), t);
    const uint32_t hb = __float_as_uint(t) & 0xffffe000u;
    h[i] = hb;
    l[i] = __float_as_uint(t - __uint_as_float(hb));
  }
}


}  // namespace
}  // namespace dcn
