// Multi-scale deformable attention (the sampler of Deformable DETR), forward and backward, for
// sm_100a.  It is the deformable convolutions' sibling: the same bilinear gather with a gate
// and per-corner validity, applied to `num_levels` feature maps that lie one after another in
// `value`, followed by a weighted sum over (level, point) instead of a contraction with weights.
//
// Replaces ms_deformable_im2col_gpu_kernel and the ms_deformable_col2im_gpu_kernel_* family
// (mmcv/ops/csrc/common/cuda/ms_deform_attn_cuda_kernel.cuh:18-66,198-259,261-795) and their
// launch loops over im2col_step chunks (mmcv/ops/csrc/pytorch/cuda/ms_deform_attn_cuda.cu:
// 203-351).  One launch covers the whole batch.
//
// Work split.  value is [B][S][M][D] (D channels of a head contiguous), so a thread owns a
// vector of V consecutive channels of one (batch, query, head): 16-byte loads for 16-bit
// tensors (V = 8) and fp32 (V = 4) when D allows, else V = 1.  The D/V threads of one
// (batch, query, head) are neighbouring lanes; they walk the same L x P samples, compute the
// same four weights (cheap, and no shared memory or synchronisation is needed), and read
// D contiguous channels of each corner between them: every corner read of a warp is a set of
// full 32-byte sectors.  The operation moves bytes, not flops: per output vector it reads
// 4 * L * P corner vectors from L2/HBM and 3 * L * P scalars; its bound is the memory system.
//
// Backward: the same walk; grad_value by fp32 atomic adds (as the reference), and the
// gradients of the sampling locations and attention weights, which are sums over the D
// channels, are reduced over the D/V neighbouring lanes with warp shuffles when D/V is a power
// of two up to 32 (one lane then stores: each (b, q, m, l, p) has exactly one owner group, no
// atomics), else by atomic adds.  All three gradients are produced in fp32.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>

#include "dcn_b200.h"

namespace dcn {

int set_error(int code, const char *msg);

namespace {

struct MsdaGeom {
  long long B, S, Q;
  int M, D, L, P;
};

template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float ld(const float *p) { return *p; }
  static __device__ __forceinline__ void st(float *p, float v) { *p = v; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float ld(const __half *p) { return __half2float(*p); }
  static __device__ __forceinline__ void st(__half *p, float v) { *p = __float2half_rn(v); }
};

// V consecutive elements as floats; V * sizeof(T) is 16 bytes (one load) or V is 1.
template <typename T, int V>
__device__ __forceinline__ void load_vec(const T *p, float (&o)[V]) {
  if constexpr (V == 1) {
    o[0] = Elem<T>::ld(p);
  } else if constexpr (sizeof(T) == 4) {
    const float4 v = __ldg(reinterpret_cast<const float4 *>(p));
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  } else {
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (std::is_same_v<T, __nv_bfloat16>) {
        o[2 * i] = __uint_as_float(w[i] << 16);
        o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        o[2 * i] = f.x;
        o[2 * i + 1] = f.y;
      }
    }
  }
}

template <typename T, int V>
__device__ __forceinline__ void store_vec(T *p, const float (&v)[V]) {
  if constexpr (V == 1) {
    Elem<T>::st(p, v[0]);
  } else if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (std::is_same_v<T, __nv_bfloat16>) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t *>(&h);
      } else {
        const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t *>(&h);
      }
    }
    *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// One sample: gate, corner weights and corner element offsets inside the level (in elements of
// value, relative to the level's first pixel of this batch entry, head and channel 0).
// Follows ms_deform_attn_im2col_bilinear and the gate of its caller
// (ms_deform_attn_cuda_kernel.cuh:18-66, :242): h_im = loc_h * H - 0.5, sampled only if
// h_im > -1 && w_im > -1 && h_im < H && w_im < W; a corner outside the map contributes 0.
struct Sample {
  float w[4];       // hh*hw, hh*lw, lh*hw, lh*lw
  int o[4];         // element offsets of the four corners (one batch entry holds fewer than 2^31 elements)
  bool ok[4];
  float hh, hw, lh, lw;
  bool live;
};
__device__ __forceinline__ Sample make_sample(float loc_w, float loc_h, int H, int W, int pix_stride) {
  Sample s;
  const float h_im = loc_h * (float)H - 0.5f, w_im = loc_w * (float)W - 0.5f;
  s.live = h_im > -1.f && w_im > -1.f && h_im < (float)H && w_im < (float)W;
  const float hf = floorf(h_im), wf = floorf(w_im);
  const int h_low = (int)hf, w_low = (int)wf;
  s.lh = h_im - hf; s.lw = w_im - wf;
  s.hh = 1.f - s.lh; s.hw = 1.f - s.lw;
  s.w[0] = s.hh * s.hw; s.w[1] = s.hh * s.lw; s.w[2] = s.lh * s.hw; s.w[3] = s.lh * s.lw;
  const bool top = h_low >= 0, left = w_low >= 0, bot = h_low + 1 <= H - 1, right = w_low + 1 <= W - 1;
  s.ok[0] = s.live && top && left; s.ok[1] = s.live && top && right;
  s.ok[2] = s.live && bot && left; s.ok[3] = s.live && bot && right;
  const int base = (h_low * W + w_low) * pix_stride;
  s.o[0] = base; s.o[1] = base + pix_stride;
  s.o[2] = base + W * pix_stride; s.o[3] = s.o[2] + pix_stride;
  return s;
}

template <typename T, int V>
__global__ void __launch_bounds__(256)
msda_forward_kernel(const MsdaGeom g, const T *__restrict__ value, const int64_t *__restrict__ shapes,
                    const int64_t *__restrict__ starts, const T *__restrict__ loc,
                    const T *__restrict__ attn, T *__restrict__ out) {
  const int vec_per_head = g.D / V;
  const long long total = g.B * g.Q * g.M * vec_per_head;
  const int pix_stride = g.M * g.D;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int cv = (int)(idx % vec_per_head);
    const long long bqm = idx / vec_per_head;          // (b * Q + q) * M + m
    const int m = (int)(bqm % g.M);
    const long long b = bqm / ((long long)g.M * g.Q);
    const T *val_b = value + b * g.S * pix_stride + (long long)m * g.D + cv * V;
    const T *loc_p = loc + bqm * g.L * g.P * 2;
    const T *att_p = attn + bqm * g.L * g.P;
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    for (int l = 0; l < g.L; ++l) {
      const int H = (int)shapes[2 * l], W = (int)shapes[2 * l + 1];
      const T *val_l = val_b + starts[l] * pix_stride;
      for (int p = 0; p < g.P; ++p) {
        const float loc_w = Elem<T>::ld(loc_p), loc_h = Elem<T>::ld(loc_p + 1);
        const float aw = Elem<T>::ld(att_p);
        loc_p += 2; att_p += 1;
        const Sample s = make_sample(loc_w, loc_h, H, W, pix_stride);
        if (!s.live) continue;
        float v[V];
#pragma unroll
        for (int i = 0; i < V; ++i) v[i] = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (!s.ok[k]) continue;
          float c[V];
          load_vec<T, V>(val_l + s.o[k], c);
#pragma unroll
          for (int i = 0; i < V; ++i) v[i] += s.w[k] * c[i];
        }
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] += v[i] * aw;
      }
    }
    store_vec<T, V>(out + bqm * g.D + cv * V, acc);
  }
}

template <typename T, int V, bool kShuffle>
__global__ void __launch_bounds__(256)
msda_backward_kernel(const MsdaGeom g, const T *__restrict__ value, const int64_t *__restrict__ shapes,
                     const int64_t *__restrict__ starts, const T *__restrict__ loc,
                     const T *__restrict__ attn, const T *__restrict__ gout,
                     float *__restrict__ gvalue, float *__restrict__ gloc, float *__restrict__ gattn) {
  const int vec_per_head = g.D / V;
  const long long total = g.B * g.Q * g.M * vec_per_head;
  const long long padded = kShuffle ? (total + 31) / 32 * 32 : total;   // whole warps take part in the shuffles
  const int pix_stride = g.M * g.D;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < padded;
       idx += (long long)gridDim.x * blockDim.x) {
    const bool active = idx < total;
    const long long id = active ? idx : total - 1;
    const int cv = (int)(id % vec_per_head);
    const long long bqm = id / vec_per_head;
    const int m = (int)(bqm % g.M);
    const long long b = bqm / ((long long)g.M * g.Q);
    const long long voff = b * g.S * pix_stride + (long long)m * g.D + cv * V;
    const T *loc_p = loc + bqm * g.L * g.P * 2;
    const T *att_p = attn + bqm * g.L * g.P;
    float *gloc_p = gloc + bqm * g.L * g.P * 2;
    float *gatt_p = gattn + bqm * g.L * g.P;
    float go[V];
    load_vec<T, V>(gout + bqm * g.D + cv * V, go);
    for (int l = 0; l < g.L; ++l) {
      const int H = (int)shapes[2 * l], W = (int)shapes[2 * l + 1];
      const long long lbase = voff + starts[l] * pix_stride;
      for (int p = 0; p < g.P; ++p) {
        const float loc_w = Elem<T>::ld(loc_p), loc_h = Elem<T>::ld(loc_p + 1);
        const float aw = Elem<T>::ld(att_p);
        const Sample s = make_sample(loc_w, loc_h, H, W, pix_stride);
        // sums over this thread's channels: d(out)/d(weight), and the h / w derivative terms
        float g_attn = 0.f, g_h = 0.f, g_w = 0.f;
        if (s.live && active) {
          float c[4][V];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
#pragma unroll
            for (int i = 0; i < V; ++i) c[k][i] = 0.f;
            if (s.ok[k]) {
              load_vec<T, V>(value + lbase + s.o[k], c[k]);
#pragma unroll
              for (int i = 0; i < V; ++i) atomicAdd(gvalue + lbase + s.o[k] + i, s.w[k] * go[i] * aw);
            }
          }
#pragma unroll
          for (int i = 0; i < V; ++i) {
            const float val = s.w[0] * c[0][i] + s.w[1] * c[1][i] + s.w[2] * c[2][i] + s.w[3] * c[3][i];
            const float tg = go[i] * aw;
            g_attn += go[i] * val;
            g_h += tg * (-s.hw * c[0][i] - s.lw * c[1][i] + s.hw * c[2][i] + s.lw * c[3][i]);
            g_w += tg * (-s.hh * c[0][i] + s.hh * c[1][i] - s.lh * c[2][i] + s.lh * c[3][i]);
          }
          g_h *= (float)H;
          g_w *= (float)W;
        }
        if constexpr (kShuffle) {
          // the vec_per_head lanes of this (b, q, m) are neighbours and never straddle a warp
#pragma unroll
          for (int d = 1; d < 32; d <<= 1) {
            if (d < vec_per_head) {
              g_attn += __shfl_xor_sync(0xffffffffu, g_attn, d);
              g_h += __shfl_xor_sync(0xffffffffu, g_h, d);
              g_w += __shfl_xor_sync(0xffffffffu, g_w, d);
            }
          }
          if (active && cv == 0) {
            gatt_p[0] = g_attn;
            gloc_p[0] = g_w;
            gloc_p[1] = g_h;
          }
        } else if (active && s.live) {
          atomicAdd(gatt_p, g_attn);
          atomicAdd(gloc_p, g_w);
          atomicAdd(gloc_p + 1, g_h);
        }
        loc_p += 2; att_p += 1; gloc_p += 2; gatt_p += 1;
      }
    }
  }
}

int grid_for(long long total) {
  long long blocks = (total + 255) / 256;
  const long long cap = 148LL * 16;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

template <typename T>
cudaError_t launch_forward(const MsdaGeom &g, const void *value, const int64_t *shapes, const int64_t *starts,
                           const void *loc, const void *attn, void *out, bool vec_ok, cudaStream_t s) {
  constexpr int V = 16 / (int)sizeof(T);
  if (vec_ok) {
    const long long total = g.B * g.Q * g.M * (g.D / V);
    msda_forward_kernel<T, V><<<grid_for(total), 256, 0, s>>>(g, (const T *)value, shapes, starts, (const T *)loc,
                                                               (const T *)attn, (T *)out);
  } else {
    const long long total = g.B * g.Q * g.M * g.D;
    msda_forward_kernel<T, 1><<<grid_for(total), 256, 0, s>>>(g, (const T *)value, shapes, starts, (const T *)loc,
                                                               (const T *)attn, (T *)out);
  }
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_backward(const MsdaGeom &g, const void *value, const int64_t *shapes, const int64_t *starts,
                            const void *loc, const void *attn, const void *gout, float *gvalue, float *gloc,
                            float *gattn, bool vec_ok, cudaStream_t s) {
  constexpr int V = 16 / (int)sizeof(T);
  const int vph = vec_ok ? g.D / V : g.D;
  const bool pow2 = vph >= 1 && vph <= 32 && (vph & (vph - 1)) == 0;
  const long long total = g.B * g.Q * g.M * vph;
#define MSDA_BWD(VV, SH)                                                                                    \
  msda_backward_kernel<T, VV, SH><<<grid_for(total), 256, 0, s>>>(g, (const T *)value, shapes, starts,      \
                                                                  (const T *)loc, (const T *)attn,          \
                                                                  (const T *)gout, gvalue, gloc, gattn)
  if (vec_ok && pow2) MSDA_BWD(V, true);
  else if (vec_ok) MSDA_BWD(V, false);
  else if (pow2) MSDA_BWD(1, true);
  else MSDA_BWD(1, false);
#undef MSDA_BWD
  return cudaGetLastError();
}

struct DeviceScopeM {
  int prev = -1;
  bool switched = false;
  cudaError_t err;
  explicit DeviceScopeM(int device) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != device) {
      err = cudaSetDevice(device);
      switched = err == cudaSuccess;
    }
  }
  ~DeviceScopeM() {
    if (switched) cudaSetDevice(prev);
  }
};

int check_geom(int32_t dtype, int64_t B, int64_t S, int64_t M, int64_t D, int64_t L, int64_t Q, int64_t P,
               MsdaGeom *g) {
  if (dtype != DCN_DTYPE_F32 && dtype != DCN_DTYPE_BF16 && dtype != DCN_DTYPE_F16)
    return set_error(DCN_ERR_UNSUPPORTED, "multi-scale deformable attention takes fp32, bf16 and fp16 tensors");
  if (B < 0 || S < 0 || Q < 0 || M <= 0 || D <= 0 || L <= 0 || P <= 0)
    return set_error(DCN_ERR_ARG, "multi-scale deformable attention: sizes must be positive");
  if (M * D > 2147483647LL / 4 || (S + 2) * M * D >= 2147483647LL || L > 1024 || P > 1024)
    return set_error(DCN_ERR_UNSUPPORTED, "multi-scale deformable attention: problem too large");
  g->B = B; g->S = S; g->Q = Q; g->M = (int)M; g->D = (int)D; g->L = (int)L; g->P = (int)P;
  return DCN_OK;
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace
}  // namespace dcn

using namespace dcn;

extern "C" {

int dcn_msda_forward(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                     const void *sampling_loc, const void *attn_weight, void *output, int32_t dtype,
                     int64_t batch, int64_t spatial_size, int64_t num_heads, int64_t channels,
                     int64_t num_levels, int64_t num_query, int64_t num_point, int32_t device,
                     void *stream) {
  MsdaGeom g;
  int rc = check_geom(dtype, batch, spatial_size, num_heads, channels, num_levels, num_query, num_point, &g);
  if (rc) return rc;
  if (g.B * g.Q == 0) return DCN_OK;   // nothing to write
  if (!value || !spatial_shapes || !level_start_index || !sampling_loc || !attn_weight || !output)
    return set_error(DCN_ERR_ARG, "multi-scale deformable attention: NULL pointer");
  DeviceScopeM scope(device);
  if (scope.err != cudaSuccess) return set_error(DCN_ERR_CUDA, cudaGetErrorString(scope.err));
  const int esz = dtype == DCN_DTYPE_F32 ? 4 : 2;
  const bool vec_ok = g.D % (16 / esz) == 0 && aligned16(value) && aligned16(output);
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e;
  if (dtype == DCN_DTYPE_F32)
    e = launch_forward<float>(g, value, spatial_shapes, level_start_index, sampling_loc, attn_weight, output, vec_ok, s);
  else if (dtype == DCN_DTYPE_BF16)
    e = launch_forward<__nv_bfloat16>(g, value, spatial_shapes, level_start_index, sampling_loc, attn_weight, output,
                                      vec_ok, s);
  else
    e = launch_forward<__half>(g, value, spatial_shapes, level_start_index, sampling_loc, attn_weight, output, vec_ok, s);
  if (e != cudaSuccess) return set_error(DCN_ERR_CUDA, cudaGetErrorString(e));
  return DCN_OK;
}

int dcn_msda_backward(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                      const void *sampling_loc, const void *attn_weight, const void *grad_output,
                      float *grad_value, float *grad_sampling_loc, float *grad_attn_weight, int32_t dtype,
                      int64_t batch, int64_t spatial_size, int64_t num_heads, int64_t channels,
                      int64_t num_levels, int64_t num_query, int64_t num_point, int32_t device,
                      void *stream) {
  MsdaGeom g;
  int rc = check_geom(dtype, batch, spatial_size, num_heads, channels, num_levels, num_query, num_point, &g);
  if (rc) return rc;
  if (g.B * g.Q == 0) return DCN_OK;
  if (!value || !spatial_shapes || !level_start_index || !sampling_loc || !attn_weight || !grad_output ||
      !grad_value || !grad_sampling_loc || !grad_attn_weight)
    return set_error(DCN_ERR_ARG, "multi-scale deformable attention: NULL pointer");
  DeviceScopeM scope(device);
  if (scope.err != cudaSuccess) return set_error(DCN_ERR_CUDA, cudaGetErrorString(scope.err));
  const int esz = dtype == DCN_DTYPE_F32 ? 4 : 2;
  const bool vec_ok = g.D % (16 / esz) == 0 && aligned16(value) && aligned16(grad_output);
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e;
  if (dtype == DCN_DTYPE_F32)
    e = launch_backward<float>(g, value, spatial_shapes, level_start_index, sampling_loc, attn_weight, grad_output,
                               grad_value, grad_sampling_loc, grad_attn_weight, vec_ok, s);
  else if (dtype == DCN_DTYPE_BF16)
    e = launch_backward<__nv_bfloat16>(g, value, spatial_shapes, level_start_index, sampling_loc, attn_weight,
                                       grad_output, grad_value, grad_sampling_loc, grad_attn_weight, vec_ok, s);
  else
    e = launch_backward<__half>(g, value, spatial_shapes, level_start_index, sampling_loc, attn_weight, grad_output,
                                grad_value, grad_sampling_loc, grad_attn_weight, vec_ok, s);
  if (e != cudaSuccess) return set_error(DCN_ERR_CUDA, cudaGetErrorString(e));
  return DCN_OK;
}

}  // extern "C"
