// SIMT (FFMA) kernels of the deformable-convolution forward: the shape-agnostic
// fp32-arithmetic path, and the on-device cross-check of the tensor-core path.
//
// Both kernels replace, in one launch, what the reference does with a gather kernel
// per sample (mmcv/ops/csrc/common/cuda/modulated_deform_conv_cuda_kernel.cuh:186-245,
// deform_conv_cuda_kernel.cuh:190-241), a column buffer in global memory, one GEMM
// per sample and group (mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:108-130) and
// a bias pass (same file, :135-137).  No column buffer is written.
#include "dcn_internal.cuh"

namespace dcn {

// ---------------------------------------------------------------------------------
// Direct kernel: one thread per output element.  Any shape, any kernel size.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
dcn_fwd_simt_direct(const Geom g, const T *__restrict__ x, const T *__restrict__ off,
                    const T *__restrict__ msk, const T *__restrict__ wgt,
                    const T *__restrict__ bias, T *__restrict__ out) {
  const long long total = g.P * g.Co;
  const long long plane = (long long)g.Ho * g.Wo;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    // pixel fastest, so that a warp reads neighbouring offsets and writes a row run
    const int wo = (int)(idx % g.Wo);
    const int ho = (int)((idx / g.Wo) % g.Ho);
    const int co = (int)((idx / plane) % g.Co);
    const int n = (int)(idx / (plane * g.Co));
    const int grp = co / g.Cog;
    const long long pix = (long long)ho * g.Wo + wo;
    const T *x_n = x + (long long)n * g.in_sn;
    const T *w_co = wgt + (long long)co * g.Cg * g.T;
    float acc = 0.f;
    const int c_begin = grp * g.Cg, c_end = c_begin + g.Cg;
    for (int c0 = c_begin; c0 < c_end;) {
      const int dgi = c0 / g.cpdg;
      const int c1 = min(c_end, (dgi + 1) * g.cpdg);
      const T *off_g = off ? off + (long long)n * g.off_sn + (long long)dgi * 2 * g.T * plane : nullptr;
      const T *msk_g = msk ? msk + (long long)n * g.msk_sn + (long long)dgi * g.T * plane : nullptr;
      for (int i = 0; i < g.kh; ++i)
        for (int j = 0; j < g.kw; ++j) {
          const int tap = i * g.kw + j;
          const float oh = off_g ? ld_as_float(off_g, (long long)(2 * tap) * plane + pix) : 0.f;
          const float ow = off_g ? ld_as_float(off_g, (long long)(2 * tap + 1) * plane + pix) : 0.f;
          const float m = msk_g ? ld_as_float(msk_g, (long long)tap * plane + pix) : 1.f;
          float4 wt;
          int h_low, w_low;
          tap_weights(oh, ow, m, ho * g.stride_h - g.pad_h + i * g.dil_h,
                      wo * g.stride_w - g.pad_w + j * g.dil_w, g.H, g.W, wt, h_low, w_low);
          if (wt.x == 0.f && wt.y == 0.f && wt.z == 0.f && wt.w == 0.f) continue;
          const long long o00 = (long long)h_low * g.in_sh + (long long)w_low * g.in_sw;
          for (int c = c0; c < c1; ++c) {
            const T *pl = x_n + (long long)c * g.in_sc + o00;
            float v = 0.f;
            if (wt.x != 0.f) v += wt.x * ld_as_float(pl, 0);
            if (wt.y != 0.f) v += wt.y * ld_as_float(pl, g.in_sw);
            if (wt.z != 0.f) v += wt.z * ld_as_float(pl, g.in_sh);
            if (wt.w != 0.f) v += wt.w * ld_as_float(pl, g.in_sh + g.in_sw);
            acc += v * ld_as_float(w_co, (long long)(c - c_begin) * g.T + tap);
          }
        }
      c0 = c1;
    }
    if (bias) acc += ld_as_float(bias, co);
    acc = apply_act(g, co, acc);
    st_from_float(out, (long long)n * g.out_sn + (long long)co * plane + pix, acc);
  }
}

cudaError_t launch_simt_direct(const Geom &g, const Ptrs &p, int dtype, cudaStream_t s) {
  const long long total = g.P * g.Co;
  if (total == 0) return cudaSuccess;
  const int block = 256;
  long long blocks = (total + block - 1) / block;
  if (blocks > 148LL * 64) blocks = 148LL * 64;
  if (dtype == DCN_DTYPE_F32)
    dcn_fwd_simt_direct<float><<<(int)blocks, block, 0, s>>>(
        g, (const float *)p.input, (const float *)p.offset, (const float *)p.mask,
        (const float *)p.weight, (const float *)p.bias, (float *)p.output);
  else
    dcn_fwd_simt_direct<__nv_bfloat16><<<(int)blocks, block, 0, s>>>(
        g, (const __nv_bfloat16 *)p.input, (const __nv_bfloat16 *)p.offset,
        (const __nv_bfloat16 *)p.mask, (const __nv_bfloat16 *)p.weight,
        (const __nv_bfloat16 *)p.bias, (__nv_bfloat16 *)p.output);
  return cudaGetLastError();
}

}  // namespace dcn
