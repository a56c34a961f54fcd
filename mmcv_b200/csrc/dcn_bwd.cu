// Backward building blocks of (modulated) deformable convolution: the sampled column
// matrix, the scatter of column gradients to the input, and the gradients of offsets and
// mask.  The two matrix products of the backward (grad_columns = W^T grad_out and
// grad_weight += grad_out columns^T) are plain GEMMs and stay with the caller's BLAS.
//
// What they follow in the reference:
//   columns ........ modulated_deformable_im2col_gpu_kernel
//                    (mmcv/ops/csrc/common/cuda/modulated_deform_conv_cuda_kernel.cuh:186-245)
//   input scatter .. modulated_deformable_col2im_gpu_kernel (same file, :247-307): each column
//                    gradient, times the mask, goes to the (up to four) bilinear corners
//   coordinates .... modulated_deformable_col2im_coord_gpu_kernel (same file, :309-397) with
//                    dmcn_get_coordinate_weight (:134-183)
// and their unmodulated twins in deform_conv_cuda_kernel.cuh:243-365.  All arithmetic is fp32;
// tensors of the problem may be fp32 or bf16, gradients and columns are fp32.
#include "dcn_internal.cuh"

namespace dcn {

namespace {

// Position of one tap of one output pixel and the pieces the three kernels share.
struct Sample {
  bool inside;          // the reference's gate: -1 < h < H and -1 < w < W
  int h_low, w_low;
  float lh, lw, hh, hw; // fractional parts and their complements
  bool v1, v2, v3, v4;  // corner validity: (top,left) (top,right) (bottom,left) (bottom,right)
};

__device__ __forceinline__ Sample locate(float off_h, float off_w, int h_base, int w_base, int H,
                                         int W) {
  Sample s;
  const float h = (float)h_base + off_h, w = (float)w_base + off_w;
  s.inside = h > -1.f && w > -1.f && h < (float)H && w < (float)W;
  const float hf = floorf(h), wf = floorf(w);
  s.h_low = s.inside ? (int)hf : 0;
  s.w_low = s.inside ? (int)wf : 0;
  s.lh = h - hf; s.lw = w - wf;
  s.hh = 1.f - s.lh; s.hw = 1.f - s.lw;
  const bool top = s.h_low >= 0, left = s.w_low >= 0;
  const bool bot = s.h_low + 1 <= H - 1, right = s.w_low + 1 <= W - 1;
  s.v1 = s.inside && top && left;
  s.v2 = s.inside && top && right;
  s.v3 = s.inside && bot && left;
  s.v4 = s.inside && bot && right;
  return s;
}

template <typename T>
__device__ __forceinline__ void tap_inputs(const Geom &g, const T *off, const T *msk, int n,
                                           int dgi, int tap, long long pix, long long plane,
                                           float &oh, float &ow, float &m) {
  oh = 0.f; ow = 0.f; m = 1.f;
  if (off) {
    const T *o = off + (long long)n * g.off_sn + ((long long)dgi * 2 * g.T + 2 * tap) * plane + pix;
    oh = ld_as_float(o, 0);
    ow = ld_as_float(o, plane);
  }
  if (msk) m = ld_as_float(msk, (long long)n * g.msk_sn + ((long long)dgi * g.T + tap) * plane + pix);
}

// columns[(s*C + c)*T + tap][p], s = n - n0
template <typename T>
__global__ void __launch_bounds__(256)
dcn_bwd_columns_kernel(const Geom g, const T *__restrict__ x, const T *__restrict__ off,
                       const T *__restrict__ msk, int n0, int ns, float *__restrict__ col) {
  const long long plane = (long long)g.Ho * g.Wo;
  const long long total = (long long)ns * g.C * g.T * plane;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long pix = idx % plane;
    const int tap = (int)((idx / plane) % g.T);
    const int c = (int)((idx / (plane * g.T)) % g.C);
    const int s = (int)(idx / (plane * g.T * g.C));
    const int n = n0 + s;
    const int ho = (int)(pix / g.Wo), wo = (int)(pix - (long long)ho * g.Wo);
    const int i = tap / g.kw, j = tap - i * g.kw;
    float oh, ow, m;
    tap_inputs(g, off, msk, n, c / g.cpdg, tap, pix, plane, oh, ow, m);
    float4 wt;
    int h_low, w_low;
    tap_weights(oh, ow, m, ho * g.stride_h - g.pad_h + i * g.dil_h,
                wo * g.stride_w - g.pad_w + j * g.dil_w, g.H, g.W, wt, h_low, w_low);
    const T *pl = x + (long long)n * g.in_sn + (long long)c * g.in_sc + (long long)h_low * g.in_sh +
                  (long long)w_low * g.in_sw;
    float v = 0.f;
    if (wt.x != 0.f) v = fmaf(wt.x, ld_as_float(pl, 0), v);
    if (wt.y != 0.f) v = fmaf(wt.y, ld_as_float(pl, g.in_sw), v);
    if (wt.z != 0.f) v = fmaf(wt.z, ld_as_float(pl, g.in_sh), v);
    if (wt.w != 0.f) v = fmaf(wt.w, ld_as_float(pl, g.in_sh + g.in_sw), v);
    col[idx] = v;
  }
}

// grad_input[n][c][h][w] (fp32, NCHW-contiguous) += grad_columns * mask * corner weight
template <typename T>
__global__ void __launch_bounds__(256)
dcn_bwd_input_kernel(const Geom g, const T *__restrict__ off, const T *__restrict__ msk, int n0,
                     int ns, const float *__restrict__ gcol, float *__restrict__ gin) {
  const long long plane = (long long)g.Ho * g.Wo;
  const long long total = (long long)ns * g.C * g.T * plane;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const float gc = gcol[idx];
    if (gc == 0.f) continue;
    const long long pix = idx % plane;
    const int tap = (int)((idx / plane) % g.T);
    const int c = (int)((idx / (plane * g.T)) % g.C);
    const int n = n0 + (int)(idx / (plane * g.T * g.C));
    const int ho = (int)(pix / g.Wo), wo = (int)(pix - (long long)ho * g.Wo);
    const int i = tap / g.kw, j = tap - i * g.kw;
    float oh, ow, m;
    tap_inputs(g, off, msk, n, c / g.cpdg, tap, pix, plane, oh, ow, m);
    float4 wt;
    int h_low, w_low;
    tap_weights(oh, ow, m, ho * g.stride_h - g.pad_h + i * g.dil_h,
                wo * g.stride_w - g.pad_w + j * g.dil_w, g.H, g.W, wt, h_low, w_low);
    float *dst = gin + ((long long)n * g.C + c) * g.H * g.W + (long long)h_low * g.W + w_low;
    if (wt.x != 0.f) atomicAdd(dst, wt.x * gc);
    if (wt.y != 0.f) atomicAdd(dst + 1, wt.y * gc);
    if (wt.z != 0.f) atomicAdd(dst + g.W, wt.z * gc);
    if (wt.w != 0.f) atomicAdd(dst + g.W + 1, wt.w * gc);
  }
}

// grad_offset[n][dg*2T + 2*tap + {0,1}][p] and grad_mask[n][dg*T + tap][p] (fp32, dense)
template <typename T>
__global__ void __launch_bounds__(256)
dcn_bwd_coord_kernel(const Geom g, const T *__restrict__ x, const T *__restrict__ off,
                     const T *__restrict__ msk, int n0, int ns, const float *__restrict__ gcol,
                     float *__restrict__ goff, float *__restrict__ gmsk) {
  const long long plane = (long long)g.Ho * g.Wo;
  const long long total = (long long)ns * g.dg * g.T * plane;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long pix = idx % plane;
    const int tap = (int)((idx / plane) % g.T);
    const int dgi = (int)((idx / (plane * g.T)) % g.dg);
    const int s = (int)(idx / (plane * g.T * g.dg));
    const int n = n0 + s;
    const int ho = (int)(pix / g.Wo), wo = (int)(pix - (long long)ho * g.Wo);
    const int i = tap / g.kw, j = tap - i * g.kw;
    float oh, ow, m;
    tap_inputs(g, off, msk, n, dgi, tap, pix, plane, oh, ow, m);
    const Sample sp = locate(oh, ow, ho * g.stride_h - g.pad_h + i * g.dil_h,
                             wo * g.stride_w - g.pad_w + j * g.dil_w, g.H, g.W);
    float val_h = 0.f, val_w = 0.f, mval = 0.f;
    if (sp.inside) {
      const long long o00 = (long long)sp.h_low * g.in_sh + (long long)sp.w_low * g.in_sw;
      for (int c = dgi * g.cpdg; c < (dgi + 1) * g.cpdg; ++c) {
        const float gc = gcol[(((long long)s * g.C + c) * g.T + tap) * plane + pix];
        const T *pl = x + (long long)n * g.in_sn + (long long)c * g.in_sc + o00;
        const float v1 = sp.v1 ? ld_as_float(pl, 0) : 0.f;
        const float v2 = sp.v2 ? ld_as_float(pl, g.in_sw) : 0.f;
        const float v3 = sp.v3 ? ld_as_float(pl, g.in_sh) : 0.f;
        const float v4 = sp.v4 ? ld_as_float(pl, g.in_sh + g.in_sw) : 0.f;
        mval += gc * (sp.hh * sp.hw * v1 + sp.hh * sp.lw * v2 + sp.lh * sp.hw * v3 + sp.lh * sp.lw * v4);
        val_h += gc * (-sp.hw * v1 - sp.lw * v2 + sp.hw * v3 + sp.lw * v4);
        val_w += gc * (-sp.hh * v1 + sp.hh * v2 - sp.lh * v3 + sp.lh * v4);
      }
    }
    const long long ob = ((long long)n * g.dg + dgi) * 2 * g.T * plane + (long long)(2 * tap) * plane + pix;
    goff[ob] = val_h * m;
    goff[ob + plane] = val_w * m;
    if (gmsk) gmsk[(((long long)n * g.dg + dgi) * g.T + tap) * plane + pix] = mval;
  }
}

int grid_for(long long total) {
  long long b = (total + 255) / 256;
  return (int)(b > 148LL * 32 ? 148LL * 32 : (b < 1 ? 1 : b));
}

}  // namespace

cudaError_t launch_bwd_columns(const Geom &g, const Ptrs &p, int dtype, int n0, int ns, float *col,
                               cudaStream_t s) {
  const long long total = (long long)ns * g.C * g.T * g.Ho * g.Wo;
  if (total == 0) return cudaSuccess;
  if (dtype == DCN_DTYPE_F32)
    dcn_bwd_columns_kernel<float><<<grid_for(total), 256, 0, s>>>(
        g, (const float *)p.input, (const float *)p.offset, (const float *)p.mask, n0, ns, col);
  else if (dtype == DCN_DTYPE_F16)
    dcn_bwd_columns_kernel<__half><<<grid_for(total), 256, 0, s>>>(
        g, (const __half *)p.input, (const __half *)p.offset, (const __half *)p.mask, n0, ns, col);
  else
    dcn_bwd_columns_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(
        g, (const __nv_bfloat16 *)p.input, (const __nv_bfloat16 *)p.offset,
        (const __nv_bfloat16 *)p.mask, n0, ns, col);
  return cudaGetLastError();
}

cudaError_t launch_bwd_input(const Geom &g, const Ptrs &p, int dtype, int n0, int ns,
                             const float *gcol, float *gin, cudaStream_t s) {
  const long long total = (long long)ns * g.C * g.T * g.Ho * g.Wo;
  if (total == 0) return cudaSuccess;
  if (dtype == DCN_DTYPE_F32)
    dcn_bwd_input_kernel<float><<<grid_for(total), 256, 0, s>>>(
        g, (const float *)p.offset, (const float *)p.mask, n0, ns, gcol, gin);
  else if (dtype == DCN_DTYPE_F16)
    dcn_bwd_input_kernel<__half><<<grid_for(total), 256, 0, s>>>(
        g, (const __half *)p.offset, (const __half *)p.mask, n0, ns, gcol, gin);
  else
    dcn_bwd_input_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(
        g, (const __nv_bfloat16 *)p.offset, (const __nv_bfloat16 *)p.mask, n0, ns, gcol, gin);
  return cudaGetLastError();
}

cudaError_t launch_bwd_coord(const Geom &g, const Ptrs &p, int dtype, int n0, int ns,
                             const float *gcol, float *goff, float *gmsk, cudaStream_t s) {
  const long long total = (long long)ns * g.dg * g.T * g.Ho * g.Wo;
  if (total == 0) return cudaSuccess;
  if (dtype == DCN_DTYPE_F32)
    dcn_bwd_coord_kernel<float><<<grid_for(total), 256, 0, s>>>(
        g, (const float *)p.input, (const float *)p.offset, (const float *)p.mask, n0, ns, gcol,
        goff, gmsk);
  else if (dtype == DCN_DTYPE_F16)
    dcn_bwd_coord_kernel<__half><<<grid_for(total), 256, 0, s>>>(
        g, (const __half *)p.input, (const __half *)p.offset, (const __half *)p.mask, n0, ns, gcol,
        goff, gmsk);
  else
    dcn_bwd_coord_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(
        g, (const __nv_bfloat16 *)p.input, (const __nv_bfloat16 *)p.offset,
        (const __nv_bfloat16 *)p.mask, n0, ns, gcol, goff, gmsk);
  return cudaGetLastError();
}

}  // namespace dcn
