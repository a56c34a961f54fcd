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
          if (!(corner_is_read(wt.x) || corner_is_read(wt.y) || corner_is_read(wt.z) || corner_is_read(wt.w))) continue;
          const long long o00 = (long long)h_low * g.in_sh + (long long)w_low * g.in_sw;
          for (int c = c0; c < c1; ++c) {
            const T *pl = x_n + (long long)c * g.in_sc + o00;
            float v = 0.f;
            if (corner_is_read(wt.x)) v += wt.x * ld_as_float(pl, 0);
            if (corner_is_read(wt.y)) v += wt.y * ld_as_float(pl, g.in_sw);
            if (corner_is_read(wt.z)) v += wt.z * ld_as_float(pl, g.in_sh);
            if (corner_is_read(wt.w)) v += wt.w * ld_as_float(pl, g.in_sh + g.in_sw);
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
  else if (dtype == DCN_DTYPE_F16)
    dcn_fwd_simt_direct<__half><<<(int)blocks, block, 0, s>>>(
        g, (const __half *)p.input, (const __half *)p.offset, (const __half *)p.mask,
        (const __half *)p.weight, (const __half *)p.bias, (__half *)p.output);
  else
    dcn_fwd_simt_direct<__nv_bfloat16><<<(int)blocks, block, 0, s>>>(
        g, (const __nv_bfloat16 *)p.input, (const __nv_bfloat16 *)p.offset,
        (const __nv_bfloat16 *)p.mask, (const __nv_bfloat16 *)p.weight,
        (const __nv_bfloat16 *)p.bias, (__nv_bfloat16 *)p.output);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------
// Tiled kernel: 8x8 output pixels x 64 output channels per block, fp32 FFMA, 4x4 outputs
// per thread.  The sampled columns of a few input channels x all taps are built in shared
// memory (never in global memory), next to the matching weight slice; the tap table of the
// current deform group (four corner weights x mask, corner position) is built once per
// tile and deform group and reused by every channel of that group.
// ---------------------------------------------------------------------------------
namespace {
constexpr int kTP = 64;        // pixels per tile (8 x 8)
constexpr int kTC = 64;        // output channels per tile
constexpr int kRowsMax = 72;   // rows (channel, tap) of a k-chunk
constexpr int kTapsMax = 25;   // taps the tap table is sized for
}  // namespace

bool simt_tiled_supported(const Geom &g) { return g.T <= kTapsMax; }

size_t simt_tiled_smem(const Geom &g) {
  return (size_t)2 * kRowsMax * kTP * sizeof(float) + (size_t)g.T * kTP * (sizeof(float4) + sizeof(int2));
}

template <typename T>
__global__ void __launch_bounds__(256)
dcn_fwd_simt_tiled(const Geom g, const T *__restrict__ x, const T *__restrict__ off,
                   const T *__restrict__ msk, const T *__restrict__ wgt,
                   const T *__restrict__ bias, T *__restrict__ out, int tiles_x, int tiles_y,
                   int n_ctile) {
  extern __shared__ __align__(16) unsigned char smem_simt[];
  float *col_s = reinterpret_cast<float *>(smem_simt);            // [rows][64 px]
  float *w_s = col_s + kRowsMax * kTP;                            // [rows][64 co]
  float4 *tab_w = reinterpret_cast<float4 *>(w_s + kRowsMax * kTP);  // [T][64 px]
  int2 *tab_p = reinterpret_cast<int2 *>(tab_w + g.T * kTP);         // (h_low, w_low)

  const int tid = threadIdx.x;
  long long item = blockIdx.x;
  const int ct = (int)(item % n_ctile); item /= n_ctile;
  const int grp = (int)(item % g.groups); item /= g.groups;
  const int tx_ = (int)(item % tiles_x); item /= tiles_x;
  const int ty_ = (int)(item % tiles_y); item /= tiles_y;
  const int n = (int)item;
  const int ho0 = ty_ * 8, wo0 = tx_ * 8;
  const int co0 = grp * g.Cog + ct * kTC;                 // first output channel of the tile
  const int nco = min(kTC, g.Cog - ct * kTC);
  const long long plane = (long long)g.Ho * g.Wo;
  const T *x_n = x + (long long)n * g.in_sn;

  // this thread's pixel for table/gather work (tid & 63) and its 4x4 output block
  const int gpx = tid & 63;
  const int gho = ho0 + (gpx >> 3), gwo = wo0 + (gpx & 7);
  const bool gvalid = gho < g.Ho && gwo < g.Wo;
  const int ty = tid >> 4, tx = tid & 15;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int cc_max = max(1, min(8, kRowsMax / g.T));
  const int c_begin = grp * g.Cg, c_end = c_begin + g.Cg;
  int cur_dg = -1;
  for (int c0 = c_begin; c0 < c_end;) {
    const int dgi = c0 / g.cpdg;
    const int c1 = min(min(c_end, (dgi + 1) * g.cpdg), c0 + cc_max);
    const int rows = (c1 - c0) * g.T;
    __syncthreads();  // the previous chunk's columns, weights (and table) are no longer read
    if (dgi != cur_dg) {
      cur_dg = dgi;
      for (int e = tid; e < g.T * kTP; e += 256) {
        const int tap = e >> 6;  // e & 63 == gpx because 256 % 64 == 0
        const int i = tap / g.kw, j = tap - i * g.kw;
        float4 wt = make_float4(0.f, 0.f, 0.f, 0.f);
        int h_low = 0, w_low = 0;
        if (gvalid) {
          const long long pix = (long long)gho * g.Wo + gwo;
          float oh = 0.f, ow = 0.f, m = 1.f;
          if (off) {
            const T *o = off + (long long)n * g.off_sn + ((long long)dgi * 2 * g.T + 2 * tap) * plane + pix;
            oh = ld_as_float(o, 0);
            ow = ld_as_float(o, plane);
          }
          if (msk) m = ld_as_float(msk, (long long)n * g.msk_sn + ((long long)dgi * g.T + tap) * plane + pix);
          tap_weights(oh, ow, m, gho * g.stride_h - g.pad_h + i * g.dil_h,
                      gwo * g.stride_w - g.pad_w + j * g.dil_w, g.H, g.W, wt, h_low, w_low);
        }
        tab_w[e] = wt;
        tab_p[e] = make_int2(h_low, w_low);
      }
      __syncthreads();
    }
    // columns of this chunk: row r = (channel c0 + r / T, tap r % T), 64 pixels each
    for (int e = tid; e < rows * kTP; e += 256) {
      const int r = e >> 6;
      const int cl = r / g.T, tap = r - cl * g.T;
      const float4 wt = tab_w[tap * kTP + gpx];
      const int2 hw = tab_p[tap * kTP + gpx];
      const T *pl = x_n + (long long)(c0 + cl) * g.in_sc + (long long)hw.x * g.in_sh +
                    (long long)hw.y * g.in_sw;
      float v = 0.f;
      if (corner_is_read(wt.x)) v = fmaf(wt.x, ld_as_float(pl, 0), v);
      if (corner_is_read(wt.y)) v = fmaf(wt.y, ld_as_float(pl, g.in_sw), v);
      if (corner_is_read(wt.z)) v = fmaf(wt.z, ld_as_float(pl, g.in_sh), v);
      if (corner_is_read(wt.w)) v = fmaf(wt.w, ld_as_float(pl, g.in_sh + g.in_sw), v);
      col_s[r * kTP + gpx] = v;
    }
    // weight slice: w_s[r][co] = W[co0 + co][c0 - c_begin + r / T][r % T]
    {
      const long long kbase = (long long)(c0 - c_begin) * g.T;
      for (int e = tid; e < rows * kTC; e += 256) {
        const int r = e >> 6, col = e & 63;
        w_s[e] = col < nco ? ld_as_float(wgt, (long long)(co0 + col) * g.Cg * g.T + kbase + r) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int r = 0; r < rows; ++r) {
      const float4 av = *reinterpret_cast<const float4 *>(col_s + r * kTP + ty * 4);
      const float4 bv = *reinterpret_cast<const float4 *>(w_s + r * kTC + tx * 4);
      const float aa[4] = {av.x, av.y, av.z, av.w};
      const float bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(aa[i], bb[j], acc[i][j]);
    }
    c0 = c1;
  }
  // pixels ty*4 .. ty*4+3 are four consecutive wo of one tile row; channels tx*4 .. +3
  const int ho = ho0 + (ty >> 1), wo_first = wo0 + (ty & 1) * 4;
  if (ho < g.Ho) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = tx * 4 + j;
      if (col >= nco) continue;
      const int co = co0 + col;
      const float bv = bias ? ld_as_float(bias, co) : 0.f;
      T *dst = out + (long long)n * g.out_sn + (long long)co * plane + (long long)ho * g.Wo;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (wo_first + i < g.Wo) st_from_float(dst, wo_first + i, apply_act(g, co, acc[i][j] + bv));
    }
  }
}

cudaError_t launch_simt_tiled(const Geom &g, const Ptrs &p, int dtype, cudaStream_t s) {
  if (g.P == 0) return cudaSuccess;
  const int tiles_x = (g.Wo + 7) / 8, tiles_y = (g.Ho + 7) / 8;
  const int n_ctile = (g.Cog + kTC - 1) / kTC;
  const long long blocks = (long long)g.N * tiles_y * tiles_x * g.groups * n_ctile;
  if (blocks > 2147483647LL) return cudaErrorInvalidConfiguration;
  const size_t smem = simt_tiled_smem(g);
  cudaError_t e;
  if (dtype == DCN_DTYPE_F32) {
    e = cudaFuncSetAttribute(dcn_fwd_simt_tiled<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dcn_fwd_simt_tiled<float><<<(unsigned)blocks, 256, smem, s>>>(
        g, (const float *)p.input, (const float *)p.offset, (const float *)p.mask,
        (const float *)p.weight, (const float *)p.bias, (float *)p.output, tiles_x, tiles_y, n_ctile);
  } else if (dtype == DCN_DTYPE_F16) {
    e = cudaFuncSetAttribute(dcn_fwd_simt_tiled<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dcn_fwd_simt_tiled<__half><<<(unsigned)blocks, 256, smem, s>>>(
        g, (const __half *)p.input, (const __half *)p.offset, (const __half *)p.mask,
        (const __half *)p.weight, (const __half *)p.bias, (__half *)p.output, tiles_x, tiles_y,
        n_ctile);
  } else {
    e = cudaFuncSetAttribute(dcn_fwd_simt_tiled<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dcn_fwd_simt_tiled<__nv_bfloat16><<<(unsigned)blocks, 256, smem, s>>>(
        g, (const __nv_bfloat16 *)p.input, (const __nv_bfloat16 *)p.offset,
        (const __nv_bfloat16 *)p.mask, (const __nv_bfloat16 *)p.weight,
        (const __nv_bfloat16 *)p.bias, (__nv_bfloat16 *)p.output, tiles_x, tiles_y, n_ctile);
  }
  return cudaGetLastError();
}

}  // namespace dcn
