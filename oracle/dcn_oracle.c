/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Plain-C restatement of the reference's CPU algorithm for the forward of
 * (modulated) deformable convolution.  Only tests, the smoke check and the
 * CPU-baseline leg of the benchmark may link or call this file; the shipped
 * CUDA path never does.
 *
 * Parity status: PINNED.  The restatement is checked (tests/test_oracle.py)
 * against the known-answer vectors of the reference's own unit tests
 * (tests/test_ops/test_modulated_deform_conv.py:28-30,
 *  tests/test_ops/test_deform_conv.py:27-35) and against outputs of the
 * unmodified reference CPU extension on seeded inputs (tests/golden/).
 *
 * What it follows, by reference file:line
 *   bilinear sample ............ mmcv/ops/csrc/pytorch/cpu/modulated_deform_conv.cpp:5-33
 *                                mmcv/ops/csrc/pytorch/cpu/deform_conv.cpp:5-37
 *   im2col with offsets/mask ... mmcv/ops/csrc/pytorch/cpu/modulated_deform_conv.cpp:109-168
 *                                mmcv/ops/csrc/pytorch/cpu/deform_conv.cpp:113-164
 *   per-sample, per-group GEMM . mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:108-130
 *                                mmcv/ops/csrc/pytorch/deform_conv.cpp:220-239
 *   bias broadcast add ......... mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:135-137
 *   output size ................ mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:87-90
 *
 * The GEMM in the reference is a library call (ATen addmm_ -> MKL sgemm); it
 * is restated here as a plain fp32 row-accumulating product, so results agree
 * with the reference to summation-order rounding, not bit for bit.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* One bilinear sample of a single H x W plane at the fractional position
 * (h, w).  Each of the four corners contributes only if it lies inside the
 * plane; the caller decides whether the position is sampled at all. */
float dcn_oracle_bilinear(const float *plane, int height, int width, float h,
                          float w) {
  int h_low = (int)floorf(h);
  int w_low = (int)floorf(w);
  int h_high = h_low + 1;
  int w_high = w_low + 1;
  float lh = h - (float)h_low;
  float lw = w - (float)w_low;
  float hh = 1.0f - lh, hw = 1.0f - lw;
  float v1 = 0.f, v2 = 0.f, v3 = 0.f, v4 = 0.f;
  if (h_low >= 0 && w_low >= 0) v1 = plane[h_low * width + w_low];
  if (h_low >= 0 && w_high <= width - 1) v2 = plane[h_low * width + w_high];
  if (h_high <= height - 1 && w_low >= 0) v3 = plane[h_high * width + w_low];
  if (h_high <= height - 1 && w_high <= width - 1)
    v4 = plane[h_high * width + w_high];
  float w1 = hh * hw, w2 = hh * lw, w3 = lh * hw, w4 = lh * lw;
  return w1 * v1 + w2 * v2 + w3 * v3 + w4 * v4;
}

int dcn_oracle_out_size(int in, int pad, int dil, int k, int stride) {
  return (in + 2 * pad - (dil * (k - 1) + 1)) / stride + 1;
}

/* Column matrix of ONE sample: col[(c*kh*kw + i*kw + j) * Ho*Wo + h*Wo + w].
 * mask == NULL means the unmodulated (v1) operator. */
void dcn_oracle_im2col(const float *im, const float *offset, const float *mask,
                       int C, int H, int W, int kh, int kw, int pad_h,
                       int pad_w, int stride_h, int stride_w, int dil_h,
                       int dil_w, int deform_groups, int Ho, int Wo,
                       float *col) {
  const int cpdg = C / deform_groups;
  const long plane_out = (long)Ho * Wo;
#pragma omp parallel for schedule(static)
  for (int c = 0; c < C; ++c) {
    const int dg = c / cpdg;
    const float *im_c = im + (long)c * H * W;
    const float *off_g = offset + (long)dg * 2 * kh * kw * plane_out;
    const float *msk_g = mask ? mask + (long)dg * kh * kw * plane_out : NULL;
    for (int i = 0; i < kh; ++i)
      for (int j = 0; j < kw; ++j) {
        const int tap = i * kw + j;
        float *col_row = col + ((long)c * kh * kw + tap) * plane_out;
        for (int h = 0; h < Ho; ++h)
          for (int w = 0; w < Wo; ++w) {
            const long p = (long)h * Wo + w;
            const float off_h = off_g[(2 * tap) * plane_out + p];
            const float off_w = off_g[(2 * tap + 1) * plane_out + p];
            const float h_im =
                (float)(h * stride_h - pad_h + i * dil_h) + off_h;
            const float w_im =
                (float)(w * stride_w - pad_w + j * dil_w) + off_w;
            float val = 0.f;
            if (h_im > -1 && w_im > -1 && h_im < H && w_im < W)
              val = dcn_oracle_bilinear(im_c, H, W, h_im, w_im);
            if (msk_g) val *= msk_g[(long)tap * plane_out + p];
            col_row[p] = val;
          }
      }
  }
}

/* Full forward.  Layouts are the reference's: input [N,C,H,W], offset
 * [N, dg*2*kh*kw, Ho, Wo] with (y,x) interleaved per tap, mask
 * [N, dg*kh*kw, Ho, Wo] or NULL, weight [Co, C/groups, kh, kw], bias [Co] or
 * NULL, output [N,Co,Ho,Wo].  Returns 0, or a negative code on bad arguments
 * (the same conditions the reference rejects). */
int dcn_oracle_forward_f32(const float *input, const float *offset,
                           const float *mask, const float *weight,
                           const float *bias, float *output, int N, int C,
                           int H, int W, int Co, int kh, int kw, int stride_h,
                           int stride_w, int pad_h, int pad_w, int dil_h,
                           int dil_w, int groups, int deform_groups) {
  if (kh <= 0 || kw <= 0 || stride_h <= 0 || stride_w <= 0 || dil_h <= 0 ||
      dil_w <= 0)
    return -1;
  if (groups <= 0 || deform_groups <= 0 || C % groups || Co % groups ||
      C % deform_groups)
    return -2;
  const int Ho = dcn_oracle_out_size(H, pad_h, dil_h, kh, stride_h);
  const int Wo = dcn_oracle_out_size(W, pad_w, dil_w, kw, stride_w);
  if (Ho < 1 || Wo < 1) return -3;
  const long P = (long)Ho * Wo;
  const int Cg = C / groups, Cog = Co / groups;
  const long K = (long)Cg * kh * kw;
  float *col = (float *)malloc(sizeof(float) * (size_t)C * kh * kw * P);
  if (!col) return -4;
  for (int n = 0; n < N; ++n) {
    dcn_oracle_im2col(input + (long)n * C * H * W,
                      offset + (long)n * deform_groups * 2 * kh * kw * P,
                      mask ? mask + (long)n * deform_groups * kh * kw * P : NULL,
                      C, H, W, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h,
                      dil_w, deform_groups, Ho, Wo, col);
#pragma omp parallel for schedule(static)
    for (int co = 0; co < Co; ++co) {
      const int g = co / Cog;
      float *out_row = output + ((long)n * Co + co) * P;
      const float *w_row = weight + (long)co * K;
      const float *col_g = col + (long)g * K * P;
      for (long p = 0; p < P; ++p) out_row[p] = 0.f;
      for (long k = 0; k < K; ++k) {
        const float wv = w_row[k];
        const float *c_row = col_g + k * P;
        for (long p = 0; p < P; ++p) out_row[p] += wv * c_row[p];
      }
      if (bias) {
        const float b = bias[co];
        for (long p = 0; p < P; ++p) out_row[p] += b;
      }
    }
  }
  free(col);
  return 0;
}

int dcn_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
