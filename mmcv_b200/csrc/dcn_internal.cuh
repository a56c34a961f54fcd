// Internal declarations shared by the kernels and the C-ABI layer.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "dcn_b200.h"

namespace dcn {

// Geometry of one forward problem as the kernels see it (all by value).
struct Geom {
  int N, C, H, W, Co, Ho, Wo;
  int kh, kw, T;  // T = kh*kw taps
  int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int groups, dg;
  int Cg, Cog, cpdg;  // channels per conv group, outputs per group, channels per deform group
  long long P;        // N*Ho*Wo output pixels
  long long in_sn, in_sc, in_sh, in_sw;  // input element strides
  long long off_sn, msk_sn, out_sn;      // per-sample strides of offset/mask/output
  long long off_cs, off_ps, msk_cs, msk_ps;  // channel and pixel strides inside a sample
  int mask_act;                          // DCN_ACT_SIGMOID: the mask holds logits
  int act, act_lo, act_hi;
};

struct Ptrs {
  const void *input, *offset, *mask, *weight, *bias;
  void *output;
};

// Workspace layout (byte offsets from the workspace base).
struct Workspace {
  size_t status_off;   // 256 B: status word
  size_t wtile_off;    // swizzled weight tiles (tcgen05 path)
  size_t wtile_bytes;
  size_t xcl_off;      // channels-last bf16 copy of the input (tcgen05 path)
  size_t xcl_bytes;
  size_t total;
};

// tcgen05 path configuration decided on the host.
struct TcPlan {
  int BN;         // accumulator columns per tile (multiple of 16, <= 256)
  int NT;         // n-tiles per conv group
  int KC;         // 64-channel chunks per conv group
  int S;          // k-stages per tile = KC*T
  int ndgc;       // max deform groups touched by one 64-channel chunk
  int a_stages, b_stages;
  int tmem_cols;  // power of two >= 2*BN
  long long items;  // tiles*groups*NT
  int grid;
  size_t smem;
  int tw_log2;             // tile = (128 >> tw_log2) x (1 << tw_log2) output pixels of one sample
  int tiles_x, tiles_y;    // tiles per sample
  int tiles_per_stage;     // 1: 16-bit operands; 2: TF32x3 (high part and remainder)
  int op_format;           // tensor-core operand format: 0 fp16, 1 bf16, 2 tf32
  int ch_per_stage;        // input channels per k-stage: 64 (bf16) or 32 (TF32x3)
  int producer_cfg;        // [flags*1000 +] groups*100 + warps_per_group*10 + rows in flight per thread
  int io_bytes;            // element size of the tensors (bias staging in the epilogue)
  // --- second-generation 16-bit kernel (dcn_tc2.cu) ---
  int version;             // 1: dcn_fwd_tc, 2: dcn_fwd_tc2
  int in_pad;              // first-generation kernel: 1 when it reads the zero-bordered copy (pitch W + 2)
  int KH;                  // 32-channel half-chunks per conv group
  int U;                   // (half-chunk, tap) units per tile = KH*T; a k-stage holds two
  int ndu;                 // max deform groups touched by one half-chunk
  int tab_span;            // half-chunks that share one tap-table segment; 0: one segment per k-stage
  int tab_slots;           // ring depth of the tap table
  int tab_slot_blocks;     // (tap, deform group) blocks per ring slot
  int win_h, win_w;        // input window held in shared memory, in pixels (0: none)
  int win_my, win_mx;      // its margin above / left of the tile's undeformed footprint
  int epi_tma;             // 1: the epilogue stores through the tensor-copy engine
  int raw_slots;           // ring depth of offset / mask planes staged for the builders (0: none)
};

enum { kBM = 128 };

// One sampling tap: bilinear corner weights (already multiplied by the modulation
// mask, and zero for corners outside the plane) and the integer position of the
// top-left corner.  Follows dmcn_im2col_bilinear
// (mmcv/ops/csrc/common/cuda/modulated_deform_conv_cuda_kernel.cuh:80-108) and the
// sampling gate of its caller (same file, :237-239).  A position that is NaN or
// outside (-1, H) x (-1, W) yields four zero weights.
//
// A weight of +0 (all bits clear) marks a corner that the reference does not read: it lies
// outside the plane, or the whole position fails the gate.  A corner inside the plane whose
// weight happens to be zero (a grid-aligned position, a zero mask value) is read by the
// reference and multiplied -- 0 * Inf and 0 * NaN give NaN there -- so its weight is returned
// as -0: consumers test the BITS (corner_is_read) and multiply whatever they read.
__device__ __forceinline__ float read_weight(float w) { return w == 0.f ? -0.f : w; }
__device__ __forceinline__ bool corner_is_read(float w) { return __float_as_uint(w) != 0u; }
__device__ __forceinline__ void tap_weights(float off_h, float off_w, float m,
                                            int h_base, int w_base, int H, int W,
                                            float4 &wt, int &h_low, int &w_low) {
  const float h_im = (float)h_base + off_h;
  const float w_im = (float)w_base + off_w;
  wt = make_float4(0.f, 0.f, 0.f, 0.f);
  h_low = 0;
  w_low = 0;
  if (h_im > -1.f && w_im > -1.f && h_im < (float)H && w_im < (float)W) {
    const float hf = floorf(h_im), wf = floorf(w_im);
    h_low = (int)hf;
    w_low = (int)wf;
    const float lh = h_im - hf, lw = w_im - wf;
    const float hh = 1.f - lh, hw = 1.f - lw;
    const bool top = h_low >= 0, left = w_low >= 0;
    const bool bot = h_low + 1 <= H - 1, right = w_low + 1 <= W - 1;
    wt.x = (top && left) ? read_weight(hh * hw * m) : 0.f;
    wt.y = (top && right) ? read_weight(hh * lw * m) : 0.f;
    wt.z = (bot && left) ? read_weight(lh * hw * m) : 0.f;
    wt.w = (bot && right) ? read_weight(lh * lw * m) : 0.f;
  }
}

__device__ __forceinline__ float ld_as_float(const float *p, long long i) { return p[i]; }
__device__ __forceinline__ float ld_as_float(const __nv_bfloat16 *p, long long i) {
  return __bfloat162float(p[i]);
}
__device__ __forceinline__ float ld_as_float(const __half *p, long long i) {
  return __half2float(p[i]);
}
__device__ __forceinline__ void st_from_float(__half *p, long long i, float v) {
  p[i] = __float2half_rn(v);
}
__device__ __forceinline__ void st_from_float(float *p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void st_from_float(__nv_bfloat16 *p, long long i, float v) {
  p[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float apply_act(const Geom &g, int co, float v) {
  if (g.act == DCN_ACT_SIGMOID && co >= g.act_lo && co < g.act_hi)
    v = 1.f / (1.f + __expf(-v));
  return v;
}

// Launchers (each enqueues on `stream` and returns the CUDA error of the launch).
cudaError_t launch_simt_direct(const Geom &g, const Ptrs &p, int dtype, cudaStream_t s);
cudaError_t launch_simt_tiled(const Geom &g, const Ptrs &p, int dtype, cudaStream_t s);
size_t simt_tiled_smem(const Geom &g);
bool simt_tiled_supported(const Geom &g);

// pad: width of the zero border around every sample of the copy (0 or 1); with a border the
// copy ends with one more all-zero row
cudaError_t launch_stage_input_cl(const Geom &g, const void *input, int dtype, void *xcl,
                                  int op_format, int pad, cudaStream_t s);
cudaError_t launch_weight_tiles(const Geom &g, const TcPlan &tp, const void *weight,
                                int dtype, void *wtiles, cudaStream_t s);
cudaError_t launch_tc(const Geom &g, const TcPlan &tp, const Ptrs &p, int dtype, const void *xcl,
                      const void *wtiles, int *status, unsigned long long *counters,
                      cudaStream_t s);
cudaError_t launch_clear_status(int *status, cudaStream_t s);

int tc_threads(const TcPlan &tp);
size_t tc2_smem_bytes(const TcPlan &tp);
// Debug knobs of the second-generation kernel (tests of the bounded waits): wait limit in
// nanoseconds (0: default) and flags (bit 0: the weight loader withholds its last copy).
cudaError_t launch_tc2(const Geom &g, const TcPlan &tp, const Ptrs &p, int dtype, const void *xpad,
                       const void *wtiles, int *status, unsigned long long *counters,
                       unsigned long long wait_limit_ns, int debug_flags, cudaStream_t s);

bool conv_tma_supported(const Geom &g, const TcPlan &tp);
cudaError_t launch_conv_tma(const Geom &g, const TcPlan &tp, const Ptrs &p, int dtype, const void *xpad,
                            const void *wtiles, int *status, unsigned long long wait_limit_ns,
                            cudaStream_t s);

cudaError_t launch_bwd_columns(const Geom &g, const Ptrs &p, int dtype, int n0, int ns, float *col,
                               cudaStream_t s);
cudaError_t launch_bwd_input(const Geom &g, const Ptrs &p, int dtype, int n0, int ns,
                             const float *gcol, float *gin, cudaStream_t s);
cudaError_t launch_bwd_coord(const Geom &g, const Ptrs &p, int dtype, int n0, int ns,
                             const float *gcol, float *goff, float *gmsk, cudaStream_t s);

// Records `msg` as the calling thread's dcn_last_error() text and returns `code`.
int set_error(int code, const char *msg);

}  // namespace dcn
