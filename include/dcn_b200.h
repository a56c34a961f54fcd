/*
 * dcn_b200 -- C ABI of the B200 (sm_100a) forward of deformable convolution
 * v1 / v2 (modulated).  Plain pointers and sizes only; no tensor-library types.
 *
 * All functions return 0 on success and a negative DCN_ERR_* code otherwise;
 * dcn_last_error() then holds a message for the calling thread.  Nothing here
 * allocates device memory except where a function says so: scratch memory is
 * sized by dcn_fwd_workspace_bytes() and handed in by the caller.  All work is
 * enqueued on the caller's stream and nothing synchronises unless stated.
 * There is no CPU path: every entry fails if the device cannot run sm_100a code.
 */
#ifndef DCN_B200_H_
#define DCN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DCN_ABI_VERSION 6

enum { DCN_DTYPE_F32 = 0, DCN_DTYPE_BF16 = 1, DCN_DTYPE_F16 = 2 };

/* Arithmetic of the contraction.
 *   BF16   tcgen05 kind::f16 MMA on 16-bit operands in the tensors' own 16-bit type (bf16
 *          or fp16), fp32 accumulation in tensor memory.
 *   TF32X3 fp32 tensors only: tcgen05 kind::tf32 MMA, every operand split into a TF32 high
 *          part and a remainder, three products per step (hi*hi + lo*hi + hi*lo); meets the
 *          same fp32 error bound as FFMA.  Shapes the tensor-core kernel does not take
 *          (it needs C/groups % 4 == 0 and C/deformable_group % 4 == 0) run on the FFMA
 *          kernel instead.
 *   FFMA   fp32 fused multiply-add on the SIMT cores, any shape.
 *   AUTO   BF16 for bf16 and fp16 tensors, TF32X3 for fp32 tensors. */
enum { DCN_MATH_AUTO = 0, DCN_MATH_FFMA = 1, DCN_MATH_TF32X3 = 2, DCN_MATH_BF16 = 3 };

enum {
  DCN_OK = 0,
  DCN_ERR_ARG = -1,        /* shape / pointer / enum rejected (message says which) */
  DCN_ERR_UNSUPPORTED = -2,/* valid in the reference, not built here (message says what) */
  DCN_ERR_WORKSPACE = -3,  /* workspace missing, too small or misaligned */
  DCN_ERR_CUDA = -4,       /* a CUDA runtime call failed (message carries its text) */
  DCN_ERR_DEVICE = -5      /* no device, or the device is not compute capability 10.x */
};

/* Kernel families a call can be routed to (reported by dcn_fwd_plan). */
enum { DCN_PATH_TCGEN05 = 1, DCN_PATH_SIMT_TILED = 2, DCN_PATH_SIMT_DIRECT = 3 };

/* Epilogue applied to output channels [act_lo, act_hi) after bias. */
enum { DCN_ACT_NONE = 0, DCN_ACT_SIGMOID = 1 };

/*
 * One forward problem.  Tensor layouts are the reference's:
 *   input  [N, C, H, W]            element strides in_stride[4] (NCHW-contiguous or
 *                                  channels-last; anything else is rejected)
 *   offset [N, dg*2*kh*kw, Ho, Wo] (y, x) interleaved per tap, contiguous per sample,
 *                                  sample stride offset_batch_stride elements (0 = dense).
 *                                  NULL = all-zero offsets (an ordinary convolution).
 *   mask   [N, dg*kh*kw, Ho, Wo]   same rules; NULL = 1 everywhere (the v1 operator).
 *   weight [Co, C/groups, kh, kw]  contiguous
 *   bias   [Co] or NULL
 *   output [N, Co, Ho, Wo]         contiguous per sample, sample stride out_batch_stride
 *                                  elements (0 = dense)
 * with Ho = (H + 2*pad_h - (dil_h*(kh-1)+1)) / stride_h + 1 (same for Wo), as in
 * mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:87-90.  All tensors share `dtype`.
 */
typedef struct DcnFwdParams {
  const void *input;
  const void *offset;
  const void *mask;
  const void *weight;
  const void *bias;
  void *output;
  int32_t dtype;      /* DCN_DTYPE_* */
  int32_t math_mode;  /* DCN_MATH_*  */
  int64_t N, C, H, W, Co;
  int32_t kh, kw, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int32_t groups, deform_groups;
  int64_t in_stride[4];
  int64_t offset_batch_stride, mask_batch_stride, out_batch_stride;
  int32_t act, act_lo, act_hi; /* DCN_ACT_* on output channels [act_lo, act_hi) */
  int32_t device;              /* CUDA device ordinal the pointers live on */
  /* Optional: the weight image dcn_prepare_weights() wrote for these weights and this
   * problem shape; dcn_fwd then skips its own re-layout of `weight`.  NULL = none. */
  const void *weight_image;
  int64_t weight_image_bytes;
  /* Optional layout of offset and mask inside a sample: element strides between channels and
   * between neighbouring output pixels (row-major over Ho x Wo).  All zero = the reference
   * layout (channel stride Ho*Wo, pixel stride 1).  A channels-last tensor of Ct channels has
   * channel stride 1 and pixel stride Ct, so the offset and mask thirds of a channels-last
   * branch output can be passed as they lie.  Tensor-core path only (others:
   * DCN_ERR_UNSUPPORTED). */
  int64_t offset_channel_stride, offset_pixel_stride, mask_channel_stride, mask_pixel_stride;
  int32_t mask_act;   /* DCN_ACT_SIGMOID: the mask tensor holds logits (what the Pack layers'
                       * branch produces before its sigmoid).  Tensor-core path only. */
  int32_t reserved0;
  /* Optional: the zero-bordered channels-last copy of `input` that dcn_pad_channels_last()
   * wrote (16-bit tensors).  The 16-bit tensor-core kernels then read it instead of making
   * their own copy, so a caller that runs several operators on the same activations (a Pack
   * layer: offset branch + deformable kernel) pays for the copy once.  NULL = none. */
  const void *padded_input;
  int64_t padded_input_bytes;
} DcnFwdParams;

/* What a call will do; filled by dcn_fwd_plan without touching the device. */
typedef struct DcnPlanInfo {
  int32_t path;           /* DCN_PATH_* */
  int32_t launches;       /* kernels dcn_fwd enqueues for this problem */
  int32_t stages_input;   /* 1 if the input is first restaged to channels-last bf16 */
  int32_t tile_m, tile_n, tile_k;
  int32_t grid, block;    /* of the main kernel */
  int64_t smem_bytes;     /* dynamic shared memory of the main kernel */
  int64_t Ho, Wo;
  size_t workspace_bytes;
  int32_t operand_stages, weight_stages; /* depth of the two shared-memory rings (tcgen05 path) */
  int32_t producer_layout; /* tcgen05 path, first-generation kernel: groups*100 + warps per
                            * group*10 + rows in flight, +1000 rows software-pipelined, +2000
                            * per-group tap tables; second generation: 16 (gather warps, which
                            * build their own tap entries) */
  int32_t kernel_version;  /* tcgen05 path: 1 = first-generation kernel (3xTF32), 2 = second generation, 16-bit operands */
  int32_t window_h, window_w; /* input window kept in shared memory, pixels (0: none) */
  int32_t table_span;      /* (unused: 0) */
  int32_t table_slots;     /* (unused: 0) */
  int32_t epilogue_tensor_stores; /* 1: output written by cp.async.bulk.tensor stores */
} DcnPlanInfo;

int dcn_abi_version(void);
const char *dcn_last_error(void);

int dcn_fwd_plan(const DcnFwdParams *p, DcnPlanInfo *info);
int dcn_fwd_workspace_bytes(const DcnFwdParams *p, size_t *bytes);

/*
 * Enqueue the forward on `stream` (a cudaStream_t).  `workspace` is device
 * memory of at least dcn_fwd_workspace_bytes() bytes, 256-byte aligned; its
 * contents are scratch, except that its first 4 bytes receive a status word
 * (0 = ok) that dcn_read_status() returns.
 *
 * Replaces the body of modulated_deform_conv_forward
 * (mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:62-138, :395-412) and of
 * deform_conv_forward (mmcv/ops/csrc/pytorch/deform_conv.cpp:140-260) together
 * with the gather kernels they launch
 * (mmcv/ops/csrc/common/cuda/modulated_deform_conv_cuda_kernel.cuh:186-245,
 *  mmcv/ops/csrc/common/cuda/deform_conv_cuda_kernel.cuh:190-241).
 */
int dcn_fwd(const DcnFwdParams *p, void *workspace, size_t workspace_bytes,
            void *stream);

/*
 * Weights change once per optimiser step at most, the forward runs every call: these two
 * let a caller keep the re-laid-out (tiled, swizzled, type-converted) weights.
 * dcn_weight_image_bytes reports the image size for the problem (0 when the problem runs on
 * a kernel that reads `weight` directly); dcn_prepare_weights enqueues the re-layout of
 * p->weight into `image` (device memory, 256-byte aligned).  The image depends on the
 * weights' values, dtype and shape, groups, and the math mode; pass it back in
 * DcnFwdParams.weight_image together with its size.  (No counterpart in the reference, which
 * feeds `weight` to its GEMM as is.)
 */
int dcn_weight_image_bytes(const DcnFwdParams *p, size_t *bytes);
int dcn_prepare_weights(const DcnFwdParams *p, void *image, size_t image_bytes, void *stream);

/* Measurement aid: dcn_fwd with every kernel bracketed by CUDA events on `stream`.
 * Waits for the work to finish and reports the device time of each launch in
 * milliseconds: ms[0] channels-last restaging of the input, ms[1] weight tiling,
 * ms[2] the main kernel (0 for a launch the plan does not contain).  Creates and
 * destroys four CUDA events; otherwise the same contract as dcn_fwd. */
int dcn_fwd_profiled(const DcnFwdParams *p, void *workspace, size_t workspace_bytes,
                     void *stream, float ms[3]);

/*
 * dcn_fwd for callers that can neither pass a workspace nor allocate one: a host that
 * gives a plugin only input/output buffers and a stream, or a process whose framework
 * has reserved all device memory so that an allocation made inside a library call fails.
 * (No counterpart in the reference, whose entry points allocate their column buffer
 * through the tensor library on every call.)
 *
 * The scratch is a fixed DCN_STATIC_SCRATCH_BYTES array inside the library's device
 * image; problems whose dcn_fwd_workspace_bytes() exceeds it are rejected with
 * DCN_ERR_WORKSPACE and a message naming both sizes.  The call performs no cudaMalloc,
 * cudaFree or other allocating routine.  The first call on each device resolves the
 * array's device address (a one-time runtime query made with that device current), so
 * make that first call outside any stream capture.  All calls on a device share the
 * array and it keeps the previous call's contents (the status word is cleared at the
 * start of every call; everything else is rewritten before use); calls that overlap on
 * the same GPU race on it and must be serialised by the caller.  If `scratch` is not
 * NULL it receives the array's device address, which dcn_read_status() accepts.
 */
#define DCN_STATIC_SCRATCH_BYTES (32u << 20)
int dcn_fwd_static_scratch(const DcnFwdParams *p, void *stream, void **scratch);

/*
 * Backward building blocks (first version: the three sampling kernels; the two matrix
 * products of the backward stay with the caller's BLAS, as in the reference, which calls
 * addmm_ for them: mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:183-230).
 * All take the forward problem description (`weight`, `bias`, `output` unused) and a sample
 * range [n0, n1).  Gradients and columns are fp32 whatever the tensors' dtype.
 *
 * dcn_bwd_columns : columns[(n-n0)*C*T + c*T + tap][Ho*Wo], the sampled (and modulated)
 *   input, K order as weight.flatten(1); replaces modulated_deformable_im2col
 *   (mmcv/ops/csrc/common/cuda/modulated_deform_conv_cuda_kernel.cuh:186-245).
 * dcn_bwd_input   : grad_input [N,C,H,W] (dense fp32) += scatter of grad_columns (same
 *   layout as columns) to the bilinear corners; replaces modulated_deformable_col2im
 *   (same file, :247-307).  Uses atomic adds: zero grad_input before the first call.
 * dcn_bwd_coord   : grad_offset [N, dg*2*T, Ho, Wo] and grad_mask [N, dg*T, Ho, Wo] (dense
 *   fp32; grad_mask may be NULL for the v1 operator), assigned for samples [n0, n1);
 *   replaces modulated_deformable_col2im_coord (same file, :309-397).
 * The unmodulated twins are mmcv/ops/csrc/common/cuda/deform_conv_cuda_kernel.cuh:243-365.
 */
int dcn_bwd_columns(const DcnFwdParams *p, int64_t n0, int64_t n1, float *columns, void *stream);
int dcn_bwd_input(const DcnFwdParams *p, int64_t n0, int64_t n1, const float *grad_columns,
                  float *grad_input, void *stream);
int dcn_bwd_coord(const DcnFwdParams *p, int64_t n0, int64_t n1, const float *grad_columns,
                  float *grad_offset, float *grad_mask, void *stream);

/* Test aid for the bounded device-side waits.  Every wait of the tensor-core kernel gives up
 * after a time limit, sets the status word and lets the kernel return.  wait_limit_ns
 * shortens that limit for later calls in this process (0 = the default of two seconds);
 * flags bit 0 makes the weight loader of the 16-bit kernel withhold its very last copy, so
 * that the wait for it runs out.  Not for production use. */
int dcn_debug_configure(uint64_t wait_limit_ns, int32_t flags);

/* Tracing aid.  When the environment variable DCN_B200_COUNTERS=1 is set, the first
 * block of the tensor-core kernel accumulates the clock cycles its roles spend in each
 * phase into 24 counters in the workspace header; this call synchronises `stream` and
 * copies them out.  Index: 0 producer other, 1 tap-table build, 2 producer rendezvous,
 * 3 wait for a free operand stage, 4 gather+blend, 5 stages produced (count), 6 tables
 * built (count), 7 publish stage; 8 MMA waits for weights, 9 MMA waits for operand,
 * 10 MMA waits for a free accumulator, 11 MMA issue; 12 epilogue waits for accumulator,
 * 13 epilogue work; 14 loader waits for a free stage, 15 loader issue. */
int dcn_read_counters(const void *workspace, void *stream, uint64_t counters[24]);

/* Synchronises `stream`, then returns the status word the last dcn_fwd on this
 * workspace left: 0 ok; non-zero = a bounded device-side wait gave up
 * (the kernel returned early, the output is not valid). */
int dcn_read_status(const void *workspace, void *stream, int32_t *status);

/*
 * Layout helper: copies a 4-D tensor [N, C, H, W] (element strides `in_stride`, dtype
 * DCN_DTYPE_*) into a dense channels-last image [N, H, W, C] of the same type at `output`
 * (16-byte aligned), on `stream`.  dcn_fwd reads such a copy without restaging it, so a caller
 * that feeds the same activations to several layers (the Pack layers: offset branch +
 * deformable kernel) makes it once.  (No counterpart in the reference, which keeps NCHW.)
 */
int dcn_to_channels_last(const void *input, void *output, int32_t dtype, int64_t N, int64_t C,
                         int64_t H, int64_t W, const int64_t in_stride[4], int32_t device,
                         void *stream);

/*
 * The copy the 16-bit tensor-core kernels sample: channels-last, every sample surrounded by a
 * one-pixel zero border, one more all-zero row at the end: [N][H+2][W+2][C] + [W+2][C]
 * elements of the tensor's own 16-bit type (bf16 / fp16; C a multiple of 8).
 * dcn_padded_bytes reports its size; dcn_pad_channels_last enqueues the copy of a 4-D tensor
 * [N, C, H, W] with element strides `in_stride` into `padded` (256-byte aligned) on `stream`.
 * Pass the result in DcnFwdParams.padded_input.  (No counterpart in the reference, which keeps
 * NCHW and pads inside its gather.)
 */
int dcn_padded_bytes(int32_t dtype, int64_t N, int64_t C, int64_t H, int64_t W, size_t *bytes);
int dcn_pad_channels_last(const void *input, void *padded, int32_t dtype, int64_t N, int64_t C,
                          int64_t H, int64_t W, const int64_t in_stride[4], int32_t device,
                          void *stream);

/*
 * Ordinary convolution (no offsets, no mask: those two fields of `p` are ignored) with the
 * problem description of dcn_fwd, on a tensor-core kernel whose operand tiles are written by
 * tensor-map box copies from the padded input: the offset / mask branch of the Pack layers
 * (mmcv/ops/modulated_deform_conv.py:311-335, mmcv/ops/deform_conv.py:397-415), for which the
 * reference calls a library convolution.  16-bit tensors; channels per group a multiple of 64
 * or one group; otherwise DCN_ERR_UNSUPPORTED (dcn_fwd with offset == NULL computes the same
 * on the general kernel).  Workspace: dcn_conv_workspace_bytes.
 */
int dcn_conv_workspace_bytes(const DcnFwdParams *p, size_t *bytes);
int dcn_conv_fwd(const DcnFwdParams *p, void *workspace, size_t workspace_bytes, void *stream);

/*
 * The two reference entry points with flat arguments, in the reference's own
 * argument order and meaning.  `elem` is DCN_DTYPE_*; sizes are in elements.
 *
 * dcn_modulated_deform_conv_forward is what a binding of
 *   modulated_deform_conv_forward(input, weight, bias, ones, offset, mask, output,
 *     columns, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w, dilation_h,
 *     dilation_w, group, deformable_group, with_bias)
 * (mmcv/ops/csrc/pytorch/pybind.cpp:157-162, :641-648) calls; the reference's
 * scratch handles `ones` and `columns` have no counterpart because no column
 * buffer exists.
 */
int dcn_modulated_deform_conv_forward(
    const void *input, const void *weight, const void *bias, const void *offset,
    const void *mask, void *output, int32_t elem, int64_t batch, int64_t channels,
    int64_t height, int64_t width, int64_t channels_out, int32_t kernel_h,
    int32_t kernel_w, int32_t stride_h, int32_t stride_w, int32_t pad_h,
    int32_t pad_w, int32_t dilation_h, int32_t dilation_w, int32_t group,
    int32_t deformable_group, int32_t with_bias, int32_t device, void *workspace,
    size_t workspace_bytes, void *stream);

/*
 * dcn_deform_conv_forward is what a binding of
 *   deform_conv_forward(input, weight, offset, output, columns, ones, kW, kH, dW, dH,
 *     padW, padH, dilationW, dilationH, group, deformable_group, im2col_step)
 * (mmcv/ops/csrc/pytorch/pybind.cpp:38-42, :525-530) calls.  Width comes before
 * height in the scalar arguments, as in the reference.  im2col_step is accepted
 * and only validated (batch % im2col_step == 0): there is no column buffer to chunk.
 */
int dcn_deform_conv_forward(
    const void *input, const void *weight, const void *offset, void *output,
    int32_t elem, int64_t batch, int64_t channels, int64_t height, int64_t width,
    int64_t channels_out, int32_t kW, int32_t kH, int32_t dW, int32_t dH,
    int32_t padW, int32_t padH, int32_t dilationW, int32_t dilationH,
    int32_t group, int32_t deformable_group, int32_t im2col_step, int32_t device,
    void *workspace, size_t workspace_bytes, void *stream);

/* Workspace size for the two flat entry points (same arguments, no pointers). */
int dcn_forward_workspace_bytes(int32_t elem, int32_t modulated, int64_t batch,
                                int64_t channels, int64_t height, int64_t width,
                                int64_t channels_out, int32_t kernel_h,
                                int32_t kernel_w, int32_t stride_h, int32_t stride_w,
                                int32_t pad_h, int32_t pad_w, int32_t dilation_h,
                                int32_t dilation_w, int32_t group,
                                int32_t deformable_group, size_t *bytes);

/*
 * Multi-scale deformable attention, the sibling sampler of the deformable convolutions
 * (same bilinear gather, gate and per-corner validity; a weighted sum over levels and points
 * instead of a contraction with weights).
 *
 * dcn_msda_forward is what a binding of
 *   ms_deform_attn_forward(value, spatial_shapes, level_start_index, sampling_loc, attn_weight,
 *                          im2col_step)
 * (mmcv/ops/csrc/pytorch/pybind.cpp:172-176, :812-816; CUDA body
 * mmcv/ops/csrc/pytorch/cuda/ms_deform_attn_cuda.cu:203-277) calls after allocating `output`
 * [batch][num_query][num_heads * channels]; the reference's loop over im2col_step chunks has no
 * counterpart (one launch covers the batch; the binding keeps the divisibility check).
 * value is [batch][spatial_size][num_heads][channels], sampling_loc
 * [batch][num_query][num_heads][num_levels][num_point][2] as (x, y) in [0, 1], attn_weight the
 * same without the last axis; all three and output have element type `dtype`;
 * spatial_shapes ([num_levels][2] as (h, w)) and level_start_index ([num_levels]) are int64
 * arrays in DEVICE memory, as in the reference.  Asynchronous on `stream`, no allocation.
 *
 * dcn_msda_backward replaces ms_deform_attn_backward (pybind.cpp:177-184, :817-824; CUDA body
 * ms_deform_attn_cuda.cu:279-351): it ADDS to grad_value ([batch][spatial_size][num_heads][channels])
 * and writes grad_sampling_loc and grad_attn_weight (shapes of sampling_loc and attn_weight); the
 * three gradient buffers are fp32 whatever `dtype` is and must be zero on entry.
 */
int dcn_msda_forward(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                     const void *sampling_loc, const void *attn_weight, void *output, int32_t dtype,
                     int64_t batch, int64_t spatial_size, int64_t num_heads, int64_t channels,
                     int64_t num_levels, int64_t num_query, int64_t num_point, int32_t device,
                     void *stream);
int dcn_msda_backward(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                      const void *sampling_loc, const void *attn_weight, const void *grad_output,
                      float *grad_value, float *grad_sampling_loc, float *grad_attn_weight, int32_t dtype,
                      int64_t batch, int64_t spatial_size, int64_t num_heads, int64_t channels,
                      int64_t num_levels, int64_t num_query, int64_t num_point, int32_t device,
                      void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DCN_B200_H_ */
