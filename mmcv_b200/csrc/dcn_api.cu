// C-ABI layer: argument checks (the reference's own, plus what a raw-pointer interface
// needs), kernel selection, workspace layout and launch sequencing.
//
// Checks restated from the reference:
//   kernel size / channel consistency .. mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:80-85
//   positive kernel/stride/dilation, C % deformable_group, output size >= 1,
//   input >= kernel (v1) ............... mmcv/ops/csrc/pytorch/deform_conv.cpp:45-138
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>

#include "dcn_internal.cuh"

namespace dcn {
size_t tc_smem_bytes(const TcPlan &tp, int T);

// Test-only knobs of the bounded waits (dcn_debug_configure).
std::atomic<unsigned long long> g_wait_limit_ns{0};
std::atomic<int> g_debug_flags{0};

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

constexpr size_t kMaxSmemOptin = 232448;  // 227 KiB per block on sm_100
constexpr int kSmCountFallback = 148;

struct DeviceInfo {
  bool probed = false;
  int err = 0;
  int sms = 0;
  int cc_major = 0;
  size_t tc_smem_set = 0;
};
DeviceInfo g_dev[64];
std::mutex g_mu;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Tuning knobs read from the environment (experiments only; defaults are the tuned values).
int env_int(const char *name, int dflt, int lo, int hi) {
  const char *v = getenv(name);
  if (!v || !*v) return dflt;
  const int x = atoi(v);
  return x < lo ? lo : (x > hi ? hi : x);
}
// All of them, read once per process (the first call that plans a problem).
struct Knobs {
  int a_stages, b_stages, producers, tile_w, simt_tiled, counters;
  int kernel;      // 1: first-generation tensor-core kernel always, 2: default routing, 3: second generation wherever it fits
  int window;      // -1: planner's choice, 0: no shared-memory input window, n: margin n
  int epi_tma;     // -1: planner's choice, 0/1
  int small_l1;    // 1: give the kernel the largest shared-memory configuration
  int a2_max;      // deepest operand ring the table-free kernel may take
};
const Knobs &knobs() {
  static Knobs k;
  static std::once_flag once;
  std::call_once(once, [] {
    k.a_stages = env_int("DCN_B200_A_STAGES", 0, 0, 8);
    k.b_stages = env_int("DCN_B200_B_STAGES", 0, 0, 8);
    k.producers = env_int("DCN_B200_PRODUCERS", 0, 0, 9999);
    k.tile_w = env_int("DCN_B200_TILE_W", 0, 0, 128);
    k.simt_tiled = env_int("DCN_B200_SIMT_TILED", 1, 0, 1);
    k.counters = env_int("DCN_B200_COUNTERS", 0, 0, 1);
    k.kernel = env_int("DCN_B200_KERNEL", 2, 1, 3);
    k.window = env_int("DCN_B200_WINDOW", -1, -1, 16);
    k.epi_tma = env_int("DCN_B200_EPI_TMA", -1, -1, 1);
    k.small_l1 = env_int("DCN_B200_SMALL_L1", 0, 0, 1);
    k.a2_max = env_int("DCN_B200_A2_MAX", 6, 2, 8);
  });
  return k;
}

// Makes `device` current for the lifetime of the object and restores the caller's device
// afterwards (the reference scopes its device switch the same way,
// mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:68).
struct DeviceScope {
  int prev = -1;
  bool switched = false;
  cudaError_t err = cudaSuccess;
  explicit DeviceScope(int device) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != device) {
      err = cudaSetDevice(device);
      switched = err == cudaSuccess;
    }
  }
  ~DeviceScope() {
    if (switched) cudaSetDevice(prev);
  }
};

int build_geom(const DcnFwdParams *p, Geom *g) {
  if (!p) return fail(DCN_ERR_ARG, "params is NULL");
  if (p->dtype != DCN_DTYPE_F32 && p->dtype != DCN_DTYPE_BF16 && p->dtype != DCN_DTYPE_F16)
    return fail(DCN_ERR_UNSUPPORTED, "unsupported element type %d (fp32, bf16 and fp16 only)",
                p->dtype);
  if (p->math_mode < DCN_MATH_AUTO || p->math_mode > DCN_MATH_BF16)
    return fail(DCN_ERR_ARG, "unknown math mode %d", p->math_mode);
  if (p->kh <= 0 || p->kw <= 0)
    return fail(DCN_ERR_ARG, "kernel size should be greater than zero, but got kH: %d kW: %d",
                p->kh, p->kw);
  if (p->stride_h <= 0 || p->stride_w <= 0)
    return fail(DCN_ERR_ARG, "stride should be greater than zero, but got dH: %d dW: %d",
                p->stride_h, p->stride_w);
  if (p->dil_h <= 0 || p->dil_w <= 0)
    return fail(DCN_ERR_ARG, "dilation should be greater than 0, but got dilationH: %d dilationW: %d",
                p->dil_h, p->dil_w);
  if (p->pad_h < 0 || p->pad_w < 0) return fail(DCN_ERR_ARG, "padding must be non-negative");
  if (p->N < 0 || p->C <= 0 || p->H <= 0 || p->W <= 0 || p->Co <= 0)
    return fail(DCN_ERR_ARG, "tensor sizes must be positive (N=%lld C=%lld H=%lld W=%lld Co=%lld)",
                (long long)p->N, (long long)p->C, (long long)p->H, (long long)p->W,
                (long long)p->Co);
  if (p->groups <= 0 || p->deform_groups <= 0)
    return fail(DCN_ERR_ARG, "group and deformable_group must be positive");
  if (p->C % p->groups != 0 || p->Co % p->groups != 0)
    return fail(DCN_ERR_ARG, "Input shape and kernel channels won't match: (%lld vs groups %d).",
                (long long)p->C, p->groups);
  if (p->C % p->deform_groups != 0)
    return fail(DCN_ERR_ARG, "input channels must divide deformable group size");
  const long long Ho = (p->H + 2LL * p->pad_h - (p->dil_h * (p->kh - 1LL) + 1)) / p->stride_h + 1;
  const long long Wo = (p->W + 2LL * p->pad_w - (p->dil_w * (p->kw - 1LL) + 1)) / p->stride_w + 1;
  if ((p->H + 2LL * p->pad_h - (p->dil_h * (p->kh - 1LL) + 1)) < 0 ||
      (p->W + 2LL * p->pad_w - (p->dil_w * (p->kw - 1LL) + 1)) < 0 || Ho < 1 || Wo < 1)
    return fail(DCN_ERR_ARG,
                "Given input size: (%lld x %lld x %lld). Calculated output size: (%lld x %lld x "
                "%lld). Output size is too small",
                (long long)p->C, (long long)p->H, (long long)p->W, (long long)p->Co, Ho, Wo);
  const long long lim = 2147483647LL;
  if (p->N > lim || p->C > lim || p->H > lim || p->W > lim || p->Co > lim || Ho * Wo > lim ||
      p->H * p->W * p->C > lim || (long long)p->kh * p->kw > 4096)
    return fail(DCN_ERR_UNSUPPORTED, "a per-sample tensor exceeds 2^31 elements");
  memset(g, 0, sizeof(*g));
  g->N = (int)p->N; g->C = (int)p->C; g->H = (int)p->H; g->W = (int)p->W; g->Co = (int)p->Co;
  g->Ho = (int)Ho; g->Wo = (int)Wo;
  g->kh = p->kh; g->kw = p->kw; g->T = p->kh * p->kw;
  g->stride_h = p->stride_h; g->stride_w = p->stride_w;
  g->pad_h = p->pad_h; g->pad_w = p->pad_w; g->dil_h = p->dil_h; g->dil_w = p->dil_w;
  g->groups = p->groups; g->dg = p->deform_groups;
  g->Cg = g->C / g->groups; g->Cog = g->Co / g->groups; g->cpdg = g->C / g->dg;
  g->P = (long long)g->N * Ho * Wo;
  g->in_sn = p->in_stride[0]; g->in_sc = p->in_stride[1];
  g->in_sh = p->in_stride[2]; g->in_sw = p->in_stride[3];
  const bool nchw = g->in_sw == 1 && g->in_sh == g->W && g->in_sc == (long long)g->H * g->W &&
                    (g->N <= 1 || g->in_sn >= (long long)g->C * g->H * g->W);
  const bool nhwc = g->in_sc == 1 && g->in_sw == g->C && g->in_sh == (long long)g->W * g->C &&
                    (g->N <= 1 || g->in_sn >= (long long)g->C * g->H * g->W);
  if (!nchw && !nhwc && !(g->C == 1 && g->in_sw == 1 && g->in_sh == g->W))
    return fail(DCN_ERR_ARG, "input must be NCHW-contiguous or channels-last");
  g->off_sn = p->offset_batch_stride ? p->offset_batch_stride : (long long)g->dg * 2 * g->T * Ho * Wo;
  g->msk_sn = p->mask_batch_stride ? p->mask_batch_stride : (long long)g->dg * g->T * Ho * Wo;
  g->out_sn = p->out_batch_stride ? p->out_batch_stride : (long long)g->Co * Ho * Wo;
  g->off_cs = p->offset_channel_stride ? p->offset_channel_stride : (long long)Ho * Wo;
  g->off_ps = p->offset_pixel_stride ? p->offset_pixel_stride : 1;
  g->msk_cs = p->mask_channel_stride ? p->mask_channel_stride : (long long)Ho * Wo;
  g->msk_ps = p->mask_pixel_stride ? p->mask_pixel_stride : 1;
  g->mask_act = p->mask_act;
  if (g->mask_act != DCN_ACT_NONE && g->mask_act != DCN_ACT_SIGMOID)
    return fail(DCN_ERR_ARG, "unknown mask activation %d", g->mask_act);
  g->act = p->act; g->act_lo = p->act_lo; g->act_hi = p->act_hi;
  if (g->act != DCN_ACT_NONE && g->act != DCN_ACT_SIGMOID)
    return fail(DCN_ERR_ARG, "unknown activation %d", g->act);
  return DCN_OK;
}

// The input can be gathered from where it lies: channels-last, dense, and already in the
// element type the mode samples (bf16 for the bf16 contraction, fp32 for TF32x3).
bool input_is_ready(const DcnFwdParams *p, const Geom &g, int op_format) {
  const int want = op_format == 2 ? DCN_DTYPE_F32 : (op_format == 0 ? DCN_DTYPE_F16 : DCN_DTYPE_BF16);
  return p->dtype == want && g.in_sc == 1 && g.in_sw == g.C &&
         g.in_sh == (long long)g.W * g.C && g.in_sn == (long long)g.H * g.W * g.C;
}

int resolved_math(const DcnFwdParams *p) {
  return p->math_mode == DCN_MATH_AUTO
             ? (p->dtype == DCN_DTYPE_F32 ? DCN_MATH_TF32X3 : DCN_MATH_BF16)
             : p->math_mode;
}


// Second-generation 16-bit kernel: K units, table segments, ring depths, input window,
// epilogue stores.  Leaves the plan on the first-generation kernel when the problem does not fit.
void plan_tc2(const DcnFwdParams *p, const Geom &g, TcPlan *tp) {
  const Knobs &kn = knobs();
  // offsets into the padded copy are 31-bit byte offsets within a sample
  if ((long long)(g.H + 3) * (g.W + 2) * g.C * 2 >= 2147483647LL) return;
  if (tp->items >= 2147483647LL) return;
  // Routing (measured on C = 64..512, 1..8 deform groups): every lane of this kernel computes
  // the tap entry of its (row, unit) afresh, while the first-generation kernel shares one tap
  // table between the chunks of a deform group.  With 64 or fewer channels per deform group
  // there is little to share and this kernel wins; above that the first generation does.
  // (one measured exception: 128 channels in one deform group, where the table would be shared by
  // two chunks only: C128 168x100 N16 0.294 ms here against 0.313 ms)
  if (kn.kernel != 3 && g.cpdg > 64 && !(g.cpdg == 128 && g.C == 128)) return;
  TcPlan t = *tp;
  t.version = 2;
  t.producer_cfg = 16;  // 16 gather warps that build their own tap entries
  // K units: (32-channel half-chunk, tap), half-chunk-major; two per k-stage
  t.KH = (g.Cg + 31) / 32;
  t.U = t.KH * g.T;
  t.S = (t.U + 1) / 2;
  // A unit must lie inside one deform group (every lane builds the tap entry of one (row, unit)
  // pair): deform groups that start or end inside a 32-channel half-chunk go to the
  // first-generation kernel.
  for (int grp = 0; grp < g.groups; ++grp)
    for (int hc = 0; hc < t.KH; ++hc) {
      const int c0 = grp * g.Cg + hc * 32;
      const int c1 = c0 + 32 < (grp + 1) * g.Cg ? c0 + 32 : (grp + 1) * g.Cg;
      if (c0 / g.cpdg != (c1 - 1) / g.cpdg) return;
    }
  // (the kernel keeps a 3 KiB lookup table of its K units: 16 bytes x 2 S entries x conv groups,
  // with 8-bit half-chunk numbers, 16-bit offset / mask channel numbers and 23-bit channel byte
  // offsets)
  if ((long long)g.groups * 2 * t.S * 16 > 3072 || t.KH > 255 || (long long)g.dg * g.T > 32767 ||
      g.C >= (1 << 22))
    return;
  // A 1x1 kernel makes every K unit a half-chunk of its own: a gather group would then pass whole
  // input windows without touching them and hand several back at once, which the two-buffer
  // window ring (one arrival per warp, window and phase) does not allow.  Such layers stay on
  // the first-generation kernel.
  if (g.T < 2) return;
  t.ndu = 1;
  t.tab_span = t.tab_slots = t.tab_slot_blocks = 0;
  // Epilogue through the tensor-copy engine: needs 16-byte multiples everywhere and tiles
  // whose 32-channel slabs never reach into another tile's channels.
  {
    const long long es = t.io_bytes;
    const bool aligned = (g.Wo * es) % 16 == 0 && ((long long)g.Ho * g.Wo * es) % 16 == 0 &&
                         (g.out_sn * es) % 16 == 0 && ((uintptr_t)p->output & 15) == 0;
    const bool slabs_ok = g.Cog % t.BN == 0 || g.groups * t.NT == 1;
    const int want = kn.epi_tma < 0 ? 1 : kn.epi_tma;
    t.epi_tma = (want && aligned && slabs_ok && g.N > 0) ? 1 : 0;
  }
  t.raw_slots = 0;
  // Input window in shared memory: the tile's undeformed footprint plus a margin of m pixels
  // on every side, 32 channels, two buffers.  Largest margin (up to 6) that fits wins; the
  // width is rounded up to an even number of pixels (bank rule of the paired reads).
  const int th = kBM >> t.tw_log2, tw = 1 << t.tw_log2;
  const int fh = (th - 1) * g.stride_h + (g.kh - 1) * g.dil_h + 2;  // + the lower/right corner
  const int fw = (tw - 1) * g.stride_w + (g.kw - 1) * g.dil_w + 2;
  // Used when the convolution has unit stride (deformable layers of detection backbones: small
  // learned offsets around a dense footprint); a strided layer samples too widely for a window
  // of this size and stays on the first-generation kernel, as does a problem whose window
  // would have a margin of less than three pixels.
  const bool auto_win = g.stride_h == 1 && g.stride_w == 1;
  const int m_max = kn.window < 0 ? (auto_win ? 6 : 0) : kn.window;
  bool found = false;
  const int epi_wanted = t.epi_tma;
  for (int m = m_max; m >= 0 && !found; --m) {
    t.win_h = m ? fh + 2 * m : 0;
    t.win_w = m ? (fw + 2 * m + 1) / 2 * 2 : 0;
    t.win_my = t.win_mx = m;
    if (m && (t.win_h > 256 || t.win_w > 256)) continue;
    // without a window the gather lives on L1: stay inside the 164 KB shared-memory
    // configuration if possible
    const size_t budgets[2] = {167936 - 1024, kMaxSmemOptin};
    for (int bi = (m || kn.small_l1) ? 1 : 0; bi < 2 && !found; ++bi)
      for (int as = kn.a2_max; as >= 2 && !found; --as) {
        if (kn.a_stages && as != kn.a_stages && !(kn.a_stages >= 4 && as > 4)) continue;
        // A deeper operand ring is worth more than tensor stores in the epilogue (c5: a fourth
        // stage -5.5 %, the store kind +-0): give up the stores' staging memory before a stage.
        for (int epi = epi_wanted; epi >= (kn.epi_tma == 1 ? 1 : 0) && !found; --epi) {
          t.epi_tma = epi;
          t.a_stages = as;
          t.b_stages = kn.b_stages ? kn.b_stages : 2;
          t.smem = tc2_smem_bytes(t);
          found = t.smem <= budgets[bi];
        }
      }
  }
  if (!found) return;
  if (kn.window < 0 && t.win_my < 3) return;   // no useful window: first-generation kernel
  *tp = t;
}

// Decide whether the tensor-core kernel can take the problem and with what tiling.
bool plan_tc(const DcnFwdParams *p, const Geom &g, int sms, TcPlan *tp, bool allow_v2 = true) {
  const int math = resolved_math(p);
  if (math != DCN_MATH_BF16 && math != DCN_MATH_TF32X3) return false;
  const bool tf32 = math == DCN_MATH_TF32X3;
  const int ch = tf32 ? 32 : 64, cpv = tf32 ? 4 : 8;
  if (g.Cg % cpv != 0 || g.cpdg % cpv != 0) return false;
  if ((long long)g.N * g.H * g.W >= 2147483647LL) return false;
  if ((long long)(g.H + 2) * (g.W + 2) * g.C * (tf32 ? 4 : 2) >= 4294967295LL) return false;
  if (g.kh > 255 || g.kw > 255 || g.T > 4095) return false;
  const Knobs &kn = knobs();
  const int a_forced = kn.a_stages, b_forced = kn.b_stages;
  // Output channels per tile: as many as fit (fewest passes over the gather); TF32x3 needs
  // twice the operand memory per stage and may have to halve it.
  bool found = false;
  for (int cap = 256; cap >= 32 && !found; cap /= 2) {
    memset(tp, 0, sizeof(*tp));
    tp->tiles_per_stage = tf32 ? 2 : 1;
    // 16-bit operands are in the tensors' own 16-bit type; fp32 tensors asked to run the
    // 16-bit contraction use bf16
    tp->op_format = tf32 ? 2 : (p->dtype == DCN_DTYPE_F16 ? 0 : 1);
    tp->ch_per_stage = ch;
    tp->io_bytes = p->dtype == DCN_DTYPE_F32 ? 4 : 2;
    tp->NT = (g.Cog + cap - 1) / cap;
    const int per = (g.Cog + tp->NT - 1) / tp->NT;
    tp->BN = (per + 31) / 32 * 32;
    tp->KC = (g.Cg + ch - 1) / ch;
    tp->S = tp->KC * g.T;
    int ndgc = 1;
    bool chunks_share_groups = false;  // two consecutive chunks of a tile with the same deform groups
    for (int grp = 0; grp < g.groups; ++grp) {
      int prev_lo = -1, prev_nd = 0;
      for (int cc = 0; cc < tp->KC; ++cc) {
        const int c0 = grp * g.Cg + cc * ch;
        const int c1 = c0 + ch < (grp + 1) * g.Cg ? c0 + ch : (grp + 1) * g.Cg;  // chunk end
        const int lo = c0 / g.cpdg, hi = (c1 - 1) / g.cpdg;
        const int nd = hi - lo + 1;
        if (nd > ndgc) ndgc = nd;
        if (lo == prev_lo && nd == prev_nd) chunks_share_groups = true;
        prev_lo = lo;
        prev_nd = nd;
      }
    }
    if (ndgc > 15) return false;
    tp->ndgc = ndgc;
    // Producer layout (measured best on every workload tried): two groups of eight warps,
    // two rows per thread in flight, rows software-pipelined.  When every chunk of a tile has
    // deform groups of its own, the tap table is rebuilt per chunk anyway, and each group
    // keeps a table of just its own taps (3282): one group rebuilds while the other gathers.
    // When chunks share deform groups the table is shared and lives as long as they do (1282).
    // The batched layouts (282: same warps, 342: three groups of four) stay selectable.
    const int cfg_default = chunks_share_groups ? 1282 : 3282;
    switch (kn.producers ? kn.producers : cfg_default) {
      case 342: tp->producer_cfg = 342; break;
      case 1282: tp->producer_cfg = 1282; break;
      case 3282: tp->producer_cfg = 3282; break;
      case 282: tp->producer_cfg = 282; break;
      default: tp->producer_cfg = cfg_default; break;
    }
    const int a_min = (tp->producer_cfg / 100) % 10;  // every producer group needs a stage of its own
    int cols = 32;
    while (cols < 2 * tp->BN) cols *= 2;
    tp->tmem_cols = cols;
    // Pipeline depth.  Shared memory the kernel does not take stays L1, and the gather's hit
    // rate depends on it, so first try to fit the 164 KB shared-memory configuration (92 KB
    // of L1), deepest A ring first; only then fall back to the largest configuration.
    const size_t budgets[2] = {167936 - 1024, kMaxSmemOptin};
    for (int bi = 0; bi < 2 && !found; ++bi)
      for (int as = 4; as >= a_min && !found; --as)
        for (int bs = (bi == 0 ? 2 : 4); bs >= 2 && !found; --bs) {
          if ((a_forced && as != a_forced) || (b_forced && bs != b_forced)) continue;
          tp->a_stages = as;
          tp->b_stages = bs;
          tp->smem = tc_smem_bytes(*tp, g.T);
          found = tp->smem <= budgets[bi];
        }
  }
  if (!found) return false;
  // Tile shape: TH x TW pixels of one sample, TH*TW = 128.  Fewest tiles wins; among
  // shapes within 3 % of the fewest, the one closest to square (smallest sampled footprint).
  int best = -1;
  {
    const int forced = kn.tile_w;
    long long tiles[8] = {0}, fewest = -1;
    for (int lg = 3; lg <= 7; ++lg) {
      const int tw = 1 << lg, th = kBM >> lg;
      tiles[lg] = (long long)((g.Wo + tw - 1) / tw) * ((g.Ho + th - 1) / th);
      if (fewest < 0 || tiles[lg] < fewest) fewest = tiles[lg];
    }
    const int preference[5] = {4, 3, 5, 6, 7};  // 8x16, 16x8, 4x32, 2x64, 1x128
    for (int k = 0; k < 5 && best < 0; ++k)
      if (tiles[preference[k]] * 100 <= fewest * 103) best = preference[k];
    for (int lg = 3; lg <= 7; ++lg)
      if (forced == (1 << lg)) best = lg;
  }
  if (best < 0) best = 4;
  tp->tw_log2 = best;
  tp->tiles_x = (g.Wo + (1 << best) - 1) >> best;
  tp->tiles_y = (g.Ho + (kBM >> best) - 1) / (kBM >> best);
  const long long mtiles = (long long)g.N * tp->tiles_x * tp->tiles_y;
  tp->items = mtiles * g.groups * tp->NT;
  tp->grid = (int)(tp->items < sms ? tp->items : sms);
  tp->version = 1;
  if (!tf32 && kn.kernel >= 2 && allow_v2) plan_tc2(p, g, tp);
  // the first-generation 16-bit kernel reads a caller's zero-bordered copy in place
  tp->in_pad = (tp->version == 1 && !tf32 && p->padded_input) ? 1 : 0;
  return true;
}

size_t padded_copy_bytes(const Geom &g) { return ((size_t)g.N * (g.H + 2) + 1) * (g.W + 2) * g.C * 2; }

void layout_workspace(const DcnFwdParams *p, const Geom &g, bool tc, const TcPlan &tp,
                      Workspace *ws) {
  memset(ws, 0, sizeof(*ws));
  size_t off = 256;
  if (tc) {
    ws->wtile_off = off;
    ws->wtile_bytes = (size_t)g.groups * tp.NT * tp.S * tp.BN * 128 * tp.tiles_per_stage;
    off = align_up(off + ws->wtile_bytes, 256);
    if (tp.version == 2) {
      // channels-last copy with a one-pixel zero border per sample and one more zero row
      // (unless the caller brings it)
      if (!p->padded_input) {
        ws->xcl_off = off;
        ws->xcl_bytes = padded_copy_bytes(g);
        off = align_up(off + ws->xcl_bytes, 256);
      }
    } else if (tp.in_pad) {
      // reads the caller's zero-bordered copy
    } else if (!input_is_ready(p, g, tp.op_format)) {
      ws->xcl_off = off;
      ws->xcl_bytes = (size_t)g.N * g.H * g.W * g.C * (tp.tiles_per_stage == 2 ? 4 : 2);
      off = align_up(off + ws->xcl_bytes, 256);
    }
  }
  ws->total = off;
}

int probe_device(int device, DeviceInfo **out) {
  if (device < 0 || device >= 64) return fail(DCN_ERR_ARG, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceInfo &d = g_dev[device];
  if (!d.probed) {
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(DCN_ERR_DEVICE, "no usable CUDA device %d: %s (there is no CPU path)", device,
                  cudaGetErrorString(e));
    }
    d.sms = prop.multiProcessorCount;
    d.cc_major = prop.major;
    d.probed = true;
  }
  if (d.cc_major != 10)
    return fail(DCN_ERR_DEVICE, "device %d is compute capability %d.x; this library is sm_100a only",
                device, d.cc_major);
  *out = &d;
  return DCN_OK;
}

struct Plan {
  Geom g;
  bool tc;
  TcPlan tp;
  Workspace ws;
  int launches;
  bool stage;
  bool have_image;
};

int make_plan(const DcnFwdParams *p, int sms, Plan *pl) {
  int rc = build_geom(p, &pl->g);
  if (rc) return rc;
  if (p->math_mode == DCN_MATH_TF32X3 && p->dtype != DCN_DTYPE_F32)
    return fail(DCN_ERR_ARG, "the 3xTF32 contraction is for fp32 tensors");
  pl->tc = plan_tc(p, pl->g, sms, &pl->tp);
  if (!pl->tc && p->math_mode == DCN_MATH_BF16)
    return fail(DCN_ERR_UNSUPPORTED,
                "bf16 tensor-core contraction needs C/groups %% 8 == 0 and C/deformable_group %% 8 "
                "== 0 (got C/groups=%d, C/deformable_group=%d)", pl->g.Cg, pl->g.cpdg);
  if (!pl->tc) {
    const Geom &g = pl->g;
    const long long plane = (long long)g.Ho * g.Wo;
    if (g.mask_act != DCN_ACT_NONE || g.off_ps != 1 || g.msk_ps != 1 || g.off_cs != plane ||
        g.msk_cs != plane)
      return fail(DCN_ERR_UNSUPPORTED, "strided offsets/masks and mask logits are taken by the "
                  "tensor-core kernel only; this problem runs on another kernel");
  }
  // 3xTF32 on a shape the tensor-core kernel does not take runs on the FFMA kernel: both
  // meet the fp32 tolerance, so the request degrades instead of failing.
  layout_workspace(p, pl->g, pl->tc, pl->tp, &pl->ws);
  pl->stage = pl->tc && pl->ws.xcl_bytes != 0;
  if (pl->tc && (pl->tp.version == 2 || pl->tp.in_pad) && p->padded_input &&
      ((size_t)p->padded_input_bytes != padded_copy_bytes(pl->g) || ((uintptr_t)p->padded_input & 255)))
    return fail(DCN_ERR_ARG, "padded_input must be %zu bytes and 256-byte aligned (got %lld)",
                padded_copy_bytes(pl->g), (long long)p->padded_input_bytes);
  pl->have_image = pl->tc && p->weight_image != nullptr;
  // status clear + main kernel, + weight tiling, + input staging (two launches when the copy
  // carries the zero border: border, interior)
  pl->launches = pl->tc ? (2 + (pl->have_image ? 0 : 1) + (pl->stage ? (pl->tp.version == 2 ? 2 : 1) : 0)) : 2;
  return DCN_OK;
}

}  // namespace

// Error channel for entry points that live in other translation units.
int set_error(int code, const char *msg) { return fail(code, "%s", msg); }

}  // namespace dcn

using namespace dcn;

extern "C" {

int dcn_abi_version(void) { return DCN_ABI_VERSION; }
const char *dcn_last_error(void) { return g_err; }

int dcn_fwd_plan(const DcnFwdParams *p, DcnPlanInfo *info) {
  if (!info) return fail(DCN_ERR_ARG, "info is NULL");
  Plan pl;
  int rc = make_plan(p, kSmCountFallback, &pl);
  if (rc) return rc;
  memset(info, 0, sizeof(*info));
  info->path = pl.tc ? DCN_PATH_TCGEN05
                     : (simt_tiled_supported(pl.g) && pl.g.P * pl.g.Co >= 4096 ? DCN_PATH_SIMT_TILED
                                                                                : DCN_PATH_SIMT_DIRECT);
  info->launches = pl.launches;
  info->stages_input = pl.stage ? 1 : 0;
  info->tile_m = pl.tc ? kBM : 1;
  info->tile_n = pl.tc ? pl.tp.BN : 1;
  info->tile_k = pl.tc ? pl.tp.ch_per_stage : 1;
  info->grid = pl.tc ? pl.tp.grid : 0;
  info->block = pl.tc ? tc_threads(pl.tp) : 256;
  info->kernel_version = pl.tc ? pl.tp.version : 0;
  info->window_h = pl.tc ? pl.tp.win_h : 0;
  info->window_w = pl.tc ? pl.tp.win_w : 0;
  info->table_span = pl.tc ? pl.tp.tab_span : 0;
  info->table_slots = pl.tc ? pl.tp.tab_slots : 0;
  info->epilogue_tensor_stores = pl.tc ? pl.tp.epi_tma : 0;
  info->smem_bytes = pl.tc ? (int64_t)pl.tp.smem : 0;
  info->Ho = pl.g.Ho;
  info->Wo = pl.g.Wo;
  info->workspace_bytes = pl.ws.total;
  info->operand_stages = pl.tc ? pl.tp.a_stages : 0;
  info->weight_stages = pl.tc ? pl.tp.b_stages : 0;
  info->producer_layout = pl.tc ? pl.tp.producer_cfg : 0;
  return DCN_OK;
}

int dcn_fwd_workspace_bytes(const DcnFwdParams *p, size_t *bytes) {
  if (!bytes) return fail(DCN_ERR_ARG, "bytes is NULL");
  Plan pl;
  int rc = make_plan(p, kSmCountFallback, &pl);
  if (rc) return rc;
  *bytes = pl.ws.total;
  return DCN_OK;
}

static int run_fwd(const DcnFwdParams *p, void *workspace, size_t workspace_bytes, void *stream,
                   cudaEvent_t *ev) {
  if (!p) return fail(DCN_ERR_ARG, "params is NULL");
  DeviceInfo *dev = nullptr;
  int rc = probe_device(p->device, &dev);
  if (rc) return rc;
  Plan pl;
  rc = make_plan(p, dev->sms, &pl);
  if (rc) return rc;
  if (pl.g.P != 0 && (!p->input || !p->weight || !p->output))
    return fail(DCN_ERR_ARG, "input, weight and output pointers must be non-NULL");
  if (!workspace || workspace_bytes < pl.ws.total)
    return fail(DCN_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", pl.ws.total,
                workspace ? workspace_bytes : (size_t)0);
  if (((uintptr_t)workspace & 255) != 0)
    return fail(DCN_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  DeviceScope scope(p->device);
  cudaError_t e = scope.err;
  if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
  cudaStream_t s = (cudaStream_t)stream;
  uint8_t *ws = (uint8_t *)workspace;
  int *status = (int *)(ws + pl.ws.status_off);
  Ptrs ptrs{p->input, p->offset, p->mask, p->weight, p->bias, p->output};
  e = launch_clear_status(status, s);
  if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "status clear: %s", cudaGetErrorString(e));
  if (ev) cudaEventRecord(ev[0], s);
  if (pl.g.P == 0) {
    if (ev) for (int i = 1; i < 4; ++i) cudaEventRecord(ev[i], s);
    return DCN_OK;
  }
  if (!pl.tc) {
    if (ev) { cudaEventRecord(ev[1], s); cudaEventRecord(ev[2], s); }
    // tiny problems stay on the one-thread-per-output kernel: a 64x64 tile would be mostly empty
    const bool tiled = simt_tiled_supported(pl.g) && knobs().simt_tiled &&
                       pl.g.P * pl.g.Co >= 4096;
    e = tiled ? launch_simt_tiled(pl.g, ptrs, p->dtype, s)
              : launch_simt_direct(pl.g, ptrs, p->dtype, s);
    if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "SIMT kernel launch: %s", cudaGetErrorString(e));
    if (ev) cudaEventRecord(ev[3], s);
    return DCN_OK;
  }
  const void *xcl = ((pl.tp.version == 2 || pl.tp.in_pad) && p->padded_input) ? p->padded_input : p->input;
  if (pl.stage) {
    void *dst = ws + pl.ws.xcl_off;
    e = launch_stage_input_cl(pl.g, p->input, p->dtype, dst, pl.tp.op_format,
                              pl.tp.version == 2 ? 1 : 0, s);
    if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "input staging launch: %s", cudaGetErrorString(e));
    xcl = dst;
  }
  if (ev) cudaEventRecord(ev[1], s);
  const void *wimage = ws + pl.ws.wtile_off;
  if (pl.have_image) {
    if ((size_t)p->weight_image_bytes != pl.ws.wtile_bytes || ((uintptr_t)p->weight_image & 255))
      return fail(DCN_ERR_ARG, "weight_image must be %zu bytes and 256-byte aligned (got %lld)",
                  pl.ws.wtile_bytes, (long long)p->weight_image_bytes);
    wimage = p->weight_image;
  } else {
    e = launch_weight_tiles(pl.g, pl.tp, p->weight, p->dtype, ws + pl.ws.wtile_off, s);
    if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "weight tiling launch: %s", cudaGetErrorString(e));
  }
  if (ev) cudaEventRecord(ev[2], s);
  // phase counters live in the workspace header, bytes [64, 256); off unless asked for
  unsigned long long *counters =
      knobs().counters ? (unsigned long long *)(ws + 64) : nullptr;
  e = pl.tp.version == 2
          ? launch_tc2(pl.g, pl.tp, ptrs, p->dtype, xcl, wimage, status, counters,
                       g_wait_limit_ns.load(), g_debug_flags.load(), s)
          : launch_tc(pl.g, pl.tp, ptrs, p->dtype, xcl, wimage, status, counters, s);
  if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "tensor-core kernel launch: %s", cudaGetErrorString(e));
  if (ev) cudaEventRecord(ev[3], s);
  return DCN_OK;
}

int dcn_fwd(const DcnFwdParams *p, void *workspace, size_t workspace_bytes, void *stream) {
  return run_fwd(p, workspace, workspace_bytes, stream, nullptr);
}

int dcn_weight_image_bytes(const DcnFwdParams *p, size_t *bytes) {
  if (!bytes) return fail(DCN_ERR_ARG, "bytes is NULL");
  Plan pl;
  int rc = make_plan(p, kSmCountFallback, &pl);
  if (rc) return rc;
  *bytes = pl.tc ? pl.ws.wtile_bytes : 0;
  return DCN_OK;
}

int dcn_prepare_weights(const DcnFwdParams *p, void *image, size_t image_bytes, void *stream) {
  if (!p) return fail(DCN_ERR_ARG, "params is NULL");
  DeviceInfo *dev = nullptr;
  int rc = probe_device(p->device, &dev);
  if (rc) return rc;
  Plan pl;
  rc = make_plan(p, dev->sms, &pl);
  if (rc) return rc;
  if (!pl.tc) return fail(DCN_ERR_ARG, "this problem runs on a kernel that reads the weights directly");
  if (!p->weight || !image || image_bytes < pl.ws.wtile_bytes || ((uintptr_t)image & 255))
    return fail(DCN_ERR_ARG, "weight and a 256-byte aligned image of %zu bytes are required",
                pl.ws.wtile_bytes);
  DeviceScope scope(p->device);
  cudaError_t e = scope.err;
  if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
  e = launch_weight_tiles(pl.g, pl.tp, p->weight, p->dtype, image, (cudaStream_t)stream);
  return e == cudaSuccess ? DCN_OK : fail(DCN_ERR_CUDA, "weight tiling launch: %s", cudaGetErrorString(e));
}

int dcn_fwd_profiled(const DcnFwdParams *p, void *workspace, size_t workspace_bytes, void *stream,
                     float ms[3]) {
  if (!ms) return fail(DCN_ERR_ARG, "ms is NULL");
  if (!p) return fail(DCN_ERR_ARG, "params is NULL");
  DeviceScope scope(p->device);
  cudaError_t e = scope.err;
  if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
  cudaEvent_t ev[4];
  for (int i = 0; i < 4; ++i) {
    e = cudaEventCreate(&ev[i]);
    if (e != cudaSuccess) {
      for (int j = 0; j < i; ++j) cudaEventDestroy(ev[j]);
      return fail(DCN_ERR_CUDA, "cudaEventCreate: %s", cudaGetErrorString(e));
    }
  }
  int rc = run_fwd(p, workspace, workspace_bytes, stream, ev);
  if (rc == DCN_OK) {
    e = cudaEventSynchronize(ev[3]);
    if (e != cudaSuccess) rc = fail(DCN_ERR_CUDA, "event synchronize: %s", cudaGetErrorString(e));
    for (int i = 0; i < 3 && rc == DCN_OK; ++i) {
      ms[i] = 0.f;
      cudaEventElapsedTime(&ms[i], ev[i], ev[i + 1]);
    }
  }
  for (int i = 0; i < 4; ++i) cudaEventDestroy(ev[i]);
  return rc;
}

static int bwd_common(const DcnFwdParams *p, int64_t n0, int64_t n1, Geom *g) {
  int rc = build_geom(p, g);
  if (rc) return rc;
  if (n0 < 0 || n1 < n0 || n1 > g->N) return fail(DCN_ERR_ARG, "sample range [%lld, %lld) is not inside the batch", (long long)n0, (long long)n1);
  if (!p->input) return fail(DCN_ERR_ARG, "input must be non-NULL");
  DeviceInfo *dev = nullptr;
  rc = probe_device(p->device, &dev);
  if (rc) return rc;
  return DCN_OK;
}

int dcn_bwd_columns(const DcnFwdParams *p, int64_t n0, int64_t n1, float *columns, void *stream) {
  Geom g;
  int rc = bwd_common(p, n0, n1, &g);
  if (rc) return rc;
  if (!columns) return fail(DCN_ERR_ARG, "columns must be non-NULL");
  DeviceScope scope(p->device);
  if (scope.err != cudaSuccess) return fail(DCN_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(scope.err));
  Ptrs ptrs{p->input, p->offset, p->mask, p->weight, p->bias, p->output};
  cudaError_t e = launch_bwd_columns(g, ptrs, p->dtype, (int)n0, (int)(n1 - n0), columns, (cudaStream_t)stream);
  return e == cudaSuccess ? DCN_OK : fail(DCN_ERR_CUDA, "column kernel launch: %s", cudaGetErrorString(e));
}

int dcn_bwd_input(const DcnFwdParams *p, int64_t n0, int64_t n1, const float *grad_columns,
                  float *grad_input, void *stream) {
  Geom g;
  int rc = bwd_common(p, n0, n1, &g);
  if (rc) return rc;
  if (!grad_columns || !grad_input) return fail(DCN_ERR_ARG, "grad_columns and grad_input must be non-NULL");
  DeviceScope scope(p->device);
  if (scope.err != cudaSuccess) return fail(DCN_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(scope.err));
  Ptrs ptrs{p->input, p->offset, p->mask, p->weight, p->bias, p->output};
  cudaError_t e = launch_bwd_input(g, ptrs, p->dtype, (int)n0, (int)(n1 - n0), grad_columns, grad_input, (cudaStream_t)stream);
  return e == cudaSuccess ? DCN_OK : fail(DCN_ERR_CUDA, "input-gradient kernel launch: %s", cudaGetErrorString(e));
}

int dcn_bwd_coord(const DcnFwdParams *p, int64_t n0, int64_t n1, const float *grad_columns,
                  float *grad_offset, float *grad_mask, void *stream) {
  Geom g;
  int rc = bwd_common(p, n0, n1, &g);
  if (rc) return rc;
  if (!grad_columns || !grad_offset) return fail(DCN_ERR_ARG, "grad_columns and grad_offset must be non-NULL");
  DeviceScope scope(p->device);
  if (scope.err != cudaSuccess) return fail(DCN_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(scope.err));
  Ptrs ptrs{p->input, p->offset, p->mask, p->weight, p->bias, p->output};
  cudaError_t e = launch_bwd_coord(g, ptrs, p->dtype, (int)n0, (int)(n1 - n0), grad_columns, grad_offset, grad_mask, (cudaStream_t)stream);
  return e == cudaSuccess ? DCN_OK : fail(DCN_ERR_CUDA, "coordinate-gradient kernel launch: %s", cudaGetErrorString(e));
}

int dcn_debug_configure(uint64_t wait_limit_ns, int32_t flags) {
  g_wait_limit_ns.store(wait_limit_ns);
  g_debug_flags.store(flags);
  return DCN_OK;
}

int dcn_read_counters(const void *workspace, void *stream, uint64_t counters[24]) {
  if (!workspace || !counters) return fail(DCN_ERR_ARG, "workspace and counters must be non-NULL");
  cudaError_t e = cudaMemcpyAsync(counters, (const uint8_t *)workspace + 64, 24 * sizeof(uint64_t),
                                  cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "counter read: %s", cudaGetErrorString(e));
  return DCN_OK;
}

int dcn_read_status(const void *workspace, void *stream, int32_t *status) {
  if (!workspace || !status) return fail(DCN_ERR_ARG, "workspace and status must be non-NULL");
  cudaError_t e = cudaMemcpyAsync(status, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost,
                                  (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "status read: %s", cudaGetErrorString(e));
  return DCN_OK;
}

int dcn_to_channels_last(const void *input, void *output, int32_t dtype, int64_t N, int64_t C,
                         int64_t H, int64_t W, const int64_t in_stride[4], int32_t device,
                         void *stream) {
  if (dtype != DCN_DTYPE_F32 && dtype != DCN_DTYPE_BF16 && dtype != DCN_DTYPE_F16)
    return fail(DCN_ERR_UNSUPPORTED, "dtype %d is not supported (fp32, bf16, fp16)", dtype);
  if (N < 0 || C < 1 || H < 1 || W < 1 || !in_stride)
    return fail(DCN_ERR_ARG, "bad shape [%lld, %lld, %lld, %lld]", (long long)N, (long long)C,
                (long long)H, (long long)W);
  if (N > 2147483647LL || C > 2147483647LL || H * W > 2147483647LL)
    return fail(DCN_ERR_UNSUPPORTED, "tensor too large for 32-bit pixel and channel indices");
  if (N == 0) return DCN_OK;
  if (!input || !output || ((uintptr_t)output & 15))
    return fail(DCN_ERR_ARG, "input and a 16-byte aligned output are required");
  DeviceInfo *dev = nullptr;
  int rc = probe_device(device, &dev);
  if (rc) return rc;
  DeviceScope scope(device);
  cudaError_t e = scope.err;
  if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
  Geom g;
  memset(&g, 0, sizeof(g));
  g.N = (int)N; g.C = (int)C; g.H = (int)H; g.W = (int)W;
  g.in_sn = in_stride[0]; g.in_sc = in_stride[1]; g.in_sh = in_stride[2]; g.in_sw = in_stride[3];
  const int op_format = dtype == DCN_DTYPE_F32 ? 2 : (dtype == DCN_DTYPE_F16 ? 0 : 1);
  e = launch_stage_input_cl(g, input, dtype, output, op_format, 0, (cudaStream_t)stream);
  return e == cudaSuccess ? DCN_OK : fail(DCN_ERR_CUDA, "layout copy launch: %s", cudaGetErrorString(e));
}


int dcn_padded_bytes(int32_t dtype, int64_t N, int64_t C, int64_t H, int64_t W, size_t *bytes) {
  if (!bytes) return fail(DCN_ERR_ARG, "bytes is NULL");
  if (dtype != DCN_DTYPE_BF16 && dtype != DCN_DTYPE_F16)
    return fail(DCN_ERR_UNSUPPORTED, "the padded copy exists for bf16 and fp16 tensors");
  if (N < 0 || C < 1 || H < 1 || W < 1 || C % 8 != 0)
    return fail(DCN_ERR_ARG, "bad shape [%lld, %lld, %lld, %lld] (C must be a multiple of 8)", (long long)N,
                (long long)C, (long long)H, (long long)W);
  *bytes = ((size_t)N * (H + 2) + 1) * (W + 2) * C * 2;
  return DCN_OK;
}

int dcn_pad_channels_last(const void *input, void *padded, int32_t dtype, int64_t N, int64_t C,
                          int64_t H, int64_t W, const int64_t in_stride[4], int32_t device,
                          void *stream) {
  size_t bytes = 0;
  int rc = dcn_padded_bytes(dtype, N, C, H, W, &bytes);
  if (rc) return rc;
  if (!in_stride) return fail(DCN_ERR_ARG, "in_stride is NULL");
  if (N > 2147483647LL || C > 2147483647LL || H * W > 2147483647LL)
    return fail(DCN_ERR_UNSUPPORTED, "tensor too large for 32-bit pixel and channel indices");
  if (N == 0) return DCN_OK;
  if (!input || !padded || ((uintptr_t)padded & 255))
    return fail(DCN_ERR_ARG, "input and a 256-byte aligned destination are required");
  DeviceInfo *dev = nullptr;
  rc = probe_device(device, &dev);
  if (rc) return rc;
  DeviceScope scope(device);
  if (scope.err != cudaSuccess) return fail(DCN_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(scope.err));
  Geom g;
  memset(&g, 0, sizeof(g));
  g.N = (int)N; g.C = (int)C; g.H = (int)H; g.W = (int)W;
  g.in_sn = in_stride[0]; g.in_sc = in_stride[1]; g.in_sh = in_stride[2]; g.in_sw = in_stride[3];
  cudaError_t e = launch_stage_input_cl(g, input, dtype, padded, dtype == DCN_DTYPE_F16 ? 0 : 1, 1,
                                        (cudaStream_t)stream);
  return e == cudaSuccess ? DCN_OK : fail(DCN_ERR_CUDA, "padded copy launch: %s", cudaGetErrorString(e));
}

namespace {
struct ConvPlan {
  Geom g;
  TcPlan tp;
  size_t wtile_off, wtile_bytes, xpad_off, xpad_bytes, total;
};
int make_conv_plan(const DcnFwdParams *p, int sms, ConvPlan *cp) {
  int rc = build_geom(p, &cp->g);
  if (rc) return rc;
  if (p->dtype == DCN_DTYPE_F32)
    return fail(DCN_ERR_UNSUPPORTED, "the tensor-map convolution takes bf16 and fp16 tensors");
  DcnFwdParams q = *p;
  q.math_mode = DCN_MATH_BF16;
  if (!plan_tc(&q, cp->g, sms, &cp->tp, false) || !conv_tma_supported(cp->g, cp->tp))
    return fail(DCN_ERR_UNSUPPORTED, "the tensor-map convolution needs channels per group to be a multiple "
                "of 64 (or one group) and a multiple of 8 (got %d)", cp->g.Cg);
  size_t off = 256;
  cp->wtile_off = off;
  cp->wtile_bytes = (size_t)cp->g.groups * cp->tp.NT * cp->tp.S * cp->tp.BN * 128;
  off = align_up(off + cp->wtile_bytes, 256);
  cp->xpad_off = cp->xpad_bytes = 0;
  if (!p->padded_input) {
    cp->xpad_off = off;
    cp->xpad_bytes = padded_copy_bytes(cp->g);
    off = align_up(off + cp->xpad_bytes, 256);
  } else if ((size_t)p->padded_input_bytes != padded_copy_bytes(cp->g) || ((uintptr_t)p->padded_input & 255)) {
    return fail(DCN_ERR_ARG, "padded_input must be %zu bytes and 256-byte aligned (got %lld)",
                padded_copy_bytes(cp->g), (long long)p->padded_input_bytes);
  }
  cp->total = off;
  return DCN_OK;
}
}  // namespace

int dcn_conv_workspace_bytes(const DcnFwdParams *p, size_t *bytes) {
  if (!bytes) return fail(DCN_ERR_ARG, "bytes is NULL");
  ConvPlan cp;
  int rc = make_conv_plan(p, kSmCountFallback, &cp);
  if (rc) return rc;
  *bytes = cp.total;
  return DCN_OK;
}

int dcn_conv_fwd(const DcnFwdParams *p, void *workspace, size_t workspace_bytes, void *stream) {
  if (!p) return fail(DCN_ERR_ARG, "params is NULL");
  DeviceInfo *dev = nullptr;
  int rc = probe_device(p->device, &dev);
  if (rc) return rc;
  ConvPlan cp;
  rc = make_conv_plan(p, dev->sms, &cp);
  if (rc) return rc;
  if (cp.g.P != 0 && (!p->input || !p->weight || !p->output))
    return fail(DCN_ERR_ARG, "input, weight and output pointers must be non-NULL");
  if (!workspace || workspace_bytes < cp.total)
    return fail(DCN_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", cp.total,
                workspace ? workspace_bytes : (size_t)0);
  if (((uintptr_t)workspace & 255) != 0) return fail(DCN_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  DeviceScope scope(p->device);
  cudaError_t e = scope.err;
  if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
  cudaStream_t s = (cudaStream_t)stream;
  uint8_t *ws = (uint8_t *)workspace;
  e = launch_clear_status((int *)ws, s);
  if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "status clear: %s", cudaGetErrorString(e));
  if (cp.g.P == 0) return DCN_OK;
  const void *xpad = p->padded_input;
  if (!xpad) {
    e = launch_stage_input_cl(cp.g, p->input, p->dtype, ws + cp.xpad_off, cp.tp.op_format, 1, s);
    if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "input staging launch: %s", cudaGetErrorString(e));
    xpad = ws + cp.xpad_off;
  }
  const void *wimage = ws + cp.wtile_off;
  if (p->weight_image) {
    if ((size_t)p->weight_image_bytes != cp.wtile_bytes || ((uintptr_t)p->weight_image & 255))
      return fail(DCN_ERR_ARG, "weight_image must be %zu bytes and 256-byte aligned (got %lld)", cp.wtile_bytes,
                  (long long)p->weight_image_bytes);
    wimage = p->weight_image;
  } else {
    e = launch_weight_tiles(cp.g, cp.tp, p->weight, p->dtype, ws + cp.wtile_off, s);
    if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "weight tiling launch: %s", cudaGetErrorString(e));
  }
  Ptrs ptrs{p->input, nullptr, nullptr, p->weight, p->bias, p->output};
  e = launch_conv_tma(cp.g, cp.tp, ptrs, p->dtype, xpad, wimage, (int *)ws, g_wait_limit_ns.load(), s);
  if (e != cudaSuccess) return fail(DCN_ERR_CUDA, "convolution kernel launch: %s", cudaGetErrorString(e));
  return DCN_OK;
}

static void fill_dense(DcnFwdParams *q, int32_t elem, int64_t batch, int64_t channels,
                       int64_t height, int64_t width, int64_t channels_out, int32_t device) {
  memset(q, 0, sizeof(*q));
  q->dtype = elem;
  q->math_mode = DCN_MATH_AUTO;
  q->N = batch; q->C = channels; q->H = height; q->W = width; q->Co = channels_out;
  q->in_stride[0] = channels * height * width;
  q->in_stride[1] = height * width;
  q->in_stride[2] = width;
  q->in_stride[3] = 1;
  q->device = device;
}

int dcn_modulated_deform_conv_forward(
    const void *input, const void *weight, const void *bias, const void *offset,
    const void *mask, void *output, int32_t elem, int64_t batch, int64_t channels,
    int64_t height, int64_t width, int64_t channels_out, int32_t kernel_h, int32_t kernel_w,
    int32_t stride_h, int32_t stride_w, int32_t pad_h, int32_t pad_w, int32_t dilation_h,
    int32_t dilation_w, int32_t group, int32_t deformable_group, int32_t with_bias,
    int32_t device, void *workspace, size_t workspace_bytes, void *stream) {
  if (!offset || !mask) return fail(DCN_ERR_ARG, "offset and mask must be non-NULL");
  if (with_bias && !bias) return fail(DCN_ERR_ARG, "with_bias is set but bias is NULL");
  DcnFwdParams q;
  fill_dense(&q, elem, batch, channels, height, width, channels_out, device);
  q.input = input; q.weight = weight; q.bias = with_bias ? bias : nullptr;
  q.offset = offset; q.mask = mask; q.output = output;
  q.kh = kernel_h; q.kw = kernel_w; q.stride_h = stride_h; q.stride_w = stride_w;
  q.pad_h = pad_h; q.pad_w = pad_w; q.dil_h = dilation_h; q.dil_w = dilation_w;
  q.groups = group; q.deform_groups = deformable_group;
  return dcn_fwd(&q, workspace, workspace_bytes, stream);
}

int dcn_deform_conv_forward(const void *input, const void *weight, const void *offset,
                            void *output, int32_t elem, int64_t batch, int64_t channels,
                            int64_t height, int64_t width, int64_t channels_out, int32_t kW,
                            int32_t kH, int32_t dW, int32_t dH, int32_t padW, int32_t padH,
                            int32_t dilationW, int32_t dilationH, int32_t group,
                            int32_t deformable_group, int32_t im2col_step, int32_t device,
                            void *workspace, size_t workspace_bytes, void *stream) {
  if (!offset) return fail(DCN_ERR_ARG, "offset must be non-NULL");
  if (im2col_step <= 0 || (batch > 0 && batch % im2col_step != 0))
    return fail(DCN_ERR_ARG, "batch size must be divisible by im2col_step");
  if (height < kH || width < kW) return fail(DCN_ERR_ARG, "input image is smaller than kernel");
  DcnFwdParams q;
  fill_dense(&q, elem, batch, channels, height, width, channels_out, device);
  q.input = input; q.weight = weight; q.offset = offset; q.output = output;
  q.kh = kH; q.kw = kW; q.stride_h = dH; q.stride_w = dW; q.pad_h = padH; q.pad_w = padW;
  q.dil_h = dilationH; q.dil_w = dilationW; q.groups = group; q.deform_groups = deformable_group;
  return dcn_fwd(&q, workspace, workspace_bytes, stream);
}

int dcn_forward_workspace_bytes(int32_t elem, int32_t modulated, int64_t batch, int64_t channels,
                                int64_t height, int64_t width, int64_t channels_out,
                                int32_t kernel_h, int32_t kernel_w, int32_t stride_h,
                                int32_t stride_w, int32_t pad_h, int32_t pad_w,
                                int32_t dilation_h, int32_t dilation_w, int32_t group,
                                int32_t deformable_group, size_t *bytes) {
  (void)modulated;
  DcnFwdParams q;
  fill_dense(&q, elem, batch, channels, height, width, channels_out, 0);
  q.kh = kernel_h; q.kw = kernel_w; q.stride_h = stride_h; q.stride_w = stride_w;
  q.pad_h = pad_h; q.pad_w = pad_w; q.dil_h = dilation_h; q.dil_w = dilation_w;
  q.groups = group; q.deform_groups = deformable_group;
  return dcn_fwd_workspace_bytes(&q, bytes);
}

}  // extern "C"
