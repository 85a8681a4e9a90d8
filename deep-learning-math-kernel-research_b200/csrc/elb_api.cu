// C-ABI layer (include/euler_b200.h): descriptor validation and algorithm choice (the reference's
// eld_conv_t::setup, src/eld_conv.cpp:59-316), the plan object that replaces `elx_conv_t *xc`,
// first-call weight preparation (setup_workspace, src/elx_conv.hpp:130-145) and execution
// (elx_conv, src/elx_conv.cpp:213-240).  There is deliberately no CPU path: when no CUDA device
// is usable every compute entry point fails with ELB_GENERAL_ERROR.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/euler_b200.h"
#include "elb_common.cuh"
#include "host_prep.hpp"
#include "wino.cuh"
#include "depthwise.cuh"

using namespace elb;

namespace {

thread_local std::string g_last_error;

// Severities and the two environment variables of the reference's logger (src/common/el_def.hpp:17-26,
// src/el_init.cpp:18-27): EULER_LOG_LEVEL = lowest severity that is printed (default: info),
// EULER_VERBOSE=1 = one "euler-perf" line per executed convolution.  Messages below perf go to
// stderr here (the reference prints them to stdout and aborts on errors; this library returns
// codes instead), perf lines go to stdout as in the reference.
enum { LOG_TRACE = 1, LOG_DEBUG = 2, LOG_INFO = 3, LOG_WARN = 4, LOG_ERROR = 5, LOG_PERF = 999 };
struct LogOptions {
  int level = LOG_INFO;
  bool verbose = false;
  LogOptions() {
    const char *v = getenv("EULER_VERBOSE");
    verbose = v && v[0] == '1';
    if (const char *l = getenv("EULER_LOG_LEVEL")) level = atoi(l);
  }
};
const LogOptions &log_options() {
  static const LogOptions o;
  return o;
}
void log_line(int severity, const char *msg) {
  if (severity < log_options().level) return;
  const char *name = severity == LOG_TRACE ? "trace" : severity == LOG_DEBUG ? "debug" : severity == LOG_INFO ? "info"
                   : severity == LOG_WARN ? "warn" : severity == LOG_ERROR ? "error" : "perf";
  fprintf(severity == LOG_PERF ? stdout : stderr, "euler-%s, %s\n", name, msg);
}

int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  // "not implemented on the GPU" is an answer, not a fault: callers probe for it
  log_line(code == ELB_UNIMPLEMENTED ? LOG_DEBUG : LOG_ERROR, buf);
  return code;
}

}  // namespace

namespace elb {
void set_last_error(const char *msg) { g_last_error = msg ? msg : ""; }
}  // namespace elb

namespace {

#define CUDA_TRY(expr)                                                                      \
  do {                                                                                      \
    cudaError_t e__ = (expr);                                                               \
    if (e__ != cudaSuccess)                                                                 \
      return fail(ELB_GENERAL_ERROR, "CUDA error %s at %s:%d (%s)", cudaGetErrorName(e__),  \
                  __FILE__, __LINE__, cudaGetErrorString(e__));                             \
  } while (0)

size_t dt_size(int dt) {
  switch (dt) {
    case ELB_F32: return 4;
    case ELB_F16: return 2;
    case ELB_U8:
    case ELB_S8: return 1;
    default: return 0;
  }
}

bool blocked_act(int f) { return f == ELB_NCHW16C || f == ELB_NCHW8C; }
bool blocked_w(int f) {
  return f == ELB_OIHW16I16O || f == ELB_OIHW8I8O || f == ELB_GOIHW16I16O || f == ELB_GOIHW8I8O;
}

// sizes exactly as src/eld_conv.cpp:99-126 computes them
void compute_sizes(const elb_conv_desc_t &d, elb_conv_info_t &info) {
  const int icg = d.ic / d.g, ocg = d.oc / d.g;
  info.size_input = (uint64_t)d.n * d.ih * d.iw * (blocked_act(d.fmt_input) ? host::alignup(d.ic, V) : d.ic);
  info.size_weights = (uint64_t)d.g * d.kh * d.kw *
                          (blocked_w(d.fmt_weights) ? (uint64_t)host::alignup(icg, V) * host::alignup(ocg, V)
                                                    : (uint64_t)ocg * icg) +
                      4 * V;
  info.size_output = (uint64_t)d.n * d.oh * d.ow * (blocked_act(d.fmt_output) ? host::alignup(d.oc, V) : d.oc);
  info.size_bias = blocked_act(d.fmt_output) ? host::alignup(d.oc, V) : d.oc;
  info.bytes_input = dt_size(d.dt_input) * info.size_input;
  info.bytes_weights = dt_size(d.dt_weights) * info.size_weights;
  info.bytes_output = dt_size(d.dt_output) * info.size_output;
  info.bytes_bias = dt_size(d.dt_bias) * info.size_bias;
}

// CONV_AUTO and Winograd tile choice as in src/eld_conv.cpp:148-159, 231-236
int resolve_algorithm(const elb_conv_desc_t &d, int &algorithm, int &tile) {
  algorithm = d.algorithm;
  tile = d.tile_size;
  if (algorithm == ELB_CONV_AUTO) {
    if (d.kh == 1 && d.kw == 1) algorithm = ELB_CONV_DIRECT_1X1;
    else if (d.ic / d.g >= V && d.kh == 3 && d.kw == 3 && d.dilation_h == 1 && d.dilation_w == 1 &&
             d.stride_h == 1 && d.stride_w == 1 && d.pad_l == 1 && d.pad_r == 1 && d.pad_t == 1 && d.pad_b == 1)
      algorithm = ELB_CONV_WINOGRAD;
    else algorithm = ELB_CONV_DIRECT;
  }
  if (algorithm == ELB_CONV_WINOGRAD && tile == 0) {
    const int t = d.n * ((d.oh + 3) / 4) * ((d.ow + 3) / 4);
    const float mac_per_read = (float)((double)t * host::alignup(d.oc, 16)) * 1.0f / (t + host::alignup(d.oc, V));
    tile = mac_per_read > 25.0f ? 6 : 4;
  }
  return ELB_OK;
}

bool is_int8_user(const elb_conv_desc_t &d) {
  return d.dt_input == ELB_U8 && d.dt_weights == ELB_F32 && d.dt_bias == ELB_F32 &&
         (d.dt_output == ELB_U8 || d.dt_output == ELB_S8 || d.dt_output == ELB_F32);
}
bool is_fp32_user(const elb_conv_desc_t &d) {
  return d.dt_input == ELB_F32 && d.dt_weights == ELB_F32 && d.dt_output == ELB_F32 && d.dt_bias == ELB_F32;
}

}  // namespace

struct elb_conv {
  elb_conv_desc_t d;
  elb_conv_info_t info;
  int device = 0;
  int num_sms = 0;
  bool prepared = false;
  uint64_t launches = 0;
  cudaStream_t stream = nullptr;        // used by elb_conv_execute
  // device workspace
  void *d_wpack = nullptr, *d_wplain = nullptr, *d_scale = nullptr, *d_shift = nullptr;
  void *d_shift_tbl = nullptr, *d_tap_cls = nullptr;     // int8 direct, zero point with padding: per-class shifts
  void *d_tap_tbl = nullptr;                             // int8 direct, BOX mode: I8ConvParams::tap_tbl
  int *d_status = nullptr;
  int *h_status = nullptr;              // pinned: the status word travels back on the stream, behind the kernels
  std::string name = "ioi";             // eld_conv_t::name, printed in the euler-perf line
  bool pending = false;                 // an asynchronous execute has not been waited for yet
  bool pending_d2h = false;
  cudaEvent_t ev_call_done = nullptr, ev_d2h_done = nullptr;   // end of the previous call on `stream` / `s_d2h`
  void *d_acc_dump = nullptr;           // caller memory
  void *d_trace = nullptr;              // caller memory (debug timeline)
  // staging for host-pointer callers
  void *d_in_stage = nullptr, *d_out_stage = nullptr;
  // int8 direct
  I8ConvParams i8{};
  I8UmmaConfig i8cfg{};
  struct TmapEntry { const void *base; int cnt; CUtensorMap m[4]; };
  std::vector<TmapEntry> tmaps;         // tensor maps encoded so far, keyed by (first image address, image count)
  // host-pointer callers: copy streams and events of the chunked, overlapped execute
  cudaStream_t s_h2d = nullptr, s_d2h = nullptr;
  std::vector<cudaEvent_t> ev_in, ev_done;
  // winograd
  WinoPlan wino{};
  // int8 depthwise
  DwPlan dw{};
  // Plain user formats (nchw / nhwc activations, oihw / hwio weights): the kernels work on the
  // blocked formats, `d` / `info` describe that internal problem and `ud` / `uinfo` what the caller
  // passes; activations are converted on the device around every call, weights once.
  elb_conv_desc_t ud{};
  elb_conv_info_t uinfo{};
  bool cvt_in = false, cvt_out = false, cvt_w = false;
  void *d_cvt_in = nullptr, *d_cvt_out = nullptr;

  ~elb_conv() {
    cudaSetDevice(device);
    for (void *p : {d_wpack, d_wplain, d_scale, d_shift, d_shift_tbl, d_tap_cls, d_tap_tbl, (void *)d_status, d_in_stage, d_out_stage,
                    d_cvt_in, d_cvt_out})
      if (p) cudaFree(p);
    wino_release(wino);
    dw_release(dw);
    if (stream) cudaStreamSynchronize(stream);
    if (s_d2h) cudaStreamSynchronize(s_d2h);
    if (h_status) cudaFreeHost(h_status);
    if (ev_call_done) cudaEventDestroy(ev_call_done);
    if (ev_d2h_done) cudaEventDestroy(ev_d2h_done);
    if (stream) cudaStreamDestroy(stream);
    if (s_h2d) cudaStreamDestroy(s_h2d);
    if (s_d2h) cudaStreamDestroy(s_d2h);
    for (cudaEvent_t e : ev_in) cudaEventDestroy(e);
    for (cudaEvent_t e : ev_done) cudaEventDestroy(e);
  }
};

namespace {

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

// format_undef defaults of the reference (src/eld_conv.cpp:77-86)
void resolve_formats(elb_conv_desc_t &d) {
  if (d.fmt_input == ELB_FMT_UNDEF) d.fmt_input = (d.g == 1 && d.ic < V) ? ELB_NCHW : ELB_NCHW16C;
  if (d.fmt_weights == ELB_FMT_UNDEF) d.fmt_weights = d.g == 1 ? ELB_HWIO : ELB_GHWIO;
  if (d.fmt_output == ELB_FMT_UNDEF) d.fmt_output = ELB_NCHW16C;
}

// The problem the kernels see: plain activation / weight formats replaced by the blocked ones.
// ghwio depthwise weights ([g][kh][kw][1][1]) are goihw ([g][1][1][kh][kw]) byte for byte.
elb_conv_desc_t internal_desc(const elb_conv_desc_t &u, bool &cvt_in, bool &cvt_out, bool &cvt_w) {
  elb_conv_desc_t d = u;
  const bool depthwise = u.g > 1 && u.g == u.ic && u.g == u.oc;
  cvt_in = u.fmt_input == ELB_NCHW || u.fmt_input == ELB_NHWC;
  cvt_out = u.fmt_output == ELB_NCHW || u.fmt_output == ELB_NHWC;
  cvt_w = !depthwise && (u.fmt_weights == ELB_OIHW || u.fmt_weights == ELB_HWIO);
  if (cvt_in) d.fmt_input = ELB_NCHW16C;
  if (cvt_out) d.fmt_output = ELB_NCHW16C;
  if (cvt_w) d.fmt_weights = ELB_OIHW16I16O;
  if (depthwise && u.fmt_weights == ELB_GHWIO) d.fmt_weights = ELB_GOIHW;
  return d;
}

int validate_common(const elb_conv_desc_t &d) {
  if (d.n <= 0 || d.g <= 0 || d.ic <= 0 || d.oc <= 0 || d.ih <= 0 || d.iw <= 0 || d.oh <= 0 || d.ow <= 0 ||
      d.kh <= 0 || d.kw <= 0 || d.stride_h <= 0 || d.stride_w <= 0)
    return fail(ELB_GENERAL_ERROR, "invalid dimensions");
  if (d.ic % d.g || d.oc % d.g) return fail(ELB_GENERAL_ERROR, "ic/oc not divisible by groups");
  if (d.prop_kind != ELB_FORWARD_INFERENCE)
    return fail(ELB_GENERAL_ERROR, "Propagation kind error");     // src/eld_conv.cpp:143-146
  return ELB_OK;
}

// Choose the kernel for a resolved algorithm; ELB_KERNEL_NONE = not implemented on this library.
int choose_kernel(const elb_conv_desc_t &d, int algorithm, int tile, const char **why) {
  *why = "";
  const bool blocked = d.fmt_input == ELB_NCHW16C && d.fmt_output == ELB_NCHW16C;
  if (!blocked) { *why = "only nChw16c activations are implemented"; return ELB_KERNEL_NONE; }
  if (d.dilation_h != 1 || d.dilation_w != 1) { *why = "dilation"; return ELB_KERNEL_NONE; }
  if (d.stride_h != d.stride_w) { *why = "anisotropic stride"; return ELB_KERNEL_NONE; }
  const bool depthwise = d.g > 1 && d.g == d.ic && d.g == d.oc;
  if (d.g != 1 && !depthwise) { *why = "grouped convolution"; return ELB_KERNEL_NONE; }
  if (algorithm == ELB_CONV_WINOGRAD) {
    if (d.stride_h != 1 || d.kh != 3 || d.kw != 3 || d.g != 1) { *why = "Winograd needs 3x3 stride 1"; return ELB_KERNEL_NONE; }
    if (tile != 6 && tile != 4) { *why = "only tile_size 6, F(4x4,3x3), and 4, F(2x2,3x3), are implemented"; return ELB_KERNEL_NONE; }
    if (d.fmt_weights != ELB_OIHW16I16O) { *why = "weights must be OIhw16i16o"; return ELB_KERNEL_NONE; }
    if (is_fp32_user(d)) return ELB_KERNEL_WINO_F32_UMMA;
    if (is_int8_user(d)) return ELB_KERNEL_WINO_I8_UMMA;
    *why = "unsupported data types for Winograd";
    return ELB_KERNEL_NONE;
  }
  if (algorithm == ELB_CONV_DIRECT_1X1 || algorithm == ELB_CONV_DIRECT) {
    if (algorithm == ELB_CONV_DIRECT_1X1 && (d.kh != 1 || d.kw != 1)) { *why = "1x1 algorithm on a non-1x1 filter"; return ELB_KERNEL_NONE; }
    if (is_fp32_user(d)) {
      if (d.g != 1) { *why = "fp32 grouped / depthwise convolution"; return ELB_KERNEL_NONE; }
      if (d.fmt_weights != ELB_OIHW16I16O) { *why = "weights must be OIhw16i16o"; return ELB_KERNEL_NONE; }
      return ELB_KERNEL_F32_DIRECT_UMMA;
    }
    if (!is_int8_user(d)) { *why = "direct convolution is implemented for fp32 and for u8 inputs"; return ELB_KERNEL_NONE; }
    if (depthwise) {
      if (d.kh != 3 || d.kw != 3 || d.dt_output == ELB_F32) { *why = "depthwise needs 3x3 and u8/s8 output"; return ELB_KERNEL_NONE; }
      if (d.fmt_weights != ELB_GOIHW) { *why = "depthwise weights must be goihw"; return ELB_KERNEL_NONE; }
      return ELB_KERNEL_I8_DEPTHWISE;
    }
    if (d.fmt_weights != ELB_OIHW16I16O) { *why = "weights must be OIhw16i16o"; return ELB_KERNEL_NONE; }
    if (d.stride_h > 2) return ELB_KERNEL_I8_SIMT;
    if (host::alignup(d.oc, V) > 2048) return ELB_KERNEL_I8_SIMT;
    if (d.ih < d.stride_h || d.iw < d.stride_w) return ELB_KERNEL_I8_SIMT;
    const char *force = getenv("ELB_FORCE_SIMT");
    if (force && atoi(force) > 0) return ELB_KERNEL_I8_SIMT;
    const bool flat = d.kh == 1 && d.kw == 1 && d.stride_h == 1 && d.pad_t == 0 && d.pad_l == 0 &&
                      d.oh == d.ih && d.ow == d.iw;
    return flat ? ELB_KERNEL_I8_GEMM_UMMA : ELB_KERNEL_I8_CONV_UMMA;
  }
  *why = "algorithm not implemented";
  return ELB_KERNEL_NONE;
}

// BOX-mode tile: BH x BW output pixels with BH*BW = 128, chosen to waste the fewest MMA rows.
void choose_box(int oh, int ow, int &BW, int &BH) {
  long best = -1;
  for (int bw = 1; bw <= 128; bw *= 2) {
    const int bh = 128 / bw;
    const long cost = (long)((ow + bw - 1) / bw) * ((oh + bh - 1) / bh);
    // prefer wide boxes on ties (longer contiguous runs per TMA row)
    if (best < 0 || cost < best || (cost == best && bw > BW && bw <= 64)) { best = cost; BW = bw; BH = bh; }
  }
}

int encode_i8_tmaps(elb_conv &pl, const void *input, int cnt, CUtensorMap *out) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return fail(ELB_GENERAL_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
  // IH/IW are the plan's view of the input plane (a 1x1 stride-1 convolution sees it as one row)
  const int s = pl.i8.stride, CB = pl.i8.CB, IH = pl.i8.IH, IW = pl.i8.IW;
  const int pv = tune_env("ELB_I8_L2PROMO", 128);                  // measured without effect on these kernels
  const CUtensorMapL2promotion promo = pv == 256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : pv == 64 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                     : pv == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE : CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
  if (pl.i8.merged_rows) {
    // stride 1: a row of the box is BW*16 contiguous bytes; describe it as 2*BW 8-byte elements so
    // the copy engine moves whole rows (4-D map: x in 8-byte units, h, channel block, image)
    cuuint64_t dims[4] = {(cuuint64_t)IW * 2, (cuuint64_t)IH, (cuuint64_t)CB, (cuuint64_t)cnt};
    cuuint64_t strides[3] = {(cuuint64_t)IW * 16, (cuuint64_t)IH * IW * 16, (cuuint64_t)CB * IH * IW * 16};
    cuuint32_t box[4] = {(cuuint32_t)pl.i8.BW * 2, (cuuint32_t)pl.i8.BH, (cuuint32_t)pl.i8.box_c, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(&out[0], CU_TENSOR_MAP_DATA_TYPE_UINT64, 4, const_cast<void *>(input), dims, strides, box,
                     estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                     promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ELB_GENERAL_ERROR, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return ELB_OK;
  }
  for (int ph = 0; ph < s; ++ph)
    for (int pw = 0; pw < s; ++pw) {
      const cuuint64_t Hp = (IH - ph + s - 1) / s, Wp = (IW - pw + s - 1) / s;
      cuuint64_t dims[5] = {16, Wp, Hp, (cuuint64_t)CB, (cuuint64_t)cnt};
      cuuint64_t strides[4] = {(cuuint64_t)s * 16, (cuuint64_t)s * IW * 16, (cuuint64_t)IH * IW * 16,
                               (cuuint64_t)CB * IH * IW * 16};
      cuuint32_t box[5] = {16, (cuuint32_t)pl.i8.BW, (cuuint32_t)pl.i8.BH, (cuuint32_t)pl.i8.box_c, 1};
      cuuint32_t estr[5] = {1, 1, 1, 1, 1};
      void *base = (void *)((const uint8_t *)input + ((size_t)ph * IW + pw) * 16);
      CUresult r = enc(&out[ph * s + pw], CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, base, dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, promo,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) return fail(ELB_GENERAL_ERROR, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    }
  return ELB_OK;
}

// ------------------------------------------------------------------------------ int8 direct
int setup_i8_direct(elb_conv &pl) {
  const elb_conv_desc_t &d = pl.d;
  I8ConvParams &p = pl.i8;
  if (d.sampling_kind != ELB_CALIBRATED)          // src/elx_int8_conv_direct.cpp:44-46, _1x1.cpp:225-226
    return fail(ELB_UNIMPLEMENTED, "int8 direct: non-calibrated sampling_kind not supported");
  p.N = d.n; p.IH = d.ih; p.IW = d.iw; p.OH = d.oh; p.OW = d.ow; p.KH = d.kh; p.KW = d.kw;
  p.stride = d.stride_h; p.pad_t = d.pad_t; p.pad_l = d.pad_l;
  p.CB = host::alignup(d.ic, V) / V;
  p.OCB = host::alignup(d.oc, V) / V;
  p.taps = d.kh * d.kw;
  p.HW = d.oh * d.ow;
  p.M = d.n * p.HW;
  p.rq.out_type = d.dt_output == ELB_F32 ? OUT_F32 : d.dt_output == ELB_U8 ? OUT_U8 : OUT_S8;
  p.rq.relu = d.with_relu;
  p.rq.relu_lo = d.relu_lower;
  p.rq.relu_hi = d.relu_upper;
  // with_ip_sum: honoured by the 1x1 algorithm (src/kernel/elk_u8s8_gemm.hxx:221-237).  The KxK
  // algorithm of the reference ignores the flag (src/elx_int8_conv_direct.cpp:121); this library
  // applies the 1x1 semantics there as well (f += prev * sum_scale); with the flag off the two agree bit for bit.
  p.rq.with_sum = d.with_ip_sum && d.dt_output != ELB_F32;
  p.rq.sum_scale = d.sum_scale;
  if (pl.info.kernel == ELB_KERNEL_I8_GEMM_UMMA || pl.info.kernel == ELB_KERNEL_I8_CONV_UMMA) {
    // A 1x1 stride-1 convolution has no halo, so its image plane is viewed as ONE row of oh*ow
    // pixels: the tile becomes 128 consecutive pixels of one image and a whole K stage of A is a
    // single tiled TMA copy.  (ELB_I8_FLAT=1 selects the variant that tiles across images with
    // per-run bulk copies instead; it issues many more, smaller copies.)
    int mode = I8_MODE_BOX;
    if (pl.info.kernel == ELB_KERNEL_I8_GEMM_UMMA) {
      if (tune_env("ELB_I8_FLAT", 0) > 0) mode = I8_MODE_FLAT;
      else { p.IH = 1; p.IW = d.ih * d.iw; p.OH = 1; p.OW = d.oh * d.ow; }
    }
    pl.i8cfg = i8_umma_config(p.OCB, p.CB, p.taps, mode);
    p.n_tiles = (p.OCB * V + pl.i8cfg.BN - 1) / pl.i8cfg.BN;
    p.CBG = (p.CB + pl.i8cfg.KC - 1) / pl.i8cfg.KC;
    p.Q = p.taps * p.CB;
    p.k_stages = (p.Q + pl.i8cfg.KC - 1) / pl.i8cfg.KC;
    // channel blocks one tiled copy fetches: the largest power of two that divides CB, at most KC
    p.box_c = 1;
    while (p.box_c * 2 <= pl.i8cfg.KC && p.CB % (p.box_c * 2) == 0) p.box_c *= 2;
    {
      const int v = tune_env("ELB_I8_BOXC", p.box_c);
      if (v >= 1 && v <= p.box_c && p.box_c % v == 0) p.box_c = v;
    }
    if (mode == I8_MODE_FLAT) {
      p.m_tiles = (p.M + 127) / 128;
    } else {
      p.merged_rows = (p.stride == 1 && tune_env("ELB_I8_NO_MERGED_ROWS", 0) <= 0) ? 1 : 0;
      choose_box(p.OH, p.OW, p.BW, p.BH);
      p.tiles_w = (p.OW + p.BW - 1) / p.BW;
      p.tiles_h = (p.OH + p.BH - 1) / p.BH;
      p.m_tiles = d.n * p.tiles_w * p.tiles_h;
    }
    {
      p.rotate_k = tune_env("ELB_I8_NO_ROTATE_K", 0) > 0 ? 0 : 1;
      // Producer warps and stages per pass.  A copy instruction occupies its warp for hundreds of
      // cycles, so the issue rate is set by how many warps issue and how many stages each serves per
      // pass; one stage per pass refills a slot as soon as it is free (a pass of two waits for both).
      // Measured on B200: short launches are fastest with 2 warps x 1 stage (1x1 benchmark layer
      // 13.2 -> 12.7 us, 3x3 stride 2 36.2 -> 34.5 us); long K loops (16 stages and more) of 128 or
      // 256 output channels with 4 warps x 1 stage (VGG conv4_2 0.091 -> 0.080 ms, conv3_2 0.081 ->
      // 0.074 ms); long launches of short K loops with 2 warps x 2 stages.  warps x stages must not
      // exceed the ring depth: a warp further ahead could not tell its slot's phase by parity.
      const bool short_launch = (long long)p.m_tiles * p.n_tiles <= 4LL * pl.num_sms;
      p.nprod = (pl.i8cfg.BN >= 128 && p.k_stages >= 16) ? 4 : 2;
      p.spp = (p.nprod == 4 || short_launch) ? 1 : 2;
      { const int v = tune_env("ELB_I8_NPROD", p.nprod); if (v == 1 || v == 2 || v == 4) p.nprod = v; }
      p.spp = tune_env("ELB_I8_SPP", p.spp) == 1 ? 1 : 2;
      while (p.nprod * p.spp > pl.i8cfg.STAGES) { if (p.spp > 1) p.spp = 1; else p.nprod /= 2; }
    }
    // Pairs of SMs (int8_conv2.cu: each CTA fetches half of the weight panel) are opt-in with
    // ELB_I8_CTA2=1: measured on B200 they are slower than the single-CTA kernel (1x1 benchmark layer
    // 16.3 vs 13.7 us, 3x3 stride 2 42.9 vs 37.6 us): the kernel is bound by the rate at which copies
    // can be ISSUED, which pairing does not change, and it pays a cluster start-up.
    {
      const char *on2 = getenv("ELB_I8_CTA2");
      const bool zp_classes = d.input_z != 0.0f && (d.pad_t || d.pad_l || d.pad_b || d.pad_r);   // (single CTAs only)
      pl.i8cfg.cta2 = (mode == I8_MODE_BOX && p.m_tiles >= 4 && on2 && atoi(on2) > 0 && !zp_classes && pl.i8cfg.KC == 8) ? 1 : 0;
    }
    if (pl.i8cfg.cta2) CUDA_TRY(init_i8_umma2(pl.i8cfg, pl.num_sms));
    CUDA_TRY(init_i8_umma(pl.i8cfg));
    // BOX mode: the copy table (where each tiled copy of each K stage reads)
    p.tap_tbl = nullptr; p.tap_n = 0; p.ncopy = pl.i8cfg.KC / p.box_c;
    if (mode == I8_MODE_BOX && !pl.i8cfg.cta2 && p.k_stages * p.ncopy <= I8_TAP_TBL_MAX && p.CB < 4096 &&
        p.KH - p.pad_t <= 7 && p.KW - p.pad_l <= 7 && p.pad_t <= 8 && p.pad_l <= 8) {
      std::vector<uint32_t> tbl(static_cast<size_t>(p.k_stages) * p.ncopy, 0u);
      auto fdiv = [](int e, int s) { return e >= 0 ? e / s : -((-e + s - 1) / s); };
      for (int ks = 0; ks < p.k_stages; ++ks)
        for (int c = 0; c < p.ncopy; ++c) {
          const int q = ks * pl.i8cfg.KC + c * p.box_c;
          if (q >= p.Q) continue;
          const int tap = q / p.CB, cb0 = q - tap * p.CB;
          // input row = stride*(oh + dh) + parity_h with dh = floor((kh - pad)/stride)
          const int kh = tap / p.KW, kw = tap - kh * p.KW;
          const int eh = kh - p.pad_t, ew = kw - p.pad_l;
          const int dh = fdiv(eh, p.stride), dw = fdiv(ew, p.stride);
          const int map = (eh - dh * p.stride) * p.stride + (ew - dw * p.stride);
          tbl[static_cast<size_t>(ks) * p.ncopy + c] = static_cast<uint32_t>(cb0) | static_cast<uint32_t>(dh + 8) << 12 |
                                                      static_cast<uint32_t>(dw + 8) << 16 | static_cast<uint32_t>(map) << 20;
        }
      CUDA_TRY(cudaMalloc(&pl.d_tap_tbl, tbl.size() * 4));
      CUDA_TRY(cudaMemcpy(pl.d_tap_tbl, tbl.data(), tbl.size() * 4, cudaMemcpyHostToDevice));
      p.tap_tbl = static_cast<const uint32_t *>(pl.d_tap_tbl);
      p.tap_n = static_cast<int>(tbl.size());
    }
  }
  pl.info.launches_per_call = 1;
  return ELB_OK;
}

int prepare_i8_direct(elb_conv &pl, const void *weights, const void *bias) {
  const elb_conv_desc_t &d = pl.d;
  std::vector<float> hw(pl.info.size_weights), hb(pl.info.size_bias, 0.0f);
  CUDA_TRY(cudaMemcpy(hw.data(), weights, pl.info.size_weights * 4, cudaMemcpyDefault));
  if (d.with_bias) {
    if (!bias) return fail(ELB_GENERAL_ERROR, "bias is null but with_bias is set");
    CUDA_TRY(cudaMemcpy(hb.data(), bias, pl.info.size_bias * 4, cudaMemcpyDefault));
  }
  host::I8Weights wq = host::quantize_weights_i8(hw.data(), d.oc, d.ic, d.kh, d.kw);
  std::vector<float> scale, shift;
  host::fold_constants_i8(wq, hb.data(), d.with_bias != 0, d.dt_output == ELB_F32, d.input_scale, d.input_z,
                          d.output_scale, d.output_z, pl.i8.rq.with_sum != 0, d.sum_scale, d.sum_z, scale, shift);
  CUDA_TRY(cudaMalloc(&pl.d_scale, scale.size() * 4));
  CUDA_TRY(cudaMalloc(&pl.d_shift, shift.size() * 4));
  CUDA_TRY(cudaMemcpy(pl.d_scale, scale.data(), scale.size() * 4, cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMemcpy(pl.d_shift, shift.data(), shift.size() * 4, cudaMemcpyHostToDevice));
  pl.info.workspace_bytes += scale.size() * 8;
  if (d.input_z != 0.0f && (d.pad_t || d.pad_l || d.pad_b || d.pad_r)) {
    // one shift vector per (valid kh range, valid kw range): src/elx_int8_conv_direct.cpp:227-423
    const host::TapClasses th = host::tap_classes(d.oh, d.ih, d.kh, d.pad_t, d.stride_h);
    const host::TapClasses tw = host::tap_classes(d.ow, d.iw, d.kw, d.pad_l, d.stride_w);
    const int nh = (int)th.ranges.size(), nw = (int)tw.ranges.size(), OCP = wq.OCP;
    std::vector<float> tbl((size_t)nh * nw * OCP), sc_c, sh_c;
    std::vector<int32_t> qs(OCP);
    for (int ch = 0; ch < nh; ++ch)
      for (int cw = 0; cw < nw; ++cw) {
        for (int o = 0; o < OCP; ++o) {
          int32_t sum = 0;
          for (int a = th.ranges[ch].first; a <= th.ranges[ch].second; ++a)
            for (int b = tw.ranges[cw].first; b <= tw.ranges[cw].second; ++b) sum += wq.qsum_tap[(size_t)o * wq.taps + a * d.kw + b];
          qs[o] = sum;
        }
        host::fold_constants_i8(wq, hb.data(), d.with_bias != 0, d.dt_output == ELB_F32, d.input_scale, d.input_z,
                                d.output_scale, d.output_z, pl.i8.rq.with_sum != 0, d.sum_scale, d.sum_z, sc_c, sh_c, qs.data());
        std::copy(sh_c.begin(), sh_c.end(), tbl.begin() + ((size_t)ch * nw + cw) * OCP);
      }
    std::vector<int> cls(th.cls);
    cls.insert(cls.end(), tw.cls.begin(), tw.cls.end());
    CUDA_TRY(cudaMalloc(&pl.d_shift_tbl, tbl.size() * 4));
    CUDA_TRY(cudaMemcpy(pl.d_shift_tbl, tbl.data(), tbl.size() * 4, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMalloc(&pl.d_tap_cls, cls.size() * 4));
    CUDA_TRY(cudaMemcpy(pl.d_tap_cls, cls.data(), cls.size() * 4, cudaMemcpyHostToDevice));
    pl.info.workspace_bytes += tbl.size() * 4 + cls.size() * 4;
    pl.i8.shift_tbl = (const float *)pl.d_shift_tbl;
    pl.i8.hclass = (const int *)pl.d_tap_cls;
    pl.i8.wclass = pl.i8.hclass + d.oh;
    pl.i8.zp_nw = nw;
    // pixels that see every tap use the vector in `shift` (kept in shared memory by the tcgen05 kernel);
    // when no pixel does (tiny images), -1 sends every pixel to the table
    pl.i8.zp_full = (th.full >= 0 && tw.full >= 0) ? th.full * nw + tw.full : -1;
  }
  if (pl.info.kernel == ELB_KERNEL_I8_SIMT) {
    CUDA_TRY(cudaMalloc(&pl.d_wplain, wq.q.size()));
    CUDA_TRY(cudaMemcpy(pl.d_wplain, wq.q.data(), wq.q.size(), cudaMemcpyHostToDevice));
    pl.info.workspace_bytes += wq.q.size();
  } else {
    int n_tiles, CBG, k_stages;
    std::vector<int8_t> pk = host::pack_b_i8(wq, pl.i8cfg.BN, pl.i8cfg.KC, n_tiles, CBG, k_stages,
                                             pl.i8cfg.cta2 ? 2 : 1);
    if (n_tiles != pl.i8.n_tiles || CBG != pl.i8.CBG || k_stages != pl.i8.k_stages)
      return fail(ELB_GENERAL_ERROR, "internal: weight packing geometry mismatch");
    CUDA_TRY(cudaMalloc(&pl.d_wpack, pk.size()));
    CUDA_TRY(cudaMemcpy(pl.d_wpack, pk.data(), pk.size(), cudaMemcpyHostToDevice));
    pl.info.workspace_bytes += pk.size();
  }
  pl.i8.wpack = (const int8_t *)pl.d_wpack;
  pl.i8.wplain = (const int8_t *)pl.d_wplain;
  pl.i8.scale = (const float *)pl.d_scale;
  pl.i8.shift = (const float *)pl.d_shift;
  return ELB_OK;
}

// Images [n0, n0 + cnt) of the batch; `out` / `in` address the FULL tensors.
int run_i8_direct(elb_conv &pl, void *out, const void *in, int n0, int cnt, cudaStream_t s) {
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(ELB_GENERAL_ERROR, "input/output tensors must be 16-byte aligned");
  I8ConvParams p = pl.i8;
  const size_t in_img = pl.info.bytes_input / pl.d.n, out_img = pl.info.bytes_output / pl.d.n;
  p.in = (const uint8_t *)in + (size_t)n0 * in_img;
  p.out = (uint8_t *)out + (size_t)n0 * out_img;
  p.acc_dump = pl.d_acc_dump ? (int32_t *)pl.d_acc_dump + (size_t)n0 * p.OCB * V * pl.d.oh * pl.d.ow : nullptr;
  p.status = pl.d_status;
  p.trace = (long long *)pl.d_trace;
  p.N = cnt;
  p.M = cnt * p.HW;
  cudaError_t e;
  if (pl.info.kernel == ELB_KERNEL_I8_SIMT) {
    e = launch_i8_simt(p, s);
  } else {
    if (pl.i8cfg.mode == I8_MODE_FLAT) {
      p.m_tiles = (p.M + 127) / 128;
    } else {
      p.m_tiles = cnt * p.tiles_w * p.tiles_h;
      const elb_conv::TmapEntry *hit = nullptr;
      for (const auto &t : pl.tmaps)
        if (t.base == p.in && t.cnt == cnt) { hit = &t; break; }
      if (!hit) {
        elb_conv::TmapEntry t{};
        t.base = p.in;
        t.cnt = cnt;
        int rc = encode_i8_tmaps(pl, p.in, cnt, t.m);
        if (rc != ELB_OK) return rc;
        if (pl.tmaps.size() >= 64) pl.tmaps.erase(pl.tmaps.begin());
        pl.tmaps.push_back(t);
        hit = &pl.tmaps.back();
      }
      for (int i = 0; i < 4; ++i) p.tmap[i] = hit->m[i];
    }
    // (a sub-range of fewer than two pixel tiles still runs on pairs: the weights are packed for them)
    e = pl.i8cfg.cta2 ? launch_i8_umma2(p, pl.i8cfg, pl.num_sms, s) : launch_i8_umma(p, pl.i8cfg, pl.num_sms, s);
  }
  pl.launches += 1;
  if (e != cudaSuccess) return fail(ELB_GENERAL_ERROR, "kernel launch failed: %s", cudaGetErrorString(e));
  return ELB_OK;
}

// The status word of the kernels follows them on the stream into pinned host memory, so the call's
// one synchronisation also brings back the verdict (no separate blocking copy).
int fetch_status_async(elb_conv &pl, cudaStream_t s) {
  CUDA_TRY(cudaMemcpyAsync(pl.h_status, pl.d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
  return ELB_OK;
}
int check_status(elb_conv &pl) {
  const int st = *pl.h_status;
  if (st != 0) {
    *pl.h_status = 0;
    cudaMemset(pl.d_status, 0, sizeof(int));
    return fail(ELB_GENERAL_ERROR, "device kernel gave up waiting (status %d)", st);
  }
  return ELB_OK;
}

const char *fmt_name(int f) {
  static const char *n[] = {"format-unknown", "nchw", "nhwc", "nChw16c", "nChw8c", "oihw", "hwio", "OIhw16i16o",
                            "OIhw8i8o", "goihw", "ghwio", "gOIhw16i16o", "gOIhw8i8o"};
  return f >= 1 && f <= 12 ? n[f] : n[0];
}
const char *dt_name(int t) {
  static const char *n[] = {"datatype-unknown", "f32", "f16", "u8", "s8", "s32"};
  return t >= 1 && t <= 5 ? n[t] : n[0];
}
const char *algo_name(int a) {
  return a == ELB_CONV_DIRECT_1X1 ? "direct_conv_1x1" : a == ELB_CONV_DIRECT ? "direct_conv"
       : a == ELB_CONV_DIRECT_VMG ? "direct_conv_vmg" : a == ELB_CONV_WINOGRAD ? "winograd_conv"
       : a == ELB_DECONV_DIRECT ? "deconv" : "algorithm-unknown";
}
// The line execute_verbose prints (src/elx_conv.cpp:190-211), same fields in the same order.
void perf_line(const elb_conv &pl, double ms) {
  char buf[512];
  const elb_conv_desc_t &u = pl.ud;
  snprintf(buf, sizeof(buf), "%s,ih:%d;oh:%d;ic:%d;oc:%d,%s;%x,src:%s;wei:%s;dst:%s,src:%s;wei:%s;dst:%s;b:%s, %lf",
           pl.name.c_str(), u.ih, u.oh, u.ic, u.oc, algo_name(pl.info.algorithm), u.execution_mode, fmt_name(u.fmt_input),
           fmt_name(u.fmt_weights), fmt_name(u.fmt_output), dt_name(u.dt_input), dt_name(u.dt_weights),
           dt_name(u.dt_output), dt_name(u.dt_bias), ms);
  log_line(LOG_PERF, buf);
}

bool is_device_ptr(const void *p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

int do_prepare_inner(elb_conv &pl, const void *weights, const void *bias) {
  if (pl.prepared) return ELB_OK;
  if (!weights) return fail(ELB_GENERAL_ERROR, "weights are null");
  int rc;
  switch (pl.info.kernel) {
    case ELB_KERNEL_I8_GEMM_UMMA:
    case ELB_KERNEL_I8_CONV_UMMA:
    case ELB_KERNEL_I8_SIMT: rc = prepare_i8_direct(pl, weights, bias); break;
    case ELB_KERNEL_WINO_F32_UMMA:
    case ELB_KERNEL_F32_DIRECT_UMMA:
    case ELB_KERNEL_F32_SMALL_IC:
    case ELB_KERNEL_WINO_I8_UMMA: {
      std::string err;
      rc = wino_prepare(pl.wino, pl.d, pl.info, weights, bias, err);
      if (rc != ELB_OK) fail(rc, "%s", err.c_str());
      break;
    }
    case ELB_KERNEL_I8_DEPTHWISE: {
      std::string err;
      rc = dw_prepare(pl.dw, pl.d, pl.info, weights, bias, err);
      if (rc != ELB_OK) fail(rc, "%s", err.c_str());
      break;
    }
    default: rc = fail(ELB_UNIMPLEMENTED, "no kernel");
  }
  if (rc == ELB_OK) pl.prepared = true;
  return rc;
}

// Weights / bias in the caller's formats -> what the kernels' one-time preparation reads: plain
// weights (oihw, hwio) are converted to OIhw16i16o on the device, a bias of oc elements (plain
// output formats, src/eld_conv.cpp:112-114) is zero-padded to a multiple of 16.
int do_prepare(elb_conv &pl, const void *weights, const void *bias) {
  if (pl.prepared) return ELB_OK;
  if (!weights) return fail(ELB_GENERAL_ERROR, "weights are null");
  const bool pad_bias = pl.d.with_bias && bias && pl.uinfo.size_bias != pl.info.size_bias;
  if (!pl.cvt_w && !pad_bias) {
    const int rc0 = do_prepare_inner(pl, weights, bias);
    // The preparation copies from pageable host memory, and such a cudaMemcpy may return while its
    // DMA into device memory is still running; the plan's streams are non-blocking, so nothing else
    // would order the first kernel behind it.
    if (cudaDeviceSynchronize() != cudaSuccess && rc0 == ELB_OK)
      return fail(ELB_GENERAL_ERROR, "preparation failed: %s", cudaGetErrorString(cudaGetLastError()));
    return rc0;
  }
  void *w_src = nullptr, *w_blk = nullptr, *b_pad = nullptr;
  int rc = ELB_OK;
  auto cleanup = [&]() { for (void *q : {w_src, w_blk, b_pad}) if (q) cudaFree(q); };
  if (pl.cvt_w) {
    bool sup = false;
    if (cudaMalloc(&w_src, pl.uinfo.bytes_weights) != cudaSuccess || cudaMalloc(&w_blk, pl.info.bytes_weights) != cudaSuccess ||
        cudaMemcpy(w_src, weights, pl.uinfo.bytes_weights, cudaMemcpyDefault) != cudaSuccess ||
        cudaMemset(w_blk, 0, pl.info.bytes_weights) != cudaSuccess ||
        launch_reorder(w_blk, ELB_OIHW16I16O, w_src, pl.ud.fmt_weights, 1, pl.d.oc, pl.d.ic, pl.d.kh, pl.d.kw, 4, nullptr, sup) != cudaSuccess ||
        !sup || cudaDeviceSynchronize() != cudaSuccess) {
      cleanup();
      return fail(ELB_GENERAL_ERROR, "weight format conversion failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
  }
  if (pad_bias) {
    if (cudaMalloc(&b_pad, pl.info.bytes_bias) != cudaSuccess || cudaMemset(b_pad, 0, pl.info.bytes_bias) != cudaSuccess ||
        cudaMemcpy(b_pad, bias, pl.uinfo.bytes_bias, cudaMemcpyDefault) != cudaSuccess) {
      cleanup();
      return fail(ELB_GENERAL_ERROR, "bias padding failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
  }
  rc = do_prepare_inner(pl, pl.cvt_w ? w_blk : weights, pad_bias ? b_pad : bias);
  cudaDeviceSynchronize();
  cleanup();
  return rc;
}

// Enqueue images [n0, n0 + cnt) of the batch on stream s; `out` / `in` address the full tensors.
int do_enqueue_range_inner(elb_conv &pl, void *out, const void *in, int n0, int cnt, cudaStream_t s) {
  switch (pl.info.kernel) {
    case ELB_KERNEL_I8_GEMM_UMMA:
    case ELB_KERNEL_I8_CONV_UMMA:
    case ELB_KERNEL_I8_SIMT: return run_i8_direct(pl, out, in, n0, cnt, s);
    case ELB_KERNEL_I8_DEPTHWISE: {
      std::string err;
      int nl = 0;
      int rc = dw_run(pl.dw, out, in, pl.d_acc_dump, n0, cnt, s, nl, err);
      pl.launches += nl;
      if (rc != ELB_OK) return fail(rc, "%s", err.c_str());
      return rc;
    }
    case ELB_KERNEL_WINO_F32_UMMA:
    case ELB_KERNEL_F32_DIRECT_UMMA:
    case ELB_KERNEL_F32_SMALL_IC:
    case ELB_KERNEL_WINO_I8_UMMA: {
      std::string err;
      int nl = 0;
      pl.wino.trace = pl.d_trace;
      int rc = wino_run(pl.wino, out, in, pl.d_acc_dump, pl.d_status, pl.num_sms, n0, cnt, s, nl, err);
      pl.launches += nl;
      if (rc != ELB_OK) return fail(rc, "%s", err.c_str());
      return rc;
    }
    default: return fail(ELB_UNIMPLEMENTED, "no kernel");
  }
}

// The same in the caller's formats: plain activations (nchw / nhwc) are converted to nChw16c
// before the kernels and the result back after them, image range by image range, on the same
// stream (the residual of an in-place sum travels with the output tensor).
int do_enqueue_range(elb_conv &pl, void *out, const void *in, int n0, int cnt, cudaStream_t s) {
  if (!pl.cvt_in && !pl.cvt_out) return do_enqueue_range_inner(pl, out, in, n0, cnt, s);
  const elb_conv_desc_t &d = pl.d;
  const int N = d.n, ebi = (int)dt_size(d.dt_input), ebo = (int)dt_size(d.dt_output);
  const size_t u_in = pl.uinfo.bytes_input / N, b_in = pl.info.bytes_input / N;
  const size_t u_out = pl.uinfo.bytes_output / N, b_out = pl.info.bytes_output / N;
  bool sup = false;
  cudaError_t e = cudaSuccess;
  if (pl.cvt_in) {
    e = launch_reorder((uint8_t *)pl.d_cvt_in + n0 * b_in, ELB_NCHW16C, (const uint8_t *)in + n0 * u_in, pl.ud.fmt_input, 1, cnt,
                       d.ic, d.ih, d.iw, ebi, s, sup);
    ++pl.launches;
  }
  if (e == cudaSuccess && pl.cvt_out && d.with_ip_sum) {
    e = launch_reorder((uint8_t *)pl.d_cvt_out + n0 * b_out, ELB_NCHW16C, (const uint8_t *)out + n0 * u_out, pl.ud.fmt_output, 1,
                       cnt, d.oc, d.oh, d.ow, ebo, s, sup);
    ++pl.launches;
  }
  if (e != cudaSuccess) return fail(ELB_GENERAL_ERROR, "format conversion launch failed: %s", cudaGetErrorString(e));
  int rc = do_enqueue_range_inner(pl, pl.cvt_out ? pl.d_cvt_out : out, pl.cvt_in ? pl.d_cvt_in : in, n0, cnt, s);
  if (rc != ELB_OK) return rc;
  if (pl.cvt_out) {
    e = launch_reorder((uint8_t *)out + n0 * u_out, pl.ud.fmt_output, (const uint8_t *)pl.d_cvt_out + n0 * b_out, ELB_NCHW16C, 1, cnt,
                       d.oc, d.oh, d.ow, ebo, s, sup);
    ++pl.launches;
    if (e != cudaSuccess) return fail(ELB_GENERAL_ERROR, "format conversion launch failed: %s", cudaGetErrorString(e));
  }
  return ELB_OK;
}

int do_enqueue(elb_conv &pl, void *out, const void *in, cudaStream_t s) {
  return do_enqueue_range(pl, out, in, 0, pl.d.n, s);
}

// Wait for an asynchronous execute that has not been waited for (returns at once when there is none).
int wait_pending(elb_conv &pl) {
  if (!pl.pending) return ELB_OK;
  pl.pending = false;
  CUDA_TRY(cudaStreamSynchronize(pl.stream));
  if (pl.pending_d2h) {
    pl.pending_d2h = false;
    CUDA_TRY(cudaStreamSynchronize(pl.s_d2h));
  }
  return check_status(pl);
}

// elx_conv (src/elx_conv.cpp:213-240).  wait = true is eager_mode (or stream_sync): the result is
// there when the call returns.  wait = false is the reference's asynchronous mode
// (src/elx_stream.cpp:54-62): copies and kernels are enqueued on the plan's streams, the call
// returns, and elb_conv_wait (or the next waiting call, or the plan's destruction) completes it.
// Calls on one plan run in submission order, as on the reference's single worker thread.
int execute_common(elb_conv &pl, void *output, const void *input, const void *weights, const void *bias, bool wait) {
  DeviceGuard guard(pl.device);
  int rc = do_prepare(pl, weights, bias);
  if (rc != ELB_OK) return rc;
  const bool verbose = log_options().verbose && wait;
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  if (verbose) {
    if (pl.pending && (rc = wait_pending(pl)) != ELB_OK) return rc;
    CUDA_TRY(cudaEventCreate(&t0));
    CUDA_TRY(cudaEventCreate(&t1));
  }
  auto finish = [&](bool used_d2h) -> int {
    int r = fetch_status_async(pl, pl.stream);
    if (r != ELB_OK) return r;
    if (!wait) {
      // the next call must not overwrite the staging buffers before this one has used them
      CUDA_TRY(cudaEventRecord(pl.ev_call_done, pl.stream));
      if (used_d2h) CUDA_TRY(cudaEventRecord(pl.ev_d2h_done, pl.s_d2h));
      pl.pending = true;
      pl.pending_d2h = pl.pending_d2h || used_d2h;
      return ELB_OK;
    }
    pl.pending = true;
    pl.pending_d2h = pl.pending_d2h || used_d2h;
    return wait_pending(pl);
  };
  const bool in_dev = is_device_ptr(input), out_dev = is_device_ptr(output);
  if (in_dev && out_dev) {
    if (verbose) CUDA_TRY(cudaEventRecord(t0, pl.stream));
    rc = do_enqueue(pl, output, input, pl.stream);
    if (rc != ELB_OK) return rc;
    if (verbose) CUDA_TRY(cudaEventRecord(t1, pl.stream));
    rc = finish(false);
  } else {
    // Host tensors (what a caller of the reference holds) are staged through device buffers of the plan.
    const int N = pl.d.n;
    const size_t in_img = pl.uinfo.bytes_input / N, out_img = pl.uinfo.bytes_output / N;
    if (!in_dev && !pl.d_in_stage) CUDA_TRY(cudaMalloc(&pl.d_in_stage, pl.uinfo.bytes_input));
    if (!out_dev && !pl.d_out_stage) CUDA_TRY(cudaMalloc(&pl.d_out_stage, pl.uinfo.bytes_output));
    if (!pl.s_h2d) {
      CUDA_TRY(cudaStreamCreateWithFlags(&pl.s_h2d, cudaStreamNonBlocking));
      CUDA_TRY(cudaStreamCreateWithFlags(&pl.s_d2h, cudaStreamNonBlocking));
    }
    const size_t moved = (in_dev ? 0 : pl.uinfo.bytes_input) + (out_dev ? 0 : pl.uinfo.bytes_output);
    // Small calls (under 8 MB moved) run in order on ONE stream: copy in, kernels, copy out, status.
    // Larger ones are cut into chunks of whole images (about 4 MB of transfers each, at most 8), and
    // the host->device copy of chunk k+1, the kernels of chunk k and the device->host copy of chunk
    // k-1 run at the same time on three streams (the two copy directions use different copy
    // engines), so the call costs about the longer of the two transfers instead of their sum
    // (measured on the 1x1 benchmark layer, 12.8 MB in / 3.2 MB out: 0.33 ms chunked, 0.35-0.40 ms on
    // one stream).  ELB_HOST_CHUNKS overrides the chunk count.
    int chunks = moved < (size_t(8) << 20) ? 1 : (int)std::min<size_t>(8, moved / (size_t(4) << 20));
    if (const char *e = getenv("ELB_HOST_CHUNKS")) {
      const int v = atoi(e);
      if (v >= 1) chunks = v;
    }
    if (chunks > N) chunks = N;
    const void *din = in_dev ? input : pl.d_in_stage;
    void *dout = out_dev ? output : pl.d_out_stage;
    if (pl.pending) {         // an unfinished asynchronous call still reads / writes the staging buffers
      CUDA_TRY(cudaStreamWaitEvent(pl.s_h2d, pl.ev_call_done, 0));
      if (pl.pending_d2h) CUDA_TRY(cudaStreamWaitEvent(pl.stream, pl.ev_d2h_done, 0));
    }
    if (verbose) CUDA_TRY(cudaEventRecord(t0, pl.stream));
    if (chunks == 1) {
      if (!in_dev) CUDA_TRY(cudaMemcpyAsync(pl.d_in_stage, input, pl.uinfo.bytes_input, cudaMemcpyHostToDevice, pl.stream));
      if (!out_dev && pl.d.with_ip_sum)
        CUDA_TRY(cudaMemcpyAsync(pl.d_out_stage, output, pl.uinfo.bytes_output, cudaMemcpyHostToDevice, pl.stream));
      rc = do_enqueue(pl, dout, din, pl.stream);
      if (rc != ELB_OK) { cudaDeviceSynchronize(); return rc; }
      if (!out_dev) CUDA_TRY(cudaMemcpyAsync(output, pl.d_out_stage, pl.uinfo.bytes_output, cudaMemcpyDeviceToHost, pl.stream));
      if (verbose) CUDA_TRY(cudaEventRecord(t1, pl.stream));
      rc = finish(false);
    } else {
      while ((int)pl.ev_in.size() < chunks) {
        cudaEvent_t a = nullptr, b = nullptr;
        CUDA_TRY(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        CUDA_TRY(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
        pl.ev_in.push_back(a);
        pl.ev_done.push_back(b);
      }
      for (int k = 0; k < chunks; ++k) {
        const int n0 = (int)((long long)N * k / chunks), n1 = (int)((long long)N * (k + 1) / chunks);
        const int cnt = n1 - n0;
        if (!in_dev)
          CUDA_TRY(cudaMemcpyAsync((uint8_t *)pl.d_in_stage + n0 * in_img, (const uint8_t *)input + n0 * in_img, cnt * in_img,
                                   cudaMemcpyHostToDevice, pl.s_h2d));
        if (!out_dev && pl.d.with_ip_sum)
          CUDA_TRY(cudaMemcpyAsync((uint8_t *)pl.d_out_stage + n0 * out_img, (const uint8_t *)output + n0 * out_img,
                                   cnt * out_img, cudaMemcpyHostToDevice, pl.s_h2d));
        CUDA_TRY(cudaEventRecord(pl.ev_in[k], pl.s_h2d));
        CUDA_TRY(cudaStreamWaitEvent(pl.stream, pl.ev_in[k], 0));
        rc = do_enqueue_range(pl, dout, din, n0, cnt, pl.stream);
        if (rc != ELB_OK) { cudaDeviceSynchronize(); return rc; }
        if (!out_dev) {
          CUDA_TRY(cudaEventRecord(pl.ev_done[k], pl.stream));
          CUDA_TRY(cudaStreamWaitEvent(pl.s_d2h, pl.ev_done[k], 0));
          CUDA_TRY(cudaMemcpyAsync((uint8_t *)output + n0 * out_img, (uint8_t *)pl.d_out_stage + n0 * out_img, cnt * out_img,
                                   cudaMemcpyDeviceToHost, pl.s_d2h));
        }
      }
      if (verbose) {
        if (!out_dev) {       // the call ends with the last copy out: bring it back onto the timed stream
          CUDA_TRY(cudaEventRecord(pl.ev_d2h_done, pl.s_d2h));
          CUDA_TRY(cudaStreamWaitEvent(pl.stream, pl.ev_d2h_done, 0));
        }
        CUDA_TRY(cudaEventRecord(t1, pl.stream));
      }
      rc = finish(!out_dev);
    }
  }
  if (verbose) {
    float ms = 0.0f;
    if (rc == ELB_OK && cudaEventElapsedTime(&ms, t0, t1) == cudaSuccess) perf_line(pl, ms);
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
  }
  return rc;
}

}  // namespace

// =============================================================================== C ABI
extern "C" {

const char *elb_last_error(void) { return g_last_error.c_str(); }

int elb_device_supported(int device) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    cudaGetLastError();
    return fail(ELB_GENERAL_ERROR, "no CUDA device available");
  }
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) return fail(ELB_GENERAL_ERROR, "cudaGetDevice failed");
  if (device >= count) return fail(ELB_GENERAL_ERROR, "device %d out of range", device);
  cudaDeviceProp prop;
  CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) return fail(ELB_UNIMPLEMENTED, "device %d is sm_%d%d; this library is built for sm_100a only",
                                    device, prop.major, prop.minor);
  return ELB_OK;
}

int elb_conv_sizes(const elb_conv_desc_t *desc, elb_conv_info_t *info) {
  if (!desc || !info) return fail(ELB_GENERAL_ERROR, "null argument");
  int rc = validate_common(*desc);
  if (rc != ELB_OK) return rc;
  memset(info, 0, sizeof(*info));
  elb_conv_desc_t ud = *desc;
  resolve_formats(ud);
  compute_sizes(ud, *info);
  resolve_algorithm(*desc, info->algorithm, info->tile_size);
  const char *why;
  bool ci, co, cw;
  info->kernel = choose_kernel(internal_desc(ud, ci, co, cw), info->algorithm, info->tile_size, &why);
  info->device = desc->device;
  return ELB_OK;
}

int elb_conv_create(const elb_conv_desc_t *desc, elb_conv_t **plan) {
  if (!desc || !plan) return fail(ELB_GENERAL_ERROR, "null argument");
  *plan = nullptr;
  int rc = validate_common(*desc);
  if (rc != ELB_OK) return rc;
  bool cvt_in = false, cvt_out = false, cvt_w = false;
  elb_conv_desc_t ud = *desc;
  resolve_formats(ud);
  // bottom/right padding follow from the output size, as the reference does with a warning
  // (src/eld_conv.cpp:128-139, src/elx_conv.cpp:36-37)
  {
    const int need_b = (ud.oh - 1) * ud.stride_h + ud.kh - ud.ih - ud.pad_t;
    const int need_r = (ud.ow - 1) * ud.stride_w + ud.kw - ud.iw - ud.pad_l;
    ud.pad_b = need_b > 0 ? need_b : 0;
    ud.pad_r = need_r > 0 ? need_r : 0;
  }
  elb_conv_desc_t d = internal_desc(ud, cvt_in, cvt_out, cvt_w);
  elb_conv_info_t info, uinfo;
  memset(&info, 0, sizeof(info));
  memset(&uinfo, 0, sizeof(uinfo));
  compute_sizes(d, info);
  compute_sizes(ud, uinfo);
  // algorithm choice uses the caller's pads, like the reference
  resolve_algorithm(*desc, info.algorithm, info.tile_size);
  const char *why;
  info.kernel = choose_kernel(d, info.algorithm, info.tile_size, &why);
  if (info.kernel == ELB_KERNEL_NONE) return fail(ELB_UNIMPLEMENTED, "not implemented on the GPU: %s", why);

  rc = elb_device_supported(d.device);
  if (rc != ELB_OK) return rc;
  int dev = d.device;
  if (dev < 0) cudaGetDevice(&dev);
  info.device = dev;
  DeviceGuard guard(dev);
  if (!guard.ok) return fail(ELB_GENERAL_ERROR, "cannot select device %d", dev);

  elb_conv *pl = new elb_conv();
  pl->d = d;
  pl->info = info;
  pl->ud = ud;
  pl->cvt_in = cvt_in; pl->cvt_out = cvt_out; pl->cvt_w = cvt_w;
  pl->device = dev;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) { delete pl; return fail(ELB_GENERAL_ERROR, "device query failed"); }
  pl->num_sms = prop.multiProcessorCount;
  if (cudaStreamCreateWithFlags(&pl->stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaMalloc(&pl->d_status, sizeof(int)) != cudaSuccess ||
      cudaMemset(pl->d_status, 0, sizeof(int)) != cudaSuccess ||
      cudaHostAlloc(&pl->h_status, sizeof(int), cudaHostAllocDefault) != cudaSuccess ||
      cudaEventCreateWithFlags(&pl->ev_call_done, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&pl->ev_d2h_done, cudaEventDisableTiming) != cudaSuccess) {
    delete pl;
    return fail(ELB_GENERAL_ERROR, "device allocation failed");
  }
  switch (info.kernel) {
    case ELB_KERNEL_I8_GEMM_UMMA:
    case ELB_KERNEL_I8_CONV_UMMA:
    case ELB_KERNEL_I8_SIMT: rc = setup_i8_direct(*pl); break;
    case ELB_KERNEL_I8_DEPTHWISE: {
      std::string err;
      rc = dw_setup(pl->dw, pl->d, pl->info, pl->num_sms, err);
      if (rc != ELB_OK) fail(rc, "%s", err.c_str());
      break;
    }
    default: {
      std::string err;
      rc = wino_setup(pl->wino, pl->d, pl->info, err);
      if (rc != ELB_OK) fail(rc, "%s", err.c_str());
    }
  }
  if (rc != ELB_OK) { delete pl; return rc; }
  // the direct kernel for at most four input channels reads an nchw tensor itself: no conversion,
  // no 16-channel copy of an image of which three channels are real
  if (cvt_in && ud.fmt_input == ELB_NCHW && pl->info.kernel == ELB_KERNEL_F32_SMALL_IC) {
    pl->wino.in_planar = true;
    pl->cvt_in = cvt_in = false;
  }
  // what the caller sees: the sizes of ITS formats, everything else from the internal plan
  uinfo.algorithm = pl->info.algorithm; uinfo.tile_size = pl->info.tile_size; uinfo.kernel = pl->info.kernel;
  uinfo.device = pl->info.device; uinfo.launches_per_call = pl->info.launches_per_call + (cvt_in ? 1 : 0) + (cvt_out ? 1 : 0);
  pl->uinfo = uinfo;
  if ((cvt_in && cudaMalloc(&pl->d_cvt_in, pl->info.bytes_input) != cudaSuccess) ||
      (cvt_out && cudaMalloc(&pl->d_cvt_out, pl->info.bytes_output) != cudaSuccess)) {
    delete pl;
    return fail(ELB_GENERAL_ERROR, "device allocation failed");
  }
  *plan = pl;
  return ELB_OK;
}

int elb_conv_info(const elb_conv_t *plan, elb_conv_info_t *info) {
  if (!plan || !info) return fail(ELB_GENERAL_ERROR, "null argument");
  *info = plan->uinfo;
  info->workspace_bytes = plan->info.workspace_bytes;
  return ELB_OK;
}

int elb_conv_prepare(elb_conv_t *plan, const void *weights, const void *bias) {
  if (!plan) return fail(ELB_GENERAL_ERROR, "null plan");
  DeviceGuard guard(plan->device);
  return do_prepare(*plan, weights, bias);
}

int elb_conv_enqueue(elb_conv_t *plan, void *output, const void *input, const void *weights, const void *bias,
                     void *cuda_stream) {
  if (!plan || !output || !input) return fail(ELB_GENERAL_ERROR, "null argument");   // src/elx_conv.cpp:218-222
  DeviceGuard guard(plan->device);
  int rc = do_prepare(*plan, weights, bias);
  if (rc != ELB_OK) return rc;
  return do_enqueue(*plan, output, input, static_cast<cudaStream_t>(cuda_stream));
}

int elb_conv_input_step_supported(elb_conv_t *plan) {
  if (!plan) return 0;
  const int k = plan->info.kernel;
  return (k == ELB_KERNEL_WINO_F32_UMMA && !plan->cvt_in && wino_input_step_supported(plan->wino)) ? 1 : 0;
}

int elb_conv_enqueue_strided(elb_conv_t *plan, void *output, const void *input, int src_h, int src_w, int step,
                             void *cuda_stream) {
  if (!plan || !output || !input) return fail(ELB_GENERAL_ERROR, "null argument");
  if (step < 1 || src_h < 1 || src_w < 1 || (src_h + step - 1) / step != plan->d.ih || (src_w + step - 1) / step != plan->d.iw)
    return fail(ELB_GENERAL_ERROR, "strided input: %d x %d read with step %d is not the %d x %d input of this plan", src_h,
                src_w, step, plan->d.ih, plan->d.iw);
  if (step == 1) return elb_conv_enqueue(plan, output, input, nullptr, nullptr, cuda_stream);
  DeviceGuard guard(plan->device);
  int rc = do_prepare(*plan, nullptr, nullptr);
  if (rc != ELB_OK) return rc;
  if (!elb_conv_input_step_supported(plan)) return fail(ELB_UNIMPLEMENTED, "this plan's kernel cannot read its input with a step");
  plan->wino.in_step = step; plan->wino.src_h = src_h; plan->wino.src_w = src_w;
  rc = do_enqueue(*plan, output, input, static_cast<cudaStream_t>(cuda_stream));
  plan->wino.in_step = 1;
  return rc;
}

int elb_conv_execute(elb_conv_t *plan, void *output, const void *input, const void *weights, const void *bias) {
  if (!plan || !output || !input) return fail(ELB_GENERAL_ERROR, "null argument");
  return execute_common(*plan, output, input, weights, bias, true);
}

int elb_conv_execute_async(elb_conv_t *plan, void *output, const void *input, const void *weights, const void *bias) {
  if (!plan || !output || !input) return fail(ELB_GENERAL_ERROR, "null argument");
  return execute_common(*plan, output, input, weights, bias, false);
}

int elb_conv_wait(elb_conv_t *plan) {
  if (!plan) return fail(ELB_GENERAL_ERROR, "null plan");
  DeviceGuard guard(plan->device);
  return wait_pending(*plan);
}

int elb_conv_set_name(elb_conv_t *plan, const char *name) {
  if (!plan) return fail(ELB_GENERAL_ERROR, "null plan");
  plan->name = name ? name : "";
  return ELB_OK;
}

int elb_conv_set_accumulator_dump(elb_conv_t *plan, void *device_int32) {
  if (!plan) return fail(ELB_GENERAL_ERROR, "null plan");
  plan->d_acc_dump = device_int32;
  return ELB_OK;
}

// Debug hook (not part of the reference surface): per-CTA timeline of the tcgen05 kernels, 64
// int64 slots per CTA in caller device memory; NULL switches it off.
ELB_API int elb_conv_set_trace(elb_conv_t *plan, void *device_int64) {
  if (!plan) return ELB_GENERAL_ERROR;
  plan->d_trace = device_int64;
  return ELB_OK;
}

// Measurement hook (not part of the reference surface): four CUDA events that the Winograd path
// records before its input transform, between its three kernels and after the output transform of
// the first chunk of every following call, so that a benchmark can time each kernel on the
// launching stream.  NULL switches it off.  Do not leave it on while capturing a CUDA graph.
ELB_API int elb_conv_set_stage_events(elb_conv_t *plan, void **cuda_events4) {
  if (!plan) return ELB_GENERAL_ERROR;
  for (int i = 0; i < 4; ++i) plan->wino.stage_ev[i] = cuda_events4 ? static_cast<cudaEvent_t>(cuda_events4[i]) : nullptr;
  return ELB_OK;
}

int elb_conv_device_status(elb_conv_t *plan) {
  if (!plan) return -1;
  DeviceGuard guard(plan->device);
  int st = -1;
  if (cudaMemcpy(&st, plan->d_status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return st;
}

uint64_t elb_conv_launch_count(const elb_conv_t *plan) { return plan ? plan->launches : 0; }

void elb_conv_destroy(elb_conv_t *plan) { delete plan; }

int elb_reorder_nchw_to_nChw16c(void *dst, const void *src, int n, int c, int h, int w, int elem_bytes,
                                void *cuda_stream) {
  if (!dst || !src || (elem_bytes != 1 && elem_bytes != 4)) return fail(ELB_GENERAL_ERROR, "bad reorder argument");
  cudaError_t e = launch_reorder_to_blocked(dst, src, n, c, h, w, elem_bytes, static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) return fail(ELB_GENERAL_ERROR, "reorder launch failed: %s", cudaGetErrorString(e));
  return ELB_OK;
}

int elb_reorder_nChw16c_to_nchw(void *dst, const void *src, int n, int c, int h, int w, int elem_bytes,
                                void *cuda_stream) {
  if (!dst || !src || (elem_bytes != 1 && elem_bytes != 4)) return fail(ELB_GENERAL_ERROR, "bad reorder argument");
  cudaError_t e = launch_reorder_from_blocked(dst, src, n, c, h, w, elem_bytes, static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) return fail(ELB_GENERAL_ERROR, "reorder launch failed: %s", cudaGetErrorString(e));
  return ELB_OK;
}

int elb_reorder(void *dst, int dst_format, const void *src, int src_format, int g, int a, int b, int h, int w,
                int elem_bytes, void *cuda_stream) {
  if (!dst || !src) return fail(ELB_GENERAL_ERROR, "bad reorder argument");
  bool supported = false;
  cudaError_t e = launch_reorder(dst, dst_format, src, src_format, g, a, b, h, w, elem_bytes,
                                 static_cast<cudaStream_t>(cuda_stream), supported);
  if (!supported) return fail(ELB_UNIMPLEMENTED, "reorder from format %d to format %d (element size %d) is not implemented",
                              src_format, dst_format, elem_bytes);
  if (e != cudaSuccess) return fail(ELB_GENERAL_ERROR, "reorder launch failed: %s", cudaGetErrorString(e));
  return ELB_OK;
}

int elb_subsample_nChw16c(void *dst, const void *src, int n, int c, int h, int w, int step_h, int step_w,
                          int elem_bytes, void *cuda_stream) {
  if (!dst || !src || (elem_bytes != 1 && elem_bytes != 4) || n < 1 || c < 1 || h < 1 || w < 1 || step_h < 1 ||
      step_w < 1)
    return fail(ELB_GENERAL_ERROR, "bad subsample argument");
  cudaError_t e = launch_subsample_blocked(dst, src, n, c, h, w, step_h, step_w, elem_bytes,
                                           static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) return fail(ELB_GENERAL_ERROR, "subsample launch failed: %s", cudaGetErrorString(e));
  return ELB_OK;
}

// Test hook (not part of the reference surface): runs the bounded-wait self test and returns the
// status word the kernel wrote (ST_WAIT_TIMEOUT_TEST = 104 when the wait gave up as designed).
ELB_API int elb_selftest_bounded_wait(int device, unsigned long long limit_ns) {
  int rc = elb_device_supported(device);
  if (rc != ELB_OK) return -rc;
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) return -1;
  DeviceGuard guard(device);
  int *st = nullptr, h = -1;
  if (cudaMalloc(&st, sizeof(int)) != cudaSuccess) return -1;
  cudaMemset(st, 0, sizeof(int));
  cudaError_t e = launch_wait_selftest(st, limit_ns, nullptr);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) cudaMemcpy(&h, st, sizeof(int), cudaMemcpyDeviceToHost);
  cudaFree(st);
  return e == cudaSuccess ? h : -1;
}

}  // extern "C"
