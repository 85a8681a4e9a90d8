// C++ host library: the reference's public C++ surface implemented on top of the C-ABI.
//
// The reference exports exactly four convolution symbols from its libel.so --
// euler::eld_conv_t::eld_conv_t(), ~eld_conv_t(), eld_conv_t::setup(bool) and
// euler::elx_conv(eld_conv_t&, void*, void*, void*, void*) (include/euler.hpp:110-190, built with
// hidden visibility) -- plus 24 reorder<T, dst, src> constructors (include/euler_reorder.hpp:9-64,
// src/elx_reorder.cpp:209-232).  This file defines the same symbols, so a program written and
// compiled against the reference's own headers links against this library instead of the
// reference's and runs its convolutions on the GPU.  It is compiled WITH the reference's headers
// (-I<reference>/include): the descriptor type, its field order and the mangled names are the
// reference's by construction, nothing is restated here.
//
// What each function does:
//   eld_conv_t()        the reference's defaults (src/eld_conv.cpp:19-50)
//   setup(fully)        descriptor -> elb_conv_desc_t -> elb_conv_sizes / elb_conv_create; fills
//                       sizes, byte_sizes, the resolved algorithm / tile_size and keeps the plan
//                       in `xc` (src/eld_conv.cpp:59-316)
//   elx_conv            first call prepares the weights, every call executes
//                       (src/elx_conv.cpp:213-240); tensors may be host or device memory
//   ~eld_conv_t()       releases the plan (src/eld_conv.cpp:52-57)
//   reorder<...>        layout conversions of HOST tensors as the reference's test harness uses them
//                       (src/elx_reorder.cpp:11-207); plain loops, not part of any timed path
// eager_mode = false enqueues the call on the plan's CUDA streams and returns (the reference hands
// it to one worker thread, src/elx_stream.cpp:54-62); stream_sync = true then waits
// (src/elx_conv.cpp:234-235), and so does the destructor.  With EULER_GPUS=G (G > 1) in the
// environment a fully set-up descriptor splits its minibatch over GPUs 0..G-1 (host tensors only).
// Differences a caller can observe: unsupported descriptors return ELD_UNIMPLEMENTED where the
// reference prints "euler-error" and aborts; the CPU tuning knobs are ignored (flatting.t is
// honoured by the int8 depthwise path, whose rounding depends on it).
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "euler.hpp"
#include "euler_reorder.hpp"
#include "euler_b200.h"

namespace euler {

// `xc` is an opaque pointer for callers; here it carries the C-ABI plan (one GPU) or the
// minibatch-split plan (EULER_GPUS > 1).
struct host_plan {
  elb_conv_t *single = nullptr;
  elb_conv_multi_t *multi = nullptr;
};
static inline host_plan *plan_of(eld_conv_t &d) { return reinterpret_cast<host_plan *>(d.xc); }
static void drop_plan(eld_conv_t &d) {
  host_plan *h = plan_of(d);
  if (h == nullptr) return;
  if (h->single) elb_conv_destroy(h->single);      // waits for asynchronous calls still in flight
  if (h->multi) elb_conv_multi_destroy(h->multi);
  delete h;
  d.xc = nullptr;
}
static int gpus_from_env() {
  const char *e = getenv("EULER_GPUS");
  return e ? atoi(e) : 1;
}

static void to_c_desc(const eld_conv_t &s, elb_conv_desc_t &d) {
  std::memset(&d, 0, sizeof(d));
  d.n = s.dims.n; d.g = s.dims.g; d.ic = s.dims.ic; d.oc = s.dims.oc;
  d.ih = s.dims.ih; d.iw = s.dims.iw; d.oh = s.dims.oh; d.ow = s.dims.ow; d.kh = s.dims.kh; d.kw = s.dims.kw;
  d.pad_l = s.pads.l; d.pad_r = s.pads.r; d.pad_t = s.pads.t; d.pad_b = s.pads.b;
  d.stride_h = s.strides.h; d.stride_w = s.strides.w;
  d.dilation_h = s.dilations.h; d.dilation_w = s.dilations.w;
  d.dt_input = s.data_type.input; d.dt_weights = s.data_type.weights;
  d.dt_output = s.data_type.output; d.dt_bias = s.data_type.bias;
  d.fmt_input = s.formats.input; d.fmt_weights = s.formats.weights; d.fmt_output = s.formats.output;
  d.prop_kind = s.prop_kind;
  d.algorithm = s.algorithm; d.tile_size = s.tile_size;
  d.with_relu = s.with_relu; d.with_bias = s.with_bias; d.with_ip_sum = s.with_ip_sum;
  d.with_op_sum = s.with_op_sum; d.with_argmax = s.with_argmax;
  d.f16c_opt = s.f16c_opt; d.disable_autoparam = s.disable_autoparam;
  d.relu_lower = s.relu_bound.lower; d.relu_upper = s.relu_bound.upper;
  d.execution_mode = s.execution_mode;
  d.input_scale = s.input_quant.scale; d.input_z = s.input_quant.z;
  d.tinput_scale = s.wino_tinput_quant.scale; d.tinput_z = s.wino_tinput_quant.z;
  d.output_scale = s.output_quant.scale; d.output_z = s.output_quant.z;
  d.sum_scale = s.sum_quant.scale; d.sum_z = s.sum_quant.z;
  d.sampling_kind = static_cast<int32_t>(s.sampling_kind);
  d.flatting_t = s.flatting.t;
  d.device = -1;      // the calling thread's current CUDA device
}

// (the C-ABI layer has already logged the message under EULER_LOG_LEVEL; nothing to add here)
static void report(const char *) {}

eld_conv_t::eld_conv_t() {
  std::memset(&dims, 0, sizeof(dims));
  dims.g = 1;
  pads = {1, 1, 1, 1};
  strides = {1, 1};
  dilations = {1, 1};
  data_type.flat = 0;
  formats = {format_undef, format_undef, format_undef};
  prop_kind = forward_inference;
  algorithm = CONV_DIRECT;
  tile_size = 0;
  with_relu = with_bias = with_ip_sum = with_op_sum = with_argmax = false;
  f16c_opt = false;
  is_inference = true;
  use_scratch_pad = false;
  disable_autoparam = false;
  eager_mode = true;
  stream_sync = false;
  nthreads = 0;
  execution_mode = 0;
  flatting = {0, 0};
  blocking = {0, 0};
  partition = {1, 1, 1};
  streaming_hint = {0, 0};
  format_as_blocked = {false, false, false};
  input_quant = {EL_NO_CALI, EL_NO_CALI};
  wino_tinput_quant = {EL_NO_CALI, EL_NO_CALI};
  output_quant = {EL_NO_CALI, EL_NO_CALI};
  sum_quant = {EL_NO_CALI, EL_NO_CALI};
  sampling_kind = FINE;
  scratch_pad = nullptr;
  name = "ioi";
  byte_sizes = {0, 0, 0, 0};
  sizes = {0, 0, 0, 0};
  xc = nullptr;
}

eld_conv_t::~eld_conv_t() { drop_plan(*this); }

int eld_conv_t::setup(bool fully_setup) {
  // a stale plan is dropped (the reference overwrites xc and leaks it, src/eld_conv.cpp:141)
  drop_plan(*this);
  // undefined formats get the reference's defaults, visibly, in the descriptor (src/eld_conv.cpp:77-86)
  if (formats.input == format_undef) formats.input = (dims.g == 1 && dims.ic / dims.g < 16) ? nchw : nChw16c;
  if (formats.weights == format_undef) formats.weights = dims.g == 1 ? hwio : ghwio;
  if (formats.output == format_undef) formats.output = nChw16c;
  elb_conv_desc_t d;
  to_c_desc(*this, d);
  elb_conv_info_t info;
  int rc = elb_conv_sizes(&d, &info);
  if (rc != ELB_OK) { report("setup"); return rc; }
  sizes = {static_cast<size_t>(info.size_input), static_cast<size_t>(info.size_weights),
           static_cast<size_t>(info.size_output), static_cast<size_t>(info.size_bias)};
  byte_sizes = {static_cast<size_t>(info.bytes_input), static_cast<size_t>(info.bytes_weights),
                static_cast<size_t>(info.bytes_output), static_cast<size_t>(info.bytes_bias)};
  algorithm = info.algorithm;
  tile_size = info.tile_size;
  if (!fully_setup) return ELD_OK;                 // src/eld_conv.cpp:161-163
  host_plan *h = new host_plan();
  const int gpus = gpus_from_env();
  if (gpus > 1 && dims.n >= 2) rc = elb_conv_multi_create(&d, nullptr, gpus, &h->multi);
  else rc = elb_conv_create(&d, &h->single);
  if (rc != ELB_OK) { delete h; report("setup"); return rc; }
  if (h->single) elb_conv_set_name(h->single, name.c_str());
  xc = reinterpret_cast<elx_conv_t *>(h);
  return ELD_OK;
}

int elx_conv(eld_conv_t &desc, void *output, void *input, void *weights, void *bias) {
  if (desc.xc == nullptr || output == nullptr || input == nullptr) return ELX_GENERAL_ERROR;   // src/elx_conv.cpp:218-222
  host_plan *h = plan_of(desc);
  int rc;
  if (h->multi) {
    rc = elb_conv_multi_execute(h->multi, output, input, weights, bias);
  } else if (desc.eager_mode) {
    rc = elb_conv_execute(h->single, output, input, weights, bias);
  } else {
    // src/elx_conv.cpp:228-236: submit, and wait only when stream_sync is set
    rc = elb_conv_execute_async(h->single, output, input, weights, bias);
    if (rc == ELB_OK && desc.stream_sync) rc = elb_conv_wait(h->single);
  }
  if (rc != ELB_OK) report("elx_conv");
  return rc;
}

// ------------------------------------------------------------------------------ reorder (host)
namespace {
inline int up16(int x) { return (x + 15) / 16 * 16; }
}

template <typename T> reorder<T, nchw, nhwc>::reorder(T *dst, T *src, int n, int c, int h, int w) {
  for (int a = 0; a < n; ++a) for (int b = 0; b < c; ++b) for (int y = 0; y < h; ++y) for (int x = 0; x < w; ++x)
    dst[((size_t(a) * c + b) * h + y) * w + x] = src[((size_t(a) * h + y) * w + x) * c + b];
}
template <typename T> reorder<T, nhwc, nchw>::reorder(T *dst, T *src, int n, int c, int h, int w) {
  for (int a = 0; a < n; ++a) for (int b = 0; b < c; ++b) for (int y = 0; y < h; ++y) for (int x = 0; x < w; ++x)
    dst[((size_t(a) * h + y) * w + x) * c + b] = src[((size_t(a) * c + b) * h + y) * w + x];
}
// blocked -> plain drops the padding lanes; plain -> blocked zero-fills them (src/elx_reorder.cpp:40-66)
template <typename T> reorder<T, nchw, nChw16c>::reorder(T *dst, T *src, int n, int c, int h, int w) {
  const int C2 = up16(c) / 16;
  for (int a = 0; a < n; ++a) for (int b = 0; b < c; ++b) for (int y = 0; y < h; ++y) for (int x = 0; x < w; ++x)
    dst[((size_t(a) * c + b) * h + y) * w + x] = src[(((size_t(a) * C2 + b / 16) * h + y) * w + x) * 16 + b % 16];
}
template <typename T> reorder<T, nChw16c, nchw>::reorder(T *dst, T *src, int n, int c, int h, int w) {
  const int C2 = up16(c) / 16;
  for (int a = 0; a < n; ++a) for (int b = 0; b < C2 * 16; ++b) for (int y = 0; y < h; ++y) for (int x = 0; x < w; ++x)
    dst[(((size_t(a) * C2 + b / 16) * h + y) * w + x) * 16 + b % 16] =
        b < c ? src[((size_t(a) * c + b) * h + y) * w + x] : T(0);
}
template <typename T> reorder<T, oihw, OIhw16i16o>::reorder(T *dst, T *src, int o, int i, int h, int w) {
  const int I2 = up16(i) / 16;
  for (int a = 0; a < o; ++a) for (int b = 0; b < i; ++b) for (int y = 0; y < h; ++y) for (int x = 0; x < w; ++x)
    dst[((size_t(a) * i + b) * h + y) * w + x] =
        src[((((size_t(a / 16) * I2 + b / 16) * h + y) * w + x) * 16 + b % 16) * 16 + a % 16];
}
template <typename T> reorder<T, OIhw16i16o, oihw>::reorder(T *dst, T *src, int o, int i, int h, int w) {
  const int O2 = up16(o) / 16, I2 = up16(i) / 16;
  for (int a = 0; a < O2 * 16; ++a) for (int b = 0; b < I2 * 16; ++b) for (int y = 0; y < h; ++y) for (int x = 0; x < w; ++x)
    dst[((((size_t(a / 16) * I2 + b / 16) * h + y) * w + x) * 16 + b % 16) * 16 + a % 16] =
        (a < o && b < i) ? src[((size_t(a) * i + b) * h + y) * w + x] : T(0);
}
template <typename T> reorder<T, goihw, gOIhw16i16o>::reorder(T *dst, T *src, int g, int o, int i, int h, int w) {
  const size_t plain = size_t(o) * i * h * w, blocked = size_t(up16(o)) * up16(i) * h * w;
  for (int a = 0; a < g; ++a) reorder<T, oihw, OIhw16i16o>(dst + a * plain, src + a * blocked, o, i, h, w);
}
template <typename T> reorder<T, gOIhw16i16o, goihw>::reorder(T *dst, T *src, int g, int o, int i, int h, int w) {
  const size_t plain = size_t(o) * i * h * w, blocked = size_t(up16(o)) * up16(i) * h * w;
  for (int a = 0; a < g; ++a) reorder<T, OIhw16i16o, oihw>(dst + a * blocked, src + a * plain, o, i, h, w);
}
template <typename T> reorder<T, oihw, hwio>::reorder(T *dst, T *src, int o, int i, int h, int w) {
  for (int a = 0; a < o; ++a) for (int b = 0; b < i; ++b) for (int y = 0; y < h; ++y) for (int x = 0; x < w; ++x)
    dst[((size_t(a) * i + b) * h + y) * w + x] = src[((size_t(y) * w + x) * i + b) * o + a];
}
template <typename T> reorder<T, hwio, oihw>::reorder(T *dst, T *src, int o, int i, int h, int w) {
  for (int a = 0; a < o; ++a) for (int b = 0; b < i; ++b) for (int y = 0; y < h; ++y) for (int x = 0; x < w; ++x)
    dst[((size_t(y) * w + x) * i + b) * o + a] = src[((size_t(a) * i + b) * h + y) * w + x];
}
template <typename T> reorder<T, goihw, ghwio>::reorder(T *dst, T *src, int g, int o, int i, int h, int w) {
  const size_t per = size_t(o) * i * h * w;
  for (int a = 0; a < g; ++a) reorder<T, oihw, hwio>(dst + a * per, src + a * per, o, i, h, w);
}
template <typename T> reorder<T, ghwio, goihw>::reorder(T *dst, T *src, int g, int o, int i, int h, int w) {
  const size_t per = size_t(o) * i * h * w;
  for (int a = 0; a < g; ++a) reorder<T, hwio, oihw>(dst + a * per, src + a * per, o, i, h, w);
}

#define ELB_INSTANTIATE_REORDERS(T)               \
  template struct reorder<T, nchw, nhwc>;         \
  template struct reorder<T, nhwc, nchw>;         \
  template struct reorder<T, nchw, nChw16c>;      \
  template struct reorder<T, nChw16c, nchw>;      \
  template struct reorder<T, oihw, OIhw16i16o>;   \
  template struct reorder<T, goihw, gOIhw16i16o>; \
  template struct reorder<T, OIhw16i16o, oihw>;   \
  template struct reorder<T, gOIhw16i16o, goihw>; \
  template struct reorder<T, oihw, hwio>;         \
  template struct reorder<T, goihw, ghwio>;       \
  template struct reorder<T, hwio, oihw>;         \
  template struct reorder<T, ghwio, goihw>;
ELB_INSTANTIATE_REORDERS(float)
ELB_INSTANTIATE_REORDERS(uint8_t)

}  // namespace euler
