// TEST INFRASTRUCTURE ONLY.  Command-line driver that runs ONE convolution through the
// unmodified reference library (Euler: include/euler.hpp, eld_conv_t::setup + elx_conv) on
// tensors read from raw files, writes the output tensor to a raw file and prints one JSON line
// with the return codes and timings.  It is linked against oracle/_ref/libel.so by
// oracle/build_ref.sh and is used (a) to pin the C restatement in oracle/euler_oracle.c,
// (b) to generate tests/golden/, (c) as the timed CPU reference in bench.py.
//
// All tensors are in the layouts the descriptor names (blocked nChw16c / OIhw16i16o unless
// stated otherwise); the caller (Python) produces them.  Arguments are key=value pairs:
//
//   n ic oc ih iw oh ow kh kw g        dims           (oh/ow default to the conv formula)
//   pt pb pl pr sh sw                  pads, strides  (default pads 1 for k=3 else 0)
//   types=fp32|u8f32u8f32|u8f32s8f32|u8f32f32f32
//   algo=auto|direct|1x1|wino   tile=6
//   relu bias sum                      0/1 fusion flags
//   iscale iz oscale oz sscale sz tscale tz      quantisation constants
//   xopt=0x.... blk_i blk_o flt_o flt_t pat_i pat_o pat_g nthreads      tuning knobs
//   wfmt=OIhw16i16o|goihw|oihw   ifmt=nChw16c|nchw   ofmt=nChw16c|nchw
//   input_file= weights_file= bias_file= output_in_file= output_file=
//                                      file paths (output_in_file preloads the output buffer,
//                                      needed when sum=1)
//   scratch_out= scratch_bytes=        use_scratch_pad with a caller buffer, dumped afterwards
//   iters=K warmup=W                   timed repetitions after the first (weight-transform) call
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cstdint>
#include <string>
#include <map>
#include <vector>
#include <chrono>
#include <algorithm>
#include "euler.hpp"

using namespace euler;

static std::map<std::string, std::string> args;

static bool has(const char *k) { return args.count(k) != 0; }
static long geti(const char *k, long dflt) {
  return has(k) ? strtol(args[k].c_str(), nullptr, 0) : dflt;
}
static double getf(const char *k, double dflt) {
  return has(k) ? atof(args[k].c_str()) : dflt;
}
static std::string gets(const char *k, const char *dflt) {
  return has(k) ? args[k] : std::string(dflt);
}

static void *alloc64(size_t bytes) {
  void *p = nullptr;
  if (posix_memalign(&p, 64, (bytes + 63) / 64 * 64 + 64) != 0) return nullptr;
  memset(p, 0, (bytes + 63) / 64 * 64 + 64);
  return p;
}

static bool read_file(const std::string &path, void *dst, size_t cap) {
  FILE *f = fopen(path.c_str(), "rb");
  if (!f) { fprintf(stderr, "ref_driver: cannot open %s\n", path.c_str()); return false; }
  size_t got = fread(dst, 1, cap, f);
  fclose(f);
  (void)got;
  return true;
}

static bool write_file(const std::string &path, const void *src, size_t bytes) {
  FILE *f = fopen(path.c_str(), "wb");
  if (!f) { fprintf(stderr, "ref_driver: cannot create %s\n", path.c_str()); return false; }
  size_t put = fwrite(src, 1, bytes, f);
  fclose(f);
  return put == bytes;
}

static int fmt_of(const std::string &s) {
  if (s == "nchw") return nchw;
  if (s == "nhwc") return nhwc;
  if (s == "nChw16c") return nChw16c;
  if (s == "oihw") return oihw;
  if (s == "hwio") return hwio;
  if (s == "OIhw16i16o") return OIhw16i16o;
  if (s == "goihw") return goihw;
  if (s == "ghwio") return ghwio;
  if (s == "gOIhw16i16o") return gOIhw16i16o;
  fprintf(stderr, "ref_driver: unknown format %s\n", s.c_str());
  exit(2);
}

int main(int argc, char **argv) {
  for (int i = 1; i < argc; ++i) {
    const char *eq = strchr(argv[i], '=');
    if (!eq) { fprintf(stderr, "ref_driver: bad argument %s\n", argv[i]); return 2; }
    args[std::string(argv[i], eq - argv[i])] = std::string(eq + 1);
  }

  eld_conv_t d;
  d.dims.n = geti("n", 1);
  d.dims.g = geti("g", 1);
  d.dims.ic = geti("ic", 16);
  d.dims.oc = geti("oc", 16);
  d.dims.ih = geti("ih", 8);
  d.dims.iw = geti("iw", d.dims.ih);
  d.dims.kh = geti("kh", 3);
  d.dims.kw = geti("kw", d.dims.kh);
  int dp = d.dims.kh / 2;
  d.pads.t = geti("pt", dp); d.pads.b = geti("pb", d.pads.t);
  d.pads.l = geti("pl", dp); d.pads.r = geti("pr", d.pads.l);
  d.strides.h = geti("sh", 1); d.strides.w = geti("sw", d.strides.h);
  d.dilations.h = 1; d.dilations.w = 1;
  d.dims.oh = geti("oh", (d.dims.ih + d.pads.t + d.pads.b - d.dims.kh) / d.strides.h + 1);
  d.dims.ow = geti("ow", (d.dims.iw + d.pads.l + d.pads.r - d.dims.kw) / d.strides.w + 1);

  std::string types = gets("types", "fp32");
  if (types == "fp32") {
    d.data_type.input = f32; d.data_type.weights = f32; d.data_type.output = f32; d.data_type.bias = f32;
  } else if (types == "u8f32u8f32") {
    d.data_type.input = u8; d.data_type.weights = f32; d.data_type.output = u8; d.data_type.bias = f32;
  } else if (types == "u8f32s8f32") {
    d.data_type.input = u8; d.data_type.weights = f32; d.data_type.output = s8; d.data_type.bias = f32;
  } else if (types == "u8f32f32f32") {
    d.data_type.input = u8; d.data_type.weights = f32; d.data_type.output = f32; d.data_type.bias = f32;
  } else {
    fprintf(stderr, "ref_driver: unknown types %s\n", types.c_str()); return 2;
  }
  d.formats.input = fmt_of(gets("ifmt", "nChw16c"));
  d.formats.weights = fmt_of(gets("wfmt", "OIhw16i16o"));
  d.formats.output = fmt_of(gets("ofmt", "nChw16c"));
  d.prop_kind = forward_inference;

  std::string algo = gets("algo", "auto");
  d.algorithm = algo == "direct" ? CONV_DIRECT : algo == "1x1" ? CONV_DIRECT_1X1
      : algo == "wino" ? CONV_WINOGRAD : CONV_AUTO;
  d.tile_size = geti("tile", 0);
  d.with_relu = geti("relu", 0) != 0;
  d.with_bias = geti("bias", 0) != 0;
  d.with_ip_sum = geti("sum", 0) != 0;
  d.with_op_sum = false;
  d.with_argmax = false;
  d.f16c_opt = false;
  d.is_inference = true;
  d.disable_autoparam = true;          // keep transform-domain buffers in fp32
  d.use_scratch_pad = false;
  d.scratch_pad = nullptr;
  d.eager_mode = true;
  d.stream_sync = false;
  d.nthreads = geti("nthreads", 0);
  d.execution_mode = geti("xopt", 0);
  d.flatting.o = geti("flt_o", 0); d.flatting.t = geti("flt_t", 0);
  d.blocking.i = geti("blk_i", 0); d.blocking.o = geti("blk_o", 0);
  d.partition.i = geti("pat_i", 1); d.partition.o = geti("pat_o", 1); d.partition.g = geti("pat_g", 1);
  d.streaming_hint.input = 0; d.streaming_hint.output = 0;
  d.input_quant.scale = has("iscale") ? (float)getf("iscale", 1) : EL_NO_CALI;
  d.input_quant.z = has("iscale") ? (float)getf("iz", 0) : EL_NO_CALI;
  d.output_quant.scale = has("oscale") ? (float)getf("oscale", 1) : EL_NO_CALI;
  d.output_quant.z = has("oscale") ? (float)getf("oz", 0) : EL_NO_CALI;
  d.sum_quant.scale = (float)getf("sscale", 1.0); d.sum_quant.z = (float)getf("sz", 0.0);
  d.wino_tinput_quant.scale = has("tscale") ? (float)getf("tscale", 1) : EL_NO_CALI;
  d.wino_tinput_quant.z = has("tscale") ? (float)getf("tz", 0) : EL_NO_CALI;
  d.sampling_kind = (d.data_type.input == u8) ? CALIBRATED : FINE;

  void *scratch = nullptr;
  size_t scratch_bytes = (size_t)geti("scratch_bytes", 0);
  if (has("scratch_out") && scratch_bytes) {
    scratch = alloc64(scratch_bytes);
    d.use_scratch_pad = true;
    d.scratch_pad = scratch;
  }

  int rc_setup = d.setup();
  if (rc_setup != ELD_OK || d.xc == nullptr) {
    printf("{\"rc_setup\": %d, \"rc\": -1}\n", rc_setup);
    return 1;
  }

  void *in = alloc64(d.byte_sizes.input), *w = alloc64(d.byte_sizes.weights);
  void *out = alloc64(d.byte_sizes.output), *b = alloc64(d.byte_sizes.bias);
  if (has("input_file") && !read_file(args["input_file"], in, d.byte_sizes.input)) return 2;
  if (has("weights_file") && !read_file(args["weights_file"], w, d.byte_sizes.weights)) return 2;
  if (has("bias_file") && !read_file(args["bias_file"], b, d.byte_sizes.bias)) return 2;
  std::vector<char> out_init;
  if (has("output_in_file")) {
    out_init.resize(d.byte_sizes.output);
    if (!read_file(args["output_in_file"], out_init.data(), d.byte_sizes.output)) return 2;
    memcpy(out, out_init.data(), d.byte_sizes.output);
  }

  // First call: weight transform happens here, so it is excluded from the timings.
  auto t0 = std::chrono::steady_clock::now();
  int rc = elx_conv(d, out, in, w, b);
  auto t1 = std::chrono::steady_clock::now();
  double first_ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
  if (has("output_file")) write_file(args["output_file"], out, d.byte_sizes.output);
  if (scratch) write_file(args["scratch_out"], scratch, scratch_bytes);

  int iters = geti("iters", 0), warmup = geti("warmup", 0);
  std::vector<double> ms;
  for (int i = 0; i < warmup + iters && rc == ELX_OK; ++i) {
    if (!out_init.empty()) memcpy(out, out_init.data(), d.byte_sizes.output);
    auto a = std::chrono::steady_clock::now();
    rc = elx_conv(d, out, in, w, b);
    auto z = std::chrono::steady_clock::now();
    if (i >= warmup) ms.push_back(std::chrono::duration<double, std::milli>(z - a).count());
  }
  double med = 0, mn = 0, sum = 0;
  if (!ms.empty()) {
    std::vector<double> s(ms); std::sort(s.begin(), s.end());
    med = s[s.size() / 2]; mn = s[0];
    for (double v : ms) sum += v;
  }
  printf("{\"rc_setup\": %d, \"rc\": %d, \"algorithm\": %d, \"tile_size\": %d, \"first_ms\": %.4f, "
         "\"iters\": %d, \"ms_median\": %.5f, \"ms_min\": %.5f, \"ms_total\": %.4f, "
         "\"bytes\": {\"input\": %zu, \"weights\": %zu, \"output\": %zu, \"bias\": %zu}}\n",
         rc_setup, rc, d.algorithm, d.tile_size, first_ms, (int)ms.size(), med, mn, sum,
         d.byte_sizes.input, d.byte_sizes.weights, d.byte_sizes.output, d.byte_sizes.bias);
  return rc == ELX_OK ? 0 : 1;
}
