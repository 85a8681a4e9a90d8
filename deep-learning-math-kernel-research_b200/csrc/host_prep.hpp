// Host-side, one-time weight preparation: quantisation and constant folding in exactly the
// reference's fp32 association order, and packing into the operand images the kernels copy with
// single bulk TMA transfers.  Plain scalar C++ on purpose: these few thousand operations define
// bit-exactness of every later output, so nothing here may be re-associated or fused except where
// the reference build itself fuses (written as an explicit fmaf).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <utility>
#include <vector>

namespace elb {
namespace host {

inline int alignup(int x, int a) { return (x + a - 1) / a * a; }

// OIhw16i16o index: [O/16][I/16][kh][kw][16 i][16 o]   (reference: src/elx_conv.hpp:10-12)
inline size_t w_index(int I2, int KH, int KW, int o, int i, int kh, int kw) {
  return (((((size_t)(o / 16) * I2 + i / 16) * KH + kh) * KW + kw) * 16 + i % 16) * 16 + o % 16;
}

struct I8Weights {
  int OCP = 0, ICP = 0, taps = 0;
  std::vector<int8_t> q;        // [OCP][taps][ICP]
  std::vector<float> absmax;    // [OCP]
  std::vector<int32_t> qsum;    // [OCP] sum of q over all taps and channels
  std::vector<int32_t> qsum_tap;   // [OCP][taps] sum of q over the channels of one tap
};

// Per output channel: absmax over the real input channels and all taps; q = rne((w*127)/absmax)
// (multiply, then divide), padded lanes 0.
// Reference: src/elx_int8_conv_direct_1x1.cpp:239-295, src/elx_int8_conv_direct.cpp:430-475.
inline I8Weights quantize_weights_i8(const float *w, int oc, int ic, int kh, int kw) {
  I8Weights r;
  r.OCP = alignup(oc, 16);
  r.ICP = alignup(ic, 16);
  r.taps = kh * kw;
  const int I2 = r.ICP / 16;
  r.q.assign((size_t)r.OCP * r.taps * r.ICP, 0);
  r.absmax.assign(r.OCP, 0.0f);
  r.qsum.assign(r.OCP, 0);
  r.qsum_tap.assign((size_t)r.OCP * r.taps, 0);
  for (int o = 0; o < r.OCP; ++o) {
    float m = 0.0f;
    for (int i = 0; i < ic; ++i)
      for (int a = 0; a < kh; ++a)
        for (int b = 0; b < kw; ++b) {
          const float v = std::fabs(w[w_index(I2, kh, kw, o, i, a, b)]);
          if (v > m) m = v;
        }
    r.absmax[o] = m;
    if (m == 0.0f) continue;
    int32_t s = 0;
    for (int a = 0; a < kh; ++a)
      for (int b = 0; b < kw; ++b)
        for (int i = 0; i < ic; ++i) {
          volatile float t = w[w_index(I2, kh, kw, o, i, a, b)] * 127.0f;   // volatile: keep the two
          volatile float u = t / m;                                        // roundings separate
          const int8_t qv = (int8_t)std::nearbyintf(u);
          r.q[((size_t)o * r.taps + a * kw + b) * r.ICP + i] = qv;
          r.qsum_tap[(size_t)o * r.taps + a * kw + b] += qv;
          s += qv;
        }
    r.qsum[o] = s;
  }
  return r;
}

// scale / shift of the requantising epilogue.
// Reference: src/elx_int8_conv_direct_1x1.cpp:316-353, src/elx_int8_conv_direct.cpp:357-419.
//   u8/s8 out: scale = (iS*Sw)*(1/oS); shift = fma(bias, 1/oS, oz) - (iz*Sq)*scale [- sum_z*sum_S]
//   f32  out: scale =  iS*Sw;         shift = bias - (iz*Sq)*scale
// qsum: the sum of q that the zero-point term uses, [OCP]; null = wq.qsum (every tap inside the image).
inline void fold_constants_i8(const I8Weights &wq, const float *bias, bool with_bias, bool out_f32,
                              float iS, float iz, float oS, float oz, bool with_sum, float sum_S,
                              float sum_z, std::vector<float> &scale, std::vector<float> &shift,
                              const int32_t *qsum = nullptr) {
  if (!qsum) qsum = wq.qsum.data();
  scale.assign(wq.OCP, 0.0f);
  shift.assign(wq.OCP, 0.0f);
  volatile float orepS = 1.0f / oS;
  for (int o = 0; o < wq.OCP; ++o) {
    volatile float Sw = wq.absmax[o] / 127.0f;
    const float b = (with_bias && bias) ? bias[o] : 0.0f;
    volatile float sc, sh;
    if (out_f32) {
      sc = iS * Sw;
      sh = b;
    } else {
      volatile float t = iS * Sw;
      sc = t * orepS;
      sh = std::fmaf(b, orepS, oz);
    }
    if (iz != 0.0f) {
      volatile float zq = iz * (float)qsum[o];
      volatile float zs = zq * sc;
      sh = sh - zs;
    }
    if (with_sum && !out_f32) {
      volatile float ss = sum_z * sum_S;
      sh = sh - ss;
    }
    scale[o] = sc;
    shift[o] = sh;
  }
}

// Output pixels near a padded border see fewer filter taps, and with a non-zero input zero point
// the shift of a pixel depends on WHICH taps lie inside the image: shift = ... - (iz * sum of q over
// those taps) * scale.  The reference keeps one shift vector per (range of kh, range of kw)
// (src/elx_int8_conv_direct.cpp:227-309 prepare_weights_acc, :311-423 __trans_weights_acc).  Here a
// class is the pair (first valid tap, last valid tap) along one axis; cls[o] is the class of output
// coordinate o and ranges[c] its tap range.  The class of coordinates that see every tap is `full`.
struct TapClasses {
  std::vector<int> cls;                          // [out extent]
  std::vector<std::pair<int, int>> ranges;       // [classes] first / last valid tap
  int full = -1;
};
inline TapClasses tap_classes(int out, int in, int k, int pad, int stride) {
  TapClasses t;
  t.cls.resize(out);
  for (int o = 0; o < out; ++o) {
    int lo = k, hi = -1;
    for (int a = 0; a < k; ++a) {
      const int i = o * stride - pad + a;
      if (i >= 0 && i < in) { lo = a < lo ? a : lo; hi = a; }
    }
    int c = -1;
    for (size_t j = 0; j < t.ranges.size(); ++j)
      if (t.ranges[j].first == lo && t.ranges[j].second == hi) c = (int)j;
    if (c < 0) { c = (int)t.ranges.size(); t.ranges.emplace_back(lo, hi); }
    if (lo == 0 && hi == k - 1) t.full = c;
    t.cls[o] = c;
  }
  return t;
}

// Operand image of B for the tcgen05 kernels: [n_tile][k_stage][KC chunks][BN rows][16 bytes].
// K runs over chunks q = tap*CB + cb of 16 input channels (tap-major); stage ks holds chunks
// ks*KC .. ks*KC+KC-1, zero where q is past the end of K or the row past the last output channel.
// halves = 2 (two-CTA kernel): the BN rows of a stage are stored as two images of BN/2 rows,
// [n_tile][k_stage][half][KC][BN/2][16], one per CTA of the pair.
inline std::vector<int8_t> pack_b_i8(const I8Weights &wq, int BN, int KC, int &n_tiles, int &CBG,
                                     int &k_stages, int halves = 1) {
  const int CB = wq.ICP / 16;
  const int Q = wq.taps * CB;
  n_tiles = (wq.OCP + BN - 1) / BN;
  CBG = (CB + KC - 1) / KC;
  k_stages = (Q + KC - 1) / KC;
  std::vector<int8_t> out((size_t)n_tiles * k_stages * KC * BN * 16, 0);
  for (int nt = 0; nt < n_tiles; ++nt)
    for (int ks = 0; ks < k_stages; ++ks)
      for (int j = 0; j < KC; ++j) {
        const int q = ks * KC + j;
        if (q >= Q) continue;
        const int tap = q / CB, cb = q % CB;
        for (int r = 0; r < BN; ++r) {
          const int o = nt * BN + r;
          if (o >= wq.OCP) continue;
          const int BH = BN / halves, h = r / BH, rr = r % BH;
          int8_t *dst = &out[(((((size_t)nt * k_stages + ks) * halves + h) * KC + j) * BH + rr) * 16];
          std::memcpy(dst, &wq.q[((size_t)o * wq.taps + tap) * wq.ICP + cb * 16], 16);
        }
      }
  return out;
}

}  // namespace host
}  // namespace elb
