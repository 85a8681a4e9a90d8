// INT8 depthwise 3x3 convolution (g = ic = oc; u8 activations, s8 weights, u8 / s8 output) for
// sm_100a.  Replaces elx_int8_conv_direct_depthwise_t (src/elx_int8_conv_direct_depthwise.cpp:14-318,
// src/elx_int8_conv_direct_depthwise_xopt.hpp:19-66) and its micro-kernel
// (src/kernel/elk_u8s8_depthwise_conv.hxx:288-474).
//
// The path is bandwidth-bound (9 multiply-adds per input byte at stride 1), so this is a CUDA-core
// kernel built around coalesced accesses and dp4a:
//   * one thread = 4 consecutive channels (one 32-bit word of an nChw16c pixel) x 4 output columns
//     x a strip of output rows; the four lanes of a pixel sit next to each other, so a warp touches
//     whole 16-byte pixels;
//   * the 4 x 4 byte block (4 pixels x 4 channels) a thread loads is transposed in registers with
//     byte permutes into per-channel words holding 4 horizontally adjacent pixels, which is exactly
//     the operand dp4a wants: one dp4a = one filter row of one output pixel of one channel (the
//     fourth tap weight is zero), as in the reference's VNNI formulation;
//   * transposed input rows are kept in registers and reused by the output rows below them.
// Out-of-image taps contribute zero (the reference skips them); the zero-point correction in
// `shift` uses the sum of all nine weights also at the border, as the reference does.
//
// Rounding follows the reference bit for bit.  Its u8 epilogue depends on the chunking of an output
// row into pieces of T = flatting.t pixels: the first 4*floor(L/4) pixels of a piece of length L
// are floored (round toward minus infinity, no saturation) and packed four at a time with
// additions that g++ compiles as 64-bit adds over channel pairs, the remaining L % 4 pixels are
// rounded to nearest even and saturated; s8 outputs are always rounded to nearest and saturated.
#include <cmath>
#include <cstdlib>
#include <string>
#include <vector>

#include "depthwise.cuh"
#include "elb_common.cuh"
#include "host_prep.hpp"

namespace elb {

namespace {

struct DwParams {
  const uint8_t *in;       // nChw16c u8
  const uint32_t *wq;      // [G][3]: bytes (w[kh][0], w[kh][1], w[kh][2], 0) of channel g, filter row kh
  const float *scale;      // [G]
  const float *shift;      // [G]
  void *out;               // nChw16c u8 / s8
  int32_t *acc_dump;       // optional nChw16c int32
  int N, CB, IH, IW, OH, OW, pad_t, pad_l;
  int T;                   // chunk length of an output row (OW when every pixel is rounded to nearest)
  int chunks;              // ceil(OW / T)
  int groups_full;         // floored 4-pixel groups in a full chunk  (T / 4, or 0 without floor mode)
  int floored_row;         // floored groups per output row
  int rest_row;            // nearest-rounded items per output row (chunk remainders, or ceil(OW/4))
  int rest_every_chunk;    // floor mode: 1 when full chunks have a remainder (T % 4 != 0)
  int rows_strip;          // output rows per thread
  int strips;              // ceil(OH / rows_strip)
  long long blocks_floored;   // blocks [0, blocks_floored) work on floored groups, the rest on nearest items
  int out_type, relu, floor_mode;   // floor_mode: u8 output with T >= 4
  float relu_lo, relu_hi;
};

__device__ __forceinline__ int dp4a_us(uint32_t a_u8x4, uint32_t b_s8x4, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_s8x4), "r"(c));
  return d;
}

// 4x4 byte transpose: in[k] = bytes (e0,e1,e2,e3) of item k  ->  out[e] = bytes (k0,k1,k2,k3) of element e
__device__ __forceinline__ void transpose4(const uint32_t (&in)[4], uint32_t (&out)[4]) {
  const uint32_t t0 = __byte_perm(in[0], in[1], 0x5140), t1 = __byte_perm(in[2], in[3], 0x5140);
  const uint32_t t2 = __byte_perm(in[0], in[1], 0x7362), t3 = __byte_perm(in[2], in[3], 0x7362);
  out[0] = __byte_perm(t0, t1, 0x5410);
  out[1] = __byte_perm(t0, t1, 0x7632);
  out[2] = __byte_perm(t2, t3, 0x5410);
  out[3] = __byte_perm(t2, t3, 0x7632);
}

// int32 result of the x86 float->int conversions for an already rounded value: anything that does
// not fit (and NaN) becomes INT_MIN.
__device__ __forceinline__ int cvt_x86(float rounded) {
  int r = __float2int_rz(rounded);
  if (!(rounded < 2147483648.0f)) r = static_cast<int>(0x80000000u);
  return r;
}

// One input row as a thread sees it: per-channel words of the pixel windows it needs.
template <int S> struct RowWin;
template <> struct RowWin<1> { uint32_t a[4], b[4]; };             // pixels base..base+3, base+2..base+5
template <> struct RowWin<2> { uint32_t a[4], b[4], c[4]; };       // base..+3, base+4..+7, (base+8, 0, 0, 0)

// col[k] = address of this thread's word of pixel base+k in row 0 of the plane, or null when the
// column lies outside the image (its taps then contribute zero)
template <int S>
__device__ __forceinline__ void load_row(const uint32_t *const (&col)[S == 1 ? 6 : 9], int ih, int IH, int row_words,
                                         RowWin<S> &w) {
  constexpr int NPIX = S == 1 ? 6 : 9;
  uint32_t px[NPIX];
  const bool row_ok = ih >= 0 && ih < IH;
  const size_t off = static_cast<size_t>(row_ok ? ih : 0) * row_words;
#pragma unroll
  for (int k = 0; k < NPIX; ++k) {
    px[k] = 0u;
    if (row_ok && col[k] != nullptr) px[k] = __ldg(col[k] + off);
  }
  if constexpr (S == 1) {
    const uint32_t wa[4] = {px[0], px[1], px[2], px[3]}, wb[4] = {px[2], px[3], px[4], px[5]};
    transpose4(wa, w.a);
    transpose4(wb, w.b);
  } else {
    const uint32_t wa[4] = {px[0], px[1], px[2], px[3]}, wb[4] = {px[4], px[5], px[6], px[7]};
    transpose4(wa, w.a);
    transpose4(wb, w.b);
#pragma unroll
    for (int c = 0; c < 4; ++c) w.c[c] = (px[NPIX - 1] >> (8 * c)) & 0xFFu;
  }
}

// Filter row of 4 channels in the alignments dp4a needs: f0 = (w0,w1,w2,0); stride 1: f1 = (0,w0,w1,w2);
// stride 2: f1 = (0,0,w0,w1), f2 = (w2,0,0,0).
struct FilterRow { uint32_t f0[4], f1[4], f2[4]; };

// acc[pixel][channel] += one filter row over one input row
template <int S>
__device__ __forceinline__ void mac_row(const RowWin<S> &w, const FilterRow &f, int (&acc)[4][4]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    if constexpr (S == 1) {
      acc[0][c] = dp4a_us(w.a[c], f.f0[c], acc[0][c]);       // pixels base+0..2
      acc[1][c] = dp4a_us(w.a[c], f.f1[c], acc[1][c]);       // base+1..3
      acc[2][c] = dp4a_us(w.b[c], f.f0[c], acc[2][c]);       // base+2..4
      acc[3][c] = dp4a_us(w.b[c], f.f1[c], acc[3][c]);       // base+3..5
    } else {
      acc[0][c] = dp4a_us(w.a[c], f.f0[c], acc[0][c]);       // base+0..2
      acc[1][c] = dp4a_us(w.a[c], f.f1[c], acc[1][c]);       // base+2,3 ...
      acc[1][c] = dp4a_us(w.b[c], f.f2[c], acc[1][c]);       // ... and base+4
      acc[2][c] = dp4a_us(w.b[c], f.f0[c], acc[2][c]);       // base+4..6
      acc[3][c] = dp4a_us(w.b[c], f.f1[c], acc[3][c]);       // base+6,7 ...
      acc[3][c] = dp4a_us(w.c[c], f.f2[c], acc[3][c]);       // ... and base+8
    }
  }
}

// Two-lane fp32 arithmetic (each lane rounds exactly as the scalar instruction with the same
// rounding mode does): the epilogue below is bound by instruction issue.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 add2_rm(f32x2 a, f32x2 b) {      // round toward minus infinity
  f32x2 d;
  asm("add.rm.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

#ifndef DW_MIN_BLOCKS
#define DW_MIN_BLOCKS 3      // resident 256-thread blocks per SM the register allocation must allow
#endif
constexpr uint32_t MAGIC_BITS = 0x4B400000u;      // bit pattern of 1.5 * 2^23
constexpr float MAGIC = 12582912.0f;              // 1.5 * 2^23: float(MAGIC_BITS + i) == MAGIC + i for |i| < 2^22

// FAST: every value the epilogue can produce is known (from the folded constants) to lie inside
// (-2^22, 2^22), and either the output is s8 or ReLU with a non-negative lower bound is on.  Then
// int <-> float conversions can be done exactly on the FMA pipe by adding 1.5 * 2^23 (the
// accumulators even start at that bit pattern), rounding toward minus infinity is an add with
// the .rm modifier, and a floored group whose four values all fit a byte is packed with three
// multiply-adds; a group with a value above 255 (possible only with an overflowing output scale)
// takes the exact 64-bit path of the general epilogue instead.
template <int S, bool FAST>
__global__ void __launch_bounds__(256, DW_MIN_BLOCKS) dw_kernel(const __grid_constant__ DwParams p) {
  const int quad = threadIdx.x & 3;
  // Blocks are split by rounding rule so that a warp never has to run both epilogues.
  const bool floored = static_cast<long long>(blockIdx.x) < p.blocks_floored;
  const int per_row = floored ? p.floored_row : p.rest_row;
  // (the host refuses problems whose item count does not fit 31 bits)
  const unsigned per_plane = static_cast<unsigned>(p.strips) * per_row;
  const unsigned lin = (floored ? blockIdx.x : blockIdx.x - static_cast<unsigned>(p.blocks_floored)) * 64u + (threadIdx.x >> 2);
  if (lin >= per_plane * static_cast<unsigned>(p.N * p.CB)) return;
  const int plane_idx = static_cast<int>(lin / per_plane);
  const int rem = static_cast<int>(lin - plane_idx * per_plane);
  const int strip = rem / per_row;
  const int item = rem - strip * per_row;
  int x0, width;
  if (floored) {
    const int chunk = min(item / p.groups_full, p.chunks - 1);        // the last chunk may hold fewer groups
    x0 = chunk * p.T + 4 * (item - chunk * p.groups_full);
    width = 4;
  } else if (p.floor_mode) {
    // remainder of a chunk: the L % 4 pixels behind its floored groups
    const int chunk = p.rest_every_chunk ? item : p.chunks - 1;
    const int L = min(p.T, p.OW - chunk * p.T);
    x0 = chunk * p.T + (L & ~3);
    width = L & 3;
  } else {
    x0 = 4 * item;
    width = min(4, p.OW - x0);
  }
  const int n = plane_idx / p.CB, cb = plane_idx - n * p.CB;
  const int ch0 = cb * 16 + quad * 4;

  FilterRow filt[3];
  float sc[4], sh[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int kh = 0; kh < 3; ++kh) {
      const uint32_t f = __ldg(p.wq + (ch0 + c) * 3 + kh);
      filt[kh].f0[c] = f;
      filt[kh].f1[c] = S == 1 ? f << 8 : f << 16;
      filt[kh].f2[c] = (f >> 16) & 0xFFu;
    }
    sc[c] = __ldg(p.scale + ch0 + c);
    sh[c] = __ldg(p.shift + ch0 + c);
  }

  constexpr int NPIX = S == 1 ? 6 : 9;
  const int base = x0 * S - p.pad_l;
  const uint32_t *plane = reinterpret_cast<const uint32_t *>(p.in + static_cast<size_t>(plane_idx) * p.IH * p.IW * 16) + quad;
  const uint32_t *col[NPIX];
#pragma unroll
  for (int k = 0; k < NPIX; ++k) {
    const int iw = base + k;
    col[k] = (iw >= 0 && iw < p.IW) ? plane + iw * 4 : nullptr;
  }
  const int row_words = p.IW * 4;
  const int oh0 = strip * p.rows_strip;
  const int oh1 = min(p.OH, oh0 + p.rows_strip);
  const bool clamp_hi = p.relu_hi < 3.0e38f;
  constexpr int ACC0 = FAST ? static_cast<int>(MAGIC_BITS) : 0;
  // rows[k] = input row oh*S - pad_t + k of the current output row
  RowWin<S> rows[3];
  load_row<S>(col, oh0 * S - p.pad_t, p.IH, row_words, rows[0]);
  if constexpr (S == 1) load_row<S>(col, oh0 * S - p.pad_t + 1, p.IH, row_words, rows[1]);

  for (int oh = oh0; oh < oh1; ++oh) {
    const int ih0 = oh * S - p.pad_t;
    if constexpr (S == 1) {
      load_row<S>(col, ih0 + 2, p.IH, row_words, rows[2]);
    } else {
      load_row<S>(col, ih0 + 1, p.IH, row_words, rows[1]);
      load_row<S>(col, ih0 + 2, p.IH, row_words, rows[2]);
    }
    int acc[4][4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[k][c] = ACC0;
#pragma unroll
    for (int kh = 0; kh < 3; ++kh) mac_row<S>(rows[kh], filt[kh], acc);

    // ---- epilogue: f = fma(acc, scale, shift), ReLU clamp, round, pack, transpose back, store
    const size_t opix = (static_cast<size_t>(plane_idx) * p.OH + oh) * p.OW + x0;
    if (p.acc_dump) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (k < width)
          *reinterpret_cast<int4 *>(p.acc_dump + (opix + k) * 16 + quad * 4) =
              make_int4(acc[k][0] - ACC0, acc[k][1] - ACC0, acc[k][2] - ACC0, acc[k][3] - ACC0);
    }
    float f[4][4];
    if (FAST) {
      // channel pairs: (acc - magic) * scale + shift in two packed instructions per pair
      const f32x2 magic2 = pack2(MAGIC, MAGIC);
      const f32x2 sc2[2] = {pack2(sc[0], sc[1]), pack2(sc[2], sc[3])}, sh2[2] = {pack2(sh[0], sh[1]), pack2(sh[2], sh[3])};
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const f32x2 a = sub2(pack2(__int_as_float(acc[k][2 * c]), __int_as_float(acc[k][2 * c + 1])), magic2);
          unpack2(fma2(a, sc2[c], sh2[c]), f[k][2 * c], f[k][2 * c + 1]);
        }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int c = 0; c < 4; ++c) f[k][c] = __fmaf_rn(__int2float_rn(acc[k][c]), sc[c], sh[c]);
    }
    if (p.relu) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          f[k][c] = fmaxf(f[k][c], p.relu_lo);
          if (clamp_hi) f[k][c] = fminf(f[k][c], p.relu_hi);
        }
    }
    uint32_t cw[4] = {0u, 0u, 0u, 0u};       // per channel: bytes = pixels 0..3
    bool packed = false;
    if (FAST) {
      if (floored) {
        uint32_t any = 0u, bits[4][4];
        const f32x2 magic2 = pack2(MAGIC, MAGIC);
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            float b0, b1;
            unpack2(add2_rm(pack2(f[k][2 * c], f[k][2 * c + 1]), magic2), b0, b1);     // MAGIC_BITS + floor(f)
            bits[k][2 * c] = __float_as_uint(b0);
            bits[k][2 * c + 1] = __float_as_uint(b1);
            any |= bits[k][2 * c] | bits[k][2 * c + 1];
          }
        if ((any & 0x003FFF00u) == 0u) {      // all sixteen floored values fit a byte: no carries anywhere
#pragma unroll
          for (int c = 0; c < 4; ++c)
            cw[c] = bits[0][c] + (bits[1][c] << 8) + (bits[2][c] << 16) + (bits[3][c] << 24) -
                    MAGIC_BITS * 0x01010101u;
          packed = true;
        }
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t b[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int r = static_cast<int>(__float_as_uint(__fadd_rn(f[k][c], MAGIC)));   // MAGIC_BITS + rne(f)
            b[k] = static_cast<uint32_t>(p.out_type == OUT_U8
                                             ? min(r, static_cast<int>(MAGIC_BITS) + 255)
                                             : max(static_cast<int>(MAGIC_BITS) - 128, min(static_cast<int>(MAGIC_BITS) + 127, r)));
          }
          // low bytes of the four words (the low byte of MAGIC_BITS is zero)
          cw[c] = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
        }
        packed = true;
      }
    }
    if (!packed) {
      if (floored) {
        // word = u0 + (u1 << 8) + (u2 << 16) + (u3 << 24) with 64-bit adds over channel pairs
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          unsigned long long sum = 0ull;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t lo = static_cast<uint32_t>(cvt_x86(floorf(f[k][2 * e]))) << (8 * k);
            const uint32_t hi = static_cast<uint32_t>(cvt_x86(floorf(f[k][2 * e + 1]))) << (8 * k);
            sum += static_cast<unsigned long long>(lo) | (static_cast<unsigned long long>(hi) << 32);
          }
          cw[2 * e] = static_cast<uint32_t>(sum);
          cw[2 * e + 1] = static_cast<uint32_t>(sum >> 32);
        }
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int r = cvt_x86(rintf(f[k][c]));
            uint32_t b;
            if (p.out_type == OUT_U8) b = static_cast<uint32_t>(r) > 255u ? 255u : static_cast<uint32_t>(r);
            else b = static_cast<uint32_t>(max(-128, min(127, r))) & 0xFFu;
            cw[c] |= b << (8 * k);
          }
      }
    }
    uint32_t pw[4];
    transpose4(cw, pw);
    uint32_t *dst = reinterpret_cast<uint32_t *>(static_cast<uint8_t *>(p.out) + opix * 16) + quad;
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (k < width) dst[k * 4] = pw[k];

    // slide the window of input rows down
    if constexpr (S == 1) { rows[0] = rows[1]; rows[1] = rows[2]; }
    else { rows[0] = rows[2]; }
  }
}

}  // namespace

struct DwImpl {
  DwParams p{};
  int stride = 1;
  int G = 0;
  bool fast = false;       // epilogue values provably inside (-2^22, 2^22), see dw_kernel
  void *d_wq = nullptr, *d_scale = nullptr, *d_shift = nullptr;
};

int dw_setup(DwPlan &pl, const elb_conv_desc_t &d, elb_conv_info_t &info, int num_sms, std::string &err) {
  // shapes the reference accepts (src/elx_int8_conv_direct_depthwise.cpp:28-40, 88-94)
  if (d.kh != 3 || d.kw != 3 || d.stride_h != d.stride_w || (d.stride_h != 1 && d.stride_h != 2) ||
      d.pad_l < 0 || d.pad_l > 1 || d.pad_r > 1 || d.pad_t < 0 || d.pad_t > 1 || d.pad_b > 1) {
    err = "direct_depthwise: int8: shape not supported";
    return ELB_UNIMPLEMENTED;
  }
  if (d.fmt_weights != ELB_GOIHW) { err = "direct_depthwise: weights must be goihw"; return ELB_UNIMPLEMENTED; }
  if (d.sampling_kind != ELB_CALIBRATED) { err = "Unsupported quantization mode in int8 direct 1x1"; return ELB_UNIMPLEMENTED; }
  if (d.dt_output != ELB_U8 && d.dt_output != ELB_S8) { err = "direct_depthwise: output must be u8 or s8"; return ELB_UNIMPLEMENTED; }
  const int T = d.flatting_t > 0 ? d.flatting_t : 1;                    // :73 (T == 0 -> 1)
  const int Tr = d.ow % T ? d.ow % T : T;                               // :79
  if (T < d.pad_l || Tr < d.pad_r) { err = "direct_depthwise: (T,Tr) < (lp,rp)"; return ELB_GENERAL_ERROR; }   // :84-86
  // Chunkings for which the reference kernel accumulates one pixel twice or reads in front of the
  // row (stride 2 with a one-pixel chunk: the "left" and "right" steps of
  // src/kernel/elk_u8s8_depthwise_conv.hxx:374-398 both address pixel 0; stride 1 with ow == 1
  // likewise, :357-371): there is no defined result to reproduce.
  if ((d.stride_h == 2 && (T == 1 || Tr == 1)) || (d.stride_h == 1 && d.ow == 1)) {
    err = "direct_depthwise: a one-pixel chunk (flatting.t or its remainder = 1) is not supported with this stride";
    return ELB_UNIMPLEMENTED;
  }
  DwImpl *w = new DwImpl();
  pl.impl = w;
  w->stride = d.stride_h;
  w->G = host::alignup(d.g, V);
  DwParams &p = w->p;
  p.N = d.n; p.CB = w->G / V; p.IH = d.ih; p.IW = d.iw; p.OH = d.oh; p.OW = d.ow;
  p.pad_t = d.pad_t; p.pad_l = d.pad_l;
  p.out_type = d.dt_output == ELB_U8 ? OUT_U8 : OUT_S8;
  p.relu = d.with_relu; p.relu_lo = d.relu_lower; p.relu_hi = d.relu_upper;
  p.floor_mode = (p.out_type == OUT_U8 && T >= 4) ? 1 : 0;
  p.T = p.floor_mode ? T : d.ow;       // without floored groups the chunking has no effect
  p.chunks = (d.ow + p.T - 1) / p.T;
  const int last = d.ow - (p.chunks - 1) * p.T;           // length of the last chunk
  if (p.floor_mode) {
    p.groups_full = p.T / 4;
    p.floored_row = (p.chunks - 1) * p.groups_full + last / 4;
    p.rest_every_chunk = (p.T % 4) != 0;
    p.rest_row = p.rest_every_chunk ? (p.chunks - 1) + ((last % 4) != 0) : ((last % 4) != 0);
  } else {
    p.groups_full = 1;
    p.floored_row = 0;
    p.rest_every_chunk = 0;
    p.rest_row = (d.ow + 3) / 4;
  }
  // rows per thread: input rows are reused down a strip (2 extra rows per strip at stride 1), but
  // short strips keep many more threads in flight; 4 to 7 rows measured best on B200
  int rs = d.oh >= 28 ? 7 : 4;
  if (d.oh < rs) rs = d.oh;
  {
    const int v = tune_env("ELB_DW_ROWS", rs);
    if (v >= 1 && v <= 64) rs = v;
  }
  p.rows_strip = rs;
  p.strips = (d.oh + rs - 1) / rs;
  p.blocks_floored = (static_cast<long long>(d.n) * p.CB * p.strips * p.floored_row + 63) / 64;
  info.launches_per_call = 1;
  return ELB_OK;
}

int dw_prepare(DwPlan &pl, const elb_conv_desc_t &d, elb_conv_info_t &info, const void *weights,
               const void *bias, std::string &err) {
  DwImpl *w = pl.impl;
  if (!w) { err = "plan not set up"; return ELB_GENERAL_ERROR; }
  const int G = w->G, g = d.g;
  std::vector<float> hw(static_cast<size_t>(g) * 9), hb(G, 0.0f);
  cudaError_t e = cudaMemcpy(hw.data(), weights, hw.size() * 4, cudaMemcpyDefault);
  if (e == cudaSuccess && d.with_bias) {
    if (!bias) { err = "bias is null but with_bias is set"; return ELB_GENERAL_ERROR; }
    e = cudaMemcpy(hb.data(), bias, static_cast<size_t>(g) * 4, cudaMemcpyDefault);
  }
  if (e != cudaSuccess) { err = std::string("cudaMemcpy: ") + cudaGetErrorString(e); return ELB_GENERAL_ERROR; }
  // src/elx_int8_conv_direct_depthwise.cpp:202-292, in its association order
  std::vector<uint32_t> wq(static_cast<size_t>(G) * 3, 0u);
  std::vector<float> scale(G, 0.0f), shift(G, 0.0f);
  volatile float orepS = 1.0f / d.output_scale;
  for (int c = 0; c < g; ++c) {
    float m = 0.0f;
    for (int k = 0; k < 9; ++k) m = std::fmax(m, std::fabs(hw[c * 9 + k]));
    int sq = 0;
    for (int kh = 0; kh < 3; ++kh) {
      uint32_t word = 0;
      for (int kw = 0; kw < 3; ++kw) {
        volatile float t = hw[c * 9 + kh * 3 + kw] * 127.0f;
        volatile float u = t / m;
        const int8_t q = m != 0.0f ? static_cast<int8_t>(std::rint(u)) : 0;
        sq += q;
        word |= static_cast<uint32_t>(static_cast<uint8_t>(q)) << (8 * kw);
      }
      wq[c * 3 + kh] = word;
    }
    volatile float Sw = m / 127.0f;
    volatile float qs = d.input_scale * Sw;
    qs = qs * orepS;
    const float b = d.with_bias ? hb[c] : 0.0f;
    const float t0 = std::fmaf(b, orepS, d.output_z);
    volatile float zq = d.input_z * static_cast<float>(sq);
    scale[c] = qs;
    shift[c] = std::fmaf(-zq, qs, t0);
  }
  for (void **ptr : {&w->d_wq, &w->d_scale, &w->d_shift}) {
    const size_t bytes = ptr == &w->d_wq ? wq.size() * 4 : static_cast<size_t>(G) * 4;
    if (cudaMalloc(ptr, bytes) != cudaSuccess) { err = "cudaMalloc failed"; return ELB_GENERAL_ERROR; }
    info.workspace_bytes += bytes;
  }
  if (cudaMemcpy(w->d_wq, wq.data(), wq.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess ||
      cudaMemcpy(w->d_scale, scale.data(), static_cast<size_t>(G) * 4, cudaMemcpyHostToDevice) != cudaSuccess ||
      cudaMemcpy(w->d_shift, shift.data(), static_cast<size_t>(G) * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
    err = "cudaMemcpy of the depthwise constants failed";
    return ELB_GENERAL_ERROR;
  }
  // largest magnitude the epilogue can see: |acc| <= 9 * 255 * 127
  float bound = 0.0f;
  for (int c = 0; c < g; ++c) bound = std::fmax(bound, 291465.0f * std::fabs(scale[c]) + std::fabs(shift[c]));
  w->fast = bound < 4194304.0f &&
            (w->p.out_type == OUT_S8 || (d.with_relu && d.relu_lower >= 0.0f));
  w->p.wq = static_cast<const uint32_t *>(w->d_wq);
  w->p.scale = static_cast<const float *>(w->d_scale);
  w->p.shift = static_cast<const float *>(w->d_shift);
  return ELB_OK;
}

int dw_run(DwPlan &pl, void *out, const void *in, void *acc_dump, int first, int count, cudaStream_t s, int &launches,
           std::string &err) {
  DwImpl *w = pl.impl;
  launches = 0;
  if (!w) { err = "plan not set up"; return ELB_GENERAL_ERROR; }
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) {
    err = "input/output tensors must be 16-byte aligned";
    return ELB_GENERAL_ERROR;
  }
  DwParams p = w->p;
  if (first < 0 || count <= 0 || first + count > p.N) { err = "image range outside the batch"; return ELB_GENERAL_ERROR; }
  const size_t in_img = static_cast<size_t>(p.CB) * p.IH * p.IW * 16, out_img = static_cast<size_t>(p.CB) * p.OH * p.OW * 16;
  p.in = static_cast<const uint8_t *>(in) + first * in_img;
  p.out = static_cast<uint8_t *>(out) + first * out_img;
  p.acc_dump = acc_dump ? static_cast<int32_t *>(acc_dump) + first * out_img : nullptr;
  p.N = count;
  p.blocks_floored = (static_cast<long long>(count) * p.CB * p.strips * p.floored_row + 63) / 64;
  const long long blocks_rest = (static_cast<long long>(p.N) * p.CB * p.strips * p.rest_row + 63) / 64;
  if ((p.blocks_floored + blocks_rest) * 64 > 0x7FFFFFFFll) { err = "depthwise: problem too large for one launch"; return ELB_UNIMPLEMENTED; }
  dim3 grid(static_cast<unsigned>(p.blocks_floored + blocks_rest));
  if (w->stride == 1) {
    if (w->fast) dw_kernel<1, true><<<grid, 256, 0, s>>>(p);
    else dw_kernel<1, false><<<grid, 256, 0, s>>>(p);
  } else {
    if (w->fast) dw_kernel<2, true><<<grid, 256, 0, s>>>(p);
    else dw_kernel<2, false><<<grid, 256, 0, s>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { err = std::string("depthwise launch failed: ") + cudaGetErrorString(e); return ELB_GENERAL_ERROR; }
  launches = 1;
  return ELB_OK;
}

void dw_release(DwPlan &pl) {
  DwImpl *w = pl.impl;
  if (!w) return;
  for (void *p : {w->d_wq, w->d_scale, w->d_shift})
    if (p) cudaFree(p);
  delete w;
  pl.impl = nullptr;
}

}  // namespace elb
