/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement ("oracle") of the reference's convolution hot paths.
 *
 * Nothing the product ships links, imports or calls this file.  It exists so that the CUDA kernels
 * can be compared, bit for bit (integer paths) or within a stated tolerance (fp32 paths), with an
 * independent scalar statement of the reference's arithmetic, and it is itself pinned against the
 * reference library built from its own sources (oracle/build_ref.sh -> oracle/_ref/libel.so) by
 * tests/test_oracle_vs_reference.py and by the committed fixtures under tests/golden/.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC (see oracle/Makefile).  Contraction is
 * switched off on purpose: every place where the reference build (g++ -O2 -mfma, which contracts
 * a*b+c written with vector operators into one fused multiply-add) fuses is written here as an
 * explicit fmaf(), and every place where it cannot fuse stays a rounded multiply followed by a
 * rounded add.
 *
 * Layouts (slowest -> fastest), V = 16:
 *   nChw16c     [n][C/16][h][w][16]
 *   OIhw16i16o  [OC/16][IC/16][kh][kw][16 ic][16 oc]
 *   goihw (depthwise, g = channels): [g][1][1][kh][kw]
 *
 * Citations are file:line inside the reference project.
 */
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#include <float.h>

#define V 16
#define ALIGNUP(x, a) (((x) + (a) - 1) / (a) * (a))

enum { ORC_F32 = 0, ORC_U8 = 1, ORC_S8 = 2 };

typedef struct orc_conv {
  int32_t n, ic, oc, ih, iw, oh, ow, kh, kw;
  int32_t pad_t, pad_l, stride_h, stride_w;
  int32_t with_relu, with_bias, with_sum;
  int32_t out_type;          /* ORC_F32 / ORC_U8 / ORC_S8 */
  float relu_lo, relu_hi;    /* include/euler.hpp:150 (defaults 0, FLT_MAX) */
  float in_scale, in_z;      /* x = scale * (q - z), include/euler.hpp:166-168 */
  float out_scale, out_z;
  float sum_scale, sum_z;
  float tin_scale, tin_z;    /* wino_tinput_quant */
  int32_t fused_epilogue;    /* 1: acc*scale+shift is one fma (what g++ -mfma emits) */
  int32_t tile;              /* Winograd tile_size A: 6 (or 0) = F(4x4,3x3), 4 = F(2x2,3x3) */
} orc_conv_t;

/* Winograd geometry: A = input tile edge, A - 2 = output tile edge */
static inline int wino_A(const orc_conv_t *p) { return p->tile == 4 ? 4 : 6; }
static inline int wino_ht(const orc_conv_t *p) { int o = wino_A(p) - 2; return (p->oh + o - 1) / o; }
static inline int wino_wt(const orc_conv_t *p) { int o = wino_A(p) - 2; return (p->ow + o - 1) / o; }

/* round to nearest even, the mode of _MM_FROUND_TO_NEAREST_INT */
static inline float rne(float x) { return nearbyintf(x); }

static inline size_t in_index(const orc_conv_t *p, int n, int c, int h, int w) {
  int C2 = ALIGNUP(p->ic, V) / V;
  return ((((size_t)n * C2 + c / V) * p->ih + h) * p->iw + w) * V + c % V;
}
static inline size_t out_index(const orc_conv_t *p, int n, int c, int h, int w) {
  int C2 = ALIGNUP(p->oc, V) / V;
  return ((((size_t)n * C2 + c / V) * p->oh + h) * p->ow + w) * V + c % V;
}
static inline size_t w_index(const orc_conv_t *p, int o, int i, int kh, int kw) {
  int I2 = ALIGNUP(p->ic, V) / V;
  return (((((size_t)(o / V) * I2 + i / V) * p->kh + kh) * p->kw + kw) * V + i % V) * V + o % V;
}

/* ------------------------------------------------------------------------------------------
 * INT8 direct convolution (1x1 and KxK), user types u8 / f32 weights / {u8,s8,f32} / f32 bias.
 *
 * Weight quantisation: per output channel abs-max over the REAL ic (and kh,kw), then
 *   q = (int8) rne((w * 127) / absmax)      -- multiply first, then divide
 *   Sw = absmax / 127
 * src/elx_int8_conv_direct_1x1.cpp:239-322 (1x1), src/elx_int8_conv_direct.cpp:427-497 (KxK).
 * Folded constants (1x1 :325-353, KxK src/elx_int8_conv_direct.cpp:357-419):
 *   u8/s8 out: scale = (iS*Sw)*(1/oS);  shift = fma(bias, 1/oS, oz) - ((iz*Sq)*scale)
 *   f32  out: scale =  iS*Sw;          shift = bias - ((iz*Sq)*scale)
 *   with sum (1x1 only): shift -= sum_z*sum_S
 * where Sq = sum of q over the taps that fall inside the image for that output position (for a
 * 1x1 filter: all ic).  Padding taps are skipped, i.e. they contribute 0, not z
 * (src/kernel/elk_u8s8_conv.hxx:566-661).
 * ------------------------------------------------------------------------------------------ */
void orc_int8_quantize_weights(const orc_conv_t *p, const float *w, int8_t *q /* [oc][kh][kw][IC] */,
                               float *absmax /* [OC] */) {
  int IC = ALIGNUP(p->ic, V), OC = ALIGNUP(p->oc, V);
  for (int o = 0; o < OC; ++o) {
    float m = 0.0f;
    for (int i = 0; i < p->ic; ++i)
      for (int kh = 0; kh < p->kh; ++kh)
        for (int kw = 0; kw < p->kw; ++kw) {
          float a = fabsf(w[w_index(p, o, i, kh, kw)]);
          if (a > m) m = a;
        }
    absmax[o] = m;
    for (int kh = 0; kh < p->kh; ++kh)
      for (int kw = 0; kw < p->kw; ++kw)
        for (int i = 0; i < IC; ++i) {
          int8_t v = 0;
          if (i < p->ic && m != 0.0f) {
            float t = w[w_index(p, o, i, kh, kw)] * 127.0f;
            t = t / m;
            v = (int8_t)rne(t);
          }
          q[(((size_t)o * p->kh + kh) * p->kw + kw) * IC + i] = v;
        }
  }
}

/* scale[OC]; shift depends on the output position only when in_z != 0, so it is returned through
 * a callback-free formulation: shift0[OC] is the part without the zero-point term. */
void orc_int8_fold_constants(const orc_conv_t *p, const float *absmax, const float *bias,
                             float *scale, float *shift0) {
  int OC = ALIGNUP(p->oc, V);
  float orepS = 1.0f / p->out_scale;
  for (int o = 0; o < OC; ++o) {
    float Sw = absmax[o] / 127.0f;
    float b = (p->with_bias && bias) ? bias[o] : 0.0f;
    if (p->out_type == ORC_F32) {
      scale[o] = p->in_scale * Sw;
      shift0[o] = b;
    } else {
      scale[o] = (p->in_scale * Sw) * orepS;
      shift0[o] = fmaf(b, orepS, p->out_z);
    }
  }
}

static inline float requant_tail(const orc_conv_t *p, float f, const void *prev, size_t idx) {
  if (p->with_sum && prev && p->out_type != ORC_F32) {
    /* src/kernel/elk_u8s8_gemm.hxx:221-237: f += (float)prev * sum_S  (one fma in the g++ build) */
    float pv = p->out_type == ORC_U8 ? (float)((const uint8_t *)prev)[idx]
                                     : (float)((const int8_t *)prev)[idx];
    f = p->fused_epilogue ? fmaf(pv, p->sum_scale, f) : f + pv * p->sum_scale;
  }
  if (p->with_relu) {            /* elk_u8s8_gemm.hxx:240-245 */
    f = f > p->relu_lo ? f : p->relu_lo;     /* max_ps(f, lower) */
    f = f < p->relu_hi ? f : p->relu_hi;     /* min_ps(f, upper) */
  }
  return f;
}

static inline void store_q(const orc_conv_t *p, void *out, size_t idx, float f) {
  if (p->out_type == ORC_F32) {
    ((float *)out)[idx] = f;
    return;
  }
  /* cvt_roundps_epi32 (nearest even); out-of-range floats give INT_MIN (0x80000000) */
  int32_t r;
  float rf = rne(f);
  if (!(rf >= -2147483648.0f && rf < 2147483648.0f)) r = INT32_MIN; else r = (int32_t)rf;
  if (p->out_type == ORC_S8) {
    /* cvtsepi32_epi8: signed saturation */
    ((int8_t *)out)[idx] = (int8_t)(r > 127 ? 127 : r < -128 ? -128 : r);
  } else {
    /* cvtusepi32_epi8: the int32 is read as UNSIGNED, so a negative value saturates to 255
     * (src/kernel/elk_u8s8_gemm.hxx:247-256) */
    uint32_t u = (uint32_t)r;
    ((uint8_t *)out)[idx] = (uint8_t)(u > 255u ? 255u : u);
  }
}

/* out: nChw16c of out_type; acc_dump (optional): nChw16c int32 raw accumulators;
 * prev (optional, with_sum): the output tensor's previous contents. */
int orc_int8_conv(const orc_conv_t *p, const uint8_t *in, const float *w, const float *bias,
                  void *out, int32_t *acc_dump, const void *prev) {
  int IC = ALIGNUP(p->ic, V), OC = ALIGNUP(p->oc, V);
  int8_t *q = (int8_t *)malloc((size_t)OC * p->kh * p->kw * IC);
  float *absmax = (float *)malloc(sizeof(float) * OC);
  float *scale = (float *)malloc(sizeof(float) * OC);
  float *shift0 = (float *)malloc(sizeof(float) * OC);
  if (!q || !absmax || !scale || !shift0) return -1;
  orc_int8_quantize_weights(p, w, q, absmax);
  orc_int8_fold_constants(p, absmax, bias, scale, shift0);
  float sum_term = p->with_sum ? p->sum_z * p->sum_scale : 0.0f;

#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < p->n; ++n)
    for (int o = 0; o < OC; ++o) {
      for (int oh = 0; oh < p->oh; ++oh)
        for (int ow = 0; ow < p->ow; ++ow) {
          int32_t acc = 0, sq = 0;
          for (int kh = 0; kh < p->kh; ++kh) {
            int ih = oh * p->stride_h - p->pad_t + kh;
            if (ih < 0 || ih >= p->ih) continue;
            for (int kw = 0; kw < p->kw; ++kw) {
              int iw = ow * p->stride_w - p->pad_l + kw;
              if (iw < 0 || iw >= p->iw) continue;
              const int8_t *qq = q + (((size_t)o * p->kh + kh) * p->kw + kw) * IC;
              for (int i = 0; i < p->ic; ++i) {
                acc += (int32_t)in[in_index(p, n, i, ih, iw)] * (int32_t)qq[i];
                sq += qq[i];
              }
            }
          }
          size_t idx = out_index(p, n, o, oh, ow);
          if (acc_dump) acc_dump[idx] = acc;
          float shift = shift0[o];
          if (p->in_z != 0.0f) shift = shift - (p->in_z * (float)sq) * scale[o];
          if (p->with_sum) shift -= sum_term;
          float f = p->fused_epilogue ? fmaf((float)acc, scale[o], shift)
                                      : (float)acc * scale[o] + shift;
          f = requant_tail(p, f, prev, idx);
          store_q(p, out, idx, f);
        }
    }
  free(q); free(absmax); free(scale); free(shift0);
  return 0;
}

/* ------------------------------------------------------------------------------------------
 * Winograd F(4x4,3x3) (reference tile_size = 6).
 *
 * 1-D input transform B^T, written in the reference's evaluation order with its six constants
 * (src/kernel/elk_conv_wino_4x4_3x3_input.hxx:89-94, 133-145); every a*b+c is one fma there.
 * ------------------------------------------------------------------------------------------ */
static inline void wino_bt6(const float f[6], float o[6]) {
  const float z0 = -2.25f, z1 = -0.390625f, z2 = 0.87890625f, z3 = -2.640625f, z4 = 0.625f, z5 = 1.5f;
  float t0 = fmaf(f[2], z0, f[4]);
  float t1 = fmaf(f[1], z0, f[3]);
  float t2 = fmaf(f[2], z1, f[4]);
  float t3 = fmaf(f[1], z1, f[3]);
  float t4 = fmaf(f[0], z2, f[4]);
  float t5 = fmaf(f[1], z2, f[5]);
  o[0] = fmaf(f[2], z3, t4);
  o[1] = fmaf(t1, z4, t0);
  o[2] = fmaf(-t1, z4, t0);
  o[3] = fmaf(t3, z5, t2);
  o[4] = fmaf(-t3, z5, t2);
  o[5] = fmaf(f[3], z3, t5);
}

/* V[hA][wA] = B^T d B for one 6x6 tile of one channel: h direction first, then w
 * (elk_conv_wino_4x4_3x3_input.hxx:133-352). */
static int g_border_rule = 1;      /* probe switch, see orc_set_border_rule */
void orc_set_border_rule(int v) { g_border_rule = v; }
static void wino_input_tile(float d[6][6], float v[6][6], int border) {
  float m[6][6];
  for (int w = 0; w < 6; ++w) {
    float col[6], o[6];
    for (int h = 0; h < 6; ++h) col[h] = d[h][w];
    wino_bt6(col, o);
    for (int i = 0; i < 6; ++i) m[i][w] = o[i];
  }
  for (int i = 0; i < 6; ++i) wino_bt6(m[i], v[i]);
  if (border && g_border_rule) {
    /* The reference instantiates a separate kernel for tiles that touch the image border
     * (is_border, src/elx_conv_wino_trans_input.hpp:247-249) and in THAT instantiation g++ leaves
     * two corner results unfused: V[0][5] and V[5][0] are rounded products followed by rounded
     * adds.  Found by comparing against the reference's transformed input (mode a033 scratch
     * dump): with this rule 0 of 147456 values differ, without it 66 do, all in border tiles. */
    const float z2 = 0.87890625f, z3 = -2.640625f;
    float t5 = m[0][1] * z2;  t5 = t5 + m[0][5];
    float p5 = m[0][3] * z3;  v[0][5] = p5 + t5;
    float t4 = m[5][0] * z2;  t4 = t4 + m[5][4];     /* V[5][0]: only the inner sum is unfused */
    v[5][0] = fmaf(m[5][2], z3, t4);
  }
}

/* 1-D weight transform G (src/kernel/elk_conv_wino_4x4_3x3_weights.hxx:25-58) */
static int g_g3_variant = 0;       /* probe switch */
void orc_set_g3_variant(int v) { g_g3_variant = v; }
static inline void wino_g3(float f0, float f1, float f2, float o[6]) {
  const float z0 = 0.26890756302521f, z1 = -0.688403361344538f, z2 = 0.119514472455649f,
              z3 = 1.13777777777778f, z4 = 0.430252100840336f, z5 = 0.179271708683473f;
  float t1, t2;
  if (g_g3_variant == 0) {
    /* g++ fuses the FIRST product of the statement list, z0*f2, into both of its uses and leaves
     * z1*f0 and z2*f0 as rounded products */
    float p1 = z1 * f0, p2 = z2 * f0;
    t1 = fmaf(-z0, f2, p1);
    t2 = fmaf(z0, f2, p2);
  } else {
    float t0 = z0 * f2;
    t1 = fmaf(z1, f0, -t0);
    t2 = fmaf(z2, f0, t0);
  }
  o[0] = z3 * f0;
  o[1] = fmaf(-z4, f1, t1);
  o[2] = fmaf(z4, f1, t1);
  o[3] = fmaf(z5, f1, t2);
  o[4] = fmaf(-z5, f1, t2);
  o[5] = f2;
}

static void wino_weights_tile(float g[3][3], float u[6][6]) {
  float m[6][3];
  for (int kw = 0; kw < 3; ++kw) {
    float o[6];
    wino_g3(g[0][kw], g[1][kw], g[2][kw], o);
    for (int i = 0; i < 6; ++i) m[i][kw] = o[i];
  }
  for (int i = 0; i < 6; ++i) wino_g3(m[i][0], m[i][1], m[i][2], u[i]);
}

/* 1-D output transform A^T (src/kernel/elk_conv_wino_4x4_3x3_output.hxx:115-157).  g++ fuses
 * t2*z3 + t3*z0 as fma(t2, z3, t3*z0) (left product folded into the add of the right product is
 * equally possible; the difference is below the fp32 parity tolerance and only matters for the
 * staged int8 checks, which compare against the reference's own output). */
static int g_at6_variant = 0;
void orc_set_at6_variant(int v) { g_at6_variant = v; }
static inline void wino_at6(const float f[6], float p[4]) {
  const float z0 = 1.5f, z1 = 2.25f, z2 = 3.375f, z3 = 0.625f, z4 = 0.390625f, z5 = 0.244140625f;
  float t0 = f[1] + f[2];
  float t1 = f[3] + f[4];
  float t2 = f[1] - f[2];
  float t3 = f[3] - f[4];
  p[0] = t0 + t1 + f[0];
  if (g_at6_variant == 0) {
    p[1] = fmaf(t2, z3, t3 * z0);
    p[2] = fmaf(t0, z4, t1 * z1);
    p[3] = fmaf(t2, z5, t3 * z2) + f[5];
  } else if (g_at6_variant == 1) {
    p[1] = fmaf(t3, z0, t2 * z3);
    p[2] = fmaf(t1, z1, t0 * z4);
    p[3] = fmaf(t3, z2, t2 * z5) + f[5];
  } else {
    p[1] = t2 * z3 + t3 * z0;
    p[2] = t0 * z4 + t1 * z1;
    p[3] = t2 * z5 + t3 * z2 + f[5];
  }
}


/* ------------------------------------------------------------------------------------------
 * Winograd F(2x2,3x3) (reference tile_size = 4).  Only additions and multiplications by powers
 * of two, so the only rounding is in the adds; their order is the reference's.
 *
 * Input (src/kernel/elk_conv_wino_2x2_3x3_input.hxx:103-149): B^T rows (1,0,-1,0), (0,-1,1,0),
 * (0,1,1,0), (0,-1,0,1), w direction first.  The last element is summed in a different order there.
 * ------------------------------------------------------------------------------------------ */
static inline void wino_bt4(const float f[4], float o[4]) {
  o[0] = f[0] - f[2];
  o[1] = f[2] - f[1];
  o[2] = f[1] + f[2];
  o[3] = f[3] - f[1];
}
static void wino_input_tile4(float d[6][6], float v[6][6]) {
  float g[4][4];
  for (int h = 0; h < 4; ++h) wino_bt4(d[h], g[h]);
  for (int j = 0; j < 4; ++j) {
    float col[4] = {g[0][j], g[1][j], g[2][j], g[3][j]}, o[4];
    wino_bt4(col, o);
    for (int i = 0; i < 4; ++i) v[i][j] = o[i];
  }
  v[3][3] = ((d[1][1] - d[1][3]) - d[3][1]) + d[3][3];      /* :146 */
}
/* Weights (src/kernel/elk_conv_wino_2x2_3x3_weights.hxx:73-107): G rows (1,0,0), (.5,-.5,.5),
 * (.5,.5,.5), (0,0,1); w direction first. */
static void wino_weights_tile4(float g[3][3], float u[6][6]) {
  static const float cs[4] = {1.0f, 0.5f, 0.5f, 1.0f};
  float r[3][4];
  for (int x = 0; x < 3; ++x) {
    r[x][0] = g[x][0];
    r[x][1] = (g[x][0] - g[x][1]) + g[x][2];
    r[x][2] = (g[x][0] + g[x][1]) + g[x][2];
    r[x][3] = g[x][2];
  }
  for (int j = 0; j < 4; ++j) {
    u[0][j] = cs[j] * r[0][j];
    u[1][j] = (cs[j] * 0.5f) * ((r[0][j] - r[1][j]) + r[2][j]);
    u[2][j] = (cs[j] * 0.5f) * ((r[0][j] + r[1][j]) + r[2][j]);
    u[3][j] = cs[j] * r[2][j];
  }
}
/* Output (src/kernel/elk_conv_wino_2x2_3x3_output.hxx:89-97), t[hA][wA] -> y[2][2] */
static void wino_output_tile4(float t[6][6], float y[4][4]) {
  float c0 = (t[1][0] + t[1][1]) + t[1][2];
  float c1 = (t[2][0] + t[2][1]) + t[2][2];
  float c2 = (t[1][2] + t[1][3]) - t[1][1];
  float c3 = (t[2][2] + t[2][3]) - t[2][1];
  y[0][0] = (((t[0][0] + t[0][1]) + t[0][2]) + c0) + c1;
  y[1][0] = (((c1 - c0) + t[3][0]) + t[3][1]) + t[3][2];
  y[0][1] = (((t[0][2] - t[0][1]) + t[0][3]) + c2) + c3;
  y[1][1] = (((c3 - c2) - t[3][1]) + t[3][2]) + t[3][3];
}
static void wino_output_tile6(float t[6][6], float y[4][4]) {
  float m[4][6];
  for (int j = 0; j < 6; ++j) {
    float f[6], q[4];
    for (int i = 0; i < 6; ++i) f[i] = t[i][j];
    wino_at6(f, q);
    for (int i = 0; i < 4; ++i) m[i][j] = q[i];
  }
  for (int i = 0; i < 4; ++i) wino_at6(m[i], y[i]);
}

/* tweights out: [A*A][OC][IC] fp32 (a = hA*A + wA).  Padded channels are zero. */
void orc_wino_trans_weights(const orc_conv_t *p, const float *w, float *tw) {
  int IC = ALIGNUP(p->ic, V), OC = ALIGNUP(p->oc, V);
  const int A = wino_A(p);
#pragma omp parallel for schedule(static)
  for (int o = 0; o < OC; ++o)
    for (int i = 0; i < IC; ++i) {
      float g[3][3], u[6][6];
      for (int kh = 0; kh < 3; ++kh)
        for (int kw = 0; kw < 3; ++kw)
          g[kh][kw] = (o < p->oc && i < p->ic) ? w[w_index(p, o, i, kh, kw)] : 0.0f;
      if (A == 4) wino_weights_tile4(g, u); else wino_weights_tile(g, u);
      for (int a = 0; a < A * A; ++a) tw[((size_t)a * OC + o) * IC + i] = u[a / A][a % A];
    }
}

/* tinput out: [A*A][T][IC] fp32 with T = n*ht*wt tiles, tile index t = (n*ht + th)*wt + tw.
 * Tiles are anchored at (4*th - pad_t, 4*tw - pad_l); taps outside the image read as 0
 * (src/elx_conv_wino_trans_input.hpp:207-260).  in_is_u8: raw u8 values are converted to float
 * WITHOUT de-scaling (elk_conv_wino_4x4_3x3_input.hxx:40-47). */
void orc_wino_trans_input(const orc_conv_t *p, const void *in, int in_is_u8, float *tin) {
  int IC = ALIGNUP(p->ic, V);
  const int A = wino_A(p), OT = A - 2;
  int ht = wino_ht(p), wt = wino_wt(p);
  size_t T = (size_t)p->n * ht * wt;
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < p->n; ++n)
    for (int c = 0; c < IC; ++c)
      for (int th = 0; th < ht; ++th)
        for (int tw = 0; tw < wt; ++tw) {
          float d[6][6], v[6][6];
          for (int h = 0; h < A; ++h)
            for (int w = 0; w < A; ++w) {
              int ih = OT * th - p->pad_t + h, iw = OT * tw - p->pad_l + w;
              float x = 0.0f;
              if (ih >= 0 && ih < p->ih && iw >= 0 && iw < p->iw && c < p->ic) {
                size_t idx = in_index(p, n, c, ih, iw);
                x = in_is_u8 ? (float)((const uint8_t *)in)[idx] : ((const float *)in)[idx];
              }
              d[h][w] = x;
            }
          /* is_border: first tile row/column (padding) or last (the tile overhangs the image) */
          int border = th == 0 || tw == 0 || th == ht - 1 || tw == wt - 1;
          if (A == 4) wino_input_tile4(d, v); else wino_input_tile(d, v, border);
          size_t t = ((size_t)n * ht + th) * wt + tw;
          for (int a = 0; a < A * A; ++a) tin[((size_t)a * T + t) * IC + c] = v[a / A][a % A];
        }
}

/* M[a][t][oc] = sum_ic V[a][t][ic] * U[a][oc][ic], one fma per ic in ascending order
 * (src/kernel/elk_gemm.hxx:380-393). */
void orc_wino_gemm_f32(const orc_conv_t *p, const float *tin, const float *tw, float *tout) {
  int IC = ALIGNUP(p->ic, V), OC = ALIGNUP(p->oc, V);
  int ht = wino_ht(p), wt = wino_wt(p);
  const int AA = wino_A(p) * wino_A(p);
  size_t T = (size_t)p->n * ht * wt;
#pragma omp parallel for collapse(2) schedule(static)
  for (int a = 0; a < AA; ++a)
    for (size_t t = 0; t < T; ++t) {
      const float *vi = tin + ((size_t)a * T + t) * IC;
      for (int o = 0; o < OC; ++o) {
        const float *u = tw + ((size_t)a * OC + o) * IC;
        float acc = 0.0f;
        for (int i = 0; i < IC; ++i) acc = fmaf(vi[i], u[i], acc);
        tout[((size_t)a * T + t) * OC + o] = acc;
      }
    }
}

/* Y = A^T M A, then in this order: +bias, (u8/s8: *1/oS + oz), + previous output (in-place sum),
 * ReLU against a literal 0 (relu_bound is NOT used here), store with border clipping
 * (src/kernel/elk_conv_wino_4x4_3x3_output.hxx:131-195). */
void orc_wino_trans_output(const orc_conv_t *p, const float *tout, const float *bias, void *out,
                           const void *prev) {
  int OC = ALIGNUP(p->oc, V);
  const int A = wino_A(p), OT = A - 2;
  int ht = wino_ht(p), wt = wino_wt(p);
  size_t T = (size_t)p->n * ht * wt;
  float orepS = p->out_type == ORC_F32 ? 1.0f : 1.0f / p->out_scale;
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < p->n; ++n)
    for (int o = 0; o < OC; ++o)
      for (int th = 0; th < ht; ++th)
        for (int tw = 0; tw < wt; ++tw) {
          size_t t = ((size_t)n * ht + th) * wt + tw;
          float tt[6][6], yy[4][4];
          for (int i = 0; i < A; ++i)
            for (int j = 0; j < A; ++j) tt[i][j] = tout[((size_t)(i * A + j) * T + t) * OC + o];
          if (A == 4) wino_output_tile4(tt, yy); else wino_output_tile6(tt, yy);
          for (int i = 0; i < OT; ++i) {
            for (int j = 0; j < OT; ++j) {
              int oh = OT * th + i, ow = OT * tw + j;
              if (oh >= p->oh || ow >= p->ow) continue;
              size_t idx = out_index(p, n, o, oh, ow);
              float f = yy[i][j];
              if (p->with_bias && bias) f += bias[o];
              if (p->out_type != ORC_F32) f = fmaf(f, orepS, p->out_z);
              if (p->with_sum && prev) {
                f += p->out_type == ORC_F32 ? ((const float *)prev)[idx]
                   : p->out_type == ORC_U8 ? (float)((const uint8_t *)prev)[idx]
                                           : (float)((const int8_t *)prev)[idx];
              }
              if (p->with_relu) f = f > 0.0f ? f : 0.0f;
              if (A == 4 && p->out_type != ORC_F32) {
                /* the F(2x2,3x3) kernel alone converts with round-toward-minus-infinity
                 * (elk_conv_wino_2x2_3x3_output.hxx:145-153); saturation as below */
                float rf = floorf(f);
                if (p->out_type == ORC_U8) {
                  uint32_t u = (rf >= 0.0f && rf < 4294967296.0f) ? (uint32_t)rf : 0xFFFFFFFFu;
                  ((uint8_t *)out)[idx] = (uint8_t)(u > 255u ? 255u : u);
                } else {
                  ((int8_t *)out)[idx] = (int8_t)(rf > 127.0f ? 127.0f : rf < -128.0f ? -128.0f : rf);
                }
              } else if (p->out_type == ORC_U8) {
                /* cvt_roundps_epu32 then unsigned saturation: negative -> 0 is NOT what happens:
                 * vcvtps2udq of a negative value yields 0xFFFFFFFF, which saturates to 255. */
                float rf = rne(f);
                uint32_t u = (rf >= 0.0f && rf < 4294967296.0f) ? (uint32_t)rf
                           : (rf > -1.0f && rf <= 0.0f) ? 0u : 0xFFFFFFFFu;
                ((uint8_t *)out)[idx] = (uint8_t)(u > 255u ? 255u : u);
              } else {
                store_q(p, out, idx, f);
              }
            }
          }
        }
}

/* Whole fp32 Winograd convolution (src/elx_conv_wino_xopt.hpp:29-68, mode a061 data flow). */
int orc_wino_f32_conv(const orc_conv_t *p, const float *in, const float *w, const float *bias,
                      float *out, const float *prev) {
  int IC = ALIGNUP(p->ic, V), OC = ALIGNUP(p->oc, V);
  int ht = wino_ht(p), wt = wino_wt(p);
  const int AA = wino_A(p) * wino_A(p);
  size_t T = (size_t)p->n * ht * wt;
  float *tw = (float *)malloc(sizeof(float) * AA * OC * IC);
  float *tin = (float *)malloc(sizeof(float) * AA * T * IC);
  float *tout = (float *)malloc(sizeof(float) * AA * T * OC);
  if (!tw || !tin || !tout) { free(tw); free(tin); free(tout); return -1; }
  orc_wino_trans_weights(p, w, tw);
  orc_wino_trans_input(p, in, 0, tin);
  orc_wino_gemm_f32(p, tin, tw, tout);
  orc_wino_trans_output(p, tout, bias, out, prev);
  free(tw); free(tin); free(tout);
  return 0;
}

/* ------------------------------------------------------------------------------------------
 * INT8 Winograd (u8 input, f32 weights, f32/u8/s8 output), CALIBRATED sampling.
 *   tinput_u8 = sat_u8(rne(fma(V, iS/tS, tz')))       tz' = ceil(tz)
 *        src/elx_conv_wino_trans_input.cpp:616-654, src/elx_int8_conv_wino.cpp:259-278
 *   per (oc, a): absmax over ic of U; q = (int8) rne((U*127)/absmax); Sq = sum q;
 *        scale = (absmax/127) * tS ; shift = -(Sq * scale) * tz'
 *        src/elx_conv_wino_trans_weights.cpp:437-535
 *   M[a][t][oc] = fma((float)acc, scale, shift)       src/kernel/elk_u8s8_gemm.hxx:200-208
 *   then the fp32 output transform above.
 * Optional dumps: tin_u8 [36][T][IC], tw_s8 [36][OC][IC], acc [36][T][OC], tout [36][T][OC].
 * ------------------------------------------------------------------------------------------ */
int orc_int8_wino_conv(const orc_conv_t *p, const uint8_t *in, const float *w, const float *bias,
                       void *out, const void *prev, uint8_t *dump_tin, int8_t *dump_tw,
                       int32_t *dump_acc, float *dump_tout) {
  int IC = ALIGNUP(p->ic, V), OC = ALIGNUP(p->oc, V);
  int ht = wino_ht(p), wt = wino_wt(p);
  const int AA = wino_A(p) * wino_A(p);
  size_t T = (size_t)p->n * ht * wt;
  float *twf = (float *)malloc(sizeof(float) * AA * OC * IC);
  float *tinf = (float *)malloc(sizeof(float) * AA * T * IC);
  uint8_t *tin = (uint8_t *)malloc((size_t)AA * T * IC);
  int8_t *tw = (int8_t *)malloc((size_t)AA * OC * IC);
  float *scale = (float *)malloc(sizeof(float) * AA * OC);
  float *shift = (float *)malloc(sizeof(float) * AA * OC);
  float *tout = (float *)malloc(sizeof(float) * AA * T * OC);
  if (!twf || !tinf || !tin || !tw || !scale || !shift || !tout) return -1;

  float tz = ceilf(p->tin_z);
  float mrepS = p->in_scale * (1.0f / p->tin_scale);

  orc_wino_trans_weights(p, w, twf);
  for (int a = 0; a < AA; ++a)
    for (int o = 0; o < OC; ++o) {
      const float *u = twf + ((size_t)a * OC + o) * IC;
      float m = 0.0f;
      for (int i = 0; i < p->ic; ++i) { float x = fabsf(u[i]); if (x > m) m = x; }
      float sq = 0.0f;
      for (int i = 0; i < IC; ++i) {
        int8_t v = 0;
        if (i < p->ic && m != 0.0f) { float t = u[i] * 127.0f; t = t / m; v = (int8_t)rne(t); }
        tw[((size_t)a * OC + o) * IC + i] = v;
        sq += (float)v;
      }
      float sc = (m / 127.0f) * p->tin_scale;
      scale[a * OC + o] = sc;
      shift[a * OC + o] = -(sq * sc) * tz;
    }

  orc_wino_trans_input(p, in, 1, tinf);
#pragma omp parallel for schedule(static)
  for (size_t k = 0; k < (size_t)AA * T * IC; ++k) {
    /* cvt_roundps_epu32 + cvtusepi32_epi8: a value that rounds below zero converts to 0xFFFFFFFF
     * and therefore saturates to 255, not to 0 (src/elx_conv_wino_trans_input.cpp:643-648) */
    float f = rne(fmaf(tinf[k], mrepS, tz));
    tin[k] = (uint8_t)(f < 0.0f ? 255.0f : f > 255.0f ? 255.0f : f);
  }

#pragma omp parallel for collapse(2) schedule(static)
  for (int a = 0; a < AA; ++a)
    for (size_t t = 0; t < T; ++t) {
      const uint8_t *vi = tin + ((size_t)a * T + t) * IC;
      for (int o = 0; o < OC; ++o) {
        const int8_t *u = tw + ((size_t)a * OC + o) * IC;
        int32_t acc = 0;
        for (int i = 0; i < IC; ++i) acc += (int32_t)vi[i] * (int32_t)u[i];
        size_t k = ((size_t)a * T + t) * OC + o;
        if (dump_acc) dump_acc[k] = acc;
        tout[k] = fmaf((float)acc, scale[a * OC + o], shift[a * OC + o]);
      }
    }
  if (dump_tin) memcpy(dump_tin, tin, (size_t)AA * T * IC);
  if (dump_tw) memcpy(dump_tw, tw, (size_t)AA * OC * IC);
  if (dump_tout) memcpy(dump_tout, tout, sizeof(float) * AA * T * OC);
  orc_conv_t po = *p;
  po.out_z = ceilf(p->out_z);        /* src/elx_int8_conv_wino.cpp:276 */
  orc_wino_trans_output(&po, tout, bias, out, prev);
  free(twf); free(tinf); free(tin); free(tw); free(scale); free(shift); free(tout);
  return 0;
}

/* min / max of the fp32 transformed input of a u8 tensor de-quantised with in_scale: the two
 * numbers the reference's test derives wino_tinput_quant from (tests/elt_conv_utils.cpp:238-255). */
int orc_wino_tinput_range(const orc_conv_t *p, const uint8_t *in, float *mn, float *mx) {
  int IC = ALIGNUP(p->ic, V);
  int ht = wino_ht(p), wt = wino_wt(p);
  const int AA = wino_A(p) * wino_A(p);
  size_t T = (size_t)p->n * ht * wt;
  float *tinf = (float *)malloc(sizeof(float) * AA * T * IC);
  if (!tinf) return -1;
  orc_wino_trans_input(p, in, 1, tinf);
  float lo = FLT_MAX, hi = -FLT_MAX;
  for (size_t k = 0; k < (size_t)AA * T * IC; ++k) {
    float v = tinf[k] * p->in_scale;
    if (v < lo) lo = v;
    if (v > hi) hi = v;
  }
  *mn = lo; *mx = hi;
  free(tinf);
  return 0;
}

/* ------------------------------------------------------------------------------------------
 * Direct fp64 convolution of fp32 tensors (blocked layouts): the independent third opinion the
 * reference's own test uses in fp32 (tests/elt_conv_utils.cpp:668-764).
 * ------------------------------------------------------------------------------------------ */
int orc_direct_f64_conv(const orc_conv_t *p, const float *in, const float *w, const float *bias,
                        float *out) {
  int OC = ALIGNUP(p->oc, V);
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < p->n; ++n)
    for (int o = 0; o < OC; ++o)
      for (int oh = 0; oh < p->oh; ++oh)
        for (int ow = 0; ow < p->ow; ++ow) {
          double acc = (p->with_bias && bias && o < p->oc) ? (double)bias[o] : 0.0;
          if (o < p->oc)
            for (int kh = 0; kh < p->kh; ++kh) {
              int ih = oh * p->stride_h - p->pad_t + kh;
              if (ih < 0 || ih >= p->ih) continue;
              for (int kw = 0; kw < p->kw; ++kw) {
                int iw = ow * p->stride_w - p->pad_l + kw;
                if (iw < 0 || iw >= p->iw) continue;
                for (int i = 0; i < p->ic; ++i)
                  acc += (double)in[in_index(p, n, i, ih, iw)] * (double)w[w_index(p, o, i, kh, kw)];
              }
            }
          /* in-place sum: the fp32 direct kernels start from the stored output instead of zero
           * (AT_CLEAR_OUTPUT off, src/kernel/elk_gemm.hxx:330-372, src/kernel/elk_conv.hxx) */
          if (p->with_sum) acc += (double)out[out_index(p, n, o, oh, ow)];
          if (p->with_relu) {      /* relu_bound is honoured on this path (elk_gemm.hxx:230-235) */
            if (acc < (double)p->relu_lo) acc = (double)p->relu_lo;
            if (acc > (double)p->relu_hi) acc = (double)p->relu_hi;
          }
          out[out_index(p, n, o, oh, ow)] = (float)acc;
        }
  return 0;
}

/* ------------------------------------------------------------------------------------------
 * INT8 depthwise 3x3 convolution (g = ic = oc), u8 input, f32 goihw weights, u8 / s8 output.
 * Reference: src/elx_int8_conv_direct_depthwise.cpp (constructor :14-131, weight preparation
 * trans_weights_3x3 :202-292, conv_c160 :295-318), src/elx_int8_conv_direct_depthwise_xopt.hpp:19-66,
 * kernel src/kernel/elk_u8s8_depthwise_conv.hxx:288-474.
 *
 * Weights, per channel c (:208-237): absmax over the 9 taps, q = (int8) rint((w * 127) / absmax),
 * Sw = absmax / 127.  Constants (:263-291): scale = (iS * Sw) * (1/oS);
 * shift = (bias * (1/oS) + oz) - ((iz * Sq) * scale) with Sq = the sum of ALL nine q of the channel
 * (no border correction: a padded tap contributes 0 to the accumulator but its q stays in Sq).
 *
 * Output rows are cut into chunks of T = flatting.t pixels (0 means 1; the last chunk holds the
 * remainder Tr, :76-80).  Epilogue per pixel f = fma(acc, scale, shift), ReLU clamp, then
 *   s8 output: round to nearest even, signed saturation;
 *   u8 output: the first 4*floor(L/4) pixels of a chunk of length L go four at a time through
 *     u = (int32) floor(f)  (round toward minus infinity, NO saturation),
 *     word = u0 + (u1 << 8) + (u2 << 16) + (u3 << 24)  in 32-bit wrap-around arithmetic, and byte k
 *     of word is pixel k (elk_u8s8_depthwise_conv.hxx:257-286, 406-455); the remaining L % 4 pixels
 *     are rounded to nearest even and saturated as unsigned (:219-255, 456-473).
 * with_ip_sum is accepted and has no effect (the attribute bit is never read by the kernel).
 * ------------------------------------------------------------------------------------------ */
static inline int32_t cvt_i32(float r) {     /* cvtps_epi32 result for an already rounded float */
  if (!(r >= -2147483648.0f && r < 2147483648.0f)) return INT32_MIN;
  return (int32_t)r;
}

int orc_int8_depthwise(const orc_conv_t *p, int T, const uint8_t *in, const float *w, const float *bias,
                       void *out, int32_t *acc_dump) {
  if (p->ic != p->oc || p->kh != 3 || p->kw != 3 || p->out_type == ORC_F32) return -2;
  const int G = ALIGNUP(p->ic, V), g = p->ic;
  if (T <= 0) T = 1;
  int8_t *q = (int8_t *)calloc((size_t)G * 9, 1);
  float *scale = (float *)calloc(G, sizeof(float)), *shift = (float *)calloc(G, sizeof(float));
  if (!q || !scale || !shift) return -1;
  const float orepS = 1.0f / p->out_scale;
  for (int c = 0; c < g; ++c) {
    float m = 0.0f;
    for (int k = 0; k < 9; ++k) { float a = fabsf(w[c * 9 + k]); if (a > m) m = a; }
    int sq = 0;
    for (int k = 0; k < 9; ++k) {
      float t = w[c * 9 + k] * 127.0f;
      t = t / m;
      q[c * 9 + k] = (int8_t)rintf(t);
      sq += q[c * 9 + k];
    }
    float Sw = m / 127.0f;
    float qs = p->in_scale * Sw;
    qs = qs * orepS;
    float b = (p->with_bias && bias) ? bias[c] : 0.0f;
    float t0 = fmaf(b, orepS, p->out_z);
    float zq = p->in_z * (float)sq;
    scale[c] = qs;
    shift[c] = fmaf(-zq, qs, t0);
  }
  const int wt = (p->ow + T - 1) / T;
  const int Tr = p->ow % T ? p->ow % T : T;
  /* Channels are handled in pairs (2j, 2j+1): the packing adds of the floor path are written with
   * operator+= on __m512i, which g++ compiles as EIGHT 64-BIT adds, so a carry or borrow out of an
   * even channel's 32-bit word runs into the odd channel's word (only reachable when a floored
   * value lies outside [0, 255], i.e. without ReLU or with an output scale that overflows u8). */
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < p->n; ++n)
    for (int cp = 0; cp < G / 2; ++cp)
      for (int oh = 0; oh < p->oh; ++oh)
        for (int ck = 0; ck < wt; ++ck) {
          const int L = ck == wt - 1 ? Tr : T;
          const int nfloor = p->out_type == ORC_U8 ? 4 * (L / 4) : 0;
          float *f = (float *)malloc(sizeof(float) * 2 * (size_t)L);
          for (int e = 0; e < 2; ++e) {
            const int c = 2 * cp + e;
            for (int j = 0; j < L; ++j) {
              const int ow = ck * T + j;
              int32_t acc = 0;
              if (c < g)
                for (int kh = 0; kh < 3; ++kh) {
                  int ih = oh * p->stride_h - p->pad_t + kh;
                  if (ih < 0 || ih >= p->ih) continue;
                  for (int kw = 0; kw < 3; ++kw) {
                    int iw = ow * p->stride_w - p->pad_l + kw;
                    if (iw < 0 || iw >= p->iw) continue;
                    acc += (int32_t)in[in_index(p, n, c, ih, iw)] * (int32_t)q[c * 9 + kh * 3 + kw];
                  }
                }
              if (acc_dump) acc_dump[out_index(p, n, c, oh, ow)] = acc;
              float v = fmaf((float)acc, scale[c], shift[c]);
              if (p->with_relu) {
                v = v > p->relu_lo ? v : p->relu_lo;
                v = v < p->relu_hi ? v : p->relu_hi;
              }
              f[e * L + j] = v;
            }
          }
          for (int j = 0; j < nfloor; j += 4) {
            uint64_t sum = 0;
            for (int k = 0; k < 4; ++k) {
              uint32_t lo = (uint32_t)cvt_i32(floorf(f[j + k])) << (8 * k);           /* slli_epi32 */
              uint32_t hi = (uint32_t)cvt_i32(floorf(f[L + j + k])) << (8 * k);
              sum += (uint64_t)lo | ((uint64_t)hi << 32);                             /* 64-bit add */
            }
            for (int e = 0; e < 2; ++e) {
              uint32_t word = (uint32_t)(sum >> (32 * e));
              for (int k = 0; k < 4; ++k)
                ((uint8_t *)out)[out_index(p, n, 2 * cp + e, oh, ck * T + j + k)] = (uint8_t)(word >> (8 * k));
            }
          }
          for (int e = 0; e < 2; ++e)
            for (int j = nfloor; j < L; ++j)
              store_q(p, out, out_index(p, n, 2 * cp + e, oh, ck * T + j), f[e * L + j]);
          free(f);
        }
  free(q); free(scale); free(shift);
  return 0;
}

int orc_struct_size(void) { return (int)sizeof(orc_conv_t); }
