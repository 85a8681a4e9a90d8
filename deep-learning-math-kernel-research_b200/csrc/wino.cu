// Winograd F(4x4,3x3) convolution (the reference's tile_size = 6) for sm_100a, fp32 and int8.
//
// Replaces elx_conv_wino_t / elx_int8_conv_wino_t (src/elx_conv_wino.cpp, src/elx_int8_conv_wino.cpp,
// their *_xopt.hpp execution modes) and the stages under them:
//   input transform   src/elx_conv_wino_trans_input.cpp + src/kernel/elk_conv_wino_4x4_3x3_input.hxx
//   weights transform src/elx_conv_wino_trans_weights.cpp + src/kernel/elk_conv_wino_4x4_3x3_weights.hxx
//   batched GEMM      src/elx_conv_wino_gemm.cpp, src/elx_int8_conv_wino_gemm.cpp,
//                     src/kernel/elk_gemm.hxx, src/kernel/elk_u8s8_gemm.hxx
//   output transform  src/elx_conv_wino_trans_output.cpp + src/kernel/elk_conv_wino_4x4_3x3_output.hxx
//
// Data flow on the device (three kernels per call, the weights are transformed once per plan):
//   1. wino_input_kernel: reads nChw16c, computes V = B^T d B for every 6x6 tile and writes it
//      DIRECTLY in the operand image of the GEMM: for each of the 36 positions a, each 128-tile
//      row block and each K stage, [K chunk of 16 B][128 rows][16 B] -- so one GEMM stage of A is
//      one contiguous bulk TMA copy.  fp32: V is stored as plain fp32; int8: V is quantised to u8
//      here (sat(rne(fma(V, iS/tS, tz)))).
//   2. wino_gemm_kernel: 36 independent GEMMs M[a] = V[a] * U[a]^T on tcgen05 tensor cores with
//      TMEM accumulators.  fp32: four splitter warps turn each landed fp32 stage of V into its
//      tf32 planes hi = tf32(V), lo = V - hi in shared memory (the weights' planes are prepared
//      once per plan), then three kind::tf32 MMAs per K step (lo*hi + hi*lo + hi*hi) with fp32
//      accumulation.  int8: kind::i8 with s32 accumulation and the fp32 de-scale
//      fma(acc, scale[a][oc], shift[a][oc]) in the epilogue.  Same warp roles, ring of
//      shared-memory stages and bounded waits as the direct-convolution kernel.
//   3. wino_output_kernel: Y = A^T M A, + bias, (requantise), + in-place sum, ReLU, clipped store
//      into nChw16c.
// Batches whose transform-domain buffers would exceed the workspace budget (6 GiB) are processed in
// chunks of whole images.  (Chunks small enough to keep those buffers in L2 were measured and lose:
// the three kernels of a small chunk each pay a fixed 15-20 us.)
// A Winograd request for a layer with at most four input channels is served by the direct kernel of
// f32_small_ic.cu instead.
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "elb_common.cuh"
#include "host_prep.hpp"
#include "umma.cuh"
#include <type_traits>

#include "wino.cuh"

namespace elb {

namespace {

constexpr int BM = 128;
constexpr int GEMM_STAGES_1 = 4;             // pipeline stages: one CTA per tile (16 KB A + 32 KB B each)
constexpr int GEMM_STAGES_2 = 6;             // pairs of CTAs (16 KB A + 16 KB of B each)
constexpr int GEMM_MAX_STAGES = 8;           // barrier slots; fp32 with A in tensor memory runs 5..8 smaller stages
constexpr int EPI_CONST_BYTES = 32768;       // int8: per-epilogue-warp copies of the tile's scale / shift slice (16 KB used); fp32: more ring
constexpr int A_STAGE_BYTES = 16384;          // in shared memory. fp32: hi + lo planes x 4 chunks x 2 KB; int8: 8 chunks x 2 KB
constexpr int A_RAW_BYTES = 8192;             // fp32 only: one stage of V as it lies in global memory (4 chunks x 2 KB)
constexpr int GEMM_CONV_WARPS = 4;            // fp32 only: warps that split a raw stage into its tf32 hi / lo planes
#ifndef GEMM_CONV_GROUPS
#define GEMM_CONV_GROUPS 1                    // groups of such warps taking turns on the stages (2 measured slower: 0.43 vs 0.42 ms on VGG conv3_2, and the extra 128 threads push the epilogue into register spills)
#endif
constexpr int MAX_BN = 256;
constexpr int B_STAGE_MAX = 128 * MAX_BN;     // fp32: 2 x 4 x BN x 16; int8: 8 x BN x 16  (= 128*BN)
constexpr int GEMM_EPI_WARPS = 8;
// Transform kernels: one thread holds a whole 6x6 patch of 4 channels (about 190 registers), so
// an SM fits ~340 threads.  Small blocks let several of them be resident and drift apart, which
// overlaps one block's loads with another's arithmetic and stores.
#ifndef TRANS_THREADS
#define TRANS_THREADS 64
#endif
constexpr int TRANS_TILES = TRANS_THREADS / 4;      // tiles per block (4 threads = the 16 channels of a block)
// Warp roles of the GEMM kernel, laid out in whole warpgroups (register reallocation works on groups of
// four warps): 0, 2 producers (3: a third one, unused by default), 1 MMA issuer | 4..11 epilogue | 12.. splitters
constexpr int GEMM_PRODUCERS = 3;             // producer warps the kernel can run
constexpr int GEMM_PRODUCERS_DEFAULT = 2;     // measured: a third changes nothing (VGG conv1_2 GEMM 0.615 vs 0.624 ms, c1 0.335 vs 0.338 ms)
constexpr int GEMM_EPI_WARP0 = 4;
constexpr int GEMM_SPLIT_WARP0 = GEMM_EPI_WARP0 + GEMM_EPI_WARPS;
constexpr int GEMM_THREADS = (GEMM_SPLIT_WARP0 + GEMM_CONV_GROUPS * GEMM_CONV_WARPS) * 32;
static_assert(GEMM_EPI_WARP0 % 4 == 0 && GEMM_EPI_WARPS % 4 == 0 && GEMM_CONV_WARPS == 4, "roles must fill whole warpgroups");
// Registers per thread after the set-up: the epilogue warpgroups hold a whole 128 x 256 accumulator
// (128 values per thread) so that tensor memory is released before the global stores; the other
// warpgroups give theirs up.  (2 x 128 x 184 + 2 x 128 x 72 = the 64 K registers the launch owns.)
constexpr int GEMM_EPI_REGS = 184, GEMM_OTHER_REGS = 72;
static_assert(GEMM_CONV_GROUPS == 1, "the register split assumes four warpgroups");
constexpr size_t WORKSPACE_BUDGET = size_t(6) << 30;   // transform-domain buffers per chunk

enum : int { KIND_F32 = 0, KIND_I8 = 1 };

// ------------------------------------------------------------------------------ 1-D transforms
// B^T with the reference's constants and evaluation order; every a*b+c is ONE fused multiply-add
// there (src/kernel/elk_conv_wino_4x4_3x3_input.hxx:89-94, 133-145).
__device__ __forceinline__ void bt6(const float (&f)[6], float (&o)[6]) {
  const float z0 = -2.25f, z1 = -0.390625f, z2 = 0.87890625f, z3 = -2.640625f, z4 = 0.625f, z5 = 1.5f;
  const float t0 = __fmaf_rn(f[2], z0, f[4]);
  const float t1 = __fmaf_rn(f[1], z0, f[3]);
  const float t2 = __fmaf_rn(f[2], z1, f[4]);
  const float t3 = __fmaf_rn(f[1], z1, f[3]);
  const float t4 = __fmaf_rn(f[0], z2, f[4]);
  const float t5 = __fmaf_rn(f[1], z2, f[5]);
  o[0] = __fmaf_rn(f[2], z3, t4);
  o[1] = __fmaf_rn(t1, z4, t0);
  o[2] = __fmaf_rn(-t1, z4, t0);
  o[3] = __fmaf_rn(t3, z5, t2);
  o[4] = __fmaf_rn(-t3, z5, t2);
  o[5] = __fmaf_rn(f[3], z3, t5);
}

// Two-lane fp32 arithmetic (add / mul / fma .f32x2: each lane rounds exactly as the scalar
// instruction does).  The output transform runs few warps per SM and the four channels of a thread go
// through identical arithmetic: as two channel pairs the same work is half the instructions and,
// as compiled, 136 registers instead of 181 (c1's output transform 0.147 -> 0.137 ms, VGG conv1_2's
// 0.282 -> 0.259 ms).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
// A^T with the reference's constants and evaluation order (src/kernel/elk_conv_wino_4x4_3x3_output.hxx:115-157),
// on two channels at once, operation for operation
__device__ __forceinline__ void at6x2(const f32x2 (&f)[6], f32x2 (&p)[4]) {
  const f32x2 z0 = pack2(1.5f, 1.5f), z1 = pack2(2.25f, 2.25f), z2 = pack2(3.375f, 3.375f), z3 = pack2(0.625f, 0.625f),
              z4 = pack2(0.390625f, 0.390625f), z5 = pack2(0.244140625f, 0.244140625f);
  const f32x2 t0 = add2(f[1], f[2]);
  const f32x2 t1 = add2(f[3], f[4]);
  const f32x2 t2 = sub2(f[1], f[2]);
  const f32x2 t3 = sub2(f[3], f[4]);
  p[0] = add2(add2(t0, t1), f[0]);
  p[1] = fma2(t2, z3, mul2(t3, z0));
  p[2] = fma2(t0, z4, mul2(t1, z1));
  p[3] = add2(fma2(t2, z5, mul2(t3, z2)), f[5]);
}

struct WinoGeom {
  int A;          // input tile edge: 6 = F(4x4,3x3), 4 = F(2x2,3x3); output tile edge A - 2.
                  // 1 = fp32 direct convolution: one "position", a GEMM row per output pixel
  int KH, KW, stride, taps;   // direct convolution only
  int N, CB, OCB, IH, IW, OH, OW, ht, wt, pad_t, pad_l;
  int T;          // tiles in this chunk = images * ht * wt
  int m_tiles;    // ceil(T / 128)
  int Tpad;       // m_tiles * 128
  int k_stages;   // fp32: CB (16 channels per stage); int8: ceil(CB / 8) (128 channels per stage)
};

// ------------------------------------------------------------------------------ input transform
// One thread = one tile x 4 consecutive channels.  A warp covers 8 consecutive tiles x the 16
// channels of one block, so its stores are 128 contiguous bytes per K chunk (8 rows x 16 B).
struct WinoInParams {
  const void *in;      // nChw16c fp32 or u8, first image of the chunk
  void *a_img;         // operand image
  WinoGeom g;
  float mrepS, tz;     // int8: u8 = sat(rne(fma(V, mrepS, tz)))
  int step, SH, SW;    // fp32 F(4x4,3x3): the input is a plane of SH x SW pixels read with this step (1: SH = IH, SW = IW)
};

template <bool IN_U8>
__global__ void __launch_bounds__(TRANS_THREADS) wino_input_kernel(const __grid_constant__ WinoInParams p) {
  const WinoGeom &g = p.g;
  const int quad = threadIdx.x & 3;
  const int t = blockIdx.x * TRANS_TILES + (threadIdx.x >> 2);
  const int cb = blockIdx.y;
  if (t >= g.Tpad) return;
  const int mt = t >> 7, row = t & 127;

  float m[6][6][4];   // first the 6x6 input patch d[h][w][channel], then (in place) the pass along h: m[i][w][channel]
  const bool live = t < g.T;
  int n = 0, th = 0, tw = 0;
  if (live) {
    n = t / (g.ht * g.wt);
    const int r = t - n * g.ht * g.wt;
    th = r / g.wt;
    tw = r - th * g.wt;
  }
  const int ih0 = 4 * th - g.pad_t, iw0 = 4 * tw - g.pad_l;
  // is_border of the reference's tile iterator (src/elx_conv_wino_trans_input.hpp:247-249)
  const bool border = th == 0 || tw == 0 || th == g.ht - 1 || tw == g.wt - 1;
  // All 36 loads of the patch are issued before the first use: the kernel is bandwidth-bound and
  // runs few warps per SM (the patch lives in registers), so the bytes in flight per thread are
  // what keeps HBM busy.
  if (IN_U8) {
    uint32_t raw[6][6];
#pragma unroll
    for (int h = 0; h < 6; ++h)
#pragma unroll
      for (int w = 0; w < 6; ++w) {
        const int ih = ih0 + h, iw = iw0 + w;
        const bool ok = live && ih >= 0 && ih < g.IH && iw >= 0 && iw < g.IW;
        const size_t pix = ((static_cast<size_t>(n) * g.CB + cb) * g.IH + (ok ? ih : 0)) * g.IW + (ok ? iw : 0);
        raw[h][w] = ok ? __ldg(reinterpret_cast<const uint32_t *>(static_cast<const uint8_t *>(p.in) + pix * 16) + quad) : 0u;
      }
    // u8 -> fp32 without the conversion unit: a byte permute builds the bit pattern of 2^23 + b,
    // subtracting 2^23 is exact
#pragma unroll
    for (int h = 0; h < 6; ++h)
#pragma unroll
      for (int w = 0; w < 6; ++w)
#pragma unroll
        for (int c = 0; c < 4; ++c)
          m[h][w][c] = __fsub_rn(__uint_as_float(__byte_perm(raw[h][w], 0x4B000000u, 0x7650 + c)), 8388608.0f);
  } else {
    // one base pointer per thread, row and column offsets added to it; tiles that do not touch the
    // image border load without any bounds test (the address arithmetic and the predicates of 36
    // separately addressed loads cost this kernel more than its transform)
    const float4 *plane = reinterpret_cast<const float4 *>(static_cast<const float *>(p.in) +
                                                           (static_cast<size_t>(n) * g.CB + cb) * p.SH * p.SW * 16) + quad;
    const int row_pitch = p.SW * p.step * 4, col_pitch = p.step * 4;      // in float4 units
    if (live && ih0 >= 0 && iw0 >= 0 && ih0 + 5 < g.IH && iw0 + 5 < g.IW) {
      const float4 *p0 = plane + static_cast<size_t>(ih0) * row_pitch + iw0 * col_pitch;
#pragma unroll
      for (int h = 0; h < 6; ++h)
#pragma unroll
        for (int w = 0; w < 6; ++w) {
          const float4 v = __ldg(p0 + h * row_pitch + w * col_pitch);
          m[h][w][0] = v.x; m[h][w][1] = v.y; m[h][w][2] = v.z; m[h][w][3] = v.w;
        }
    } else {
#pragma unroll
      for (int h = 0; h < 6; ++h)
#pragma unroll
        for (int w = 0; w < 6; ++w) {
          const int ih = ih0 + h, iw = iw0 + w;
          const bool ok = live && ih >= 0 && ih < g.IH && iw >= 0 && iw < g.IW;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (ok) v = __ldg(plane + static_cast<size_t>(ih) * row_pitch + iw * col_pitch);
          m[h][w][0] = v.x; m[h][w][1] = v.y; m[h][w][2] = v.z; m[h][w][3] = v.w;
        }
    }
  }
  // pass along h, in place.  (Two channels per instruction, as in the output transform, measured
  // SLOWER here: c1's input transform 0.127 -> 0.137 ms, VGG conv1_2's 0.245 -> 0.264 ms; and without
  // effect in the u8 kernel below: c4's 0.084 ms either way.)
#pragma unroll
  for (int w = 0; w < 6; ++w)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float f[6] = {m[0][w][c], m[1][w][c], m[2][w][c], m[3][w][c], m[4][w][c], m[5][w][c]};
      float o[6];
      bt6(f, o);
#pragma unroll
      for (int i = 0; i < 6; ++i) m[i][w][c] = o[i];
    }
  // pass along w, one transformed row at a time, stored as soon as it is ready
  float *v_base = static_cast<float *>(p.a_img) +
                  ((static_cast<size_t>(mt) * g.k_stages + cb) * (A_RAW_BYTES / 4) + (quad * BM + row) * 4);   // fp32: position 0
  const size_t v_step = static_cast<size_t>(g.m_tiles) * g.k_stages * (A_RAW_BYTES / 4);                        // ... to the next position
#pragma unroll
  for (int i = 0; i < 6; ++i) {
    float v[6][4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float f[6] = {m[i][0][c], m[i][1][c], m[i][2][c], m[i][3][c], m[i][4][c], m[i][5][c]};
      float o[6];
      bt6(f, o);
#pragma unroll
      for (int j = 0; j < 6; ++j) v[j][c] = o[j];
      // The reference compiles a separate kernel for tiles that touch the image border, and in it
      // two corner results are not fully fused: V[0][5] is rounded products + rounded adds,
      // V[5][0] keeps only its outer fma.  Reproduced so that the quantised u8 transform matches
      // the reference bit for bit (found against its mode-a033 scratch dump).
      if (border) {
        const float z2 = 0.87890625f, z3 = -2.640625f;
        if (i == 0) v[5][c] = __fadd_rn(__fmul_rn(f[3], z3), __fadd_rn(__fmul_rn(f[1], z2), f[5]));
        if (i == 5) v[0][c] = __fmaf_rn(f[2], z3, __fadd_rn(__fmul_rn(f[0], z2), f[4]));
      }
    }
#pragma unroll
    for (int j = 0; j < 6; ++j) {
      const int a = i * 6 + j;
      if (IN_U8) {
        // stage = 8 channel blocks; chunk = cb % 8; 4 bytes per thread
        // sat_u8(rne(fma(V, mrepS, tz))): adding 1.5 * 2^23 rounds to nearest even and leaves the
        // integer in the low bits; as an UNSIGNED number a negative result is huge, so one min()
        // gives the reference's unsigned saturation (below zero -> 255, above 255 -> 255).  Exact
        // while |fma| < 2^22; anything larger takes the plain conversion.
        uint32_t b[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float f = __fmaf_rn(v[j][c], p.mrepS, p.tz);
          const uint32_t u = __float_as_uint(__fadd_rn(f, 12582912.0f)) - 0x4B400000u;
          b[c] = min(u, 255u);
          if (!(fabsf(f) < 4194304.0f)) {
            const float q = rintf(f);
            b[c] = (q < 0.0f || q > 255.0f || q != q) ? 255u : static_cast<uint32_t>(q);
          }
        }
        const uint32_t w = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
        const size_t off = ((((static_cast<size_t>(a) * g.m_tiles + mt) * g.k_stages + (cb >> 3)) * 8 + (cb & 7)) * BM + row) * 16 + quad * 4;
        *reinterpret_cast<uint32_t *>(static_cast<uint8_t *>(p.a_img) + off) = live ? w : 0u;
      } else {
        // stage = this channel block, chunk = quad; plain fp32 (the GEMM kernel splits it into its
        // tf32 hi / lo planes in shared memory, so V crosses HBM once, not twice)
        // (one base address per thread + a constant step per position)
        *reinterpret_cast<float4 *>(v_base + static_cast<size_t>(a) * v_step) = make_float4(v[j][0], v[j][1], v[j][2], v[j][3]);
      }
    }
  }
}

// u8 variant (INT8 Winograd): the 36 input words of a thread stay packed (4 channels per word)
// and the four channels are transformed ONE AFTER THE OTHER, so a thread needs ~36 + 36 + 36
// registers instead of 36 + 144.  That doubles the warps an SM can hold; the kernel is bound by
// instruction latency (few warps, long dependent fma chains), not by its 51 MB + 116 MB of traffic.
// FAST: the host has checked that |fma(V, mrepS, tz)| < 2^22 for every possible input (|V| <= 255 *
// 5.28125^2, the largest absolute row sum of B^T squared), so the rounding by magic-number addition
// is exact and the general conversion is not even compiled in.
template <bool FAST>
__global__ void __launch_bounds__(TRANS_THREADS, 512 / TRANS_THREADS) wino_input_u8_kernel(const __grid_constant__ WinoInParams p) {
  const WinoGeom &g = p.g;
  const int quad = threadIdx.x & 3;
  const int t = blockIdx.x * TRANS_TILES + (threadIdx.x >> 2);
  const int cb = blockIdx.y;
  if (t >= g.Tpad) return;
  const int mt = t >> 7, row = t & 127;
  const bool live = t < g.T;
  int n = 0, th = 0, tw = 0;
  if (live) {
    n = t / (g.ht * g.wt);
    const int r = t - n * g.ht * g.wt;
    th = r / g.wt;
    tw = r - th * g.wt;
  }
  const int ih0 = 4 * th - g.pad_t, iw0 = 4 * tw - g.pad_l;
  const bool border = th == 0 || tw == 0 || th == g.ht - 1 || tw == g.wt - 1;   // src/elx_conv_wino_trans_input.hpp:247-249
  uint32_t raw[6][6], outw[36];
  // one base pointer per thread; tiles inside the image load without bounds tests (see the fp32 kernel)
  const uint32_t *plane = reinterpret_cast<const uint32_t *>(static_cast<const uint8_t *>(p.in) +
                                                             (static_cast<size_t>(n) * g.CB + cb) * g.IH * g.IW * 16) + quad;
  if (live && ih0 >= 0 && iw0 >= 0 && ih0 + 5 < g.IH && iw0 + 5 < g.IW) {
    const uint32_t *p0 = plane + (static_cast<size_t>(ih0) * g.IW + iw0) * 4;
#pragma unroll
    for (int h = 0; h < 6; ++h)
#pragma unroll
      for (int w = 0; w < 6; ++w) raw[h][w] = __ldg(p0 + (h * g.IW + w) * 4);
  } else {
#pragma unroll
    for (int h = 0; h < 6; ++h)
#pragma unroll
      for (int w = 0; w < 6; ++w) {
        const int ih = ih0 + h, iw = iw0 + w;
        const bool ok = live && ih >= 0 && ih < g.IH && iw >= 0 && iw < g.IW;
        raw[h][w] = ok ? __ldg(plane + (static_cast<size_t>(ih) * g.IW + iw) * 4) : 0u;
      }
  }
#pragma unroll
  for (int a = 0; a < 36; ++a) outw[a] = 0u;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    const uint32_t sel_in = 0x7650u + c;                        // byte c of x, then the three high bytes of y
    const uint32_t sel_out = 0x3210u ^ ((4u ^ c) << (4 * c));   // byte c of the result <- byte 0 of y
    float m[6][6];
    // u8 -> fp32 without the conversion unit: the permute builds the bit pattern of 2^23 + b
#pragma unroll
    for (int h = 0; h < 6; ++h)
#pragma unroll
      for (int w = 0; w < 6; ++w)
        m[h][w] = __fsub_rn(__uint_as_float(__byte_perm(raw[h][w], 0x4B000000u, sel_in)), 8388608.0f);
#pragma unroll
    for (int w = 0; w < 6; ++w) {          // pass along h, in place
      const float f[6] = {m[0][w], m[1][w], m[2][w], m[3][w], m[4][w], m[5][w]};
      float o[6];
      bt6(f, o);
#pragma unroll
      for (int i = 0; i < 6; ++i) m[i][w] = o[i];
    }
#pragma unroll
    for (int i = 0; i < 6; ++i) {          // pass along w, quantise
      const float f[6] = {m[i][0], m[i][1], m[i][2], m[i][3], m[i][4], m[i][5]};
      float v[6];
      bt6(f, v);
      // border tiles: the reference's border kernel leaves two corner results partly unfused (see
      // the fp32 kernel above)
      if (border) {
        const float z2 = 0.87890625f, z3 = -2.640625f;
        if (i == 0) v[5] = __fadd_rn(__fmul_rn(f[3], z3), __fadd_rn(__fmul_rn(f[1], z2), f[5]));
        if (i == 5) v[0] = __fmaf_rn(f[2], z3, __fadd_rn(__fmul_rn(f[0], z2), f[4]));
      }
#pragma unroll
      for (int j = 0; j < 6; ++j) {
        // sat_u8(rne(fma(V, mrepS, tz))): adding 1.5 * 2^23 rounds to nearest even and leaves the
        // integer in the low bits; read as UNSIGNED a negative result is huge, so one min() gives
        // the reference's unsigned saturation (below zero -> 255, above 255 -> 255).  Exact while
        // |fma| < 2^22; anything larger takes the plain conversion.
        const float q = __fmaf_rn(v[j], p.mrepS, p.tz);
        uint32_t b = min(__float_as_uint(__fadd_rn(q, 12582912.0f)) - 0x4B400000u, 255u);
        if (!FAST) {
          if (!(fabsf(q) < 4194304.0f)) {
            const float r = rintf(q);
            b = (r < 0.0f || r > 255.0f || r != r) ? 255u : static_cast<uint32_t>(r);
          }
        }
        outw[i * 6 + j] = __byte_perm(outw[i * 6 + j], b, sel_out);
      }
    }
  }
  // stage = 8 channel blocks; chunk = cb % 8; 4 bytes per thread, 128 contiguous bytes per warp
  uint32_t *v_base = reinterpret_cast<uint32_t *>(static_cast<uint8_t *>(p.a_img) +
                     (((static_cast<size_t>(mt) * g.k_stages + (cb >> 3)) * 8 + (cb & 7)) * BM + row) * 16 + quad * 4);   // position 0
  const size_t v_step = static_cast<size_t>(g.m_tiles) * g.k_stages * 8 * BM * 4;                                        // words to the next one
#pragma unroll
  for (int a = 0; a < 36; ++a) v_base[a * v_step] = live ? outw[a] : 0u;
}


// ------------------------------------------------------------------------------ F(2x2,3x3), tile_size 4
// Same data flow with 16 transform positions, 4x4 input tiles anchored every 2 pixels and 2x2
// output tiles.  The matrices hold only 0, +-1 (and powers of two on the weight side), so the
// transforms are sums; they are written in the reference's order
// (src/kernel/elk_conv_wino_2x2_3x3_input.hxx:103-149, ..._output.hxx:89-97).
__device__ __forceinline__ void bt4(const float (&f)[4], float (&o)[4]) {
  o[0] = __fsub_rn(f[0], f[2]);
  o[1] = __fsub_rn(f[2], f[1]);
  o[2] = __fadd_rn(f[1], f[2]);
  o[3] = __fsub_rn(f[3], f[1]);
}

// One thread = one 4x4 tile x 4 consecutive channels (64 values).  IN_U8: quantises to u8 like the
// F(4x4,3x3) kernel; |V| <= 4 * 255, so the magic-number rounding is exact whenever the host found
// 1020 * |mrepS| + |tz| < 2^22 (FAST), else the general conversion is kept.
template <bool IN_U8, bool FAST>
__global__ void __launch_bounds__(128) wino4_input_kernel(const __grid_constant__ WinoInParams p) {
  const WinoGeom &g = p.g;
  const int quad = threadIdx.x & 3;
  const int t = blockIdx.x * 32 + (threadIdx.x >> 2);
  const int cb = blockIdx.y;
  if (t >= g.Tpad) return;
  const int mt = t >> 7, row = t & 127;
  const bool live = t < g.T;
  int n = 0, th = 0, tw = 0;
  if (live) {
    n = t / (g.ht * g.wt);
    const int r = t - n * g.ht * g.wt;
    th = r / g.wt;
    tw = r - th * g.wt;
  }
  const int ih0 = 2 * th - g.pad_t, iw0 = 2 * tw - g.pad_l;
  float d[4][4][4];
#pragma unroll
  for (int h = 0; h < 4; ++h)
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const int ih = ih0 + h, iw = iw0 + w;
      const bool ok = live && ih >= 0 && ih < g.IH && iw >= 0 && iw < g.IW;
      const size_t pix = ((static_cast<size_t>(n) * g.CB + cb) * g.IH + (ok ? ih : 0)) * g.IW + (ok ? iw : 0);
      if (IN_U8) {
        const uint32_t raw = ok ? __ldg(reinterpret_cast<const uint32_t *>(static_cast<const uint8_t *>(p.in) + pix * 16) + quad) : 0u;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          d[h][w][c] = __fsub_rn(__uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7650 + c)), 8388608.0f);
      } else {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ok) v = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(p.in) + pix * 16) + quad);
        d[h][w][0] = v.x; d[h][w][1] = v.y; d[h][w][2] = v.z; d[h][w][3] = v.w;
      }
    }
  float v[4][4][4];   // v[i][j][channel]
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    float gg[4][4];
#pragma unroll
    for (int h = 0; h < 4; ++h) {       // along w
      const float f[4] = {d[h][0][c], d[h][1][c], d[h][2][c], d[h][3][c]};
      bt4(f, gg[h]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {       // along h
      const float f[4] = {gg[0][j], gg[1][j], gg[2][j], gg[3][j]};
      float o[4];
      bt4(f, o);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i][j][c] = o[i];
    }
    // the reference sums the last element in another order (elk_conv_wino_2x2_3x3_input.hxx:146)
    v[3][3][c] = __fadd_rn(__fsub_rn(__fsub_rn(d[1][1][c], d[1][3][c]), d[3][1][c]), d[3][3][c]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int a = i * 4 + j;
      if (IN_U8) {
        uint32_t b[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float f = __fmaf_rn(v[i][j][c], p.mrepS, p.tz);
          b[c] = min(__float_as_uint(__fadd_rn(f, 12582912.0f)) - 0x4B400000u, 255u);
          if (!FAST) {
            if (!(fabsf(f) < 4194304.0f)) {
              const float q = rintf(f);
              b[c] = (q < 0.0f || q > 255.0f || q != q) ? 255u : static_cast<uint32_t>(q);
            }
          }
        }
        const uint32_t w = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
        const size_t off = ((((static_cast<size_t>(a) * g.m_tiles + mt) * g.k_stages + (cb >> 3)) * 8 + (cb & 7)) * BM + row) * 16 + quad * 4;
        *reinterpret_cast<uint32_t *>(static_cast<uint8_t *>(p.a_img) + off) = live ? w : 0u;
      } else {
        const size_t stage = (static_cast<size_t>(a) * g.m_tiles + mt) * g.k_stages + cb;
        float *base = static_cast<float *>(p.a_img) + stage * (A_RAW_BYTES / 4);
        *reinterpret_cast<float4 *>(base + (quad * BM + row) * 4) = make_float4(v[i][j][0], v[i][j][1], v[i][j][2], v[i][j][3]);
      }
    }
}


// ------------------------------------------------------------------------------ fp32 direct / 1x1
// The fp32 direct convolutions (reference: elx_conv_direct_1x1_t and elx_conv_direct_t,
// src/elx_conv_direct_1x1.cpp, src/elx_conv_direct.cpp, kernels src/kernel/elk_gemm.hxx and
// src/kernel/elk_conv.hxx) run as ONE implicit GEMM on the same 3xTF32 tensor-core kernel as the
// Winograd path: rows = output pixels (n, oh, ow), K = (kh, kw, ic) in chunks of 16 channels,
// columns = output channels.
//   f32_gather_kernel   writes the operand image [m tile][K stage = (tap, channel block)][4 chunks]
//                       [128 rows][4 floats]: the input pixel each row reads for that tap, zero
//                       where the tap falls into the padding;
//   wino_gemm_kernel    with one position;
//   f32_epilogue_kernel result + bias (+ the stored output for the in-place sum), clamped to
//                       relu_bound when ReLU is on (elk_gemm.hxx:230-235), written as nChw16c.
// One thread moves the 4 channels (16 bytes) of one row.
__global__ void __launch_bounds__(128) f32_gather_kernel(const __grid_constant__ WinoInParams p) {
  const WinoGeom &g = p.g;
  const int quad = threadIdx.x & 3;
  const int t = blockIdx.x * 32 + (threadIdx.x >> 2);
  const int ks = blockIdx.y;                 // tap * CB + cb
  if (t >= g.Tpad) return;
  const int tap = ks / g.CB, cb = ks - tap * g.CB;
  const int kh = tap / g.KW, kw = tap - kh * g.KW;
  const int mt = t >> 7, row = t & 127;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (t < g.T) {
    const int hw = g.OH * g.OW;
    const int n = t / hw;
    const int r = t - n * hw;
    const int oh = r / g.OW, ow = r - oh * g.OW;
    const int ih = oh * g.stride - g.pad_t + kh, iw = ow * g.stride - g.pad_l + kw;
    if (ih >= 0 && ih < g.IH && iw >= 0 && iw < g.IW) {
      const size_t pix = ((static_cast<size_t>(n) * g.CB + cb) * g.IH + ih) * g.IW + iw;
      v = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(p.in) + pix * 16) + quad);
    }
  }
  const size_t stage = static_cast<size_t>(mt) * g.k_stages + ks;
  float *base = static_cast<float *>(p.a_img) + stage * (A_RAW_BYTES / 4);
  *reinterpret_cast<float4 *>(base + (quad * BM + row) * 4) = v;
}

// ------------------------------------------------------------------------------ batched GEMM
struct WinoGemmParams {
  // flat mode (fp32 1x1 stride 1 without padding): 3-D map over the nChw16c input -- 16 floats of a
  // pixel, the pixels of a plane, (image, channel block) planes -- read in boxes of 4 floats x 128 pixels
  alignas(64) CUtensorMap tmap_a;
  const uint8_t *a_img;     // [36][m_tiles][k_stages][A_STAGE_BYTES]
  const uint8_t *b_img;     // [36][n_tiles][k_stages][128*BN bytes]
  float *m_out;             // [36][OCB*4 channel quads][Tpad][4] fp32
  const float *scale;       // int8: [36][OCP]
  const float *shift;       // int8: [36][OCP]
  int32_t *acc_dump;        // int8, optional: [36][T][OCP]
  int *status;
  long long *trace;         // optional per-CTA timeline (SM cycle counter), 64 slots per CTA (debug)
  int m_tiles, m_pitch, n_tiles, k_stages, BN, OCB, Tpad, T, kind;
  int positions;            // A*A independent GEMMs: 36 for F(4x4,3x3), 16 for F(2x2,3x3)
  // flat mode: the whole convolution in this kernel.  Row block mt = (image, block of 128 pixels);
  // A is fetched from the user's tensor by tiled copies, the epilogue adds bias (+ stored output),
  // clamps and writes nChw16c.
  int flat, HW, tiles_img, CB;
  int rotate_k;             // tiles start their K loop at different stages (spreads the weight reads over L2)
  int producers;            // producer warps taking turns on the stages (1..3)
  int kmul;                 // fp32 with A in tensor memory: K stages (16 channels each) fetched, split and handed over as ONE
                            // pipeline step (1 or 2; divides k_stages; the kernel's KMUL).  The hand-overs between the roles cost about a
                            // thousand cycles per step whatever its size, which narrow tiles cannot hide behind their MMAs.
  int a_tmem;               // fp32, single CTAs: A planes in tensor memory (see the kernel)
  int stack;                // fp32, single CTAs, BN <= 128: the hi and lo weight rows of a K chunk lie one after the
                            // other, so hi*[hi;lo] is ONE MMA of 2*BN columns and the 3xTF32 product takes two MMAs
  int ablate;               // -DELB_TUNING builds only: bit mask of pipeline roles switched off to find the bound (results are then wrong)
  const float *bias;
  float *out;
  int with_bias, with_relu, with_sum;
  float relu_lo, relu_hi;
};
// CTA2 = true: the kernel runs as clusters of two CTAs.  A pair multiplies TWO 128-tile row blocks
// (one per CTA) by the BN transformed weights with one tcgen05.mma.cta_group::2 per K step; each
// CTA stages only ITS half of the weight rows, which halves both the bytes it pulls from L2 and the
// shared-memory reads of the B operand per MMA (the fp32 path is bound by shared-memory bandwidth:
// three tf32 MMAs per K step, each reading A and B).  Warp 1 of the peer CTA forwards "my stage is
// ready" to the leader; commits are multicast to both CTAs.
#ifdef ELB_TUNING
#define ABL(bit) ((p.ablate & (bit)) != 0)      // 1 no split, 2 no MMA, 4 no result store, 8 no A copy, 16 no B copy
#else
#define ABL(bit) false
#endif
#ifdef ELB_TUNING
#define WG_TRACE2(slot) do { if (tracing && (slot) < 64) p.trace[(gridDim.x + blockIdx.x) * 64 + (slot)] = clock64(); } while (0)
#else
#define WG_TRACE2(slot) do { } while (0)
#endif
#ifdef ELB_TUNING
#define TR0 (static_cast<uint32_t>(p.ablate) >> 16)     // first pipeline stage the timeline records (steady state instead of start-up)
#else
#define TR0 0u
#endif
#define WG_TRACE(slot) do { if (tracing && (slot) < 64) p.trace[blockIdx.x * 64 + (slot)] = clock64(); } while (0)

// KMUL: K stages per pipeline step (WinoGemmParams::kmul); a template argument because the role
// loops are single threads bound by instruction latency -- as a run-time loop count the same code
// measured 10-20 % slower at kmul = 1.
// SPEC: 0 = every mode decided at run time from the parameters; 1 / 2 = fp32 with A in tensor memory
// and stacked / plain weight rows, 3 = int8; none of them flat: the modes of the long launches,
// compiled with their flags as constants (every instruction the one-thread role loops do not
// execute is ~6 cycles; measured against the generic kernel on the same GPU: c1 GEMM 0.333 -> 0.265
// ms, VGG conv1_2 0.45 -> 0.35 ms, conv4_2 0.19 -> 0.14 ms).
// TBN: the tile's output channels as a constant (0 = p.BN): descriptors, ring geometry and the
// epilogue's block loop then fold at compile time.
template <bool CTA2, int KMUL = 1, int SPEC = 0, int TBN = 0>
__global__ void __launch_bounds__(GEMM_THREADS, 1) wino_gemm_kernel(const __grid_constant__ WinoGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  constexpr int GEMM_STAGES = CTA2 ? GEMM_STAGES_2 : GEMM_STAGES_1;
  constexpr int STAGE_BYTES = A_STAGE_BYTES + (CTA2 ? B_STAGE_MAX / 2 : B_STAGE_MAX);
  // ring of operand stages (fp32: the copy of V lands in the first half of the A region and is split
  // IN PLACE into its hi plane there and its lo plane behind it), then the epilogue constants
  uint8_t *consts_area = smem + GEMM_STAGES * STAGE_BYTES;
  uint64_t *full = reinterpret_cast<uint64_t *>(consts_area + EPI_CONST_BYTES);
  uint64_t *empty = full + GEMM_MAX_STAGES;
  uint64_t *cfull = empty + GEMM_MAX_STAGES;       // fp32: hi / lo planes of stage s are written
  uint64_t *pfull = cfull + GEMM_MAX_STAGES;       // pairs, leader only: the peer's stage s is ready
  uint64_t *tfull = pfull + GEMM_MAX_STAGES;
  uint64_t *tempty = tfull + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  // int8 only: per-epilogue-warp copies of the scale / shift slice of the current tile
  float *epi_consts = reinterpret_cast<float *>(consts_area);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BN = TBN != 0 ? TBN : p.BN;
  const int kind = SPEC == 3 ? static_cast<int>(KIND_I8) : SPEC != 0 ? static_cast<int>(KIND_F32) : p.kind;
  const bool flat = SPEC != 0 ? false : p.flat != 0;
  const bool tracing = SPEC != 0 ? false : p.trace != nullptr;      // (timelines are taken from the generic kernel)
  const uint32_t rank = CTA2 ? cluster_ctarank() : 0u;
  const bool leader = rank == 0;
  const int BNL = CTA2 ? BN / 2 : BN;                      // weight rows this CTA stages
  const uint32_t b_stage_bytes = 128u * BNL;
  const int m_units = CTA2 ? (p.m_tiles + 1) / 2 : p.m_tiles;    // row blocks (pairs of them) per position and n tile
  const int tiles_per_a = m_units * p.n_tiles;
  const int total_tiles = p.positions * tiles_per_a;
  const int first = CTA2 ? blockIdx.x >> 1 : blockIdx.x, step = CTA2 ? gridDim.x >> 1 : gridDim.x;
  constexpr uint32_t TMEM_COLS = 512;     // two accumulator buffers of up to 256 columns
  // fp32 on single CTAs: ONE accumulator buffer (columns 0..255) and, behind it, a ring of A-operand
  // slots in tensor memory, one per shared-memory stage: 16 columns of tf32 hi + 16 of lo
  constexpr uint32_t A_TMEM_COL0 = MAX_BN;
  const bool a_in_tmem = SPEC == 3 ? false : SPEC != 0 ? true : (!CTA2 && kind == KIND_F32 && p.a_tmem != 0);
  // Stacked weights (see WinoGemmParams::stack): the accumulator is 2*BN columns wide, columns
  // [BN, 2*BN) collect hi*lo and are added to [0, BN) by the epilogue.
  const bool stack = SPEC == 1 ? true : SPEC != 0 ? false : (!CTA2 && kind == KIND_F32 && p.stack != 0);
  const int acc_width = stack ? 2 * BN : BN;
  // Accumulator buffers: two (the epilogue of a tile overlaps the next tile's MMAs) unless the A
  // slots in tensor memory leave room for one only: columns [0,256) hold the accumulators (two of at
  // most 128 columns, or one wider), [256,512) the A slots.
  const int acc_bufs = (a_in_tmem && acc_width > 128) ? 1 : 2;
  const uint32_t acc_stride = a_in_tmem ? 128u : static_cast<uint32_t>(MAX_BN);
  // Ring geometry.  A stage holds A (16 KB of hi / lo planes or int8 chunks; only the raw 8 KB when
  // the planes go to tensor memory) and the BN weight rows, so tiles of fewer output channels get a
  // deeper ring: 4 stages at BN = 256 (5 with A in tensor memory), 6 at 128, up to 8 below.
  // (Measured: the extra depth changes nothing on the 64- and 128-channel VGG layers, whose stages
  // land about 1400 cycles apart however many are in flight.)
  constexpr int kmul = KMUL;                      // (KMUL > 1 is launched only with A in tensor memory, not in flat mode)
  const int ksteps = p.k_stages / kmul;           // pipeline steps per tile
  const int stage_bytes = a_in_tmem ? kmul * (A_RAW_BYTES + 128 * BN) : CTA2 ? STAGE_BYTES : A_STAGE_BYTES + 128 * BN;
  const int b_off = a_in_tmem ? kmul * A_RAW_BYTES : A_STAGE_BYTES;
  // the ring may also use the area of the int8 epilogue constants when the kernel runs fp32
  // (Staging the result of a one-accumulator tile through shared memory and bulk-storing it from
  // there, so that tensor memory is released after it has been read, was measured and is SLOWER: c1
  // GEMM 0.367 -> 0.429 ms.  The kernel is bound by shared-memory bandwidth -- per stage 48 KB of B
  // reads by the MMAs, 40 KB of incoming copies and 8 KB of splitter reads against 128 B/clk -- and
  // the detour adds 256 KB of shared-memory traffic per tile.)
  const int ring_bytes = GEMM_STAGES * STAGE_BYTES + (kind == KIND_F32 ? EPI_CONST_BYTES : 0);
  const int nstages = CTA2 ? GEMM_STAGES : min(GEMM_MAX_STAGES / kmul, ring_bytes / stage_bytes);     // (8 A slots of 16 channels in tensor memory)

  if (threadIdx.x == 0) {
    for (int s = 0; s < GEMM_MAX_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&cfull[s], GEMM_CONV_WARPS);
      mbar_init(&pfull[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], CTA2 ? 2 * GEMM_EPI_WARPS : GEMM_EPI_WARPS);      // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    if (CTA2) tmem_alloc2(tmem_slot, TMEM_COLS);
    else tmem_alloc(tmem_slot, TMEM_COLS);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (CTA2) cluster_sync_all();          // the peer's barriers exist before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  int fail_code = 0;

  if (warp < GEMM_EPI_WARP0) {
  reg_dealloc<GEMM_OTHER_REGS>();      // (one instruction for the whole warpgroup, before its warps part ways)
  if (warp != 1) {
    // -------- producers (warps 0, 2 and optionally 3): two contiguous bulk copies per stage, issued by
    // lanes 0 (A) and 1 (B).  Issuing a copy costs its lane a few hundred cycles and a pass through
    // this loop about a thousand, all of it latency of a single warp -- so the warps take turns on
    // the stages: stage i belongs to producer i mod p.producers.
    const int pw = warp == 0 ? 0 : warp - 1;
    const int np = SPEC != 0 ? GEMM_PRODUCERS_DEFAULT : p.producers;
    int turn = 0;               // whose stage the current one is
    // ring slot / phase of the current stage, kept as counters (an integer division costs this
    // one-warp loop more than the copy instructions it issues)
    int s = 0;
    uint32_t ph = 0;
    uint32_t my_pass = 0;       // (timeline only)
    auto next_stage = [&]() {
      if (++s == nstages) { s = 0; ph ^= 1u; }
      if (++turn == np) turn = 0;
    };
    bool ok = pw < np;
    if (flat) {
      // flat mode: lanes 0..3 fetch the four 16-byte channel chunks of a stage (boxes of 4 floats x
      // 128 pixels, rows past the end of the plane arrive as zeros), lane 4 the weights
      if (lane == 0) tma_prefetch_desc(&p.tmap_a);
      for (int tile = first; tile < total_tiles && ok; tile += step) {
        const int nt = tile / p.m_tiles, mt = tile - nt * p.m_tiles;
        const int n = mt / p.tiles_img, ptile = mt - n * p.tiles_img;
        const uint8_t *b_src = p.b_img + static_cast<size_t>(nt) * p.k_stages * b_stage_bytes;
        // CTAs that run side by side multiply by the same weights: each tile may start its K loop at a
        // different stage so that they do not all ask the same L2 lines at the same moment
        const int rot = p.rotate_k ? tile % p.k_stages : 0;
        for (int ks = 0; ks < p.k_stages; ++ks, next_stage()) {
          if (turn != pw) continue;
          const int ksr = ks + rot < p.k_stages ? ks + rot : ks + rot - p.k_stages;     // rotated K stage
          int w_ok = 1;
          if (lane == 0) w_ok = mbar_wait(&empty[s], ph ^ 1u, abort_flag) ? 1 : 0;
          if (!__all_sync(0xFFFFFFFFu, w_ok)) { ok = false; fail_code = ST_WAIT_TIMEOUT_PRODUCER; break; }
          uint8_t *stage = smem + s * stage_bytes;
          if (lane == 0) mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(A_RAW_BYTES) + b_stage_bytes);
          __syncwarp();
          if (lane < 4) tma_tile_3d(stage + lane * 2048, &p.tmap_a, 4 * lane, ptile * BM, n * p.CB + ksr, &full[s]);
          else if (lane == 4) tma_bulk_g2s(stage + b_off, b_src + static_cast<size_t>(ksr) * b_stage_bytes, b_stage_bytes, &full[s]);
          __syncwarp();
        }
      }
    }
    // fp32: A arrives as plain fp32 (8 KB per stage) in the raw ring; int8: straight into the stage
    const uint32_t a_gbytes = kind == KIND_F32 ? A_RAW_BYTES : A_STAGE_BYTES;
    const size_t b_pitch = static_cast<size_t>(CTA2 ? 2 : 1) * b_stage_bytes;
    // position a and index r within it of the current tile, carried along instead of divided out
    int a = first / tiles_per_a, r = first - a * tiles_per_a;
    uint32_t tcount = 0;
    for (int tile = first; tile < total_tiles && ok && !flat; tile += step, ++tcount) {
      int nt = 0, mu = r;
      while (mu >= m_units) { mu -= m_units; ++nt; }        // (one or two n tiles)
      const int mt = CTA2 ? 2 * mu + static_cast<int>(rank) : mu;
      const bool live = mt < p.m_tiles;            // an odd number of row blocks leaves the last peer without one
      const uint8_t *a_src = p.a_img + (static_cast<size_t>(a) * p.m_pitch + (live ? mt : 0)) * p.k_stages * a_gbytes;
      // pairs: the weight image holds the two halves of every stage one after the other
      const uint8_t *b_src = p.b_img + (static_cast<size_t>(a) * p.n_tiles + nt) * p.k_stages * b_pitch +
                             (CTA2 ? rank * b_stage_bytes : 0);
      const int rot = (SPEC == 0 && p.rotate_k) ? tile % ksteps : 0;      // see the flat-mode loop above
      if (pw == 0 && lane == 0 && tcount < 8) WG_TRACE(tcount);
      for (int ks = 0; ks < ksteps; ++ks, next_stage()) {
        if (turn != pw) continue;            // another producer warp's stage
        const int ksr = ks + rot < ksteps ? ks + rot : ks + rot - ksteps;
        // empty[s] is committed by the MMAs of the stage's previous use, which also implies that the
        // splitter warps are done with raw slot s
        int w_ok = 1;
        if (pw == 0 && lane == 0 && my_pass - TR0 < 12u) WG_TRACE2(2 * (my_pass - TR0));
        if (lane == 0) w_ok = mbar_wait(&empty[s], ph ^ 1u, abort_flag) ? 1 : 0;
        if (!__all_sync(0xFFFFFFFFu, w_ok)) { ok = false; fail_code = ST_WAIT_TIMEOUT_PRODUCER; break; }
        if (pw == 0 && lane == 0 && my_pass - TR0 < 12u) WG_TRACE2(2 * (my_pass - TR0) + 1);
        uint8_t *stage = smem + s * stage_bytes;
        // (the kmul K stages of a step lie one after the other in both operand images)
        if (lane == 0) mbar_arrive_expect_tx(&full[s], (live && !ABL(8) ? a_gbytes * kmul : 0u) + (ABL(16) ? 0u : b_stage_bytes * kmul));
        __syncwarp();
        if (lane == 0) {
          if (live && !ABL(8)) tma_bulk_g2s(stage, a_src + static_cast<size_t>(ksr) * a_gbytes * kmul, a_gbytes * kmul, &full[s]);
        } else if (lane == 1 && !ABL(16)) {
          tma_bulk_g2s(stage + b_off, b_src + static_cast<size_t>(ksr) * b_pitch * kmul, b_stage_bytes * kmul, &full[s]);
        }
        __syncwarp();
        if (pw == 0 && lane == 0 && my_pass - TR0 < 6u) WG_TRACE2(24 + (my_pass - TR0));
        ++my_pass;
      }
      r += step;
      while (r >= tiles_per_a) { r -= tiles_per_a; ++a; }
    }
  } else if (warp == 1) {
    // -------- MMA issuer (pairs: in the leader CTA only; the peer's lane forwards stage readiness)
    if (lane == 0 && CTA2 && !leader) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = first; tile < total_tiles && ok; tile += step) {
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const int s = static_cast<int>(it % static_cast<uint32_t>(nstages));
          const uint32_t ph = (it / static_cast<uint32_t>(nstages)) & 1u;
          if (!mbar_wait(&full[s], ph, abort_flag) ||
              (kind == KIND_F32 && !mbar_wait(&cfull[s], ph, abort_flag))) { ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; break; }
          mbar_arrive_cluster(mapa_u32(&pfull[s], 0));
        }
      }
    } else if (lane == 0) {
      const int MM = CTA2 ? 2 * BM : BM;
      const uint32_t idesc = kind == KIND_F32 ? umma_idesc(1, 2, 2, MM, BN) : umma_idesc(2, 0, 1, MM, BN);
      const uint32_t b_lbo = 16u * BNL;
      uint32_t it = 0, tcount = 0;
      // This loop is ONE thread: every instruction in it costs its full latency (measured ~330 cycles
      // per stage for two integer divisions and eight descriptor constructions alone), so the ring
      // slot and its phase are counters and the descriptors are a constant upper half OR-ed with the
      // stage's shared-memory address.
      int s = 0;
      uint32_t ph = 0;
      const uint64_t a_desc_hi = umma_desc_kmajor(0, 2048, 128), b_desc_hi = umma_desc_kmajor(0, b_lbo, 128);
      // stacked weights: a K chunk is [hi rows | lo rows] = 2*BN rows of 16 bytes
      const uint32_t st_lbo = 32u * BN;
      const uint64_t st_desc_hi = umma_desc_kmajor(0, st_lbo, 128);
      const uint32_t idesc2 = umma_idesc(1, 2, 2, MM, 2 * BN);
      const uint32_t smem_base = smem_u32(smem);
      bool ok = true;
      bool staged = false;        // the first stage of this tile was already waited for (behind the previous tile's MMAs)
      for (int tile = first; tile < total_tiles && ok; tile += step, ++tcount) {
        const uint32_t b = acc_bufs == 1 ? 0u : (tcount & 1u), tph = acc_bufs == 1 ? (tcount & 1u) : ((tcount >> 1) & 1u);
        const uint32_t d_tmem = tmem_base + b * acc_stride;
        // The waits for stage ks + 1 are issued BETWEEN the two K steps of stage ks: a wait costs this
        // thread ~300 cycles of latency even when the barrier has completed, and behind the first K
        // step's three MMAs (queued in the tensor pipe) that latency is hidden; done between the
        // stages it left the pipe idle a third of the time (measured timeline, 256-channel layer).
        // fp32 on single CTAs: the splitter warps arrive on cfull only after they have seen full (the
        // weights of the stage come with the same transaction count), so cfull alone orders this
        // thread behind both copies -- one barrier round trip less per stage.
        auto wait_stage = [&](int st, uint32_t phase) -> bool {
          if ((CTA2 || kind != KIND_F32) && !mbar_wait(&full[st], phase, abort_flag)) return false;
          if (kind == KIND_F32 && !mbar_wait(&cfull[st], phase, abort_flag)) return false;
          if (CTA2 && !mbar_wait(&pfull[st], phase, abort_flag)) return false;
          tc_fence_after_sync();
          return true;
        };
        // first the operands (long there unless `staged` already), then the accumulator buffer: the
        // wait that really blocks comes last
        if (!staged && !wait_stage(s, ph)) { ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; break; }
        staged = false;
        if (!mbar_wait(&tempty[b], tph ^ 1u, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; break; }
        tc_fence_after_sync();
        if (tcount < 8) WG_TRACE(8 + tcount);
        for (int ks = 0; ks < ksteps; ++ks, ++it) {
          if (it - TR0 < 6u) WG_TRACE2(33 + 3 * (it - TR0));
          if (ks == 0 && tcount < 8) WG_TRACE(16 + tcount);
          const uint32_t a_addr = smem_base + s * stage_bytes;
          const uint32_t b_addr = a_addr + b_off;
          const uint64_t a_desc = a_desc_hi | (a_addr >> 4), b_desc = b_desc_hi | (b_addr >> 4);   // (addresses < 256 KB: 14 bits)
          int s_next = s + 1;
          uint32_t ph_next = ph;
          if (s_next == nstages) { s_next = 0; ph_next ^= 1u; }
          // (the look-ahead crosses into the next tile: its first stage follows in the ring)
          const bool last_ks = ks + 1 == ksteps;
          const bool more = !last_ks || tile + step < total_tiles;
          if (last_ks && more) staged = true;
          if (ABL(2)) {
            if (more && !wait_stage(s_next, ph_next)) { ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; break; }
          } else if (stack) {
            // hi * [hi; lo] in one MMA of 2*BN columns, lo * hi in one of BN columns (same descriptor:
            // the first BN rows of a chunk are the hi rows)
            // (j: the K stages of this pipeline step; more than one only with A in tensor memory)
#pragma unroll
            for (int j = 0; j < kmul; ++j) {
            const uint64_t st_desc = st_desc_hi | ((b_addr + j * 128 * BN) >> 4);
#pragma unroll
            for (int k2 = 0; k2 < 2; ++k2) {
              const uint64_t bst = st_desc + ((k2 * 2 * st_lbo) >> 4);
              if (a_in_tmem) {
                const uint32_t t_hi = tmem_base + A_TMEM_COL0 + (s * kmul + j) * 32 + k2 * 8, t_lo = t_hi + 16;
#ifdef ELB_TUNING
                // timing experiments (wrong results): 32 = the lo MMA accumulates elsewhere, 64 = the two K steps do
                const uint32_t d_hi = (ABL(64) && k2) ? (d_tmem ^ 256u) : d_tmem;
                const uint32_t d_lo = ABL(32) ? (d_hi ^ 128u) : d_hi;
                if (it == TR0 + 2) WG_TRACE2(52 + (j * 2 + k2) * 3);
                umma_tf32_ts(d_hi, t_hi, bst, idesc2, (ks | j | k2) != 0 ? 1u : 0u);
                if (it == TR0 + 2) WG_TRACE2(53 + (j * 2 + k2) * 3);
                umma_tf32_ts(d_lo, t_lo, bst, idesc, 1u);
                if (it == TR0 + 2) WG_TRACE2(54 + (j * 2 + k2) * 3);
#else
                umma_tf32_ts(d_tmem, t_hi, bst, idesc2, (ks | j | k2) != 0 ? 1u : 0u);
                umma_tf32_ts(d_tmem, t_lo, bst, idesc, 1u);
#endif
              } else {
                umma_tf32(d_tmem, a_desc + ((k2 * 4096) >> 4), bst, idesc2, (ks | k2) != 0 ? 1u : 0u);
                umma_tf32(d_tmem, a_desc + ((8192 + k2 * 4096) >> 4), bst, idesc, 1u);
              }
              if (j == 0 && k2 == 0 && more && !wait_stage(s_next, ph_next)) { ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; }
            }
            }
            if (!ok) break;
          } else if (kind == KIND_F32) {
            // planes: A hi at +0, lo at +8 KB; B hi at +0, lo at +4 chunks.  K step = 2 chunks.
#pragma unroll
            for (int j = 0; j < kmul; ++j) {
#pragma unroll
            for (int k2 = 0; k2 < 2; ++k2) {
              const uint64_t ahi = a_desc + ((k2 * 4096) >> 4);
              const uint64_t alo = a_desc + ((8192 + k2 * 4096) >> 4);
              const uint64_t bhi = b_desc + ((j * 128 * BN + k2 * 2 * b_lbo) >> 4);
              const uint64_t blo = b_desc + ((j * 128 * BN + 4 * b_lbo + k2 * 2 * b_lbo) >> 4);
              if (a_in_tmem) {
                // A planes in tensor memory: hi at columns [0,16) of the stage's slot, lo at [16,32)
                const uint32_t t_hi = tmem_base + A_TMEM_COL0 + (s * kmul + j) * 32 + k2 * 8, t_lo = t_hi + 16;
                umma_tf32_ts(d_tmem, t_lo, bhi, idesc, (ks | j | k2) != 0 ? 1u : 0u);
                umma_tf32_ts(d_tmem, t_hi, blo, idesc, 1u);
                umma_tf32_ts(d_tmem, t_hi, bhi, idesc, 1u);
              } else if (CTA2) {
                umma_tf32_2cta(d_tmem, alo, bhi, idesc, (ks | k2) != 0 ? 1u : 0u);
                umma_tf32_2cta(d_tmem, ahi, blo, idesc, 1u);
                umma_tf32_2cta(d_tmem, ahi, bhi, idesc, 1u);
              } else {
                umma_tf32(d_tmem, alo, bhi, idesc, (ks | k2) != 0 ? 1u : 0u);
                umma_tf32(d_tmem, ahi, blo, idesc, 1u);
                umma_tf32(d_tmem, ahi, bhi, idesc, 1u);
              }
              if (j == 0 && k2 == 0 && more && !wait_stage(s_next, ph_next)) { ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; }
            }
            }
            if (!ok) break;
          } else {
#pragma unroll
            for (int k2 = 0; k2 < 4; ++k2) {
              const uint64_t ad = a_desc + ((k2 * 4096) >> 4);
              const uint64_t bd = b_desc + ((k2 * 2 * b_lbo) >> 4);
              if (CTA2) umma_i8_2cta(d_tmem, ad, bd, idesc, (ks | k2) != 0 ? 1u : 0u);
              else umma_i8(d_tmem, ad, bd, idesc, (ks | k2) != 0 ? 1u : 0u);
              if (k2 == 1 && more && !wait_stage(s_next, ph_next)) { ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; }
            }
            if (!ok) break;
          }
          if (CTA2) umma_commit_2cta(&empty[s]);
          else umma_commit(&empty[s]);
          if (it - TR0 < 6u) WG_TRACE2(34 + 3 * (it - TR0));
          s = s_next;
          ph = ph_next;
        }
        if (ok) {
          if (CTA2) umma_commit_2cta(&tfull[b]);
          else umma_commit(&tfull[b]);
        }
        if (tcount < 8) WG_TRACE(24 + tcount);
      }
    }
    __syncwarp();
  }
  } else if (warp >= GEMM_SPLIT_WARP0) {
    reg_dealloc<GEMM_OTHER_REGS>();
    // -------- splitter (fp32 only): raw fp32 stage -> tf32 hi plane + residual lo plane, the
    // operands of the 3xTF32 product.  hi = round-to-nearest tf32(x), lo = x - hi (exact).
    if (kind == KIND_F32) {
      const int cgrp = (warp - GEMM_SPLIT_WARP0) / GEMM_CONV_WARPS;       // this warp's group
      const int tid_c = ((warp - GEMM_SPLIT_WARP0) % GEMM_CONV_WARPS) * 32 + lane;
      uint32_t it = 0;
      int s = 0;
      uint32_t ph = 0;
      auto next_slot = [&]() { if (++s == nstages) { s = 0; ph ^= 1u; } };      // (no divisions: see the MMA loop)
      bool ok = true;
      for (int tile = first; tile < total_tiles && ok; tile += step) {
        for (int ks = 0; ks < ksteps; ++ks, ++it, next_slot()) {
          if (GEMM_CONV_GROUPS > 1 && static_cast<int>(it % GEMM_CONV_GROUPS) != cgrp) continue;       // the other group's stage
          if (tid_c == 0 && it - TR0 < 2u) WG_TRACE2(50 + (it - TR0));
          if (!mbar_wait_warp(&full[s], ph, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; break; }
          if (tid_c == 0 && it - TR0 < 8u) WG_TRACE(48 + 2 * (it - TR0));
          if (ABL(1)) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&cfull[s]);
            continue;
          }
          if (a_in_tmem) {
            // single CTAs: the planes go to TENSOR memory, row r of the stage = lane r, so the MMAs
            // read A without touching shared memory (three MMAs per K step re-reading A and B from
            // shared memory, next to the incoming copies, saturated its port).  Warp w may only
            // address lanes 32*(w%4)..: the four splitter warps cover the four quarters.
            const int quarter = warp & 3, srow = quarter * 32 + lane;
#pragma unroll
            for (int q = 0; q < kmul; ++q) {        // the K stages of this pipeline step
              const float4 *raw4 = reinterpret_cast<const float4 *>(smem + s * stage_bytes + q * A_RAW_BYTES);
              uint32_t h[16], l[16];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float4 v = raw4[j * BM + srow];
                const float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  uint32_t hb;
                  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(x[c]));
                  h[4 * j + c] = hb;
                  l[4 * j + c] = __float_as_uint(__fsub_rn(x[c], __uint_as_float(hb)));
                }
              }
              const uint32_t t_slot = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + A_TMEM_COL0 + (s * kmul + q) * 32;
              tmem_st16(t_slot, h);
              tmem_st16(t_slot + 16, l);
            }
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&cfull[s]);
            if (tid_c == 0 && it - TR0 < 8u) WG_TRACE(49 + 2 * (it - TR0));
            continue;
          }
          float4 *hi = reinterpret_cast<float4 *>(smem + s * stage_bytes);     // holds the raw fp32 values on arrival
          const float4 *raw = hi;
          float4 *lo = hi + A_RAW_BYTES / 16;
#pragma unroll
          for (int j = 0; j < A_RAW_BYTES / 16 / (GEMM_CONV_WARPS * 32); ++j) {
            const int u = tid_c + j * GEMM_CONV_WARPS * 32;
            const float4 v = raw[u];
            const float x[4] = {v.x, v.y, v.z, v.w};
            float h[4], l[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t hb;
              asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(x[c]));
              h[c] = __uint_as_float(hb);
              l[c] = __fsub_rn(x[c], h[c]);
            }
            hi[u] = make_float4(h[0], h[1], h[2], h[3]);
            lo[u] = make_float4(l[0], l[1], l[2], l[3]);
          }
          fence_proxy_async_smem();      // generic-proxy stores -> visible to the tensor core's reads
          __syncwarp();
          if (lane == 0) mbar_arrive(&cfull[s]);
          if (tid_c == 0 && it < 8) WG_TRACE(49 + 2 * it);
        }
      }
    }
  } else {
    // -------- epilogue: one tile row (= one Winograd tile) per thread, 16 channels at a time
    reg_alloc<GEMM_EPI_REGS>();
    const int quarter = warp & 3, half = (warp - GEMM_EPI_WARP0) >> 2;
    const int row = quarter * 32 + lane;
    const int OCP = p.OCB * 16;
    uint32_t tcount = 0;
    bool ok = true;
    const uint32_t tempty_leader0 = CTA2 ? mapa_u32(&tempty[0], 0) : 0u, tempty_leader1 = CTA2 ? mapa_u32(&tempty[1], 0) : 0u;
    // The tile loop exists twice (EARLY = one accumulator buffer, whose contents go to registers
    // first): compiled as one loop with both bodies the register allocator kept both sets of
    // accumulator registers alive and spilled.
    auto tile_loop = [&](auto early_tag) {
    constexpr bool EARLY = decltype(early_tag)::value;
    for (int tile = first; tile < total_tiles && ok; tile += step, ++tcount) {
      const int a = tile / tiles_per_a;
      const int r = tile - a * tiles_per_a;
      const int nt = r / m_units, mu = r - nt * m_units;
      const int mt = CTA2 ? 2 * mu + static_cast<int>(rank) : mu;
      const bool live = mt < p.m_tiles;
      const uint32_t b = acc_bufs == 1 ? 0u : (tcount & 1u), tph = acc_bufs == 1 ? (tcount & 1u) : ((tcount >> 1) & 1u);
      const int t = mt * BM + row;
      if (!mbar_wait_warp(&tfull[b], tph, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_EPILOGUE; break; }
      tc_fence_after_sync();
      if (threadIdx.x == GEMM_EPI_WARP0 * 32 && tcount < 8) WG_TRACE(32 + tcount);
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + b * acc_stride;
      // int8: this warp's slice of the per-(position, channel) constants goes to a warp-private
      // piece of shared memory first (one 16-byte load per lane and array), so that the loop below
      // reads them with broadcast shared-memory loads instead of waiting on global memory
      float *w_sc = epi_consts + (warp - GEMM_EPI_WARP0) * 2 * MAX_BN, *w_sh = w_sc + MAX_BN;
      if (kind == KIND_I8) {
        __syncwarp();
#pragma unroll
        for (int c = lane * 4; c < MAX_BN; c += 128) {
          if (c < BN) {
            const size_t gi = static_cast<size_t>(a) * OCP + nt * BN + c;
            const bool in = nt * BN + c < OCP;
            *reinterpret_cast<float4 *>(w_sc + c) = in ? __ldg(reinterpret_cast<const float4 *>(p.scale + gi)) : make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4 *>(w_sh + c) = in ? __ldg(reinterpret_cast<const float4 *>(p.shift + gi)) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
        __syncwarp();
      }
      // flat mode: this thread's row is pixel flat_pix of image flat_n
      const int flat_n = flat ? mt / p.tiles_img : 0;
      const int flat_pix = flat ? (mt - flat_n * p.tiles_img) * BM + row : 0;
      auto emit = [&](int k, uint32_t (&rr)[16], bool partner_added) {      // k-th 16-column block of this warp
        const int blk = half + 2 * k;
        const int ocb = nt * (BN / 16) + blk;
        if (stack && !partner_added) {
          // columns [BN, 2*BN) hold the hi*lo part of the same outputs
          uint32_t r2[16];
          tmem_ld16(t_addr + BN + blk * 16, r2);
          tmem_ld_wait16(r2);
#pragma unroll
          for (int i = 0; i < 16; ++i) rr[i] = __float_as_uint(__fadd_rn(__uint_as_float(rr[i]), __uint_as_float(r2[i])));
        }
        if (flat) {
          if (flat_pix < p.HW && ocb < p.OCB) {
            float4 *o = reinterpret_cast<float4 *>(p.out + ((static_cast<size_t>(flat_n) * p.OCB + ocb) * p.HW + flat_pix) * 16);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float4 v = make_float4(__uint_as_float(rr[4 * i]), __uint_as_float(rr[4 * i + 1]),
                                     __uint_as_float(rr[4 * i + 2]), __uint_as_float(rr[4 * i + 3]));
              if (p.with_bias) {
                const float4 bb = __ldg(reinterpret_cast<const float4 *>(p.bias + ocb * 16) + i);
                v.x = __fadd_rn(v.x, bb.x); v.y = __fadd_rn(v.y, bb.y); v.z = __fadd_rn(v.z, bb.z); v.w = __fadd_rn(v.w, bb.w);
              }
              if (p.with_sum) {
                const float4 pv = o[i];
                v.x = __fadd_rn(v.x, pv.x); v.y = __fadd_rn(v.y, pv.y); v.z = __fadd_rn(v.z, pv.z); v.w = __fadd_rn(v.w, pv.w);
              }
              if (p.with_relu) {
                v.x = fminf(fmaxf(v.x, p.relu_lo), p.relu_hi); v.y = fminf(fmaxf(v.y, p.relu_lo), p.relu_hi);
                v.z = fminf(fmaxf(v.z, p.relu_lo), p.relu_hi); v.w = fminf(fmaxf(v.w, p.relu_lo), p.relu_hi);
              }
              o[i] = v;
            }
          }
          return;
        }
        if (live && ocb < p.OCB && !ABL(4)) {
          float f[16];
          if (kind == KIND_F32) {
#pragma unroll
            for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(rr[i]);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 c = reinterpret_cast<const float4 *>(w_sc)[blk * 4 + i];
              const float4 h = reinterpret_cast<const float4 *>(w_sh)[blk * 4 + i];
              f[4 * i + 0] = __fmaf_rn(__int2float_rn(static_cast<int>(rr[4 * i + 0])), c.x, h.x);
              f[4 * i + 1] = __fmaf_rn(__int2float_rn(static_cast<int>(rr[4 * i + 1])), c.y, h.y);
              f[4 * i + 2] = __fmaf_rn(__int2float_rn(static_cast<int>(rr[4 * i + 2])), c.z, h.z);
              f[4 * i + 3] = __fmaf_rn(__int2float_rn(static_cast<int>(rr[4 * i + 3])), c.w, h.w);
            }
            if (SPEC == 0 && p.acc_dump && t < p.T) {
              int32_t *d = p.acc_dump + (static_cast<size_t>(a) * p.T + t) * OCP + ocb * 16;
#pragma unroll
              for (int i = 0; i < 16; ++i) d[i] = static_cast<int>(rr[i]);
            }
          }
          // M[a][channel quad][tile][4]: the 32 lanes of a warp are 32 consecutive tiles, so each of
          // the four stores below writes 512 contiguous bytes
          float *o = p.m_out + ((static_cast<size_t>(a) * p.OCB + ocb) * 4 * p.Tpad + t) * 4;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            *reinterpret_cast<float4 *>(o + static_cast<size_t>(i) * p.Tpad * 4) =
                make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
        }
      };
      // This warp owns every second 16-column block (half, half+2, ...).  The loads of tensor
      // memory are software-pipelined: while one pair of blocks is converted and stored, the next
      // pair is already on its way (wait::ld covers every load issued so far).
      const int nblk = (BN / 16 - half + 1) / 2;      // blocks of this warp (may be 0)
      const uint32_t w_addr = t_addr + half * 16;     // k-th block at +32*k columns
      if constexpr (EARLY) {
        // One accumulator buffer: the next tile's MMAs wait for this epilogue.  The whole share of the
        // warp (up to 8 blocks = 128 values per thread, stacked partners included) is read into
        // registers, tensor memory is handed back, and only then are the results converted and stored:
        // the MMAs stand still for the ~600 cycles of the loads instead of the ~9000 of the stores.
        uint32_t acc[8][16];
        const int nmain = stack ? min(nblk, 4) : nblk;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (!stack) { if (k < nblk) tmem_ld16(w_addr + k * 32, acc[k]); }
          else if (k < 4) { if (k < nblk) tmem_ld16(w_addr + k * 32, acc[k]); }
          else if (k - 4 < nblk) tmem_ld16(w_addr + BN + (k - 4) * 32, acc[k]);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) tmem_ld_wait16(acc[k]);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[b]);
        if (threadIdx.x == GEMM_EPI_WARP0 * 32 && tcount < 8) WG_TRACE(40 + tcount);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (k < nmain) {
            if (stack) {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                acc[k][i] = __float_as_uint(__fadd_rn(__uint_as_float(acc[k][i]), __uint_as_float(acc[(k + 4) & 7][i])));
            }
            emit(k, acc[k], true);
          }
        }
      } else {
      uint32_t r0[16], r1[16], r2[16], r3[16];
      if (0 < nblk) tmem_ld16(w_addr, r0);
      if (1 < nblk) tmem_ld16(w_addr + 32, r1);
#pragma unroll 1
      for (int k = 0; k < nblk; k += 4) {
        tmem_ld_wait16(r0);
        tmem_ld_wait16(r1);
        if (k + 2 < nblk) tmem_ld16(w_addr + (k + 2) * 32, r2);
        if (k + 3 < nblk) tmem_ld16(w_addr + (k + 3) * 32, r3);
        emit(k, r0, false);
        if (k + 1 < nblk) emit(k + 1, r1, false);
        tmem_ld_wait16(r2);
        tmem_ld_wait16(r3);
        if (k + 4 < nblk) tmem_ld16(w_addr + (k + 4) * 32, r0);
        if (k + 5 < nblk) tmem_ld16(w_addr + (k + 5) * 32, r1);
        if (k + 2 < nblk) emit(k + 2, r2, false);
        if (k + 3 < nblk) emit(k + 3, r3, false);
      }
      tc_fence_before_sync();
      // one arrival per warp (pairs: on the LEADER's barrier, the accumulator is reused by MMAs that
      // write both CTAs' tensor memory); the warp barrier puts every lane's tensor-memory loads in front of it
      __syncwarp();
      if (lane == 0) {
        if (CTA2) mbar_arrive_cluster(b ? tempty_leader1 : tempty_leader0);
        else mbar_arrive(&tempty[b]);
      }
      if (threadIdx.x == GEMM_EPI_WARP0 * 32 && tcount < 8) WG_TRACE(40 + tcount);
      }
    }
    };
    if (acc_bufs == 1) tile_loop(std::true_type{});
    else tile_loop(std::false_type{});
  }

  if (fail_code != 0) atomicCAS(p.status, 0, fail_code);
  tc_fence_before_sync();
  __syncthreads();
  if (CTA2) cluster_sync_all();    // nobody leaves (or frees tensor memory) while the other CTA may still signal it
  tc_fence_after_sync();
  if (warp == 1) {
    __syncwarp();
    if (CTA2) tmem_dealloc2(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

constexpr int GEMM_SMEM_BYTES_1 = GEMM_STAGES_1 * (A_STAGE_BYTES + B_STAGE_MAX) + EPI_CONST_BYTES + (4 * GEMM_MAX_STAGES + 4) * 8 + 16 + 128;
constexpr int GEMM_SMEM_BYTES_2 = GEMM_STAGES_2 * (A_STAGE_BYTES + B_STAGE_MAX / 2) + EPI_CONST_BYTES + (4 * GEMM_MAX_STAGES + 4) * 8 + 16 + 128;
constexpr int GEMM_SMEM_BYTES = GEMM_SMEM_BYTES_1 > GEMM_SMEM_BYTES_2 ? GEMM_SMEM_BYTES_1 : GEMM_SMEM_BYTES_2;
static_assert(GEMM_SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
static_assert(GEMM_EPI_WARPS * 2 * MAX_BN * 4 <= EPI_CONST_BYTES, "epilogue constants must fit their area");

// The single-CTA instantiations of the GEMM kernel: the generic one, the two K stages per step one,
// and the ones specialised for fp32 with A in tensor memory (see SPEC).
inline cudaError_t gemm_set_attributes() {
  cudaError_t e = cudaSuccess;
  auto set = [&](const void *f) {
    if (e == cudaSuccess) e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES);
  };
  set(reinterpret_cast<const void *>(wino_gemm_kernel<false, 1, 0>));
  set(reinterpret_cast<const void *>(wino_gemm_kernel<false, 1, 1>));
  set(reinterpret_cast<const void *>(wino_gemm_kernel<false, 1, 2>));
  set(reinterpret_cast<const void *>(wino_gemm_kernel<false, 2, 0>));
  set(reinterpret_cast<const void *>(wino_gemm_kernel<false, 2, 1>));
  set(reinterpret_cast<const void *>(wino_gemm_kernel<false, 2, 1, 64>));
  set(reinterpret_cast<const void *>(wino_gemm_kernel<false, 2, 1, 128>));
  set(reinterpret_cast<const void *>(wino_gemm_kernel<false, 1, 2, 256>));
  set(reinterpret_cast<const void *>(wino_gemm_kernel<false, 1, 3, 256>));
  return e;
}
inline void gemm_launch(const WinoGemmParams &gp, int ctas, cudaStream_t s) {
  // specialised kernels: fp32, A in tensor memory, not flat, no timeline requested
  const bool plain = !gp.flat && !gp.trace && !gp.ablate && !gp.rotate_k && gp.producers == GEMM_PRODUCERS_DEFAULT;
  if (plain && gp.kind == KIND_I8 && gp.BN == 256 && !gp.acc_dump) {
    wino_gemm_kernel<false, 1, 3, 256><<<ctas, GEMM_THREADS, GEMM_SMEM_BYTES, s>>>(gp);
    return;
  }
  const int spec = (plain && gp.kind == KIND_F32 && gp.a_tmem) ? (gp.stack ? 1 : 2) : 0;
  if (gp.kmul == 2) {
    if (spec == 1 && gp.BN == 64) wino_gemm_kernel<false, 2, 1, 64><<<ctas, GEMM_THREADS, GEMM_SMEM_BYTES, s>>>(gp);
    else if (spec == 1 && gp.BN == 128) wino_gemm_kernel<false, 2, 1, 128><<<ctas, GEMM_THREADS, GEMM_SMEM_BYTES, s>>>(gp);
    else if (spec == 1) wino_gemm_kernel<false, 2, 1><<<ctas, GEMM_THREADS, GEMM_SMEM_BYTES, s>>>(gp);
    else wino_gemm_kernel<false, 2, 0><<<ctas, GEMM_THREADS, GEMM_SMEM_BYTES, s>>>(gp);
  } else if (spec == 1) {
    wino_gemm_kernel<false, 1, 1><<<ctas, GEMM_THREADS, GEMM_SMEM_BYTES, s>>>(gp);
  } else if (spec == 2 && gp.BN == 256) {
    wino_gemm_kernel<false, 1, 2, 256><<<ctas, GEMM_THREADS, GEMM_SMEM_BYTES, s>>>(gp);
  } else if (spec == 2) {
    wino_gemm_kernel<false, 1, 2><<<ctas, GEMM_THREADS, GEMM_SMEM_BYTES, s>>>(gp);
  } else {
    wino_gemm_kernel<false, 1, 0><<<ctas, GEMM_THREADS, GEMM_SMEM_BYTES, s>>>(gp);
  }
}

// ------------------------------------------------------------------------------ output transform
struct WinoOutParams {
  const float *m_in;    // [36][OCB*4 channel quads][Tpad][4]
  const float *bias;    // [OCP] or null
  void *out;            // nChw16c f32 / u8 / s8, first image of the chunk
  WinoGeom g;
  int out_type, with_bias, with_relu, with_sum;
  float orepS, oz;
  float relu_lo, relu_hi;   // fp32 direct convolution only (the Winograd output transform uses a literal 0)
};

__global__ void __launch_bounds__(TRANS_THREADS) wino_output_kernel(const __grid_constant__ WinoOutParams p) {
  const WinoGeom &g = p.g;
  const int quad = threadIdx.x & 3;
  const int t = blockIdx.x * TRANS_TILES + (threadIdx.x >> 2);
  const int ocb = blockIdx.y;
  if (t >= g.T) return;
  const int n = t / (g.ht * g.wt);
  const int r = t - n * g.ht * g.wt;
  const int th = r / g.wt, tw = r - th * g.wt;

  // all 36 loads first (bytes in flight, see the input transform), then the pass along h
  float4 raw[6][6];
  // (a hand-made "base + position * step" for these addresses measured slower: 0.107 -> 0.113 ms on c1)
#pragma unroll
  for (int i = 0; i < 6; ++i)
#pragma unroll
    for (int j = 0; j < 6; ++j)
      raw[i][j] = __ldg(reinterpret_cast<const float4 *>(
          p.m_in + (((static_cast<size_t>(i * 6 + j) * g.OCB + ocb) * 4 + quad) * g.Tpad + t) * 4));
  f32x2 m[4][6][2];   // after the pass along h: m[i][j][channel pair]
#pragma unroll
  for (int j = 0; j < 6; ++j) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      f32x2 f[6], q[4];
#pragma unroll
      for (int i = 0; i < 6; ++i) f[i] = c == 0 ? pack2(raw[i][j].x, raw[i][j].y) : pack2(raw[i][j].z, raw[i][j].w);
      at6x2(f, q);
#pragma unroll
      for (int i = 0; i < 4; ++i) m[i][j][c] = q[i];
    }
  }
  float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (p.with_bias && p.bias) bias4 = *reinterpret_cast<const float4 *>(p.bias + ocb * 16 + quad * 4);
  const float bb[4] = {bias4.x, bias4.y, bias4.z, bias4.w};
  const f32x2 bias_lo = pack2(bias4.x, bias4.y), bias_hi = pack2(bias4.z, bias4.w);
  const int elt = p.out_type == OUT_F32 ? 4 : 1;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int oh = 4 * th + i;
    float y[4][4];
    f32x2 yp[4][2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const f32x2 f[6] = {m[i][0][c], m[i][1][c], m[i][2][c], m[i][3][c], m[i][4][c], m[i][5][c]};
      f32x2 q[4];
      at6x2(f, q);
#pragma unroll
      for (int j = 0; j < 4; ++j) { yp[j][c] = q[j]; unpack2(q[j], y[j][2 * c], y[j][2 * c + 1]); }
    }
    if (oh >= g.OH) continue;
    if (p.out_type == OUT_F32 && !p.with_sum) {
      // the common case (fp32 result, no residual): bias on channel pairs, one address per row
      float *row0 = static_cast<float *>(p.out) +
                    ((((static_cast<size_t>(n) * g.OCB + ocb) * g.OH + oh) * g.OW + 4 * tw) * 16 + quad * 4);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (4 * tw + j >= g.OW) continue;
        float4 v;
        if (p.with_bias) {
          unpack2(add2(yp[j][0], bias_lo), v.x, v.y);
          unpack2(add2(yp[j][1], bias_hi), v.z, v.w);
        } else {
          v = make_float4(y[j][0], y[j][1], y[j][2], y[j][3]);
        }
        if (p.with_relu) { v.x = fmaxf(v.x, 0.0f); v.y = fmaxf(v.y, 0.0f); v.z = fmaxf(v.z, 0.0f); v.w = fmaxf(v.w, 0.0f); }
        *reinterpret_cast<float4 *>(row0 + j * 16) = v;
      }
      continue;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int ow = 4 * tw + j;
      if (ow >= g.OW) continue;
      const size_t pix = ((static_cast<size_t>(n) * g.OCB + ocb) * g.OH + oh) * g.OW + ow;
      uint8_t *dst = static_cast<uint8_t *>(p.out) + (pix * 16 + quad * 4) * elt;
      float f[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        f[c] = y[j][c];
        if (p.with_bias) f[c] = __fadd_rn(f[c], bb[c]);
        if (p.out_type != OUT_F32) f[c] = __fmaf_rn(f[c], p.orepS, p.oz);
      }
      if (p.with_sum) {
        if (p.out_type == OUT_F32) {
          const float4 pv = *reinterpret_cast<const float4 *>(dst);
          f[0] = __fadd_rn(f[0], pv.x); f[1] = __fadd_rn(f[1], pv.y);
          f[2] = __fadd_rn(f[2], pv.z); f[3] = __fadd_rn(f[3], pv.w);
        } else {
          const uint32_t pv = *reinterpret_cast<const uint32_t *>(dst);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint32_t b = (pv >> (8 * c)) & 0xFFu;
            f[c] = __fadd_rn(f[c], p.out_type == OUT_U8 ? static_cast<float>(b)
                                                        : static_cast<float>(static_cast<int>(static_cast<int8_t>(b))));
          }
        }
      }
      if (p.with_relu) {          // literal zero: relu_bound is not used on this path in the reference
#pragma unroll
        for (int c = 0; c < 4; ++c) f[c] = fmaxf(f[c], 0.0f);
      }
      if (p.out_type == OUT_F32) {
        *reinterpret_cast<float4 *>(dst) = make_float4(f[0], f[1], f[2], f[3]);
      } else {
        uint32_t w = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float q = rintf(f[c]);
          uint32_t b;
          if (p.out_type == OUT_U8) b = (q < 0.0f || q > 255.0f) ? 255u : static_cast<uint32_t>(q);
          else b = static_cast<uint32_t>(static_cast<int>(fminf(fmaxf(q, -128.0f), 127.0f))) & 0xFFu;
          w |= b << (8 * c);
        }
        *reinterpret_cast<uint32_t *>(dst) = w;
      }
    }
  }
}


// F(2x2,3x3) output transform: one thread = one tile x 4 channels.  Sums in the reference's order
// (src/kernel/elk_conv_wino_2x2_3x3_output.hxx:89-97); the epilogue is the one above except that
// u8 / s8 results are rounded toward minus infinity (:145-153), where every other tile size
// rounds to nearest even.
__global__ void __launch_bounds__(128) wino4_output_kernel(const __grid_constant__ WinoOutParams p) {
  const WinoGeom &g = p.g;
  const int quad = threadIdx.x & 3;
  const int t = blockIdx.x * 32 + (threadIdx.x >> 2);
  const int ocb = blockIdx.y;
  if (t >= g.T) return;
  const int n = t / (g.ht * g.wt);
  const int r = t - n * g.ht * g.wt;
  const int th = r / g.wt, tw = r - th * g.wt;
  float4 raw[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      raw[i][j] = __ldg(reinterpret_cast<const float4 *>(
          p.m_in + (((static_cast<size_t>(i * 4 + j) * g.OCB + ocb) * 4 + quad) * g.Tpad + t) * 4));
  float y[2][2][4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    float m[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        m[i][j] = c == 0 ? raw[i][j].x : c == 1 ? raw[i][j].y : c == 2 ? raw[i][j].z : raw[i][j].w;
    const float c0 = __fadd_rn(__fadd_rn(m[1][0], m[1][1]), m[1][2]);
    const float c1 = __fadd_rn(__fadd_rn(m[2][0], m[2][1]), m[2][2]);
    const float c2 = __fsub_rn(__fadd_rn(m[1][2], m[1][3]), m[1][1]);
    const float c3 = __fsub_rn(__fadd_rn(m[2][2], m[2][3]), m[2][1]);
    y[0][0][c] = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(m[0][0], m[0][1]), m[0][2]), c0), c1);
    y[1][0][c] = __fadd_rn(__fadd_rn(__fadd_rn(__fsub_rn(c1, c0), m[3][0]), m[3][1]), m[3][2]);
    y[0][1][c] = __fadd_rn(__fadd_rn(__fadd_rn(__fsub_rn(m[0][2], m[0][1]), m[0][3]), c2), c3);
    y[1][1][c] = __fadd_rn(__fadd_rn(__fsub_rn(__fsub_rn(c3, c2), m[3][1]), m[3][2]), m[3][3]);
  }
  float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (p.with_bias && p.bias) bias4 = *reinterpret_cast<const float4 *>(p.bias + ocb * 16 + quad * 4);
  const float bb[4] = {bias4.x, bias4.y, bias4.z, bias4.w};
  const int elt = p.out_type == OUT_F32 ? 4 : 1;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int oh = 2 * th + i, ow = 2 * tw + j;
      if (oh >= g.OH || ow >= g.OW) continue;
      const size_t pix = ((static_cast<size_t>(n) * g.OCB + ocb) * g.OH + oh) * g.OW + ow;
      uint8_t *dst = static_cast<uint8_t *>(p.out) + (pix * 16 + quad * 4) * elt;
      float f[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        f[c] = y[i][j][c];
        if (p.with_bias) f[c] = __fadd_rn(f[c], bb[c]);
        if (p.out_type != OUT_F32) f[c] = __fmaf_rn(f[c], p.orepS, p.oz);
      }
      if (p.with_sum) {
        if (p.out_type == OUT_F32) {
          const float4 pv = *reinterpret_cast<const float4 *>(dst);
          f[0] = __fadd_rn(f[0], pv.x); f[1] = __fadd_rn(f[1], pv.y);
          f[2] = __fadd_rn(f[2], pv.z); f[3] = __fadd_rn(f[3], pv.w);
        } else {
          const uint32_t pv = *reinterpret_cast<const uint32_t *>(dst);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint32_t b = (pv >> (8 * c)) & 0xFFu;
            f[c] = __fadd_rn(f[c], p.out_type == OUT_U8 ? static_cast<float>(b)
                                                        : static_cast<float>(static_cast<int>(static_cast<int8_t>(b))));
          }
        }
      }
      if (p.with_relu) {
#pragma unroll
        for (int c = 0; c < 4; ++c) f[c] = fmaxf(f[c], 0.0f);
      }
      if (p.out_type == OUT_F32) {
        *reinterpret_cast<float4 *>(dst) = make_float4(f[0], f[1], f[2], f[3]);
      } else {
        uint32_t w = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float q = floorf(f[c]);
          uint32_t b;
          // u8: the unsigned conversion of a negative value saturates to 255
          if (p.out_type == OUT_U8) b = (q >= 0.0f && q <= 255.0f) ? static_cast<uint32_t>(q) : 255u;
          else b = static_cast<uint32_t>(static_cast<int>(fminf(fmaxf(q, -128.0f), 127.0f))) & 0xFFu;
          w |= b << (8 * c);
        }
        *reinterpret_cast<uint32_t *>(dst) = w;
      }
    }
}


// fp32 direct convolution: GEMM result [OCB*4 channel quads][Tpad][4] -> nChw16c with the fused
// epilogue.  Row t of the GEMM is output pixel (n, oh, ow) in nChw16c order.
__global__ void __launch_bounds__(128) f32_epilogue_kernel(const __grid_constant__ WinoOutParams p) {
  const WinoGeom &g = p.g;
  const int quad = threadIdx.x & 3;
  const int t = blockIdx.x * 32 + (threadIdx.x >> 2);
  const int ocb = blockIdx.y;
  if (t >= g.T) return;
  const int hw = g.OH * g.OW;
  const int n = t / hw;
  const int r = t - n * hw;
  float4 v = __ldg(reinterpret_cast<const float4 *>(p.m_in + ((static_cast<size_t>(ocb) * 4 + quad) * g.Tpad + t) * 4));
  if (p.with_bias && p.bias) {
    const float4 b = *reinterpret_cast<const float4 *>(p.bias + ocb * 16 + quad * 4);
    v.x = __fadd_rn(v.x, b.x); v.y = __fadd_rn(v.y, b.y); v.z = __fadd_rn(v.z, b.z); v.w = __fadd_rn(v.w, b.w);
  }
  float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(p.out) +
                                           ((static_cast<size_t>(n) * g.OCB + ocb) * hw + r) * 16) + quad;
  if (p.with_sum) {
    const float4 pv = *dst;
    v.x = __fadd_rn(v.x, pv.x); v.y = __fadd_rn(v.y, pv.y); v.z = __fadd_rn(v.z, pv.z); v.w = __fadd_rn(v.w, pv.w);
  }
  if (p.with_relu) {
    v.x = fminf(fmaxf(v.x, p.relu_lo), p.relu_hi); v.y = fminf(fmaxf(v.y, p.relu_lo), p.relu_hi);
    v.z = fminf(fmaxf(v.z, p.relu_lo), p.relu_hi); v.w = fminf(fmaxf(v.w, p.relu_lo), p.relu_hi);
  }
  *dst = v;
}

// ------------------------------------------------------------------------------ host side
inline float tf32_rna(float x) {            // what cvt.rna.tf32.f32 returns for finite x
  uint32_t u;
  std::memcpy(&u, &x, 4);
  u = (u + 0x1000u) & 0xFFFFE000u;
  float r;
  std::memcpy(&r, &u, 4);
  return r;
}

// G with the reference's constants and order (src/kernel/elk_conv_wino_4x4_3x3_weights.hxx:25-58)
inline void g3(float f0, float f1, float f2, float o[6]) {
  const float z0 = 0.26890756302521f, z1 = -0.688403361344538f, z2 = 0.119514472455649f,
              z3 = 1.13777777777778f, z4 = 0.430252100840336f, z5 = 0.179271708683473f;
  // In the reference build the first product, z0*f2, is the one fused into both of its uses;
  // z1*f0 and z2*f0 stay rounded products.  (Pinned against the reference's int8 Winograd
  // output: with this structure the quantised weights agree everywhere, with the other one
  // roughly one s8 code in 10^5 flips.)
  volatile float p1 = z1 * f0;
  volatile float p2 = z2 * f0;
  const float t1 = std::fmaf(-z0, f2, p1);
  const float t2 = std::fmaf(z0, f2, p2);
  volatile float o0 = z3 * f0;
  o[0] = o0;
  o[1] = std::fmaf(-z4, f1, t1);
  o[2] = std::fmaf(z4, f1, t1);
  o[3] = std::fmaf(z5, f1, t2);
  o[4] = std::fmaf(-z5, f1, t2);
  o[5] = f2;
}

// F(2x2,3x3): G rows (1,0,0), (.5,-.5,.5), (.5,.5,.5), (0,0,1); kw direction first, the sums in the
// reference's order, the power-of-two factors applied last (exact)
// (src/kernel/elk_conv_wino_2x2_3x3_weights.hxx:73-107).
inline void weights_tile4(const float (&g)[3][3], float (&u)[4][4]) {
  const float cs[4] = {1.0f, 0.5f, 0.5f, 1.0f};
  float r[3][4];
  for (int x = 0; x < 3; ++x) {
    volatile float d = g[x][0] - g[x][1];
    volatile float a = g[x][0] + g[x][1];
    volatile float s1 = d + g[x][2];
    volatile float s2 = a + g[x][2];
    r[x][0] = g[x][0]; r[x][1] = s1; r[x][2] = s2; r[x][3] = g[x][2];
  }
  for (int j = 0; j < 4; ++j) {
    volatile float d = r[0][j] - r[1][j];
    volatile float a = r[0][j] + r[1][j];
    volatile float s1 = d + r[2][j];
    volatile float s2 = a + r[2][j];
    u[0][j] = cs[j] * r[0][j];
    u[1][j] = cs[j] * 0.5f * s1;
    u[2][j] = cs[j] * 0.5f * s2;
    u[3][j] = cs[j] * r[2][j];
  }
}

// U[a][oc][ic] = G g G^T in the reference's order, zero for padded channels; a = hA*A + wA.
std::vector<float> transform_weights(const float *w, int oc, int ic, int OCP, int ICP, int A) {
  std::vector<float> u(static_cast<size_t>(A) * A * OCP * ICP, 0.0f);
  const int I2 = ICP / 16;
  for (int o = 0; o < oc; ++o)
    for (int i = 0; i < ic; ++i) {
      float g[3][3], m[6][3], r[6];
      for (int kh = 0; kh < 3; ++kh)
        for (int kw = 0; kw < 3; ++kw) g[kh][kw] = w[host::w_index(I2, 3, 3, o, i, kh, kw)];
      if (A == 4) {
        float u4[4][4];
        weights_tile4(g, u4);
        for (int a = 0; a < 4; ++a)
          for (int b = 0; b < 4; ++b) u[(static_cast<size_t>(a * 4 + b) * OCP + o) * ICP + i] = u4[a][b];
        continue;
      }
      for (int kw = 0; kw < 3; ++kw) {
        g3(g[0][kw], g[1][kw], g[2][kw], r);
        for (int a = 0; a < 6; ++a) m[a][kw] = r[a];
      }
      for (int a = 0; a < 6; ++a) {
        g3(m[a][0], m[a][1], m[a][2], r);
        for (int b = 0; b < 6; ++b) u[(static_cast<size_t>(a * 6 + b) * OCP + o) * ICP + i] = r[b];
      }
    }
  return u;
}

// Tuning switches of the GEMM kernel (tune_env: overridable only in -DELB_TUNING builds).
// fp32: A in tensor memory relieves the shared-memory port and deepens the ring; with an accumulator
// wider than 128 columns it leaves room for one accumulator buffer only, whose epilogue therefore
// hands tensor memory back before it stores (see the kernel).  The Winograd / direct GEMMs (not flat)
// always use it: they then run the kernels specialised for it, which beat the generic kernel with A
// in shared memory on every layer of the VGG-16 stack (same GPU, 32 images: conv2_1 GEMM 0.176 ->
// 0.126 ms, conv3_1 0.116 -> 0.087 ms; the layers from 256 input channels up had it before).  The
// flat 1x1 kernel keeps the rule it was measured with: long K loops, or a CTA that runs a single tile
// (1x1 benchmark layer 68.9 -> 55.9 us), or accumulators of at most 128 columns.
inline int tune_a_tmem(int kind, int k_stages, long long total_tiles, int num_sms, int acc_width, bool flat) {
  const int dflt = kind != KIND_F32 ? 0 : !flat ? 1 : (k_stages >= 16 || total_tiles <= num_sms || acc_width <= 128) ? 1 : 0;
  return tune_env("ELB_F32_A_TMEM", dflt) > 0 ? 1 : 0;
}
// K rotation spreads the weight reads of CTAs running side by side over L2; measured without effect
// on this kernel (the weights of one position are 0.5 MB and stay hot), so it is off.
inline int tune_rotate_k() {
  return tune_env("ELB_WINO_ROTATE_K", 0) > 0 ? 1 : 0;
}
// K stages per pipeline step (WinoGemmParams::kmul).  Tiles of at most 128 output channels spend
// more time handing a stage from role to role than multiplying it, so they move two stages at a
// time (VGG conv1_2, 64 -> 64 channels: GEMM 0.610 -> 0.447 ms); 256-wide tiles are bound by their
// MMAs and keep the deeper ring of single stages.
inline int tune_kmul(int kind, int a_tmem, int k_stages, int BN) {
  int v = tune_env("ELB_WINO_KMUL", (kind == KIND_F32 && a_tmem && BN <= 128) ? 2 : 1);
  if (kind != KIND_F32 || !a_tmem || v != 2) return 1;
  const int ring_bytes = GEMM_STAGES_1 * (A_STAGE_BYTES + B_STAGE_MAX) + EPI_CONST_BYTES;
  while (v > 1 && (k_stages % v != 0 || ring_bytes / (v * (A_RAW_BYTES + 128 * BN)) < 2)) v /= 2;
  return v;
}
// Producer warps taking turns on the stages (1..GEMM_PRODUCERS).
inline int tune_producers() {
  const int n = tune_env("ELB_WINO_PRODUCERS", GEMM_PRODUCERS_DEFAULT);
  return n < 1 ? 1 : n > GEMM_PRODUCERS ? GEMM_PRODUCERS : n;
}

}  // namespace

struct WinoImpl {
  int kind = KIND_F32;
  WinoGeom g{};            // geometry of a full chunk
  int N = 0, imgs_per_chunk = 0;
  int ICP = 0, OCP = 0, BN = 0, n_tiles = 0;
  int out_type = OUT_F32, with_bias = 0, with_relu = 0, with_sum = 0;
  float orepS = 1.f, oz = 0.f, mrepS = 1.f, tz = 0.f;
  float relu_lo = 0.f, relu_hi = 3.402823466e38f;
  bool direct = false;     // fp32 direct convolution on the GEMM kernel (g.A == 1)
  bool flat = false;       // ... 1x1 stride 1 without padding: the GEMM kernel alone, reading the user's tensor
  bool small_ic = false;   // fp32 Winograd asked for a layer with <= 4 input channels: the CUDA-core direct kernel
  void *d_w_small = nullptr;
  int ic_real = 0;
  size_t in_img_bytes = 0, out_img_bytes = 0;
  size_t a_bytes = 0, b_bytes = 0, m_bytes = 0;
  bool cta2 = false;       // GEMM on pairs of CTAs (weight rows split over the pair)
  bool stack = false;      // fp32, BN <= 128: hi and lo weight rows stacked per K chunk (two MMAs per K step instead of three)
  int max_clusters = 0;    // pairs the device holds at once
  void *d_a = nullptr, *d_b = nullptr, *d_m = nullptr, *d_bias = nullptr, *d_scale = nullptr, *d_shift = nullptr;
};

int wino_setup(WinoPlan &pl, const elb_conv_desc_t &d, elb_conv_info_t &info, std::string &err) {
  const bool direct = info.kernel == ELB_KERNEL_F32_DIRECT_UMMA;
  if (!direct) {
    if (d.pad_t != 1 || d.pad_l != 1) { err = "Winograd needs pad 1"; return ELB_UNIMPLEMENTED; }
    if (info.tile_size != 6 && info.tile_size != 4) { err = "Winograd tile_size must be 6 or 4"; return ELB_UNIMPLEMENTED; }
  }
  WinoImpl *w = new WinoImpl();
  pl.impl = w;
  w->direct = direct;
  // 1x1, stride 1, no padding: the operand rows are the input pixels themselves
  w->flat = direct && d.kh == 1 && d.kw == 1 && d.stride_h == 1 && d.stride_w == 1 && d.pad_t == 0 && d.pad_l == 0 &&
            d.oh == d.ih && d.ow == d.iw && !(getenv("ELB_F32_NO_FLAT") && atoi(getenv("ELB_F32_NO_FLAT")) > 0);
  w->relu_lo = d.relu_lower; w->relu_hi = d.relu_upper;
  w->kind = info.kernel == ELB_KERNEL_WINO_I8_UMMA ? KIND_I8 : KIND_F32;
  // fp32 Winograd on a layer with at most four input channels (an image network's first layer): 13 of
  // the 16 transformed channels would be zeros; the direct CUDA-core kernel does it in one pass over
  // the input and the output
  w->small_ic = info.kernel == ELB_KERNEL_WINO_F32_UMMA && d.ic <= 4 && host::alignup(d.oc, V) <= 256 &&
                f32_small_ic_smem_bytes(host::alignup(d.oc, V) / V) <= 200 * 1024;
  w->ic_real = d.ic;
  if (w->small_ic) info.kernel = ELB_KERNEL_F32_SMALL_IC;
  if (w->kind == KIND_I8) {
    if (d.sampling_kind != ELB_CALIBRATED) { err = "int8 Winograd: only CALIBRATED sampling is implemented"; return ELB_UNIMPLEMENTED; }
    if (d.input_z != 0.0f) { err = "Support abs-max scaling for input only in Conv Winograd"; return ELB_UNIMPLEMENTED; }  // src/eld_conv.cpp:224-229
  }
  w->N = d.n;
  w->ICP = host::alignup(d.ic, V);
  w->OCP = host::alignup(d.oc, V);
  WinoGeom &g = w->g;
  g.CB = w->ICP / V; g.OCB = w->OCP / V;
  g.IH = d.ih; g.IW = d.iw; g.OH = d.oh; g.OW = d.ow;
  g.A = direct ? 1 : info.tile_size;
  const int OT = direct ? 1 : g.A - 2, AA = g.A * g.A;
  g.ht = (d.oh + OT - 1) / OT; g.wt = (d.ow + OT - 1) / OT;      // direct: one GEMM row per output pixel
  g.pad_t = d.pad_t; g.pad_l = d.pad_l;
  g.KH = d.kh; g.KW = d.kw; g.stride = d.stride_h; g.taps = direct ? d.kh * d.kw : 1;
  g.k_stages = w->kind == KIND_F32 ? g.CB * g.taps : (g.CB + 7) / 8;
  w->n_tiles = (w->OCP + MAX_BN - 1) / MAX_BN;
  w->BN = host::alignup((w->OCP + w->n_tiles - 1) / w->n_tiles, 16);
  // chunk of whole images whose transform-domain buffers fit the budget
  const size_t tiles_img = static_cast<size_t>(g.ht) * g.wt;
  const size_t a_gbytes = w->kind == KIND_F32 ? A_RAW_BYTES : A_STAGE_BYTES;    // one stage of A in global memory
  const size_t per_tile = static_cast<size_t>(AA) * (static_cast<size_t>(g.k_stages) * a_gbytes / BM + static_cast<size_t>(w->OCP) * 4);
  size_t budget = WORKSPACE_BUDGET;
  budget = static_cast<size_t>(tune_env("ELB_WINO_CHUNK_MB", static_cast<int>(budget >> 20))) << 20;
  size_t imgs = budget / (per_tile * tiles_img);
  if (imgs < 1) imgs = 1;
  if (imgs > static_cast<size_t>(d.n) || w->flat || w->small_ic) imgs = d.n;       // (no transform-domain buffers in these modes)
  w->imgs_per_chunk = static_cast<int>(imgs);
  g.N = w->imgs_per_chunk;
  g.T = static_cast<int>(imgs * tiles_img);
  g.m_tiles = (g.T + BM - 1) / BM;
  g.Tpad = g.m_tiles * BM;
  w->a_bytes = static_cast<size_t>(AA) * g.m_tiles * g.k_stages * a_gbytes;
  w->b_bytes = static_cast<size_t>(AA) * w->n_tiles * g.k_stages * 128 * w->BN;
  w->m_bytes = static_cast<size_t>(AA) * g.OCB * g.Tpad * 16 * 4;
  if (w->flat || w->small_ic) { w->a_bytes = 256; w->m_bytes = 256; }
  w->in_img_bytes = static_cast<size_t>(w->ICP) * d.ih * d.iw * (d.dt_input == ELB_F32 ? 4 : 1);
  w->out_type = d.dt_output == ELB_F32 ? OUT_F32 : d.dt_output == ELB_U8 ? OUT_U8 : OUT_S8;
  w->out_img_bytes = static_cast<size_t>(w->OCP) * d.oh * d.ow * (w->out_type == OUT_F32 ? 4 : 1);
  w->with_bias = d.with_bias; w->with_relu = d.with_relu; w->with_sum = d.with_ip_sum;
  if (w->out_type != OUT_F32) {
    w->orepS = 1.0f / d.output_scale;
    w->oz = w->kind == KIND_I8 ? std::ceil(d.output_z) : d.output_z;      // src/elx_int8_conv_wino.cpp:276
  }
  if (w->kind == KIND_I8) {
    w->tz = std::ceil(d.tinput_z);                                       // src/elx_int8_conv_wino.cpp:274
    volatile float rep = 1.0f / d.tinput_scale;
    w->mrepS = d.input_scale * rep;                                      // src/elx_conv_wino_trans_input.cpp:617
  }
  cudaError_t e = gemm_set_attributes();
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(wino_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES);
  if (e != cudaSuccess) { err = std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e); return ELB_GENERAL_ERROR; }
  {
    // Pairs of CTAs are opt-in (ELB_WINO_CTA2=1): measured on B200 they are not faster than single
    // CTAs (VGG conv3_2 GEMM 0.417 ms either way, int8 0.152 vs 0.120 ms), because the kernel is
    // bound by the hi/lo splitter warps and the epilogue, not by the bytes of B.
    const char *on2 = getenv("ELB_WINO_CTA2");
    w->cta2 = g.m_tiles >= 4 && w->BN % 32 == 0 && on2 && atoi(on2) > 0 && !w->flat;
    if (w->cta2) {
      int dev = 0, sms = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(2 * (sms / 2));
      cfg.blockDim = dim3(GEMM_THREADS);
      cfg.dynamicSmemBytes = GEMM_SMEM_BYTES;
      cudaLaunchAttribute at{};
      at.id = cudaLaunchAttributeClusterDimension;
      at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
      cfg.attrs = &at;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, wino_gemm_kernel<true>, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = sms / 2;
      }
      w->max_clusters = n;
    }
  }
  w->stack = w->kind == KIND_F32 && !w->cta2 && w->BN <= 128 && tune_env("ELB_F32_STACK", 1) > 0;
  info.launches_per_call = (w->flat || w->small_ic) ? 1 : 3 * ((d.n + w->imgs_per_chunk - 1) / w->imgs_per_chunk);
  if (w->small_ic) {
    e = init_f32_small_ic(g.OCB);
    if (e != cudaSuccess) { err = std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e); return ELB_GENERAL_ERROR; }
  }
  return ELB_OK;
}

#define W_TRY(expr)                                                                   \
  do {                                                                                \
    cudaError_t e__ = (expr);                                                         \
    if (e__ != cudaSuccess) { err = std::string(#expr) + ": " + cudaGetErrorString(e__); return ELB_GENERAL_ERROR; } \
  } while (0)

int wino_prepare(WinoPlan &pl, const elb_conv_desc_t &d, elb_conv_info_t &info, const void *weights,
                 const void *bias, std::string &err) {
  WinoImpl *w = pl.impl;
  if (!w) { err = "plan not set up"; return ELB_GENERAL_ERROR; }
  const WinoGeom &g = w->g;
  std::vector<float> hw(info.size_weights), hb(w->OCP, 0.0f);
  W_TRY(cudaMemcpy(hw.data(), weights, info.size_weights * 4, cudaMemcpyDefault));
  if (d.with_bias) {
    if (!bias) { err = "bias is null but with_bias is set"; return ELB_GENERAL_ERROR; }
    W_TRY(cudaMemcpy(hb.data(), bias, static_cast<size_t>(w->OCP) * 4, cudaMemcpyDefault));
  }
  if (w->small_ic) {
    // [tap][channel 0..3][OCP]: the layout the direct kernel reads as broadcast float4s
    std::vector<float> ws(static_cast<size_t>(9) * 4 * w->OCP, 0.0f);
    for (int o = 0; o < d.oc; ++o)
      for (int i = 0; i < d.ic; ++i)
        for (int tap = 0; tap < 9; ++tap)
          ws[(static_cast<size_t>(tap) * 4 + i) * w->OCP + o] = hw[host::w_index(w->ICP / 16, 3, 3, o, i, tap / 3, tap % 3)];
    W_TRY(cudaMalloc(&w->d_w_small, ws.size() * 4));
    W_TRY(cudaMemcpy(w->d_w_small, ws.data(), ws.size() * 4, cudaMemcpyHostToDevice));
    W_TRY(cudaMalloc(&w->d_bias, static_cast<size_t>(w->OCP) * 4));
    W_TRY(cudaMemcpy(w->d_bias, hb.data(), static_cast<size_t>(w->OCP) * 4, cudaMemcpyHostToDevice));
    info.workspace_bytes += ws.size() * 4 + static_cast<size_t>(w->OCP) * 4;
    return ELB_OK;
  }
  std::vector<float> u;
  if (w->direct) {
    // U[oc][tap][ic]: K runs over (kh, kw) taps, then the input channels
    u.assign(static_cast<size_t>(w->OCP) * g.taps * w->ICP, 0.0f);
    for (int o = 0; o < d.oc; ++o)
      for (int tap = 0; tap < g.taps; ++tap)
        for (int i = 0; i < d.ic; ++i)
          u[(static_cast<size_t>(o) * g.taps + tap) * w->ICP + i] =
              hw[host::w_index(w->ICP / 16, d.kh, d.kw, o, i, tap / d.kw, tap % d.kw)];
  } else {
    u = transform_weights(hw.data(), d.oc, d.ic, w->OCP, w->ICP, g.A);
  }
  const int BN = w->BN, KS = g.k_stages, AA = g.A * g.A;
  const size_t KTOT = static_cast<size_t>(g.taps) * w->ICP;      // K extent of one position
  std::vector<uint8_t> img(w->b_bytes, 0);
  if (w->kind == KIND_F32) {
    // [a][nt][ks = channel block][plane][chunk j = 4 channels][BN rows][4 floats]
    float *dst = reinterpret_cast<float *>(img.data());
    for (int a = 0; a < AA; ++a)
      for (int nt = 0; nt < w->n_tiles; ++nt)
        for (int ks = 0; ks < KS; ++ks)
          for (int r = 0; r < BN; ++r) {
            const int o = nt * BN + r;
            if (o >= w->OCP) continue;
            const float *src = &u[(static_cast<size_t>(a) * w->OCP + o) * KTOT + static_cast<size_t>(ks) * 16];
            // pairs: a stage is stored as two half images of BN/2 rows, one per CTA
            const int BNH = w->cta2 ? BN / 2 : BN, hf = r / BNH, rr = r % BNH;
            float *stage = dst + ((static_cast<size_t>(a) * w->n_tiles + nt) * KS + ks) * (32 * BN) + static_cast<size_t>(hf) * 32 * BNH;
            for (int c = 0; c < 16; ++c) {
              const float hi = tf32_rna(src[c]);
              volatile float lo = src[c] - hi;
              const int j = c >> 2, e = c & 3;
              if (w->stack) {      // [chunk j][hi rows | lo rows][4 floats]
                stage[(static_cast<size_t>(j) * 2 * BN + rr) * 4 + e] = hi;
                stage[(static_cast<size_t>(j) * 2 * BN + BN + rr) * 4 + e] = lo;
              } else {             // [plane hi / lo][chunk j][rows][4 floats]
                stage[(static_cast<size_t>(j) * BNH + rr) * 4 + e] = hi;
                stage[(static_cast<size_t>(4 + j) * BNH + rr) * 4 + e] = lo;
              }
            }
          }
  } else {
    // per (a, oc): abs-max over ic, q = rne((U*127)/absmax), scale = (absmax/127)*tS,
    // shift = -(sum q * scale) * ceil(tz)      (src/elx_conv_wino_trans_weights.cpp:437-535)
    std::vector<float> scale(static_cast<size_t>(AA) * w->OCP, 0.0f), shift(scale.size(), 0.0f);
    for (int a = 0; a < AA; ++a)
      for (int o = 0; o < w->OCP; ++o) {
        const float *src = &u[(static_cast<size_t>(a) * w->OCP + o) * w->ICP];
        float m = 0.0f;
        for (int i = 0; i < w->ICP; ++i) m = std::fmax(m, std::fabs(src[i]));
        float sq = 0.0f;
        const int nt = o / BN, r = o % BN;
        for (int i = 0; i < w->ICP; ++i) {
          int8_t q = 0;
          if (m != 0.0f) {
            volatile float t = src[i] * 127.0f;
            volatile float v = t / m;
            q = static_cast<int8_t>(std::nearbyintf(v));
          }
          sq += static_cast<float>(q);
          const int cb = i >> 4, ks = cb >> 3, j = cb & 7;
          const int BNH = w->cta2 ? BN / 2 : BN, hf = r / BNH, rr = r % BNH;
          img[((static_cast<size_t>(a) * w->n_tiles + nt) * KS + ks) * (128 * BN) + static_cast<size_t>(hf) * 128 * BNH +
              (static_cast<size_t>(j) * BNH + rr) * 16 + (i & 15)] = static_cast<uint8_t>(q);
        }
        volatile float sw = m / 127.0f;
        volatile float sc = sw * d.tinput_scale;
        volatile float z1 = -sq * sc;
        volatile float zw = z1 * w->tz;
        scale[static_cast<size_t>(a) * w->OCP + o] = sc;
        shift[static_cast<size_t>(a) * w->OCP + o] = zw;
      }
    W_TRY(cudaMalloc(&w->d_scale, scale.size() * 4));
    W_TRY(cudaMalloc(&w->d_shift, shift.size() * 4));
    W_TRY(cudaMemcpy(w->d_scale, scale.data(), scale.size() * 4, cudaMemcpyHostToDevice));
    W_TRY(cudaMemcpy(w->d_shift, shift.data(), shift.size() * 4, cudaMemcpyHostToDevice));
  }
  W_TRY(cudaMalloc(&w->d_b, w->b_bytes));
  W_TRY(cudaMemcpy(w->d_b, img.data(), w->b_bytes, cudaMemcpyHostToDevice));
  W_TRY(cudaMalloc(&w->d_bias, static_cast<size_t>(w->OCP) * 4));
  W_TRY(cudaMemcpy(w->d_bias, hb.data(), static_cast<size_t>(w->OCP) * 4, cudaMemcpyHostToDevice));
  W_TRY(cudaMalloc(&w->d_a, w->a_bytes));
  W_TRY(cudaMemset(w->d_a, 0, w->a_bytes));          // K padding chunks stay zero for ever
  W_TRY(cudaMalloc(&w->d_m, w->m_bytes));
  info.workspace_bytes += w->a_bytes + w->b_bytes + w->m_bytes + static_cast<size_t>(w->OCP) * 4;
  return ELB_OK;
}

int wino_run(WinoPlan &pl, void *out, const void *in, void *acc_dump, int *status, int num_sms,
             int first, int count, cudaStream_t s, int &launches, std::string &err) {
  WinoImpl *w = pl.impl;
  launches = 0;
  if (!w) { err = "plan not set up"; return ELB_GENERAL_ERROR; }
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) {
    err = "input/output tensors must be 16-byte aligned";
    return ELB_GENERAL_ERROR;
  }
  if (first < 0 || count <= 0 || first + count > w->N) { err = "image range outside the batch"; return ELB_GENERAL_ERROR; }
  const bool stepped = pl.in_step > 1;
  if (stepped && !wino_input_step_supported(pl)) { err = "this kernel cannot read its input with a step"; return ELB_UNIMPLEMENTED; }
  if (w->small_ic) {
    const WinoGeom &g = w->g;
    SmallIcParams sp{};
    sp.planar = pl.in_planar ? 1 : 0;
    sp.trace = static_cast<long long *>(pl.trace);
    sp.in = static_cast<const float *>(in) +
            static_cast<size_t>(first) * (pl.in_planar ? static_cast<size_t>(w->ic_real) * g.IH * g.IW : w->in_img_bytes / 4);
    sp.out = static_cast<float *>(out) + static_cast<size_t>(first) * (w->out_img_bytes / 4);
    sp.w = static_cast<const float *>(w->d_w_small);
    sp.bias = static_cast<const float *>(w->d_bias);
    sp.N = count; sp.H = g.IH; sp.W = g.IW; sp.CB = g.CB; sp.OCB = g.OCB;
    sp.ic = w->ic_real;
    sp.with_bias = w->with_bias; sp.with_relu = w->with_relu; sp.with_sum = w->with_sum;
    const bool timed = pl.stage_ev[0] != nullptr;
    if (timed) { W_TRY(cudaEventRecord(pl.stage_ev[0], s)); W_TRY(cudaEventRecord(pl.stage_ev[1], s)); }
    if (f32_rgb_umma_supported(sp) && tune_env("ELB_RGB_UMMA", 1) != 0) W_TRY(launch_f32_rgb_umma(sp, num_sms, status, s));
    else W_TRY(launch_f32_small_ic(sp, s));
    if (timed) { W_TRY(cudaEventRecord(pl.stage_ev[2], s)); W_TRY(cudaEventRecord(pl.stage_ev[3], s)); }
    launches = 1;
    return ELB_OK;
  }
  if (w->flat) {
    // the whole convolution in the GEMM kernel: A straight from the user's tensor, fused epilogue
    const WinoGeom &g = w->g;
    const int HW = g.OH * g.OW, tiles_img = (HW + BM - 1) / BM;
    PFN_encodeTiled enc = get_encode_tiled();
    if (!enc) { err = "cuTensorMapEncodeTiled is not available from the driver"; return ELB_GENERAL_ERROR; }
    WinoGemmParams gp{};
    const float *src = static_cast<const float *>(in) + static_cast<size_t>(first) * (w->in_img_bytes / 4);
    cuuint64_t dims[3] = {16, static_cast<cuuint64_t>(HW), static_cast<cuuint64_t>(count) * g.CB};
    cuuint64_t strides[2] = {64, static_cast<cuuint64_t>(HW) * 64};
    cuuint32_t box[3] = {4, BM, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult cr = enc(&gp.tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(src), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) { err = "cuTensorMapEncodeTiled failed (" + std::to_string(static_cast<int>(cr)) + ")"; return ELB_GENERAL_ERROR; }
    gp.b_img = static_cast<const uint8_t *>(w->d_b);
    gp.status = status;
    gp.trace = static_cast<long long *>(pl.trace);
    gp.m_tiles = count * tiles_img;
    gp.m_pitch = gp.m_tiles;
    gp.n_tiles = w->n_tiles; gp.k_stages = g.k_stages; gp.BN = w->BN;
    gp.OCB = g.OCB; gp.Tpad = 0; gp.T = count * HW; gp.kind = KIND_F32;
    gp.positions = 1;
    gp.flat = 1; gp.HW = HW; gp.tiles_img = tiles_img; gp.CB = g.CB;
    gp.producers = tune_producers();
    gp.rotate_k = tune_rotate_k();
    gp.stack = w->stack ? 1 : 0;
    gp.a_tmem = tune_a_tmem(KIND_F32, gp.k_stages, static_cast<long long>(gp.m_tiles) * gp.n_tiles, num_sms,
                            w->stack ? 2 * w->BN : w->BN, true);
    gp.kmul = 1;
    gp.bias = static_cast<const float *>(w->d_bias);
    gp.out = static_cast<float *>(out) + static_cast<size_t>(first) * (w->out_img_bytes / 4);
    gp.with_bias = w->with_bias; gp.with_relu = w->with_relu; gp.with_sum = w->with_sum;
    gp.relu_lo = w->relu_lo; gp.relu_hi = w->relu_hi;
    const bool timed = pl.stage_ev[0] != nullptr;
    if (timed) { W_TRY(cudaEventRecord(pl.stage_ev[0], s)); W_TRY(cudaEventRecord(pl.stage_ev[1], s)); }
    const int total = gp.m_tiles * gp.n_tiles;
    gemm_launch(gp, total < num_sms ? total : num_sms, s);
    W_TRY(cudaGetLastError());
    if (timed) { W_TRY(cudaEventRecord(pl.stage_ev[2], s)); W_TRY(cudaEventRecord(pl.stage_ev[3], s)); }
    launches = 1;
    return ELB_OK;
  }
  for (int n0 = first; n0 < first + count; n0 += w->imgs_per_chunk) {
    WinoGeom g = w->g;
    const int imgs = std::min(w->imgs_per_chunk, first + count - n0);
    g.N = imgs;
    g.T = imgs * g.ht * g.wt;
    g.m_tiles = (g.T + BM - 1) / BM;
    g.Tpad = w->g.Tpad;                   // buffers keep the full-chunk pitch
    const int m_tiles_run = g.m_tiles;
    g.m_tiles = w->g.m_tiles;             // operand image pitch
    // 1. input transform (covers every row of the m-tiles that will be multiplied)
    WinoInParams ip{};
    ip.in = static_cast<const uint8_t *>(in) + static_cast<size_t>(n0) * (stepped ? static_cast<size_t>(g.CB) * pl.src_h * pl.src_w * 64 : w->in_img_bytes);
    ip.a_img = w->d_a;
    ip.g = g;
    ip.step = stepped ? pl.in_step : 1; ip.SH = stepped ? pl.src_h : g.IH; ip.SW = stepped ? pl.src_w : g.IW;
    ip.g.Tpad = m_tiles_run * BM;
    ip.mrepS = w->mrepS; ip.tz = w->tz;
    dim3 gi((m_tiles_run * BM + TRANS_TILES - 1) / TRANS_TILES, g.CB);
    const bool timed = pl.stage_ev[0] != nullptr && n0 == first;
    if (timed) W_TRY(cudaEventRecord(pl.stage_ev[0], s));
    if (w->direct) {
      f32_gather_kernel<<<dim3((m_tiles_run * BM + 31) / 32, g.k_stages), 128, 0, s>>>(ip);
    } else if (g.A == 4) {
      dim3 g4((m_tiles_run * BM + 31) / 32, g.CB);
      const bool fast = 1020.0f * std::fabs(w->mrepS) + std::fabs(w->tz) < 4194304.0f;
      if (w->kind != KIND_I8) wino4_input_kernel<false, true><<<g4, 128, 0, s>>>(ip);
      else if (fast) wino4_input_kernel<true, true><<<g4, 128, 0, s>>>(ip);
      else wino4_input_kernel<true, false><<<g4, 128, 0, s>>>(ip);
    } else if (w->kind == KIND_I8) {
      // largest |V| for u8 inputs: 255 * (largest absolute row sum of B^T = 5.28125)^2
      const bool fast = 255.0f * 27.8916f * std::fabs(w->mrepS) + std::fabs(w->tz) < 4194304.0f;
      if (fast) wino_input_u8_kernel<true><<<gi, TRANS_THREADS, 0, s>>>(ip);
      else wino_input_u8_kernel<false><<<gi, TRANS_THREADS, 0, s>>>(ip);
    }
    else wino_input_kernel<false><<<gi, TRANS_THREADS, 0, s>>>(ip);
    W_TRY(cudaGetLastError());
    if (timed) W_TRY(cudaEventRecord(pl.stage_ev[1], s));
    // 2. batched GEMM
    WinoGemmParams gp{};
    gp.a_img = static_cast<const uint8_t *>(w->d_a);
    gp.b_img = static_cast<const uint8_t *>(w->d_b);
    gp.m_out = static_cast<float *>(w->d_m);
    gp.scale = static_cast<const float *>(w->d_scale);
    gp.shift = static_cast<const float *>(w->d_shift);
    gp.acc_dump = (w->kind == KIND_I8 && acc_dump && n0 == 0 && imgs == w->N) ? static_cast<int32_t *>(acc_dump) : nullptr;
    gp.status = status;
    gp.trace = static_cast<long long *>(pl.trace);
    gp.m_tiles = m_tiles_run;            // tiles multiplied in this chunk
    gp.m_pitch = w->g.m_tiles;           // pitch of the operand image (full chunk)
    gp.n_tiles = w->n_tiles; gp.k_stages = g.k_stages; gp.BN = w->BN;
    gp.OCB = g.OCB; gp.Tpad = w->g.Tpad; gp.T = g.T; gp.kind = w->kind;
    gp.positions = g.A * g.A;
    gp.producers = tune_producers();
    gp.rotate_k = tune_rotate_k();
    gp.ablate = tune_env("ELB_ABL", 0);
    gp.stack = w->stack ? 1 : 0;
    gp.a_tmem = tune_a_tmem(w->kind, gp.k_stages, static_cast<long long>(gp.positions) * gp.m_tiles * gp.n_tiles, num_sms,
                            w->stack ? 2 * w->BN : w->BN, false);
    gp.kmul = tune_kmul(w->kind, gp.a_tmem, gp.k_stages, w->BN);
    if (w->cta2) {
      const int pairs = gp.positions * ((gp.m_tiles + 1) / 2) * gp.n_tiles;
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(2 * (pairs < w->max_clusters ? pairs : w->max_clusters));
      cfg.blockDim = dim3(GEMM_THREADS);
      cfg.dynamicSmemBytes = GEMM_SMEM_BYTES;
      cfg.stream = s;
      cudaLaunchAttribute at{};
      at.id = cudaLaunchAttributeClusterDimension;
      at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
      cfg.attrs = &at;
      cfg.numAttrs = 1;
      W_TRY(cudaLaunchKernelEx(&cfg, wino_gemm_kernel<true>, gp));
    } else {
      const int total = gp.positions * gp.m_tiles * gp.n_tiles;
      gemm_launch(gp, total < num_sms ? total : num_sms, s);
      W_TRY(cudaGetLastError());
    }
    if (timed) W_TRY(cudaEventRecord(pl.stage_ev[2], s));
    // 3. output transform
    WinoOutParams op{};
    op.m_in = static_cast<const float *>(w->d_m);
    op.bias = static_cast<const float *>(w->d_bias);
    op.out = static_cast<uint8_t *>(out) + static_cast<size_t>(n0) * w->out_img_bytes;
    op.g = g;
    op.g.Tpad = w->g.Tpad;
    op.out_type = w->out_type; op.with_bias = w->with_bias; op.with_relu = w->with_relu; op.with_sum = w->with_sum;
    op.orepS = w->orepS; op.oz = w->oz;
    op.relu_lo = w->relu_lo; op.relu_hi = w->relu_hi;
    dim3 go((g.T + TRANS_TILES - 1) / TRANS_TILES, g.OCB);
    if (w->direct) f32_epilogue_kernel<<<dim3((g.T + 31) / 32, g.OCB), 128, 0, s>>>(op);
    else if (g.A == 4) wino4_output_kernel<<<dim3((g.T + 31) / 32, g.OCB), 128, 0, s>>>(op);
    else wino_output_kernel<<<go, TRANS_THREADS, 0, s>>>(op);
    W_TRY(cudaGetLastError());
    if (timed) W_TRY(cudaEventRecord(pl.stage_ev[3], s));
    launches += 3;
  }
  return ELB_OK;
}

bool wino_input_step_supported(const WinoPlan &pl) {
  const WinoImpl *w = pl.impl;
  return w && w->kind == KIND_F32 && !w->small_ic && !w->flat && !w->direct && w->g.A == 6;
}

void wino_release(WinoPlan &pl) {
  WinoImpl *w = pl.impl;
  if (!w) return;
  for (void *p : {w->d_a, w->d_b, w->d_m, w->d_bias, w->d_scale, w->d_shift, w->d_w_small})
    if (p) cudaFree(p);
  delete w;
  pl.impl = nullptr;
}

// =================================================================================================
// Allocation-free FP32 Winograd entry point.
//
// Some hosts may not allocate device memory where they call a convolution: a serving process whose
// memory was carved up at start-up and handed to an arena it must not grow, a real-time loop that
// must not take the driver's allocation lock, a plug-in running inside another framework's memory
// budget.  For them elb_wino_f32_conv_noalloc() runs the same three kernels as the plan-based path
// (plus a device-side weight transform) with every transform-domain buffer -- packed weights,
// operand image of the transformed input, GEMM result, status word -- carved out of ONE file-scope
// device array of fixed size.  Every GPU that loads the library holds that array until the process
// exits.  The call uses no cudaMalloc / cudaFree and no allocating library routine; the caller
// passes device pointers for input, weights, bias and output.
//
// Rules that follow from sharing one static array:
//   * problems whose buffers exceed ELB_NOALLOC_SCRATCH_BYTES are rejected with ELB_UNIMPLEMENTED;
//   * the array keeps the previous call's contents; this path rewrites everything it reads (the
//     operand image has no K padding in fp32) and clears the status word at the start of each call;
//   * two calls that overlap on the GPU (different streams, or different host threads) race on the
//     array -- serialise them;
//   * the first call on each device resolves the array's device address and sets the GEMM kernel's
//     shared-memory attribute; make that first call before any stream capture begins.
// =================================================================================================
namespace {

constexpr size_t ELB_NOALLOC_SCRATCH_BYTES = size_t(64) << 20;     // 64 MiB per GPU
static __device__ __align__(256) unsigned char g_noalloc_scratch[ELB_NOALLOC_SCRATCH_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
unsigned char *g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};     // device address of the array, per device

__device__ __forceinline__ void g3_dev(float f0, float f1, float f2, float (&o)[6]) {
  const float z0 = 0.26890756302521f, z1 = -0.688403361344538f, z2 = 0.119514472455649f,
              z3 = 1.13777777777778f, z4 = 0.430252100840336f, z5 = 0.179271708683473f;
  const float t1 = __fmaf_rn(-z0, f2, __fmul_rn(z1, f0));      // same fusion structure as the host path
  const float t2 = __fmaf_rn(z0, f2, __fmul_rn(z2, f0));
  o[0] = __fmul_rn(z3, f0);
  o[1] = __fmaf_rn(-z4, f1, t1);
  o[2] = __fmaf_rn(z4, f1, t1);
  o[3] = __fmaf_rn(z5, f1, t2);
  o[4] = __fmaf_rn(-z5, f1, t2);
  o[5] = f2;
}

// One thread = one (oc, ic) pair: U = G g G^T, 3xTF32 split, written into the GEMM's B image
// [a][n tile][k stage = ic/16][plane][chunk = (ic%16)/4][BN rows][4 floats].
__global__ void wino_weights_f32_kernel(const float *__restrict__ w, float *__restrict__ b_img, int oc, int ic,
                                        int OCP, int ICP, int BN, int n_tiles, int stack) {
  // one thread per row of EVERY n tile (n_tiles * BN >= OCP): rows past the last output channel are
  // written as zeros, because the scratch behind them still holds an earlier call's bytes
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_tiles * BN * ICP) return;
  (void)OCP;
  const int o = idx / ICP, i = idx - o * ICP;
  float g[3][3];
#pragma unroll
  for (int kh = 0; kh < 3; ++kh)
#pragma unroll
    for (int kw = 0; kw < 3; ++kw) {
      float v = 0.0f;
      if (o < oc && i < ic)
        v = w[((((static_cast<size_t>(o >> 4) * (ICP >> 4) + (i >> 4)) * 3 + kh) * 3 + kw) * 16 + (i & 15)) * 16 + (o & 15)];
      g[kh][kw] = v;
    }
  float m[6][3];
#pragma unroll
  for (int kw = 0; kw < 3; ++kw) {
    float r[6];
    g3_dev(g[0][kw], g[1][kw], g[2][kw], r);
#pragma unroll
    for (int a = 0; a < 6; ++a) m[a][kw] = r[a];
  }
  const int nt = o / BN, row = o - nt * BN;
  const int ks = i >> 4, j = (i & 15) >> 2, e = i & 3;
  const int KS = ICP >> 4;
#pragma unroll
  for (int a = 0; a < 6; ++a) {
    float r[6];
    g3_dev(m[a][0], m[a][1], m[a][2], r);
#pragma unroll
    for (int b = 0; b < 6; ++b) {
      uint32_t hb;
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(r[b]));
      const float hi = __uint_as_float(hb);
      const float lo = __fsub_rn(r[b], hi);
      float *stage = b_img + ((static_cast<size_t>(a * 6 + b) * n_tiles + nt) * KS + ks) * (32 * BN);
      if (stack) {       // [chunk j][hi rows | lo rows][4 floats]
        stage[(static_cast<size_t>(j) * 2 * BN + row) * 4 + e] = hi;
        stage[(static_cast<size_t>(j) * 2 * BN + BN + row) * 4 + e] = lo;
      } else {           // [plane hi / lo][chunk j][rows][4 floats]
        stage[(static_cast<size_t>(j) * BN + row) * 4 + e] = hi;
        stage[(static_cast<size_t>(4 + j) * BN + row) * 4 + e] = lo;
      }
    }
  }
}

}  // namespace

void set_last_error(const char *msg);   // elb_api.cu: text returned by elb_last_error()

}  // namespace elb

// No counterpart in the reference (its allocators, src/common/el_allocator.hpp:40-136, always own
// their memory); see the block comment above for who needs this and the limits that come with it.
// All pointers are device pointers of the current device; weights are OIhw16i16o fp32 as the
// caller holds them (they are transformed on the device inside this call), bias may be NULL when
// desc->with_bias is 0.  Returns ELB_OK / ELB_UNIMPLEMENTED / ELB_GENERAL_ERROR; the text of a
// failure is returned by elb_last_error().
extern "C" ELB_API int elb_wino_f32_conv_noalloc(const elb_conv_desc_t *desc, void *output, const void *input,
                                                 const void *weights, const void *bias, void *cuda_stream) {
  using namespace elb;
  auto fail = [](int code, const std::string &msg) { set_last_error(msg.c_str()); return code; };
  if (!desc || !output || !input || !weights) return fail(ELB_GENERAL_ERROR, "null argument");
  const elb_conv_desc_t &d = *desc;
  const bool shape_ok = d.kh == 3 && d.kw == 3 && d.stride_h == 1 && d.stride_w == 1 && d.pad_t == 1 && d.pad_l == 1 &&
                        d.dilation_h == 1 && d.dilation_w == 1 && d.g == 1 && d.n > 0 && d.ic > 0 && d.oc > 0 &&
                        d.oh == d.ih && d.ow == d.iw && (d.tile_size == 6 || d.tile_size == 0);
  const bool type_ok = d.dt_input == ELB_F32 && d.dt_weights == ELB_F32 && d.dt_output == ELB_F32 && d.dt_bias == ELB_F32 &&
                       d.fmt_input == ELB_NCHW16C && d.fmt_output == ELB_NCHW16C && d.fmt_weights == ELB_OIHW16I16O;
  if (!shape_ok || !type_ok)
    return fail(ELB_UNIMPLEMENTED, "elb_wino_f32_conv_noalloc: needs fp32 nChw16c/OIhw16i16o, 3x3, stride 1, pad 1, F(4x4,3x3)");
  if (d.with_bias && !bias) return fail(ELB_GENERAL_ERROR, "bias is null but with_bias is set");
  if ((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(output) | reinterpret_cast<uintptr_t>(weights)) & 15)
    return fail(ELB_GENERAL_ERROR, "tensors must be 16-byte aligned");

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= NOALLOC_MAX_DEVICES) return fail(ELB_GENERAL_ERROR, "no usable CUDA device");
  if (!g_noalloc_ptr[dev]) {
    // first call on this device: the array's NAME is a host-side handle, the kernels need its
    // device address
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return fail(ELB_GENERAL_ERROR, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    e = gemm_set_attributes();
    if (e != cudaSuccess) return fail(ELB_GENERAL_ERROR, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    g_noalloc_ptr[dev] = static_cast<unsigned char *>(p);
  }
  int num_sms = 0;
  if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
    return fail(ELB_GENERAL_ERROR, "cannot query the SM count");

  // geometry (one chunk: the whole batch must fit)
  const int ICP = host::alignup(d.ic, V), OCP = host::alignup(d.oc, V);
  WinoGeom g{};
  g.N = d.n; g.CB = ICP / V; g.OCB = OCP / V;
  g.IH = d.ih; g.IW = d.iw; g.OH = d.oh; g.OW = d.ow;
  g.A = 6;
  g.ht = (d.oh + 3) / 4; g.wt = (d.ow + 3) / 4;
  g.pad_t = 1; g.pad_l = 1;
  g.k_stages = g.CB;
  const long long T = static_cast<long long>(d.n) * g.ht * g.wt;
  if (T > (1ll << 24)) return fail(ELB_UNIMPLEMENTED, "elb_wino_f32_conv_noalloc: problem exceeds the static scratch array");
  g.T = static_cast<int>(T);
  g.m_tiles = (g.T + BM - 1) / BM;
  g.Tpad = g.m_tiles * BM;
  const int n_tiles = (OCP + MAX_BN - 1) / MAX_BN;
  const int BN = host::alignup((OCP + n_tiles - 1) / n_tiles, 16);
  const size_t b_bytes = static_cast<size_t>(36) * n_tiles * g.k_stages * 128 * BN;
  const size_t a_bytes = static_cast<size_t>(36) * g.m_tiles * g.k_stages * A_RAW_BYTES;
  const size_t m_bytes = static_cast<size_t>(36) * g.OCB * g.Tpad * 16 * 4;
  const size_t need = 256 + b_bytes + a_bytes + m_bytes;
  if (need > ELB_NOALLOC_SCRATCH_BYTES) {
    char buf[200];
    snprintf(buf, sizeof(buf), "elb_wino_f32_conv_noalloc: needs %zu bytes of scratch, the static array holds %zu",
             need, ELB_NOALLOC_SCRATCH_BYTES);
    return fail(ELB_UNIMPLEMENTED, buf);
  }
  unsigned char *base = g_noalloc_ptr[dev];
  int *status = reinterpret_cast<int *>(base);
  float *b_img = reinterpret_cast<float *>(base + 256);
  unsigned char *a_img = base + 256 + b_bytes;
  float *m_buf = reinterpret_cast<float *>(base + 256 + b_bytes + a_bytes);
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);

  // the status word must start at zero; everything else the kernels read is rewritten below
  if (cudaMemsetAsync(status, 0, 256, s) != cudaSuccess) return fail(ELB_GENERAL_ERROR, "cudaMemsetAsync failed");
  const int stack = BN <= 128 ? 1 : 0;
  wino_weights_f32_kernel<<<(n_tiles * BN * ICP + 255) / 256, 256, 0, s>>>(static_cast<const float *>(weights), b_img, d.oc,
                                                                         d.ic, OCP, ICP, BN, n_tiles, stack);
  WinoInParams ip{};
  ip.in = input; ip.a_img = a_img; ip.g = g;
  ip.step = 1; ip.SH = g.IH; ip.SW = g.IW;
  wino_input_kernel<false><<<dim3((g.Tpad + TRANS_TILES - 1) / TRANS_TILES, g.CB), TRANS_THREADS, 0, s>>>(ip);
  WinoGemmParams gp{};
  gp.a_img = a_img; gp.b_img = reinterpret_cast<const uint8_t *>(b_img); gp.m_out = m_buf;
  gp.status = status;
  gp.m_tiles = g.m_tiles; gp.m_pitch = g.m_tiles; gp.n_tiles = n_tiles; gp.k_stages = g.k_stages; gp.BN = BN;
  gp.OCB = g.OCB; gp.Tpad = g.Tpad; gp.T = g.T; gp.kind = KIND_F32;
  gp.positions = 36;
  gp.producers = GEMM_PRODUCERS_DEFAULT;
  const int total = 36 * gp.m_tiles * gp.n_tiles;
  gp.stack = stack;
  gp.a_tmem = 1;
  gp.kmul = tune_kmul(KIND_F32, gp.a_tmem, gp.k_stages, BN);
  gemm_launch(gp, total < num_sms ? total : num_sms, s);
  WinoOutParams op{};
  op.m_in = m_buf; op.bias = static_cast<const float *>(bias); op.out = output; op.g = g;
  op.out_type = OUT_F32; op.with_bias = d.with_bias; op.with_relu = d.with_relu; op.with_sum = d.with_ip_sum;
  op.orepS = 1.0f; op.oz = 0.0f;
  wino_output_kernel<<<dim3((g.T + TRANS_TILES - 1) / TRANS_TILES, g.OCB), TRANS_THREADS, 0, s>>>(op);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(ELB_GENERAL_ERROR, std::string("kernel launch failed: ") + cudaGetErrorString(e));
  return ELB_OK;
}

// Status word of the allocation-free path on the current device: 0 = every bounded wait of the last
// elb_wino_f32_conv_noalloc call completed, otherwise the code of the wait that gave up (the output
// of that call is then invalid); -1 = the entry point has not run on this device yet or the read
// failed.  Call it after synchronising the stream the convolution was enqueued on.  It copies four
// bytes from the static array to the host and allocates nothing.
extern "C" ELB_API int elb_wino_f32_noalloc_status(void) {
  using namespace elb;
  int dev = 0, st = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= NOALLOC_MAX_DEVICES || !g_noalloc_ptr[dev]) return -1;
  if (cudaMemcpy(&st, g_noalloc_ptr[dev], sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return st;
}
