// FP32 3x3 stride-1 pad-1 convolution for layers with at most FOUR input channels (the first layer
// of an image network: VGG-16 conv1_1 has 3), on CUDA cores.
//
// The reference runs such a layer through the same Winograd F(4x4,3x3) pipeline as any other when
// CONV_WINOGRAD is asked for (src/elx_conv_wino.cpp; the blocked input is zero-padded to 16
// channels, src/eld_conv.cpp:99-101), and its CONV_AUTO picks the direct algorithm for ic < 16
// (src/eld_conv.cpp:148-159).  Here the Winograd request is served by this direct kernel: with 3 of
// 16 channels real, the transform-domain tensors would be 13/16 zeros and the batched GEMM one
// 16-channel stage deep, i.e. all the traffic of Winograd (36/16 of the output size, written and read
// again) for none of its savings.  Measured on B200, VGG-16 conv1_1 at 32 images: 0.59 ms through the
// Winograd kernels, the figure of this kernel is in the profile notes.  The result differs from the
// reference's Winograd output by fp32 rounding only (both are within 1e-6 of the exact convolution).
//
// One thread computes 4 consecutive output pixels of a row for every output channel, eight channels
// at a time: its 3 x 6 input window (float4 = the four real channels of a pixel) stays in registers,
// the weights [tap][channel][OC] and the bias sit in shared memory and are read as broadcast float4s
// (16 FMAs per load).
#include <cuda_runtime.h>

#include "wino.cuh"

namespace elb {

namespace {

constexpr int SI_THREADS = 128;

// Two fp32 fused multiply-adds in one instruction (each lane rounds exactly as fma.rn.f32 does): in
// its scalar form the kernel was bound by instruction issue, 70 % of its instructions being FMAs.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// One 256-bit store: a whole 32-byte sector from one lane (two 128-bit stores of the same sector are two
// partial writes for the L2 to merge).  The address must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void *ptr, const float (&v)[8]) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "f"(v[0]), "f"(v[1]), "f"(v[2]),
               "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}

// Output channels are processed eight at a time: 32 accumulators + the 18 float4 of the window + the
// weights loaded ahead keep the thread near 140 registers, i.e. three resident blocks per SM.  (With
// sixteen channels at a time the kernel ran two blocks per SM and its issue slots were 30 % busy,
// most stalls waiting on the per-block bias loads from global memory; the bias now sits in shared
// memory behind the weights.)  Measured on B200, VGG-16 conv1_1 at 32 images: 0.192 ms with four
// blocks of 125 registers, a run-time channel test and two 128-bit stores per pixel; 0.183 ms with
// the channel count compiled in and three blocks; 0.157 ms with the 256-bit store on top.
//
// IC = 3 compiles the kernel for three input channels (an RGB image, the case that matters): the 27
// (tap, channel) steps then form one straight-line block whose weight loads the compiler can issue
// ahead of the arithmetic; IC = 0 tests the channel count at run time.
//
// PLANAR reads the caller's nchw tensor (how the reference's own first-layer runs pass an image,
// --input-format=nchw): three planes of floats instead of 16-channel blocks of which three channels
// are real, i.e. less than a fifth of the input bytes over PCIe and from HBM, and loads that
// neighbouring lanes share lines of (a lane's strip is 16 contiguous bytes of each plane row).
__device__ __forceinline__ void set_channel(float4 &v, int ch, float x) {
  if (ch == 0) v.x = x; else if (ch == 1) v.y = x; else if (ch == 2) v.z = x; else v.w = x;
}

template <int IC, bool PLANAR>
__global__ void __launch_bounds__(SI_THREADS, 3) f32_small_ic_kernel(const SmallIcParams p) {
  extern __shared__ float4 s_w4[];                 // [9 taps][4 channels][OCP] floats, then [OCP] bias
  float *s_w = reinterpret_cast<float *>(s_w4);
  const int OCP = p.OCB * 16;
  float *s_b = s_w + 9 * 4 * OCP;
  for (int i = threadIdx.x; i < 9 * 4 * OCP / 4; i += SI_THREADS) s_w4[i] = reinterpret_cast<const float4 *>(p.w)[i];
  for (int i = threadIdx.x; i < OCP; i += SI_THREADS) s_b[i] = p.with_bias ? p.bias[i] : 0.0f;
  __syncthreads();
  const int w4 = (p.W + 3) >> 2;                   // groups of 4 pixels per row
  const long long idx = static_cast<long long>(blockIdx.x) * SI_THREADS + threadIdx.x;
  if (idx >= static_cast<long long>(p.N) * p.H * w4) return;
  const int g = static_cast<int>(idx % w4);
  const int oh = static_cast<int>((idx / w4) % p.H);
  const int n = static_cast<int>(idx / (static_cast<long long>(w4) * p.H));
  const int ow0 = g * 4;

  // the four real channels of the 3 x 6 input pixels around the strip (zero outside the image)
  float4 win[3][6];
  if (PLANAR) {
    const float *in_n = p.in + static_cast<size_t>(n) * p.ic * p.H * p.W;
    const bool vec = (p.W & 3) == 0;               // rows start on 16-byte boundaries: one float4 for the strip itself
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int ih = oh - 1 + r;
      const bool row_ok = ih >= 0 && ih < p.H;
#pragma unroll
      for (int c = 0; c < 6; ++c) win[r][c] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        if ((IC != 0 ? ch < IC : ch < p.ic) && row_ok) {
          const float *row = in_n + (static_cast<size_t>(ch) * p.H + ih) * p.W;
          if (vec) {
            const float4 m = __ldg(reinterpret_cast<const float4 *>(row + ow0));
            set_channel(win[r][1], ch, m.x); set_channel(win[r][2], ch, m.y);
            set_channel(win[r][3], ch, m.z); set_channel(win[r][4], ch, m.w);
          } else {
#pragma unroll
            for (int c = 1; c < 5; ++c)
              if (ow0 + c - 1 < p.W) set_channel(win[r][c], ch, __ldg(row + ow0 + c - 1));
          }
          if (ow0 > 0) set_channel(win[r][0], ch, __ldg(row + ow0 - 1));
          if (ow0 + 4 < p.W) set_channel(win[r][5], ch, __ldg(row + ow0 + 4));
        }
      }
    }
  } else {
    const float *in_n = p.in + static_cast<size_t>(n) * p.CB * p.H * p.W * 16;    // channel block 0 holds every real channel
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int ih = oh - 1 + r;
#pragma unroll
      for (int c = 0; c < 6; ++c) {
        const int iw = ow0 - 1 + c;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ih >= 0 && ih < p.H && iw >= 0 && iw < p.W)
          v = __ldg(reinterpret_cast<const float4 *>(in_n + (static_cast<size_t>(ih) * p.W + iw) * 16));
        win[r][c] = v;
      }
    }
  }

  const int groups = OCP >> 3;                     // groups of eight output channels
#pragma unroll 1
  for (int og = 0; og < groups; ++og) {
    unsigned long long acc[4][4];                  // [pixel][pair of output channels]
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const unsigned long long b = pack2(s_b[og * 8 + 2 * i], s_b[og * 8 + 2 * i + 1]);
#pragma unroll
      for (int px = 0; px < 4; ++px) acc[px][i] = b;
    }
#pragma unroll
    for (int kh = 0; kh < 3; ++kh)
#pragma unroll
      for (int kw = 0; kw < 3; ++kw)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (IC != 0 ? c < IC : c < p.ic) {       // uniform: the same for every thread
            const float4 *wr = reinterpret_cast<const float4 *>(s_w + ((kh * 3 + kw) * 4 + c) * OCP + og * 8);
            const float4 w0 = wr[0], w1 = wr[1];
            const unsigned long long wv[4] = {pack2(w0.x, w0.y), pack2(w0.z, w0.w), pack2(w1.x, w1.y), pack2(w1.z, w1.w)};
#pragma unroll
            for (int px = 0; px < 4; ++px) {
              const float4 xv = win[kh][px + kw];
              const float x = c == 0 ? xv.x : c == 1 ? xv.y : c == 2 ? xv.z : xv.w;
              const unsigned long long xx = pack2(x, x);
#pragma unroll
              for (int i = 0; i < 4; ++i) acc[px][i] = fma2(xx, wv[i], acc[px][i]);
            }
          }
        }
    // bias is in; + stored output (in-place sum), ReLU, store: 32 bytes of each of the four pixels
    const int ocb = og >> 1, half = og & 1;
#pragma unroll
    for (int px = 0; px < 4; ++px) {
      const int ow = ow0 + px;
      if (ow < p.W) {
        float4 *dst = reinterpret_cast<float4 *>(p.out + (((static_cast<size_t>(n) * p.OCB + ocb) * p.H + oh) * p.W + ow) * 16) + half * 2;
        if (!p.with_sum) {                         // the eight channels are one 32-byte sector: one store
          float v[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) unpack2(acc[px][i], v[2 * i], v[2 * i + 1]);
          if (p.with_relu) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = fmaxf(v[i], 0.0f);
          }
          st_global_v8(dst, v);
          continue;
        }
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          float4 v;
          unpack2(acc[px][2 * q], v.x, v.y);
          unpack2(acc[px][2 * q + 1], v.z, v.w);
          if (p.with_sum) {
            const float4 pv = dst[q];
            v.x = __fadd_rn(v.x, pv.x); v.y = __fadd_rn(v.y, pv.y); v.z = __fadd_rn(v.z, pv.z); v.w = __fadd_rn(v.w, pv.w);
          }
          if (p.with_relu) {                       // the Winograd output transform's ReLU: a plain max with 0
            v.x = fmaxf(v.x, 0.0f); v.y = fmaxf(v.y, 0.0f); v.z = fmaxf(v.z, 0.0f); v.w = fmaxf(v.w, 0.0f);
          }
          dst[q] = v;
        }
      }
    }
  }
}

}  // namespace

size_t f32_small_ic_smem_bytes(int OCB) { return (static_cast<size_t>(9) * 4 + 1) * OCB * 16 * 4; }

cudaError_t init_f32_small_ic(int OCB) {
  const int bytes = static_cast<int>(f32_small_ic_smem_bytes(OCB));
  cudaError_t e = cudaFuncSetAttribute(f32_small_ic_kernel<0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(f32_small_ic_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(f32_small_ic_kernel<0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(f32_small_ic_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  return e;
}

cudaError_t launch_f32_small_ic(const SmallIcParams &p, cudaStream_t s) {
  const long long threads = static_cast<long long>(p.N) * p.H * ((p.W + 3) / 4);
  const unsigned blocks = static_cast<unsigned>((threads + SI_THREADS - 1) / SI_THREADS);
  const size_t smem = f32_small_ic_smem_bytes(p.OCB);
  if (p.planar) {
    if (p.ic == 3) f32_small_ic_kernel<3, true><<<blocks, SI_THREADS, smem, s>>>(p);
    else f32_small_ic_kernel<0, true><<<blocks, SI_THREADS, smem, s>>>(p);
  } else {
    if (p.ic == 3) f32_small_ic_kernel<3, false><<<blocks, SI_THREADS, smem, s>>>(p);
    else f32_small_ic_kernel<0, false><<<blocks, SI_THREADS, smem, s>>>(p);
  }
  return cudaGetLastError();
}

}  // namespace elb
