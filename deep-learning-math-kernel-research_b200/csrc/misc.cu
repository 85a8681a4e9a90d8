// Layout converters nchw <-> nChw16c on the device (reference: reorder<T, nChw16c, nchw> and
// reorder<T, nchw, nChw16c>, src/elx_reorder.cpp:11-66).  Bandwidth-bound permutes staged through
// shared memory so that both the plain-side reads (contiguous along w) and the blocked-side
// writes (16 channels contiguous) are coalesced.  Channel padding lanes are written as zero.
#include <algorithm>
#include "../../include/euler_b200.h"
#include "elb_common.cuh"

namespace elb {
namespace {

// One CTA handles one (n, channel block) and a strip of TILE pixels.
template <typename T, bool TO_BLOCKED>
__global__ void __launch_bounds__(256) reorder_kernel(T *__restrict__ dst, const T *__restrict__ src, int c, int hw) {
  constexpr int TILE = 128;
  __shared__ T tile[16][TILE + 1];
  const int cb = blockIdx.y, n = blockIdx.z;
  const int p0 = blockIdx.x * TILE;
  const int C2 = (c + 15) / 16;
  if (TO_BLOCKED) {
    for (int i = threadIdx.x; i < 16 * TILE; i += blockDim.x) {
      const int ch = i / TILE, px = i % TILE;
      const int cc = cb * 16 + ch;
      T v = T(0);
      if (cc < c && p0 + px < hw) v = src[((size_t)n * c + cc) * hw + p0 + px];
      tile[ch][px] = v;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * TILE; i += blockDim.x) {
      const int px = i / 16, ch = i % 16;
      if (p0 + px < hw) dst[(((size_t)n * C2 + cb) * hw + p0 + px) * 16 + ch] = tile[ch][px];
    }
  } else {
    for (int i = threadIdx.x; i < 16 * TILE; i += blockDim.x) {
      const int px = i / 16, ch = i % 16;
      if (p0 + px < hw) tile[ch][px] = src[(((size_t)n * C2 + cb) * hw + p0 + px) * 16 + ch];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * TILE; i += blockDim.x) {
      const int ch = i / TILE, px = i % TILE;
      const int cc = cb * 16 + ch;
      if (cc < c && p0 + px < hw) dst[((size_t)n * c + cc) * hw + p0 + px] = tile[ch][px];
    }
  }
}

// u8 nchw -> nChw16c when a plane is a whole number of 4-pixel groups: one thread = 4 pixels of one
// channel block.  It reads one 32-bit word per real channel (a warp: 128 contiguous bytes of a plane)
// and writes the four pixels' 16-byte blocks, padding lanes zero.  (The byte-wise kernel above moves
// one byte per access: measured 43 us for 32 RGB images of 224x224 against a few us of traffic.)
__global__ void __launch_bounds__(256) reorder_u8_planes_kernel(uint4 *__restrict__ dst, const uint8_t *__restrict__ src,
                                                                int c, int hw4, long long total) {
  griddep_launch_dependents();      // an INT8 kernel behind this one may set itself up (see launch_overlapped)
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int C2 = (c + 15) / 16;
  const int q = static_cast<int>(idx % hw4);
  const int cb = static_cast<int>((idx / hw4) % C2);
  const long long n = idx / (static_cast<long long>(hw4) * C2);
  uint32_t pl[16];
#pragma unroll
  for (int ch = 0; ch < 16; ++ch) {
    const int cc = cb * 16 + ch;
    pl[ch] = cc < c ? __ldg(reinterpret_cast<const uint32_t *>(src) + (n * c + cc) * hw4 + q) : 0u;
  }
  uint4 *o = dst + ((n * C2 + cb) * hw4 + q) * 4;
#pragma unroll
  for (int px = 0; px < 4; ++px) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // byte px of the four planes 4j .. 4j+3, in channel order
      const uint32_t lo = __byte_perm(pl[4 * j], pl[4 * j + 1], 0x0040 + px * 0x0011);
      const uint32_t hi = __byte_perm(pl[4 * j + 2], pl[4 * j + 3], 0x0040 + px * 0x0011);
      w[j] = __byte_perm(lo, hi, 0x5410);
    }
    o[px] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

template <bool TO_BLOCKED>
cudaError_t launch(void *dst, const void *src, int n, int c, int h, int w, int eb, cudaStream_t s) {
  const int hw = h * w;
  if (TO_BLOCKED && eb == 1 && hw % 4 == 0 && ((reinterpret_cast<uintptr_t>(src) & 3) == 0) &&
      ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
    const long long total = static_cast<long long>(n) * ((c + 15) / 16) * (hw / 4);
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    reorder_u8_planes_kernel<<<blocks, 256, 0, s>>>((uint4 *)dst, (const uint8_t *)src, c, hw / 4, total);
    return cudaGetLastError();
  }
  dim3 grid((hw + 127) / 128, (c + 15) / 16, n);
  if (eb == 1)
    reorder_kernel<uint8_t, TO_BLOCKED><<<grid, 256, 0, s>>>((uint8_t *)dst, (const uint8_t *)src, c, hw);
  else
    reorder_kernel<float, TO_BLOCKED><<<grid, 256, 0, s>>>((float *)dst, (const float *)src, c, hw);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// General converter between any two of the reference's formats of one tensor family
// (reference: every reorder<T, dst, src> of src/elx_reorder.cpp:11-207).  A tensor is addressed by
// the logical coordinate (g, a, b, h, w) -- a = n or o, b = c or i -- and a format is a list of
// physical axes, each one a whole logical dimension, its quotient by 16 or its remainder by 16.
// One thread writes one destination element (coalesced writes); lanes of a blocked destination
// past the logical extent are written as zero, lanes of a blocked source past it are not read.
struct Layout {
  int naxes;
  int dim[7];      // logical dimension of the axis: 0 g, 1 a, 2 b, 3 h, 4 w
  int kind[7];     // 0 whole, 1 quotient by 16, 2 remainder by 16
  int extent[7];
  long long stride[7];
};

template <typename T>
__global__ void __launch_bounds__(256) reorder_generic_kernel(T *__restrict__ dst, const T *__restrict__ src,
                                                              Layout ld, Layout ls, int da, int db,
                                                              long long total) {
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    int co[5] = {0, 0, 0, 0, 0};
    long long r = idx;
#pragma unroll
    for (int k = 6; k >= 0; --k) {
      if (k >= ld.naxes) continue;
      const int e = ld.extent[k];
      const int v = (int)(r % e);
      r /= e;
      co[ld.dim[k]] += ld.kind[k] == 1 ? v * 16 : v;
    }
    T v = T(0);
    if (co[1] < da && co[2] < db) {
      long long off = 0;
#pragma unroll
      for (int k = 0; k < 7; ++k) {
        if (k >= ls.naxes) continue;
        const int c = co[ls.dim[k]];
        off += (long long)(ls.kind[k] == 0 ? c : ls.kind[k] == 1 ? c / 16 : c % 16) * ls.stride[k];
      }
      v = src[off];
    }
    dst[idx] = v;
  }
}

// Batched 2-D transpose [rows][cols] -> [cols][rows] through a padded 32x32 shared-memory tile:
// nchw <-> nhwc is this with (rows, cols) = (c, h*w) or (h*w, c) per image.
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(T *__restrict__ dst, const T *__restrict__ src, int rows, int cols) {
  __shared__ T tile[32][33];
  const size_t base = (size_t)blockIdx.z * rows * cols;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
  for (int j = ty; j < 32; j += 8)
    if (r0 + j < rows && c0 + tx < cols) tile[j][tx] = src[base + (size_t)(r0 + j) * cols + c0 + tx];
  __syncthreads();
  for (int j = ty; j < 32; j += 8)
    if (c0 + j < cols && r0 + tx < rows) dst[base + (size_t)(c0 + j) * rows + r0 + tx] = tile[tx][j];
}

// Keep every step_h-th row and step_w-th column of an nChw16c tensor (the spatial subsample between
// two layers of a stack).  One thread moves the 16 channels of one pixel as 16-byte pieces.
template <int PIECES>
__global__ void __launch_bounds__(256) subsample_kernel(int4 *__restrict__ dst, const int4 *__restrict__ src, int planes,
                                                        int h, int w, int oh, int ow, int sh, int sw) {
  griddep_launch_dependents();      // an INT8 kernel behind this one may set itself up (see launch_overlapped)
  const long long total = (long long)planes * oh * ow * PIECES;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int piece = (int)(idx % PIECES);
    long long r = idx / PIECES;
    const int x = (int)(r % ow);
    r /= ow;
    const int y = (int)(r % oh);
    const long long pl = r / oh;
    dst[idx] = __ldg(&src[((pl * h + (long long)y * sh) * w + (long long)x * sw) * PIECES + piece]);
  }
}

// Format code (the reference's enum, include/euler.hpp:75-89) -> physical axes for (g, a, b, h, w).
bool make_layout(int fmt, int g, int a, int b, int h, int w, Layout &L) {
  const int A2 = (a + 15) / 16, B2 = (b + 15) / 16;
  int n = 0;
  auto ax = [&](int dim, int kind, int extent) { L.dim[n] = dim; L.kind[n] = kind; L.extent[n] = extent; ++n; };
  switch (fmt) {
    case ELB_NCHW: case ELB_OIHW: case ELB_GOIHW:
      ax(0, 0, g); ax(1, 0, a); ax(2, 0, b); ax(3, 0, h); ax(4, 0, w); break;
    case ELB_NHWC:
      ax(0, 0, g); ax(1, 0, a); ax(3, 0, h); ax(4, 0, w); ax(2, 0, b); break;
    case ELB_HWIO: case ELB_GHWIO:
      ax(0, 0, g); ax(3, 0, h); ax(4, 0, w); ax(2, 0, b); ax(1, 0, a); break;
    case ELB_NCHW16C:
      ax(0, 0, g); ax(1, 0, a); ax(2, 1, B2); ax(3, 0, h); ax(4, 0, w); ax(2, 2, 16); break;
    case ELB_OIHW16I16O: case ELB_GOIHW16I16O:
      ax(0, 0, g); ax(1, 1, A2); ax(2, 1, B2); ax(3, 0, h); ax(4, 0, w); ax(2, 2, 16); ax(1, 2, 16); break;
    default: return false;
  }
  L.naxes = n;
  long long st = 1;
  for (int k = n - 1; k >= 0; --k) { L.stride[k] = st; st *= L.extent[k]; }
  for (int k = n; k < 7; ++k) { L.dim[k] = 0; L.kind[k] = 0; L.extent[k] = 1; L.stride[k] = 0; }
  return true;
}

int family_of(int fmt) {
  switch (fmt) {
    case ELB_NCHW: case ELB_NHWC: case ELB_NCHW16C: return 1;
    case ELB_OIHW: case ELB_HWIO: case ELB_OIHW16I16O: return 2;
    case ELB_GOIHW: case ELB_GHWIO: case ELB_GOIHW16I16O: return 3;
    default: return 0;
  }
}

}  // namespace

cudaError_t launch_reorder(void *dst, int dst_fmt, const void *src, int src_fmt, int g, int a, int b, int h,
                           int w, int eb, cudaStream_t s, bool &supported) {
  supported = false;
  const int fam = family_of(dst_fmt);
  if (fam == 0 || fam != family_of(src_fmt) || dst_fmt == src_fmt) return cudaSuccess;
  if (fam != 3) g = 1;
  if (g < 1 || a < 1 || b < 1 || h < 1 || w < 1 || (eb != 1 && eb != 4)) return cudaSuccess;
  supported = true;
  // fast paths for activations
  if (dst_fmt == ELB_NCHW16C && src_fmt == ELB_NCHW) return launch<true>(dst, src, a, b, h, w, eb, s);
  if (dst_fmt == ELB_NCHW && src_fmt == ELB_NCHW16C) return launch<false>(dst, src, a, b, h, w, eb, s);
  if ((dst_fmt == ELB_NCHW && src_fmt == ELB_NHWC) || (dst_fmt == ELB_NHWC && src_fmt == ELB_NCHW)) {
    const int rows = src_fmt == ELB_NCHW ? b : h * w, cols = src_fmt == ELB_NCHW ? h * w : b;
    if (a <= 65535 && (rows + 31) / 32 <= 65535) {
      dim3 grid((cols + 31) / 32, (rows + 31) / 32, a);
      if (eb == 1) transpose_kernel<uint8_t><<<grid, 256, 0, s>>>((uint8_t *)dst, (const uint8_t *)src, rows, cols);
      else transpose_kernel<float><<<grid, 256, 0, s>>>((float *)dst, (const float *)src, rows, cols);
      return cudaGetLastError();
    }
  }
  Layout ld, ls;
  make_layout(dst_fmt, g, a, b, h, w, ld);
  make_layout(src_fmt, g, a, b, h, w, ls);
  long long total = 1;
  for (int k = 0; k < ld.naxes; ++k) total *= ld.extent[k];
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148 * 32);
  if (eb == 1)
    reorder_generic_kernel<uint8_t><<<blocks, 256, 0, s>>>((uint8_t *)dst, (const uint8_t *)src, ld, ls, a, b, total);
  else
    reorder_generic_kernel<float><<<blocks, 256, 0, s>>>((float *)dst, (const float *)src, ld, ls, a, b, total);
  return cudaGetLastError();
}

cudaError_t launch_subsample_blocked(void *dst, const void *src, int n, int c, int h, int w, int sh, int sw, int eb,
                                     cudaStream_t s) {
  const int planes = n * ((c + 15) / 16);
  const int oh = (h + sh - 1) / sh, ow = (w + sw - 1) / sw;
  const long long total = (long long)planes * oh * ow * (eb == 4 ? 4 : 1);
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148 * 32);
  if (eb == 4)
    subsample_kernel<4><<<blocks, 256, 0, s>>>((int4 *)dst, (const int4 *)src, planes, h, w, oh, ow, sh, sw);
  else
    subsample_kernel<1><<<blocks, 256, 0, s>>>((int4 *)dst, (const int4 *)src, planes, h, w, oh, ow, sh, sw);
  return cudaGetLastError();
}

cudaError_t launch_reorder_to_blocked(void *dst, const void *src, int n, int c, int h, int w, int eb, cudaStream_t s) {
  return launch<true>(dst, src, n, c, h, w, eb, s);
}
cudaError_t launch_reorder_from_blocked(void *dst, const void *src, int n, int c, int h, int w, int eb, cudaStream_t s) {
  return launch<false>(dst, src, n, c, h, w, eb, s);
}

}  // namespace elb
