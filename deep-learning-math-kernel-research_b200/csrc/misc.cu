// Layout converters nchw <-> nChw16c on the device (reference: reorder<T, nChw16c, nchw> and
// reorder<T, nchw, nChw16c>, src/elx_reorder.cpp:11-66).  Bandwidth-bound permutes staged through
// shared memory so that both the plain-side reads (contiguous along w) and the blocked-side
// writes (16 channels contiguous) are coalesced.  Channel padding lanes are written as zero.
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

template <bool TO_BLOCKED>
cudaError_t launch(void *dst, const void *src, int n, int c, int h, int w, int eb, cudaStream_t s) {
  const int hw = h * w;
  dim3 grid((hw + 127) / 128, (c + 15) / 16, n);
  if (eb == 1)
    reorder_kernel<uint8_t, TO_BLOCKED><<<grid, 256, 0, s>>>((uint8_t *)dst, (const uint8_t *)src, c, hw);
  else
    reorder_kernel<float, TO_BLOCKED><<<grid, 256, 0, s>>>((float *)dst, (const float *)src, c, hw);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_reorder_to_blocked(void *dst, const void *src, int n, int c, int h, int w, int eb, cudaStream_t s) {
  return launch<true>(dst, src, n, c, h, w, eb, s);
}
cudaError_t launch_reorder_from_blocked(void *dst, const void *src, int n, int c, int h, int w, int eb, cudaStream_t s) {
  return launch<false>(dst, src, n, c, h, w, eb, s);
}

}  // namespace elb
