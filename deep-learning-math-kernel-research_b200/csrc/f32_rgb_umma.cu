// FP32 3x3 stride-1 pad-1 convolution of an nchw image with at most four channels into 64 output
// channels (the first layer of an image network: VGG-16 conv1_1) on the tensor cores.
//
// The reference runs such a layer through its Winograd pipeline like any other
// (src/elx_conv_wino.cpp); this library serves it directly (see f32_small_ic.cu for why).  The
// CUDA-core kernel there needs 1728 FMAs per output pixel and runs at 2.3x the time its output
// alone takes to write.  Here the same convolution is an implicit GEMM on tcgen05:
//
//   rows    = 128 output pixels, a tile of 4 image rows x 32 pixels (TMEM lane r = row r)
//   K       = 9 taps x ic channels, index tap*ic + channel (27 for an RGB image), in steps of 8
//   columns = the 64 output channels, twice: the weights are STACKED, rows [0,64) of the operand
//             image their tf32 hi parts and rows [64,128) the lo parts
//   3xTF32: per K step  D[:, 0:128] += A_hi * [B_hi ; B_lo]  and  D[:, 0:64] += A_lo * B_hi  with
//   hi = cvt.rna.tf32(x), lo = x - hi, fp32 accumulate; the epilogue adds columns [64,128) to
//   [0,64) -- the arithmetic of the Winograd GEMM (wino.cu), ~1e-6 of the exact result.  (An MMA
//   this small costs its fixed latency, ~110 cycles, whatever it multiplies: 8 per tile instead
//   of the 15 of five 4-slot K steps with three MMAs each.)
//
// Measured on B200, VGG-16 conv1_1 inside the fp32 stack, 64 images: 0.29 ms with the CUDA-core
// kernel, 0.20-0.22 ms with this one (the 822 MB of output alone take 0.13 ms).  The per-CTA
// timeline shows a tile every ~1600 cycles with builders, issuer and epilogue groups each busy
// most of that; with the stores switched off it is 1380 cycles, i.e. the launch writes at the
// rate of HBM while an epilogue group stores.
//
// Nothing of A ever touches shared memory: the thread that owns output pixel r reads its 27 input
// values from the three planes (neighbouring lanes read neighbouring floats), splits them and writes
// both planes to ITS lane of tensor memory (tcgen05.st), from where the MMAs read them
// (tcgen05.mma with the A operand in tensor memory).  B, the weights, is split once per CTA into a
// K-major shared-memory image.  One CTA per SM, warp roles:
//   warps 0-3, 4-7   two groups of A builders, taking turns on the CTA's tiles (buffer g = group g)
//   warps 8-11, 12-15 two epilogue groups, taking turns likewise (accumulator e = group e):
//                    accumulator -> registers -> bias, ReLU -> 256-bit stores (nChw16c).  The stores of
//                    a tile take as long as everything else about it (the launch writes at the
//                    rate of HBM while they last), so one group's stores overlap the other's loads
//   warp  16         lane 0 issues the MMAs of a tile
// Every wait is bounded (mbar_wait); a wait that gives up raises the CTA's abort flag, the roles
// leave their loops and the status word is set.
#include <cuda_runtime.h>

#include "elb_common.cuh"
#include "umma.cuh"
#include "wino.cuh"

namespace elb {

namespace {

constexpr int RGB_BN = 64;                  // output channels (columns)
constexpr int RGB_TW = 32, RGB_TH = 4;      // tile: 4 rows of 32 pixels = 128 GEMM rows
constexpr int RGB_KCH = 10;                 // K chunks of 4 values (at most 9 taps x 4 channels = 36 -> 40)
constexpr int RGB_THREADS = 17 * 32;
constexpr int RGB_EPI_WARP0 = 8, RGB_MMA_WARP = 16;
constexpr uint32_t RGB_TMEM_COLS = 512;
constexpr uint32_t RGB_ACC = 2 * RGB_BN;    // columns of one accumulator (hi and lo halves)
constexpr uint32_t RGB_A_COL0 = 2 * RGB_ACC;// two accumulators, the A planes behind them
constexpr uint32_t RGB_A_PLANE = 48;        // columns of one plane (40 used; written 16 at a time)

__device__ __forceinline__ void st_global_v8(void *ptr, const float (&v)[8]) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "f"(v[0]), "f"(v[1]), "f"(v[2]),
               "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}

template <int IC>      // input channels (1..4; 3 = an RGB image)
__global__ void __launch_bounds__(RGB_THREADS, 1) f32_rgb_umma_kernel(const __grid_constant__ SmallIcParams p,
                                                                       int *__restrict__ status) {
  __shared__ __align__(128) float s_b[RGB_KCH][2 * RGB_BN][4];     // weights: [K chunk][hi rows | lo rows][4 K values]
  __shared__ float s_bias[RGB_BN];
  __shared__ __align__(8) uint64_t s_bar[8];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  uint64_t *a_full = s_bar, *a_empty = s_bar + 2, *tfull = s_bar + 4, *tempty = s_bar + 6;
  volatile int *abort_flag = &s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int g = 0; g < 2; ++g) {
      mbar_init(&a_full[g], 4);       // one arrival per builder warp of the group
      mbar_init(&a_empty[g], 1);      // the commit behind the tile's MMAs
      mbar_init(&tfull[g], 1);
      mbar_init(&tempty[g], 4);       // one arrival per epilogue warp
    }
    s_abort = 0;
    fence_barrier_init();
  }
  if (warp == RGB_MMA_WARP) tmem_alloc(&s_tmem, RGB_TMEM_COLS);
  // the operand image of the weights: K index kk = tap * ic + channel, chunk kk / 4
  constexpr int kreal = 9 * IC;                     // 27 for an RGB image
  constexpr int ksteps = (kreal + 7) >> 3;
  for (int i = threadIdx.x; i < RGB_KCH * RGB_BN * 4; i += RGB_THREADS) {
    const int kk = (i / (RGB_BN * 4)) * 4 + (i & 3), n = (i >> 2) % RGB_BN;
    const int tap = kk / IC, c = kk - tap * IC;
    const float w = kk < kreal ? p.w[(tap * 4 + c) * (p.OCB * 16) + n] : 0.0f;
    uint32_t hb;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(w));
    s_b[kk >> 2][n][kk & 3] = __uint_as_float(hb);
    s_b[kk >> 2][RGB_BN + n][kk & 3] = __fsub_rn(w, __uint_as_float(hb));
  }
  for (int i = threadIdx.x; i < RGB_BN; i += RGB_THREADS) s_bias[i] = p.with_bias ? p.bias[i] : 0.0f;
  fence_proxy_async_smem();           // the MMAs read the image through the asynchronous proxy
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = s_tmem;
  int fail_code = 0;
  // optional timeline: stamp `what` (0..7) of the CTA's j-th tile, first eight tiles
#define RGB_TRACE(j, what) do { if (p.trace && (j) < 8u) p.trace[blockIdx.x * 64 + (j) * 8 + (what)] = clock64(); } while (0)

  const int tiles_w = (p.W + RGB_TW - 1) / RGB_TW, tiles_h = (p.H + RGB_TH - 1) / RGB_TH;
  const int per_img = tiles_w * tiles_h;
  const int total_tiles = p.N * per_img;

  if (warp < RGB_EPI_WARP0) {
    // ---------------------------------------------------------------- A builders
    const int g = warp >> 2, quarter = warp & 3;
    const size_t plane = static_cast<size_t>(p.H) * p.W;
    uint32_t k = 0;
    bool ok = true;
    for (int tile = blockIdx.x + g * gridDim.x; tile < total_tiles && ok; tile += 2 * gridDim.x, ++k) {
      if ((threadIdx.x & 127) == 0) RGB_TRACE(g + 2 * k, 0);
      const int n = tile / per_img, r = tile - n * per_img;
      const int oh = (r / tiles_w) * RGB_TH + quarter, ow = (r % tiles_w) * RGB_TW + lane;
      const float *in_n = p.in + static_cast<size_t>(n) * IC * plane;
      // All 27 loads are issued before any value is used (clamped addresses, so none of them is
      // conditional): issued one by one behind their uses they cost the warp 27 memory latencies per
      // tile (measured: 6400 cycles per tile, twice the CUDA-core kernel's time).
      const bool live = oh < p.H && ow < p.W;
      float xv[9][IC];
#pragma unroll
      for (int kh = 0; kh < 3; ++kh) {
        const int ihc = min(max(oh - 1 + kh, 0), p.H - 1);
#pragma unroll
        for (int kw = 0; kw < 3; ++kw) {
          const int iwc = min(max(ow - 1 + kw, 0), p.W - 1);
          const float *px = in_n + static_cast<size_t>(ihc) * p.W + iwc;
#pragma unroll
          for (int c = 0; c < IC; ++c) xv[kh * 3 + kw][c] = __ldg(px + c * plane);
        }
      }
      // which taps lie inside the image (bit tap); dead rows of a ragged tile contribute zeros
      uint32_t okmask = 0;
#pragma unroll
      for (int kh = 0; kh < 3; ++kh)
#pragma unroll
        for (int kw = 0; kw < 3; ++kw) {
          const int ih = oh - 1 + kh, iw = ow - 1 + kw;
          if (live && ih >= 0 && ih < p.H && iw >= 0 && iw < p.W) okmask |= 1u << (kh * 3 + kw);
        }
      // the thread's row of A, column tap * IC + channel, split into its planes BEFORE the wait for the
      // buffer, so that only the stores to tensor memory stand between that wait and the hand-over
      constexpr int NBLK = (ksteps + 1) / 2;      // blocks of 16 columns
      uint32_t h[NBLK][16], l[NBLK][16];
#pragma unroll
      for (int i = 0; i < NBLK; ++i) {
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
          const int col = i * 16 + jj;
          if (col < kreal) {
            const int tap = col / IC, c = col - tap * IC;
            const float x = ((okmask >> tap) & 1u) ? xv[tap][c] : 0.0f;
            uint32_t hb;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(x));
            h[i][jj] = hb;
            l[i][jj] = __float_as_uint(__fsub_rn(x, __uint_as_float(hb)));
          } else {
            h[i][jj] = 0u;
            l[i][jj] = 0u;
          }
        }
      }
      if ((threadIdx.x & 127) == 0) RGB_TRACE(g + 2 * k, 1);
      // the buffer is free once the MMAs of this group's previous tile have read it
      if (!mbar_wait_warp(&a_empty[g], (k & 1u) ^ 1u, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_PRODUCER; break; }
      tc_fence_after_sync();
      const uint32_t t_hi = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + RGB_A_COL0 + g * 2 * RGB_A_PLANE;
#pragma unroll
      for (int i = 0; i < NBLK; ++i) {
        tmem_st16(t_hi + i * 16, h[i]);
        tmem_st16(t_hi + RGB_A_PLANE + i * 16, l[i]);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[g]);
      if ((threadIdx.x & 127) == 0) RGB_TRACE(g + 2 * k, 2);
    }
  } else if (warp == RGB_MMA_WARP) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t IDESC_HI = umma_idesc(1, 2, 2, 128, RGB_BN);           // rows [0,64) of the image: hi
      constexpr uint32_t IDESC_BOTH = umma_idesc(1, 2, 2, 128, 2 * RGB_BN);     // all 128 rows: hi and lo
      constexpr uint32_t LBO = 2 * RGB_BN * 16;      // distance between the two K chunks of one instruction
      const uint64_t b_desc = umma_desc_kmajor(smem_u32(&s_b[0][0][0]), LBO, 128);
      uint32_t j = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++j) {
        const uint32_t g = j & 1u, ph = (j >> 1) & 1u;
        if (!mbar_wait(&tempty[g], ph ^ 1u, abort_flag) || !mbar_wait(&a_full[g], ph, abort_flag)) {
          fail_code = ST_WAIT_TIMEOUT_MMA;
          break;
        }
        tc_fence_after_sync();
        RGB_TRACE(j, 3);
        const uint32_t d = tmem_base + g * RGB_ACC;
        const uint32_t a_hi = tmem_base + RGB_A_COL0 + g * 2 * RGB_A_PLANE, a_lo = a_hi + RGB_A_PLANE;
#pragma unroll
        for (int ks = 0; ks < RGB_KCH / 2; ++ks) {
          if (ks < ksteps) {
            const uint64_t b = b_desc + ((ks * 2 * LBO) >> 4);
            umma_tf32_ts(d, a_hi + ks * 8, b, IDESC_BOTH, ks != 0 ? 1u : 0u);      // [0,64) += hi*hi, [64,128) += hi*lo
            umma_tf32_ts(d, a_lo + ks * 8, b, IDESC_HI, 1u);                        // [0,64) += lo*hi
          }
        }
        umma_commit(&a_empty[g]);      // the A buffer may be rewritten ...
        umma_commit(&tfull[g]);        // ... and the accumulator read, once these MMAs are done
        RGB_TRACE(j, 4);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (warp & 3 = its TMEM lane quarter)
    const int quarter = warp & 3;
    const uint32_t g = static_cast<uint32_t>(warp - RGB_EPI_WARP0) >> 2;      // group = accumulator buffer
    uint32_t j = g;
    bool ok = true;
    for (int tile = blockIdx.x + g * gridDim.x; tile < total_tiles && ok; tile += 2 * gridDim.x, j += 2) {
      const uint32_t ph = (j >> 1) & 1u;
      const int n = tile / per_img, r = tile - n * per_img;
      const int oh = (r / tiles_w) * RGB_TH + quarter, ow = (r % tiles_w) * RGB_TW + lane;
      if (!mbar_wait_warp(&tfull[g], ph, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_EPILOGUE; break; }
      tc_fence_after_sync();
      if ((threadIdx.x & 127) == 0) RGB_TRACE(j, 5);
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + g * RGB_ACC;
      // Columns [0,64) and their partners [64,128) are added block by block as they arrive (32 registers
      // in flight, 64 kept), the accumulator is handed back, and only then does the warp store: the
      // stores are the slow part, and the MMAs of the group's next tile wait for this buffer.
      float sum[4][16];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        uint32_t acc[16], part[16];
        tmem_ld16(t_addr + b * 16, acc);
        tmem_ld16(t_addr + RGB_BN + b * 16, part);
        tmem_ld_wait16(acc);
        tmem_ld_wait16(part);
#pragma unroll
        for (int i = 0; i < 16; ++i) sum[b][i] = __fadd_rn(__uint_as_float(acc[i]), __uint_as_float(part[i]));
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[g]);
      if ((threadIdx.x & 127) == 0) RGB_TRACE(j, 6);
      if (oh < p.H && ow < p.W) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          float *dst = p.out + (((static_cast<size_t>(n) * p.OCB + b) * p.H + oh) * p.W + ow) * 16;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              v[i] = __fadd_rn(sum[b][half * 8 + i], s_bias[b * 16 + half * 8 + i]);
              if (p.with_relu) v[i] = fmaxf(v[i], 0.0f);
            }
            st_global_v8(dst + half * 8, v);
          }
        }
      }
      if ((threadIdx.x & 127) == 0) RGB_TRACE(j, 7);
    }
  }

  if (fail_code != 0) atomicCAS(status, 0, fail_code);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == RGB_MMA_WARP) {
    __syncwarp();
    tmem_dealloc(tmem_base, RGB_TMEM_COLS);
  }
}

}  // namespace

// The shapes this kernel takes: an nchw image, exactly 64 (padded) output channels, no in-place sum.
bool f32_rgb_umma_supported(const SmallIcParams &p) {
  return p.planar && p.OCB * 16 == RGB_BN && !p.with_sum && p.ic >= 1 && p.ic <= 4;
}

cudaError_t launch_f32_rgb_umma(const SmallIcParams &p, int num_sms, int *status, cudaStream_t s) {
  const long long tiles = static_cast<long long>(p.N) * ((p.W + RGB_TW - 1) / RGB_TW) * ((p.H + RGB_TH - 1) / RGB_TH);
  const int grid = static_cast<int>(tiles < num_sms ? tiles : num_sms);
  switch (p.ic) {
    case 1: f32_rgb_umma_kernel<1><<<grid, RGB_THREADS, 0, s>>>(p, status); break;
    case 2: f32_rgb_umma_kernel<2><<<grid, RGB_THREADS, 0, s>>>(p, status); break;
    case 3: f32_rgb_umma_kernel<3><<<grid, RGB_THREADS, 0, s>>>(p, status); break;
    default: f32_rgb_umma_kernel<4><<<grid, RGB_THREADS, 0, s>>>(p, status); break;
  }
  return cudaGetLastError();
}

}  // namespace elb
