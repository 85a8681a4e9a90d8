// Shared declarations of the CUDA translation units: kernel parameter blocks, the fused
// requantisation epilogue, status codes and the launcher prototypes the C-ABI layer calls.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cuda.h>
#include <cuda_runtime.h>

namespace elb {

constexpr int V = 16;   // channel block of nChw16c / OIhw16i16o

// Kernel tuning switches.  They read the environment only in builds made with -DELB_TUNING (kernel
// experiments); the library as shipped ignores the environment and always returns the default, so
// a user's environment cannot change which kernel variant runs.
inline int tune_env(const char *name, int dflt) {
#ifdef ELB_TUNING
  if (const char *e = getenv(name)) return atoi(e);
#endif
  (void)name;
  return dflt;
}

// A kernel launched with programmatic stream serialisation (launch_overlapped below) may
// start while the kernel before it in the stream is still running, once every CTA of that kernel has
// executed griddep_launch_dependents() or has finished.  Such a kernel must execute griddep_wait()
// before its first access to global memory that an earlier kernel writes or reads: the wait returns
// when the earlier kernel has completed and its writes are visible.  What runs before the wait (barrier
// initialisation, tensor-memory allocation, loading per-plan constants) overlaps the tail of the
// earlier kernel.  In a kernel launched the plain way both instructions do nothing.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launch a kernel that may overlap its set-up with the tail of the kernel before it in the stream
// (the kernel must contain griddep_wait).  Captured into a CUDA graph the
// dependency becomes a programmatic edge.  Only the INT8 tensor-core kernels are launched this way:
// their set-up (barriers, tensor memory, per-channel constants, the copy table) is 2-3 us of a launch
// that may last 10 us.  Measured on the fp32 Winograd path: overlapped launches of the GEMM and the
// input transform change nothing, and the output transform launched as an early dependent is SLOWER
// (c1 0.506 -> 0.550 ms, with all three 0.592 ms; the fp32 stack 24.2 -> 28.5 ms), so those stay plain.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                     Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = tune_env("ELB_NO_OVERLAP", 0) ? 0 : 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// device status word values (0 = ok)
enum : int {
  ST_OK = 0,
  ST_WAIT_TIMEOUT_PRODUCER = 101,   // producer waited too long for a free shared-memory stage
  ST_WAIT_TIMEOUT_MMA = 102,        // MMA issuer waited too long for operands or a free accumulator
  ST_WAIT_TIMEOUT_EPILOGUE = 103,   // epilogue waited too long for an accumulator
  ST_WAIT_TIMEOUT_TEST = 104        // the deliberate give-up of the wait self-test
};

enum : int { OUT_F32 = 0, OUT_U8 = 1, OUT_S8 = 2 };

// ---------------------------------------------------------------------------------------------
// Requantisation of 16 consecutive output channels of one pixel.
// Arithmetic of the reference's int8 epilogues (src/kernel/elk_u8s8_gemm.hxx:200-256,
// src/kernel/elk_u8s8_conv.hxx:218-243), in its order:
//   f = fma((float)acc, scale, shift)            (one fused multiply-add in the reference build)
//   f = fma((float)prev, sum_scale, f)           if in-place sum (u8/s8 outputs only)
//   f = min(max(f, relu_lo), relu_hi)            if ReLU
//   q = round-to-nearest-even(f); u8: values outside [0,255] -> 255 (unsigned saturation of the
//       int32 bit pattern, so negatives become 255); s8: clamp to [-128,127]
// ---------------------------------------------------------------------------------------------
struct Requant {
  int out_type;
  int relu;
  int with_sum;
  float relu_lo, relu_hi, sum_scale;
};

__device__ __forceinline__ float requant_one(int acc, float sc, float sh) {
  return __fmaf_rn(__int2float_rn(acc), sc, sh);
}

// acc: 16 int32 accumulators; sc/sh: 16 per-channel constants; out/prev: address of the 16-channel
// group in the output tensor (prev == out for the in-place sum).
__device__ __forceinline__ void requant_store16(const int (&acc)[16], const float *__restrict__ sc,
                                                const float *__restrict__ sh, void *out, const Requant &rq) {
  float f[16];
  // the constants of the 16 channels are 64-byte aligned: four 16-byte loads per array
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 c = reinterpret_cast<const float4 *>(sc)[i], h = reinterpret_cast<const float4 *>(sh)[i];
    f[4 * i + 0] = requant_one(acc[4 * i + 0], c.x, h.x);
    f[4 * i + 1] = requant_one(acc[4 * i + 1], c.y, h.y);
    f[4 * i + 2] = requant_one(acc[4 * i + 2], c.z, h.z);
    f[4 * i + 3] = requant_one(acc[4 * i + 3], c.w, h.w);
  }
  // (an upper bound of +inf -- plain ReLU -- needs no min; the test is uniform)
  const bool clamp_hi = rq.relu_hi < 3.0e38f;
  if (rq.out_type == OUT_F32) {
    if (rq.relu) {
      if (clamp_hi) {
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] = fminf(fmaxf(f[i], rq.relu_lo), rq.relu_hi);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] = fmaxf(f[i], rq.relu_lo);
      }
    }
    float4 *o = reinterpret_cast<float4 *>(out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
    return;
  }
  if (rq.with_sum) {
    const uint4 pv = *reinterpret_cast<const uint4 *>(out);
    const uint32_t w[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t b = (w[i >> 2] >> (8 * (i & 3))) & 0xFFu;
      const float p = rq.out_type == OUT_U8 ? static_cast<float>(b)
                                            : static_cast<float>(static_cast<int>(static_cast<int8_t>(b)));
      f[i] = __fmaf_rn(p, rq.sum_scale, f[i]);
    }
  }
  if (rq.relu) {
    if (clamp_hi) {
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = fminf(fmaxf(f[i], rq.relu_lo), rq.relu_hi);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = fmaxf(f[i], rq.relu_lo);
    }
  }
  uint32_t w[4];
  // Packing with saturation.  s8: signed saturation is what the reference does.  u8: the reference
  // saturates the int32 bit pattern as UNSIGNED (negatives -> 255); when ReLU with a non-negative
  // lower bound is on no negative value can reach this point and the plain saturating pack is
  // identical, otherwise the unsigned rule is applied explicitly.
  if (rq.out_type == OUT_S8 || (rq.relu && rq.relu_lo >= 0.0f)) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r0 = __float2int_rn(f[4 * i]), r1 = __float2int_rn(f[4 * i + 1]);
      const int r2 = __float2int_rn(f[4 * i + 2]), r3 = __float2int_rn(f[4 * i + 3]);
      uint32_t hi, lo;
      if (rq.out_type == OUT_S8) {
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(r3), "r"(r2));
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(lo) : "r"(r1), "r"(r0), "r"(hi));
      } else {
        asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(r3), "r"(r2));
        asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(lo) : "r"(r1), "r"(r0), "r"(hi));
      }
      w[i] = lo;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int r = __float2int_rn(f[i]);
      const uint32_t b = (static_cast<uint32_t>(r) > 255u) ? 255u : static_cast<uint32_t>(r);
      w[i >> 2] |= b << (8 * (i & 3));
    }
  }
  *reinterpret_cast<uint4 *>(out) = make_uint4(w[0], w[1], w[2], w[3]);
}

// ---------------------------------------------------------------------------------------------
// INT8 direct convolution (1x1 and KxK) parameter block, shared by the tcgen05 kernels and the
// CUDA-core kernel.
// ---------------------------------------------------------------------------------------------
struct I8ConvParams {
  alignas(64) CUtensorMap tmap[4];   // BOX mode: one map per (row parity, column parity) input plane
  const uint8_t *in;                 // nChw16c u8
  const int8_t *wpack;               // UMMA operand image [n_tile][k_stage][KC][BN][16]
  const int8_t *wplain;              // [OCpad][taps][ICpad] (CUDA-core kernel)
  const float *scale;                // [OCpad] folded iS*Sw(/oS)
  const float *shift;                // [OCpad] folded bias/oS + oz - ...  (pixels that see every filter tap)
  // non-zero input zero point with padding: pixels near a border see fewer taps and take their shift
  // from shift_tbl[hclass[oh] * zp_nw + wclass[ow]][OCpad]; null when one shift vector serves all
  const float *shift_tbl;
  const int *hclass, *wclass;
  int zp_nw, zp_full;                // classes along w; index of the class `shift` holds
  void *out;                         // nChw16c u8 / s8 / f32
  int32_t *acc_dump;                 // optional raw accumulators, nChw16c int32
  int *status;
  long long *trace;                  // optional timeline, 64 slots per CTA (debug)
  Requant rq;
  int N, IH, IW, OH, OW, KH, KW, stride, pad_t, pad_l;
  int CB, OCB;                       // channel blocks of 16 (input / output)
  int M, HW;                         // FLAT mode: M = N*OH*OW rows, HW = OH*OW
  int taps, CBG, k_stages;           // K loop over chunks q = tap*CB + cb (16 channels each), KC chunks per stage
  int Q, box_c;                      // Q = taps*CB chunks in all; one tiled copy fetches box_c chunks of one tap
  int n_tiles, m_tiles;
  int BW, BH, tiles_w, tiles_h;      // BOX mode tile = BH x BW output pixels (BH*BW = 128)
  int merged_rows;                   // BOX mode, stride 1: 4-D tensor map over 8-byte elements
  int spp;                           // BOX mode: pipeline stages a producer warp fills per pass (1 or 2)
  int nprod;                         // BOX mode: producer warps taking turns on the passes (1, 2 or 4)
  int rotate_k;                      // tiles start their K loop at different stages (spreads the weight reads over L2)
  // BOX mode: where each tiled copy of a K stage reads, worked out once on the host instead of with four
  // integer divisions per copy in the one-warp producer loop.  Entry [stage * ncopy + copy] =
  // channel block | (row shift + 8) << 12 | (column shift + 8) << 16 | tensor map << 20; null: compute.
  const uint32_t *tap_tbl;
  int tap_n, ncopy;                  // entries in all; tiled copies per full stage (KC / box_c)
};
constexpr int I8_TAP_TBL_MAX = 1024;   // entries the kernels keep in shared memory

enum : int { I8_MODE_FLAT = 0, I8_MODE_BOX = 1 };

// geometry the host needs to pack weights / size grids for the tcgen05 kernels
struct I8UmmaConfig {
  int BN, KC, STAGES, mode;
  size_t smem_bytes;
  int cta2;            // 1: the two-CTA kernel (int8_conv2.cu): weight rows split over a pair of SMs
  int max_clusters;    // two-CTA kernel: clusters the device holds at once (persistent grid size)
};
I8UmmaConfig i8_umma_config(int ocb, int cb, int taps, int mode);
cudaError_t init_i8_umma(const I8UmmaConfig &cfg);   // per-device kernel attributes, call once per plan
cudaError_t launch_i8_umma(const I8ConvParams &p, const I8UmmaConfig &cfg, int num_sms, cudaStream_t s);
cudaError_t launch_i8_simt(const I8ConvParams &p, cudaStream_t s);
cudaError_t init_i8_umma2(I8UmmaConfig &cfg, int num_sms);    // two-CTA kernel: attributes + cluster occupancy
cudaError_t launch_i8_umma2(const I8ConvParams &p, const I8UmmaConfig &cfg, int num_sms, cudaStream_t s);

// Bounded-wait self test: one CTA waits on an mbarrier nobody arrives at, gives up after
// `limit_ns`, writes ST_WAIT_TIMEOUT_TEST to *status and returns normally.
cudaError_t launch_wait_selftest(int *status, unsigned long long limit_ns, cudaStream_t s);

// layout converters
cudaError_t launch_reorder_to_blocked(void *dst, const void *src, int n, int c, int h, int w, int eb,
                                      cudaStream_t s);
cudaError_t launch_reorder_from_blocked(void *dst, const void *src, int n, int c, int h, int w, int eb,
                                        cudaStream_t s);

// cuTensorMapEncodeTiled, resolved through the runtime (no link-time dependency on libcuda)
typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);
inline PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_encodeTiled>(p);
  }
  return fn;
}

// Any reorder<T, dst, src> of the reference; supported = false when the pair is not one of them.
cudaError_t launch_reorder(void *dst, int dst_fmt, const void *src, int src_fmt, int g, int a, int b, int h,
                           int w, int eb, cudaStream_t s, bool &supported);
// dst[n][C/16][ceil(h/sh)][ceil(w/sw)][16] = src[n][C/16][y*sh][x*sw][16]
cudaError_t launch_subsample_blocked(void *dst, const void *src, int n, int c, int h, int w, int sh, int sw, int eb,
                                     cudaStream_t s);

}  // namespace elb
