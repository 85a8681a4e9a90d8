// Winograd F(4x4,3x3) and depthwise plans: interface between the C-ABI layer and wino.cu.
#pragma once
#include <string>
#include <cuda_runtime.h>
#include "../../include/euler_b200.h"

namespace elb {

struct WinoImpl;
struct WinoPlan {
  WinoImpl *impl = nullptr;
  void *trace = nullptr;     // optional debug timeline of the GEMM kernel (64 int64 slots per CTA)
  cudaEvent_t stage_ev[4] = {nullptr, nullptr, nullptr, nullptr};   // optional: recorded before / between / after the three kernels
  // next call only: the input tensor is a plane of src_h x src_w pixels of which the convolution reads
  // every in_step-th row and column (a subsample folded into the input transform); 1 = plain
  int in_step = 1, src_h = 0, src_w = 0;
  // the input tensor is the caller's nchw tensor (only the direct kernel for at most four input
  // channels reads one; set by the C-ABI layer after wino_setup)
  bool in_planar = false;
};
// Can this plan read its input with a step (fp32 Winograd F(4x4,3x3) through the transform kernels)?
bool wino_input_step_supported(const WinoPlan &pl);

// Build the launch geometry for pl from the descriptor (no device work).
int wino_setup(WinoPlan &pl, const elb_conv_desc_t &d, elb_conv_info_t &info, std::string &err);
// One-time weight transform / quantisation / packing into device memory.
int wino_prepare(WinoPlan &pl, const elb_conv_desc_t &d, elb_conv_info_t &info, const void *weights,
                 const void *bias, std::string &err);
// Enqueue the kernels for images [first, first + count) of the batch on stream s (out / in address
// the full tensors); launches = number of kernels launched.
int wino_run(WinoPlan &pl, void *out, const void *in, void *acc_dump, int *status, int num_sms,
             int first, int count, cudaStream_t s, int &launches, std::string &err);
void wino_release(WinoPlan &pl);

// fp32 3x3 stride-1 pad-1 convolution with at most four input channels (f32_small_ic.cu)
struct SmallIcParams {
  const float *in;      // nChw16c fp32 (planar: nchw), first image of the range
  const float *w;       // [9 taps][4 channels][OCP] fp32
  const float *bias;    // [OCP]
  float *out;           // nChw16c fp32
  int N, H, W, CB, OCB, ic;
  int with_bias, with_relu, with_sum;
  int planar;           // the input is the caller's nchw tensor
  long long *trace;     // optional per-CTA timeline of the tensor-core kernel (64 slots per CTA), else null
};
size_t f32_small_ic_smem_bytes(int OCB);
cudaError_t init_f32_small_ic(int OCB);        // once per plan and device (kernel attribute)
cudaError_t launch_f32_small_ic(const SmallIcParams &p, cudaStream_t s);
// the same convolution on the tensor cores for an nchw image and 64 output channels (f32_rgb_umma.cu);
// status = the plan's device status word (a bounded wait that gives up leaves its code there)
bool f32_rgb_umma_supported(const SmallIcParams &p);
cudaError_t launch_f32_rgb_umma(const SmallIcParams &p, int num_sms, int *status, cudaStream_t s);

}  // namespace elb
