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
};

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

}  // namespace elb
