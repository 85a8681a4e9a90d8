// INT8 depthwise 3x3 plan: interface between the C-ABI layer and depthwise.cu.
#pragma once
#include <string>
#include <cuda_runtime.h>
#include "../../include/euler_b200.h"

namespace elb {

struct DwImpl;
struct DwPlan {
  DwImpl *impl = nullptr;
};

// Validate the descriptor the way the reference's constructor does and fix the launch geometry.
int dw_setup(DwPlan &pl, const elb_conv_desc_t &d, elb_conv_info_t &info, int num_sms, std::string &err);
// One-time weight quantisation and constant folding (first execute).
int dw_prepare(DwPlan &pl, const elb_conv_desc_t &d, elb_conv_info_t &info, const void *weights,
               const void *bias, std::string &err);
// Enqueue images [first, first + count) of the batch on stream s (out / in address the full tensors).
int dw_run(DwPlan &pl, void *out, const void *in, void *acc_dump, int first, int count, cudaStream_t s, int &launches,
           std::string &err);
void dw_release(DwPlan &pl);

}  // namespace elb
