#include "wino.cuh"
namespace elb {
int wino_setup(WinoPlan &, const elb_conv_desc_t &, elb_conv_info_t &, std::string &err) { err = "Winograd path not built yet"; return ELB_UNIMPLEMENTED; }
int wino_prepare(WinoPlan &, const elb_conv_desc_t &, elb_conv_info_t &, const void *, const void *, std::string &err) { err = "not built"; return ELB_UNIMPLEMENTED; }
int wino_run(WinoPlan &, void *, const void *, void *, int *, int, cudaStream_t, int &, std::string &err) { err = "not built"; return ELB_UNIMPLEMENTED; }
void wino_release(WinoPlan &) {}
}
