// tcgen05 implicit-GEMM path (placeholder until the tensor-core kernel lands).
#include "common.cuh"

int wdc_tc_conv2d(wdc_context*, const wdc_conv_desc*, const float*, const float*, const float*,
                  const float*, const float*, float*) {
  return WDC_ERR_UNSUPPORTED;
}
int wdc_tc_gemm(wdc_context*, const wdc_gemm_desc*, const float*, const float*, const float*, float*) {
  return WDC_ERR_UNSUPPORTED;
}
void wdc_tc_destroy(wdc_context*) {}
