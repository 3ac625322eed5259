// Entry points whose kernels are not built yet answer CROQ_ERR_UNSUPPORTED.
#include "croq_host.h"

extern "C" {
int croq_gemm_sp_f16(const croq_view2*, const croq_view2*, const croq_view2*, const croq_view2*,
                     int, croq_stream) {
  return CROQ_ERR_UNSUPPORTED;
}
}
