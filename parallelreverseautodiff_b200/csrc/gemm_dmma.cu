// placeholder until the DMMA kernel lands: reports every shape as unsupported
#include "common.cuh"
namespace prad {
prad_status gemm_f64_dmma(prad_ctx*, bool, bool, int, int, int, double, const void*, int,
                          const void*, int, double, void*, int, int, int64_t, int64_t, int64_t,
                          const GemmEpilogue&, bool) {
  return PRAD_ERR_UNSUPPORTED;
}
}  // namespace prad
