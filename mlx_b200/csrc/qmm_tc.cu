// Prefill-regime quantized GEMM (TMA + tcgen05 + TMEM).  Placeholder until the
// kernel lands: reports "unsupported" so callers take the decode kernel in
// 16-row passes.
#include "internal.h"

namespace luxcuda {
bool qmm_tc_supported(const QmmArgs&) { return false; }
cudaError_t launch_qmm_tc(const QmmArgs&, int, cudaStream_t, const char**) { return cudaErrorNotSupported; }
}  // namespace luxcuda
