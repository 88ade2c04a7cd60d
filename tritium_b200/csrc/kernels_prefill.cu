// Prefill GEMM placeholder translation unit (replaced by the tcgen05 kernel).
#include "tb_internal.h"

bool tb_prefill_supported(const tb_weights*, uint32_t) { return false; }
size_t tb_prefill_scratch_bytes(const tb_weights*, uint32_t) { return 0; }
cudaError_t tb_launch_prefill(const PrefillArgs&, int, cudaStream_t) { return cudaErrorNotSupported; }
