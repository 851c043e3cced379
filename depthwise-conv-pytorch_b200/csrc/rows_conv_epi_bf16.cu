// Rows family, forward with a fused epilogue in bf16.
#include "rows_conv_epi_ops.cuh"

namespace dwb {

int rows_conv_epi_bf16_take_error() { return conv_take_error_here(); }

template int rows_forward_epilogue<__nv_bfloat16>(const __nv_bfloat16 *, const __nv_bfloat16 *, __nv_bfloat16 *, const Shape &, const EpilogueArgs &, cudaStream_t);

}  // namespace dwb
