// Rows family, forward and backward-input in bf16: the instantiations of rows_conv_ops.cuh.
#include "rows_conv_ops.cuh"

namespace dwb {

int rows_conv_bf16_take_error() { return conv_take_error_here(); }

template int rows_forward<__nv_bfloat16>(const __nv_bfloat16 *, const __nv_bfloat16 *, __nv_bfloat16 *, const Shape &, cudaStream_t);
template int rows_backward_input<__nv_bfloat16>(const __nv_bfloat16 *, const __nv_bfloat16 *, __nv_bfloat16 *, const Shape &, cudaStream_t);

}  // namespace dwb
