// Rows family, forward and backward-input in f16: the instantiations of rows_conv_ops.cuh.
#include "rows_conv_ops.cuh"

namespace dwb {

int rows_conv_f16_take_error() { return conv_take_error_here(); }

int rows_conv_f16_debug_plan(int op, const Shape &s, int a16, int *out) {
  return rows_debug_conv_plan_t<__half>(op, s, a16, out);
}

template int rows_forward<__half>(const __half *, const __half *, __half *, const Shape &, cudaStream_t);
template int rows_backward_input<__half>(const __half *, const __half *, __half *, const Shape &, cudaStream_t);

}  // namespace dwb
