// Rows family, forward and backward-input: the plain operators (fp32; fp64 declines), the plan
// inspection and the error flags of the family's forward / backward-input translation units.
#include "rows_conv_ops.cuh"

namespace dwb {

int rows_conv_f16_debug_plan(int op, const Shape &s, int a16, int *out);  // rows_conv_f16.cu

// Plan inspection (rows_debug_conv_plan_t) for an element size: the planner treats both 16-bit
// types alike.
int rows_debug_conv_plan(int op, int esize, const Shape &s, int a16, int *out) {
  if (esize == 4) return rows_debug_conv_plan_t<float>(op, s, a16, out);
  if (esize == 2) return rows_conv_f16_debug_plan(op, s, a16, out);
  return 0;
}

int rows_conv_epi_take_error();  // rows_conv_epi.cu (and its 16-bit siblings)
int rows_conv_f16_take_error();   // rows_conv_f16.cu
int rows_conv_bf16_take_error();  // rows_conv_bf16.cu
int tiles_tma_take_error();      // tiles_tma.cu
int nhwc_tma_take_error();       // nhwc_tma.cu

int rows_conv_take_error() {
  return conv_take_error_here() | rows_conv_f16_take_error() | rows_conv_bf16_take_error() |
         rows_conv_epi_take_error() | rows_bigk_take_error() |
         tiles_tma_take_error() | nhwc_tma_take_error();
}

template int rows_forward<float>(const float *, const float *, float *, const Shape &, cudaStream_t);
template int rows_forward<double>(const double *, const double *, double *, const Shape &, cudaStream_t);
template int rows_backward_input<float>(const float *, const float *, float *, const Shape &, cudaStream_t);
template int rows_backward_input<double>(const double *, const double *, double *, const Shape &, cudaStream_t);

}  // namespace dwb
