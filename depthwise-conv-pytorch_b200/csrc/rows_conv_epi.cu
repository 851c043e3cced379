// Rows family, forward with a fused epilogue: fp32 (fp64 declines) and the error flags of the
// three translation units.
#include "rows_conv_epi_ops.cuh"

namespace dwb {

int rows_conv_epi_f16_take_error();   // rows_conv_epi_f16.cu
int rows_conv_epi_bf16_take_error();  // rows_conv_epi_bf16.cu

int rows_conv_epi_take_error() {
  return conv_take_error_here() | rows_conv_epi_f16_take_error() | rows_conv_epi_bf16_take_error();
}

template int rows_forward_epilogue<float>(const float *, const float *, float *, const Shape &, const EpilogueArgs &, cudaStream_t);
template int rows_forward_epilogue<double>(const double *, const double *, double *, const Shape &, const EpilogueArgs &, cudaStream_t);

}  // namespace dwb
