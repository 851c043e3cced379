// Rows family, forward with a fused epilogue in f16.
#include "rows_conv_epi_ops.cuh"

namespace dwb {

int rows_conv_epi_f16_take_error() { return conv_take_error_here(); }

template int rows_forward_epilogue<__half>(const __half *, const __half *, __half *, const Shape &, const EpilogueArgs &, cudaStream_t);

}  // namespace dwb
