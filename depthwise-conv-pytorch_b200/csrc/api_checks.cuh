// Argument checks shared by the translation units that define C entry points.
#pragma once

#include <cstdint>

#include "common.cuh"

namespace dwb {

inline bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline size_t elem_size(int dtype) {
  switch (dtype) {
    case DWCONV_B200_F32: return 4;
    case DWCONV_B200_F16: return 2;
    case DWCONV_B200_BF16: return 2;
    case DWCONV_B200_F64: return 8;
    default: return 0;
  }
}

inline int check_shape(const Shape *s) {
  if (s == nullptr) return DWCONV_B200_BAD_ARGUMENT;
  if (s->N <= 0 || s->C <= 0 || s->H <= 0 || s->W <= 0 || s->kh <= 0 || s->kw <= 0 ||
      s->sh <= 0 || s->sw <= 0 || s->ph < 0 || s->pw < 0 || s->Ho <= 0 || s->Wo <= 0)
    return DWCONV_B200_BAD_ARGUMENT;
  // Index arithmetic inside one plane is 32-bit; whole-tensor offsets are 64-bit.
  const long long lim = 1ll << 30;
  if ((long long)s->H * s->W >= lim || (long long)s->Ho * s->Wo >= lim ||
      (long long)s->kh * s->kw >= (1ll << 20) || (long long)s->N * s->C >= (1ll << 31) - 1 ||
      (long long)s->Ho * s->sh + s->kh >= lim || (long long)s->Wo * s->sw + s->kw >= lim)
    return DWCONV_B200_TOO_LARGE;
  return DWCONV_B200_OK;
}


// Defined in api.cu: status of the launches made so far on this thread (records the CUDA error
// for dwconv_b200_last_cuda_error), and the kernel family dwconv_b200_last_path reports.
int api_launch_status();
void api_note_path(int path);

}  // namespace dwb
