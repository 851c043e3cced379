// placeholder: rows engine not yet built; every request is declined.
#pragma once
#include "common.cuh"
namespace dwb {
enum { ROWS_DECLINED = 0, ROWS_SERVED = 1 };
template <typename T> int rows_forward(const T *, const T *, T *, const Shape &, cudaStream_t) { return ROWS_DECLINED; }
template <typename T> int rows_backward_input(const T *, const T *, T *, const Shape &, cudaStream_t) { return ROWS_DECLINED; }
template <typename T> int rows_backward_filter_slices(const Shape &) { return 0; }
template <typename T> int rows_backward_filter(const T *, const T *, typename Elem<T>::acc_t *, const Shape &, cudaStream_t, int *) { return ROWS_DECLINED; }
}
