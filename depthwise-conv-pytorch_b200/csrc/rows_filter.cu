// Rows family, backward-filter first pass: variant selection and launch.
#include "rows_plan.cuh"

namespace dwb {

namespace {

__device__ int g_filter_error_flag;

constexpr int filter_u(int K, int S) { return S == 1 ? (K == 3 ? 4 : 2) : (K <= 5 ? 2 : 1); }
constexpr int filter_minb(int K) { return K <= 5 ? 2 : 1; }

inline bool filter_shape_ok(const Shape &s) {
  if (s.kh != s.kw || (s.kh != 3 && s.kh != 5 && s.kh != 7)) return false;
  if (s.sh != s.sw || (s.sh != 1 && s.sh != 2)) return false;
  if (s.ph != s.kh / 2 || s.pw != s.kw / 2) return false;
  if (s.Ho != (s.H + 2 * s.ph - s.kh) / s.sh + 1 || s.Wo != (s.W + 2 * s.pw - s.kw) / s.sw + 1)
    return false;
  return true;
}

// (VI, VO) for the map widths; 0 if none applies.  a16: both tensors 16-byte aligned.
inline int pick_v(int S, int W, int Wo, bool a16, int &VI, int &VO) {
  if (S == 1) {
    if (a16 && W % 4 == 0 && W <= 128 && W > 16) { VI = VO = 4; return 1; }
    if (a16 && W % 2 == 0 && W <= 64 && W > 8) { VI = VO = 2; return 1; }
    if (W <= 32) { VI = VO = 1; return 1; }
    return 0;
  }
  if (a16 && W % 4 == 0 && Wo % 2 == 0 && W <= 128 && W > 16) { VI = 4; VO = 2; return 1; }
  if (a16 && W % 2 == 0 && W <= 64) { VI = 2; VO = 1; return 1; }
  return 0;
}

template <typename T>
bool plan_filter(const Shape &s, bool a16, RowsFilterParams &p, int &VI, int &VO) {
  if (!filter_shape_ok(s)) return false;
  const int K = s.kh, S = s.sh;
  if (!pick_v(S, s.W, s.Wo, a16, VI, VO)) return false;
  const int lanes = max(ceil_div(s.W, VI), ceil_div(s.Wo, VO));
  p.LW = pick_lw(lanes);
  if (p.LW == 0) return false;
  const int NSEG = ROWS_WARPS * (32 / p.LW);
  const int U = filter_u(K, S);
  TilePlan t;
  // the dy region starts on a 128-byte boundary: keep that slack out of the budget
  if (!plan_tiles(t, K, S, MODE_FWD, U, s.H, s.Ho, s.W * (int)sizeof(T), s.Wo * (int)sizeof(T),
                  NSEG, ROWS_STAGE_BYTES - 128))
    return false;
  p.N = s.N; p.C = s.C; p.H = s.H; p.W = s.W; p.Ho = s.Ho; p.Wo = s.Wo;
  p.G = t.G; p.NRT = t.NRT; p.TH = t.TH; p.NRB = t.NRB; p.RBH = t.RBH;
  const int xrows = (p.G > 1) ? s.H : min(s.H, (p.TH - 1) * S + K);
  p.XPL = xrows * s.W;
  p.DPL = p.TH * s.Wo;
  p.DYOFF = round_up(p.G * p.XPL * (int)sizeof(T), 128);
  if (p.DYOFF + p.G * p.DPL * (int)sizeof(T) > ROWS_STAGE_BYTES) return false;
  p.TPC = ceil_div(s.N, p.G) * p.NRT;
  int SL = ceil_div(4 * sm_count(), s.C);
  if (SL > p.TPC) SL = p.TPC;
  if (SL < 1) SL = 1;
  p.SL = SL;
  p.x_bulk = ((size_t)s.H * s.W * sizeof(T)) % 16 == 0;
  p.dy_bulk = ((size_t)s.Ho * s.Wo * sizeof(T)) % 16 == 0;
  return true;
}

template <typename T, int K, int S, int VI, int VO>
int launch_filter(const RowsFilterParams &p, cudaStream_t st) {
  constexpr int U = filter_u(K, S);
  constexpr int MINB = filter_minb(K);
  auto kernel = rows_filter_kernel<T, K, S, VI, VO, U, MINB>;
  static std::atomic<unsigned long long> smem_done{0};
  if (!ensure_smem(kernel, ROWS_SMEM_BYTES, smem_done)) return ROWS_DECLINED;
  int *flag = nullptr;
  if (cudaGetSymbolAddress((void **)&flag, g_filter_error_flag) != cudaSuccess) {
    (void)cudaGetLastError();
    return ROWS_DECLINED;
  }
  kernel<<<p.C * p.SL, ROWS_THREADS, ROWS_SMEM_BYTES, st>>>(p, flag);
  return ROWS_SERVED;
}

template <typename T, int K, int S>
int select_filter_v(const RowsFilterParams &p, int VI, cudaStream_t st) {
  if (S == 1) {
    if (VI == 4) return launch_filter<T, K, 1, 4, 4>(p, st);
    if (VI == 2) return launch_filter<T, K, 1, 2, 2>(p, st);
    return launch_filter<T, K, 1, 1, 1>(p, st);
  }
  if (VI == 4) return launch_filter<T, K, 2, 4, 2>(p, st);
  return launch_filter<T, K, 2, 2, 1>(p, st);
}

template <typename T> struct RowsDtype { static constexpr bool ok = false; };
template <> struct RowsDtype<float> { static constexpr bool ok = true; };
template <> struct RowsDtype<__half> { static constexpr bool ok = true; };

}  // namespace

template <typename T> int rows_backward_filter_slices(const Shape &s) {
  if constexpr (!RowsDtype<T>::ok) {
    return 0;
  } else {
    // alignment is not known here: report the largest slice count either choice would use
    RowsFilterParams p{};
    int VI, VO, best = 0;
    for (int a16 = 0; a16 < 2; ++a16)
      if (plan_filter<T>(s, a16 != 0, p, VI, VO) && p.SL > best) best = p.SL;
    return best;
  }
}

template <typename T>
int rows_backward_filter(const T *x, const T *dy, typename Elem<T>::acc_t *partial, const Shape &s,
                         cudaStream_t st, int *slices_out) {
  if constexpr (!RowsDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    const bool a16 = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy)) & 15) == 0;
    RowsFilterParams p{};
    int VI, VO;
    if (!plan_filter<T>(s, a16, p, VI, VO)) return ROWS_DECLINED;
    p.x = x; p.dy = dy; p.partial = partial;
    *slices_out = p.SL;
    switch (s.kh * 10 + s.sh) {
      case 31: return select_filter_v<T, 3, 1>(p, VI, st);
      case 51: return select_filter_v<T, 5, 1>(p, VI, st);
      case 71: return select_filter_v<T, 7, 1>(p, VI, st);
      case 32: return select_filter_v<T, 3, 2>(p, VI, st);
      case 52: return select_filter_v<T, 5, 2>(p, VI, st);
      case 72: return select_filter_v<T, 7, 2>(p, VI, st);
      default: return ROWS_DECLINED;
    }
  }
}

int rows_filter_take_error() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_filter_error_flag, sizeof(int)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (v) {
    const int zero = 0;
    (void)cudaMemcpyToSymbol(g_filter_error_flag, &zero, sizeof(int));
  }
  return v;
}

int rows_take_device_error() { return rows_conv_take_error() | rows_filter_take_error(); }

template int rows_backward_filter_slices<float>(const Shape &);
template int rows_backward_filter_slices<__half>(const Shape &);
template int rows_backward_filter_slices<double>(const Shape &);
template int rows_backward_filter<float>(const float *, const float *, float *, const Shape &, cudaStream_t, int *);
template int rows_backward_filter<__half>(const __half *, const __half *, float *, const Shape &, cudaStream_t, int *);
template int rows_backward_filter<double>(const double *, const double *, double *, const Shape &, cudaStream_t, int *);

}  // namespace dwb
