// Rows family, backward-filter first pass: variant selection and launch.
#include "rows_plan.cuh"

namespace dwb {

// large filters: rows_bigk.cu
template <typename T> int rows_bigk_filter_slices(const Shape &s);
template <typename T>
int rows_bigk_filter(const T *x, const T *dy, float *partial, const Shape &s, cudaStream_t st,
                     int *slices_out);

namespace {

__device__ int g_filter_error_flag;

constexpr int filter_minb(int K) { return K <= 5 ? 2 : 1; }

// Rows-per-chunk choices compiled for each (K, S); the planner picks per shape.
template <int K, int S> struct FilterU;
template <> struct FilterU<3, 1> { static constexpr int n = 3; static constexpr int v[4] = {4, 7, 8, 8}; };  // 14 measured slower than 7 on 14-row maps
template <> struct FilterU<5, 1> { static constexpr int n = 2; static constexpr int v[4] = {2, 4, 4, 4}; };
template <> struct FilterU<7, 1> { static constexpr int n = 2; static constexpr int v[4] = {2, 4, 4, 4}; };  // 4: 77.9 vs 81.4 us on the 56x56 fp16 layer
template <> struct FilterU<3, 2> { static constexpr int n = 1; static constexpr int v[4] = {2, 2, 2, 2}; };  // 4 and 7 measured slower
template <> struct FilterU<5, 2> { static constexpr int n = 1; static constexpr int v[4] = {2, 2, 2, 2}; };
template <> struct FilterU<7, 2> { static constexpr int n = 1; static constexpr int v[4] = {1, 1, 1, 1}; };

inline bool filter_shape_ok(const Shape &s) {
  if (s.kh != s.kw || (s.kh != 3 && s.kh != 5 && s.kh != 7)) return false;
  if (s.sh != s.sw || (s.sh != 1 && s.sh != 2)) return false;
  if (s.ph != s.kh / 2 || s.pw != s.kw / 2) return false;
  if (s.Ho != (s.H + 2 * s.ph - s.kh) / s.sh + 1 || s.Wo != (s.W + 2 * s.pw - s.kw) / s.sw + 1)
    return false;
  return true;
}

// (VI, VO) for the map widths; false if none applies.  a16: both tensors 16-byte aligned.
inline bool pick_v(int S, int W, int Wo, bool a16, int &VI, int &VO) {
  if (S == 1) {
    if (a16 && W % 4 == 0 && W <= 128 && W > 16) { VI = VO = 4; return true; }
    if (a16 && W % 2 == 0 && W <= 64 && W > 8) { VI = VO = 2; return true; }
    if (W <= 32) { VI = VO = 1; return true; }
    return false;
  }
  if (a16 && W % 4 == 0 && Wo % 2 == 0 && W <= 128 && W > 16) { VI = 4; VO = 2; return true; }
  if (a16 && W % 2 == 0 && W <= 64) { VI = 2; VO = 1; return true; }
  return false;
}

struct FilterPlan {
  RowsFilterParams p;
  int VI, VO, U;
  bool mask, exact;
};

// Options above this height spill registers for the given vector width (ptxas -v); the tables
// are ascending, so a cap keeps a prefix.
constexpr int filter_u_cap(int K, int S, int VI) {
  return (VI == 4 && K == 3 && S == 1) ? 8 : (1 << 20);
}
template <int K, int S> constexpr int filter_u_count(int VI) {
  int n = 0;
  for (int i = 0; i < FilterU<K, S>::n; ++i)
    if (FilterU<K, S>::v[i] <= filter_u_cap(K, S, VI)) ++n;
  return n;
}

template <typename T, int K, int S>
bool plan_filter_ks(const Shape &s, bool a16, FilterPlan &f) {
  if (!pick_v(S, s.W, s.Wo, a16, f.VI, f.VO)) return false;
  const int lanes_in = ceil_div(s.W, f.VI);
  const int lanes = max(lanes_in, ceil_div(s.Wo, f.VO));
  RowsFilterParams &p = f.p;
  p.LW = pick_lw(lanes);
  if (p.LW == 0) return false;
  PlanInput in{K, S, MODE_FWD, s.H, s.W, s.Ho, s.Wo, (int)sizeof(T),
               ROWS_CWARPS * (32 / p.LW), s.C, 0, 0, true};
  const TilePlan t = plan_best(in, FilterU<K, S>::v, filter_u_count<K, S>(f.VI));
  if (!t.ok) return false;
  p.N = s.N; p.C = s.C; p.H = s.H; p.W = s.W; p.Ho = s.Ho; p.Wo = s.Wo;
  p.G = t.G; p.NRT = t.NRT; p.TH = t.TH; p.NRB = t.NRB; p.RBH = t.RBH;
  p.inv_NRB = magic_of(p.NRB);
  p.NST = t.NST;
  p.DYOFF = t.DYOFF;
  f.U = t.U;
  f.exact = t.exact;
  const long long tpc = (long long)s.N * p.NRT;
  if (tpc > (1ll << 30)) return false;
  p.TPC = (int)tpc;
  p.NCG = ceil_div(s.C, p.G);
  // One equal work item per resident CTA when the channel groups divide the CTA slots well
  // (no tail, fewest reductions); otherwise about two items per slot.  At least one tile each.
  const int slots = sm_count() * filter_minb(K);
  int SL = slots / p.NCG;
  if (SL < 1 || (long long)SL * p.NCG * 100 < 85ll * slots) SL = ceil_div(2 * slots, p.NCG);
  if (SL > p.TPC) SL = p.TPC;
  if (SL < 1) SL = 1;
  p.SL = SL;
  // halo reach in lanes (column geometry does not depend on U)
  const int cmin = geo_min_rel(K, S, MODE_FWD, f.VO), cmax = geo_max_rel(K, S, MODE_FWD, f.VO);
  const int hl = -geo_fdiv(cmin, f.VI), hr = geo_fdiv(cmax, f.VI);
  f.mask = (p.LW - lanes_in) < (hl > hr ? hl : hr);
  return true;
}

template <typename T>
bool plan_filter(const Shape &s, bool a16, FilterPlan &f) {
  if (!filter_shape_ok(s)) return false;
  switch (s.kh * 10 + s.sh) {
    case 31: return plan_filter_ks<T, 3, 1>(s, a16, f);
    case 51: return plan_filter_ks<T, 5, 1>(s, a16, f);
    case 71: return plan_filter_ks<T, 7, 1>(s, a16, f);
    case 32: return plan_filter_ks<T, 3, 2>(s, a16, f);
    case 52: return plan_filter_ks<T, 5, 2>(s, a16, f);
    case 72: return plan_filter_ks<T, 7, 2>(s, a16, f);
    default: return false;
  }
}

int *filter_flag_address() {
  static std::atomic<int *> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  int *p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress((void **)&p, g_filter_error_flag) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    cached[dev].store(p, std::memory_order_release);
  }
  return p;
}

template <typename T, int K, int S, int VI, int VO, int U, bool MASK, bool EXACT>
int launch_variant(const RowsFilterParams &p, cudaStream_t st) {
  constexpr int MINB = filter_minb(K);
  auto kernel = rows_filter_kernel<T, K, S, VI, VO, U, MASK, EXACT, MINB>;
  static std::atomic<unsigned long long> smem_done{0};
  if (!ensure_smem(kernel, ROWS_SMEM_BYTES, smem_done)) return ROWS_DECLINED;
  int *flag = filter_flag_address();
  if (flag == nullptr) return ROWS_DECLINED;
  const long long items = (long long)p.NCG * p.SL;
  const int grid = (int)min((long long)sm_count() * MINB, items);
  launch_dependent(kernel, grid, ROWS_THREADS, ROWS_SMEM_BYTES, st, p, flag);
  return ROWS_SERVED;
}

template <typename T, int K, int S, int VI, int VO, int I>
int launch_filter_u(const FilterPlan &f, cudaStream_t st) {
  constexpr int UI = FilterU<K, S>::v[I];
  constexpr int N = filter_u_count<K, S>(VI);
  if (f.U == UI || I + 1 >= N) {
    if (f.mask)
      return f.exact ? launch_variant<T, K, S, VI, VO, UI, true, true>(f.p, st)
                     : launch_variant<T, K, S, VI, VO, UI, true, false>(f.p, st);
    return f.exact ? launch_variant<T, K, S, VI, VO, UI, false, true>(f.p, st)
                   : launch_variant<T, K, S, VI, VO, UI, false, false>(f.p, st);
  }
  if constexpr (I + 1 < N)
    return launch_filter_u<T, K, S, VI, VO, I + 1>(f, st);
  else
    return ROWS_DECLINED;
}
template <typename T, int K, int S, int VI, int VO>
int launch_filter_v(const FilterPlan &f, cudaStream_t st) {
  return launch_filter_u<T, K, S, VI, VO, 0>(f, st);
}

template <typename T, int K, int S>
int launch_filter(const FilterPlan &f, cudaStream_t st) {
  if (S == 1) {
    if (f.VI == 4) return launch_filter_v<T, K, 1, 4, 4>(f, st);
    if (f.VI == 2) return launch_filter_v<T, K, 1, 2, 2>(f, st);
    return launch_filter_v<T, K, 1, 1, 1>(f, st);
  }
  if (f.VI == 4) return launch_filter_v<T, K, 2, 4, 2>(f, st);
  return launch_filter_v<T, K, 2, 2, 1>(f, st);
}

template <typename T> struct RowsDtype { static constexpr bool ok = false; };
template <> struct RowsDtype<float> { static constexpr bool ok = true; };
template <> struct RowsDtype<__half> { static constexpr bool ok = true; };
template <> struct RowsDtype<__nv_bfloat16> { static constexpr bool ok = true; };

}  // namespace

template <typename T> int rows_backward_filter_slices(const Shape &s) {
  if constexpr (!RowsDtype<T>::ok) {
    return 0;
  } else {
    // alignment is not known here: report the largest slice count either choice would use
    if (s.kh > 7) return rows_bigk_filter_slices<T>(s);
    FilterPlan f{};
    int best = 0;
    for (int a16 = 0; a16 < 2; ++a16)
      if (plan_filter<T>(s, a16 != 0, f) && f.p.SL > best) best = f.p.SL;
    return best;
  }
}

template <typename T>
int rows_backward_filter(const T *x, const T *dy, typename Elem<T>::acc_t *partial, const Shape &s,
                         cudaStream_t st, int *slices_out) {
  if constexpr (!RowsDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    if (s.kh > 7) return rows_bigk_filter<T>(x, dy, partial, s, st, slices_out);
    const bool a16 = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy)) & 15) == 0;
    FilterPlan f{};
    if (!plan_filter<T>(s, a16, f)) return ROWS_DECLINED;
    f.p.x = x; f.p.dy = dy; f.p.partial = partial;
    *slices_out = f.p.SL;
    switch (s.kh * 10 + s.sh) {
      case 31: return launch_filter<T, 3, 1>(f, st);
      case 51: return launch_filter<T, 5, 1>(f, st);
      case 71: return launch_filter<T, 7, 1>(f, st);
      case 32: return launch_filter<T, 3, 2>(f, st);
      case 52: return launch_filter<T, 5, 2>(f, st);
      case 72: return launch_filter<T, 7, 2>(f, st);
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

int rows_take_device_error() {
  return rows_conv_take_error() | rows_filter_take_error() | rows_backward_take_error();
}

template int rows_backward_filter_slices<float>(const Shape &);
template int rows_backward_filter_slices<__half>(const Shape &);
template int rows_backward_filter_slices<__nv_bfloat16>(const Shape &);
template int rows_backward_filter_slices<double>(const Shape &);
template int rows_backward_filter<float>(const float *, const float *, float *, const Shape &, cudaStream_t, int *);
template int rows_backward_filter<__half>(const __half *, const __half *, float *, const Shape &, cudaStream_t, int *);
template int rows_backward_filter<__nv_bfloat16>(const __nv_bfloat16 *, const __nv_bfloat16 *, float *, const Shape &, cudaStream_t, int *);
template int rows_backward_filter<double>(const double *, const double *, double *, const Shape &, cudaStream_t, int *);

// Tiling the backward-filter first pass would use, for inspection: the test-suite models the
// kernel's index arithmetic on the CPU from these numbers.
int rows_debug_filter_plan(int esize, const Shape &s, int a16, int *out) {
  FilterPlan f{};
  bool ok = esize == 4 ? plan_filter<float>(s, a16 != 0, f) : plan_filter<__half>(s, a16 != 0, f);
  if (!ok) return 0;
  const RowsFilterParams &p = f.p;
  const int v[24] = {f.VI, f.VO, f.U, f.mask ? 1 : 0, p.LW, p.G, p.NRT, p.TH, p.NRB, p.RBH, p.NST,
                     f.exact ? 1 : 0, 0, 0, 0, p.DYOFF, p.TPC, p.SL, 0, p.NCG, 0, 0, 0, 0};
  for (int i = 0; i < 24; ++i) out[i] = v[i];
  return 1;
}

}  // namespace dwb
