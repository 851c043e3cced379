// Rows family, fused backward (dx and the partial sums of dW in one pass over dy): variant
// selection and launch.
#include "lanerow_backward.cuh"
#include "rows_backward.cuh"
#include "rows_plan.cuh"

namespace dwb {

namespace {

__device__ int g_backward_error_flag;

// The cluster form of the second pass needs one CTA per work item, all resident at once, and a
// cluster of at most 8 CTAs (the portable limit).
inline bool direct_possible(long long items, int slots, int SL) {
  return items <= slots && SL >= 1 && SL <= 8 && tuning_int("CLUSTER", 1) != 0;
}

// One CTA per SM where the taps plus the gradient accumulators (2 * K * K registers) leave no
// room for two.
constexpr int backward_minb(int K) { return K <= 3 ? 2 : 1; }

// Rows-per-chunk choices compiled for each (K, S); the planner picks per shape.
template <int K, int S> struct BackwardU;
template <> struct BackwardU<3, 1> { static constexpr int n = 2; static constexpr int v[4] = {4, 7, 7, 7}; };
template <> struct BackwardU<5, 1> { static constexpr int n = 2; static constexpr int v[4] = {2, 4, 4, 4}; };
template <> struct BackwardU<7, 1> { static constexpr int n = 1; static constexpr int v[4] = {2, 2, 2, 2}; };
template <> struct BackwardU<3, 2> { static constexpr int n = 2; static constexpr int v[4] = {4, 8, 8, 8}; };
template <> struct BackwardU<5, 2> { static constexpr int n = 1; static constexpr int v[4] = {4, 4, 4, 4}; };
template <> struct BackwardU<7, 2> { static constexpr int n = 1; static constexpr int v[4] = {2, 2, 2, 2}; };

constexpr int backward_u_cap(int K, int S, int VO) {
  return (VO == 4 && K == 3 && S == 1) ? 4 : (1 << 20);
}
template <int K, int S> constexpr int backward_u_count(int VO) {
  int n = 0;
  for (int i = 0; i < BackwardU<K, S>::n; ++i)
    if (BackwardU<K, S>::v[i] <= backward_u_cap(K, S, VO)) ++n;
  return n;
}

inline bool backward_shape_ok(const Shape &s) {
  if (s.kh != s.kw || (s.kh != 3 && s.kh != 5 && s.kh != 7)) return false;
  if (s.sh != s.sw || (s.sh != 1 && s.sh != 2)) return false;
  if (s.ph != s.kh / 2 || s.pw != s.kw / 2) return false;
  if (s.Ho != (s.H + 2 * s.ph - s.kh) / s.sh + 1 || s.Wo != (s.W + 2 * s.pw - s.kw) / s.sw + 1)
    return false;
  return true;
}

// (VI, VO) = dy / dx columns per lane for the map widths; false if none applies.
// a16: x, dy and dx are all 16-byte aligned.
inline bool pick_v(int S, int W, int Wo, bool a16, int &VI, int &VO) {
  if (S == 1) {
    if (a16 && W % 4 == 0 && W <= 128 && W > 16) { VI = VO = 4; return true; }
    if (a16 && W % 2 == 0 && W <= 64 && W > 8) { VI = VO = 2; return true; }
    if (W <= 32) { VI = VO = 1; return true; }
    return false;
  }
  if (a16 && Wo % 2 == 0 && W % 4 == 0 && Wo <= 64 && W <= 128 && W > 16) { VI = 2; VO = 4; return true; }
  if (a16 && W % 2 == 0 && Wo <= 32 && W <= 64) { VI = 1; VO = 2; return true; }
  return false;
}

struct BackwardPlan {
  RowsBackwardParams p;
  int VI, VO, U;
  bool mask, exact;
};

template <typename T, int K, int S>
bool plan_backward_ks(const Shape &s, bool a16, BackwardPlan &f) {
  constexpr int MODE = (S == 1) ? MODE_FWD : MODE_BWD;
  if (!pick_v(S, s.W, s.Wo, a16, f.VI, f.VO)) return false;
  // Where the one-CTA-per-SM fused kernel measured slower than the two operators run one after
  // the other (32x32 maps, four columns per lane: 5x5 fp32 65 against 51 us, 7x7 fp32 108
  // against 104 us), the caller falls back to them.
  if (S == 1 && f.VO == 4 && (K == 5 || (K == 7 && sizeof(T) == 4))) return false;
  const int lanes_in = ceil_div(s.Wo, f.VI);
  const int lanes = max(lanes_in, ceil_div(s.W, f.VO));
  RowsBackwardParams &p = f.p;
  p.LW = pick_lw(lanes);
  if (p.LW == 0) return false;
  // the window source ("in") is dy, the rows the tasks walk ("out") are those of x / dx
  PlanInput in{K, S, MODE, s.Ho, s.Wo, s.H, s.W, (int)sizeof(T),
               ROWS_CWARPS * (32 / p.LW), s.C, 0, 0, true};
  const TilePlan t = plan_best(in, BackwardU<K, S>::v, backward_u_count<K, S>(f.VO));
  if (!t.ok) return false;
  p.N = s.N; p.C = s.C; p.H = s.H; p.W = s.W; p.Ho = s.Ho; p.Wo = s.Wo;
  p.G = t.G; p.NRT = t.NRT; p.TH = t.TH; p.NRB = t.NRB; p.RBH = t.RBH;
  p.inv_NRB = magic_of(p.NRB);
  p.NST = t.NST;
  p.XOFF = t.DYOFF;
  f.U = t.U;
  f.exact = t.exact;
  const long long tpc = (long long)s.N * p.NRT;
  if (tpc > (1ll << 30)) return false;
  p.TPC = (int)tpc;
  p.NCG = ceil_div(s.C, p.G);
  // One equal work item per resident CTA when the channel groups divide the CTA slots well;
  // otherwise about two items per slot.  At least one tile each.
  const int slots = sm_count() * backward_minb(K);
  int SL = slots / p.NCG;
  if (SL < 1 || (long long)SL * p.NCG * 100 < 85ll * slots) SL = ceil_div(2 * slots, p.NCG);
  if (SL > p.TPC) SL = p.TPC;
  if (SL < 1) SL = 1;
  p.SL = SL;
  const int cmin = geo_min_rel(K, S, MODE, f.VO), cmax = geo_max_rel(K, S, MODE, f.VO);
  const int hl = -geo_fdiv(cmin, f.VI), hr = geo_fdiv(cmax, f.VI);
  f.mask = (p.LW - lanes_in) < (hl > hr ? hl : hr);
  return true;
}

template <typename T>
bool plan_backward(const Shape &s, bool a16, BackwardPlan &f) {
  if (!backward_shape_ok(s)) return false;
  switch (s.kh * 10 + s.sh) {
    case 31: return plan_backward_ks<T, 3, 1>(s, a16, f);
    case 51: return plan_backward_ks<T, 5, 1>(s, a16, f);
    case 71: return plan_backward_ks<T, 7, 1>(s, a16, f);
    case 32: return plan_backward_ks<T, 3, 2>(s, a16, f);
    case 52: return plan_backward_ks<T, 5, 2>(s, a16, f);
    case 72: return plan_backward_ks<T, 7, 2>(s, a16, f);
    default: return false;
  }
}

int *backward_flag_address() {
  static std::atomic<int *> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  int *p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress((void **)&p, g_backward_error_flag) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    cached[dev].store(p, std::memory_order_release);
  }
  return p;
}

template <typename T, int K, int S, int VI, int VO, int U, bool MASK, bool EXACT>
int launch_variant(const RowsBackwardParams &p, cudaStream_t st) {
  constexpr int MINB = backward_minb(K);
  constexpr int MODE = (S == 1) ? MODE_FWD : MODE_BWD;
  auto kernel = rows_backward_kernel<T, K, S, MODE, VI, VO, U, MASK, EXACT, MINB>;
  static std::atomic<unsigned long long> smem_done{0};
  if (!ensure_smem(kernel, ROWS_SMEM_BYTES, smem_done)) return ROWS_DECLINED;
  int *flag = backward_flag_address();
  if (flag == nullptr) return ROWS_DECLINED;
  const long long items = (long long)p.NCG * p.SL;
  const int grid = (int)min((long long)sm_count() * MINB, items);
  if (p.dw_direct != nullptr) {
    // every item has its own CTA: the SL CTAs of a channel group form a cluster that finishes dW
    static ClusterLimits cluster_ok;
    if (direct_possible(items, sm_count() * MINB, p.SL) &&
        launch_dependent_cluster(kernel, grid, ROWS_THREADS, ROWS_SMEM_BYTES, st, p.SL, cluster_ok, p, flag))
      return ROWS_SERVED_DW;
    RowsBackwardParams q = p;
    q.dw_direct = nullptr;
    launch_dependent(kernel, grid, ROWS_THREADS, ROWS_SMEM_BYTES, st, q, flag);
    return ROWS_SERVED;
  }
  launch_dependent(kernel, grid, ROWS_THREADS, ROWS_SMEM_BYTES, st, p, flag);
  return ROWS_SERVED;
}

template <typename T, int K, int S, int VI, int VO, int I>
int launch_backward_u(const BackwardPlan &f, cudaStream_t st) {
  constexpr int UI = BackwardU<K, S>::v[I];
  constexpr int N = backward_u_count<K, S>(VO);
  if (f.U == UI || I + 1 >= N) {
    if (f.mask)
      return f.exact ? launch_variant<T, K, S, VI, VO, UI, true, true>(f.p, st)
                     : launch_variant<T, K, S, VI, VO, UI, true, false>(f.p, st);
    return f.exact ? launch_variant<T, K, S, VI, VO, UI, false, true>(f.p, st)
                   : launch_variant<T, K, S, VI, VO, UI, false, false>(f.p, st);
  }
  if constexpr (I + 1 < N)
    return launch_backward_u<T, K, S, VI, VO, I + 1>(f, st);
  else
    return ROWS_DECLINED;
}

template <typename T, int K, int S>
int launch_backward(const BackwardPlan &f, cudaStream_t st) {
  if (S == 1) {
    // (the variants the planner never picks, see plan_backward_ks, are not compiled)
    if constexpr (!(K == 5 || (K == 7 && sizeof(T) == 4))) {
      if (f.VI == 4) return launch_backward_u<T, K, 1, 4, 4, 0>(f, st);
    }
    if (f.VI == 2) return launch_backward_u<T, K, 1, 2, 2, 0>(f, st);
    return launch_backward_u<T, K, 1, 1, 1, 0>(f, st);
  }
  if (f.VI == 2) return launch_backward_u<T, K, 2, 2, 4, 0>(f, st);
  return launch_backward_u<T, K, 2, 1, 2, 0>(f, st);
}

template <typename T> struct RowsDtype { static constexpr bool ok = false; };
template <> struct RowsDtype<float> { static constexpr bool ok = true; };
template <> struct RowsDtype<__half> { static constexpr bool ok = true; };
template <> struct RowsDtype<__nv_bfloat16> { static constexpr bool ok = true; };

// ---- small maps: a lane owns a row (lanerow_backward.cuh) ----
// Stride 1, padding k/2, maps 7, 14 or 28 columns wide and at most 32 rows high; fp32 and fp16.
// One CTA per SM where 3 * W row registers plus 2 * K * K taps and sums do not leave room for two.
constexpr bool lanerow_compiled(int K, int W) {
  return (K == 3 || K == 5 || K == 7) && (W == 7 || W == 14 || W == 28) && !(K == 7 && W == 7);
}
constexpr int lanerow_minb(int K, int W) { return (3 * W + 2 * K * K + 24 <= 128) ? 2 : 1; }

inline bool lanerow_shape_ok(const Shape &s) {
  return s.kh == s.kw && s.sh == 1 && s.sw == 1 && s.ph == s.kh / 2 && s.pw == s.kw / 2 &&
         lanerow_compiled(s.kh, s.W) && s.H <= 32 && s.Ho == s.H && s.Wo == s.W;
}

// Where the column-per-lane kernel measured faster: 3x3 fp32 on 28-column maps (four columns per
// lane there: 43.9 against 49.5 us on N128 C192 28x28).
inline bool lanerow_not_worth_it(const Shape &s, int esize) { return s.kh == 3 && s.W == 28 && esize == 4; }

inline bool plan_lanerow(const Shape &s, int esize, LaneRowParams &p) {
  if (!lanerow_shape_ok(s)) return false;
  const int lanes = ROWS_CWARPS * 32;
  int G = lanes / s.H;
  if (G > s.C) G = s.C;
  if (G < 1) return false;
  const int plane_bytes = s.H * s.W * esize;
  auto region = [&](int g) { return round_up(g * plane_bytes + 16, 16); };
  auto stage_need = [&](int g) { return LANEROW_ZERO_BYTES + 3 * region(g); };
  while (G > 1 && stage_need(G) > ROWS_RING_BYTES / 2) --G;
  if (stage_need(G) > ROWS_RING_BYTES / 2) return false;
  p.NST = stage_need(G) <= ROWS_RING_BYTES / 3 ? 3 : 2;
  p.N = s.N; p.C = s.C; p.H = s.H; p.G = G;
  p.DYOFF = LANEROW_ZERO_BYTES;
  p.XOFF = p.DYOFF + region(G);
  p.OUTOFF = p.XOFF + region(G);
  p.NCG = ceil_div(s.C, G);
  const int slots = sm_count() * lanerow_minb(s.kh, s.W);
  int SL = slots / p.NCG;
  if (SL < 1 || (long long)SL * p.NCG * 100 < 85ll * slots) SL = ceil_div(2 * slots, p.NCG);
  if (SL > s.N) SL = s.N;
  if (SL < 1) SL = 1;
  p.SL = SL;
  return true;
}

template <typename T, int K, int W>
int launch_lanerow(const LaneRowParams &p, cudaStream_t st) {
  if constexpr (!lanerow_compiled(K, W)) {
    return ROWS_DECLINED;
  } else {
    constexpr int MINB = lanerow_minb(K, W);
    auto kernel = lanerow_backward_kernel<T, K, W, MINB>;
    static std::atomic<unsigned long long> smem_done{0};
    if (!ensure_smem(kernel, ROWS_SMEM_BYTES, smem_done)) return ROWS_DECLINED;
    int *flag = backward_flag_address();
    if (flag == nullptr) return ROWS_DECLINED;
    const long long items = (long long)p.NCG * p.SL;
    const int grid = (int)min((long long)sm_count() * MINB, items);
    if (p.dw_direct != nullptr) {
      static ClusterLimits cluster_ok;
      if (direct_possible(items, sm_count() * MINB, p.SL) &&
          launch_dependent_cluster(kernel, grid, ROWS_THREADS, ROWS_SMEM_BYTES, st, p.SL, cluster_ok, p, flag))
        return ROWS_SERVED_DW;
      LaneRowParams q = p;
      q.dw_direct = nullptr;
      launch_dependent(kernel, grid, ROWS_THREADS, ROWS_SMEM_BYTES, st, q, flag);
      return ROWS_SERVED;
    }
    launch_dependent(kernel, grid, ROWS_THREADS, ROWS_SMEM_BYTES, st, p, flag);
    return ROWS_SERVED;
  }
}

template <typename T, int K>
int launch_lanerow_w(const LaneRowParams &p, int W, cudaStream_t st) {
  switch (W) {
    case 7: return launch_lanerow<T, K, 7>(p, st);
    case 14: return launch_lanerow<T, K, 14>(p, st);
    case 28: return launch_lanerow<T, K, 28>(p, st);
    default: return ROWS_DECLINED;
  }
}

}  // namespace

template <typename T> int rows_backward_slices(const Shape &s) {
  if constexpr (!RowsDtype<T>::ok) {
    return 0;
  } else {
    // alignment is not known here: report the largest slice count either choice would use
    BackwardPlan f{};
    int best = 0;
    for (int a16 = 0; a16 < 2; ++a16)
      if (plan_backward<T>(s, a16 != 0, f) && f.p.SL > best) best = f.p.SL;
    LaneRowParams lp{};
    if (plan_lanerow(s, (int)sizeof(T), lp) && lp.SL > best) best = lp.SL;
    return best;
  }
}

template <typename T>
int rows_backward(const T *x, const T *dy, const T *w, T *dx, typename Elem<T>::acc_t *partial,
                  const Shape &s, cudaStream_t st, int *slices_out, T *dw_direct) {
  if constexpr (!RowsDtype<T>::ok) {
    return ROWS_DECLINED;
  } else {
    const bool a16 = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) |
                       reinterpret_cast<uintptr_t>(dx)) & 15) == 0;
    {
      LaneRowParams lp{};
      const int mode = tuning_int("LANEROW", 1);
      if (a16 && mode != 0 && (mode == 2 || !lanerow_not_worth_it(s, (int)sizeof(T))) &&
          plan_lanerow(s, (int)sizeof(T), lp)) {
        lp.x = x; lp.dy = dy; lp.w = w; lp.dx = dx; lp.partial = partial;
        lp.dw_direct = dw_direct;
        *slices_out = lp.SL;
        int r = ROWS_DECLINED;
        switch (s.kh) {
          case 3: r = launch_lanerow_w<T, 3>(lp, s.W, st); break;
          case 5: r = launch_lanerow_w<T, 5>(lp, s.W, st); break;
          case 7: r = launch_lanerow_w<T, 7>(lp, s.W, st); break;
          default: break;
        }
        if (r != ROWS_DECLINED) return r;
      }
    }
    BackwardPlan f{};
    if (!plan_backward<T>(s, a16, f)) return ROWS_DECLINED;
    f.p.x = x; f.p.dy = dy; f.p.w = w; f.p.dx = dx; f.p.partial = partial;
    f.p.dw_direct = dw_direct;
    *slices_out = f.p.SL;
    switch (s.kh * 10 + s.sh) {
      case 31: return launch_backward<T, 3, 1>(f, st);
      case 51: return launch_backward<T, 5, 1>(f, st);
      case 71: return launch_backward<T, 7, 1>(f, st);
      case 32: return launch_backward<T, 3, 2>(f, st);
      case 52: return launch_backward<T, 5, 2>(f, st);
      case 72: return launch_backward<T, 7, 2>(f, st);
      default: return ROWS_DECLINED;
    }
  }
}

int rows_backward_take_error() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_backward_error_flag, sizeof(int)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (v) {
    const int zero = 0;
    (void)cudaMemcpyToSymbol(g_backward_error_flag, &zero, sizeof(int));
  }
  return v;
}

template int rows_backward_slices<float>(const Shape &);
template int rows_backward_slices<__half>(const Shape &);
template int rows_backward_slices<__nv_bfloat16>(const Shape &);
template int rows_backward_slices<double>(const Shape &);
template int rows_backward<float>(const float *, const float *, const float *, float *, float *, const Shape &, cudaStream_t, int *, float *);
template int rows_backward<__half>(const __half *, const __half *, const __half *, __half *, float *, const Shape &, cudaStream_t, int *, __half *);
template int rows_backward<__nv_bfloat16>(const __nv_bfloat16 *, const __nv_bfloat16 *, const __nv_bfloat16 *, __nv_bfloat16 *, float *, const Shape &, cudaStream_t, int *, __nv_bfloat16 *);
template int rows_backward<double>(const double *, const double *, const double *, double *, double *, const Shape &, cudaStream_t, int *, double *);

// Tiling the fused backward pass would use, for inspection (same layout as the other plans).
int rows_debug_backward_plan(int esize, const Shape &s, int a16, int *out) {
  LaneRowParams lp{};
  if (a16 && plan_lanerow(s, esize, lp) && !lanerow_not_worth_it(s, esize)) {
    // the lane-per-row kernel: W columns per lane, one row each
    const int v[24] = {s.W, s.W, 1, 0, 1, lp.G, 1, s.H, s.H, 1, lp.NST, 1, 0, 0, 0, lp.XOFF, s.N, lp.SL, 0,
                       lp.NCG, 2 /* lane per row */, 0, 0, 0};
    for (int i = 0; i < 24; ++i) out[i] = v[i];
    return 1;
  }
  BackwardPlan f{};
  bool ok = esize == 4 ? plan_backward<float>(s, a16 != 0, f) : plan_backward<__half>(s, a16 != 0, f);
  if (!ok) return 0;
  const RowsBackwardParams &p = f.p;
  const int v[24] = {f.VI, f.VO, f.U, f.mask ? 1 : 0, p.LW, p.G, p.NRT, p.TH, p.NRB, p.RBH, p.NST,
                     f.exact ? 1 : 0, 0, 0, 0, p.XOFF, p.TPC, p.SL, 0, p.NCG, 0, 0, 0, 0};
  for (int i = 0; i < 24; ++i) out[i] = v[i];
  return 1;
}

}  // namespace dwb
