// Rows family, forward and backward-input: variant selection and launch templates, shared by
// the translation units that instantiate them (rows_conv.cu: the plain operators;
// rows_conv_epi.cu: the forward with a fused epilogue).  Everything here has internal linkage:
// each translation unit has its own error flag and its own once-only kernel set-up.
#pragma once

#include "lanerow_conv.cuh"
#include "rows_plan.cuh"

namespace dwb {

namespace {

__device__ int g_conv_error_flag;

// When set (rows_debug_conv_plan), the selected variant and tiling are written here and
// nothing is launched.
thread_local int *t_plan_out = nullptr;

template <typename T> struct RowsDtype { static constexpr bool ok = false; };
template <> struct RowsDtype<float> { static constexpr bool ok = true; };
template <> struct RowsDtype<__half> { static constexpr bool ok = true; };
template <> struct RowsDtype<__nv_bfloat16> { static constexpr bool ok = true; };

constexpr int conv_minb(int K) { return K <= 5 ? 2 : 1; }  // 49 tap registers: one CTA per SM

// Rows-per-chunk choices compiled for each (K, S, MODE); the planner picks per shape.
template <int K, int S, int MODE> struct ConvU;
template <> struct ConvU<3, 1, MODE_FWD> { static constexpr int n = 3; static constexpr int v[4] = {4, 7, 8, 8}; };  // 14 measured slower than 7 on 14-row maps
template <> struct ConvU<5, 1, MODE_FWD> { static constexpr int n = 2; static constexpr int v[4] = {4, 7, 7, 7}; };
template <> struct ConvU<7, 1, MODE_FWD> { static constexpr int n = 1; static constexpr int v[4] = {2, 2, 2, 2}; };  // 4 measured the same (no spill, 33.1 vs 32.7 us on 32x32 maps)
template <> struct ConvU<3, 2, MODE_FWD> { static constexpr int n = 3; static constexpr int v[4] = {2, 4, 7, 7}; };
template <> struct ConvU<5, 2, MODE_FWD> { static constexpr int n = 1; static constexpr int v[4] = {2, 2, 2, 2}; };  // 4 measured slower (and spills at VI = 4)
template <> struct ConvU<7, 2, MODE_FWD> { static constexpr int n = 1; static constexpr int v[4] = {2, 2, 2, 2}; };
template <> struct ConvU<3, 2, MODE_BWD> { static constexpr int n = 3; static constexpr int v[4] = {4, 8, 14, 14}; };
template <> struct ConvU<5, 2, MODE_BWD> { static constexpr int n = 2; static constexpr int v[4] = {4, 14, 14, 14}; };
template <> struct ConvU<7, 2, MODE_BWD> { static constexpr int n = 2; static constexpr int v[4] = {2, 4, 4, 4}; };

// Options above this height spill registers for the given vector width (ptxas -v) and measured
// slower; the tables are ascending, so a cap keeps a prefix.
constexpr int conv_u_cap(int K, int S, int mode, int VI) {
  if (VI == 4 && K == 3 && S == 1) return 8;
  if (VI == 4 && K == 5 && S == 1) return 4;
  return 1 << 20;
}
template <int K, int S, int MODE, int VI> constexpr int conv_u_count() {
  int n = 0;
  for (int i = 0; i < ConvU<K, S, MODE>::n; ++i)
    if (ConvU<K, S, MODE>::v[i] <= conv_u_cap(K, S, MODE, VI)) ++n;
  return n;
}

int *conv_flag_address() {
  static std::atomic<int *> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  int *p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress((void **)&p, g_conv_error_flag) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    cached[dev].store(p, std::memory_order_release);
  }
  return p;
}

template <typename T, int K, int S, int MODE, int VI, int VO, int U, bool MASK, bool EXACT, bool EPI>
int launch_variant(const RowsParams &p, cudaStream_t st) {
  constexpr int MINB = conv_minb(K);
  auto kernel = rows_conv_kernel<T, K, S, MODE, VI, VO, U, MASK, EXACT, MINB, EPI>;
  static std::atomic<unsigned long long> smem_done{0};
  if (!ensure_smem(kernel, ROWS_SMEM_BYTES, smem_done)) return ROWS_DECLINED;
  int *flag = conv_flag_address();
  if (flag == nullptr) return ROWS_DECLINED;
  const int grid = (int)min((long long)sm_count() * MINB, (long long)p.ntiles);
  launch_dependent(kernel, grid, ROWS_THREADS, ROWS_SMEM_BYTES, st, p, flag);
  return ROWS_SERVED;
}

// Dispatch on the planner's runtime choices (U among the compiled options, mask, exact).
template <typename T, int K, int S, int MODE, int VI, int VO, bool EPI, int I>
int launch_u(const RowsParams &p, int U, bool mask, bool exact, cudaStream_t st) {
  constexpr int UI = ConvU<K, S, MODE>::v[I];
  constexpr int N = conv_u_count<K, S, MODE, VI>();
  if (U == UI || I + 1 >= N) {
    if (mask)
      return exact ? launch_variant<T, K, S, MODE, VI, VO, UI, true, true, EPI>(p, st)
                   : launch_variant<T, K, S, MODE, VI, VO, UI, true, false, EPI>(p, st);
    return exact ? launch_variant<T, K, S, MODE, VI, VO, UI, false, true, EPI>(p, st)
                 : launch_variant<T, K, S, MODE, VI, VO, UI, false, false, EPI>(p, st);
  }
  if constexpr (I + 1 < N)
    return launch_u<T, K, S, MODE, VI, VO, EPI, I + 1>(p, U, mask, exact, st);
  else
    return ROWS_DECLINED;
}

template <typename T, int K, int S, int MODE, int VI, int VO, bool EPI>
int launch_conv(RowsParams p, cudaStream_t st) {
  using Geo = RowsGeo<K, S, MODE, VI, VO, ConvU<K, S, MODE>::v[0]>;  // column geometry: U-independent
  const int lanes_in = ceil_div(p.Win, VI);
  const int lanes = max(lanes_in, ceil_div(p.Wout, VO));
  p.LW = pick_lw(lanes);
  if (p.LW == 0) return ROWS_DECLINED;
  PlanInput in{K, S, MODE, p.Hin, p.Win, p.Hout, p.Wout, (int)sizeof(T),
               ROWS_CWARPS * (32 / p.LW), p.NC, 0, sm_count() * conv_minb(K), false};
  const TilePlan t = plan_best(in, ConvU<K, S, MODE>::v, conv_u_count<K, S, MODE, VI>());
  if (!t.ok) return ROWS_DECLINED;
  p.G = t.G; p.NRT = t.NRT; p.TH = t.TH; p.NRB = t.NRB; p.RBH = t.RBH;
  p.inv_NRB = magic_of(p.NRB);
  p.NST = t.NST;
  p.TAPB = t.TAPB;
  const long long ntiles = (long long)ceil_div(p.NC, p.G) * p.NRT;
  if (ntiles > (1ll << 30)) return ROWS_DECLINED;
  p.ntiles = (int)ntiles;
  // halo columns reach this many lanes to either side; spare (zero) lanes at the end of each
  // segment make explicit masking unnecessary
  constexpr int halo_lanes = (-Geo::fdiv(Geo::CMIN, VI) > Geo::fdiv(Geo::CMAX, VI))
                                 ? -Geo::fdiv(Geo::CMIN, VI)
                                 : Geo::fdiv(Geo::CMAX, VI);
  const bool mask = (p.LW - lanes_in) < halo_lanes;
  if (t_plan_out != nullptr) {
    const int v[24] = {VI, VO, t.U, mask ? 1 : 0, p.LW, p.G, p.NRT, p.TH, p.NRB, p.RBH, p.NST,
                       t.exact ? 1 : 0, 0, p.TAPB, 0, 0, p.ntiles, 0, MODE, 0, 0, 0, 0, 0};
    for (int i = 0; i < 24; ++i) t_plan_out[i] = v[i];
    return ROWS_SERVED;
  }
  return launch_u<T, K, S, MODE, VI, VO, EPI, 0>(p, t.U, mask, t.exact, st);
}

// Picks the widest per-lane vector the widths and pointers allow.
template <typename T, int K, int S, int MODE, bool EPI>
int select_conv(const RowsParams &p, cudaStream_t st) {
  const bool a16 = ((reinterpret_cast<uintptr_t>(p.in) | reinterpret_cast<uintptr_t>(p.out)) & 15) == 0;
  if (S == 1) {
    if (a16 && p.Win % 4 == 0 && p.Wout % 4 == 0 && p.Win <= 128 && p.Wout <= 128 && p.Win > 16)
      return launch_conv<T, K, 1, MODE_FWD, 4, 4, EPI>(p, st);
    if (a16 && p.Win % 2 == 0 && p.Wout % 2 == 0 && p.Win <= 64 && p.Wout <= 64 && p.Win > 8)
      return launch_conv<T, K, 1, MODE_FWD, 2, 2, EPI>(p, st);
    if (p.Win <= 32 && p.Wout <= 32) return launch_conv<T, K, 1, MODE_FWD, 1, 1, EPI>(p, st);
    return ROWS_DECLINED;
  }
  if (MODE == MODE_FWD) {
    if (a16 && p.Win % 4 == 0 && p.Wout % 2 == 0 && p.Win <= 128 && p.Wout <= 64 && p.Win > 16)
      return launch_conv<T, K, 2, MODE_FWD, 4, 2, EPI>(p, st);
    if (a16 && p.Win % 2 == 0 && p.Win <= 64 && p.Wout <= 32)
      return launch_conv<T, K, 2, MODE_FWD, 2, 1, EPI>(p, st);
    return ROWS_DECLINED;
  }
  if (a16 && p.Win % 2 == 0 && p.Wout % 4 == 0 && p.Win <= 64 && p.Wout <= 128 && p.Wout > 16)
    return launch_conv<T, K, 2, MODE_BWD, 2, 4, EPI>(p, st);
  if (a16 && p.Wout % 2 == 0 && p.Win <= 32 && p.Wout <= 64)
    return launch_conv<T, K, 2, MODE_BWD, 1, 2, EPI>(p, st);
  return ROWS_DECLINED;
}

// ---- small maps, stride 1: a lane owns a row (lanerow_conv.cuh) ----
constexpr bool lanerow_conv_compiled(int K, int W) {
  return (K == 3 || K == 5 || K == 7) && (W == 7 || W == 14 || W == 28) && !(K == 7 && W == 7);
}
constexpr int lanerow_conv_minb(int K, int W) { return (2 * W + K * K + 20 <= 128) ? 2 : 1; }

template <typename T, int K, int W>
int launch_lanerow_conv(const LaneRowConvParams &p, cudaStream_t st) {
  if constexpr (!lanerow_conv_compiled(K, W)) {
    return ROWS_DECLINED;
  } else {
    constexpr int MINB = lanerow_conv_minb(K, W);
    auto kernel = lanerow_conv_kernel<T, K, W, MINB>;
    static std::atomic<unsigned long long> smem_done{0};
    if (!ensure_smem(kernel, ROWS_SMEM_BYTES, smem_done)) return ROWS_DECLINED;
    int *flag = conv_flag_address();
    if (flag == nullptr) return ROWS_DECLINED;
    const int grid = (int)min((long long)sm_count() * MINB, (long long)p.ntiles);
    launch_dependent(kernel, grid, ROWS_THREADS, ROWS_SMEM_BYTES, st, p, flag);
    return ROWS_SERVED;
  }
}

template <typename T, int K>
int launch_lanerow_conv_w(const LaneRowConvParams &p, int W, cudaStream_t st) {
  switch (W) {
    case 7: return launch_lanerow_conv<T, K, 7>(p, st);
    case 14: return launch_lanerow_conv<T, K, 14>(p, st);
    case 28: return launch_lanerow_conv<T, K, 28>(p, st);
    default: return ROWS_DECLINED;
  }
}

// Maps 7, 14 or 28 columns wide and at most 32 rows high, 16-byte aligned tensors.  3x3 on 14-
// and 28-column maps stays with the window kernel, which already runs at the speed of a plain
// copy there (22.0 us against 22.8 us in this layout on N128 C576 14x14, 28.7 against 30.6 us
// on N128 C192 28x28); 5x5 on 14-column maps: 28.6 against 32.0 us; 7x7: 37.3 against 48.6 us.
template <typename T>
int try_lanerow_conv(const RowsParams &rp, int K, int S, cudaStream_t st) {
  if (S != 1 || !lanerow_conv_compiled(K, rp.Win) || rp.Hin > 32 || rp.Hout != rp.Hin ||
      rp.Wout != rp.Win || t_plan_out != nullptr)
    return ROWS_DECLINED;
  if (((reinterpret_cast<uintptr_t>(rp.in) | reinterpret_cast<uintptr_t>(rp.out)) & 15) != 0)
    return ROWS_DECLINED;
  const int mode = tuning_int("LANEROW", 1);
  if (mode == 0) return ROWS_DECLINED;
  if (K == 3 && rp.Win >= 14 && mode != 2) return ROWS_DECLINED;
  LaneRowConvParams p{};
  const int lanes = ROWS_CWARPS * 32;
  const int plane_bytes = rp.Hin * rp.Win * (int)sizeof(T);
  int G = lanes / rp.Hin;
  if (G > rp.NC) G = rp.NC;
  auto region = [&](int g) { return round_up(g * plane_bytes + 16, 16); };
  auto need = [&](int g) { return LANEROW_ZERO_BYTES + 2 * region(g); };
  while (G > 1 && need(G) > ROWS_RING_BYTES / 2) --G;
  if (G < 1 || need(G) > ROWS_RING_BYTES / 2) return ROWS_DECLINED;
  p.NST = need(G) <= ROWS_RING_BYTES / 3 ? 3 : 2;
  p.in = rp.in; p.w = rp.w; p.out = rp.out;
  p.NC = rp.NC; p.C = rp.C; p.H = rp.Hin; p.G = G;
  p.INOFF = LANEROW_ZERO_BYTES;
  p.OUTOFF = p.INOFF + region(G);
  p.ntiles = ceil_div(rp.NC, G);
  p.flip = rp.flip;
  p.ep = rp.ep;
  switch (K) {
    case 3: return launch_lanerow_conv_w<T, 3>(p, rp.Win, st);
    case 5: return launch_lanerow_conv_w<T, 5>(p, rp.Win, st);
    case 7: return launch_lanerow_conv_w<T, 7>(p, rp.Win, st);
    default: return ROWS_DECLINED;
  }
}

template <typename T, int MODE, bool EPI>
int select_k(const RowsParams &p, int K, int S, cudaStream_t st) {
  if (try_lanerow_conv<T>(p, K, S, st) == ROWS_SERVED) return ROWS_SERVED;
  switch (K * 10 + S) {
    case 31: return select_conv<T, 3, 1, MODE_FWD, EPI>(p, st);
    case 51: return select_conv<T, 5, 1, MODE_FWD, EPI>(p, st);
    case 71: return select_conv<T, 7, 1, MODE_FWD, EPI>(p, st);
    case 32: return select_conv<T, 3, 2, MODE, EPI>(p, st);
    case 52: return select_conv<T, 5, 2, MODE, EPI>(p, st);
    case 72: return select_conv<T, 7, 2, MODE, EPI>(p, st);
    default: return ROWS_DECLINED;
  }
}

// The family covers square odd filters, equal strides 1 or 2, padding k/2, and the output
// extent that padding implies: 3/5/7 here, 9..31 at stride 1 in rows_bigk.cu.
inline bool conv_shape_ok(const Shape &s, bool big) {
  if (s.kh != s.kw) return false;
  if (!big && s.kh != 3 && s.kh != 5 && s.kh != 7) return false;
  if (big && (s.kh < 9 || s.kh > 31 || (s.kh & 1) == 0 || s.sh != 1)) return false;
  if (s.sh != s.sw || (s.sh != 1 && s.sh != 2)) return false;
  if (s.ph != s.kh / 2 || s.pw != s.kw / 2) return false;
  if (s.Ho != (s.H + 2 * s.ph - s.kh) / s.sh + 1 || s.Wo != (s.W + 2 * s.pw - s.kw) / s.sw + 1)
    return false;
  return true;
}


// Reads and clears this translation unit's error flag.
inline int conv_take_error_here() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_conv_error_flag, sizeof(int)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (v) {
    const int zero = 0;
    (void)cudaMemcpyToSymbol(g_conv_error_flag, &zero, sizeof(int));
  }
  return v;
}

}  // namespace

}  // namespace dwb
