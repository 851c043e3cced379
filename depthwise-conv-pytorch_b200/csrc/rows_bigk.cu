// Rows family, large filters (odd k 9..31, stride 1, padding k/2, maps up to 32 wide):
// forward and backward-input launches.
#include "rows_bigk.cuh"
#include "rows_plan.cuh"

namespace dwb {

namespace {

__device__ int g_bigk_error_flag;

int *bigk_flag_address() {
  static std::atomic<int *> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  int *p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress((void **)&p, g_bigk_error_flag) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    cached[dev].store(p, std::memory_order_release);
  }
  return p;
}

template <typename T, int KMAX>
int launch_bigk(RowsParams p, int K, cudaStream_t st) {
  constexpr int MINB = 2;
  p.LW = pick_lw(p.Win);
  if (p.LW == 0) return ROWS_DECLINED;
  const int NSEG = ROWS_CWARPS * (32 / p.LW);
  // whole planes only; a stage holds, per plane, its rows and K*KMAX fp32 taps
  const int plane_bytes = p.Hin * p.Win * (int)sizeof(T);
  const int tap_bytes = K * KMAX * 4;
  int best_G = 0, best_nst = 3, best_NRB = 1;
  double best_eff = 0;
  for (int nst = 3; nst >= 2; --nst) {
    const int cap = ROWS_RING_BYTES / nst;
    for (int G = NSEG; G >= 1; --G) {
      if (round_up(G * tap_bytes, 128) + 32 + G * plane_bytes > cap) continue;
      const int nrb_max = NSEG / G;
      for (int NRB = 1; NRB <= nrb_max; ++NRB) {
        if (NRB > 1 && p.Hout / NRB < BIGK_U) break;  // blocks shorter than U waste window rows
        const int len = ceil_div(p.Hout, NRB);
        const int rbh = round_up(len, BIGK_U);
        // useful rows / (segment slots x rows looped incl. the k-1 extra input rows per block)
        const double eff = (double)G * p.Hout / (NSEG * (double)(rbh + (K - 1) * (rbh / BIGK_U)));
        if (eff > best_eff * (nst == 2 ? 1.25 : 1.0)) {
          best_eff = eff; best_G = G; best_nst = nst; best_NRB = NRB;
        }
      }
    }
  }
  if (best_G == 0) return ROWS_DECLINED;
  p.G = best_G; p.NRT = 1; p.TH = p.Hout; p.NRB = best_NRB; p.NST = best_nst;
  p.RBH = round_up(ceil_div(p.Hout, p.NRB) + 0, BIGK_U);
  p.inv_NRB = magic_of(p.NRB);
  p.TAPB = round_up(p.G * tap_bytes, 128);
  const long long ntiles = ceil_div(p.NC, p.G);
  if (ntiles > (1ll << 30)) return ROWS_DECLINED;
  p.ntiles = (int)ntiles;
  auto kernel = rows_bigk_conv_kernel<T, KMAX, MINB>;
  static std::atomic<unsigned long long> smem_done{0};
  if (!ensure_smem(kernel, ROWS_SMEM_BYTES, smem_done)) return ROWS_DECLINED;
  int *flag = bigk_flag_address();
  if (flag == nullptr) return ROWS_DECLINED;
  const int grid = (int)min((long long)sm_count() * MINB, ntiles);
  kernel<<<grid, ROWS_THREADS, ROWS_SMEM_BYTES, st>>>(p, K, magic_of(K * KMAX), flag);
  return ROWS_SERVED;
}

}  // namespace

struct BigkFilterPlan {
  RowsFilterParams p;
  int KMAX;
};

// Tiling of the large-filter backward-filter pass; false if the family declines.
template <typename T> bool plan_bigk_filter(const Shape &s, BigkFilterPlan &f) {
  const int K = s.kh;
  if (s.kh != s.kw || K < 9 || K > 31 || (K & 1) == 0) return false;
  if (s.sh != 1 || s.sw != 1 || s.ph != K / 2 || s.pw != K / 2) return false;
  if (s.Ho != s.H || s.Wo != s.W || s.W > 32 || s.W % 4 != 0) return false;
  const int plane_bytes = s.H * s.W * (int)sizeof(T);
  RowsFilterParams &p = f.p;
  int best_G = 0, best_nst = 3, best_NRB = 1;
  double best_eff = 0;
  for (int nst = 3; nst >= 2; --nst) {
    const int cap = ROWS_RING_BYTES / nst;
    for (int G = ROWS_CWARPS; G >= 1; --G) {
      if (G > s.C) continue;
      if (64 + 2 * (G * plane_bytes + 16) > cap) continue;
      for (int NRB = 1; NRB <= ROWS_CWARPS / G; ++NRB) {
        if (NRB > 1 && s.Ho / NRB < 8) break;
        const int len = ceil_div(s.Ho, NRB);
        // busy warps x useful dy rows / (all warps x x-rows walked)
        const double eff = (double)G * s.Ho / (ROWS_CWARPS * (double)(len + K - 1));
        if (eff > best_eff * (nst == 2 ? 1.25 : 1.0)) {
          best_eff = eff; best_G = G; best_nst = nst; best_NRB = NRB;
        }
      }
    }
  }
  if (best_G == 0) return false;
  p.N = s.N; p.C = s.C; p.H = s.H; p.W = s.W; p.Ho = s.Ho; p.Wo = s.Wo;
  p.G = best_G; p.NRT = 1; p.TH = s.Ho; p.NRB = best_NRB; p.RBH = 0; p.LW = 32;
  p.inv_NRB = magic_of(p.NRB);
  p.NST = best_nst;
  p.NCG = ceil_div(s.C, p.G);
  p.TPC = s.N;
  p.DYOFF = round_up(16 + 16 + p.G * plane_bytes, 16);
  const int slots = sm_count() * 2;
  int SL = slots / p.NCG;
  if (SL < 1 || (long long)SL * p.NCG * 100 < 85ll * slots) SL = ceil_div(2 * slots, p.NCG);
  if (SL > p.TPC) SL = p.TPC;
  if (SL < 1) SL = 1;
  p.SL = SL;
  f.KMAX = K <= 15 ? 16 : 32;
  return true;
}

// in/out as RowsParams expects them (backward-input: in = dy, out = dx, flip = 1).
template <typename T> int rows_bigk_conv(const RowsParams &p, int K, cudaStream_t st) {
  if (K < 9 || K > 31 || (K & 1) == 0) return ROWS_DECLINED;
  if (p.Win > 32 || p.Win != p.Wout || p.Hin != p.Hout) return ROWS_DECLINED;
  if (p.Hin * p.Win * (int)sizeof(T) + 31 * 32 * 4 + 256 > ROWS_RING_BYTES / 2) return ROWS_DECLINED;
  return K <= 15 ? launch_bigk<T, 16>(p, K, st) : launch_bigk<T, 32>(p, K, st);
}

// Slots per channel the finalize kernel must add (slices x row blocks); 0: declined.
template <typename T> int rows_bigk_filter_slices(const Shape &s) {
  BigkFilterPlan f{};
  return plan_bigk_filter<T>(s, f) ? f.p.SL * f.p.NRB : 0;
}

template <typename T>
int rows_bigk_filter(const T *x, const T *dy, float *partial, const Shape &s, cudaStream_t st,
                     int *slices_out) {
  BigkFilterPlan f{};
  if (!plan_bigk_filter<T>(s, f)) return ROWS_DECLINED;
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy)) & 15) != 0)
    return ROWS_DECLINED;  // 128-bit loads of dy rows need the staged phase to be a multiple of 4
  f.p.x = x; f.p.dy = dy; f.p.partial = partial;
  *slices_out = f.p.SL * f.p.NRB;
  int *flag = bigk_flag_address();
  if (flag == nullptr) return ROWS_DECLINED;
  const long long items = (long long)f.p.NCG * f.p.SL;
  const int grid = (int)min((long long)sm_count() * 2, items);
  if (f.KMAX == 16) {
    auto kernel = rows_bigk_filter_kernel<T, 16, 2>;
    static std::atomic<unsigned long long> done{0};
    if (!ensure_smem(kernel, ROWS_SMEM_BYTES, done)) return ROWS_DECLINED;
    kernel<<<grid, ROWS_THREADS, ROWS_SMEM_BYTES, st>>>(f.p, s.kh, flag);
  } else {
    auto kernel = rows_bigk_filter_kernel<T, 32, 2>;
    static std::atomic<unsigned long long> done{0};
    if (!ensure_smem(kernel, ROWS_SMEM_BYTES, done)) return ROWS_DECLINED;
    kernel<<<grid, ROWS_THREADS, ROWS_SMEM_BYTES, st>>>(f.p, s.kh, flag);
  }
  return ROWS_SERVED;
}

int rows_bigk_take_error() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_bigk_error_flag, sizeof(int)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (v) {
    const int zero = 0;
    (void)cudaMemcpyToSymbol(g_bigk_error_flag, &zero, sizeof(int));
  }
  return v;
}

template int rows_bigk_filter_slices<float>(const Shape &);
template int rows_bigk_filter_slices<__half>(const Shape &);
template int rows_bigk_filter_slices<__nv_bfloat16>(const Shape &);
template int rows_bigk_filter<float>(const float *, const float *, float *, const Shape &, cudaStream_t, int *);
template int rows_bigk_filter<__half>(const __half *, const __half *, float *, const Shape &, cudaStream_t, int *);
template int rows_bigk_filter<__nv_bfloat16>(const __nv_bfloat16 *, const __nv_bfloat16 *, float *, const Shape &, cudaStream_t, int *);
template int rows_bigk_conv<float>(const RowsParams &, int, cudaStream_t);
template int rows_bigk_conv<__half>(const RowsParams &, int, cudaStream_t);
template int rows_bigk_conv<__nv_bfloat16>(const RowsParams &, int, cudaStream_t);

}  // namespace dwb
