// Host-side tiling decisions of the rows family, shared by its translation units.
#pragma once

#include <atomic>

#include "rows_engine.cuh"

namespace dwb {

inline int gcd_int(int a, int b) {
  while (b) {
    const int t = a % b;
    a = b;
    b = t;
  }
  return a;
}
inline int round_up(int a, int b) { return ceil_div(a, b) * b; }
inline int pick_lw(int lanes) { return lanes <= 8 ? 8 : lanes <= 16 ? 16 : lanes <= 32 ? 32 : 0; }

inline int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int v = cached[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      v = 148;
    cached[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

// Opt the kernel in to more than 48 KB of dynamic shared memory, once per device.
template <typename KernelT> inline bool ensure_smem(KernelT kernel, int bytes, std::atomic<unsigned long long> &done) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  const unsigned long long bit = 1ull << dev;
  if (done.load(std::memory_order_acquire) & bit) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  done.fetch_or(bit, std::memory_order_release);
  return true;
}

// Row/plane tiling for a map of Hin x Win inputs and Hout x Wout outputs whose per-stage
// footprint is `in_bytes_per_row` per input row plus `out_bytes_per_row` per output row
// (the latter is 0 for forward/backward-input, which do not stage their outputs).
// budget: bytes one stage may hold.  Fills G, NRT, TH, NRB, RBH; false if nothing fits.
struct TilePlan {
  int G, NRT, TH, NRB, RBH;
};
inline bool plan_tiles(TilePlan &t, int K, int S, int mode, int U, int Hin, int Hout,
                       int in_bytes_per_row, int out_bytes_per_row, int NSEG, int budget) {
  const int RS = (mode == MODE_BWD) ? S : 1;
  const long long plane_bytes = (long long)Hin * in_bytes_per_row + (long long)Hout * out_bytes_per_row;
  int maxlen;
  if (plane_bytes <= budget / 2) {
    const int Gmax = (int)(budget / plane_bytes);
    int G = 1;
    if (Gmax >= NSEG) {
      int m = Gmax / NSEG;
      if (m > 4) m = 4;
      G = NSEG * m;
    } else {
      for (int d = NSEG / 2; d >= 1; d /= 2)
        if (d <= Gmax) {
          G = d;
          break;
        }
    }
    int NRB = G >= NSEG ? 1 : NSEG / G;
    const int row_units = Hout / RS > 0 ? Hout / RS : 1;
    if (NRB > row_units) NRB = row_units;
    t.G = G;
    t.NRT = 1;
    t.TH = Hout;
    t.NRB = NRB;
    maxlen = ceil_div(Hout, NRB) + (RS - 1);
  } else {
    // largest tile height whose input rows (plus staged output rows) fit the budget
    int best = 0;
    for (int th = RS; th <= Hout + RS; th += RS) {
      int lo, hi;
      // worst case over tile positions: an interior tile
      const int in_rows = (mode == MODE_FWD) ? (th - 1) * S + K : (th + K - 2) / S + 2;
      (void)lo; (void)hi;
      if ((long long)in_rows * in_bytes_per_row + (long long)th * out_bytes_per_row <= budget)
        best = th;
      else
        break;
    }
    if (best == 0) return false;
    int NRT = ceil_div(Hout, best);
    int TH = round_up(ceil_div(Hout, NRT), RS);
    if (TH > best) TH = best;
    NRT = ceil_div(Hout, TH);
    int NRB = NSEG;
    const int row_units = TH / RS > 0 ? TH / RS : 1;
    if (NRB > row_units) NRB = row_units;
    t.G = 1;
    t.NRT = NRT;
    t.TH = TH;
    t.NRB = NRB;
    maxlen = ceil_div(TH, NRB) + (RS - 1);
  }
  t.RBH = round_up(maxlen, U);
  return true;
}

}  // namespace dwb
