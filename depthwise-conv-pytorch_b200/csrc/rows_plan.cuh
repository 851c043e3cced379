// Host-side tiling decisions of the rows family, shared by its translation units.
#pragma once

#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

#include "rows_engine.cuh"

namespace dwb {

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
template <typename KernelT>
inline bool ensure_smem(KernelT kernel, int bytes, std::atomic<unsigned long long> &done) {
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

// What the planner needs to know about one problem.
struct PlanInput {
  int K, S, mode;    // mode of the x/in window (backward-filter: MODE_FWD)
  int Hin, Win;      // staged input map
  int Hout, Wout;    // rows the tasks iterate over / their width
  int esize;         // bytes per element
  int NSEG;          // segments per CTA
  bool taps;         // the stage holds the tile's taps (forward / backward-input)
  bool stage_out;    // the stage also holds the Hout x Wout map (backward-filter: dy)
};

// One tiling of the problem for a given rows-per-chunk U.
struct TilePlan {
  bool ok;
  int U;
  int G, NRT, TH, NRB, RBH;
  int PS, ZT, ZBF, TAPB, DPL, DYOFF;
  int bytes;   // stage bytes in use
  double eff;  // useful output rows / segment-row slots spent
};

inline int plan_base_row(int mode, int S, int r) { return mode == MODE_FWD ? r * S : r / S; }

// Fills margins / slot sizes for a candidate (G, NRT, TH, NRB) and scores it.
inline bool plan_finish(const PlanInput &in, int U, TilePlan &t) {
  const int RS = (in.mode == MODE_BWD) ? in.S : 1;
  const int RMIN = geo_min_rel(in.K, in.S, in.mode, U), RMAX = geo_max_rel(in.K, in.S, in.mode, U);
  const int b = in.esize;
  int lenmax = 0;
  for (int rt = 0; rt < t.NRT; ++rt) {
    const int R0 = rt * t.TH, th = (in.Hout - R0 < t.TH) ? in.Hout - R0 : t.TH;
    for (int rb = 0; rb < t.NRB; ++rb) {
      int r0, r1;
      task_rows(rb, t.NRB, R0, th, RS, r0, r1);
      if (r1 - r0 > lenmax) lenmax = r1 - r0;
    }
  }
  if (lenmax <= 0) return false;
  t.RBH = round_up(lenmax, U);
  int qmin = 0, rows_need = 0;
  for (int rt = 0; rt < t.NRT; ++rt) {
    const int R0 = rt * t.TH, th = (in.Hout - R0 < t.TH) ? in.Hout - R0 : t.TH;
    int lo = 0, hi = in.Hin;
    if (t.NRT > 1) tile_in_rows(in.K, in.S, in.mode, R0, th, in.Hin, lo, hi);
    int need = hi - lo;
    if (t.NRT > 1 && hi == in.Hin) need += in.K;  // cleared rows below the map
    for (int rb = 0; rb < t.NRB; ++rb) {
      int r0, r1;
      task_rows(rb, t.NRB, R0, th, RS, r0, r1);
      const int q0 = plan_base_row(in.mode, in.S, r0) + RMIN - lo;
      const int q1 = plan_base_row(in.mode, in.S, r0 + t.RBH - U) + RMAX - lo;  // last row read
      if (q0 < qmin) qmin = q0;
      if (q1 + 1 > need) need = q1 + 1;
    }
    if (need > rows_need) rows_need = need;
  }
  const int above_bytes = (-qmin) * in.Win * b;
  t.ZT = round_up(above_bytes < 16 ? 16 : above_bytes, 16) / b;
  // + 32 bytes: the data may sit up to 15 bytes behind the slot's aligned start (it keeps its
  // source's phase) and 16 bytes behind it are cleared
  t.PS = round_up((t.ZT + rows_need * in.Win) * b + 32, 16) / b;
  t.ZBF = (t.NRT > 1) ? in.K * in.Win : 0;
  t.TAPB = in.taps ? round_up(t.G * in.K * in.K * 4, 128) : 0;
  int total = t.TAPB + t.G * t.PS * b;
  t.DPL = 0;
  t.DYOFF = 0;
  if (in.stage_out) {
    t.DYOFF = round_up(total, 128);
    t.DPL = round_up(t.TH * in.Wout * b + 32, 16) / b;
    total = t.DYOFF + t.G * t.DPL * b;
  }
  t.bytes = total;
  if (total > ROWS_STAGE_BYTES) return false;
  const int rounds = ceil_div(t.G * t.NRB, in.NSEG);
  t.eff = (double)in.Hout * t.G / ((double)t.NRT * rounds * in.NSEG * t.RBH);
  t.U = U;
  t.ok = true;
  return true;
}

// Best tiling for a given U: whole planes when they fit (several per tile if small), else row
// tiles of one plane.
inline TilePlan plan_for_u(const PlanInput &in, int U) {
  TilePlan best{};
  best.ok = false;
  const int RS = (in.mode == MODE_BWD) ? in.S : 1;
  auto consider = [&](TilePlan &c) -> bool {
    if (!plan_finish(in, U, c)) return false;
    // higher efficiency wins; at (near) equal efficiency the larger tile
    if (!best.ok || c.eff > best.eff * 1.02 || (c.eff >= best.eff * 0.98 && c.bytes > best.bytes))
      best = c;
    return true;
  };
  // whole planes: every group size up to four rounds of segments
  for (int G = 4 * in.NSEG; G >= 1; --G) {
    const int nrb_max = (G >= in.NSEG) ? 1 : in.NSEG / G;
    for (int NRB = 1; NRB <= nrb_max; ++NRB) {
      if (NRB > 1 && NRB * RS > in.Hout) break;
      TilePlan c{};
      c.G = G; c.NRT = 1; c.TH = in.Hout; c.NRB = NRB;
      consider(c);
    }
  }
  if (best.ok) return best;
  // row tiles of a single plane: the few largest tile heights that fit
  int fits = 0;
  for (int NRT = 2; NRT <= in.Hout && fits < 4; ++NRT) {
    const int TH = round_up(ceil_div(in.Hout, NRT), RS);
    if (ceil_div(in.Hout, TH) != NRT) continue;
    bool fit = false;
    for (int NRB = 1; NRB <= in.NSEG; ++NRB) {
      if (NRB > 1 && NRB * RS > TH) break;
      TilePlan c{};
      c.G = 1; c.NRT = NRT; c.TH = TH; c.NRB = NRB;
      fit = consider(c) || fit;
    }
    if (fit) ++fits;
  }
  return best;
}

inline TilePlan plan_search(const PlanInput &in, const int *u_options, int n_options) {
  TilePlan best{};
  best.ok = false;
  for (int i = 0; i < n_options; ++i) {
    TilePlan c = plan_for_u(in, u_options[i]);
    if (!c.ok) continue;
    // prefer efficiency; at near-equal efficiency the larger U (less loop overhead)
    if (!best.ok || c.eff > best.eff * 1.02 || (c.eff >= best.eff * 0.98 && c.U > best.U)) best = c;
  }
  return best;
}

// Planning walks a few hundred candidates; results are remembered per problem so that a
// repeated launch costs one table lookup.
inline TilePlan plan_best(const PlanInput &in, const int *u_options, int n_options) {
  struct Entry {
    int key[16];
    TilePlan plan;
  };
  static std::mutex mu;
  static std::vector<Entry> table;
  int key[16] = {in.K, in.S, in.mode, in.Hin, in.Win, in.Hout, in.Wout, in.esize, in.NSEG,
                 in.taps ? 1 : 0, in.stage_out ? 1 : 0, n_options, 0, 0, 0, 0};
  for (int i = 0; i < n_options && i < 4; ++i) key[12 + i] = u_options[i];
  {
    std::lock_guard<std::mutex> lock(mu);
    for (const Entry &e : table)
      if (std::memcmp(e.key, key, sizeof(key)) == 0) return e.plan;
  }
  Entry e;
  std::memcpy(e.key, key, sizeof(key));
  e.plan = plan_search(in, u_options, n_options);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (table.size() < 4096) table.push_back(e);
  }
  return e.plan;
}

}  // namespace dwb
