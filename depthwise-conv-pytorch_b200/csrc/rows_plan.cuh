// Host-side tiling decisions of the rows family, shared by its translation units.
#pragma once

#include <atomic>
#include <cstdio>
#include <cstdlib>
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

// Launch with the programmatic-serialization attribute: the kernel may become resident while the
// kernel before it in the stream drains; it calls pdl_wait() before touching global memory.
template <typename KernelT, typename... Args>
inline void launch_dependent(KernelT kernel, int grid, int block, int smem_bytes, cudaStream_t st,
                             Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  (void)cudaLaunchKernelEx(&cfg, kernel, args...);  // errors are read by the caller (peek)
}

// The same with the grid cut into thread-block clusters of `cluster` consecutive CTAs (at most 8).
// False, with nothing launched, unless ALL the grid's clusters can be resident at once (a cluster
// needs its CTAs inside one GPC, so fewer CTAs fit than without clusters; a grid that needs a
// second wave of clusters measured much slower than the two-kernel form: 50 against 32 us on the
// N128 C576 14x14 layer).  The device is asked once per kernel and cluster size.
struct ClusterLimits {
  std::atomic<int> max_active[9];  // 0: not asked yet; -1: impossible
};
template <typename KernelT, typename... Args>
inline bool launch_dependent_cluster(KernelT kernel, int grid, int block, int smem_bytes, cudaStream_t st,
                                     int cluster, ClusterLimits &limits, Args... args) {
  if (cluster < 1 || cluster > 8 || grid % cluster != 0) return false;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  int limit = limits.max_active[cluster].load(std::memory_order_acquire);
  if (limit == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = -1;
    }
    limits.max_active[cluster].store(n, std::memory_order_release);
    limit = n;
  }
  if (limit < grid / cluster) return false;
  (void)cudaLaunchKernelEx(&cfg, kernel, args...);
  return true;
}

// What the planner needs to know about one problem.
struct PlanInput {
  int K, S, mode;    // mode of the x/in window (backward-filter: MODE_FWD)
  int Hin, Win;      // staged input map
  int Hout, Wout;    // rows the tasks iterate over / their width
  int esize;         // bytes per element
  int NSEG;          // segments per CTA
  int maxG;          // planes that can share a tile (forward: N*C; backward-filter: C)
  int stage_bytes;   // capacity of one stage (set by the planner: 32 KB x 3 or 48 KB x 2)
  int slots;         // CTAs resident on the device at once (forward / backward-input: a small
                     // problem should still be cut into at least this many tiles); 0 = ignore
  bool filter;       // backward-filter: the stage also holds the Hout x Wout rows (dy), no taps,
                     // and a segment keeps one task for a whole item (G * NRB <= NSEG)
};

// One tiling of the problem for a given rows-per-chunk U.
struct TilePlan {
  bool ok;
  int U;
  int G, NRT, TH, NRB, RBH;
  int TAPB, DYOFF;
  int NST;     // stages the ring is cut into
  bool exact;  // every task of every tile has exactly RBH rows
  int bytes;   // stage bytes in use
  double eff;  // useful output rows / segment-row slots spent
};

// Fills RBH and the stage layout for a candidate (G, NRT, TH, NRB) and scores it.
inline bool plan_finish(const PlanInput &in, int U, TilePlan &t) {
  const int RS = (in.mode == MODE_BWD) ? in.S : 1;
  const int b = in.esize;
  int lenmax = 0, lenmin = 1 << 30, rows_in = 0;
  for (int rt = 0; rt < t.NRT; ++rt) {
    const int R0 = rt * t.TH, th = (in.Hout - R0 < t.TH) ? in.Hout - R0 : t.TH;
    int lo = 0, hi = in.Hin;
    if (t.NRT > 1) tile_in_rows(in.K, in.S, in.mode, R0, th, in.Hin, lo, hi);
    if (hi - lo > rows_in) rows_in = hi - lo;
    for (int rb = 0; rb < t.NRB; ++rb) {
      int r0, r1;
      task_rows(rb, t.NRB, R0, th, RS, r0, r1);
      if (r1 - r0 > lenmax) lenmax = r1 - r0;
      if (r1 - r0 < lenmin) lenmin = r1 - r0;
    }
  }
  if (lenmax <= 0) return false;
  if (in.filter && t.G * t.NRB > in.NSEG) return false;
  t.RBH = round_up(lenmax, U);
  t.exact = (lenmin == t.RBH);
  // stage: [taps][16 zero bytes][rows, up to 15 bytes behind their aligned start]
  // taps: up to two ranges, each up to 15 bytes behind a 16-byte boundary
  t.TAPB = in.filter ? 0 : round_up(t.G * in.K * in.K * b + 48, 128);
  int total = t.TAPB + 16 + 16 + t.G * rows_in * in.Win * b;
  t.DYOFF = 0;
  if (in.filter) {
    t.DYOFF = round_up(total, 16);
    total = t.DYOFF + 16 + t.G * t.TH * in.Wout * b;
  }
  t.bytes = total;
  if (total > in.stage_bytes) return false;
  // Cost in segment-row slots: every task pays its rows, the window rows it re-reads above its
  // first row, and a fixed set-up; every tile pays a fixed hand-over.  Score = useful rows / cost.
  const int rounds = ceil_div(t.G * t.NRB, in.NSEG);
  const double halo = (in.mode == MODE_FWD) ? (double)(in.K - in.S) / in.S : (double)(in.K - 1) / in.S;
  const double task_rows_cost = t.RBH + halo + 2.0;
  t.eff = (double)in.Hout * t.G /
          ((double)t.NRT * in.NSEG * (rounds * task_rows_cost + 2.0));
  if (t.exact) t.eff *= 1.03;  // no per-row tests in the inner loop
  if (in.slots > 0) {
    const double ntiles = (double)ceil_div(in.maxG, t.G) * t.NRT;
    if (ntiles < in.slots) {
      t.eff *= ntiles / in.slots;  // too few tiles leave SMs idle
    } else {
      // tiles are dealt round-robin to the resident CTAs: the last round is only partly full
      const double rounds_of_tiles = ntiles / in.slots;
      t.eff *= rounds_of_tiles / (double)ceil_div((int)ntiles, in.slots);
    }
  }
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
  int gmax = 4 * in.NSEG;
  if (in.filter) gmax = in.NSEG;
  if (gmax > in.maxG) gmax = in.maxG;
  for (int G = gmax; G >= 1; --G) {
    const int nrb_max = (G >= in.NSEG) ? 1 : in.NSEG / G;
    for (int NRB = 1; NRB <= nrb_max; ++NRB) {
      if (NRB > 1 && NRB * RS > in.Hout) break;
      TilePlan c{};
      c.G = G; c.NRT = 1; c.TH = in.Hout; c.NRB = NRB;
      consider(c);
    }
  }
  if (best.ok && !(in.slots > 0 && (double)ceil_div(in.maxG, best.G) < in.slots)) return best;
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

inline TilePlan plan_search(PlanInput in, const int *u_options, int n_options) {
  TilePlan best{};
  best.ok = false;
  // three 32 KB stages unless two 48 KB stages are clearly more efficient (small planes whose
  // groups do not fit 32 KB): a deeper ring hides more latency
  for (int nst = 3; nst >= 2; --nst) {
    in.stage_bytes = ROWS_RING_BYTES / nst;
    TilePlan cfg{};
    cfg.ok = false;
    for (int i = 0; i < n_options; ++i) {
      TilePlan c = plan_for_u(in, u_options[i]);
      if (!c.ok) continue;
      // prefer efficiency; at near-equal efficiency the larger U (less loop overhead)
      if (!cfg.ok || c.eff > cfg.eff * 1.02 || (c.eff >= cfg.eff * 0.98 && c.U > cfg.U)) cfg = c;
    }
    if (!cfg.ok) continue;
    cfg.NST = nst;
    if (!best.ok || cfg.eff > best.eff * 1.25) best = cfg;
  }
  return best;
}

// Tuning aids, compiled only into a library built with -DDWCONV_B200_TUNING (never the shipped
// one): environment variables that override the planner and the variant selection, for sweeps.
//   DWCONV_B200_FORCE_PLAN="fwd=U,G,NRT,TH,NRB,NST;bwd=...;flt=..."  one tiling (refused if it
//       does not fit) for forward / stride-1 backward-input, stride-2 backward-input, backward-filter
//   DWCONV_B200_FORCE_U="fwd=U;bwd=U;flt=U"   one chunk height
//   DWCONV_B200_<NAME>=int                     switches read with tuning_int("<NAME>", default)
#ifdef DWCONV_B200_TUNING
inline int tuning_int(const char *name, int dflt) {
  char key[96];
  std::snprintf(key, sizeof(key), "DWCONV_B200_%s", name);
  const char *v = std::getenv(key);
  return v ? std::atoi(v) : dflt;
}
inline bool forced_plan(const PlanInput &in, TilePlan &out) {
  const char *env = std::getenv("DWCONV_B200_FORCE_PLAN");
  if (env == nullptr) return false;
  const char *key = in.filter ? "flt=" : (in.mode == MODE_BWD ? "bwd=" : "fwd=");
  const char *at = std::strstr(env, key);
  if (at == nullptr) return false;
  int v[6] = {0, 0, 0, 0, 0, 0};
  if (std::sscanf(at + 4, "%d,%d,%d,%d,%d,%d", &v[0], &v[1], &v[2], &v[3], &v[4], &v[5]) != 6) return false;
  PlanInput pin = in;
  TilePlan c{};
  c.G = v[1]; c.NRT = v[2]; c.TH = v[3]; c.NRB = v[4];
  if (v[5] < 2 || v[5] > 3 || c.G < 1 || c.NRT < 1 || c.TH < 1 || c.NRB < 1 || c.G > in.maxG ||
      ceil_div(in.Hout, c.TH) != c.NRT)
    return false;
  pin.stage_bytes = ROWS_RING_BYTES / v[5];
  if (!plan_finish(pin, v[0], c)) return false;
  c.NST = v[5];
  out = c;
  return true;
}
inline int forced_u(const PlanInput &in) {
  const char *env = std::getenv("DWCONV_B200_FORCE_U");
  if (env == nullptr) return 0;
  const char *at = std::strstr(env, in.filter ? "flt=" : (in.mode == MODE_BWD ? "bwd=" : "fwd="));
  return at ? std::atoi(at + 4) : 0;
}
#else
inline int tuning_int(const char *, int dflt) { return dflt; }
#endif

// Planning walks a few hundred candidates; results are remembered per problem so that a
// repeated launch costs one table lookup.
inline TilePlan plan_best(const PlanInput &in, const int *u_options, int n_options) {
#ifdef DWCONV_B200_TUNING
  {
    TilePlan forced{};
    if (forced_plan(in, forced)) {
      for (int i = 0; i < n_options; ++i)
        if (u_options[i] == forced.U) return forced;
    }
    const int fu = forced_u(in);
    for (int i = 0; fu > 0 && i < n_options; ++i)
      if (u_options[i] == fu) return plan_search(in, &u_options[i], 1);
  }
#endif
  struct Entry {
    int key[16];
    TilePlan plan;
  };
  static std::mutex mu;
  static std::vector<Entry> table;
  int key[16] = {in.K, in.S, in.mode, in.Hin, in.Win, in.Hout, in.Wout, in.esize, in.NSEG,
                 in.maxG, in.filter ? 1 : 0, n_options, 0, 0, 0, 0};  // stage_bytes: planner-set
  key[15] = in.slots;
  for (int i = 0; i < n_options && i < 3; ++i) key[12 + i] = u_options[i];
  if (n_options > 4) n_options = 4;
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
