// AutoPipe: heuristic search for the pipeline-stage partition of a layer sequence that minimises
// the simulated 1F1B iteration time (2*stages micro-batches), given per-layer forward and
// backward costs.  Native because the search evaluates thousands of candidate partitions.
//
// Same cost model and search moves as the reference partitioner (Merak/cpp/autopipe.cpp:77-578),
// so it returns the same stage boundaries on the same cost vectors:
//   1. seed: min-max contiguous partition of (fwd+bwd) cost by dynamic programming;
//   2. cost of a candidate: event-time simulation of the 1F1B steady phase, detection of the
//      critical stage (the stage that never idles in steady state, searched from the last stage),
//      then the cool-down phase seen from that stage;
//   3. breadth-first exploration: (a) shift first layers of the stages behind the critical stage
//      one stage forward while they have slack, (b) move one layer across the critical stage's
//      front or back boundary and re-balance everything in front of it with the DP table.
//
// A partition is stored as the start index of every stage (`starts`, one entry per stage), stage i
// owning layers [starts[i], starts[i+1]).  Exposed through a C ABI for ctypes.
#include <algorithm>
#include <array>
#include <climits>
#include <cstdint>
#include <queue>
#include <set>
#include <utility>
#include <vector>

namespace {

using i64 = long long;
constexpr i64 kInf = LLONG_MAX;

struct Costs {
  std::vector<i64> fwd, bwd, prefix;           // prefix over fwd+bwd
  std::vector<std::vector<i64>> minmax;        // minmax[n][k]: best bottleneck of first n layers in k parts
  int layers = 0, stages = 0;

  Costs(const i64* f, const i64* b, int n, int s) : fwd(f, f + n), bwd(b, b + n), layers(n), stages(s) {
    prefix.assign(n + 1, 0);
    for (int i = 0; i < n; ++i) prefix[i + 1] = prefix[i] + fwd[i] + bwd[i];
    const int kmax = std::min(n, s);
    minmax.assign(n + 1, std::vector<i64>(kmax + 1, kInf));
    minmax[0][0] = 0;
    for (int cnt = 1; cnt <= n; ++cnt)
      for (int k = 1; k <= std::min(cnt, s); ++k)
        for (int p = 0; p < cnt; ++p)
          minmax[cnt][k] = std::min(minmax[cnt][k], std::max(minmax[p][k - 1], prefix[cnt] - prefix[p]));
  }

  // Start indices of the optimal min-max split of the first `count` layers into `parts` stages.
  // Ties are resolved by the smallest start of the LAST stage first (widest last stage).
  bool balanced_starts(int count, int parts, std::vector<int>& out) const {
    out.assign(parts, 0);
    int n = count;
    for (int k = parts; k >= 1; --k) {
      if (n <= 0 || n < k) return false;
      int p = 0;
      while (p < n && minmax[n][k] != std::max(minmax[p][k - 1], prefix[n] - prefix[p])) ++p;
      if (p >= n) return false;
      out[k - 1] = p;
      n = p;
    }
    return n == 0;
  }
};

struct StageTimes {
  std::vector<i64> f, b;   // 1-based per stage, zero sentinels at 0 and S+1
};

StageTimes stage_times(const Costs& c, const std::vector<int>& starts) {
  const int S = (int)starts.size();
  StageTimes t;
  t.f.assign(S + 2, 0);
  t.b.assign(S + 2, 0);
  for (int s = 0; s < S; ++s) {
    const int lo = starts[s], hi = (s + 1 < S) ? starts[s + 1] : c.layers;
    for (int l = lo; l < hi; ++l) {
      t.f[s + 1] += c.fwd[l];
      t.b[s + 1] += c.bwd[l];
    }
  }
  return t;
}

struct SimResult {
  i64 time = kInf;
  int critical = -1;
};

// Event-time model of one 1F1B iteration with 2*S micro-batches.
SimResult simulate(const StageTimes& t) {
  const int S = (int)t.f.size() - 2;
  const int MB = 2 * S;
  auto last_mb = [&](int stage) { return MB - S + stage; };
  // start[stage+1][mb][0|1]: start of the forward | backward of micro-batch mb on `stage`
  std::vector<std::vector<std::array<i64, 2>>> start(S + 2, std::vector<std::array<i64, 2>>(MB, {0, 0}));
  i64 first_bwd = 0;
  for (int s = 0; s < S; ++s) first_bwd += t.f[s + 1];
  for (int s = S - 1; s >= 0; --s) {
    start[s + 1][0][0] = INT32_MIN;
    start[s + 1][0][1] = first_bwd;
    first_bwd += t.b[s + 1];
  }
  for (int mb = 1; mb < MB; ++mb) {
    for (int s = 0; s < S; ++s)
      if (mb <= last_mb(s))
        start[s + 1][mb][0] = std::max(start[s][mb - 1][0] + t.f[s], start[s + 1][mb - 1][1] + t.b[s + 1]);
    for (int s = S - 1; s >= 0; --s)
      if (mb <= last_mb(s))
        start[s + 1][mb][1] = std::max(start[s + 2][mb][1] + t.b[s + 2], start[s + 1][mb][0] + t.f[s + 1]);
  }
  // critical stage: no idle gap between consecutive slots during the steady phase
  int crit = S - 1;
  for (; crit >= 0; --crit) {
    int mb = 1;
    for (; mb <= last_mb(crit); ++mb) {
      if (start[crit + 1][mb][0] != start[crit + 1][mb - 1][1] + t.b[crit + 1]) break;
      if (start[crit + 1][mb][1] != start[crit + 1][mb][0] + t.f[crit + 1]) break;
    }
    if (mb == last_mb(crit) + 1) break;
  }
  SimResult r;
  if (crit < 0) return r;
  // cool-down seen from the critical stage
  const int V = S - crit;
  std::vector<std::vector<i64>> cd(V, std::vector<i64>(V, 0));
  i64 bst = start[crit + 1][last_mb(crit)][0];
  for (int i = 0; i < V; ++i) {
    bst += t.f[crit + 1 + i];
    cd[i][V - 1 - i] = bst;
  }
  for (int col = V - 2; col >= 0; --col)
    for (int row = V - col - 2; row >= 0; --row) {
      cd[row][col] = std::max(cd[row][col + 1] + t.b[crit + 1 + row], cd[row + 1][col] + t.b[crit + 2 + row]);
      if (row > 0) cd[row][col] = std::max(cd[row][col], cd[row - 1][col + 1]);
    }
  i64 total = cd[0][0];
  for (int s = crit; s > 0; --s) total += t.b[s + 1];
  total += t.b[1];
  r.time = total;
  r.critical = crit;
  return r;
}

struct Best {
  std::vector<int> starts;
  i64 time = kInf;
  void offer(const std::vector<int>& s, const SimResult& r) {
    if (r.time < time) {
      time = r.time;
      starts = s;
    }
  }
};

int stage_size(const Costs& c, const std::vector<int>& starts, int s) {
  const int hi = (s + 1 < (int)starts.size()) ? starts[s + 1] : c.layers;
  return hi - starts[s];
}

// Move (a): let the stages after the critical one absorb layers from their successors while the
// critical stage still hides their work.
void relax_tail(const Costs& c, const std::vector<int>& seed, int crit_base, Best& best) {
  const int S = (int)seed.size();
  std::vector<int> cur = seed;
  int upto = crit_base + 1;
  i64 gap = 0;
  for (;;) {
    const StageTimes t = stage_times(c, cur);
    const SimResult r = simulate(t);
    if (upto == S) {
      best.offer(cur, r);
      return;
    }
    if (r.critical != crit_base) return;
    best.offer(cur, r);
    i64 tail = 0;
    for (int s = crit_base + 1; s <= upto; ++s) tail += t.f[s + 1] + t.b[s + 1];
    const i64 hidden = (i64)(upto - crit_base) * t.b[crit_base + 1] + gap;
    if (tail <= hidden) {
      ++upto;
      continue;
    }
    bool moved = false;
    for (int bt = crit_base + 1; bt < upto; ++bt) {
      if (bt + 1 >= S || stage_size(c, cur, bt + 1) <= 1) continue;   // never empty a stage
      const int blk = cur[bt + 1];
      const i64 crit_cost = t.f[crit_base + 1] + t.b[crit_base + 1];
      const i64 bt_cost = t.f[bt + 1] + t.b[bt + 1];
      if (crit_cost > bt_cost + c.fwd[blk] + c.bwd[blk]) {
        cur[bt + 1] += 1;   // first layer of stage bt+1 joins stage bt
        i64 upto_bt = 0;
        for (int s = crit_base + 1; s <= bt; ++s) upto_bt += t.f[s + 1] + t.b[s + 1];
        const i64 hidden_bt = (i64)(bt - crit_base) * t.b[crit_base + 1] + gap;
        gap += std::max<i64>(0, upto_bt - hidden_bt);
        upto = bt + 1;
        moved = true;
        break;
      }
    }
    if (!moved) return;
  }
}

std::vector<int> search(const Costs& c) {
  const int S = c.stages;
  std::vector<int> seed;
  if (!c.balanced_starts(c.layers, S, seed)) {
    seed.resize(S);
    for (int s = 0; s < S; ++s) seed[s] = (int)((i64)s * c.layers / S);
    return seed;
  }
  Best best;
  std::set<std::vector<int>> seen;
  std::queue<std::vector<int>> frontier;
  frontier.push(seed);
  while (!frontier.empty()) {
    const std::vector<int> cur = frontier.front();
    frontier.pop();
    const SimResult base = simulate(stage_times(c, cur));
    best.offer(cur, base);
    if (base.critical < 0) continue;
    relax_tail(c, cur, base.critical, best);

    const int crit = base.critical;
    if (crit == 0) continue;
    // Move (b1): the critical stage gives its first layer to the stages in front of it.
    if (stage_size(c, cur, crit) > 1) {   // a stage is never left empty
      const int count = cur[crit] + 1;
      std::vector<int> head;
      if (c.balanced_starts(count, crit, head)) {
        std::vector<int> cand = cur;
        for (int s = 0; s < crit; ++s) cand[s] = head[s];
        cand[crit] = count;
        if (seen.insert(cand).second) frontier.push(cand);
      }
    }
    // Move (b2): the critical stage gives its last layer to the stage behind it.
    if (crit < S - 1 && stage_size(c, cur, crit) > 1) {
      const int count = cur[crit + 1] - 1;
      std::vector<int> head;
      if (count >= crit + 1 && c.balanced_starts(count, crit + 1, head)) {
        std::vector<int> cand = cur;
        for (int s = 0; s <= crit; ++s) cand[s] = head[s];
        cand[crit + 1] = count;
        const SimResult r = simulate(stage_times(c, cand));
        if (r.critical <= crit && seen.insert(cand).second) frontier.push(cand);
      }
    }
  }
  return best.starts.empty() ? seed : best.starts;
}

}  // namespace

extern "C" {

// Writes the first layer index of every stage into out[0..stages).  Returns 0 on success.
__attribute__((visibility("default"))) int mrk_autopipe_partition(const long long* fwd, const long long* bwd,
                                                                   int layers, int stages, int* out) {
  if (!fwd || !bwd || !out || layers <= 0 || stages <= 0 || stages > layers) return 1;
  Costs c(fwd, bwd, layers, stages);
  const std::vector<int> starts = search(c);
  for (int s = 0; s < stages; ++s) out[s] = starts[s];
  return 0;
}

// Simulated 1F1B iteration time (2*stages micro-batches) of a given partition; `critical` receives
// the index of the critical stage.  Returns -1 when the model has no steady-state critical stage.
__attribute__((visibility("default"))) long long mrk_autopipe_simulate(const long long* fwd, const long long* bwd,
                                                                        int layers, const int* starts, int stages,
                                                                        int* critical) {
  if (!fwd || !bwd || !starts || layers <= 0 || stages <= 0) return -1;
  Costs c(fwd, bwd, layers, stages);
  const std::vector<int> st(starts, starts + stages);
  const SimResult r = simulate(stage_times(c, st));
  if (critical) *critical = r.critical;
  return r.time == kInf ? -1 : r.time;
}

}  // extern "C"
