#include "auto_tuner.h"

#include <algorithm>
#include <cmath>

namespace gvrt {

SplitChoice pick_decode_splits(int batch, int kv_heads, int max_kv_len, int num_sms,
                               int ctas_per_sm, int max_splits) {
  constexpr int kWarpTile = 32;      // tokens per warp tile
  constexpr int kRound = 4 * 32;     // tokens a 4-warp CTA consumes per round
  constexpr int kMinChunk = 256;     // do not split below this many tokens per task
  SplitChoice best{1, std::max(kWarpTile, (max_kv_len + kWarpTile - 1) / kWarpTile * kWarpTile), -1.0};
  if (batch <= 0 || kv_heads <= 0 || max_kv_len <= 0) return best;
  const int slots = std::max(1, num_sms * std::max(1, ctas_per_sm));
  int limit = std::max(1, std::min(max_splits, (max_kv_len + kMinChunk - 1) / kMinChunk));
  // Measured on B200 (64 requests, context 1060 - 1168, 128-wide heads): once the unsplit grid has
  // about two thirds of an SM count of tasks, every split costs more in partial writes and merge
  // work than it wins in balance (512 tasks: 51 us unsplit, 78 us with 2 splits; 128 tasks: 20.5
  // against 24.0), while 64 tasks do gain from 4 splits (20.0 -> 17.2 us). So such grids stay
  // unsplit, and the others get at most enough splits for about 1.75 tasks per SM.
  const long long base_tasks = (long long)batch * kv_heads;
  int lowest = 1;
  if (base_tasks * 3 >= (long long)num_sms * 2) {
    limit = 1;
  } else {
    limit = (int)std::max<long long>(1, std::min<long long>(limit, (long long)num_sms * 7 / 4 / base_tasks));
    lowest = limit;                       // small grids: fill the device (about 1.75 tasks per SM)
  }
  for (int s = lowest; s <= limit; ++s) {
    int chunk = (max_kv_len + s - 1) / s;
    chunk = (chunk + kWarpTile - 1) / kWarpTile * kWarpTile;
    if ((long long)chunk * (s - 1) >= max_kv_len && s > 1) continue;  // last split would be empty
    const long long tasks = (long long)batch * kv_heads * s;
    const long long waves = (tasks + slots - 1) / slots;
    const double wave_eff = (double)tasks / (double)(waves * slots);
    const int rounds = (chunk + kRound - 1) / kRound;
    const double round_eff = (double)chunk / (double)(rounds * kRound);
    // time model: waves * (rounds + fixed per-task cost) (+ merge pass when s > 1)
    const double per_task = rounds + 1.5;
    const double time = (double)waves * per_task / std::max(round_eff, 0.25) + (s > 1 ? 1.0 + 0.05 * s : 0.0);
    const double ideal = (double)batch * kv_heads * ((double)max_kv_len / kRound) / slots;
    const double score = 0.7 * (ideal / time) + 0.2 * wave_eff + 0.1 * round_eff;
    if (score > best.score + 1e-9) best = SplitChoice{s, chunk, score};
  }
  return best;
}

}  // namespace gvrt
