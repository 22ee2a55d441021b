// The lane planner: how many drafts each lane of a batched window should carry.
//
// Replaces plan_rows / explore_rows (engine/src/batch_plan.hpp:63-141; its caller src/batch.cpp): host arithmetic only.
// Lane i offers up to avail[i] drafts, of which the first j + 1 all stand with probability reach[i][j]; a window of n lanes with
// d[i] drafts each is expected to yield n + sum_i sum_{j < d[i]} reach[i][j] tokens and to cost
//   base_ms + sum over the rows past the lanes' first of their price (row_lo up to the knee'th row of the window, row_hi past it)
//           + chain_ms for every draft after a chain lane's first (each is one more draft-layer call).
// The plan with the most expected tokens per ms is found exactly: for a rate lam the best plan of value tokens - lam * ms is a
// knapsack over the lanes (state: drafts handed out so far, since the rows' price depends only on their total), and lam is
// raised to the rate of the plan found until no plan beats it (the parametric method for a ratio of two linear costs).
#include <algorithm>
#include <vector>

#include "fnx_common.cuh"

namespace fnxb {

static double rows_ms(const fnx_row_cost& c, int from, int to) {   // the price of window rows from + 1 .. to
    double ms = 0.0;
    for (int t = from + 1; t <= to; ++t) ms += t <= c.knee ? c.row_lo : c.row_hi;
    return ms;
}

}  // namespace fnxb

using namespace fnxb;

extern "C" int fnx_plan_rows(int n_lanes, const int* avail, const double* reach, const int* chain, int max_rows, double base_ms, const fnx_row_cost* cost,
                             int* drafts, double* rate_out) {
    FNX_REQUIRE(avail && reach && drafts && cost, "fnx_plan_rows: null pointer");
    FNX_REQUIRE(n_lanes >= 1 && n_lanes <= FNX_MAX_ROWS && max_rows >= n_lanes && max_rows <= FNX_MAX_ROWS, "fnx_plan_rows: %d lanes in %d rows", n_lanes, max_rows);
    FNX_REQUIRE(base_ms > 0.0, "fnx_plan_rows: the window's base cost must be positive");
    constexpr int MAXD = FNX_LANE_ROWS - 1;   // drafts a lane can carry
    const int room = max_rows - n_lanes;
    // gain[i][k], call[i][k]: expected tokens and chain calls' ms of lane i's first k drafts
    std::vector<double> gain((size_t) n_lanes * (MAXD + 1), 0.0), call((size_t) n_lanes * (MAXD + 1), 0.0);
    std::vector<int> most((size_t) n_lanes, 0);
    for (int i = 0; i < n_lanes; ++i) {
        FNX_REQUIRE(avail[i] >= 0, "fnx_plan_rows: lane %d offers %d drafts", i, avail[i]);
        most[i] = std::min(std::min(avail[i], MAXD), room);
        for (int k = 1; k <= most[i]; ++k) {
            const double r = reach[(size_t) i * MAXD + k - 1];
            FNX_REQUIRE(r >= 0.0 && r <= 1.0 && (k == 1 || r <= reach[(size_t) i * MAXD + k - 2] + 1e-12), "fnx_plan_rows: lane %d's reach is not a non-increasing probability", i);
            gain[(size_t) i * (MAXD + 1) + k] = gain[(size_t) i * (MAXD + 1) + k - 1] + r;
            call[(size_t) i * (MAXD + 1) + k] = chain && chain[i] ? (k - 1) * cost->chain_ms : 0.0;
        }
    }
    auto rate_of = [&](const int* d) {
        double tokens = n_lanes, ms = base_ms;
        int t = 0;
        for (int i = 0; i < n_lanes; ++i) {
            tokens += gain[(size_t) i * (MAXD + 1) + d[i]];
            ms += call[(size_t) i * (MAXD + 1) + d[i]];
            t += d[i];
        }
        return tokens / (ms + rows_ms(*cost, n_lanes, n_lanes + t));
    };
    std::vector<int> best((size_t) n_lanes, 0), cand((size_t) n_lanes, 0);
    double lam = rate_of(best.data());
    const double NEG = -1e300;
    std::vector<double> f((size_t) (n_lanes + 1) * (room + 1));
    std::vector<int> pick((size_t) (n_lanes + 1) * (room + 1));
    for (int round = 0; round < 64; ++round) {
        std::fill(f.begin(), f.end(), NEG);
        f[0] = 0.0;
        for (int i = 0; i < n_lanes; ++i)
            for (int t = 0; t <= room; ++t) {
                const double have = f[(size_t) i * (room + 1) + t];
                if (have == NEG) continue;
                for (int k = 0; k <= most[i] && t + k <= room; ++k) {
                    const double v = have + gain[(size_t) i * (MAXD + 1) + k] - lam * call[(size_t) i * (MAXD + 1) + k];
                    double& slot = f[(size_t) (i + 1) * (room + 1) + t + k];
                    if (v > slot) {
                        slot = v;
                        pick[(size_t) (i + 1) * (room + 1) + t + k] = k;
                    }
                }
            }
        int bt = 0;
        double bv = NEG;
        for (int t = 0; t <= room; ++t) {
            const double have = f[(size_t) n_lanes * (room + 1) + t];
            if (have == NEG) continue;
            const double v = n_lanes + have - lam * (base_ms + rows_ms(*cost, n_lanes, n_lanes + t));
            if (v > bv) {
                bv = v;
                bt = t;
            }
        }
        for (int i = n_lanes, t = bt; i > 0; --i) {
            cand[i - 1] = pick[(size_t) i * (room + 1) + t];
            t -= cand[i - 1];
        }
        const double r = rate_of(cand.data());
        if (r <= lam * (1.0 + 1e-12)) break;
        best = cand;
        lam = r;
    }
    for (int i = 0; i < n_lanes; ++i) drafts[i] = best[i];
    if (rate_out) *rate_out = lam;
    return FNX_OK;
}
