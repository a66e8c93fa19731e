#include "stream_plan.h"

namespace ogle {

namespace {

bool Overlap(const std::vector<MemSpan>& a, const std::vector<MemSpan>& b) {
    for (const MemSpan& x : a)
        for (const MemSpan& y : b)
            if (x.lo < y.hi && y.lo < x.hi) return true;
    return false;
}

}  // namespace

StreamPlan PlanStreamsFor(const std::vector<NodeAccess>& nodes, int streams) {
    const size_t n = nodes.size();
    StreamPlan plan;
    plan.lane.assign(n, 0);
    plan.waits.assign(n, std::vector<int>());
    plan.signals.assign(n, false);
    if (streams <= 1 || n == 0) return plan;
    // direct dependencies, then without those already implied by a later one
    std::vector<std::vector<bool>> anc(n, std::vector<bool>(n, false));
    std::vector<std::vector<int>> deps(n);
    for (size_t i = 0; i < n; ++i) {
        std::vector<int> all;
        for (size_t j = 0; j < i; ++j)
            if (Overlap(nodes[j].writes, nodes[i].reads) || Overlap(nodes[j].writes, nodes[i].writes) ||
                Overlap(nodes[j].reads, nodes[i].writes))
                all.push_back(int(j));
        for (int j : all) {
            anc[i][size_t(j)] = true;
            for (int a = 0; a < j; ++a)
                if (anc[size_t(j)][size_t(a)]) anc[i][size_t(a)] = true;
        }
        for (int j : all) {
            bool implied = false;
            for (int k : all)
                if (k > j && anc[size_t(k)][size_t(j)]) { implied = true; break; }
            if (!implied) deps[i].push_back(j);
        }
    }
    std::vector<int> tail(size_t(streams), -1);
    for (size_t i = 0; i < n; ++i) {
        int best = -1;
        for (int l = 0; l < streams; ++l) {
            bool is_dep = false;
            for (int j : deps[i]) is_dep = is_dep || j == tail[size_t(l)];
            if (is_dep && (best < 0 || tail[size_t(l)] > tail[size_t(best)])) best = l;
        }
        if (best < 0) {
            best = 0;
            for (int l = 1; l < streams; ++l)
                if (tail[size_t(l)] < tail[size_t(best)]) best = l;
            if (i > 0) ++plan.branches;
        }
        plan.lane[i] = best;
        for (int j : deps[i]) {
            if (plan.lane[size_t(j)] == best) continue;     // same stream: ordered by the stream itself
            plan.waits[i].push_back(j);
            plan.signals[size_t(j)] = true;
        }
        tail[size_t(best)] = int(i);
    }
    return plan;
}

}  // namespace ogle
