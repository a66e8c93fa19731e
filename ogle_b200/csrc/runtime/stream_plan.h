// Stream plan of a node sequence: which stream each node is recorded on and which nodes on
// other streams it has to wait for, from the memory spans the nodes read and write. Pure
// host logic (no CUDA calls), used by FBOSession when it captures its graph. The reference
// runs its nodes strictly in file order (ogl_runtime/opengl/core/fbo_session.cc:127-156).
#ifndef OGLE_RUNTIME_STREAM_PLAN_H_
#define OGLE_RUNTIME_STREAM_PLAN_H_

#include <cstdint>
#include <vector>

namespace ogle {

struct MemSpan {
    uintptr_t lo, hi;      // [lo, hi)
};

struct NodeAccess {
    std::vector<MemSpan> reads, writes;
};

struct StreamPlan {
    std::vector<int> lane;                  // stream of each node, 0 = the main stream
    std::vector<std::vector<int>> waits;    // earlier nodes on other streams to wait for
    std::vector<bool> signals;              // some node on another stream waits for this one
    int branches = 0;                       // nodes that did not continue a predecessor's stream
};

// Node i depends on an earlier node j when j writes what i reads or writes, or reads what i
// writes; dependencies implied by a later dependency are dropped. A node continues the stream
// whose last node it depends on (the most recent such); otherwise it starts a branch on the
// stream that has been idle longest. streams <= 1 gives a chain on stream 0.
StreamPlan PlanStreamsFor(const std::vector<NodeAccess>& nodes, int streams);

}  // namespace ogle

#endif
