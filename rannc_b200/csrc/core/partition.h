// Automatic partitioning: multi-level coarsening of the operator graph followed
// by a dynamic-programming search over (stage boundaries x devices x pipeline
// depth).  Same structure as the reference's MLPartitioner + DPStaging
// (src/graph/Partitioner.cpp:875-939, src/graph/DPStaging.cpp:295-792) with an
// additive, measured cost model instead of running every candidate on the GPU.
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

#include "ir.h"
#include "profile.h"

namespace rannc {

// ---- multi-level graph (reference: src/graph/MLGraph.h:14-99) -------------
struct MLBaseEdge {
    std::string src_id, tgt_id, value;
    mp::Value pack() const;
    static MLBaseEdge unpack(const mp::Value& v);
};
struct MLEdge {
    std::string src_id, tgt_id;
    std::vector<MLBaseEdge> base_edges;  // value-level edges this edge stands for
    mp::Value pack() const;
    static MLEdge unpack(const mp::Value& v);
};
struct MLNode {
    std::string id;
    IRGraph graph;                        // operators of this node (empty for the nodes of lower levels)
    std::vector<std::string> sub_nodes;   // ids of the operators merged into it
    std::vector<MLNode> children;         // the nodes of the level below that were merged into this one
    int level = 0;                        // 0: an atomic block (one batch / criterion operator)
    mp::Value pack() const;
    static MLNode unpack(const mp::Value& v);
};
struct MLGraph {
    std::vector<MLNode> nodes;  // topological order after sortMLGraph
    std::vector<MLEdge> edges;
    int level() const;          // the highest level among the nodes
    mp::Value pack() const;
    static MLGraph unpack(const mp::Value& v);
};

// One level down: every node is replaced by its children (a node without children stays); edges are
// rebuilt from the operator graph `g` (reference: toLowerLevel, src/graph/MLGraph.cpp).
MLGraph toLowerLevel(const IRGraph& g, const MLGraph& ml);
// One level up: `groups[k]` lists the indices of the nodes of `ml` that become node k of the result, which
// keeps them as its children (reference: liftUp, src/graph/MLGraph.cpp).  The groups must partition the nodes.
MLGraph liftUp(const IRGraph& g, const MLGraph& ml, const std::vector<std::vector<int>>& groups);
// Sum over the edges of the bytes of the values that cross between nodes.
int64_t cutBytes(const IRGraph& g, const MLGraph& ml);

// Cuts `g` by a node -> part label into per-part IRGraphs.  Non-batch nodes are
// copied into every part that consumes them (reference: fixNonBatchRanks,
// Decomposition.cpp:1230-1287).  Parts are returned in label order.
std::vector<IRGraph> createSubGraphs(const IRGraph& g, const std::vector<int>& label, int num_parts,
                                     const std::string& prefix);
// Merges consecutive subgraphs [first, last] of a partition of `g`.
IRGraph mergeSubGraphs(const IRGraph& g, const std::vector<IRGraph>& parts, int first, int last,
                       const std::string& name);

class MLPartitioner {
public:
    MLPartitioner(const ProfileModel& pm, const PartitioningConf& conf) : pm_(pm), conf_(conf) {}
    MLGraph partition();  // atomic blocks -> coarsen -> (uncoarsen) -> sort -> mergeSmall
    int levels() const { return levels_; }
    int moves() const { return moves_; }          // boundary moves made by the uncoarsening passes
    int64_t cutBefore() const { return cut_before_; }
    int64_t cutAfter() const { return cut_after_; }

private:
    const ProfileModel& pm_;
    PartitioningConf conf_;
    int levels_ = 0;
    int moves_ = 0;
    int64_t cut_before_ = 0, cut_after_ = 0;
};

// ---- stage search ---------------------------------------------------------
struct AllocSolution {
    std::vector<IRGraph> graphs;           // one per stage, in pipeline order
    std::unordered_map<std::string, int> repl_nums;
    int pipeline_num = 1;
    bool checkpointing = false;
    std::vector<int> boundaries;           // index of the first ML node of each stage, plus the end
    std::vector<int> dev_nums;             // devices per stage
    double est_time_us = 0;
    mp::Value pack() const;
    static AllocSolution unpack(const mp::Value& v);
};

struct StageEstimate {
    std::string name;
    int repl = 1;
    int64_t micro_batch = 0;
    GraphProfile profile;
    double allreduce_us = 0, in_comm_us = 0, out_comm_us = 0;
    int64_t total_mem = 0, opt_mem = 0, comm_mem = 0;
};

class DPStaging {
public:
    DPStaging(const ProfileModel& pm, const MLGraph& ml, const PartitioningConf& conf)
        : pm_(pm), ml_(ml), conf_(conf) {}
    // throws std::runtime_error when nothing fits in memory
    AllocSolution run();
    const std::vector<StageEstimate>& estimates() const { return estimates_; }
    std::string dumpNodeProfiles() const;  // JSON (reference: DPStaging.cpp:172-238)

private:
    bool runOnce(int stage_num, int pipeline_num, bool checkpointing, AllocSolution* sol,
                 std::vector<StageEstimate>* est);
    const ProfileModel& pm_;
    const MLGraph& ml_;
    PartitioningConf conf_;
    std::vector<StageEstimate> estimates_;
};

// Fixed-shape alternative: split the topological order by cumulative value
// bytes (reference: src/graph/FairWeightDecomposer.cpp:116-230).
AllocSolution fairWeightDecompose(const ProfileModel& pm, const PartitioningConf& conf);

// DP re-run from a dumped cache, without a GPU (reference: DPStaging.cpp:820-881).
struct DPStagingCache {
    MLGraph graph;
    IRGraph ir_graph;
    std::unordered_map<std::string, NodeProfile> node_profiles;
    PartitioningConf conf;
    mp::Value pack() const;
    static DPStagingCache unpack(const mp::Value& v);
};
AllocSolution runDpDry(const DPStagingCache& cache);

}  // namespace rannc
