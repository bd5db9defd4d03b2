// Deployment: which stage runs on which ranks, and the routes that move values
// between stages and between the caller ("MASTER") and the stages.
//
// Same content and msgpack layout as the reference's Deployment / RouteDP /
// DeploymentState (src/graph/Decomposition.h:156-183, src/comm/SCommCommon.h:20-94,
// src/graph/DeploymentSerializer.h:11-26), so a saved partitioning can be shown,
// reloaded and re-used.
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "ir.h"
#include "partition.h"

namespace rannc {

enum class RouteTypeDP : int {
    P2P = 0, REDIST, SCATTER, GATHER, REDUCE, WEIGHTED_REDUCE, BROADCAST, SCATTER_ANY, ALL_GATHER, ANY,
    ANY_TO_ALL, NA
};

struct RouteDP {
    IValueLocation location;
    std::vector<int> sources;
    std::string source_graph;
    int source_order = 0;
    std::vector<int> dests;
    std::string dest_graph;
    int dest_order = 0;
    int tag = 0;
    int source_tag = 0;
    RouteTypeDP type = RouteTypeDP::NA;
    IRValue ir_value;
    mp::Value pack() const;
    static RouteDP unpack(const mp::Value& v);
};

// per-stage description of tensor-partitioned (distop) parameters
// (reference: src/distop/PartitionTensor.h:40-42)
struct TensorPartitioningGraphInfo {
    IRGraph graph;
    std::vector<int> ranks;
    std::unordered_map<std::string, std::pair<int, int>> param_partitions;  // name -> (arg index, dim)
    std::vector<std::string> rank_values;
    std::unordered_map<std::string, int> dim_values;
    std::unordered_map<std::string, std::string> rank_value_names;
    mp::Value pack() const;
    static TensorPartitioningGraphInfo unpack(const mp::Value& v);
};

struct Deployment {
    std::string id;
    IRGraph graph;
    std::unordered_map<std::string, IRGraph> subgraphs;
    std::unordered_map<std::string, std::vector<int>> allocation;  // stage -> ranks
    std::unordered_map<std::string, TensorPartitioningGraphInfo> part_info;
    std::vector<RouteDP> fwd_routes, fwd_in_routes, fwd_out_routes;
    std::vector<std::string> fwd_graph_order;
    std::vector<RouteDP> bwd_routes, bwd_in_routes, bwd_out_routes;
    std::vector<std::string> bwd_graph_order;
    int pipeline_num = 1;
    bool checkpointing = false;
    bool offload_params = false;
    bool force_dist_matmul = false;
    mp::Value pack() const;
    static Deployment unpack(const mp::Value& v);
    std::string toString() const;
};

struct DeploymentState {
    Deployment deployment;
    int world_size = 1;
    int64_t dev_mem = 0;
    std::string dumps() const;
    static DeploymentState loads(const std::string& data);
};

// rank assignment (reference: Decomposition.cpp:1109-1225)
std::unordered_map<std::string, std::vector<int>> searchAllocationFlat(
    const std::vector<std::string>& order, const std::unordered_map<std::string, int>& repl_nums, int dev_num);
std::unordered_map<std::string, std::vector<int>> searchAllocationSimple(
    const std::vector<std::string>& order, const std::unordered_map<std::string, int>& repl_nums, int dev_num);

// stable tag of a rank set, used as the key of a communicator
// (reference: TagMap, src/comm/SComm.h:32-76)
int tagOfRanks(const std::vector<int>& ranks);

// Builds the deployment (subgraphs scaled to the replica micro-batch, routes,
// orders) from a stage solution.  `gather_inputs = false` makes rank 0 the only
// MASTER endpoint (reference: GraphLauncher.cpp:41-57).
Deployment createDeployment(const IRGraph& graph, const AllocSolution& sol, int dev_num, bool alloc_repl_flat,
                            const std::string& id);
// Every subgraph input / output must have a forward route, and a backward
// route when it carries a gradient (reference: Decomposition.cpp:1348-1429).
// Returns an empty string when the deployment is consistent, else the reason.
std::string verifyDeployment(const Deployment& d);

// ---- batch arithmetic (reference: src/comp/BatchSizeCalculator.cpp:19-175) ----
class BatchSizeCalculator {
public:
    BatchSizeCalculator(int pipeline_num, int64_t global_batch) : P_(pipeline_num), B_(global_batch) {}
    // size of micro-batch `split`: floor(B/P) (+1 for the first B mod P splits)
    int64_t splitSize(int split) const;
    // rows rank index `idx` of `n` sorted ranks gets from micro-batch `split`; the "+1"s rotate
    // by the sum of the previous split sizes
    int64_t localSplitSize(int idx, int n, int split) const;
    // sum over all splits for a rank
    int64_t localBatchSize(int idx, int n) const;
    // rows per rank for a tensor whose first dimension is `dim0` for the whole global batch
    std::vector<int64_t> localDims(int64_t dim0, int n, int split) const;

private:
    int P_;
    int64_t B_;
};

struct RedistArgs {
    std::vector<int64_t> sendcounts, recvcounts, sdispls, rdispls;  // rows, indexed by global rank
};
// Contiguous-row all-to-all-v plan between the rank set that holds a tensor and
// the rank set that needs it (reference: src/comm/SComm.cpp:16-177,465-524).
RedistArgs getRedistArgs(int my_rank, int world_size, int64_t total_rows, const std::vector<int>& src_ranks,
                         const std::vector<int>& dst_ranks, int split, int pipeline_num, int64_t global_batch);

// ---- ZeRO / dist_param segment math (reference: TorchUtil.cpp:1579-1591,
//      DistributedParamLocatorBase.cpp:14-46) ----
int64_t alignedNumel(int64_t numel, int elem_size, int nranks);
// [begin, end) element range of rank index `idx`, clipped to numel (may be empty)
std::pair<int64_t, int64_t> segmentRange(int64_t numel, int elem_size, int nranks, int idx);

}  // namespace rannc
