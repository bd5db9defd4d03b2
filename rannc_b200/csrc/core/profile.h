// Profiles and the cost model the partitioner plans with.
//
// The reference measures every candidate subgraph by running it on the GPU
// (src/comp/GraphProfiler.cpp:245-415) and assumes fixed link speeds of
// 20 GiB/s between stages and 10 GiB/s for all-reduce
// (src/graph/ProfilerUtil.cpp:37-53).  Here each operator node is profiled
// once (measured with CUDA events on the sm_100a kernels, or estimated from a
// roofline when no GPU is present) and subgraph profiles are accumulated from
// node profiles, scaled to the micro-batch size.  Link constants default to
// what NVLink 5 / NVSwitch delivers on an 8 x B200 box and are configurable.
#pragma once
#include <cstdint>
#include <functional>
#include <string>
#include <unordered_map>
#include <vector>

#include "ir.h"

namespace rannc {

// Serialised field order follows the reference (src/comp/GraphProfiler.h:54-57,133-160).
struct GraphProfile {
    std::string name;
    int64_t fwd_time = 0, fwd_cpu_time = 0, fwd_cuda_time = 0;  // microseconds
    int64_t bwd_time = 0, bwd_cpu_time = 0, bwd_cuda_time = 0;
    int64_t max_allocated_mem = 0;
    int64_t param_size = 0, input_size = 0, output_size = 0;
    int64_t working_mem = 0, activation_size = 0;
    bool checkpointing = false;
    mp::Value pack() const;
    static GraphProfile unpack(const mp::Value& v);
};

// What is known about one operator node at the graph's reference batch size.
struct NodeProfile {
    double fwd_us = 0, bwd_us = 0;
    int64_t activation_bytes = 0;  // tensors kept for the backward
    int64_t working_bytes = 0;     // transient workspace
    bool scales_with_batch = true;
};

struct LinkModel {
    double p2p_bytes_per_us = 770e3;        // stage <-> stage, one direction (770 GB/s measured peer copy)
    double allreduce_bytes_per_us = 725e3;  // bus bandwidth of an 8-rank all-reduce (725 GB/s measured)
    double latency_us = 8.0;                // per transfer / collective launch
    double launch_overhead_us = 4.0;        // part of a node's time that does not scale with batch
};

struct PartitioningConf {
    int dev_num = 1;
    int64_t batch_size = 1;
    int64_t dev_mem = 0;          // bytes usable per device (after the margin)
    bool use_amp_master_params = false;
    bool enable_zero = false;
    bool offload_params = false;
    bool force_dist_matmul = false;
    int opt_param_factor = 2;
    int min_pipeline = 1, max_pipeline = 32;
    int min_pipeline_bs = 1;
    int min_partition_num = 5, max_partition_num = 32;
    int cfg_partition_num = 0, cfg_replica_num = 0, cfg_pipeline_num = 0;
    bool limit_dev_num_pot = true;
    bool limit_dev_num_more_than_bs = true;
    bool dp_search_all = false;
    bool do_coarsening = true, do_uncoarsening = false, coarsen_by_time = true;
    bool checkpointing = false;          // force recompute
    bool checkpointing_no_last = false;
    bool prefer_no_checkpointing = true; // keep activations resident when they fit (180 GB HBM)
    // a plan of ONE stage runs each micro-batch's backward right after its forward (interleave_backward), so
    // only one micro-batch's activations are alive whatever the number of micro-batches
    bool interleave_single_stage = false;
    LinkModel link;
    mp::Value pack() const;
    static PartitioningConf unpack(const mp::Value& v);
};

class ProfileModel {
public:
    ProfileModel(const IRGraph& g, std::unordered_map<std::string, NodeProfile> node_profiles, LinkModel link);
    // profile of the nodes `ids` (indices into graph.nodes) run as one stage at micro-batch `bs`
    GraphProfile profile(const IRGraph& sub, int64_t bs, bool checkpointing) const;
    const IRGraph& graph() const { return g_; }
    const LinkModel& link() const { return link_; }
    const NodeProfile* nodeProfile(const std::string& id) const;

    // Measurement of a whole candidate subgraph (reference: GraphProfiler::computeGraph,
    // src/comp/GraphProfiler.cpp:245-415): given the ids of its operators, the micro-batch size and whether it
    // recomputes, the callback runs forward + backward on the device and fills times (microseconds), the
    // allocator peak, activation and working bytes.  It returns false when it cannot measure (no device, too
    // large), and the additive estimate is used.  Results are cached per (operators, batch, checkpointing), at
    // most `limit` subgraphs are measured per model.
    using SubgraphMeasure =
        std::function<bool(const std::vector<std::string>& node_ids, int64_t bs, bool checkpointing, GraphProfile*)>;
    void setSubgraphMeasure(SubgraphMeasure f, int limit) {
        measure_ = std::move(f);
        measure_limit_ = limit;
    }
    bool hasSubgraphMeasure() const { return static_cast<bool>(measure_); }
    int measuredCount() const { return measured_; }
    // fwd + bwd microseconds of the operators `ids` run as one graph; false: no measurement available
    bool measuredSubgraphTime(const std::vector<std::string>& ids, int64_t bs, double* us) const;

private:
    bool measured(const std::vector<std::string>& ids, int64_t bs, bool checkpointing, GraphProfile* out) const;
    IRGraph g_;
    std::unordered_map<std::string, NodeProfile> np_;
    LinkModel link_;
    SubgraphMeasure measure_;
    int measure_limit_ = 0;
    mutable int measured_ = 0;
    mutable std::unordered_map<std::string, std::pair<bool, GraphProfile>> measure_cache_;
};

// microseconds to move `bytes` between two stages / to all-reduce `bytes` over n ranks
double calcCommTime(const LinkModel& l, int64_t bytes);
double calcAllReduceTime(const LinkModel& l, int64_t bytes, int nranks);
// optimizer + master-copy + gradient memory of a stage (reference: ProfilerUtil.cpp:55-105)
int64_t getOptMemSize(const IRGraph& g, const PartitioningConf& conf, int zero_ranks);
// device memory a stage needs (reference: ProfilerUtil.cpp:120-139)
int64_t calcGraphMem(const IRGraph& g, const GraphProfile& prof, const PartitioningConf& conf, int repl,
                     int pipeline_num, bool checkpointing);

// msgpack-persisted profile cache keyed like the reference's ProfileDB
// (src/comp/GraphProfiler.cpp:18-62,937-963).
struct ProfileItemKey {
    std::unordered_map<std::string, IRGraph> ir_graphs;
    int64_t batch_size = 0;
    std::unordered_map<std::string, int> repl_nums;
    int iteration = 1;
    bool checkpointing = false;
    mp::Value pack() const;
    static ProfileItemKey unpack(const mp::Value& v);
    uint64_t hash() const;
};
struct ProfilingResult {
    std::unordered_map<std::string, GraphProfile> node_profiles;
    std::unordered_map<std::string, IRType> value_types;
    mp::Value pack() const;
    static ProfilingResult unpack(const mp::Value& v);
};
class ProfileDB {
public:
    void add(const ProfileItemKey& key, const ProfilingResult& res);
    bool get(const ProfileItemKey& key, ProfilingResult* out) const;
    size_t size() const { return items_.size(); }
    std::string dumps() const;
    void loads(const std::string& data);

private:
    std::unordered_map<uint64_t, std::pair<ProfileItemKey, ProfilingResult>> items_;
};

}  // namespace rannc
