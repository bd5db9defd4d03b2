#include "profile.h"

#include "runtime_util.h"

#include <algorithm>
#include <cmath>
#include <functional>

namespace rannc {

// ---------------------------------------------------------------- GraphProfile
mp::Value GraphProfile::pack() const {
    auto I = [](int64_t v) { return mp::Value::integer(v); };
    return mp::Value::array({mp::Value::str(name), I(fwd_time), I(fwd_cpu_time), I(fwd_cuda_time), I(bwd_time),
                             I(bwd_cpu_time), I(bwd_cuda_time), I(max_allocated_mem), I(param_size), I(input_size),
                             I(output_size), I(working_mem), I(activation_size), mp::Value::boolean(checkpointing)});
}
GraphProfile GraphProfile::unpack(const mp::Value& v) {
    GraphProfile p;
    p.name = v.at(0).as_str();
    p.fwd_time = v.at(1).as_int();
    p.fwd_cpu_time = v.at(2).as_int();
    p.fwd_cuda_time = v.at(3).as_int();
    p.bwd_time = v.at(4).as_int();
    p.bwd_cpu_time = v.at(5).as_int();
    p.bwd_cuda_time = v.at(6).as_int();
    p.max_allocated_mem = v.at(7).as_int();
    p.param_size = v.at(8).as_int();
    p.input_size = v.at(9).as_int();
    p.output_size = v.at(10).as_int();
    p.working_mem = v.at(11).as_int();
    p.activation_size = v.at(12).as_int();
    p.checkpointing = v.at(13).as_bool();
    return p;
}

// ---------------------------------------------------------------- PartitioningConf
mp::Value PartitioningConf::pack() const {
    auto I = [](int64_t v) { return mp::Value::integer(v); };
    auto B = [](bool v) { return mp::Value::boolean(v); };
    return mp::Value::array({I(dev_num), I(batch_size), I(dev_mem), B(use_amp_master_params), B(enable_zero),
                             I(opt_param_factor), I(min_pipeline), I(max_pipeline), I(min_partition_num),
                             I(max_partition_num), I(cfg_partition_num), I(cfg_replica_num), I(cfg_pipeline_num),
                             B(offload_params), B(force_dist_matmul)});
}
PartitioningConf PartitioningConf::unpack(const mp::Value& v) {
    PartitioningConf c;
    c.dev_num = static_cast<int>(v.at(0).as_int());
    c.batch_size = v.at(1).as_int();
    c.dev_mem = v.at(2).as_int();
    c.use_amp_master_params = v.at(3).as_bool();
    c.enable_zero = v.at(4).as_bool();
    c.opt_param_factor = static_cast<int>(v.at(5).as_int());
    c.min_pipeline = static_cast<int>(v.at(6).as_int());
    c.max_pipeline = static_cast<int>(v.at(7).as_int());
    c.min_partition_num = static_cast<int>(v.at(8).as_int());
    c.max_partition_num = static_cast<int>(v.at(9).as_int());
    c.cfg_partition_num = static_cast<int>(v.at(10).as_int());
    c.cfg_replica_num = static_cast<int>(v.at(11).as_int());
    c.cfg_pipeline_num = static_cast<int>(v.at(12).as_int());
    c.offload_params = v.at(13).as_bool();
    c.force_dist_matmul = v.at(14).as_bool();
    return c;
}

// ---------------------------------------------------------------- ProfileModel
ProfileModel::ProfileModel(const IRGraph& g, std::unordered_map<std::string, NodeProfile> np, LinkModel link)
    : g_(g), np_(std::move(np)), link_(link) {}

const NodeProfile* ProfileModel::nodeProfile(const std::string& id) const {
    auto it = np_.find(id);
    return it == np_.end() ? nullptr : &it->second;
}

bool ProfileModel::measured(const std::vector<std::string>& ids, int64_t bs, bool checkpointing,
                            GraphProfile* out) const {
    if (!measure_ || ids.empty()) return false;
    std::vector<std::string> sorted = ids;
    std::sort(sorted.begin(), sorted.end());
    std::string key = std::to_string(bs) + (checkpointing ? "|c|" : "|n|");
    for (const auto& s : sorted) {
        key += s;
        key += ',';
    }
    auto it = measure_cache_.find(key);
    if (it != measure_cache_.end()) {
        if (it->second.first) *out = it->second.second;
        return it->second.first;
    }
    if (measured_ >= measure_limit_) return false;
    GraphProfile gp;
    bool ok = false;
    try {
        ok = measure_(sorted, bs, checkpointing, &gp);
    } catch (...) {
        ok = false;
    }
    ++measured_;
    measure_cache_[key] = {ok, gp};
    if (ok) *out = gp;
    return ok;
}

bool ProfileModel::measuredSubgraphTime(const std::vector<std::string>& ids, int64_t bs, double* us) const {
    GraphProfile gp;
    if (!measured(ids, bs, false, &gp)) return false;
    *us = static_cast<double>(gp.fwd_time + gp.bwd_time);
    return true;
}

GraphProfile ProfileModel::profile(const IRGraph& sub, int64_t bs, bool checkpointing) const {
    GraphProfile p;
    p.name = sub.name;
    const double ref_bs = static_cast<double>(std::max<int64_t>(1, g_.batch_size));
    const double ratio = static_cast<double>(std::max<int64_t>(1, bs)) / ref_bs;
    double fwd = 0, bwd = 0, act = 0, work = 0;
    for (const auto& n : sub.nodes) {
        const NodeProfile* np = nodeProfile(n.id);
        if (!np) continue;
        const bool scales = np->scales_with_batch && (n.is_batch || n.is_criterion);
        const double r = scales ? ratio : 1.0;
        const double oh = link_.launch_overhead_us;
        fwd += np->fwd_us > oh ? oh + (np->fwd_us - oh) * r : np->fwd_us;
        bwd += np->bwd_us > oh ? oh + (np->bwd_us - oh) * r : np->bwd_us;
        act += static_cast<double>(np->activation_bytes) * r;
        work = std::max(work, static_cast<double>(np->working_bytes) * r);
    }
    IRGraph scaled = scaleGraph(sub, bs > 0 ? bs : sub.batch_size);
    p.param_size = scaled.paramSizeInByte();
    p.input_size = scaled.inputSizeInByte();
    p.output_size = scaled.outputSizeInByte();
    p.checkpointing = checkpointing;
    if (checkpointing) {
        bwd += fwd;  // recompute
    }
    p.fwd_time = static_cast<int64_t>(std::ceil(fwd));
    p.bwd_time = static_cast<int64_t>(std::ceil(bwd));
    p.fwd_cuda_time = p.fwd_time;
    p.bwd_cuda_time = p.bwd_time;
    p.activation_size = static_cast<int64_t>(act);
    p.working_mem = static_cast<int64_t>(work);
    p.max_allocated_mem = p.param_size + p.input_size + p.output_size + p.activation_size + p.working_mem;
    if (measure_) {
        // a measurement of this very subgraph replaces the sums of operator figures: times, and the memory
        // the allocator really needed
        std::vector<std::string> ids;
        for (const auto& n : sub.nodes)
            if (n.is_batch || n.is_criterion) ids.push_back(n.id);
        GraphProfile m;
        if (measured(ids, bs, checkpointing, &m)) {
            p.fwd_time = m.fwd_time;
            p.bwd_time = m.bwd_time;
            p.fwd_cuda_time = m.fwd_cuda_time ? m.fwd_cuda_time : m.fwd_time;
            p.bwd_cuda_time = m.bwd_cuda_time ? m.bwd_cuda_time : m.bwd_time;
            p.fwd_cpu_time = m.fwd_cpu_time;
            p.bwd_cpu_time = m.bwd_cpu_time;
            if (m.activation_size > 0) p.activation_size = m.activation_size;
            if (m.working_mem > 0) p.working_mem = m.working_mem;
            if (m.max_allocated_mem > 0)
                p.max_allocated_mem = std::max<int64_t>(m.max_allocated_mem + p.param_size,
                                                        p.param_size + p.input_size + p.output_size);
        }
    }
    return p;
}

double calcCommTime(const LinkModel& l, int64_t bytes) {
    if (bytes <= 0) return 0;
    return l.latency_us + static_cast<double>(bytes) / l.p2p_bytes_per_us;
}

double calcAllReduceTime(const LinkModel& l, int64_t bytes, int nranks) {
    if (bytes <= 0 || nranks <= 1) return 0;
    // bus-bandwidth convention: time = bytes * 2(n-1)/n / busbw
    const double factor = 2.0 * (nranks - 1) / nranks;
    return l.latency_us + static_cast<double>(bytes) * factor / l.allreduce_bytes_per_us;
}

// Bytes of the device window through which 16-bit parameters and their gradients are streamed from host memory
// (offload_params with offload_param_window_mb > 0); 0: they are resident.
static int64_t paramWindowBytes(const PartitioningConf& conf) {
    if (!conf.offload_params || !conf.use_amp_master_params) return 0;
    return std::max<int64_t>(0, Config::get().getInt("offload_param_window_mb")) << 20;
}

int64_t getOptMemSize(const IRGraph& g, const PartitioningConf& conf, int zero_ranks) {
    const int z = conf.enable_zero ? std::max(1, zero_ranks) : 1;
    const bool streamed = paramWindowBytes(conf) > 0;
    int64_t total = 0;
    for (const auto& n : g.input_names) {
        const IRValue& v = g.value(n);
        if (!v.is_param || !v.type.holdsGradient()) continue;
        const int64_t sz = v.type.sizeInByte();
        const bool half = v.type.tensor_elem_type == IRTensorElemType::HALF ||
                          v.type.tensor_elem_type == IRTensorElemType::BFLOAT16;
        if (conf.use_amp_master_params && half) {
            // fp32 gradient buffer (whole), fp32 master copy and optimizer state (sharded under ZeRO);
            // with offload_params the master copy and the optimizer state live in pinned host memory and
            // only a fixed staging window is on the device
            if (!streamed) total += 2 * sz;   // streamed: the gradients live on the host too
            if (!conf.offload_params) {
                total += (2 * sz) / z;
                total += (static_cast<int64_t>(conf.opt_param_factor) * 2 * sz) / z;
            }
        } else {
            total += sz;  // gradient
            total += (static_cast<int64_t>(conf.opt_param_factor) * sz) / z;
        }
    }
    return total;
}

int64_t calcGraphMem(const IRGraph& g, const GraphProfile& prof, const PartitioningConf& conf, int repl,
                     int pipeline_num, bool checkpointing) {
    const int64_t opt = getOptMemSize(g, conf, repl);
    const int64_t P = std::max(1, pipeline_num);
    const int64_t window = paramWindowBytes(conf);
    if (window > 0 && prof.param_size > 0) {
        // streamed parameters: two segments' parameters (half a window each) and one segment's fp32 gradients
        // are on the device; the stage recomputes segment by segment, keeping the inputs of every segment for
        // every micro-batch in flight
        const int64_t half = std::max<int64_t>(1, window / 2);
        const int64_t nseg = std::max<int64_t>(1, (prof.param_size + half - 1) / half);
        const int64_t params = std::min(prof.param_size, window) + std::min(2 * prof.param_size, window);
        const int64_t act_s = P * prof.input_size * nseg + prof.activation_size / nseg;
        IRGraph scaled_s = g;
        return params + act_s + prof.working_mem + opt + scaled_s.commBufSize() * std::min<int64_t>(P, 2);
    }
    int64_t act;
    const int64_t segs = Config::get().getInt("checkpoint_segments");
    if (checkpointing && segs > 1) {
        // recomputation segment by segment: the values at the segment boundaries (about a stage input each) of
        // every in-flight micro-batch + one segment's activations of one micro-batch
        act = P * segs * prof.input_size + prof.activation_size / segs;
    } else if (checkpointing) {
        // stage inputs of every in-flight micro-batch + one micro-batch's activations
        act = P * prof.input_size + prof.activation_size;
    } else {
        act = P * prof.activation_size;
    }
    // comm buffers are per micro-batch in flight (inputs, outputs and their gradients stay on the device)
    IRGraph scaled = g;
    const int64_t comm = scaled.commBufSize();
    return prof.param_size + act + prof.working_mem + opt + comm * std::min<int64_t>(P, 2);
}

// ---------------------------------------------------------------- profile DB
mp::Value ProfileItemKey::pack() const {
    mp::MapItems gs;
    std::vector<std::string> keys;
    for (const auto& kv : ir_graphs) keys.push_back(kv.first);
    std::sort(keys.begin(), keys.end());
    for (const auto& k : keys) gs.emplace_back(mp::Value::str(k), ir_graphs.at(k).pack());
    mp::MapItems rs;
    keys.clear();
    for (const auto& kv : repl_nums) keys.push_back(kv.first);
    std::sort(keys.begin(), keys.end());
    for (const auto& k : keys) rs.emplace_back(mp::Value::str(k), mp::Value::integer(repl_nums.at(k)));
    return mp::Value::array({mp::Value::mapping(std::move(gs)), mp::Value::integer(batch_size),
                             mp::Value::mapping(std::move(rs)), mp::Value::integer(iteration),
                             mp::Value::boolean(checkpointing)});
}
ProfileItemKey ProfileItemKey::unpack(const mp::Value& v) {
    ProfileItemKey k;
    for (const auto& kv : v.at(0).as_map()) k.ir_graphs[kv.first.as_str()] = IRGraph::unpack(kv.second);
    k.batch_size = v.at(1).as_int();
    for (const auto& kv : v.at(2).as_map()) k.repl_nums[kv.first.as_str()] = static_cast<int>(kv.second.as_int());
    k.iteration = static_cast<int>(v.at(3).as_int());
    k.checkpointing = v.at(4).as_bool();
    return k;
}
uint64_t ProfileItemKey::hash() const {
    // hash of the printed graphs + batch size + iterations + checkpointing
    std::vector<std::string> keys;
    for (const auto& kv : ir_graphs) keys.push_back(kv.first);
    std::sort(keys.begin(), keys.end());
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](const std::string& s) {
        for (unsigned char c : s) {
            h ^= c;
            h *= 1099511628211ull;
        }
    };
    for (const auto& k : keys) mix(ir_graphs.at(k).toString());
    mix(std::to_string(batch_size));
    mix(std::to_string(iteration));
    mix(checkpointing ? "c1" : "c0");
    return h;
}
mp::Value ProfilingResult::pack() const {
    mp::MapItems ps, ts;
    std::vector<std::string> keys;
    for (const auto& kv : node_profiles) keys.push_back(kv.first);
    std::sort(keys.begin(), keys.end());
    for (const auto& k : keys) ps.emplace_back(mp::Value::str(k), node_profiles.at(k).pack());
    keys.clear();
    for (const auto& kv : value_types) keys.push_back(kv.first);
    std::sort(keys.begin(), keys.end());
    for (const auto& k : keys) ts.emplace_back(mp::Value::str(k), value_types.at(k).pack());
    return mp::Value::array({mp::Value::mapping(std::move(ps)), mp::Value::mapping(std::move(ts))});
}
ProfilingResult ProfilingResult::unpack(const mp::Value& v) {
    ProfilingResult r;
    for (const auto& kv : v.at(0).as_map()) r.node_profiles[kv.first.as_str()] = GraphProfile::unpack(kv.second);
    for (const auto& kv : v.at(1).as_map()) r.value_types[kv.first.as_str()] = IRType::unpack(kv.second);
    return r;
}
void ProfileDB::add(const ProfileItemKey& key, const ProfilingResult& res) { items_[key.hash()] = {key, res}; }
bool ProfileDB::get(const ProfileItemKey& key, ProfilingResult* out) const {
    auto it = items_.find(key.hash());
    if (it == items_.end()) return false;
    if (out) *out = it->second.second;
    return true;
}
std::string ProfileDB::dumps() const {
    mp::MapItems m;
    std::vector<uint64_t> keys;
    for (const auto& kv : items_) keys.push_back(kv.first);
    std::sort(keys.begin(), keys.end());
    for (auto k : keys) {
        const auto& it = items_.at(k);
        m.emplace_back(mp::Value::uinteger(k), mp::Value::array({it.first.pack(), it.second.pack()}));
    }
    return mp::pack(mp::Value::mapping(std::move(m)));
}
void ProfileDB::loads(const std::string& data) {
    items_.clear();
    mp::Value v = mp::unpack(data);
    for (const auto& kv : v.as_map())
        items_[kv.first.as_uint()] = {ProfileItemKey::unpack(kv.second.at(0)), ProfilingResult::unpack(kv.second.at(1))};
}

}  // namespace rannc
