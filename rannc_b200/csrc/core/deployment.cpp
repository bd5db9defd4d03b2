#include "deployment.h"

#include <algorithm>
#include <numeric>
#include <set>
#include <sstream>
#include <stdexcept>

namespace rannc {

namespace {
mp::Value packIntVec(const std::vector<int>& v) {
    mp::Array a;
    for (int x : v) a.push_back(mp::Value::integer(x));
    return mp::Value::array(std::move(a));
}
std::vector<int> unpackIntVec(const mp::Value& v) {
    std::vector<int> r;
    for (const auto& e : v.as_array()) r.push_back(static_cast<int>(e.as_int()));
    return r;
}
template <typename T, typename F>
mp::Value packStrMap(const std::unordered_map<std::string, T>& m, F f) {
    std::vector<std::string> keys;
    for (const auto& kv : m) keys.push_back(kv.first);
    std::sort(keys.begin(), keys.end());
    mp::MapItems items;
    for (const auto& k : keys) items.emplace_back(mp::Value::str(k), f(m.at(k)));
    return mp::Value::mapping(std::move(items));
}
mp::Value packRoutes(const std::vector<RouteDP>& rs) {
    mp::Array a;
    for (const auto& r : rs) a.push_back(r.pack());
    return mp::Value::array(std::move(a));
}
std::vector<RouteDP> unpackRoutes(const mp::Value& v) {
    std::vector<RouteDP> r;
    for (const auto& e : v.as_array()) r.push_back(RouteDP::unpack(e));
    return r;
}
}  // namespace

// ---------------------------------------------------------------- serialisation
mp::Value RouteDP::pack() const {
    return mp::Value::array({location.pack(), packIntVec(sources), mp::Value::str(source_graph),
                             mp::Value::integer(source_order), packIntVec(dests), mp::Value::str(dest_graph),
                             mp::Value::integer(dest_order), mp::Value::integer(tag), mp::Value::integer(source_tag),
                             mp::Value::integer(static_cast<int>(type)), ir_value.pack()});
}
RouteDP RouteDP::unpack(const mp::Value& v) {
    RouteDP r;
    r.location = IValueLocation::unpack(v.at(0));
    r.sources = unpackIntVec(v.at(1));
    r.source_graph = v.at(2).as_str();
    r.source_order = static_cast<int>(v.at(3).as_int());
    r.dests = unpackIntVec(v.at(4));
    r.dest_graph = v.at(5).as_str();
    r.dest_order = static_cast<int>(v.at(6).as_int());
    r.tag = static_cast<int>(v.at(7).as_int());
    r.source_tag = static_cast<int>(v.at(8).as_int());
    r.type = static_cast<RouteTypeDP>(v.at(9).as_int());
    r.ir_value = IRValue::unpack(v.at(10));
    return r;
}

mp::Value TensorPartitioningGraphInfo::pack() const {
    mp::MapItems pp;
    std::vector<std::string> keys;
    for (const auto& kv : param_partitions) keys.push_back(kv.first);
    std::sort(keys.begin(), keys.end());
    for (const auto& k : keys)
        pp.emplace_back(mp::Value::str(k), mp::Value::array({mp::Value::integer(param_partitions.at(k).first),
                                                            mp::Value::integer(param_partitions.at(k).second)}));
    return mp::Value::array({graph.pack(), packIntVec(ranks), mp::Value::mapping(std::move(pp)),
                             packStrings(rank_values),
                             packStrMap(dim_values, [](int x) { return mp::Value::integer(x); }),
                             packStrMap(rank_value_names, [](const std::string& s) { return mp::Value::str(s); })});
}
TensorPartitioningGraphInfo TensorPartitioningGraphInfo::unpack(const mp::Value& v) {
    TensorPartitioningGraphInfo t;
    t.graph = IRGraph::unpack(v.at(0));
    t.ranks = unpackIntVec(v.at(1));
    for (const auto& kv : v.at(2).as_map())
        t.param_partitions[kv.first.as_str()] = {static_cast<int>(kv.second.at(0).as_int()),
                                                 static_cast<int>(kv.second.at(1).as_int())};
    t.rank_values = unpackStrings(v.at(3));
    for (const auto& kv : v.at(4).as_map()) t.dim_values[kv.first.as_str()] = static_cast<int>(kv.second.as_int());
    for (const auto& kv : v.at(5).as_map()) t.rank_value_names[kv.first.as_str()] = kv.second.as_str();
    return t;
}

mp::Value Deployment::pack() const {
    return mp::Value::array(
        {mp::Value::str(id), graph.pack(), packStrMap(subgraphs, [](const IRGraph& g) { return g.pack(); }),
         packStrMap(allocation, [](const std::vector<int>& r) { return packIntVec(r); }),
         packStrMap(part_info, [](const TensorPartitioningGraphInfo& t) { return t.pack(); }),
         packRoutes(fwd_routes), packRoutes(fwd_in_routes), packRoutes(fwd_out_routes),
         packStrings(fwd_graph_order), packRoutes(bwd_routes), packRoutes(bwd_in_routes),
         packRoutes(bwd_out_routes), packStrings(bwd_graph_order), mp::Value::integer(pipeline_num),
         mp::Value::boolean(checkpointing), mp::Value::boolean(offload_params),
         mp::Value::boolean(force_dist_matmul)});
}
Deployment Deployment::unpack(const mp::Value& v) {
    Deployment d;
    d.id = v.at(0).as_str();
    d.graph = IRGraph::unpack(v.at(1));
    for (const auto& kv : v.at(2).as_map()) d.subgraphs[kv.first.as_str()] = IRGraph::unpack(kv.second);
    for (const auto& kv : v.at(3).as_map()) d.allocation[kv.first.as_str()] = unpackIntVec(kv.second);
    for (const auto& kv : v.at(4).as_map())
        d.part_info[kv.first.as_str()] = TensorPartitioningGraphInfo::unpack(kv.second);
    d.fwd_routes = unpackRoutes(v.at(5));
    d.fwd_in_routes = unpackRoutes(v.at(6));
    d.fwd_out_routes = unpackRoutes(v.at(7));
    d.fwd_graph_order = unpackStrings(v.at(8));
    d.bwd_routes = unpackRoutes(v.at(9));
    d.bwd_in_routes = unpackRoutes(v.at(10));
    d.bwd_out_routes = unpackRoutes(v.at(11));
    d.bwd_graph_order = unpackStrings(v.at(12));
    d.pipeline_num = static_cast<int>(v.at(13).as_int());
    d.checkpointing = v.at(14).as_bool();
    d.offload_params = v.at(15).as_bool();
    d.force_dist_matmul = v.at(16).as_bool();
    return d;
}

std::string Deployment::toString() const {
    std::ostringstream ss;
    ss << "deployment " << id << ": " << fwd_graph_order.size() << " stage(s), pipeline_num=" << pipeline_num
       << ", checkpointing=" << (checkpointing ? "true" : "false") << "\n";
    for (const auto& name : fwd_graph_order) {
        const IRGraph& sg = subgraphs.at(name);
        ss << "  " << name << ": " << sg.nodes.size() << " nodes, params " << sg.paramSizeInByte()
           << " B, in " << sg.inputSizeInByte() << " B, out " << sg.outputSizeInByte() << " B, ranks [";
        const auto& rs = allocation.at(name);
        for (size_t i = 0; i < rs.size(); ++i) ss << (i ? "," : "") << rs[i];
        ss << "]\n";
    }
    ss << "  routes: fwd " << fwd_routes.size() << " / in " << fwd_in_routes.size() << " / out "
       << fwd_out_routes.size() << "; bwd " << bwd_routes.size() << " / in " << bwd_in_routes.size() << " / out "
       << bwd_out_routes.size() << "\n";
    return ss.str();
}

std::string DeploymentState::dumps() const {
    return mp::pack(mp::Value::array({deployment.pack(), mp::Value::integer(world_size), mp::Value::integer(dev_mem)}));
}
DeploymentState DeploymentState::loads(const std::string& data) {
    mp::Value v = mp::unpack(data);
    DeploymentState s;
    s.deployment = Deployment::unpack(v.at(0));
    s.world_size = static_cast<int>(v.at(1).as_int());
    s.dev_mem = v.at(2).as_int();
    return s;
}

// ---------------------------------------------------------------- allocation
std::unordered_map<std::string, std::vector<int>> searchAllocationFlat(
    const std::vector<std::string>& order, const std::unordered_map<std::string, int>& repl_nums, int dev_num) {
    // keep one pipeline replica on neighbouring devices: for each of gcd(repl) groups, for each
    // stage, take consecutive device ids
    int g = 0;
    for (const auto& n : order) g = std::gcd(g, repl_nums.at(n));
    g = std::max(1, g);
    std::unordered_map<std::string, std::vector<int>> alloc;
    int dev = 0;
    for (int grp = 0; grp < g; ++grp)
        for (const auto& n : order) {
            const int per = repl_nums.at(n) / g;
            for (int k = 0; k < per; ++k) alloc[n].push_back((dev++) % std::max(1, dev_num));
        }
    for (auto& kv : alloc) std::sort(kv.second.begin(), kv.second.end());
    return alloc;
}

std::unordered_map<std::string, std::vector<int>> searchAllocationSimple(
    const std::vector<std::string>& order, const std::unordered_map<std::string, int>& repl_nums, int dev_num) {
    std::vector<std::string> sorted = order;
    std::stable_sort(sorted.begin(), sorted.end(),
                     [&](const std::string& a, const std::string& b) { return repl_nums.at(a) > repl_nums.at(b); });
    std::unordered_map<std::string, std::vector<int>> alloc;
    int dev = 0;
    for (const auto& n : sorted)
        for (int k = 0; k < repl_nums.at(n); ++k) alloc[n].push_back((dev++) % std::max(1, dev_num));
    return alloc;
}

int tagOfRanks(const std::vector<int>& ranks) {
    std::vector<int> s = ranks;
    std::sort(s.begin(), s.end());
    s.erase(std::unique(s.begin(), s.end()), s.end());
    uint32_t h = 2166136261u;
    for (int r : s) {
        h ^= static_cast<uint32_t>(r + 1);
        h *= 16777619u;
    }
    return 100 + static_cast<int>(h % 29000u);  // below the reference's tag upper bound of 30000
}

// ---------------------------------------------------------------- routes
Deployment createDeployment(const IRGraph& graph, const AllocSolution& sol, int dev_num, bool alloc_repl_flat,
                            const std::string& id) {
    Deployment d;
    d.id = id;
    d.graph = graph;
    d.pipeline_num = sol.pipeline_num;
    d.checkpointing = sol.checkpointing;
    std::vector<std::string> order;
    for (const auto& g : sol.graphs) order.push_back(g.name);
    d.fwd_graph_order = order;
    d.bwd_graph_order.assign(order.rbegin(), order.rend());
    d.allocation = alloc_repl_flat ? searchAllocationFlat(order, sol.repl_nums, dev_num)
                                   : searchAllocationSimple(order, sol.repl_nums, dev_num);
    std::vector<int> all_ranks(dev_num);
    std::iota(all_ranks.begin(), all_ranks.end(), 0);

    // subgraphs are stored at the per-replica, per-micro-batch size (reference: replicate/scaleGraph)
    for (const auto& g : sol.graphs) {
        const int repl = sol.repl_nums.at(g.name);
        const int64_t mb = std::max<int64_t>(1, (graph.batch_size + static_cast<int64_t>(repl) * sol.pipeline_num - 1) /
                                                    (static_cast<int64_t>(repl) * sol.pipeline_num));
        d.subgraphs[g.name] = scaleGraph(g, mb);
    }

    std::unordered_map<std::string, int> order_of;
    for (size_t i = 0; i < order.size(); ++i) order_of[order[i]] = static_cast<int>(i);
    std::unordered_map<std::string, std::string> producer_stage;
    for (const auto& g : sol.graphs)
        for (const auto& o : g.output_names) producer_stage[o] = g.name;

    auto makeRoute = [&](const IRValue& v, const std::string& sg, const std::vector<int>& src, const std::string& dg,
                         const std::vector<int>& dst, RouteTypeDP type) {
        RouteDP r;
        r.location.value_name = v.name;
        r.sources = src;
        r.source_graph = sg;
        r.source_order = order_of.count(sg) ? order_of[sg] : -1;
        r.dests = dst;
        r.dest_graph = dg;
        r.dest_order = order_of.count(dg) ? order_of[dg] : -1;
        std::vector<int> u = src;
        u.insert(u.end(), dst.begin(), dst.end());
        r.tag = tagOfRanks(u);
        r.source_tag = tagOfRanks(src);
        r.type = type;
        r.ir_value = v;
        return r;
    };
    const std::string MASTER = "MASTER";
    std::set<std::pair<std::string, std::string>> done;  // (value, dest stage)
    for (const auto& g : sol.graphs) {
        const auto& dst = d.allocation.at(g.name);
        for (const auto& in : g.input_names) {
            const IRValue& v = g.value(in);
            if (v.is_param) continue;
            if (!done.insert({in, g.name}).second) continue;
            auto pit = producer_stage.find(in);
            if (pit == producer_stage.end() || pit->second == g.name) {
                // graph input: MASTER -> stage
                d.fwd_in_routes.push_back(makeRoute(v, MASTER, all_ranks, g.name, dst, RouteTypeDP::REDIST));
                if (v.type.holdsGradient() && v.type.requires_grad)
                    d.bwd_out_routes.push_back(makeRoute(v, g.name, dst, MASTER, all_ranks, RouteTypeDP::REDIST));
            } else {
                const auto& src = d.allocation.at(pit->second);
                const RouteTypeDP t = v.is_loss ? RouteTypeDP::BROADCAST : RouteTypeDP::REDIST;
                d.fwd_routes.push_back(makeRoute(v, pit->second, src, g.name, dst, t));
                if (v.type.holdsGradient())
                    d.bwd_routes.push_back(makeRoute(v, g.name, dst, pit->second, src,
                                                     v.is_loss ? RouteTypeDP::WEIGHTED_REDUCE : RouteTypeDP::REDIST));
            }
        }
    }
    for (const auto& o : graph.output_names) {
        auto pit = producer_stage.find(o);
        if (pit == producer_stage.end()) continue;
        const IRValue& v = graph.value(o);
        const auto& src = d.allocation.at(pit->second);
        d.fwd_out_routes.push_back(makeRoute(v, pit->second, src, MASTER, all_ranks,
                                             v.is_loss ? RouteTypeDP::WEIGHTED_REDUCE : RouteTypeDP::REDIST));
        if (v.type.holdsGradient())
            d.bwd_in_routes.push_back(makeRoute(v, MASTER, all_ranks, pit->second, src,
                                                v.is_loss ? RouteTypeDP::BROADCAST : RouteTypeDP::REDIST));
    }
    std::reverse(d.bwd_routes.begin(), d.bwd_routes.end());
    return d;
}

std::string verifyDeployment(const Deployment& d) {
    std::ostringstream err;
    std::set<std::pair<std::string, std::string>> fwd_to, fwd_from, bwd_to, bwd_from;
    auto collect = [](const std::vector<RouteDP>& rs, std::set<std::pair<std::string, std::string>>& to,
                      std::set<std::pair<std::string, std::string>>& from) {
        for (const auto& r : rs) {
            to.insert({r.location.value_name, r.dest_graph});
            from.insert({r.location.value_name, r.source_graph});
        }
    };
    collect(d.fwd_routes, fwd_to, fwd_from);
    collect(d.fwd_in_routes, fwd_to, fwd_from);
    collect(d.fwd_out_routes, fwd_to, fwd_from);
    collect(d.bwd_routes, bwd_to, bwd_from);
    collect(d.bwd_in_routes, bwd_to, bwd_from);
    collect(d.bwd_out_routes, bwd_to, bwd_from);
    std::unordered_set<std::string> graph_inputs(d.graph.input_names.begin(), d.graph.input_names.end());
    std::unordered_set<std::string> graph_outputs(d.graph.output_names.begin(), d.graph.output_names.end());
    for (const auto& name : d.fwd_graph_order) {
        auto it = d.subgraphs.find(name);
        if (it == d.subgraphs.end()) return "stage " + name + " has no subgraph";
        if (!d.allocation.count(name) || d.allocation.at(name).empty()) return "stage " + name + " has no ranks";
        const IRGraph& sg = it->second;
        for (const auto& in : sg.input_names) {
            const IRValue& v = sg.value(in);
            if (v.is_param) continue;
            if (!fwd_to.count({in, name})) err << "input " << in << " of " << name << " has no forward route; ";
            if (v.type.holdsGradient() && !graph_inputs.count(in) && !bwd_from.count({in, name}))
                err << "input " << in << " of " << name << " has no backward route; ";
        }
        for (const auto& o : sg.output_names) {
            if (!fwd_from.count({o, name})) err << "output " << o << " of " << name << " has no forward route; ";
            if (sg.value(o).type.holdsGradient() && !bwd_to.count({o, name}))
                err << "output " << o << " of " << name << " has no backward route; ";
        }
    }
    for (const auto& o : d.graph.output_names)
        if (!fwd_to.count({o, "MASTER"})) err << "graph output " << o << " never reaches the caller; ";
    return err.str();
}

// ---------------------------------------------------------------- batch arithmetic
int64_t BatchSizeCalculator::splitSize(int split) const {
    const int64_t P = std::max(1, P_);
    return B_ / P + (split < B_ % P ? 1 : 0);
}
int64_t BatchSizeCalculator::localSplitSize(int idx, int n, int split) const {
    if (n <= 0) return 0;
    const int64_t b = splitSize(split);
    int64_t prev = 0;
    for (int j = 0; j < split; ++j) prev += splitSize(j);
    const int64_t rem = b % n;
    const int64_t off = prev % n;
    const int64_t pos = ((idx - off) % n + n) % n;
    return b / n + (pos < rem ? 1 : 0);
}
int64_t BatchSizeCalculator::localBatchSize(int idx, int n) const {
    int64_t s = 0;
    for (int j = 0; j < P_; ++j) s += localSplitSize(idx, n, j);
    return s;
}
std::vector<int64_t> BatchSizeCalculator::localDims(int64_t dim0, int n, int split) const {
    // the first dimension may be a multiple of the batch (reference: BatchSizeCalculator.cpp:169-172)
    const int64_t b = splitSize(split);
    const int64_t mult = b > 0 && dim0 % b == 0 ? dim0 / b : 1;
    std::vector<int64_t> r(n);
    for (int i = 0; i < n; ++i) r[i] = localSplitSize(i, n, split) * mult;
    return r;
}

RedistArgs getRedistArgs(int my_rank, int world_size, int64_t total_rows, const std::vector<int>& src_ranks_in,
                         const std::vector<int>& dst_ranks_in, int split, int pipeline_num, int64_t global_batch) {
    std::vector<int> src = src_ranks_in, dst = dst_ranks_in;
    std::sort(src.begin(), src.end());
    std::sort(dst.begin(), dst.end());
    BatchSizeCalculator calc(pipeline_num, global_batch);
    const std::vector<int64_t> sdim = calc.localDims(total_rows, static_cast<int>(src.size()), split);
    const std::vector<int64_t> ddim = calc.localDims(total_rows, static_cast<int>(dst.size()), split);
    auto ranges = [](const std::vector<int64_t>& dims) {
        std::vector<std::pair<int64_t, int64_t>> r;
        int64_t off = 0;
        for (auto d : dims) {
            r.emplace_back(off, off + d);
            off += d;
        }
        return r;
    };
    const auto sr = ranges(sdim), dr = ranges(ddim);
    RedistArgs a;
    a.sendcounts.assign(world_size, 0);
    a.recvcounts.assign(world_size, 0);
    a.sdispls.assign(world_size, 0);
    a.rdispls.assign(world_size, 0);
    auto overlap = [](std::pair<int64_t, int64_t> x, std::pair<int64_t, int64_t> y) {
        const int64_t lo = std::max(x.first, y.first), hi = std::min(x.second, y.second);
        return std::make_pair(lo, std::max<int64_t>(0, hi - lo));
    };
    for (size_t si = 0; si < src.size(); ++si) {
        if (src[si] != my_rank) continue;
        for (size_t di = 0; di < dst.size(); ++di) {
            auto ov = overlap(sr[si], dr[di]);
            if (ov.second == 0) continue;
            a.sendcounts[dst[di]] = ov.second;
            a.sdispls[dst[di]] = ov.first - sr[si].first;
        }
    }
    for (size_t di = 0; di < dst.size(); ++di) {
        if (dst[di] != my_rank) continue;
        for (size_t si = 0; si < src.size(); ++si) {
            auto ov = overlap(sr[si], dr[di]);
            if (ov.second == 0) continue;
            a.recvcounts[src[si]] = ov.second;
            a.rdispls[src[si]] = ov.first - dr[di].first;
        }
    }
    return a;
}

// ---------------------------------------------------------------- segments
int64_t alignedNumel(int64_t numel, int elem_size, int nranks) {
    const int64_t unit = static_cast<int64_t>(16 / std::max(1, elem_size)) * std::max(1, nranks);
    return (numel + unit - 1) / unit * unit;
}
std::pair<int64_t, int64_t> segmentRange(int64_t numel, int elem_size, int nranks, int idx) {
    const int64_t seg = alignedNumel(numel, elem_size, nranks) / std::max(1, nranks);
    const int64_t b = std::min(numel, seg * idx), e = std::min(numel, seg * (idx + 1));
    return {b, e};
}

}  // namespace rannc
