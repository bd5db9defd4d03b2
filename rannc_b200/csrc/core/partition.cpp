#include "partition.h"

#include <algorithm>
#include <cmath>
#include <functional>
#include <limits>
#include <map>
#include <numeric>
#include <queue>
#include <set>
#include <sstream>
#include <stdexcept>

namespace rannc {

// ---------------------------------------------------------------- ML graph serialisation
mp::Value MLBaseEdge::pack() const {
    return mp::Value::array({mp::Value::str(src_id), mp::Value::str(tgt_id), mp::Value::str(value)});
}
MLBaseEdge MLBaseEdge::unpack(const mp::Value& v) { return {v.at(0).as_str(), v.at(1).as_str(), v.at(2).as_str()}; }
mp::Value MLEdge::pack() const {
    mp::Array be;
    for (const auto& e : base_edges) be.push_back(e.pack());
    // field order: src_id, tgt_id, sub_edges, base_edges (reference: MLGraph.h:41-62)
    return mp::Value::array({mp::Value::str(src_id), mp::Value::str(tgt_id), mp::Value::array({}),
                             mp::Value::array(std::move(be))});
}
MLEdge MLEdge::unpack(const mp::Value& v) {
    MLEdge e;
    e.src_id = v.at(0).as_str();
    e.tgt_id = v.at(1).as_str();
    for (const auto& b : v.at(3).as_array()) e.base_edges.push_back(MLBaseEdge::unpack(b));
    return e;
}
mp::Value MLNode::pack() const {
    // field order: id, graph, sub_nodes, sub_edges (reference: MLGraph.h:14-39).  sub_nodes holds the nodes of
    // the level below as nested records; an atomic block lists the ids of its operators instead.
    mp::Value subs;
    if (!children.empty()) {
        mp::Array cs;
        for (const auto& c : children) cs.push_back(c.pack());
        subs = mp::Value::array(std::move(cs));
    } else {
        subs = packStrings(sub_nodes);
    }
    return mp::Value::array({mp::Value::str(id), graph.pack(), std::move(subs), mp::Value::array({})});
}
namespace {
void collectOps(const MLNode& n, std::vector<std::string>* out) {
    if (n.children.empty()) {
        out->insert(out->end(), n.sub_nodes.begin(), n.sub_nodes.end());
        return;
    }
    for (const auto& c : n.children) collectOps(c, out);
}
}  // namespace
MLNode MLNode::unpack(const mp::Value& v) {
    MLNode n;
    n.id = v.at(0).as_str();
    n.graph = IRGraph::unpack(v.at(1));
    const mp::Value& sn = v.at(2);
    for (const auto& s : sn.as_array()) {
        if (s.kind == mp::Value::STR) {
            n.sub_nodes.push_back(s.as_str());
        } else {
            n.children.push_back(MLNode::unpack(s));
            n.level = std::max(n.level, n.children.back().level + 1);
        }
    }
    if (!n.children.empty()) collectOps(n, &n.sub_nodes);
    return n;
}
int MLGraph::level() const {
    int l = 0;
    for (const auto& n : nodes) l = std::max(l, n.level);
    return l;
}
mp::Value MLGraph::pack() const {
    mp::Array ns, es;
    for (const auto& n : nodes) ns.push_back(n.pack());
    for (const auto& e : edges) es.push_back(e.pack());
    return mp::Value::array({mp::Value::array(std::move(ns)), mp::Value::array(std::move(es))});
}
MLGraph MLGraph::unpack(const mp::Value& v) {
    MLGraph g;
    for (const auto& n : v.at(0).as_array()) g.nodes.push_back(MLNode::unpack(n));
    for (const auto& e : v.at(1).as_array()) g.edges.push_back(MLEdge::unpack(e));
    return g;
}

// ---------------------------------------------------------------- subgraph extraction
namespace {

// Index structure over the full graph used by every cut / merge operation.
struct GraphIndex {
    const IRGraph& g;
    std::vector<bool> owned_kind;  // true: batch / criterion node (owned by exactly one part)
    std::unordered_map<std::string, size_t> producer;
    std::unordered_map<std::string, std::vector<size_t>> consumer;
    // for a replicated (non-batch) node: owned nodes that depend on it through replicated nodes only
    std::vector<std::vector<int>> dependants;
    std::unordered_set<std::string> graph_outputs;

    explicit GraphIndex(const IRGraph& graph) : g(graph) {
        producer = producers(g);
        consumer = consumers(g);
        graph_outputs.insert(g.output_names.begin(), g.output_names.end());
        const size_t n = g.nodes.size();
        owned_kind.assign(n, false);
        bool any = false;
        for (size_t i = 0; i < n; ++i) {
            owned_kind[i] = g.nodes[i].is_batch || g.nodes[i].is_criterion;
            any = any || owned_kind[i];
        }
        if (!any) std::fill(owned_kind.begin(), owned_kind.end(), true);
        dependants.assign(n, {});
        for (size_t k = n; k-- > 0;) {
            if (owned_kind[k]) continue;
            std::set<int> deps;
            for (const auto& o : g.nodes[k].output_names) {
                auto it = consumer.find(o);
                if (it == consumer.end()) continue;
                for (size_t c : it->second) {
                    if (owned_kind[c]) deps.insert(static_cast<int>(c));
                    else deps.insert(dependants[c].begin(), dependants[c].end());
                }
            }
            dependants[k].assign(deps.begin(), deps.end());
        }
    }

    // owned nodes + the replicated nodes they (transitively) read from
    std::vector<int> closure(const std::vector<int>& own) const {
        std::vector<bool> in(g.nodes.size(), false);
        std::vector<int> stack(own.begin(), own.end());
        for (int i : own) in[i] = true;
        while (!stack.empty()) {
            const int i = stack.back();
            stack.pop_back();
            for (const auto& name : g.nodes[i].input_names) {
                auto it = producer.find(name);
                if (it == producer.end()) continue;
                const size_t p = it->second;
                if (!owned_kind[p] && !in[p]) {
                    in[p] = true;
                    stack.push_back(static_cast<int>(p));
                }
            }
        }
        std::vector<int> r;
        for (size_t i = 0; i < in.size(); ++i)
            if (in[i]) r.push_back(static_cast<int>(i));
        return r;
    }

    IRGraph extract(const std::vector<int>& own, const std::string& name, bool take_orphan_outputs) const {
        std::vector<bool> is_own(g.nodes.size(), false);
        for (int i : own) is_own[i] = true;
        const std::vector<int> all = closure(own);
        std::vector<bool> in_set(g.nodes.size(), false);
        for (int i : all) in_set[i] = true;

        IRGraph r;
        r.name = name;
        r.batch_size = g.batch_size;
        r.is_replicable = g.is_replicable;
        std::unordered_set<std::string> produced;
        std::vector<std::string> in_batch, in_param;
        std::unordered_set<std::string> seen_in;
        for (int i : all) {
            const IRNode& node = g.nodes[i];
            for (const auto& in : node.input_names) {
                if (produced.count(in) || seen_in.count(in)) continue;
                auto pit = producer.find(in);
                if (pit != producer.end() && in_set[pit->second]) continue;
                seen_in.insert(in);
                (g.value(in).is_param ? in_param : in_batch).push_back(in);
                r.values[in] = g.value(in);
            }
            r.nodes.push_back(node);
            for (const auto& o : node.output_names) {
                produced.insert(o);
                r.values[o] = g.value(o);
            }
        }
        r.input_names = in_batch;
        r.input_names.insert(r.input_names.end(), in_param.begin(), in_param.end());
        // outputs: produced by an owned node here and needed by an owned node elsewhere or by the caller
        for (int i : all) {
            if (!is_own[i] && !(take_orphan_outputs && !owned_kind[i])) continue;
            for (const auto& o : g.nodes[i].output_names) {
                bool needed = false;
                if (graph_outputs.count(o)) {
                    // a graph output computed by a replicated node belongs to the last part only
                    needed = is_own[i] || take_orphan_outputs;
                }
                if (!needed && is_own[i]) {
                    auto cit = consumer.find(o);
                    if (cit != consumer.end()) {
                        for (size_t c : cit->second) {
                            if (owned_kind[c]) {
                                if (!is_own[c]) needed = true;
                            } else {
                                for (int d : dependants[c])
                                    if (!is_own[d]) needed = true;
                            }
                            if (needed) break;
                        }
                    }
                }
                if (needed && std::find(r.output_names.begin(), r.output_names.end(), o) == r.output_names.end())
                    r.output_names.push_back(o);
            }
        }
        return r;
    }
};

}  // namespace

std::vector<IRGraph> createSubGraphs(const IRGraph& g, const std::vector<int>& label, int num_parts,
                                     const std::string& prefix) {
    GraphIndex idx(g);
    std::vector<std::vector<int>> own(num_parts);
    for (size_t i = 0; i < g.nodes.size(); ++i)
        if (idx.owned_kind[i] && label[i] >= 0 && label[i] < num_parts) own[label[i]].push_back(static_cast<int>(i));
    std::vector<IRGraph> parts;
    for (int k = 0; k < num_parts; ++k)
        parts.push_back(idx.extract(own[k], prefix + std::to_string(k), k == num_parts - 1));
    return parts;
}

namespace {
std::vector<int> ownedIndices(const GraphIndex& idx, const IRGraph& part,
                              const std::unordered_map<std::string, int>& node_pos) {
    std::vector<int> own;
    for (const auto& n : part.nodes) {
        auto it = node_pos.find(n.id);
        if (it != node_pos.end() && idx.owned_kind[it->second]) own.push_back(it->second);
    }
    return own;
}
}  // namespace

IRGraph mergeSubGraphs(const IRGraph& g, const std::vector<IRGraph>& parts, int first, int last,
                       const std::string& name) {
    GraphIndex idx(g);
    std::unordered_map<std::string, int> pos;
    for (size_t i = 0; i < g.nodes.size(); ++i) pos[g.nodes[i].id] = static_cast<int>(i);
    std::vector<int> own;
    for (int k = first; k <= last; ++k) {
        auto o = ownedIndices(idx, parts[k], pos);
        own.insert(own.end(), o.begin(), o.end());
    }
    std::sort(own.begin(), own.end());
    own.erase(std::unique(own.begin(), own.end()), own.end());
    return idx.extract(own, name, last == static_cast<int>(parts.size()) - 1);
}

// ---------------------------------------------------------------- coarsening
namespace {

struct Block {
    std::vector<int> own;   // owned node indices (sorted)
    double eval = 0;        // fwd + bwd microseconds at the planning micro-batch
    int64_t mem = 0;        // parameter + activation bytes, rough
    bool alive = true;
};

struct BlockGraph {
    std::vector<Block> blocks;
    std::vector<int> block_of;  // owned node -> block
    // adjacency with cut bytes
    std::vector<std::unordered_map<int, int64_t>> succ, pred;
};

bool reachableWithout(const BlockGraph& bg, int from, int to) {
    // is `to` reachable from `from` by a path that does not use the direct edge from->to?
    std::vector<int> stack;
    std::unordered_set<int> seen;
    for (const auto& kv : bg.succ[from])
        if (kv.first != to) stack.push_back(kv.first);
    while (!stack.empty()) {
        const int v = stack.back();
        stack.pop_back();
        if (v == to) return true;
        if (!seen.insert(v).second) continue;
        for (const auto& kv : bg.succ[v]) stack.push_back(kv.first);
    }
    return false;
}

void mergeInto(BlockGraph& bg, int a, int b) {
    // merge block b into a (edge a->b exists and the merge is convex)
    Block& A = bg.blocks[a];
    Block& B = bg.blocks[b];
    A.own.insert(A.own.end(), B.own.begin(), B.own.end());
    std::sort(A.own.begin(), A.own.end());
    A.eval += B.eval;
    A.mem += B.mem;
    B.alive = false;
    for (int n : B.own) bg.block_of[n] = a;
    B.own.clear();
    for (const auto& kv : bg.succ[b]) {
        bg.pred[kv.first].erase(b);
        if (kv.first == a) continue;
        bg.succ[a][kv.first] += kv.second;
        bg.pred[kv.first][a] += kv.second;
    }
    for (const auto& kv : bg.pred[b]) {
        bg.succ[kv.first].erase(b);
        if (kv.first == a) continue;
        bg.pred[a][kv.first] += kv.second;
        bg.succ[kv.first][a] += kv.second;
    }
    bg.succ[a].erase(b);
    bg.pred[a].erase(b);
    bg.succ[b].clear();
    bg.pred[b].clear();
}

int aliveCount(const BlockGraph& bg) {
    int n = 0;
    for (const auto& b : bg.blocks) n += b.alive ? 1 : 0;
    return n;
}

std::vector<int> topoOrder(const BlockGraph& bg) {
    const int n = static_cast<int>(bg.blocks.size());
    std::vector<int> indeg(n, 0), order;
    // tie-break by the first owned node so the order follows the original program order
    auto key = [&](int b) { return bg.blocks[b].own.empty() ? 1 << 30 : bg.blocks[b].own.front(); };
    auto cmp = [&](int x, int y) { return key(x) > key(y); };
    std::priority_queue<int, std::vector<int>, decltype(cmp)> q(cmp);
    for (int b = 0; b < n; ++b) {
        if (!bg.blocks[b].alive) continue;
        indeg[b] = static_cast<int>(bg.pred[b].size());
        if (indeg[b] == 0) q.push(b);
    }
    while (!q.empty()) {
        const int b = q.top();
        q.pop();
        order.push_back(b);
        for (const auto& kv : bg.succ[b])
            if (--indeg[kv.first] == 0) q.push(kv.first);
    }
    return order;
}

}  // namespace

namespace {

// Skeleton of the multi-level hierarchy: which blocks of the level below a block was merged from.
struct Skel {
    int level = 0;
    std::vector<int> own;        // operator indices (sorted)
    std::vector<Skel> kids;
};

using Adj = std::vector<std::unordered_map<int, int64_t>>;

// Group-level adjacency (bytes of the values that go from group a to group b) for a node -> group labelling.
void buildAdjacency(const GraphIndex& idx, const std::vector<int>& group_of, int ngroups, double ratio, Adj* succ,
                    Adj* pred) {
    const IRGraph& g = idx.g;
    succ->assign(ngroups, {});
    pred->assign(ngroups, {});
    for (size_t i = 0; i < g.nodes.size(); ++i) {
        if (!idx.owned_kind[i] || group_of[i] < 0) continue;
        for (const auto& o : g.nodes[i].output_names) {
            auto cit = idx.consumer.find(o);
            if (cit == idx.consumer.end()) continue;
            const int64_t bytes = static_cast<int64_t>(g.value(o).type.sizeInByte() * ratio);
            std::set<int> targets;
            for (size_t c : cit->second) {
                if (idx.owned_kind[c]) targets.insert(group_of[c]);
                else
                    for (int d : idx.dependants[c]) targets.insert(group_of[d]);
            }
            for (int t : targets) {
                if (t < 0 || t == group_of[i]) continue;
                (*succ)[group_of[i]][t] += bytes;
                (*pred)[t][group_of[i]] += bytes;
            }
        }
    }
}

bool reaches(const Adj& succ, int from, int to) {
    if (from == to) return true;
    std::vector<int> stack{from};
    std::unordered_set<int> seen;
    while (!stack.empty()) {
        const int v = stack.back();
        stack.pop_back();
        if (v == to) return true;
        if (!seen.insert(v).second) continue;
        for (const auto& kv : succ[v]) stack.push_back(kv.first);
    }
    return false;
}

MLNode skelToNode(const GraphIndex& idx, const Skel& s, const std::string& id, bool with_graph, bool last) {
    MLNode n;
    n.id = id;
    if (with_graph) n.graph = idx.extract(s.own, id, last);
    for (int i : s.own) n.sub_nodes.push_back(idx.g.nodes[i].id);
    // the level of a node is the height of the hierarchy below it (what a reader of the file can recompute)
    n.level = 0;
    for (size_t k = 0; k < s.kids.size(); ++k) {
        n.children.push_back(skelToNode(idx, s.kids[k], id + "_" + std::to_string(k), false, false));
        n.level = std::max(n.level, n.children.back().level + 1);
    }
    return n;
}

}  // namespace

MLGraph MLPartitioner::partition() {
    const IRGraph& g = pm_.graph();
    GraphIndex idx(g);
    const int n = static_cast<int>(g.nodes.size());

    // atomic blocks: one per batch / criterion operator (reference: Partitioner.cpp:885-896)
    BlockGraph bg;
    bg.block_of.assign(n, -1);
    const int64_t plan_bs =
        std::max<int64_t>(1, conf_.batch_size / std::max(1, conf_.dev_num) / std::max(1, conf_.max_pipeline));
    const double ratio = static_cast<double>(plan_bs) / std::max<int64_t>(1, g.batch_size);
    std::vector<double> node_time(n, 0.0);
    std::vector<int64_t> node_mem(n, 0);
    for (int i = 0; i < n; ++i) {
        if (!idx.owned_kind[i]) continue;
        Block b;
        b.own = {i};
        const NodeProfile* np = pm_.nodeProfile(g.nodes[i].id);
        if (np) {
            node_time[i] = (np->fwd_us + np->bwd_us) * (np->scales_with_batch ? ratio : 1.0);
            b.mem = static_cast<int64_t>(np->activation_bytes * ratio);
        }
        for (const auto& in : g.nodes[i].input_names)
            if (g.hasValue(in) && g.value(in).is_param) b.mem += g.value(in).type.sizeInByte();
        node_mem[i] = b.mem;
        // what a block is weighed by: its time, or (coarsen_by_time = false) the memory it needs
        // (reference: Partitioner.cpp:44-55)
        b.eval = conf_.coarsen_by_time ? node_time[i] : static_cast<double>(b.mem);
        bg.block_of[i] = static_cast<int>(bg.blocks.size());
        bg.blocks.push_back(std::move(b));
    }
    const int nb = static_cast<int>(bg.blocks.size());
    buildAdjacency(idx, bg.block_of, nb, ratio, &bg.succ, &bg.pred);
    std::vector<Skel> skel(nb);
    for (int b = 0; b < nb; ++b) skel[b].own = bg.blocks[b].own;

    const int min_parts = std::max(1, std::min(conf_.max_partition_num,
                                               std::max(conf_.min_partition_num, 2 * conf_.dev_num)));
    auto mergeSkel = [&](int a, int b, int level) {
        Skel m;
        m.level = level;
        m.kids.push_back(std::move(skel[a]));
        m.kids.push_back(std::move(skel[b]));
        m.own = m.kids[0].own;
        m.own.insert(m.own.end(), m.kids[1].own.begin(), m.kids[1].own.end());
        std::sort(m.own.begin(), m.own.end());
        skel[a] = std::move(m);
        skel[b] = Skel{};
    };
    levels_ = 0;
    if (conf_.do_coarsening) {
        int last = -1;
        while (aliveCount(bg) != last) {
            last = aliveCount(bg);
            if (last <= 3 || last <= min_parts) break;
            // statistics for the "not an outlier" rule
            double sum = 0, sq = 0;
            std::vector<int> order;
            for (int b = 0; b < nb; ++b)
                if (bg.blocks[b].alive) {
                    order.push_back(b);
                    sum += bg.blocks[b].eval;
                }
            const double mean = sum / order.size();
            for (int b : order) sq += (bg.blocks[b].eval - mean) * (bg.blocks[b].eval - mean);
            const double sigma = std::sqrt(sq / order.size());
            std::sort(order.begin(), order.end(), [&](int x, int y) {
                if (bg.blocks[x].eval != bg.blocks[y].eval) return bg.blocks[x].eval < bg.blocks[y].eval;
                return x < y;
            });
            std::vector<bool> matched(nb, false);
            int remaining = last;
            for (int v : order) {
                if (matched[v] || !bg.blocks[v].alive) continue;
                if (remaining <= min_parts) break;
                int best = -1;
                double best_imprv = -1;
                for (const auto& kv : bg.succ[v]) {
                    const int adj = kv.first;
                    if (matched[adj] || !bg.blocks[adj].alive) continue;
                    const double merged_eval = bg.blocks[v].eval + bg.blocks[adj].eval;
                    if (order.size() > 8 && merged_eval > mean + 2 * sigma && merged_eval > 2.5 * mean) continue;
                    if (conf_.dev_mem > 0 && bg.blocks[v].mem + bg.blocks[adj].mem > conf_.dev_mem) continue;
                    if (reachableWithout(bg, v, adj)) continue;  // merge would not be convex
                    // gain of the merge = t(v) + t(adj) + comm(v -> adj) - t(merged)
                    // (reference: Partitioner.cpp:90-238).  The merged time comes from a measurement of the
                    // merged subgraph when the profile model has one (measured subgraph profiles), and is
                    // the sum of the two otherwise, which leaves the saved transfer as the gain.
                    double imprv = calcCommTime(pm_.link(), kv.second);
                    if (conf_.coarsen_by_time) {
                        std::vector<int> both = bg.blocks[v].own;
                        both.insert(both.end(), bg.blocks[adj].own.begin(), bg.blocks[adj].own.end());
                        std::vector<std::string> ids;
                        for (int i : both) ids.push_back(g.nodes[i].id);
                        double t_merged = 0;
                        if (pm_.measuredSubgraphTime(ids, plan_bs, &t_merged))
                            imprv += merged_eval - t_merged;
                    }
                    if (imprv > best_imprv) {
                        best_imprv = imprv;
                        best = adj;
                    }
                }
                if (best >= 0) {
                    matched[v] = matched[best] = true;
                    mergeInto(bg, v, best);
                    mergeSkel(v, best, levels_ + 1);
                    --remaining;
                }
            }
            ++levels_;
        }
    }

    // uncoarsening: walk the hierarchy back down; at every level the blocks of the level below that sit at a
    // boundary may change sides when that shrinks the cut and keeps the block sizes in bounds
    // (reference: uncoarsen / adjustBoundaries, Partitioner.cpp:511-771)
    moves_ = 0;
    cut_before_ = cut_after_ = 0;
    for (int b = 0; b < nb; ++b)
        if (bg.blocks[b].alive)
            for (const auto& kv : bg.succ[b]) cut_before_ += kv.second;
    cut_after_ = cut_before_;
    if (conf_.do_uncoarsening && conf_.do_coarsening && levels_ > 0) {
        // parts = the alive blocks; units = pieces of the hierarchy, refined level by level
        std::vector<int> part_ids;
        for (int b = 0; b < nb; ++b)
            if (bg.blocks[b].alive) part_ids.push_back(b);
        struct Unit {
            Skel skel;
            int part;
        };
        std::vector<Unit> units;
        for (int b : part_ids) {
            if (skel[b].kids.empty()) units.push_back({skel[b], b});
            else
                for (auto& k : skel[b].kids) units.push_back({k, b});
        }
        auto unitEval = [&](const Skel& s) {
            double e = 0;
            for (int i : s.own) e += conf_.coarsen_by_time ? node_time[i] : static_cast<double>(node_mem[i]);
            return e;
        };
        auto unitMem = [&](const Skel& s) {
            int64_t m = 0;
            for (int i : s.own) m += node_mem[i];
            return m;
        };
        for (int level = levels_; level >= 1; --level) {
            for (int pass = 0; pass < 2; ++pass) {
                int moved_this_pass = 0;
                const int nu = static_cast<int>(units.size());
                std::vector<int> unit_of(n, -1), part_of_node(n, -1);
                for (int u = 0; u < nu; ++u)
                    for (int i : units[u].skel.own) {
                        unit_of[i] = u;
                        part_of_node[i] = units[u].part;
                    }
                Adj usucc, upred, psucc, ppred;
                buildAdjacency(idx, unit_of, nu, ratio, &usucc, &upred);
                buildAdjacency(idx, part_of_node, nb, ratio, &psucc, &ppred);
                std::vector<double> part_eval(nb, 0.0);
                std::vector<int64_t> part_mem(nb, 0);
                std::vector<int> part_units(nb, 0);
                for (int u = 0; u < nu; ++u) {
                    part_eval[units[u].part] += unitEval(units[u].skel);
                    part_mem[units[u].part] += unitMem(units[u].skel);
                    part_units[units[u].part] += 1;
                }
                double sum = 0, sq = 0, mx = 0;
                for (int b : part_ids) {
                    sum += part_eval[b];
                    mx = std::max(mx, part_eval[b]);
                }
                const double mean = sum / part_ids.size();
                for (int b : part_ids) sq += (part_eval[b] - mean) * (part_eval[b] - mean);
                const double limit = std::max(mx, mean + 2 * std::sqrt(sq / part_ids.size()));
                for (int u = 0; u < nu; ++u) {
                    const int A = units[u].part;
                    if (part_units[A] < 2) continue;
                    bool succ_in_A = false, pred_in_A = false;
                    std::unordered_map<int, int64_t> to_part, from_part;
                    for (const auto& kv : usucc[u]) {
                        if (units[kv.first].part == A) succ_in_A = true;
                        else to_part[units[kv.first].part] += kv.second;
                    }
                    int64_t from_A = 0, to_A = 0;
                    for (const auto& kv : upred[u]) {
                        if (units[kv.first].part == A) {
                            pred_in_A = true;
                            from_A += kv.second;
                        } else {
                            from_part[units[kv.first].part] += kv.second;
                        }
                    }
                    for (const auto& kv : usucc[u])
                        if (units[kv.first].part == A) to_A += kv.second;
                    const double ue = unitEval(units[u].skel);
                    const int64_t um = unitMem(units[u].skel);
                    int best = -1;
                    int64_t best_gain = 0;
                    auto fits = [&](int B) {
                        if (part_eval[B] + ue > limit) return false;
                        if (conf_.dev_mem > 0 && part_mem[B] + um > conf_.dev_mem) return false;
                        return true;
                    };
                    if (!succ_in_A) {
                        // a sink of its part: may move forward into a part it feeds
                        for (const auto& kv : to_part) {
                            const int B = kv.first;
                            if (!fits(B)) continue;
                            bool cyc = false;
                            for (const auto& o : to_part)
                                if (o.first != B && reaches(psucc, o.first, B)) cyc = true;
                            if (cyc) continue;
                            const int64_t gain = kv.second - from_A;
                            if (gain > best_gain) {
                                best_gain = gain;
                                best = B;
                            }
                        }
                    }
                    if (!pred_in_A) {
                        // a source of its part: may move backward into a part that feeds it
                        for (const auto& kv : from_part) {
                            const int B = kv.first;
                            if (!fits(B)) continue;
                            bool cyc = false;
                            for (const auto& o : from_part)
                                if (o.first != B && reaches(psucc, B, o.first)) cyc = true;
                            if (cyc) continue;
                            const int64_t gain = kv.second - to_A;
                            if (gain > best_gain) {
                                best_gain = gain;
                                best = B;
                            }
                        }
                    }
                    if (best < 0) continue;
                    units[u].part = best;
                    part_eval[A] -= ue;
                    part_eval[best] += ue;
                    part_mem[A] -= um;
                    part_mem[best] += um;
                    part_units[A] -= 1;
                    part_units[best] += 1;
                    for (int i : units[u].skel.own) part_of_node[i] = best;
                    buildAdjacency(idx, part_of_node, nb, ratio, &psucc, &ppred);
                    ++moves_;
                    ++moved_this_pass;
                }
                if (!moved_this_pass) break;
            }
            if (level > 1) {
                // one level down: every unit is replaced by the blocks it was merged from
                std::vector<Unit> lower;
                for (auto& u : units) {
                    if (u.skel.kids.empty()) lower.push_back(std::move(u));
                    else
                        for (auto& k : u.skel.kids) lower.push_back({k, u.part});
                }
                units = std::move(lower);
            }
        }
        // rebuild the blocks from the final assignment
        for (int b : part_ids) {
            bg.blocks[b].own.clear();
            bg.blocks[b].eval = 0;
            bg.blocks[b].mem = 0;
            skel[b] = Skel{};
            skel[b].level = levels_;
        }
        for (auto& u : units) {
            Block& B = bg.blocks[u.part];
            B.own.insert(B.own.end(), u.skel.own.begin(), u.skel.own.end());
            B.eval += unitEval(u.skel);
            B.mem += unitMem(u.skel);
            skel[u.part].kids.push_back(std::move(u.skel));
        }
        for (int b : part_ids) {
            std::sort(bg.blocks[b].own.begin(), bg.blocks[b].own.end());
            skel[b].own = bg.blocks[b].own;
            for (int i : bg.blocks[b].own) bg.block_of[i] = b;
        }
        buildAdjacency(idx, bg.block_of, nb, ratio, &bg.succ, &bg.pred);
        cut_after_ = 0;
        for (int b : part_ids)
            for (const auto& kv : bg.succ[b]) cut_after_ += kv.second;
    }

    // mergeSmall: cheapest block joins its cheaper convex neighbour until <= max_partition_num
    // (reference: Partitioner.cpp:773-873)
    while (aliveCount(bg) > std::max(1, conf_.max_partition_num)) {
        std::vector<int> order = topoOrder(bg);
        int cheapest = -1;
        for (int b : order)
            if (cheapest < 0 || bg.blocks[b].eval < bg.blocks[cheapest].eval) cheapest = b;
        int best = -1;
        bool best_is_succ = false;
        auto consider = [&](int other, bool is_succ) {
            const int a = is_succ ? cheapest : other, b = is_succ ? other : cheapest;
            if (reachableWithout(bg, a, b)) return;
            if (best < 0 || bg.blocks[other].eval < bg.blocks[best].eval) {
                best = other;
                best_is_succ = is_succ;
            }
        };
        for (const auto& kv : bg.succ[cheapest]) consider(kv.first, true);
        for (const auto& kv : bg.pred[cheapest]) consider(kv.first, false);
        if (best < 0) {
            // isolated block: attach to its neighbour in the topological order
            auto it = std::find(order.begin(), order.end(), cheapest);
            const size_t p = it - order.begin();
            const int other = p + 1 < order.size() ? order[p + 1] : order[p - 1];
            bg.succ[cheapest][other] += 0;
            bg.pred[other][cheapest] += 0;
            best = other;
            best_is_succ = true;
        }
        if (best_is_succ) {
            mergeInto(bg, cheapest, best);
            mergeSkel(cheapest, best, std::max(skel[cheapest].level, skel[best].level) + 1);
        } else {
            mergeInto(bg, best, cheapest);
            mergeSkel(best, cheapest, std::max(skel[cheapest].level, skel[best].level) + 1);
        }
    }

    // emit in topological order (reference: sortMLGraph)
    MLGraph out;
    std::vector<int> order = topoOrder(bg);
    std::unordered_map<int, std::string> id_of;
    for (size_t k = 0; k < order.size(); ++k) id_of[order[k]] = "ML_" + std::to_string(k);
    for (size_t k = 0; k < order.size(); ++k) {
        skel[order[k]].own = bg.blocks[order[k]].own;
        out.nodes.push_back(skelToNode(idx, skel[order[k]], id_of[order[k]], true, k + 1 == order.size()));
    }
    for (int b : order) {
        for (const auto& kv : bg.succ[b]) {
            MLEdge e;
            e.src_id = id_of[b];
            e.tgt_id = id_of[kv.first];
            out.edges.push_back(std::move(e));
        }
    }
    // value-level edges
    std::unordered_map<std::string, std::string> producer_block;
    for (const auto& node : out.nodes)
        for (const auto& o : node.graph.output_names) producer_block[o] = node.id;
    for (auto& e : out.edges) {
        for (const auto& node : out.nodes) {
            if (node.id != e.tgt_id) continue;
            for (const auto& in : node.graph.input_names) {
                auto it = producer_block.find(in);
                if (it != producer_block.end() && it->second == e.src_id)
                    e.base_edges.push_back({e.src_id, e.tgt_id, in});
            }
        }
    }
    return out;
}

namespace {
// edges (with value-level base edges) of an ML graph whose nodes carry operator ids
void rebuildEdges(const IRGraph& g, MLGraph* ml) {
    GraphIndex idx(g);
    std::unordered_map<std::string, int> pos;
    for (size_t i = 0; i < g.nodes.size(); ++i) pos[g.nodes[i].id] = static_cast<int>(i);
    std::vector<int> group_of(g.nodes.size(), -1);
    for (size_t k = 0; k < ml->nodes.size(); ++k)
        for (const auto& id : ml->nodes[k].sub_nodes) {
            auto it = pos.find(id);
            if (it != pos.end() && idx.owned_kind[it->second]) group_of[it->second] = static_cast<int>(k);
        }
    ml->edges.clear();
    std::unordered_map<std::string, int> producer_node;
    for (size_t k = 0; k < ml->nodes.size(); ++k)
        for (const auto& o : ml->nodes[k].graph.output_names) producer_node[o] = static_cast<int>(k);
    std::map<std::pair<int, int>, std::vector<std::string>> found;
    for (size_t k = 0; k < ml->nodes.size(); ++k)
        for (const auto& in : ml->nodes[k].graph.input_names) {
            auto it = producer_node.find(in);
            if (it != producer_node.end() && it->second != static_cast<int>(k))
                found[{it->second, static_cast<int>(k)}].push_back(in);
        }
    for (const auto& kv : found) {
        MLEdge e;
        e.src_id = ml->nodes[kv.first.first].id;
        e.tgt_id = ml->nodes[kv.first.second].id;
        for (const auto& v : kv.second) e.base_edges.push_back({e.src_id, e.tgt_id, v});
        ml->edges.push_back(std::move(e));
    }
}

std::vector<int> opsOf(const IRGraph& g, const GraphIndex& idx, const MLNode& n) {
    std::unordered_map<std::string, int> pos;
    for (size_t i = 0; i < g.nodes.size(); ++i) pos[g.nodes[i].id] = static_cast<int>(i);
    std::vector<int> own;
    for (const auto& id : n.sub_nodes) {
        auto it = pos.find(id);
        if (it != pos.end() && idx.owned_kind[it->second]) own.push_back(it->second);
    }
    std::sort(own.begin(), own.end());
    return own;
}
}  // namespace

MLGraph toLowerLevel(const IRGraph& g, const MLGraph& ml) {
    GraphIndex idx(g);
    MLGraph out;
    for (const auto& node : ml.nodes) {
        if (node.children.empty()) {
            out.nodes.push_back(node);
            continue;
        }
        for (const auto& c : node.children) out.nodes.push_back(c);
    }
    for (size_t k = 0; k < out.nodes.size(); ++k)
        out.nodes[k].graph = idx.extract(opsOf(g, idx, out.nodes[k]), out.nodes[k].id, false);
    rebuildEdges(g, &out);
    return out;
}

MLGraph liftUp(const IRGraph& g, const MLGraph& ml, const std::vector<std::vector<int>>& groups) {
    GraphIndex idx(g);
    std::vector<bool> used(ml.nodes.size(), false);
    MLGraph out;
    for (size_t k = 0; k < groups.size(); ++k) {
        MLNode up;
        up.id = "ML_" + std::to_string(k);
        for (int i : groups[k]) {
            if (i < 0 || i >= static_cast<int>(ml.nodes.size()) || used[i])
                throw std::invalid_argument("liftUp: the groups must partition the nodes");
            used[i] = true;
            MLNode child = ml.nodes[i];
            child.graph = IRGraph{};
            up.level = std::max(up.level, child.level + 1);
            up.sub_nodes.insert(up.sub_nodes.end(), child.sub_nodes.begin(), child.sub_nodes.end());
            up.children.push_back(std::move(child));
        }
        up.graph = idx.extract(opsOf(g, idx, up), up.id, k + 1 == groups.size());
        out.nodes.push_back(std::move(up));
    }
    if (std::find(used.begin(), used.end(), false) != used.end())
        throw std::invalid_argument("liftUp: the groups must partition the nodes");
    rebuildEdges(g, &out);
    return out;
}

int64_t cutBytes(const IRGraph& g, const MLGraph& ml) {
    int64_t total = 0;
    for (const auto& e : ml.edges)
        for (const auto& b : e.base_edges)
            if (g.hasValue(b.value)) total += g.value(b.value).type.sizeInByte();
    return total;
}

// ---------------------------------------------------------------- stage search
mp::Value AllocSolution::pack() const {
    mp::Array gs;
    for (const auto& g : graphs) gs.push_back(g.pack());
    mp::MapItems rn;
    std::vector<std::string> keys;
    for (const auto& kv : repl_nums) keys.push_back(kv.first);
    std::sort(keys.begin(), keys.end());
    for (const auto& k : keys) rn.emplace_back(mp::Value::str(k), mp::Value::integer(repl_nums.at(k)));
    std::vector<int64_t> b(boundaries.begin(), boundaries.end()), d(dev_nums.begin(), dev_nums.end());
    // field order: graphs, repl_nums, part_info, pipeline_num, checkpointing, boundaries, dev_nums
    // (reference: DPStaging.h:33-35)
    return mp::Value::array({mp::Value::array(std::move(gs)), mp::Value::mapping(std::move(rn)),
                             mp::Value::mapping({}), mp::Value::integer(pipeline_num),
                             mp::Value::boolean(checkpointing), packInts(b), packInts(d)});
}
AllocSolution AllocSolution::unpack(const mp::Value& v) {
    AllocSolution s;
    for (const auto& g : v.at(0).as_array()) s.graphs.push_back(IRGraph::unpack(g));
    for (const auto& kv : v.at(1).as_map()) s.repl_nums[kv.first.as_str()] = static_cast<int>(kv.second.as_int());
    s.pipeline_num = static_cast<int>(v.at(3).as_int());
    s.checkpointing = v.at(4).as_bool();
    for (auto x : unpackInts(v.at(5))) s.boundaries.push_back(static_cast<int>(x));
    for (auto x : unpackInts(v.at(6))) s.dev_nums.push_back(static_cast<int>(x));
    return s;
}

namespace {
bool isPow2(int x) { return x > 0 && (x & (x - 1)) == 0; }
int64_t ceilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Σ over the S + P - 1 pipeline steps of (max fwd + max bwd among the active stages) + max all-reduce
// (reference: DPStaging.cpp:240-276)
double estimateTime(const std::vector<StageEstimate>& st, int P) {
    const int S = static_cast<int>(st.size());
    double total = 0;
    for (int t = 0; t < S + P - 1; ++t) {
        double mf = 0, mb = 0;
        for (int s = 0; s < S; ++s) {
            const int mbi = t - s;
            if (mbi < 0 || mbi >= P) continue;
            mf = std::max(mf, st[s].profile.fwd_time + st[s].in_comm_us);
            mb = std::max(mb, st[s].profile.bwd_time + st[s].out_comm_us);
        }
        total += mf + mb;
    }
    double ar = 0;
    for (const auto& s : st) ar = std::max(ar, s.allreduce_us);
    return total + ar;
}
}  // namespace

bool DPStaging::runOnce(int S, int P, bool ckpt, AllocSolution* sol, std::vector<StageEstimate>* est) {
    const int L = static_cast<int>(ml_.nodes.size());
    const int D = conf_.dev_num;
    if (S > L || S > D) return false;
    const int64_t B = conf_.batch_size;
    const IRGraph& g = pm_.graph();
    std::vector<IRGraph> parts;
    for (const auto& n : ml_.nodes) parts.push_back(n.graph);

    struct Cell {
        double value = std::numeric_limits<double>::infinity();
        double max_fwd = 0, max_bwd = 0;
        int prev_b = -1, prev_d = -1;
    };
    // table[s][b][d]: best value for the first b ML nodes on d devices in s stages
    std::vector<std::vector<std::vector<Cell>>> table(
        S + 1, std::vector<std::vector<Cell>>(L + 1, std::vector<Cell>(D + 1)));
    table[0][0][0].value = 0;

    // cache of merged ranges and their profiles
    std::map<std::pair<int, int>, IRGraph> merged;
    auto rangeGraph = [&](int b0, int b1) -> const IRGraph& {
        auto key = std::make_pair(b0, b1);
        auto it = merged.find(key);
        if (it == merged.end()) {
            std::ostringstream nm;
            nm << "MERGE_" << b0 << "_" << (b1 - 1);
            it = merged.emplace(key, mergeSubGraphs(g, parts, b0, b1 - 1, nm.str())).first;
        }
        return it->second;
    };
    struct Eval {
        bool ok = false;
        StageEstimate e;
    };
    std::map<std::tuple<int, int, int>, Eval> evals;
    auto evalStage = [&](int b0, int b1, int repl) -> const Eval& {
        auto key = std::make_tuple(b0, b1, repl);
        auto it = evals.find(key);
        if (it != evals.end()) return it->second;
        Eval ev;
        const IRGraph& sg = rangeGraph(b0, b1);
        const int64_t mb = ceilDiv(B, static_cast<int64_t>(repl) * P);
        ev.e.name = sg.name;
        ev.e.repl = repl;
        ev.e.micro_batch = mb;
        // checkpointing_no_last: the last stage keeps its activations instead of recomputing them when they
        // fit (its backward is the first to run, so its recomputation would sit on the critical path)
        // (reference: config item checkpointing_no_last)
        const bool stage_ckpt = ckpt && !(conf_.checkpointing_no_last && b1 == L);
        ev.e.profile = pm_.profile(sg, mb, stage_ckpt);
        IRGraph scaled = scaleGraph(sg, mb);
        ev.e.in_comm_us = calcCommTime(pm_.link(), scaled.inputSizeInByte());
        ev.e.out_comm_us = calcCommTime(pm_.link(), scaled.outputSizeInByte());
        ev.e.allreduce_us = calcAllReduceTime(pm_.link(), sg.paramSizeInByte(), repl);
        ev.e.opt_mem = getOptMemSize(sg, conf_, repl);
        ev.e.comm_mem = scaled.commBufSize();
        // a single stage that interleaves forward and backward per micro-batch holds one micro-batch at a time
        const int P_mem = (conf_.interleave_single_stage && b0 == 0 && b1 == L) ? 1 : P;
        ev.e.total_mem = calcGraphMem(scaled, ev.e.profile, conf_, repl, P_mem, stage_ckpt);
        ev.ok = conf_.dev_mem <= 0 || ev.e.total_mem < conf_.dev_mem;
        return evals.emplace(key, std::move(ev)).first->second;
    };

    for (int s = 1; s <= S; ++s) {
        for (int b = s; b <= L - (S - s); ++b) {
            for (int d = D; d >= s; --d) {
                Cell& cell = table[s][b][d];
                for (int bp = s - 1; bp < b; ++bp) {
                    for (int dp = s - 1; dp < d; ++dp) {
                        const Cell& prev = table[s - 1][bp][dp];
                        if (!std::isfinite(prev.value)) continue;
                        const int repl = d - dp;
                        if (conf_.limit_dev_num_pot && !isPow2(repl)) continue;
                        if (conf_.limit_dev_num_more_than_bs && repl > ceilDiv(B, P)) continue;
                        if (B / (static_cast<int64_t>(repl) * P) < conf_.min_pipeline_bs) continue;
                        if (conf_.cfg_replica_num > 0 && repl != conf_.cfg_replica_num) continue;
                        const Eval& ev = evalStage(bp, b, repl);
                        if (!ev.ok) continue;
                        const double f = std::max(ev.e.profile.fwd_time + ev.e.in_comm_us, prev.max_fwd);
                        const double w = std::max(ev.e.profile.bwd_time + ev.e.out_comm_us, prev.max_bwd);
                        const double val = f + w;
                        if (val < cell.value) {
                            cell.value = val;
                            cell.max_fwd = f;
                            cell.max_bwd = w;
                            cell.prev_b = bp;
                            cell.prev_d = dp;
                        }
                    }
                }
            }
        }
    }
    // the final state must use every device (reference: DPStaging.cpp:743-750)
    if (!std::isfinite(table[S][L][D].value)) return false;
    std::vector<int> bnd(S + 1), devs(S);
    int b = L, d = D;
    bnd[S] = L;
    for (int s = S; s >= 1; --s) {
        const Cell& c = table[s][b][d];
        devs[s - 1] = d - c.prev_d;
        bnd[s - 1] = c.prev_b;
        b = c.prev_b;
        d = c.prev_d;
    }
    sol->graphs.clear();
    sol->repl_nums.clear();
    est->clear();
    for (int s = 0; s < S; ++s) {
        const Eval& ev = evalStage(bnd[s], bnd[s + 1], devs[s]);
        sol->graphs.push_back(rangeGraph(bnd[s], bnd[s + 1]));
        sol->repl_nums[ev.e.name] = devs[s];
        est->push_back(ev.e);
    }
    sol->pipeline_num = P;
    sol->checkpointing = ckpt;
    sol->boundaries = bnd;
    sol->dev_nums = devs;
    sol->est_time_us = estimateTime(*est, P);
    return true;
}

AllocSolution DPStaging::run() {
    const int L = static_cast<int>(ml_.nodes.size());
    const int D = conf_.dev_num;
    const int64_t B = conf_.batch_size;
    AllocSolution best;
    bool found = false;
    const int s_min = conf_.cfg_partition_num > 0 ? conf_.cfg_partition_num : 1;
    const int s_max = conf_.cfg_partition_num > 0 ? conf_.cfg_partition_num : std::min(L, D);
    for (int S = s_min; S <= s_max; ++S) {
        AllocSolution best_s;
        std::vector<StageEstimate> best_est;
        bool found_s = false;
        std::vector<int> pls;
        if (conf_.cfg_pipeline_num > 0) pls.push_back(conf_.cfg_pipeline_num);
        else
            for (int64_t P = std::max(1, conf_.min_pipeline); P <= std::min<int64_t>(B, conf_.max_pipeline); P *= 2)
                pls.push_back(static_cast<int>(P));
        for (int P : pls) {
            // recompute is required only when memory demands it (or when asked for)
            std::vector<bool> modes;
            if (conf_.checkpointing) modes = {true};
            else if (P > 1 && !conf_.prefer_no_checkpointing) modes = {true};
            else if (P > 1) modes = {false, true};
            else modes = {false};
            for (bool ckpt : modes) {
                AllocSolution sol;
                std::vector<StageEstimate> est;
                if (!runOnce(S, P, ckpt, &sol, &est)) continue;
                if (!found_s || sol.est_time_us < best_s.est_time_us) {
                    best_s = sol;
                    best_est = est;
                    found_s = true;
                }
                break;  // the cheaper mode fits: do not also try the recomputing one
            }
        }
        if (found_s && (!found || best_s.est_time_us < best.est_time_us)) {
            best = best_s;
            estimates_ = best_est;
            found = true;
        }
        if (found && !conf_.dp_search_all) break;  // first feasible stage count wins
    }
    if (!found)
        throw std::runtime_error(
            "partitioning failed: no assignment of stages to devices fits in device memory");
    return best;
}

std::string DPStaging::dumpNodeProfiles() const {
    std::ostringstream ss;
    ss << "{\"nodes\":[";
    const int64_t mb = std::max<int64_t>(1, conf_.batch_size / std::max(1, conf_.dev_num));
    for (size_t i = 0; i < ml_.nodes.size(); ++i) {
        const GraphProfile p = pm_.profile(ml_.nodes[i].graph, mb, false);
        ss << (i ? "," : "") << "{\"id\":\"" << ml_.nodes[i].id << "\",\"fwd_time\":" << p.fwd_time
           << ",\"bwd_time\":" << p.bwd_time << ",\"param_size\":" << p.param_size
           << ",\"activation_size\":" << p.activation_size << ",\"input_size\":" << p.input_size
           << ",\"output_size\":" << p.output_size << "}";
    }
    ss << "],\"batch_size\":" << mb << "}";
    return ss.str();
}

// ---------------------------------------------------------------- fair weight
AllocSolution fairWeightDecompose(const ProfileModel& pm, const PartitioningConf& conf) {
    const IRGraph& g = pm.graph();
    GraphIndex idx(g);
    const int parts = std::max(1, conf.cfg_partition_num > 0 ? conf.cfg_partition_num : 1);
    const int repl = std::max(1, conf.cfg_replica_num > 0 ? conf.cfg_replica_num : conf.dev_num / parts);
    const int P = std::max(1, conf.cfg_pipeline_num > 0 ? conf.cfg_pipeline_num : 1);
    // cumulative bytes of the values each owned node produces or reads as parameters
    std::vector<int> owned;
    std::vector<double> w;
    double total = 0;
    for (size_t i = 0; i < g.nodes.size(); ++i) {
        if (!idx.owned_kind[i]) continue;
        double bytes = 0;
        for (const auto& o : g.nodes[i].output_names) bytes += g.value(o).type.sizeInByte();
        for (const auto& in : g.nodes[i].input_names)
            if (g.hasValue(in) && g.value(in).is_param) bytes += g.value(in).type.sizeInByte();
        owned.push_back(static_cast<int>(i));
        w.push_back(bytes);
        total += bytes;
    }
    std::vector<int> label(g.nodes.size(), -1);
    double acc = 0;
    for (size_t k = 0; k < owned.size(); ++k) {
        int part = static_cast<int>(acc / (total / parts + 1e-9));
        part = std::min(part, parts - 1);
        label[owned[k]] = part;
        acc += w[k];
    }
    AllocSolution sol;
    sol.graphs = createSubGraphs(g, label, parts, "FW_");
    for (const auto& sg : sol.graphs) sol.repl_nums[sg.name] = repl;
    sol.pipeline_num = P;
    sol.checkpointing = conf.checkpointing || (P > 1 && !conf.prefer_no_checkpointing);
    sol.dev_nums.assign(parts, repl);
    for (int k = 0; k <= parts; ++k) sol.boundaries.push_back(k);
    return sol;
}

// ---------------------------------------------------------------- DP cache / dry run
mp::Value DPStagingCache::pack() const {
    mp::MapItems np;
    std::vector<std::string> keys;
    for (const auto& kv : node_profiles) keys.push_back(kv.first);
    std::sort(keys.begin(), keys.end());
    for (const auto& k : keys) {
        const NodeProfile& p = node_profiles.at(k);
        np.emplace_back(mp::Value::str(k),
                        mp::Value::array({mp::Value::real(p.fwd_us), mp::Value::real(p.bwd_us),
                                          mp::Value::integer(p.activation_bytes), mp::Value::integer(p.working_bytes),
                                          mp::Value::boolean(p.scales_with_batch)}));
    }
    // field order: graph, ml_profile_cache, ir_graph, conf (reference: DPStaging.h, DPStagingCache)
    return mp::Value::array({graph.pack(), mp::Value::mapping(std::move(np)), ir_graph.pack(), conf.pack()});
}
DPStagingCache DPStagingCache::unpack(const mp::Value& v) {
    DPStagingCache c;
    c.graph = MLGraph::unpack(v.at(0));
    for (const auto& kv : v.at(1).as_map()) {
        NodeProfile p;
        p.fwd_us = kv.second.at(0).as_double();
        p.bwd_us = kv.second.at(1).as_double();
        p.activation_bytes = kv.second.at(2).as_int();
        p.working_bytes = kv.second.at(3).as_int();
        p.scales_with_batch = kv.second.at(4).as_bool();
        c.node_profiles[kv.first.as_str()] = p;
    }
    c.ir_graph = IRGraph::unpack(v.at(2));
    c.conf = PartitioningConf::unpack(v.at(3));
    return c;
}
AllocSolution runDpDry(const DPStagingCache& cache) {
    ProfileModel pm(cache.ir_graph, cache.node_profiles, cache.conf.link);
    DPStaging dp(pm, cache.graph, cache.conf);
    return dp.run();
}

}  // namespace rannc
