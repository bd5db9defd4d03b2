// pybind11 module `_core`: the host-side native core of the framework.
// Counterpart of the reference's `_pyrannc` binding layer (src/main.cpp:30-522)
// for everything that is not tensor traffic.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "deployment.h"
#include "ir.h"
#include "msgpack.h"
#include "partition.h"
#include "profile.h"
#include "runtime_util.h"

namespace py = pybind11;
using namespace rannc;

namespace {

mp::Value toValue(const py::handle& o) {
    if (o.is_none()) return mp::Value::nil();
    if (py::isinstance<py::bool_>(o)) return mp::Value::boolean(o.cast<bool>());
    if (py::isinstance<py::int_>(o)) {
        py::int_ i = py::reinterpret_borrow<py::int_>(o);
        if (PyObject_RichCompareBool(i.ptr(), py::int_(0).ptr(), Py_LT) == 1) return mp::Value::integer(i.cast<int64_t>());
        return mp::Value::uinteger(i.cast<uint64_t>());
    }
    if (py::isinstance<py::float_>(o)) return mp::Value::real(o.cast<double>());
    if (py::isinstance<py::str>(o)) return mp::Value::str(o.cast<std::string>());
    if (py::isinstance<py::bytes>(o)) return mp::Value::bin(o.cast<std::string>());
    if (py::isinstance<py::dict>(o)) {
        mp::MapItems m;
        for (auto kv : py::reinterpret_borrow<py::dict>(o)) m.emplace_back(toValue(kv.first), toValue(kv.second));
        return mp::Value::mapping(std::move(m));
    }
    if (py::isinstance<py::list>(o) || py::isinstance<py::tuple>(o)) {
        mp::Array a;
        for (auto e : o) a.push_back(toValue(e));
        return mp::Value::array(std::move(a));
    }
    throw std::runtime_error("msgpack: unsupported Python type");
}

py::object fromValue(const mp::Value& v) {
    switch (v.kind) {
        case mp::Value::NIL: return py::none();
        case mp::Value::BOOL: return py::bool_(v.b);
        case mp::Value::INT: return py::int_(v.i);
        case mp::Value::UINT: return py::int_(v.u);
        case mp::Value::FLOAT: return py::float_(v.f);
        case mp::Value::STR: return py::str(v.s);
        case mp::Value::BIN: return py::bytes(v.s);
        case mp::Value::ARRAY: {
            py::list l;
            for (const auto& e : *v.arr) l.append(fromValue(e));
            return std::move(l);
        }
        case mp::Value::MAP: {
            py::dict d;
            for (const auto& kv : *v.map) {
                py::object k = fromValue(kv.first);
                if (py::isinstance<py::list>(k)) k = py::tuple(k);
                d[k] = fromValue(kv.second);
            }
            return std::move(d);
        }
    }
    return py::none();
}

}  // namespace

PYBIND11_MODULE(_core, m) {
    m.doc() = "native core: IR, msgpack codec, value classification, partitioner, stage search, deployment";

    // ---- msgpack
    m.def("msgpack_pack", [](py::object o) { return py::bytes(mp::pack(toValue(o))); });
    m.def("msgpack_unpack", [](const std::string& data) { return fromValue(mp::unpack(data)); });

    // ---- IR
    py::enum_<IRBaseType>(m, "IRBaseType")
        .value("SCALAR", IRBaseType::SCALAR).value("TENSOR", IRBaseType::TENSOR).value("STRING", IRBaseType::STRING)
        .value("LIST", IRBaseType::LIST).value("TUPLE", IRBaseType::TUPLE).value("OPTIONAL", IRBaseType::OPTIONAL)
        .value("NONE", IRBaseType::NONE).value("FUNCTION", IRBaseType::FUNCTION);
    py::enum_<IRTensorElemType>(m, "IRTensorElemType")
        .value("UNDEF", IRTensorElemType::UNDEF).value("INT", IRTensorElemType::INT)
        .value("DOUBLE", IRTensorElemType::DOUBLE).value("FLOAT", IRTensorElemType::FLOAT)
        .value("HALF", IRTensorElemType::HALF).value("BFLOAT16", IRTensorElemType::BFLOAT16)
        .value("LONG", IRTensorElemType::LONG).value("BOOL", IRTensorElemType::BOOL);
    py::enum_<IRListType>(m, "IRListType")
        .value("INT", IRListType::INT).value("FLOAT", IRListType::FLOAT).value("BOOL", IRListType::BOOL)
        .value("TENSOR", IRListType::TENSOR).value("GENERIC", IRListType::GENERIC);
    py::enum_<IRScalarType>(m, "IRScalarType")
        .value("NONE", IRScalarType::NONE).value("INT", IRScalarType::INT).value("FLOAT", IRScalarType::FLOAT)
        .value("NUMBER", IRScalarType::NUMBER).value("BOOL", IRScalarType::BOOL).value("DEVICE", IRScalarType::DEVICE);

    py::class_<IRType>(m, "IRType")
        .def(py::init<>())
        .def_static("tensor", &IRType::tensor, py::arg("elem"), py::arg("dims"), py::arg("requires_grad") = false)
        .def_static("scalar", &IRType::scalar)
        .def_static("list", &IRType::list)
        .def_static("tuple", &IRType::tuple)
        .def_static("none", &IRType::none)
        .def_static("string", &IRType::string)
        .def_readwrite("base_type", &IRType::base_type)
        .def_readwrite("scalar_type", &IRType::scalar_type)
        .def_readwrite("tensor_dim", &IRType::tensor_dim)
        .def_readwrite("tensor_elem_type", &IRType::tensor_elem_type)
        .def_readwrite("requires_grad", &IRType::requires_grad)
        .def_readwrite("list_type", &IRType::list_type)
        .def_readwrite("compound_types", &IRType::compound_types)
        .def_readwrite("list_size", &IRType::list_size)
        .def_readwrite("func_name", &IRType::func_name)
        .def("numel", &IRType::numel)
        .def("size_in_byte", &IRType::sizeInByte)
        .def("holds_gradient", &IRType::holdsGradient);

    py::class_<IRValue>(m, "IRValue")
        .def(py::init<>())
        .def(py::init([](std::string name, IRType type, bool is_param) {
                 IRValue v;
                 v.name = std::move(name);
                 v.type = std::move(type);
                 v.is_param = is_param;
                 return v;
             }),
             py::arg("name"), py::arg("type"), py::arg("is_param") = false)
        .def_readwrite("name", &IRValue::name)
        .def_readwrite("type", &IRValue::type)
        .def_readwrite("is_param", &IRValue::is_param)
        .def_readwrite("is_batch", &IRValue::is_batch)
        .def_readwrite("is_loss", &IRValue::is_loss)
        .def_readwrite("batch_size", &IRValue::batch_size)
        .def_readwrite("split_dim", &IRValue::split_dim)
        .def_readwrite("batch_hint", &IRValue::batch_hint);

    py::class_<IRNode>(m, "IRNode")
        .def(py::init<>())
        .def(py::init([](std::string op, std::vector<std::string> ins, std::vector<std::string> outs, std::string id) {
                 IRNode n;
                 n.name = std::move(op);
                 n.input_names = std::move(ins);
                 n.output_names = std::move(outs);
                 n.id = std::move(id);
                 return n;
             }),
             py::arg("op"), py::arg("inputs"), py::arg("outputs"), py::arg("id"))
        .def_readwrite("name", &IRNode::name)
        .def_readwrite("input_names", &IRNode::input_names)
        .def_readwrite("output_names", &IRNode::output_names)
        .def_readwrite("id", &IRNode::id)
        .def_readwrite("is_criterion", &IRNode::is_criterion)
        .def_readwrite("is_batch", &IRNode::is_batch)
        .def_readwrite("batch_size", &IRNode::batch_size);

    py::class_<IRGraph>(m, "IRGraph")
        .def(py::init<>())
        .def_readwrite("name", &IRGraph::name)
        .def_readwrite("nodes", &IRGraph::nodes)
        .def_readwrite("input_names", &IRGraph::input_names)
        .def_readwrite("output_names", &IRGraph::output_names)
        .def_readwrite("is_replicable", &IRGraph::is_replicable)
        .def_readwrite("batch_size", &IRGraph::batch_size)
        .def_property_readonly("values", [](const IRGraph& g) { return g.values; })
        .def("add_value", [](IRGraph& g, const IRValue& v) { g.values[v.name] = v; })
        .def("add_input", [](IRGraph& g, const IRValue& v) {
            g.values[v.name] = v;
            g.input_names.push_back(v.name);
        })
        .def("add_node", [](IRGraph& g, const IRNode& n) { g.nodes.push_back(n); })
        .def("add_output", [](IRGraph& g, const std::string& n) { g.output_names.push_back(n); })
        .def("value", [](const IRGraph& g, const std::string& n) { return g.value(n); })
        .def("has_value", &IRGraph::hasValue)
        .def("param_input_names", &IRGraph::paramInputNames)
        .def("non_param_input_names", &IRGraph::nonParamInputNames)
        .def("param_size_in_byte", &IRGraph::paramSizeInByte)
        .def("input_size_in_byte", &IRGraph::inputSizeInByte)
        .def("output_size_in_byte", &IRGraph::outputSizeInByte)
        .def("comm_buf_size", &IRGraph::commBufSize)
        .def("check", &IRGraph::check)
        .def("dumps", [](const IRGraph& g) { return py::bytes(mp::pack(g.pack())); })
        .def_static("loads", [](const std::string& d) { return IRGraph::unpack(mp::unpack(d)); })
        .def("__str__", &IRGraph::toString)
        .def("to_dot", &IRGraph::toDot);

    m.def("guess_value_types", [](IRGraph g) {
        guessValueTypes(g);
        return g;
    });
    m.def("find_unused_values", &findUnusedValues);
    m.def("remove_unused_nodes", &removeUnusedNodes);
    m.def("scale_graph", &scaleGraph);
    m.def("shared_inputs", &sharedInputs);
    m.def("create_subgraphs", &createSubGraphs);
    m.def("merge_subgraphs", &mergeSubGraphs);

    // ---- profiles / cost model
    py::class_<GraphProfile>(m, "GraphProfile")
        .def(py::init<>())
        .def_readwrite("name", &GraphProfile::name)
        .def_readwrite("fwd_time", &GraphProfile::fwd_time)
        .def_readwrite("bwd_time", &GraphProfile::bwd_time)
        .def_readwrite("fwd_cpu_time", &GraphProfile::fwd_cpu_time)
        .def_readwrite("bwd_cpu_time", &GraphProfile::bwd_cpu_time)
        .def_readwrite("fwd_cuda_time", &GraphProfile::fwd_cuda_time)
        .def_readwrite("bwd_cuda_time", &GraphProfile::bwd_cuda_time)
        .def_readwrite("max_allocated_mem", &GraphProfile::max_allocated_mem)
        .def_readwrite("param_size", &GraphProfile::param_size)
        .def_readwrite("input_size", &GraphProfile::input_size)
        .def_readwrite("output_size", &GraphProfile::output_size)
        .def_readwrite("working_mem", &GraphProfile::working_mem)
        .def_readwrite("activation_size", &GraphProfile::activation_size)
        .def_readwrite("checkpointing", &GraphProfile::checkpointing)
        .def("dumps", [](const GraphProfile& p) { return py::bytes(mp::pack(p.pack())); })
        .def_static("loads", [](const std::string& d) { return GraphProfile::unpack(mp::unpack(d)); });
    py::class_<NodeProfile>(m, "NodeProfile")
        .def(py::init<>())
        .def(py::init([](double f, double b, int64_t act, int64_t work, bool scales) {
                 NodeProfile p;
                 p.fwd_us = f;
                 p.bwd_us = b;
                 p.activation_bytes = act;
                 p.working_bytes = work;
                 p.scales_with_batch = scales;
                 return p;
             }),
             py::arg("fwd_us"), py::arg("bwd_us"), py::arg("activation_bytes") = 0, py::arg("working_bytes") = 0,
             py::arg("scales_with_batch") = true)
        .def_readwrite("fwd_us", &NodeProfile::fwd_us)
        .def_readwrite("bwd_us", &NodeProfile::bwd_us)
        .def_readwrite("activation_bytes", &NodeProfile::activation_bytes)
        .def_readwrite("working_bytes", &NodeProfile::working_bytes)
        .def_readwrite("scales_with_batch", &NodeProfile::scales_with_batch);
    py::class_<LinkModel>(m, "LinkModel")
        .def(py::init<>())
        .def_readwrite("p2p_bytes_per_us", &LinkModel::p2p_bytes_per_us)
        .def_readwrite("allreduce_bytes_per_us", &LinkModel::allreduce_bytes_per_us)
        .def_readwrite("latency_us", &LinkModel::latency_us)
        .def_readwrite("launch_overhead_us", &LinkModel::launch_overhead_us);
    py::class_<PartitioningConf>(m, "PartitioningConf")
        .def(py::init<>())
        .def_readwrite("dev_num", &PartitioningConf::dev_num)
        .def_readwrite("batch_size", &PartitioningConf::batch_size)
        .def_readwrite("dev_mem", &PartitioningConf::dev_mem)
        .def_readwrite("use_amp_master_params", &PartitioningConf::use_amp_master_params)
        .def_readwrite("enable_zero", &PartitioningConf::enable_zero)
        .def_readwrite("offload_params", &PartitioningConf::offload_params)
        .def_readwrite("interleave_single_stage", &PartitioningConf::interleave_single_stage)
        .def_readwrite("force_dist_matmul", &PartitioningConf::force_dist_matmul)
        .def_readwrite("opt_param_factor", &PartitioningConf::opt_param_factor)
        .def_readwrite("min_pipeline", &PartitioningConf::min_pipeline)
        .def_readwrite("max_pipeline", &PartitioningConf::max_pipeline)
        .def_readwrite("min_pipeline_bs", &PartitioningConf::min_pipeline_bs)
        .def_readwrite("min_partition_num", &PartitioningConf::min_partition_num)
        .def_readwrite("max_partition_num", &PartitioningConf::max_partition_num)
        .def_readwrite("cfg_partition_num", &PartitioningConf::cfg_partition_num)
        .def_readwrite("cfg_replica_num", &PartitioningConf::cfg_replica_num)
        .def_readwrite("cfg_pipeline_num", &PartitioningConf::cfg_pipeline_num)
        .def_readwrite("limit_dev_num_pot", &PartitioningConf::limit_dev_num_pot)
        .def_readwrite("limit_dev_num_more_than_bs", &PartitioningConf::limit_dev_num_more_than_bs)
        .def_readwrite("dp_search_all", &PartitioningConf::dp_search_all)
        .def_readwrite("do_coarsening", &PartitioningConf::do_coarsening)
        .def_readwrite("do_uncoarsening", &PartitioningConf::do_uncoarsening)
        .def_readwrite("coarsen_by_time", &PartitioningConf::coarsen_by_time)
        .def_readwrite("checkpointing", &PartitioningConf::checkpointing)
        .def_readwrite("checkpointing_no_last", &PartitioningConf::checkpointing_no_last)
        .def_readwrite("prefer_no_checkpointing", &PartitioningConf::prefer_no_checkpointing)
        .def_readwrite("link", &PartitioningConf::link);
    py::class_<ProfileModel>(m, "ProfileModel")
        .def(py::init<const IRGraph&, std::unordered_map<std::string, NodeProfile>, LinkModel>())
        .def("profile", &ProfileModel::profile)
        .def("set_subgraph_measure",
             [](ProfileModel& pm, py::function fn, int limit) {
                 // fn(node_ids, batch, checkpointing) -> GraphProfile or None; may be called from the stage
                 // search, which runs without the interpreter lock
                 pm.setSubgraphMeasure(
                     [fn](const std::vector<std::string>& ids, int64_t bs, bool ckpt, GraphProfile* out) {
                         py::gil_scoped_acquire gil;
                         py::object r = fn(ids, bs, ckpt);
                         if (r.is_none()) return false;
                         *out = r.cast<GraphProfile>();
                         return true;
                     },
                     limit);
             })
        .def("measured_count", &ProfileModel::measuredCount);
    m.def("calc_comm_time", &calcCommTime);
    m.def("calc_allreduce_time", &calcAllReduceTime);
    m.def("get_opt_mem_size", &getOptMemSize);
    m.def("calc_graph_mem", &calcGraphMem);
    py::class_<ProfileDB>(m, "ProfileDB")
        .def(py::init<>())
        .def("add", [](ProfileDB& db, const std::unordered_map<std::string, IRGraph>& graphs, int64_t bs, int iter,
                       bool ckpt, const std::unordered_map<std::string, GraphProfile>& profiles) {
            ProfileItemKey k;
            k.ir_graphs = graphs;
            k.batch_size = bs;
            k.iteration = iter;
            k.checkpointing = ckpt;
            ProfilingResult r;
            r.node_profiles = profiles;
            db.add(k, r);
        })
        .def("get", [](const ProfileDB& db, const std::unordered_map<std::string, IRGraph>& graphs, int64_t bs,
                       int iter, bool ckpt) -> py::object {
            ProfileItemKey k;
            k.ir_graphs = graphs;
            k.batch_size = bs;
            k.iteration = iter;
            k.checkpointing = ckpt;
            ProfilingResult r;
            if (!db.get(k, &r)) return py::none();
            return py::cast(r.node_profiles);
        })
        .def("__len__", &ProfileDB::size)
        .def("dumps", [](const ProfileDB& db) { return py::bytes(db.dumps()); })
        .def("loads", &ProfileDB::loads);

    // ---- partitioner
    py::class_<MLNode>(m, "MLNode")
        .def_readonly("id", &MLNode::id)
        .def_readonly("graph", &MLNode::graph)
        .def_readonly("sub_nodes", &MLNode::sub_nodes)
        .def_readonly("children", &MLNode::children)
        .def_readonly("level", &MLNode::level);
    py::class_<MLEdge>(m, "MLEdge").def_readonly("src_id", &MLEdge::src_id).def_readonly("tgt_id", &MLEdge::tgt_id);
    py::class_<MLGraph>(m, "MLGraph")
        .def(py::init<>())
        .def_readonly("nodes", &MLGraph::nodes)
        .def_readonly("edges", &MLGraph::edges)
        .def("level", &MLGraph::level)
        .def("dumps", [](const MLGraph& g) { return py::bytes(mp::pack(g.pack())); })
        .def_static("loads", [](const std::string& d) { return MLGraph::unpack(mp::unpack(d)); });
    m.def("ml_partition", [](const ProfileModel& pm, const PartitioningConf& conf) {
        MLPartitioner p(pm, conf);
        return p.partition();
    });
    // the same, with what the passes did: (graph, coarsening levels, boundary moves, cut bytes before / after
    // the uncoarsening)
    m.def("ml_partition_stats", [](const ProfileModel& pm, const PartitioningConf& conf) {
        MLPartitioner p(pm, conf);
        MLGraph g = p.partition();
        return py::make_tuple(g, p.levels(), p.moves(), p.cutBefore(), p.cutAfter());
    });
    m.def("ml_to_lower_level", &toLowerLevel);
    m.def("ml_lift_up", &liftUp);
    m.def("ml_cut_bytes", &cutBytes);
    py::class_<AllocSolution>(m, "AllocSolution")
        .def(py::init<>())
        .def_readwrite("graphs", &AllocSolution::graphs)
        .def_readwrite("repl_nums", &AllocSolution::repl_nums)
        .def_readwrite("pipeline_num", &AllocSolution::pipeline_num)
        .def_readwrite("checkpointing", &AllocSolution::checkpointing)
        .def_readwrite("boundaries", &AllocSolution::boundaries)
        .def_readwrite("dev_nums", &AllocSolution::dev_nums)
        .def_readwrite("est_time_us", &AllocSolution::est_time_us)
        .def("dumps", [](const AllocSolution& s) { return py::bytes(mp::pack(s.pack())); })
        .def_static("loads", [](const std::string& d) { return AllocSolution::unpack(mp::unpack(d)); });
    py::class_<StageEstimate>(m, "StageEstimate")
        .def_readonly("name", &StageEstimate::name)
        .def_readonly("repl", &StageEstimate::repl)
        .def_readonly("micro_batch", &StageEstimate::micro_batch)
        .def_readonly("profile", &StageEstimate::profile)
        .def_readonly("allreduce_us", &StageEstimate::allreduce_us)
        .def_readonly("in_comm_us", &StageEstimate::in_comm_us)
        .def_readonly("out_comm_us", &StageEstimate::out_comm_us)
        .def_readonly("total_mem", &StageEstimate::total_mem)
        .def_readonly("opt_mem", &StageEstimate::opt_mem)
        .def_readonly("comm_mem", &StageEstimate::comm_mem);
    m.def("dp_staging", [](const ProfileModel& pm, const MLGraph& ml, const PartitioningConf& conf) {
        DPStaging dp(pm, ml, conf);
        AllocSolution sol;
        {
            py::gil_scoped_release rel;
            sol = dp.run();
        }
        return py::make_tuple(sol, dp.estimates(), dp.dumpNodeProfiles());
    });
    m.def("fair_weight_decompose", &fairWeightDecompose);
    m.def("dump_dp_cache", [](const MLGraph& ml, const IRGraph& g,
                              const std::unordered_map<std::string, NodeProfile>& np, const PartitioningConf& conf) {
        DPStagingCache c;
        c.graph = ml;
        c.ir_graph = g;
        c.node_profiles = np;
        c.conf = conf;
        return py::bytes(mp::pack(c.pack()));
    });
    m.def("run_dp_dry", [](const std::string& data, py::object dev_num, py::object dev_mem) {
        DPStagingCache c = DPStagingCache::unpack(mp::unpack(data));
        if (!dev_num.is_none()) c.conf.dev_num = dev_num.cast<int>();
        if (!dev_mem.is_none()) c.conf.dev_mem = dev_mem.cast<int64_t>();
        return runDpDry(c);
    }, py::arg("data"), py::arg("dev_num") = py::none(), py::arg("dev_mem") = py::none());

    // ---- deployment
    py::enum_<RouteTypeDP>(m, "RouteType")
        .value("P2P", RouteTypeDP::P2P).value("REDIST", RouteTypeDP::REDIST).value("SCATTER", RouteTypeDP::SCATTER)
        .value("GATHER", RouteTypeDP::GATHER).value("REDUCE", RouteTypeDP::REDUCE)
        .value("WEIGHTED_REDUCE", RouteTypeDP::WEIGHTED_REDUCE).value("BROADCAST", RouteTypeDP::BROADCAST)
        .value("SCATTER_ANY", RouteTypeDP::SCATTER_ANY).value("ALL_GATHER", RouteTypeDP::ALL_GATHER)
        .value("ANY", RouteTypeDP::ANY).value("ANY_TO_ALL", RouteTypeDP::ANY_TO_ALL).value("NA", RouteTypeDP::NA);
    py::class_<RouteDP>(m, "Route")
        .def_property_readonly("value_name", [](const RouteDP& r) { return r.location.value_name; })
        .def_readonly("sources", &RouteDP::sources)
        .def_readonly("source_graph", &RouteDP::source_graph)
        .def_readonly("source_order", &RouteDP::source_order)
        .def_readonly("dests", &RouteDP::dests)
        .def_readonly("dest_graph", &RouteDP::dest_graph)
        .def_readonly("dest_order", &RouteDP::dest_order)
        .def_readonly("tag", &RouteDP::tag)
        .def_readonly("source_tag", &RouteDP::source_tag)
        .def_readonly("type", &RouteDP::type)
        .def_readonly("ir_value", &RouteDP::ir_value);
    py::class_<Deployment>(m, "Deployment")
        .def(py::init<>())
        .def_readwrite("id", &Deployment::id)
        .def_readwrite("graph", &Deployment::graph)
        .def_readwrite("subgraphs", &Deployment::subgraphs)
        .def_readwrite("allocation", &Deployment::allocation)
        .def_readwrite("fwd_routes", &Deployment::fwd_routes)
        .def_readwrite("fwd_in_routes", &Deployment::fwd_in_routes)
        .def_readwrite("fwd_out_routes", &Deployment::fwd_out_routes)
        .def_readwrite("fwd_graph_order", &Deployment::fwd_graph_order)
        .def_readwrite("bwd_routes", &Deployment::bwd_routes)
        .def_readwrite("bwd_in_routes", &Deployment::bwd_in_routes)
        .def_readwrite("bwd_out_routes", &Deployment::bwd_out_routes)
        .def_readwrite("bwd_graph_order", &Deployment::bwd_graph_order)
        .def_readwrite("pipeline_num", &Deployment::pipeline_num)
        .def_readwrite("checkpointing", &Deployment::checkpointing)
        .def_readwrite("offload_params", &Deployment::offload_params)
        .def_readwrite("force_dist_matmul", &Deployment::force_dist_matmul)
        .def("__str__", &Deployment::toString);
    m.def("create_deployment", &createDeployment);
    m.def("verify_deployment", &verifyDeployment);
    m.def("save_deployment", [](const Deployment& d, int world_size, int64_t dev_mem) {
        DeploymentState s{d, world_size, dev_mem};
        return py::bytes(s.dumps());
    });
    m.def("load_deployment", [](const std::string& data) {
        DeploymentState s = DeploymentState::loads(data);
        return py::make_tuple(s.deployment, s.world_size, s.dev_mem);
    });
    m.def("search_allocation_flat", &searchAllocationFlat);
    m.def("search_allocation_simple", &searchAllocationSimple);
    m.def("tag_of_ranks", &tagOfRanks);

    // ---- batch arithmetic, redist, segments
    py::class_<BatchSizeCalculator>(m, "BatchSizeCalculator")
        .def(py::init<int, int64_t>())
        .def("split_size", &BatchSizeCalculator::splitSize)
        .def("local_split_size", &BatchSizeCalculator::localSplitSize)
        .def("local_batch_size", &BatchSizeCalculator::localBatchSize)
        .def("local_dims", &BatchSizeCalculator::localDims);
    py::class_<RedistArgs>(m, "RedistArgs")
        .def_readonly("sendcounts", &RedistArgs::sendcounts)
        .def_readonly("recvcounts", &RedistArgs::recvcounts)
        .def_readonly("sdispls", &RedistArgs::sdispls)
        .def_readonly("rdispls", &RedistArgs::rdispls);
    m.def("get_redist_args", &getRedistArgs);
    m.def("aligned_numel", &alignedNumel);
    m.def("segment_range", &segmentRange);

    // ---- config / logging / trace / watchdog
    m.def("config_reload", [] { Config::get().reload(); });
    m.def("config_get", [](const std::string& name) -> py::object {
        for (const auto& it : Config::get().items()) {
            if (it.name != name) continue;
            switch (it.type) {
                case ConfigItem::INT: return py::int_(Config::get().getInt(name));
                case ConfigItem::FLOAT: return py::float_(Config::get().getFloat(name));
                case ConfigItem::BOOL: return py::bool_(Config::get().getBool(name));
                default: return py::str(Config::get().getString(name));
            }
        }
        throw std::runtime_error("unknown config item: " + name);
    });
    m.def("config_set", [](const std::string& name, const std::string& value) { Config::get().set(name, value); });
    m.def("config_items", [] {
        py::dict d;
        for (const auto& it : Config::get().items()) d[py::str(it.name)] = py::make_tuple(it.value, it.default_value);
        return d;
    });
    m.def("config_warnings", [] { return Config::get().warnings(); });
    m.def("parse_toml", &Config::parseToml);
    m.def("log", [](const std::string& logger, int level, const std::string& msg) {
        getLogger(logger).log(static_cast<LogLevel>(level), msg);
    });
    m.def("set_log_level", [](const std::string& logger, const std::string& level) {
        setLogLevel(logger, parseLogLevel(level));
    });
    m.def("set_log_rank", &setLogRank);
    m.def("configure_logging_from_toml", &configureLoggingFromToml);
    m.def("log_enabled", [](const std::string& logger, int level) {
        return getLogger(logger).enabled(static_cast<LogLevel>(level));
    });

    m.def("trace_enable", [](bool on) { EventRecorder::get().enable(on); });
    m.def("trace_enabled", [] { return EventRecorder::get().enabled(); });
    m.def("trace_begin", [](const std::string& n, int tid) { EventRecorder::get().begin(n, tid); },
          py::arg("name"), py::arg("tid") = 0);
    m.def("trace_end", [](const std::string& n, int tid) { EventRecorder::get().end(n, tid); }, py::arg("name"),
          py::arg("tid") = 0);
    m.def("trace_size", [] { return EventRecorder::get().size(); });
    m.def("trace_clear", [] { EventRecorder::get().clear(); });
    m.def("trace_dump_local", [](int rank) { return EventRecorder::get().dumpLocal(rank); });
    m.def("trace_merge", &EventRecorder::merge);
    m.def("func_key", &funcKey);
    m.def("comm_key", &commKey);

    py::class_<TimeCounter>(m, "TimeCounter")
        .def(py::init<bool>(), py::arg("enable") = true)
        .def("start", &TimeCounter::start)
        .def("stop", &TimeCounter::stop)
        .def("total_us", &TimeCounter::totalUs)
        .def("count", &TimeCounter::count)
        .def("summary", &TimeCounter::summary)
        .def("clear", &TimeCounter::clear);

    py::class_<Watchdog>(m, "Watchdog")
        .def(py::init<>())
        .def("start", [](Watchdog& w, const std::string& dir, int rank, int world, double period, double stale,
                         py::object cb) {
            std::function<void(int)> f;
            if (!cb.is_none()) {
                py::function pf = cb.cast<py::function>();
                f = [pf](int peer) {
                    py::gil_scoped_acquire g;
                    pf(peer);
                };
            }
            w.start(dir, rank, world, period, stale, f);
        }, py::arg("dir"), py::arg("rank"), py::arg("world_size"), py::arg("period_s") = 10.0,
             py::arg("stale_s") = 60.0, py::arg("on_failure") = py::none())
        .def("stop", [](Watchdog& w, bool remove) {
            py::gil_scoped_release rel;
            w.stop(remove);
        }, py::arg("remove_own_file") = true)
        .def("running", &Watchdog::running)
        .def("failed_peer", &Watchdog::failedPeer)
        .def_static("lock_path", &Watchdog::lockPath);
    m.def("resident_mem_bytes", &residentMemBytes);
}
