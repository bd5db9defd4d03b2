// Stand-alone self-test of the native core, built with the host sanitizers
// (python -m rannc_b200.build --selftest): AddressSanitizer + UndefinedBehaviorSanitizer in one binary,
// ThreadSanitizer in another.  It drives the code paths the Python bindings drive -- msgpack codec, IR
// construction and classification, multi-level partitioning with uncoarsening, stage search, deployment and
// its serialisation, batch arithmetic, redistribution plans -- and the two components that own threads (event
// recorder under concurrent writers, heartbeat watchdog).  Exit code 0 = every check held and no sanitizer
// report was produced.  The reference has no sanitizer configuration; this program is how the rebuilt host
// code is checked for memory errors, undefined behaviour and data races without a GPU.
#ifdef RANNC_SELFTEST
#include <cstdio>
#include <cstdlib>
#include <filesystem>
#include <unistd.h>
#include <thread>

#include "deployment.h"
#include "ir.h"
#include "partition.h"
#include "profile.h"
#include "runtime_util.h"

using namespace rannc;

#define CHECK(cond)                                                               \
    do {                                                                          \
        if (!(cond)) {                                                            \
            std::fprintf(stderr, "selftest: %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            std::exit(1);                                                         \
        }                                                                         \
    } while (0)

static IRGraph makeMlp(int layers, int hidden, int batch) {
    IRGraph g;
    g.name = "mlp";
    g.batch_size = batch;
    auto addValue = [&](const std::string& n, IRType t, bool param) {
        IRValue v;
        v.name = n;
        v.type = std::move(t);
        v.is_param = param;
        g.values[n] = v;
    };
    addValue("x", IRType::tensor(IRTensorElemType::FLOAT, {batch, hidden}), false);
    g.input_names.push_back("x");
    for (int i = 0; i < layers; ++i) {
        const std::string w = "w" + std::to_string(i), b = "b" + std::to_string(i);
        addValue(w, IRType::tensor(IRTensorElemType::FLOAT, {hidden, hidden}, true), true);
        addValue(b, IRType::tensor(IRTensorElemType::FLOAT, {hidden}, true), true);
        g.input_names.push_back(w);
        g.input_names.push_back(b);
    }
    std::string prev = "x";
    for (int i = 0; i < layers; ++i) {
        const std::string h = "h" + std::to_string(i), a = "a" + std::to_string(i);
        addValue(h, IRType::tensor(IRTensorElemType::FLOAT, {batch, hidden}), false);
        IRNode lin;
        lin.name = "aten::linear";
        lin.input_names = {prev, "w" + std::to_string(i), "b" + std::to_string(i)};
        lin.output_names = {h};
        lin.id = "lin" + std::to_string(i);
        g.nodes.push_back(lin);
        addValue(a, IRType::tensor(IRTensorElemType::FLOAT, {batch, hidden}), false);
        IRNode act;
        act.name = "aten::relu";
        act.input_names = {h};
        act.output_names = {a};
        act.id = "relu" + std::to_string(i);
        g.nodes.push_back(act);
        prev = a;
    }
    g.output_names.push_back(prev);
    g.check();
    guessValueTypes(g);
    return g;
}

static void testCodecAndIr() {
    IRGraph g = makeMlp(6, 32, 16);
    const std::string bytes = mp::pack(g.pack());
    IRGraph back = IRGraph::unpack(mp::unpack(bytes));
    CHECK(back.toString() == g.toString());
    CHECK(g.value("h2").is_batch && g.value("w0").is_param);
    IRGraph half = scaleGraph(g, 8);
    CHECK(half.value("h2").type.tensor_dim[0] == 8);
    CHECK(findUnusedValues(g).empty());
    // size_t(-1) survives the codec (list_size default)
    IRType t = IRType::tensor(IRTensorElemType::HALF, {2, 3});
    IRType t2 = IRType::unpack(mp::unpack(mp::pack(t.pack())));
    CHECK(t2.list_size == static_cast<uint64_t>(-1) && t2.tensor_dim.size() == 2);
}

static void testPlanning() {
    IRGraph g = makeMlp(24, 64, 32);
    std::unordered_map<std::string, NodeProfile> np;
    unsigned seed = 7;
    for (const auto& n : g.nodes) {
        NodeProfile p;
        seed = seed * 1103515245u + 12345u;
        p.fwd_us = 50 + (seed >> 16) % 100;
        p.bwd_us = 2 * p.fwd_us;
        p.activation_bytes = 1 << 14;
        np[n.id] = p;
    }
    PartitioningConf conf;
    conf.dev_num = 4;
    conf.batch_size = 32;
    conf.min_partition_num = 6;
    conf.do_uncoarsening = true;
    ProfileModel pm(g, np, conf.link);
    MLPartitioner part(pm, conf);
    MLGraph ml = part.partition();
    CHECK(!ml.nodes.empty() && part.levels() > 0 && part.cutAfter() <= part.cutBefore());
    size_t ops = 0;
    for (const auto& n : ml.nodes) ops += n.sub_nodes.size();
    CHECK(ops == g.nodes.size());
    MLGraph ml2 = MLGraph::unpack(mp::unpack(mp::pack(ml.pack())));
    CHECK(ml2.nodes.size() == ml.nodes.size() && ml2.level() == ml.level());
    MLGraph low = toLowerLevel(g, ml);
    CHECK(low.nodes.size() >= ml.nodes.size());
    conf.cfg_partition_num = 2;
    conf.cfg_pipeline_num = 2;
    DPStaging dp(pm, ml, conf);
    AllocSolution sol = dp.run();
    CHECK(sol.graphs.size() == 2 && sol.pipeline_num == 2);
    AllocSolution sol2 = AllocSolution::unpack(mp::unpack(mp::pack(sol.pack())));
    CHECK(sol2.boundaries == sol.boundaries);
    Deployment dep = createDeployment(g, sol, 4, true, "selftest");
    CHECK(verifyDeployment(dep).empty());
    DeploymentState st;
    st.deployment = dep;
    st.world_size = 4;
    st.dev_mem = 123;
    DeploymentState st2 = DeploymentState::loads(st.dumps());
    CHECK(st2.world_size == 4 && st2.deployment.fwd_graph_order == dep.fwd_graph_order);
    // a measuring callback that throws must not take the search down
    pm.setSubgraphMeasure([](const std::vector<std::string>&, int64_t, bool, GraphProfile*) -> bool {
        throw std::runtime_error("boom");
    }, 4);
    DPStaging dp2(pm, ml, conf);
    CHECK(dp2.run().graphs.size() == 2);
    AllocSolution fw = fairWeightDecompose(pm, conf);
    CHECK(!fw.graphs.empty());
}

static void testBatchMath() {
    BatchSizeCalculator calc(3, 17);
    int64_t total = 0;
    for (int s = 0; s < 3; ++s) {
        total += calc.splitSize(s);
        int64_t rows = 0;
        for (int i = 0; i < 4; ++i) rows += calc.localSplitSize(i, 4, s);
        CHECK(rows == calc.splitSize(s));
    }
    CHECK(total == 17);
    for (int me = 0; me < 4; ++me) {
        RedistArgs a = getRedistArgs(me, 4, 6, {0, 1}, {2, 3}, 1, 3, 17);
        CHECK(a.sendcounts.size() == 4 && a.recvcounts.size() == 4);
    }
    CHECK(alignedNumel(10, 4, 4) % 16 == 0);
    auto r = segmentRange(10, 4, 4, 3);
    CHECK(r.first <= r.second && r.second <= 10);
    CHECK(tagOfRanks({0, 1, 2}) == tagOfRanks({2, 1, 0}));
}

static void testThreads() {
    // concurrent writers + a reader on the event recorder
    EventRecorder& rec = EventRecorder::get();
    rec.clear();
    rec.enable(true);
    std::vector<std::thread> th;
    for (int t = 0; t < 4; ++t)
        th.emplace_back([t, &rec] {
            for (int i = 0; i < 500; ++i) {
                const std::string k = funcKey("forward", "g" + std::to_string(t), i % 3, false);
                rec.begin(k, t);
                rec.end(k, t);
            }
        });
    th.emplace_back([&rec] {
        for (int i = 0; i < 50; ++i) (void)rec.dumpLocal(0).size();
    });
    for (auto& x : th) x.join();
    CHECK(rec.size() == 4 * 500 * 2);
    const std::string doc = EventRecorder::merge({rec.dumpLocal(0), rec.dumpLocal(1)});
    CHECK(doc.find("traceEvents") != std::string::npos);
    rec.enable(false);
    rec.clear();
    TimeCounter tc(true);
    std::vector<std::thread> th2;
    for (int t = 0; t < 3; ++t)
        th2.emplace_back([t, &tc] {
            for (int i = 0; i < 200; ++i) {
                tc.start("k" + std::to_string(t));
                tc.stop("k" + std::to_string(t));
            }
        });
    for (auto& x : th2) x.join();
    CHECK(tc.count("k0") == 200);
    // watchdog: two "ranks" in one process; the second stops and removes its file, the first notices
    namespace fs = std::filesystem;
    const fs::path dir = fs::temp_directory_path() / ("rannc_selftest_" + std::to_string(::getpid()));
    fs::create_directories(dir);
    std::atomic<int> failed{-1};
    {
        Watchdog a, b;
        a.start(dir.string(), 0, 2, 0.02, 5.0, [&failed](int peer) { failed = peer; });
        b.start(dir.string(), 1, 2, 0.02, 5.0, [](int) {});
        std::this_thread::sleep_for(std::chrono::milliseconds(150));
        CHECK(failed.load() == -1);
        b.stop(true);
        for (int i = 0; i < 200 && failed.load() < 0; ++i) std::this_thread::sleep_for(std::chrono::milliseconds(10));
        CHECK(failed.load() == 1 && a.failedPeer() == 1);
        a.stop(true);
    }
    fs::remove_all(dir);
    // configuration reads while another thread overrides a value
    std::thread w([] {
        for (int i = 0; i < 200; ++i) Config::get().set("profiling_iter", std::to_string(1 + i % 3));
    });
    for (int i = 0; i < 200; ++i) CHECK(Config::get().getInt("profiling_iter") >= 1);
    w.join();
}

int main() {
    testCodecAndIr();
    testPlanning();
    testBatchMath();
    testThreads();
    std::printf("selftest ok\n");
    return 0;
}
#endif  // RANNC_SELFTEST
