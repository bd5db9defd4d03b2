#include "runtime_util.h"

#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <cstdio>
#include <chrono>
#include <cstdlib>
#include <ctime>
#include <fstream>
#include <iostream>
#include <sstream>
#include <stdexcept>

namespace rannc {

// ---------------------------------------------------------------- config
namespace {
std::string trim(const std::string& s) {
    size_t b = 0, e = s.size();
    while (b < e && std::isspace(static_cast<unsigned char>(s[b]))) ++b;
    while (e > b && std::isspace(static_cast<unsigned char>(s[e - 1]))) --e;
    return s.substr(b, e - b);
}
std::string upper(std::string s) {
    for (auto& c : s) c = static_cast<char>(std::toupper(static_cast<unsigned char>(c)));
    return s;
}
std::string lower(std::string s) {
    for (auto& c : s) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
    return s;
}
struct Def {
    const char* name;
    ConfigItem::Type type;
    const char* def;
};
// the reference's items with their defaults, followed by the items specific to this runtime
const Def kDefs[] = {
    {"show_config_items", ConfigItem::BOOL, "false"},
    {"profiling", ConfigItem::BOOL, "false"},
    {"graph_profiling", ConfigItem::BOOL, "false"},
    {"profile_dump_path", ConfigItem::STRING, "test_default_config"},
    {"dump_graph", ConfigItem::BOOL, "false"},
    {"dump_graph_prefix", ConfigItem::STRING, "/tmp/rannc_graph"},
    {"partition_num", ConfigItem::INT, "0"},
    {"replica_num", ConfigItem::INT, "0"},
    {"pipeline_num", ConfigItem::INT, "0"},
    {"validate_comm", ConfigItem::BOOL, "false"},
    {"display_comm_value", ConfigItem::BOOL, "false"},
    {"display_act_value", ConfigItem::BOOL, "false"},
    {"consolidate_grads", ConfigItem::BOOL, "false"},
    {"profiling_iter", ConfigItem::INT, "3"},
    {"checkpointing", ConfigItem::BOOL, "false"},
    {"checkpointing_no_last", ConfigItem::BOOL, "false"},
    {"disable_balancing", ConfigItem::BOOL, "true"},
    {"opt_param_factor", ConfigItem::INT, "2"},
    {"auto_parallel", ConfigItem::BOOL, "false"},
    {"p2p_comm", ConfigItem::BOOL, "true"},
    {"decomposer", ConfigItem::STRING, "ml_part"},
    {"mem_limit_gb", ConfigItem::INT, "0"},
    {"min_partition_num", ConfigItem::INT, "5"},
    {"max_partition_num", ConfigItem::INT, "32"},
    {"mem_margin", ConfigItem::FLOAT, "0.1"},
    {"max_mp_num", ConfigItem::INT, "8"},
    {"do_uncoarsening", ConfigItem::BOOL, "false"},
    {"do_coarsening", ConfigItem::BOOL, "true"},
    {"min_pipeline", ConfigItem::INT, "1"},
    {"max_pipeline", ConfigItem::INT, "32"},
    {"save_deployment", ConfigItem::BOOL, "false"},
    {"load_deployment", ConfigItem::BOOL, "false"},
    {"deployment_file", ConfigItem::STRING, "/tmp/rannc_deployment.bin"},
    {"save_graph_profile", ConfigItem::BOOL, "false"},
    {"load_graph_profile", ConfigItem::BOOL, "false"},
    {"graph_profile_file", ConfigItem::STRING, "/tmp/rannc_graph_profiles.bin"},
    {"trace_events", ConfigItem::BOOL, "false"},
    {"event_trace_file", ConfigItem::STRING, "/tmp/rannc_event_trace.json"},
    {"verify_recomp", ConfigItem::BOOL, "false"},
    {"dp_search_all", ConfigItem::BOOL, "false"},
    {"min_pipeline_bs", ConfigItem::INT, "1"},
    {"coarsen_by_time", ConfigItem::BOOL, "true"},
    {"limit_dev_num_pot", ConfigItem::BOOL, "true"},
    {"limit_dev_num_more_than_bs", ConfigItem::BOOL, "true"},
    {"profile_by_acc", ConfigItem::BOOL, "false"},
    {"verify_partitioning", ConfigItem::BOOL, "false"},
    {"alloc_repl_flat", ConfigItem::BOOL, "true"},
    {"sync_allreduce", ConfigItem::BOOL, "false"},
    {"save_mlpart_results", ConfigItem::BOOL, "false"},
    {"load_mlpart_results", ConfigItem::BOOL, "false"},
    {"mlpart_results_file", ConfigItem::STRING, "/tmp/rannc_mlpart_results.bin"},
    {"save_alloc_solutions", ConfigItem::BOOL, "false"},
    {"load_alloc_solutions", ConfigItem::BOOL, "false"},
    {"alloc_solutions_file_prefix", ConfigItem::STRING, "/tmp/rannc_alloc_sols"},
    {"dump_dp_node_profiles", ConfigItem::STRING, ""},
    {"dump_dp_cache", ConfigItem::STRING, ""},
    {"partitioning_dry_run_np", ConfigItem::INT, "0"},
    {"use_mpi_to_gather_dist_params", ConfigItem::BOOL, "false"},
    {"run_watchdog", ConfigItem::BOOL, "false"},
    {"watchdog_lockfile_dir", ConfigItem::STRING, ""},
    {"force_dist_matmul", ConfigItem::BOOL, "false"},
    {"offload_chunk_numel", ConfigItem::INT, "33554432"},
    {"offload_param_window_mb", ConfigItem::INT, "0"},
    {"checkpoint_segments", ConfigItem::INT, "0"},
    {"conv_implicit_gemm", ConfigItem::BOOL, "true"},
    {"interleave_backward", ConfigItem::BOOL, "false"},
    {"conv_implicit_max_overhead", ConfigItem::FLOAT, "1.2"},
    {"use_named_tensors", ConfigItem::BOOL, "false"},
    {"profiler_cache_size", ConfigItem::INT, "0"},
    {"enable_kineto", ConfigItem::BOOL, "false"},
    {"conf_dir", ConfigItem::STRING, ""},
    // --- items of this runtime (no counterpart in the reference) ---
    {"fused_kernels", ConfigItem::BOOL, "true"},          // false: stock ATen ops + NCCL collectives
    {"fused_grad_allreduce", ConfigItem::BOOL, "true"},   // peer-memory reduce-scatter + Adam + all-gather
    {"measure_profiles", ConfigItem::BOOL, "true"},       // on a CUDA device: time operators and blocks when planning
    {"measure_subgraphs", ConfigItem::BOOL, "false"},     // the stage search measures its candidate stages
    {"max_measured_subgraphs", ConfigItem::INT, "64"},
    {"p2p_gbs", ConfigItem::FLOAT, "770"},                // stage <-> stage bandwidth, GB/s
    {"allreduce_gbs", ConfigItem::FLOAT, "725"},          // all-reduce bus bandwidth, GB/s
    {"dev_tflops", ConfigItem::FLOAT, "1388"},            // sustained bf16 GEMM throughput for estimates
    {"dev_hbm_gbs", ConfigItem::FLOAT, "6553"},           // copy bandwidth for estimates
    {"prefer_no_checkpointing", ConfigItem::BOOL, "true"},
    {"watchdog_period_s", ConfigItem::FLOAT, "10"},
    {"watchdog_stale_s", ConfigItem::FLOAT, "60"},
    {"comm_timeout_s", ConfigItem::FLOAT, "1800"},
    {"grad_bucket_mb", ConfigItem::FLOAT, "64"},          // gradient bytes per reduction bucket under ZeRO
    {"overlap_grad_reduce", ConfigItem::BOOL, "true"},    // reduce each bucket while backward still runs
    {"fused_update_in_backward", ConfigItem::BOOL, "true"},  // the overlapped launches also update + publish
    {"fused_reduce_ctas", ConfigItem::INT, "32"},         // CTAs of a reduction launch that overlaps backward
    {"comm_retry", ConfigItem::INT, "1"},                 // retries of a failed collective after re-creating groups
    {"comm_retry_wait_s", ConfigItem::FLOAT, "1"},
    {"check_device_error_every_step", ConfigItem::BOOL, "true"},
    {"keep_dist_params_sharded", ConfigItem::BOOL, "false"},  // dist_param weights of linear layers stay sliced
};
}  // namespace

std::map<std::string, std::string> Config::parseToml(const std::string& text) {
    std::map<std::string, std::string> kv;
    std::istringstream ss(text);
    std::string line;
    while (std::getline(ss, line)) {
        bool in_str = false;
        std::string clean;
        for (char c : line) {
            if (c == '"') in_str = !in_str;
            if (c == '#' && !in_str) break;
            clean.push_back(c);
        }
        clean = trim(clean);
        if (clean.empty() || clean[0] == '[') continue;
        const size_t eq = clean.find('=');
        if (eq == std::string::npos) continue;
        std::string key = trim(clean.substr(0, eq));
        std::string val = trim(clean.substr(eq + 1));
        if (val.size() >= 2 && ((val.front() == '"' && val.back() == '"') || (val.front() == '\'' && val.back() == '\'')))
            val = val.substr(1, val.size() - 2);
        kv[key] = val;
    }
    return kv;
}

Config::Config() { reload(); }

Config& Config::get() {
    static Config c;
    return c;
}

std::string Config::confDir() const {
    const char* e = std::getenv("RANNC_CONF_DIR");
    if (e && *e) return e;
    const char* home = std::getenv("HOME");
    return std::string(home ? home : ".") + "/.pyrannc";
}

void Config::reload() {
    std::lock_guard<std::mutex> lk(mu_);
    items_.clear();
    warnings_.clear();
    for (const auto& d : kDefs) {
        ConfigItem it;
        it.type = d.type;
        it.name = d.name;
        it.value = it.default_value = d.def;
        items_[it.name] = it;
    }
    const std::string dir = confDir();
    items_["conf_dir"].value = dir;
    std::ifstream f(dir + "/rannc_conf.toml");
    if (f) {
        std::stringstream buf;
        buf << f.rdbuf();
        for (const auto& kv : parseToml(buf.str())) {
            auto it = items_.find(kv.first);
            if (it == items_.end()) {
                warnings_.push_back("unknown config item ignored: " + kv.first);
                continue;
            }
            it->second.value = kv.second;
        }
    }
    for (auto& kv : items_) {
        const std::string env = "RANNC_" + upper(kv.first);
        const char* v = std::getenv(env.c_str());
        if (v) kv.second.value = v;
    }
}

const ConfigItem& Config::item(const std::string& name) const {
    auto it = items_.find(name);
    if (it == items_.end()) throw std::runtime_error("unknown config item: " + name);
    return it->second;
}
bool Config::has(const std::string& name) const {
    std::lock_guard<std::mutex> lk(mu_);
    return items_.count(name) != 0;
}
int64_t Config::getInt(const std::string& name) const {
    std::lock_guard<std::mutex> lk(mu_);
    return std::stoll(item(name).value);
}
double Config::getFloat(const std::string& name) const {
    std::lock_guard<std::mutex> lk(mu_);
    return std::stod(item(name).value);
}
bool Config::getBool(const std::string& name) const {
    std::lock_guard<std::mutex> lk(mu_);
    const std::string v = lower(item(name).value);
    return v == "true" || v == "1" || v == "yes" || v == "on";
}
std::string Config::getString(const std::string& name) const {
    std::lock_guard<std::mutex> lk(mu_);
    return item(name).value;
}
void Config::set(const std::string& name, const std::string& value) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = items_.find(name);
    if (it == items_.end()) throw std::runtime_error("unknown config item: " + name);
    it->second.value = value;
}
std::vector<ConfigItem> Config::items() const {
    std::lock_guard<std::mutex> lk(mu_);
    std::vector<ConfigItem> r;
    for (const auto& kv : items_) r.push_back(kv.second);
    return r;
}

// ---------------------------------------------------------------- logging
namespace {
std::mutex g_log_mu;
std::map<std::string, LogLevel> g_levels;
LogLevel g_default_level = LogLevel::INFO;
int g_log_rank = -1;
std::map<std::string, Logger*> g_loggers;
const char* levelName(LogLevel l) {
    switch (l) {
        case LogLevel::TRACE: return "trace";
        case LogLevel::DEBUG: return "debug";
        case LogLevel::INFO: return "info";
        case LogLevel::WARN: return "warning";
        case LogLevel::ERR: return "error";
        case LogLevel::CRITICAL: return "critical";
        default: return "off";
    }
}
}  // namespace

LogLevel parseLogLevel(const std::string& s) {
    const std::string l = lower(s);
    if (l == "trace") return LogLevel::TRACE;
    if (l == "debug") return LogLevel::DEBUG;
    if (l == "info") return LogLevel::INFO;
    if (l == "warn" || l == "warning") return LogLevel::WARN;
    if (l == "err" || l == "error") return LogLevel::ERR;
    if (l == "critical") return LogLevel::CRITICAL;
    return LogLevel::OFF;
}
bool Logger::enabled(LogLevel lv) const {
    std::lock_guard<std::mutex> lk(g_log_mu);
    auto it = g_levels.find(name_);
    const LogLevel th = it == g_levels.end() ? g_default_level : it->second;
    return static_cast<int>(lv) >= static_cast<int>(th);
}
void Logger::log(LogLevel lv, const std::string& msg) const {
    if (!enabled(lv)) return;
    // one write per line (ranks share the terminal), wall-clock time first as spdlog's default pattern does in
    // the reference
    const auto now = std::chrono::system_clock::now();
    const std::time_t tt = std::chrono::system_clock::to_time_t(now);
    const int ms = static_cast<int>(
        std::chrono::duration_cast<std::chrono::milliseconds>(now.time_since_epoch()).count() % 1000);
    std::tm tmv{};
    localtime_r(&tt, &tmv);
    char stamp[40];
    std::snprintf(stamp, sizeof stamp, "[%04d-%02d-%02d %02d:%02d:%02d.%03d] ", tmv.tm_year + 1900, tmv.tm_mon + 1,
                  tmv.tm_mday, tmv.tm_hour, tmv.tm_min, tmv.tm_sec, ms);
    std::ostringstream line;
    line << stamp << "[" << name_ << "] [" << levelName(lv) << "]";
    if (g_log_rank >= 0) line << " [rank " << g_log_rank << "]";
    line << " " << msg << "\n";
    const std::string text = line.str();
    std::lock_guard<std::mutex> lk(g_log_mu);
    std::cerr.write(text.data(), static_cast<std::streamsize>(text.size()));
    std::cerr.flush();
}
Logger& getLogger(const std::string& name) {
    std::lock_guard<std::mutex> lk(g_log_mu);
    auto it = g_loggers.find(name);
    if (it == g_loggers.end()) it = g_loggers.emplace(name, new Logger(name)).first;
    return *it->second;
}
void setLogLevel(const std::string& logger_name, LogLevel lv) {
    std::lock_guard<std::mutex> lk(g_log_mu);
    if (logger_name.empty()) g_default_level = lv;
    else g_levels[logger_name] = lv;
}
void setLogRank(int rank) {
    std::lock_guard<std::mutex> lk(g_log_mu);
    g_log_rank = rank;
}
void configureLoggingFromToml(const std::string& text) {
    // [[logger]] tables with name / level keys; a `global_level`-style top key sets the default
    std::istringstream ss(text);
    std::string line, cur_name, cur_level;
    bool in_logger = false;
    auto flush = [&]() {
        if (in_logger && !cur_name.empty() && !cur_level.empty()) setLogLevel(cur_name, parseLogLevel(cur_level));
        cur_name.clear();
        cur_level.clear();
    };
    while (std::getline(ss, line)) {
        std::string t = trim(line);
        if (t.empty() || t[0] == '#') continue;
        if (t[0] == '[') {
            flush();
            in_logger = t.find("logger") != std::string::npos;
            continue;
        }
        auto kv = Config::parseToml(t);
        for (const auto& p : kv) {
            if (p.first == "name") cur_name = p.second;
            else if (p.first == "level") {
                if (in_logger) cur_level = p.second;
                else setLogLevel("", parseLogLevel(p.second));
            } else if (p.first == "global_level") setLogLevel("", parseLogLevel(p.second));
        }
    }
    flush();
}

// ---------------------------------------------------------------- event recorder
static int64_t nowUs() {
    return std::chrono::duration_cast<std::chrono::microseconds>(
               std::chrono::system_clock::now().time_since_epoch())
        .count();
}
EventRecorder& EventRecorder::get() {
    static EventRecorder r;
    return r;
}
void EventRecorder::begin(const std::string& name, int tid) {
    if (!enabled_) return;
    std::lock_guard<std::mutex> lk(mu_);
    if (events_.size() < kMaxEvents) events_.push_back({name, 'B', nowUs(), tid});
}
void EventRecorder::end(const std::string& name, int tid) {
    if (!enabled_) return;
    std::lock_guard<std::mutex> lk(mu_);
    if (events_.size() < kMaxEvents) events_.push_back({name, 'E', nowUs(), tid});
}
size_t EventRecorder::size() const {
    std::lock_guard<std::mutex> lk(mu_);
    return events_.size();
}
void EventRecorder::clear() {
    std::lock_guard<std::mutex> lk(mu_);
    events_.clear();
}
static std::string jsonEscape(const std::string& s) {
    std::string o;
    for (char c : s) {
        if (c == '"' || c == '\\') o.push_back('\\');
        if (c == '\n') { o += "\\n"; continue; }
        o.push_back(c);
    }
    return o;
}
std::string EventRecorder::dumpLocal(int rank) const {
    std::lock_guard<std::mutex> lk(mu_);
    std::ostringstream ss;
    bool first = true;
    for (const auto& e : events_) {
        if (!first) ss << ",";
        first = false;
        ss << "{\"name\":\"" << jsonEscape(e.name) << "\",\"cat\":\"rannc\",\"ph\":\"" << e.phase
           << "\",\"ts\":" << e.ts_us << ",\"pid\":" << rank << ",\"tid\":" << e.tid << "}";
    }
    return ss.str();
}
std::string EventRecorder::merge(const std::vector<std::string>& fragments) {
    std::ostringstream ss;
    ss << "{\"traceEvents\":[";
    bool first = true;
    for (const auto& f : fragments) {
        if (f.empty()) continue;
        if (!first) ss << ",";
        first = false;
        ss << f;
    }
    ss << "]}";
    return ss.str();
}
std::string funcKey(const std::string& func, const std::string& graph, int split, bool bwd) {
    std::ostringstream ss;
    ss << func << "[graph=" << graph << ",split=" << split << "," << (bwd ? "bwd" : "fwd") << "]";
    return ss.str();
}
std::string commKey(const std::string& func, const std::string& value, int split, bool bwd) {
    std::ostringstream ss;
    ss << func << "[value=" << value << ",split=" << split << "," << (bwd ? "bwd" : "fwd") << "]";
    return ss.str();
}

// ---------------------------------------------------------------- time counter
void TimeCounter::start(const std::string& name) {
    if (!enabled_) return;
    std::lock_guard<std::mutex> lk(mu_);
    Acc& a = acc_[name];
    a.t0 = std::chrono::steady_clock::now();
    a.running = true;
}
void TimeCounter::stop(const std::string& name) {
    if (!enabled_) return;
    std::lock_guard<std::mutex> lk(mu_);
    auto it = acc_.find(name);
    if (it == acc_.end() || !it->second.running) return;
    it->second.total_us +=
        std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - it->second.t0).count();
    it->second.count++;
    it->second.running = false;
}
int64_t TimeCounter::totalUs(const std::string& name) const {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = acc_.find(name);
    return it == acc_.end() ? 0 : it->second.total_us;
}
int64_t TimeCounter::count(const std::string& name) const {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = acc_.find(name);
    return it == acc_.end() ? 0 : it->second.count;
}
std::string TimeCounter::summary() const {
    std::lock_guard<std::mutex> lk(mu_);
    std::ostringstream ss;
    for (const auto& kv : acc_) {
        const double avg = kv.second.count ? static_cast<double>(kv.second.total_us) / kv.second.count : 0.0;
        ss << kv.first << ": total=" << kv.second.total_us << "us count=" << kv.second.count << " avg=" << avg
           << "us\n";
    }
    return ss.str();
}
void TimeCounter::clear() {
    std::lock_guard<std::mutex> lk(mu_);
    acc_.clear();
}

// ---------------------------------------------------------------- watchdog
std::string Watchdog::lockPath(const std::string& dir, int rank) {
    return dir + "/rannc_" + std::to_string(rank) + ".lock";
}
Watchdog::~Watchdog() { stop(false); }
static void touchFile(const std::string& path) {
    std::ofstream f(path, std::ios::trunc);
    f << nowUs();
}
void Watchdog::start(const std::string& dir, int rank, int world_size, double period_s, double stale_s,
                     std::function<void(int)> on_failure) {
    stop(false);
    dir_ = dir;
    rank_ = rank;
    world_ = world_size;
    period_s_ = period_s;
    stale_s_ = stale_s;
    on_failure_ = std::move(on_failure);
    failed_peer_ = -1;
    touchFile(lockPath(dir_, rank_));
    running_ = true;
    th_ = std::thread([this] { loop(); });
}
void Watchdog::stop(bool remove_own_file) {
    const bool was = running_.exchange(false);
    if (th_.joinable()) th_.join();
    if (was && remove_own_file) ::unlink(lockPath(dir_, rank_).c_str());
}
void Watchdog::loop() {
    const auto step = std::chrono::milliseconds(20);
    auto next = std::chrono::steady_clock::now();
    // give the peers one period to create their files
    auto armed_at = std::chrono::steady_clock::now() + std::chrono::duration<double>(period_s_);
    while (running_) {
        std::this_thread::sleep_for(step);
        const auto now = std::chrono::steady_clock::now();
        if (now < next) continue;
        next = now + std::chrono::duration_cast<std::chrono::steady_clock::duration>(
                         std::chrono::duration<double>(period_s_));
        touchFile(lockPath(dir_, rank_));
        if (now < armed_at) continue;
        for (int r = 0; r < world_ && running_; ++r) {
            if (r == rank_) continue;
            struct stat st;
            bool bad = ::stat(lockPath(dir_, r).c_str(), &st) != 0;
            if (!bad) {
                const double age = std::difftime(::time(nullptr), st.st_mtime);
                bad = age > stale_s_;
            }
            if (bad) {
                failed_peer_ = r;
                running_ = false;
                if (on_failure_) on_failure_(r);
                return;
            }
        }
    }
}

int64_t residentMemBytes() {
    std::ifstream f("/proc/self/statm");
    long pages = 0, rss = 0;
    if (!(f >> pages >> rss)) return 0;
    return static_cast<int64_t>(rss) * ::sysconf(_SC_PAGESIZE);
}

}  // namespace rannc
