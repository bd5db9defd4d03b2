// Host-side runtime utilities: configuration, named loggers, event trace,
// time counters and the peer-liveness watchdog.
#pragma once
#include <atomic>
#include <chrono>
#include <cstdint>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace rannc {

// ---- configuration (reference: src/Config.cpp:133-280) ---------------------
// Typed items with defaults; values come from <conf_dir>/rannc_conf.toml and are
// overridden by environment variables RANNC_<UPPERCASE_NAME>.
struct ConfigItem {
    enum Type { INT, FLOAT, BOOL, STRING } type = STRING;
    std::string name;
    std::string value;  // canonical text form
    std::string default_value;
};

class Config {
public:
    static Config& get();
    void reload();  // defaults -> toml -> environment
    bool has(const std::string& name) const;
    int64_t getInt(const std::string& name) const;
    double getFloat(const std::string& name) const;
    bool getBool(const std::string& name) const;
    std::string getString(const std::string& name) const;
    void set(const std::string& name, const std::string& value);  // programmatic override (tests)
    std::vector<ConfigItem> items() const;
    std::string confDir() const;
    std::vector<std::string> warnings() const { return warnings_; }
    // minimal TOML subset: `key = value` lines, comments, strings, ints, floats, booleans
    static std::map<std::string, std::string> parseToml(const std::string& text);

private:
    Config();
    const ConfigItem& item(const std::string& name) const;
    std::map<std::string, ConfigItem> items_;
    std::vector<std::string> warnings_;
    mutable std::mutex mu_;
};

// ---- logging (reference: src/Logging.cpp:26-47, documents/logging.rst) -----
enum class LogLevel : int { TRACE = 0, DEBUG, INFO, WARN, ERR, CRITICAL, OFF };
class Logger {
public:
    explicit Logger(std::string name) : name_(std::move(name)) {}
    void log(LogLevel lv, const std::string& msg) const;
    bool enabled(LogLevel lv) const;
    const std::string& name() const { return name_; }

private:
    std::string name_;
};
Logger& getLogger(const std::string& name);
void setLogLevel(const std::string& logger_name, LogLevel lv);  // "" = default of every logger
void setLogRank(int rank);
LogLevel parseLogLevel(const std::string& s);
// reads `[[logger]] name = "...", level = "..."` tables of a logging.toml
void configureLoggingFromToml(const std::string& text);

// ---- event trace (reference: src/comp/EventRecorder.cpp:49-99) --------------
struct TraceEventRec {
    std::string name;
    char phase;  // 'B' or 'E'
    int64_t ts_us;
    int tid;
};
class EventRecorder {
public:
    static EventRecorder& get();
    void enable(bool on) { enabled_ = on; }
    bool enabled() const { return enabled_; }
    void begin(const std::string& name, int tid = 0);
    void end(const std::string& name, int tid = 0);
    size_t size() const;
    void clear();
    // events of this rank as a JSON array fragment (no brackets); pid = rank
    std::string dumpLocal(int rank) const;
    // full Chrome-trace document from the fragments of every rank
    static std::string merge(const std::vector<std::string>& fragments);
    static constexpr size_t kMaxEvents = 100000;

private:
    std::atomic<bool> enabled_{false};
    mutable std::mutex mu_;
    std::vector<TraceEventRec> events_;
};
std::string funcKey(const std::string& func, const std::string& graph, int split, bool bwd);
std::string commKey(const std::string& func, const std::string& value, int split, bool bwd);

// ---- time counters (reference: src/comp/TimeCounter.cpp) --------------------
class TimeCounter {
public:
    explicit TimeCounter(bool enable = true) : enabled_(enable) {}
    void start(const std::string& name);
    void stop(const std::string& name);
    int64_t totalUs(const std::string& name) const;
    int64_t count(const std::string& name) const;
    std::string summary() const;
    void clear();

private:
    struct Acc {
        int64_t total_us = 0, count = 0;
        std::chrono::steady_clock::time_point t0;
        bool running = false;
    };
    bool enabled_;
    mutable std::mutex mu_;
    std::map<std::string, Acc> acc_;
};

// ---- watchdog (reference: src/cuda/CudaSync.cpp:22-112) ---------------------
// Every rank keeps a heartbeat file <dir>/rannc_<rank>.lock fresh; a thread
// checks the peers' files and calls `on_failure` when one is missing or stale,
// so that blocked collectives can be aborted.  Removing the own file is how a
// failing rank tells the others.
class Watchdog {
public:
    Watchdog() = default;
    ~Watchdog();
    void start(const std::string& dir, int rank, int world_size, double period_s, double stale_s,
               std::function<void(int)> on_failure);
    void stop(bool remove_own_file);
    bool running() const { return running_; }
    int failedPeer() const { return failed_peer_; }
    static std::string lockPath(const std::string& dir, int rank);

private:
    void loop();
    std::string dir_;
    int rank_ = 0, world_ = 1;
    double period_s_ = 10, stale_s_ = 60;
    std::function<void(int)> on_failure_;
    std::atomic<bool> running_{false};
    std::atomic<int> failed_peer_{-1};
    std::thread th_;
};

int64_t residentMemBytes();  // RSS of this process (reference: src/Common.cpp:216-238)

}  // namespace rannc
