// Leveled, timestamped logging to stderr for the host runtime.
// The level comes from the environment variable LYAPUNOV_LOG
// (debug, info, warn, error; default warn).  The reference has a Logger
// singleton with the same four levels (csrc/include/utils/logging.hpp:30-73).
#pragma once

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

namespace lyapunov::host {

enum class LogLevel : int { kDebug = 0, kInfo = 1, kWarn = 2, kError = 3 };

class Log {
public:
  static Log &get() {
    static Log instance;
    return instance;
  }
  bool enabled(LogLevel level) const { return static_cast<int>(level) >= static_cast<int>(level_); }
  void set_level(LogLevel level) { level_ = level; }
  void write(LogLevel level, const std::string &text) {
    if (!enabled(level)) return;
    static const char *names[] = {"debug", "info", "warn", "error"};
    using clock = std::chrono::system_clock;
    const double now = std::chrono::duration<double>(clock::now().time_since_epoch()).count();
    std::lock_guard<std::mutex> guard(mutex_);
    std::fprintf(stderr, "[lyapunov %.3f %s] %s\n", now, names[static_cast<int>(level)], text.c_str());
  }

private:
  Log() {
    const char *env = std::getenv("LYAPUNOV_LOG");
    if (env == nullptr) return;
    if (!std::strcmp(env, "debug")) level_ = LogLevel::kDebug;
    else if (!std::strcmp(env, "info")) level_ = LogLevel::kInfo;
    else if (!std::strcmp(env, "error")) level_ = LogLevel::kError;
  }
  LogLevel level_{LogLevel::kWarn};
  std::mutex mutex_;
};

inline void log(LogLevel level, const std::string &text) { Log::get().write(level, text); }

}  // namespace lyapunov::host
