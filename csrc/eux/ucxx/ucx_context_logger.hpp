// Logging: an interface, a default logger that prints ERROR and above to
// stderr and drops the rest, a process-wide manager, and stream-style macros
// (reference: ucx_context/ucx_context_logger.hpp, macros at :319-330).
#pragma once

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <string_view>

namespace eux::ucxx {

enum class LogLevel : int { TRACE = 0, DEBUG = 1, INFO = 2, WARN = 3, ERROR = 4, FATAL = 5, OFF = 6 };

inline const char* to_string(LogLevel l) {
  switch (l) {
    case LogLevel::TRACE: return "TRACE";
    case LogLevel::DEBUG: return "DEBUG";
    case LogLevel::INFO: return "INFO";
    case LogLevel::WARN: return "WARN";
    case LogLevel::ERROR: return "ERROR";
    case LogLevel::FATAL: return "FATAL";
    default: return "OFF";
  }
}

class UcxLogger {
 public:
  virtual ~UcxLogger() = default;
  virtual void log(LogLevel level, std::string_view component, std::string_view message) = 0;
  virtual bool enabled(LogLevel level) const = 0;
};

class DefaultUcxLogger final : public UcxLogger {
 public:
  explicit DefaultUcxLogger(LogLevel threshold = LogLevel::ERROR) : threshold_(threshold) {}
  void set_threshold(LogLevel l) { threshold_.store(l); }
  bool enabled(LogLevel level) const override { return level >= threshold_.load(std::memory_order_relaxed); }
  void log(LogLevel level, std::string_view component, std::string_view message) override {
    if (!enabled(level)) return;
    std::lock_guard lk(mu_);
    std::fprintf(stderr, "[%s][%.*s] %.*s\n", to_string(level), (int)component.size(), component.data(),
                 (int)message.size(), message.data());
  }

 private:
  std::atomic<LogLevel> threshold_;
  std::mutex mu_;
};

class UcxLoggerManager {
 public:
  static UcxLoggerManager& instance() {
    static UcxLoggerManager m;
    return m;
  }
  std::shared_ptr<UcxLogger> get() {
    std::lock_guard lk(mu_);
    return logger_;
  }
  void set(std::shared_ptr<UcxLogger> l) {
    std::lock_guard lk(mu_);
    logger_ = l ? std::move(l) : std::make_shared<DefaultUcxLogger>();
  }

 private:
  // EUX_LOG_LEVEL=TRACE|DEBUG|INFO|WARN|ERROR|FATAL|OFF sets the default logger's threshold
  UcxLoggerManager() : logger_(std::make_shared<DefaultUcxLogger>(level_from_env())) {}
  static LogLevel level_from_env() {
    const char* e = std::getenv("EUX_LOG_LEVEL");
    if (!e) return LogLevel::ERROR;
    const std::string_view v(e);
    for (int l = 0; l <= static_cast<int>(LogLevel::OFF); ++l)
      if (v == to_string(static_cast<LogLevel>(l))) return static_cast<LogLevel>(l);
    return LogLevel::ERROR;
  }
  std::mutex mu_;
  std::shared_ptr<UcxLogger> logger_;
};

// Collects a message with operator<< and emits it when the temporary dies.
class LogLine {
 public:
  LogLine(LogLevel level, std::string_view component) : level_(level), component_(component) {
    logger_ = UcxLoggerManager::instance().get();
    on_ = logger_ && logger_->enabled(level);
  }
  ~LogLine() {
    if (on_) logger_->log(level_, component_, ss_.str());
  }
  template <class T>
  LogLine& operator<<(const T& v) {
    if (on_) ss_ << v;
    return *this;
  }

 private:
  LogLevel level_;
  std::string_view component_;
  std::shared_ptr<UcxLogger> logger_;
  bool on_ = false;
  std::ostringstream ss_;
};

}  // namespace eux::ucxx

#define UCX_CTX_TRACE ::eux::ucxx::LogLine(::eux::ucxx::LogLevel::TRACE, "ctx")
#define UCX_CTX_DEBUG ::eux::ucxx::LogLine(::eux::ucxx::LogLevel::DEBUG, "ctx")
#define UCX_CTX_INFO ::eux::ucxx::LogLine(::eux::ucxx::LogLevel::INFO, "ctx")
#define UCX_CTX_WARN ::eux::ucxx::LogLine(::eux::ucxx::LogLevel::WARN, "ctx")
#define UCX_CTX_ERROR ::eux::ucxx::LogLine(::eux::ucxx::LogLevel::ERROR, "ctx")
#define UCX_CONN_TRACE ::eux::ucxx::LogLine(::eux::ucxx::LogLevel::TRACE, "conn")
#define UCX_CONN_DEBUG ::eux::ucxx::LogLine(::eux::ucxx::LogLevel::DEBUG, "conn")
#define UCX_CONN_INFO ::eux::ucxx::LogLine(::eux::ucxx::LogLevel::INFO, "conn")
#define UCX_CONN_WARN ::eux::ucxx::LogLine(::eux::ucxx::LogLevel::WARN, "conn")
#define UCX_CONN_ERROR ::eux::ucxx::LogLine(::eux::ucxx::LogLevel::ERROR, "conn")
