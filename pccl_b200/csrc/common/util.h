// Process-wide utilities: environment options, leveled logging, hex encoding,
// NVTX ranges.  Option names match the reference's environment variables
// (reference: csrc/common/environ.cc:10-21, csrc/common/logging.cc:6-35,
// csrc/common/serialize.cc:6-57, include/common/nvtx.h:7-16).
#pragma once
#include <cstdint>
#include <cstdio>
#include <map>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace pccl {

// ---- environment ------------------------------------------------------------------------------
class Environs {
 public:
  // Value of `name`, or `fallback` when unset / empty.
  static std::string get(const std::string& name, const std::string& fallback = "");
  static int64_t get_int(const std::string& name, int64_t fallback);
  static bool get_flag(const std::string& name, bool fallback = false);
  // Throws std::runtime_error naming the variable when it is unset.
  static std::string require(const std::string& name);
  // Registry of documented options (name -> description), exposed to Python.
  static void register_option(const std::string& name, const std::string& description);
  static std::map<std::string, std::string> list_options();
};

// ---- logging ------------------------------------------------------------------------------------
enum class LogLevel { kTrace = 0, kDebug, kInfo, kWarn, kError, kCritical, kOff };
LogLevel log_level();                       // from PCCL_LOG_LEVEL, default WARN
void log_write(LogLevel level, const std::string& message);

#define PCCL_LOG(LEVEL, ...)                                                      \
  do {                                                                            \
    if (::pccl::LogLevel::LEVEL >= ::pccl::log_level()) {                         \
      std::ostringstream pccl_log_stream;                                         \
      pccl_log_stream << __VA_ARGS__;                                             \
      ::pccl::log_write(::pccl::LogLevel::LEVEL, pccl_log_stream.str());          \
    }                                                                             \
  } while (0)
#define PCCL_LOG_DEBUG(...) PCCL_LOG(kDebug, __VA_ARGS__)
#define PCCL_LOG_INFO(...) PCCL_LOG(kInfo, __VA_ARGS__)
#define PCCL_LOG_WARN(...) PCCL_LOG(kWarn, __VA_ARGS__)
#define PCCL_LOG_ERROR(...) PCCL_LOG(kError, __VA_ARGS__)

// ---- errors -------------------------------------------------------------------------------------
struct Error : std::runtime_error { using std::runtime_error::runtime_error; };
struct TimeoutError : Error { using Error::Error; };

#define PCCL_CHECK(COND, ...)                                                     \
  do {                                                                            \
    if (!(COND)) {                                                                \
      std::ostringstream pccl_chk_stream;                                         \
      pccl_chk_stream << __VA_ARGS__;                                             \
      throw ::pccl::Error(pccl_chk_stream.str());                                 \
    }                                                                             \
  } while (0)

// ---- hex ------------------------------------------------------------------------------------------
std::string to_hex(const void* data, size_t bytes);
std::vector<uint8_t> from_hex(const std::string& hex);

// ---- NVTX -------------------------------------------------------------------------------------------
// RAII range; a no-op unless a profiler injected the NVTX library.
class NvtxRange {
 public:
  explicit NvtxRange(const char* name);
  ~NvtxRange();
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

}  // namespace pccl
