#include "util.h"

#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>

namespace pccl {

std::string Environs::get(const std::string& name, const std::string& fallback) {
  const char* v = std::getenv(name.c_str());
  return (v && *v) ? std::string(v) : fallback;
}

int64_t Environs::get_int(const std::string& name, int64_t fallback) {
  const std::string v = get(name);
  if (v.empty()) return fallback;
  char* end = nullptr;
  long long parsed = std::strtoll(v.c_str(), &end, 10);
  if (end == v.c_str()) return fallback;
  // Accept K / M / G suffixes for sizes.
  switch (*end) {
    case 'k': case 'K': parsed <<= 10; break;
    case 'm': case 'M': parsed <<= 20; break;
    case 'g': case 'G': parsed <<= 30; break;
    default: break;
  }
  return parsed;
}

bool Environs::get_flag(const std::string& name, bool fallback) {
  std::string v = get(name);
  if (v.empty()) return fallback;
  std::transform(v.begin(), v.end(), v.begin(), ::tolower);
  return !(v == "0" || v == "false" || v == "off" || v == "no");
}

std::string Environs::require(const std::string& name) {
  const char* v = std::getenv(name.c_str());
  if (!v) throw Error("environment variable " + name + " is not set");
  return v;
}

namespace {
std::mutex& registry_mutex() { static std::mutex m; return m; }
std::map<std::string, std::string>& registry() { static std::map<std::string, std::string> r; return r; }
}  // namespace

void Environs::register_option(const std::string& name, const std::string& description) {
  std::lock_guard<std::mutex> lock(registry_mutex());
  registry()[name] = description;
}

std::map<std::string, std::string> Environs::list_options() {
  std::lock_guard<std::mutex> lock(registry_mutex());
  return registry();
}

LogLevel log_level() {
  static const LogLevel level = [] {
    std::string v = Environs::get("PCCL_LOG_LEVEL", "WARN");
    std::transform(v.begin(), v.end(), v.begin(), ::toupper);
    if (v == "TRACE") return LogLevel::kTrace;
    if (v == "DEBUG") return LogLevel::kDebug;
    if (v == "INFO") return LogLevel::kInfo;
    if (v == "ERROR") return LogLevel::kError;
    if (v == "CRITICAL") return LogLevel::kCritical;
    if (v == "OFF") return LogLevel::kOff;
    return LogLevel::kWarn;
  }();
  return level;
}

void log_write(LogLevel level, const std::string& message) {
  static const char* names[] = {"trace", "debug", "info", "warn", "error", "critical", "off"};
  static std::mutex m;
  const auto now = std::chrono::system_clock::now().time_since_epoch();
  const long long ms = std::chrono::duration_cast<std::chrono::milliseconds>(now).count();
  std::lock_guard<std::mutex> lock(m);
  std::fprintf(stderr, "[pccl %lld.%03lld %s] %s\n", ms / 1000, ms % 1000,
               names[static_cast<int>(level)], message.c_str());
}

std::string to_hex(const void* data, size_t bytes) {
  static const char digits[] = "0123456789abcdef";
  const auto* p = static_cast<const uint8_t*>(data);
  std::string out(bytes * 2, '0');
  for (size_t i = 0; i < bytes; ++i) {
    out[2 * i] = digits[p[i] >> 4];
    out[2 * i + 1] = digits[p[i] & 15];
  }
  return out;
}

std::vector<uint8_t> from_hex(const std::string& hex) {
  if (hex.size() % 2) throw Error("hex string has odd length");
  auto nibble = [](char c) -> int {
    if (c >= '0' && c <= '9') return c - '0';
    if (c >= 'a' && c <= 'f') return c - 'a' + 10;
    if (c >= 'A' && c <= 'F') return c - 'A' + 10;
    throw Error("invalid hex digit");
  };
  std::vector<uint8_t> out(hex.size() / 2);
  for (size_t i = 0; i < out.size(); ++i)
    out[i] = static_cast<uint8_t>(nibble(hex[2 * i]) << 4 | nibble(hex[2 * i + 1]));
  return out;
}

NvtxRange::NvtxRange(const char* name) { nvtxRangePushA(name); }
NvtxRange::~NvtxRange() { nvtxRangePop(); }

}  // namespace pccl
