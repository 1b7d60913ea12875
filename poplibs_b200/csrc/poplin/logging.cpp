// Logging front end: levels and destinations are taken from the environment
// variables the reference reads (lib/poplibs_support/logging.cpp:118-171).
#include "poplibs_support/logging.hpp"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace poplibs_support {
namespace logging {

namespace {

const char *const moduleNames[] = {"POPFLOAT", "POPLIN", "POPNN", "POPOPS",
                                   "POPRAND", "POPSPARSE", "POPUTIL"};
const char *const levelNames[] = {"T", "D", "I", "W", "E", "C", "O"};

Level parseLevel(const char *s, Level dflt) {
  if (!s) return dflt;
  static const struct { const char *name; Level level; } table[] = {
      {"TRACE", Level::Trace}, {"DEBUG", Level::Debug}, {"INFO", Level::Info},
      {"WARN", Level::Warn},   {"ERR", Level::Err},     {"OFF", Level::Off}, {"", Level::Off}};
  for (const auto &e : table)
    if (std::strcmp(s, e.name) == 0) return e.level;
  std::fprintf(stderr, "Unknown POPLIBS log level '%s': expected TRACE, DEBUG, INFO, WARN, ERR or OFF\n", s);
  return dflt;
}

struct State {
  Level levels[int(Module::size)];
  std::FILE *dest = stderr;
  std::mutex mutex;
  State() {
    const Level base = parseLevel(std::getenv("POPLIBS_LOG_LEVEL"), Level::Off);
    for (int m = 0; m < int(Module::size); ++m) {
      const std::string var = std::string("POPLIBS_") + moduleNames[m] + "_LOG_LEVEL";
      levels[m] = parseLevel(std::getenv(var.c_str()), base);
    }
    if (const char *d = std::getenv("POPLIBS_LOG_DEST")) {
      if (std::strcmp(d, "stdout") == 0) dest = stdout;
      else if (std::strcmp(d, "stderr") == 0) dest = stderr;
      else if (std::FILE *f = std::fopen(d, "a")) dest = f;
    }
  }
};

State &state() {
  static State s;
  return s;
}

}  // namespace

bool shouldLog(Module m, Level l) { return l != Level::Off && l >= state().levels[int(m)]; }

void log(Module m, Level l, const std::string &msg) {
  if (!shouldLog(m, l)) return;
  State &s = state();
  std::lock_guard<std::mutex> lock(s.mutex);
  std::fprintf(s.dest, "PL:%s [%s] %s\n", moduleNames[int(m)], levelNames[int(l)], msg.c_str());
  std::fflush(s.dest);
}

}  // namespace logging
}  // namespace poplibs_support
