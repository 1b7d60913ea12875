// Logging with the environment variables of the reference's
// lib/poplibs_support/logging.cpp:118-171: POPLIBS_LOG_LEVEL,
// POPLIBS_POPLIN_LOG_LEVEL (overrides it for the poplin module) and
// POPLIBS_LOG_DEST ("stdout", "stderr" or a file name).  Levels: TRACE, DEBUG,
// INFO, WARN, ERR, OFF.
#ifndef poplibs_support_logging_hpp
#define poplibs_support_logging_hpp

#include <string>

namespace poplibs_support {
namespace logging {

enum class Level { Trace = 0, Debug = 1, Info = 2, Warn = 3, Err = 4, Critical = 5, Off = 6 };
enum class Module { popfloat, poplin, popnn, popops, poprand, popsparse, poputil, size };

bool shouldLog(Module m, Level l);
void log(Module m, Level l, const std::string &msg);

namespace poplin {
inline void trace(const std::string &s) { log(Module::poplin, Level::Trace, s); }
inline void debug(const std::string &s) { log(Module::poplin, Level::Debug, s); }
inline void info(const std::string &s) { log(Module::poplin, Level::Info, s); }
inline void warn(const std::string &s) { log(Module::poplin, Level::Warn, s); }
inline void err(const std::string &s) { log(Module::poplin, Level::Err, s); }
} // namespace poplin

} // namespace logging
} // namespace poplibs_support

#endif // poplibs_support_logging_hpp
