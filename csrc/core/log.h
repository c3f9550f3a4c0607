// Leveled, per-component logging owned by the library (the reference borrows UCS logging,
// src/utils/xccl_log.h:13-27). Levels come from XCCL_LOG_LEVEL and, per team library,
// XCCL_TEAM_<TL>_LOG_LEVEL. Messages go to stderr, or to the file named by XCCL_LOG_FILE.
#pragma once
#include <cstdarg>
#include <string>

namespace xccl {

enum LogLevel { LOG_FATAL = 0, LOG_ERROR, LOG_WARN, LOG_INFO, LOG_DEBUG, LOG_TRACE, LOG_LEVEL_LAST };

struct LogComponent {
    const char *name;
    int         level;
};

LogComponent &global_log();
int           parse_log_level(const std::string &s, int dflt);
const char   *log_level_name(int level);
void          log_write(const LogComponent &c, int level, const char *file, int line, const char *fmt, ...)
    __attribute__((format(printf, 5, 6)));

}  // namespace xccl

#define XCCL_LOG_AT(comp, lvl, ...)                                              \
    do {                                                                         \
        if ((lvl) <= (comp).level) {                                             \
            ::xccl::log_write((comp), (lvl), __FILE__, __LINE__, __VA_ARGS__);   \
        }                                                                        \
    } while (0)

#define xccl_error(...) XCCL_LOG_AT(::xccl::global_log(), ::xccl::LOG_ERROR, __VA_ARGS__)
#define xccl_warn(...)  XCCL_LOG_AT(::xccl::global_log(), ::xccl::LOG_WARN, __VA_ARGS__)
#define xccl_info(...)  XCCL_LOG_AT(::xccl::global_log(), ::xccl::LOG_INFO, __VA_ARGS__)
#define xccl_debug(...) XCCL_LOG_AT(::xccl::global_log(), ::xccl::LOG_DEBUG, __VA_ARGS__)
#define xccl_trace(...) XCCL_LOG_AT(::xccl::global_log(), ::xccl::LOG_TRACE, __VA_ARGS__)
