#include "log.h"

#include <algorithm>
#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unistd.h>

namespace xccl {

static const char *const kLevelNames[LOG_LEVEL_LAST] = {"FATAL", "ERROR", "WARN", "INFO", "DEBUG", "TRACE"};

const char *log_level_name(int level)
{
    return (level >= 0 && level < LOG_LEVEL_LAST) ? kLevelNames[level] : "?";
}

int parse_log_level(const std::string &s, int dflt)
{
    std::string u(s);
    std::transform(u.begin(), u.end(), u.begin(), [](unsigned char c) { return std::toupper(c); });
    for (int i = 0; i < LOG_LEVEL_LAST; i++) {
        if (u == kLevelNames[i]) {
            return i;
        }
    }
    if (u == "WARNING") return LOG_WARN;
    if (u == "DATA" || u == "POLL" || u == "REQ" || u == "FUNC") return LOG_TRACE;
    if (!u.empty() && std::isdigit((unsigned char)u[0])) {
        return std::min(std::max(std::atoi(u.c_str()), 0), (int)LOG_TRACE);
    }
    return dflt;
}

LogComponent &global_log()
{
    static LogComponent c = [] {
        LogComponent g{"XCCL", LOG_WARN};
        const char  *e = std::getenv("XCCL_LOG_LEVEL");
        if (e != nullptr) {
            g.level = parse_log_level(e, LOG_WARN);
        }
        return g;
    }();
    return c;
}

static FILE *log_stream()
{
    static FILE *f = [] {
        const char *path = std::getenv("XCCL_LOG_FILE");
        if (path != nullptr && path[0] != '\0') {
            std::string p(path);
            size_t      pos = p.find("%p");
            if (pos != std::string::npos) {
                p.replace(pos, 2, std::to_string((long)getpid()));
            }
            FILE *out = std::fopen(p.c_str(), "a");
            if (out != nullptr) {
                return out;
            }
        }
        return stderr;
    }();
    return f;
}

void log_write(const LogComponent &c, int level, const char *file, int line, const char *fmt, ...)
{
    static std::mutex mu;
    char              msg[1024];
    va_list           ap;
    va_start(ap, fmt);
    std::vsnprintf(msg, sizeof(msg), fmt, ap);
    va_end(ap);
    const char *base = std::strrchr(file, '/');
    base             = (base != nullptr) ? base + 1 : file;
    std::lock_guard<std::mutex> lock(mu);
    std::fprintf(log_stream(), "[%ld] %-5s %s %s:%d  %s\n", (long)getpid(), log_level_name(level), c.name, base,
                 line, msg);
    std::fflush(log_stream());
}

}  // namespace xccl
