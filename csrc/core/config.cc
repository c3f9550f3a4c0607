#include "config.h"

#include <algorithm>
#include <cctype>
#include <climits>
#include <cstdlib>
#include <cstring>
#include <fstream>

#include "log.h"

namespace xccl {

static std::string lower(std::string s)
{
    std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return std::tolower(c); });
    return s;
}

long long parse_memunits(const std::string &in, bool *ok)
{
    std::string s = lower(in);
    if (ok != nullptr) *ok = true;
    if (s == "inf" || s == "infinity" || s == "auto") {
        return LLONG_MAX;
    }
    char     *end = nullptr;
    double    v   = std::strtod(s.c_str(), &end);
    long long mul = 1;
    if (end == s.c_str()) {
        if (ok != nullptr) *ok = false;
        return 0;
    }
    while (*end == ' ') end++;
    switch (*end) {
    case 'k': mul = 1ll << 10; end++; break;
    case 'm': mul = 1ll << 20; end++; break;
    case 'g': mul = 1ll << 30; end++; break;
    case 't': mul = 1ll << 40; end++; break;
    default: break;
    }
    if (*end == 'i') end++;
    if (*end == 'b') end++;
    if (*end != '\0') {
        if (ok != nullptr) *ok = false;
        return 0;
    }
    return (long long)(v * (double)mul);
}

static bool parse_bool(const std::string &in, bool *out)
{
    std::string s = lower(in);
    if (s == "y" || s == "yes" || s == "1" || s == "on" || s == "true") {
        *out = true;
        return true;
    }
    if (s == "n" || s == "no" || s == "0" || s == "off" || s == "false") {
        *out = false;
        return true;
    }
    return false;
}

OptTable::OptTable(std::string scope, std::vector<OptField> fields)
    : scope_(std::move(scope)), fields_(std::move(fields))
{
    for (const auto &f : fields_) {
        values_[f.name] = f.dflt;
    }
}

void OptTable::append(const std::vector<OptField> &more)
{
    for (const auto &f : more) {
        fields_.push_back(f);
        values_[f.name] = f.dflt;
    }
}

bool OptTable::valid(const OptField &f, const std::string &v) const
{
    bool ok = true, b;
    switch (f.type) {
    case OptType::STRING: return true;
    case OptType::INT:
        parse_memunits(v, &ok);
        return ok;
    case OptType::UINT:
    case OptType::MEMUNITS:
        return parse_memunits(v, &ok) >= 0 && ok;  // counts and sizes: a negative value is a mistake, not a huge number
    case OptType::BOOL: return parse_bool(v, &b);
    case OptType::TERNARY: return parse_bool(v, &b) || lower(v) == "try";
    case OptType::LOG_LEVEL: return parse_log_level(v, -1) >= 0;
    case OptType::DOUBLE: {
        char *end = nullptr;
        std::strtod(v.c_str(), &end);
        return end != v.c_str() && *end == '\0';
    }
    }
    return false;
}

bool OptTable::set(const std::string &name, const std::string &value)
{
    for (const auto &f : fields_) {
        if (name == f.name) {
            if (!valid(f, value)) {
                xccl_warn("option %s%s: value '%s' rejected", scope_.c_str(), f.name, value.c_str());
                return false;
            }
            values_[name] = value;
            return true;
        }
    }
    return false;
}

void OptTable::read(const char *env_prefix, const char *filename)
{
    if (filename != nullptr) {
        std::ifstream in(filename);
        std::string   line;
        while (in && std::getline(in, line)) {
            size_t eq = line.find('=');
            if (line.empty() || line[0] == '#' || eq == std::string::npos) continue;
            std::string key = line.substr(0, eq), val = line.substr(eq + 1);
            std::string want = "XCCL_" + scope_;
            if (key.compare(0, want.size(), want) == 0) {
                set(key.substr(want.size()), val);
            }
        }
    }
    for (const auto &f : fields_) {
        std::string base = "XCCL_" + scope_ + f.name;
        const char *v    = nullptr;
        if (env_prefix != nullptr && env_prefix[0] != '\0') {
            v = std::getenv((std::string(env_prefix) + "_" + base).c_str());
        }
        if (v == nullptr) {
            v = std::getenv(base.c_str());
        }
        if (v != nullptr) {
            set(f.name, v);
        }
    }
}

bool OptTable::has(const std::string &name) const { return values_.count(name) != 0; }

std::string OptTable::str(const std::string &name) const
{
    auto it = values_.find(name);
    return it == values_.end() ? std::string() : it->second;
}

long long OptTable::num(const std::string &name) const
{
    bool ok = true;
    return parse_memunits(str(name), &ok);
}

bool OptTable::flag(const std::string &name) const
{
    bool        b = false;
    std::string v = str(name);
    if (parse_bool(v, &b)) return b;
    return lower(v) == "try";
}

double OptTable::real(const std::string &name) const { return std::strtod(str(name).c_str(), nullptr); }

void OptTable::print(FILE *out, const char *title, unsigned flags) const
{
    if ((flags & XCCL_CONFIG_PRINT_HEADER) && title != nullptr) {
        std::fprintf(out, "#\n# %s\n#\n", title);
    }
    for (const auto &f : fields_) {
        if (flags & XCCL_CONFIG_PRINT_DOC) {
            std::fprintf(out, "# %s (default: %s)\n", f.doc, f.dflt);
        }
        std::fprintf(out, "XCCL_%s%s=%s\n", scope_.c_str(), f.name, str(f.name).c_str());
    }
}

}  // namespace xccl
