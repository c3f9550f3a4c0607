// Typed option tables filled from the environment, a NAME=VALUE file and programmatic
// overrides. Naming scheme follows the reference (src/core/xccl_global_opts.c:10-37,
// src/core/xccl_context.c:134-220): global options are XCCL_<NAME>, team-library options are
// XCCL_TEAM_<TL>_<NAME>, and a caller prefix P is tried first as P_XCCL_... .
#pragma once
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

#include "xccl/xccl.h"

namespace xccl {

enum class OptType { STRING, INT, UINT, BOOL, MEMUNITS, TERNARY, LOG_LEVEL, DOUBLE };

struct OptField {
    const char *name;
    const char *dflt;
    const char *doc;
    OptType     type;
};

// A named set of fields plus the values read for them.
class OptTable {
public:
    OptTable() = default;
    OptTable(std::string scope, std::vector<OptField> fields);

    // scope is "" for the global table or "TEAM_<TL>_" for a team library
    void        read(const char *env_prefix, const char *filename);
    bool        set(const std::string &name, const std::string &value);  // false: unknown name or bad value
    bool        has(const std::string &name) const;
    std::string str(const std::string &name) const;
    long long   num(const std::string &name) const;  // INT/UINT/MEMUNITS ("inf" -> LLONG_MAX)
    bool        flag(const std::string &name) const; // BOOL; TERNARY "try" counts as true
    double      real(const std::string &name) const;
    void        print(FILE *out, const char *title, unsigned flags) const;
    void        append(const std::vector<OptField> &more);
    const std::string &scope() const { return scope_; }

private:
    bool valid(const OptField &f, const std::string &v) const;
    std::string                        scope_;
    std::vector<OptField>              fields_;
    std::map<std::string, std::string> values_;
};

long long parse_memunits(const std::string &s, bool *ok);

}  // namespace xccl
