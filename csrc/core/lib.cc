// Library object, global options, TL registry and queries.
// Reference behaviour: src/core/xccl_lib.c:27-122, src/core/xccl_init.c:59-164,
// src/core/xccl_query.c:12-80, src/core/xccl_global_opts.c:10-37.
#include <algorithm>
#include <chrono>
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <glob.h>
#include <mutex>
#include <unistd.h>

#include "../utils/mem.h"
#include "../utils/topo.h"
#include "core.h"

namespace xccl {

static const std::vector<OptField> kGlobalFields = {
    {"LOG_LEVEL", "warn", "Verbosity: fatal, error, warn, info, debug, trace", OptType::LOG_LEVEL},
    {"TEAM_LIB_PATH", "", "Directory searched for extra team-library plugins (xccl_team_lib_*.so)", OptType::STRING},
    {"MEM_COMPONENT_CACHE_SIZE", "4096", "Bytes of scratch kept cached per memory type", OptType::MEMUNITS},
    {"LF_TASKS_QUEUE_SIZE", "8", "Slots per pool of the multi-thread progress queue; tasks beyond twice this go to a locked overflow list", OptType::UINT},
    {"OOB_TIMEOUT", "120", "Seconds a blocking out-of-band exchange may take before it fails", OptType::DOUBLE},
    {"WAIT_TIMEOUT", "600", "Seconds xccl_collective_wait may spin before it returns XCCL_ERR_TIMED_OUT", OptType::DOUBLE},
    {"NVTX", "n", "Wrap xccl_collective_post and xccl_collective_wait in NVTX ranges named after the collective", OptType::BOOL},
};

GlobalState &global_state()
{
    static GlobalState g = [] {
        GlobalState s;
        s.opts = OptTable("", kGlobalFields);
        s.opts.read(nullptr, nullptr);
        global_log().level = parse_log_level(s.opts.str("LOG_LEVEL"), LOG_WARN);
        char host[256]     = {0};
        gethostname(host, sizeof(host) - 1);
        s.host_name = host;
        s.host_hash = str_hash_djb2(host);
        s.pid       = (int)getpid();
        s.socket_id = bound_socket_id();
        return s;
    }();
    return g;
}

// ------------------------------------------------------------------ TL base + registry

static const char *tl_name_or_unknown(xccl_tl_id_t id)
{
    const char *n = xccl_tl_str(id);
    return n != nullptr ? n : "unknown";
}

TeamLib::TeamLib(xccl_tl_id_t id_, int default_priority)
    : id(id_), name(tl_name_or_unknown(id_)), priority(default_priority), log{name, LOG_WARN}
{
}

std::string TeamLib::upper_name() const
{
    std::string u(name);
    std::transform(u.begin(), u.end(), u.begin(), [](unsigned char c) { return std::toupper(c); });
    return u;
}

xccl_status_t TeamLib::query(xccl_tl_attr_t *attr)
{
    if (attr->field_mask & XCCL_TL_ATTR_FIELD_CONTEXT_CREATE_MODE) {
        attr->context_create_mode = caps.ctx_mode;
    }
    if (attr->field_mask & XCCL_TL_ATTR_FIELD_DEVICES_COUNT) {
        attr->devices_count = 0;
    }
    if (attr->field_mask & XCCL_TL_ATTR_FIELD_DEVICES) {
        attr->devices = nullptr;
    }
    return XCCL_OK;
}

std::vector<TeamLib *> &team_lib_registry()
{
    static std::vector<TeamLib *> reg;
    return reg;
}

void register_team_lib(TeamLib *tl)
{
    for (TeamLib *t : team_lib_registry()) {
        if (t->id == tl->id) return;
    }
    team_lib_registry().push_back(tl);
}

TeamLib *find_team_lib(xccl_tl_id_t id)
{
    for (TeamLib *t : team_lib_registry()) {
        if (t->id == id) return t;
    }
    return nullptr;
}

namespace {
struct Plugin {
    void    *handle;
    TeamLib *tl;
};
std::vector<Plugin> &plugins()
{
    static std::vector<Plugin> p;
    return p;
}

// End of the process (reference: the library destructor, src/core/xccl_finalize.c:18-42): every team library
// that was opened is closed, newest first, the scratch cache of the memory component is dropped and plugin
// objects are unloaded. Registered with atexit when the team libraries are opened, so it runs before the
// destructors of the statically registered team-library objects, which were constructed earlier.
void close_all_team_libs()
{
    auto &reg = team_lib_registry();
    for (auto it = reg.rbegin(); it != reg.rend(); ++it) {
        if ((*it)->opened) {
            (*it)->close();
            (*it)->opened = false;
        }
    }
    mem_cache_release();
    for (auto it = plugins().rbegin(); it != plugins().rend(); ++it) {
        reg.erase(std::remove(reg.begin(), reg.end(), it->tl), reg.end());
        dlclose(it->handle);
    }
    plugins().clear();
}
}  // namespace

static void load_plugins(const std::string &dir)
{
    glob_t      g{};
    std::string pattern = dir + "/xccl_team_lib_*.so";
    if (glob(pattern.c_str(), 0, nullptr, &g) != 0) {
        globfree(&g);
        return;
    }
    for (size_t i = 0; i < g.gl_pathc; i++) {
        void *h = dlopen(g.gl_pathv[i], RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) {
            xccl_warn("cannot load plugin %s: %s", g.gl_pathv[i], dlerror());
            continue;
        }
        using CreateFn = TeamLib *(*)();
        auto fn        = (CreateFn)dlsym(h, "xccl_team_lib_create");
        if (fn == nullptr) {
            xccl_warn("plugin %s has no xccl_team_lib_create", g.gl_pathv[i]);
            dlclose(h);
            continue;
        }
        TeamLib *tl = fn();
        if (tl == nullptr || find_team_lib(tl->id) != nullptr) {
            xccl_warn("plugin %s offers no team library, or one whose id is already registered", g.gl_pathv[i]);
            dlclose(h);
            continue;
        }
        register_team_lib(tl);
        plugins().push_back(Plugin{h, tl});
    }
    globfree(&g);
}

void open_all_team_libs()
{
    static std::once_flag once;
    std::call_once(once, [] {
        GlobalState &g    = global_state();
        std::string  path = g.opts.str("TEAM_LIB_PATH");
        if (!path.empty()) {
            load_plugins(path);
        }
        for (TeamLib *tl : team_lib_registry()) {
            std::vector<OptField> fields = {
                {"LOG_LEVEL", "warn", "Verbosity of this team library", OptType::LOG_LEVEL},
                {"PRIORITY", "-1", "Selection priority; -1 keeps the built-in value", OptType::INT},
            };
            for (const auto &f : tl->lib_options()) fields.push_back(f);
            tl->lib_cfg = OptTable(tl->scope(), fields);
            tl->lib_cfg.read(nullptr, nullptr);
            tl->log.level = parse_log_level(tl->lib_cfg.str("LOG_LEVEL"), LOG_WARN);
            if (tl->log.level < global_log().level) tl->log.level = global_log().level;
            long long prio = tl->lib_cfg.num("PRIORITY");
            if (prio >= 0) tl->priority = (int)prio;
            xccl_status_t st = tl->open();
            tl->opened       = (st == XCCL_OK);
            if (!tl->opened) {
                xccl_debug("team library %s not available (%s)", tl->name, xccl_status_str(st));
            }
        }
        std::atexit(close_all_team_libs);
    });
}

xccl_status_t oob_allgather_blocking(const xccl_oob_collectives_t &oob, void *sbuf, void *rbuf, size_t size)
{
    void           *req = nullptr;
    xccl_ep_range_t r{};
    r.type = XCCL_EP_RANGE_UNDEFINED;
    if (oob.allgather(sbuf, rbuf, size, oob.rank, r, oob.coll_context, &req) != 0) {
        return XCCL_ERR_NO_MESSAGE;
    }
    double        limit = global_state().opts.real("OOB_TIMEOUT");
    auto          t0    = std::chrono::steady_clock::now();
    xccl_status_t st;
    while ((st = oob.req_test(req)) == XCCL_INPROGRESS) {
        double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (limit > 0 && dt > limit) {
            oob.req_free(req);
            xccl_error("out-of-band allgather of %zu bytes timed out after %.0f s", size, dt);
            return XCCL_ERR_TIMED_OUT;
        }
    }
    oob.req_free(req);
    return st;
}

}  // namespace xccl

using namespace xccl;

// ------------------------------------------------------------------ C entry points

extern "C" {

const char *xccl_status_str(xccl_status_t st)
{
    switch (st) {
    case XCCL_OK: return "ok";
    case XCCL_INPROGRESS: return "in progress";
    case XCCL_ERR_NO_MESSAGE: return "no message";
    case XCCL_ERR_NO_RESOURCE: return "no resource";
    case XCCL_ERR_NO_MEMORY: return "out of memory";
    case XCCL_ERR_INVALID_PARAM: return "invalid parameter";
    case XCCL_ERR_UNREACHABLE: return "unreachable";
    case XCCL_ERR_NOT_IMPLEMENTED: return "not implemented";
    case XCCL_ERR_MESSAGE_TRUNCATED: return "message truncated";
    case XCCL_ERR_NO_PROGRESS: return "no progress";
    case XCCL_ERR_BUFFER_TOO_SMALL: return "buffer too small";
    case XCCL_ERR_NO_ELEM: return "no such element";
    case XCCL_ERR_UNSUPPORTED: return "unsupported";
    case XCCL_ERR_TIMED_OUT: return "timed out";
    default: return "unknown status";
    }
}

xccl_status_t xccl_lib_config_read(const char *env_prefix, const char *filename, xccl_lib_config_t **config_p)
{
    if (config_p == nullptr) return XCCL_ERR_INVALID_PARAM;
    auto *cfg       = new xccl_lib_config;
    cfg->global     = OptTable("", kGlobalFields);
    cfg->env_prefix = env_prefix != nullptr ? env_prefix : "";
    cfg->global.read(env_prefix, filename);
    *config_p = cfg;
    return XCCL_OK;
}

void xccl_lib_config_release(xccl_lib_config_t *config) { delete config; }

void xccl_lib_config_print(const xccl_lib_config_t *config, FILE *stream, const char *title,
                           xccl_config_print_flags_t flags)
{
    if (config == nullptr || stream == nullptr) return;
    config->global.print(stream, title, flags);
    open_all_team_libs();
    for (TeamLib *tl : team_lib_registry()) {
        tl->lib_cfg.print(stream, tl->name, flags & ~XCCL_CONFIG_PRINT_HEADER);
    }
}

xccl_status_t xccl_lib_init(const xccl_lib_params_t *params, const xccl_lib_config_t *config, xccl_lib_h *lib_p)
{
    if (params == nullptr || lib_p == nullptr) return XCCL_ERR_INVALID_PARAM;
    GlobalState &g = global_state();
    if (config != nullptr) {
        int lvl = parse_log_level(config->global.str("LOG_LEVEL"), -1);
        if (lvl >= 0) global_log().level = lvl;
    }
    (void)g;
    open_all_team_libs();
    auto *lib   = new xccl_lib;
    lib->params = *params;
    for (TeamLib *tl : team_lib_registry()) {
        if (!tl->opened) continue;
        const TlCaps &c = tl->caps;
        if ((params->field_mask & XCCL_LIB_PARAM_FIELD_REPRODUCIBLE) && !(params->reproducible & c.reproducible)) continue;
        if ((params->field_mask & XCCL_LIB_PARAM_FIELD_THREAD_MODE) && !(params->thread_mode & c.thread_mode)) continue;
        if ((params->field_mask & XCCL_LIB_PARAM_FIELD_TEAM_USAGE) && !(params->team_usage & c.team_usage)) continue;
        if ((params->field_mask & XCCL_LIB_PARAM_FIELD_COLL_TYPES) && !(params->coll_types & c.coll_types)) continue;
        lib->tls.push_back(tl);
    }
    if (lib->tls.empty()) {
        xccl_error("no team library matches the requested library parameters");
        delete lib;
        return XCCL_ERR_NO_MESSAGE;
    }
    *lib_p = lib;
    return XCCL_OK;
}

void xccl_lib_cleanup(xccl_lib_h lib) { delete lib; }

xccl_status_t xccl_get_tl_list(xccl_lib_h lib, xccl_tl_id_t **tls, unsigned *tl_count)
{
    if (lib == nullptr || tls == nullptr || tl_count == nullptr) return XCCL_ERR_INVALID_PARAM;
    *tl_count = (unsigned)lib->tls.size();
    *tls      = (xccl_tl_id_t *)std::malloc(sizeof(xccl_tl_id_t) * (lib->tls.size() + 1));
    if (*tls == nullptr) return XCCL_ERR_NO_MEMORY;
    for (size_t i = 0; i < lib->tls.size(); i++) (*tls)[i] = lib->tls[i]->id;
    return XCCL_OK;
}

void xccl_free_tl_list(xccl_tl_id_t *tls) { std::free(tls); }

xccl_status_t xccl_tl_query(xccl_lib_h lib, xccl_tl_id_t *tl, xccl_tl_attr_t *attr)
{
    if (lib == nullptr || tl == nullptr || attr == nullptr) return XCCL_ERR_INVALID_PARAM;
    for (TeamLib *t : lib->tls) {
        if (t->id == *tl) return t->query(attr);
    }
    return XCCL_ERR_NO_ELEM;
}

void xccl_free_tl_attr(xccl_tl_attr_t *attr)
{
    if (attr != nullptr && (attr->field_mask & XCCL_TL_ATTR_FIELD_DEVICES) && attr->devices != nullptr) {
        std::free(attr->devices);
        attr->devices = nullptr;
    }
}

}  // extern "C"
