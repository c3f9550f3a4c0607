// Context: one TlContext per selected team library plus the task progress queue.
// Reference behaviour: src/core/xccl_context.c:29-238.
#include <cstring>

#include "core.h"

using namespace xccl;

extern "C" {

xccl_status_t xccl_context_config_read(xccl_lib_h lib, const char *env_prefix, const char *filename,
                                       xccl_context_config_t **config)
{
    if (lib == nullptr || config == nullptr) return XCCL_ERR_INVALID_PARAM;
    auto *cfg       = new xccl_context_config;
    cfg->lib        = lib;
    cfg->env_prefix = env_prefix != nullptr ? env_prefix : "";
    for (TeamLib *tl : lib->tls) {
        OptTable t(tl->scope(), tl->context_options());
        t.read(env_prefix, filename);
        cfg->tables.push_back(std::move(t));
    }
    *config = cfg;
    return XCCL_OK;
}

xccl_status_t xccl_context_config_modify(xccl_tl_id_t *tl_id, xccl_context_config_t *config, const char *name,
                                         const char *value)
{
    if (tl_id == nullptr || config == nullptr || name == nullptr || value == nullptr) return XCCL_ERR_INVALID_PARAM;
    for (size_t i = 0; i < config->lib->tls.size(); i++) {
        if (config->lib->tls[i]->id == *tl_id) {
            return config->tables[i].set(name, value) ? XCCL_OK : XCCL_ERR_INVALID_PARAM;
        }
    }
    return XCCL_ERR_NO_ELEM;
}

void xccl_context_config_release(xccl_context_config_t *config) { delete config; }

xccl_status_t xccl_context_create(xccl_lib_h lib, const xccl_context_params_t *params,
                                  const xccl_context_config_t *config, xccl_context_h *context)
{
    if (lib == nullptr || params == nullptr || context == nullptr) return XCCL_ERR_INVALID_PARAM;
    auto *ctx   = new xccl_context;
    ctx->lib    = lib;
    ctx->params = *params;
    if (!(params->field_mask & XCCL_CONTEXT_PARAM_FIELD_THREAD_MODE)) {
        ctx->params.thread_mode = XCCL_THREAD_MODE_SINGLE;
    }
    uint64_t want = (params->field_mask & XCCL_CONTEXT_PARAM_FIELD_TLS) ? params->tls : (uint64_t)XCCL_TL_ALL;
    ctx->pq       = ProgressQueue::create(ctx->params.thread_mode, (int)global_state().opts.num("LF_TASKS_QUEUE_SIZE"));

    for (size_t i = 0; i < lib->tls.size(); i++) {
        TeamLib *tl = lib->tls[i];
        if (!(want & (uint64_t)tl->id)) continue;
        OptTable fallback;
        const OptTable *table = nullptr;
        if (config != nullptr && config->lib == lib) {
            table = &config->tables[i];
        } else {
            fallback = OptTable(tl->scope(), tl->context_options());
            fallback.read(nullptr, nullptr);
            table = &fallback;
        }
        TlContext    *tctx = nullptr;
        xccl_status_t st   = tl->context_create(lib, ctx->params, *table, &tctx);
        if (st != XCCL_OK) {
            // a TL that cannot come up here (no GPU, no library) is skipped, not fatal
            xccl_debug("team library %s: no context (%s)", tl->name, xccl_status_str(st));
            continue;
        }
        tctx->tl   = tl;
        tctx->core = ctx;
        ctx->tl_ctxs.emplace_back(tctx);
    }
    if (ctx->tl_ctxs.empty()) {
        xccl_error("none of the requested team libraries (mask 0x%llx) could create a context",
                   (unsigned long long)want);
        delete ctx;
        return XCCL_ERR_NO_MESSAGE;
    }
    *context = ctx;
    return XCCL_OK;
}

xccl_status_t xccl_context_progress(xccl_context_h context)
{
    if (context == nullptr) return XCCL_ERR_INVALID_PARAM;
    for (auto &t : context->tl_ctxs) {
        if (t->has_progress()) {
            xccl_status_t st = t->progress();
            if (st < 0) return st;
        }
    }
    return context->pq->progress();
}

xccl_status_t xccl_context_destroy(xccl_context_h context)
{
    delete context;
    return XCCL_OK;
}

xccl_status_t xccl_ctx_query(xccl_context_h ctx, xccl_ctx_attr_t *attr)
{
    if (ctx == nullptr || attr == nullptr) return XCCL_ERR_INVALID_PARAM;
    if (attr->field_mask & XCCL_CTX_ATTR_FIELD_SUPPORTED_COLLS) {
        attr->supported_colls = 0;
        for (auto &t : ctx->tl_ctxs) attr->supported_colls |= t->tl->caps.coll_types;
    }
    return XCCL_OK;
}

void xccl_free_ctx_attr(xccl_ctx_attr_t *) {}

}  // extern "C"
