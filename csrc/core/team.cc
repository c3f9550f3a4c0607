// Team creation and the (collective, memory type) -> team library table.
// Reference behaviour: src/core/xccl_team.c:14-131. TL teams are created one after another
// because only one out-of-band allgather may be in flight per context; once all exist they are
// ordered by descending priority and the first capable TL wins each (collective, memory) slot.
#include <algorithm>
#include <chrono>
#include <cstring>

#include "core.h"

namespace xccl {

OobGroup make_oob_group(const xccl_team_params_t &p, const xccl_oob_collectives_t &ctx_oob)
{
    OobGroup g;
    if (p.field_mask & XCCL_TEAM_PARAM_FIELD_OOB) {
        g.oob        = p.oob;
        g.range.type = XCCL_EP_RANGE_UNDEFINED;
        g.rank       = p.oob.rank;
        g.size       = p.oob.size;
        return g;
    }
    g.oob = ctx_oob;
    if ((p.field_mask & XCCL_TEAM_PARAM_FIELD_EP_RANGE) && p.range.type != XCCL_EP_RANGE_UNDEFINED) {
        g.range = p.range;
        g.size  = p.range.ep_num;
        g.rank  = -1;
        for (int i = 0; i < g.size; i++) {
            if (xccl_range_to_rank(p.range, i) == ctx_oob.rank) {
                g.rank = i;
                break;
            }
        }
    } else {
        g.range.type = XCCL_EP_RANGE_UNDEFINED;
        g.rank       = ctx_oob.rank;
        g.size       = ctx_oob.size;
    }
    return g;
}

xccl_status_t OobGroup::allgather_blocking(void *sbuf, void *rbuf, size_t bytes) const
{
    void *req = nullptr;
    if (allgather(sbuf, rbuf, bytes, &req) != 0) {
        return XCCL_ERR_NO_MESSAGE;
    }
    double        limit = global_state().opts.real("OOB_TIMEOUT");
    auto          t0    = std::chrono::steady_clock::now();
    xccl_status_t st;
    while ((st = test(req)) == XCCL_INPROGRESS) {
        double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (limit > 0 && dt > limit) {
            free(req);
            return XCCL_ERR_TIMED_OUT;
        }
    }
    free(req);
    return st;
}

static xccl_status_t post_next(xccl_team *team)
{
    while (team->n_posted < team->ctx->tl_ctxs.size()) {
        TlContext    *tctx = team->ctx->tl_ctxs[team->n_posted].get();
        TlTeam       *tt   = nullptr;
        xccl_status_t st   = tctx->team_create_post(team->params, &tt);
        team->n_posted++;
        if (st < 0 || tt == nullptr) {
            // this TL cannot serve the team (e.g. nvlink without peer access): skip it
            xccl_debug("team library %s declined the team (%s)", tctx->tl->name, xccl_status_str(st));
            continue;
        }
        tt->ctx = tctx;
        team->tl_teams.emplace_back(tt);
        return XCCL_INPROGRESS;  // test it before posting the next one
    }
    return XCCL_OK;
}

static void build_selection(xccl_team *team)
{
    std::stable_sort(team->tl_teams.begin(), team->tl_teams.end(),
                     [](const std::unique_ptr<TlTeam> &a, const std::unique_ptr<TlTeam> &b) {
                         return a->ctx->tl->priority > b->ctx->tl->priority;
                     });
    for (int c = 0; c < XCCL_COLL_LAST; c++) {
        for (int m = 0; m < XCCL_MEMORY_TYPE_LAST; m++) {
            team->coll_team_id[c][m] = -1;
            for (size_t i = 0; i < team->tl_teams.size(); i++) {
                const TlCaps &caps = team->tl_teams[i]->ctx->tl->caps;
                const bool    sync = (c == XCCL_BARRIER || c == XCCL_FANIN || c == XCCL_FANOUT);
                const uint64_t mems = (sync && caps.sync_mem_types != ~0ull) ? caps.sync_mem_types : caps.mem_types;
                if ((caps.coll_types & XCCL_BIT(c)) && (mems & XCCL_BIT(m))) {
                    team->coll_team_id[c][m] = (int)i;
                    break;
                }
            }
        }
    }
}

}  // namespace xccl

using namespace xccl;

extern "C" {

xccl_status_t xccl_team_create_post(xccl_context_h context, xccl_team_params_t *params, xccl_team_h *team_p)
{
    if (context == nullptr || params == nullptr || team_p == nullptr) return XCCL_ERR_INVALID_PARAM;
    auto *team   = new xccl_team;
    team->ctx    = context;
    team->params = *params;
    if ((params->field_mask & XCCL_TEAM_PARAM_FIELD_EP_RANGE) && params->range.type == XCCL_EP_RANGE_MAP &&
        params->range.map.map != nullptr) {
        team->range_map.assign(params->range.map.map, params->range.map.map + params->range.ep_num);
        team->params.range.map.map = team->range_map.data();
    }
    if (!(params->field_mask & XCCL_TEAM_PARAM_FIELD_OOB) &&
        !(context->params.field_mask & XCCL_CONTEXT_PARAM_FIELD_OOB)) {
        xccl_error("team creation needs an out-of-band allgather on the team or on the context");
        delete team;
        return XCCL_ERR_INVALID_PARAM;
    }
    std::memset(team->coll_team_id, 0xff, sizeof(team->coll_team_id));
    post_next(team);
    *team_p = team;
    return XCCL_OK;
}

xccl_status_t xccl_team_create_test(xccl_team_h team)
{
    if (team == nullptr) return XCCL_ERR_INVALID_PARAM;
    if (team->created) return XCCL_OK;
    if (team->failed != XCCL_OK) return team->failed;
    // Creation is non-blocking, but not open-ended: a member that never joins must not leave the others
    // polling forever. The deadline is the same as for a blocking out-of-band exchange (XCCL_OOB_TIMEOUT).
    auto now_s = [] { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); };
    if (team->t_posted == 0.0) team->t_posted = now_s();
    const double limit = global_state().opts.real("OOB_TIMEOUT");
    if (limit > 0 && now_s() - team->t_posted > limit) {
        team->failed = XCCL_ERR_TIMED_OUT;
        xccl_error("team creation did not finish within %.1f s (a member never joined?)", limit);
        return team->failed;
    }
    if (!team->tl_teams.empty()) {
        TlTeam       *last = team->tl_teams.back().get();
        xccl_status_t st   = last->create_test();
        if (st == XCCL_INPROGRESS) return st;
        if (st < 0) {
            xccl_debug("team library %s failed to create its team (%s)", last->ctx->tl->name, xccl_status_str(st));
            team->tl_teams.pop_back();
        }
    }
    if (post_next(team) == XCCL_INPROGRESS) return XCCL_INPROGRESS;
    if (team->tl_teams.empty()) {
        team->failed = XCCL_ERR_NO_RESOURCE;
        xccl_error("no team library could create this team");
        return team->failed;
    }
    build_selection(team);
    team->created = true;
    return XCCL_OK;
}

void xccl_team_destroy(xccl_team_h team) { delete team; }

xccl_status_t xccl_team_query(xccl_team_h team, int *rank, int *size)
{
    if (team == nullptr) return XCCL_ERR_INVALID_PARAM;
    OobGroup g = make_oob_group(team->params, team->ctx->params.oob);
    if (rank != nullptr) *rank = g.rank;
    if (size != nullptr) *size = g.size;
    return XCCL_OK;
}

xccl_status_t xccl_team_mem_alloc(xccl_team_h team, size_t bytes, void **ptr)
{
    if (team == nullptr || ptr == nullptr || bytes == 0 || !team->created) return XCCL_ERR_INVALID_PARAM;
    for (auto &tt : team->tl_teams) {
        xccl_status_t st = tt->sym_alloc(bytes, ptr);
        if (st != XCCL_ERR_NOT_IMPLEMENTED) return st;
    }
    return XCCL_ERR_NOT_IMPLEMENTED;
}

xccl_status_t xccl_team_mem_free(xccl_team_h team, void *ptr)
{
    if (team == nullptr || ptr == nullptr) return XCCL_ERR_INVALID_PARAM;
    for (auto &tt : team->tl_teams) {
        xccl_status_t st = tt->sym_free(ptr);
        if (st != XCCL_ERR_NOT_IMPLEMENTED && st != XCCL_ERR_NO_ELEM) return st;
    }
    return XCCL_ERR_NO_ELEM;
}

xccl_tl_id_t xccl_team_coll_tl(xccl_team_h team, xccl_collective_type_t coll, xccl_memory_type_t mem)
{
    if (team == nullptr || !team->created || coll >= XCCL_COLL_LAST || mem >= XCCL_MEMORY_TYPE_LAST) return XCCL_TL_NULL;
    int id = team->coll_team_id[coll][mem];
    return id < 0 ? XCCL_TL_NULL : team->tl_teams[(size_t)id]->ctx->tl->id;
}

}  // extern "C"
