// A collective request made of collectives on other teams (and small local actions), wired as
// fragments of steps over the task engine. Composite team libraries (pod split, multirail)
// describe WHAT runs WHERE; this class owns the persistent sub-requests, posts them in
// dependency order and drives them from the context's progress queue.
//
//   fragment   an ordered list of steps; step i starts when step i-1 completed (or all at once)
//   window     at most `depth` fragments are in flight; fragment f starts when f-depth completed
// Sub-requests are initialised at build time in fragment order, so every member of a sub-team
// creates its requests in the same order.
#pragma once
#include <functional>
#include <memory>
#include <vector>

#include "core.h"

namespace xccl {

struct CompositeStep {
    xccl_team_h                    team = nullptr;  // collective on this team, or
    xccl_coll_op_args_t            args{};
    std::function<xccl_status_t()> local;           // a local action that completes immediately
};

class CompositeReq : public xccl_coll_req {
public:
    explicit CompositeReq(xccl_context *progress_ctx) : ctx_(progress_ctx) {}
    ~CompositeReq() override;

    xccl_status_t add_fragment(const std::vector<CompositeStep> &steps, bool parallel = false);
    void          set_depth(int depth) { depth_ = depth < 1 ? 1 : depth; }
    // keeps arrays referenced by step arguments alive for the life of the request
    uint32_t     *keep(std::vector<uint32_t> v);

    xccl_status_t post() override;
    xccl_status_t test() override;
    xccl_status_t finalize() override { return sched_.state.load() == TASK_INPROGRESS ? XCCL_INPROGRESS : XCCL_OK; }
    // hook run once per post after everything completed (e.g. releasing a serialisation slot)
    std::function<void()> on_complete;

private:
    struct StepTask final : public Task {
        CompositeStep   step;
        xccl_coll_req_h req = nullptr;
        ~StepTask() override
        {
            if (req != nullptr) xccl_collective_finalize(req);
        }
    };
    void wire();
    xccl_context                           *ctx_;
    Schedule                                sched_;
    std::vector<std::unique_ptr<StepTask>>  tasks_;
    std::vector<std::unique_ptr<Schedule>>  frags_;
    std::vector<std::unique_ptr<std::vector<uint32_t>>> kept_;
    int  depth_ = 1 << 30;
    bool wired_ = false, notified_ = true;
};

}  // namespace xccl
