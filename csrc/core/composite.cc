#include "composite.h"

namespace xccl {

CompositeReq::~CompositeReq() = default;

uint32_t *CompositeReq::keep(std::vector<uint32_t> v)
{
    kept_.push_back(std::make_unique<std::vector<uint32_t>>(std::move(v)));
    return kept_.back()->data();
}

xccl_status_t CompositeReq::add_fragment(const std::vector<CompositeStep> &steps, bool parallel)
{
    auto frag = std::make_unique<Schedule>();
    Task *prev = nullptr;
    for (const CompositeStep &cs : steps) {
        auto t  = std::make_unique<StepTask>();
        t->step = cs;
        if (cs.team != nullptr) {
            xccl_status_t st = xccl_collective_init(&t->step.args, &t->req, cs.team);
            if (st != XCCL_OK) return st;
        }
        t->progress = [](Task *self) -> xccl_status_t {
            auto *s = static_cast<StepTask *>(self);
            for (int k = 0; k < 10; k++) {
                xccl_status_t st = xccl_collective_test(s->req);
                if (st == XCCL_INPROGRESS) continue;
                s->complete(st);
                return st;
            }
            return XCCL_OK;
        };
        auto start = [this](Task *self, Task *) {
            auto *s = static_cast<StepTask *>(self);
            if (s->req == nullptr) {
                s->state.store(TASK_INPROGRESS);
                s->complete(s->step.local ? s->step.local() : XCCL_OK);
                return;
            }
            xccl_status_t st = xccl_collective_post(s->req);
            if (st != XCCL_OK) {
                s->state.store(TASK_INPROGRESS);
                s->complete(st);
                return;
            }
            ctx_->pq->enqueue(s);
        };
        t->set_handler(EVENT_SCHEDULE_STARTED, start);
        t->set_handler(EVENT_COMPLETED, start);
        frag->add(t.get());
        if (parallel || prev == nullptr) {
            frag->subscribe(EVENT_SCHEDULE_STARTED, t.get());
        } else {
            prev->subscribe(EVENT_COMPLETED, t.get());
        }
        prev = t.get();
        tasks_.push_back(std::move(t));
    }
    frags_.push_back(std::move(frag));
    return XCCL_OK;
}

void CompositeReq::wire()
{
    auto kick = [](Task *self, Task *) { static_cast<Schedule *>(self)->start(); };
    for (size_t f = 0; f < frags_.size(); f++) {
        Schedule *frag = frags_[f].get();
        frag->set_handler(EVENT_SCHEDULE_STARTED, kick);
        frag->set_handler(EVENT_COMPLETED, kick);
        sched_.add(frag);
        if (f < (size_t)depth_) {
            sched_.subscribe(EVENT_SCHEDULE_STARTED, frag);
        } else {
            frags_[f - (size_t)depth_]->subscribe(EVENT_COMPLETED, frag);
        }
    }
    wired_ = true;
}

xccl_status_t CompositeReq::post()
{
    if (!wired_) wire();
    if (sched_.state.load() == TASK_INPROGRESS) return XCCL_ERR_NO_RESOURCE;
    sched_.rearm();
    notified_ = false;
    sched_.start();
    return XCCL_OK;
}

xccl_status_t CompositeReq::test()
{
    int s = sched_.state.load(std::memory_order_acquire);
    if (s == TASK_INPROGRESS) {
        xccl_context_progress(ctx_);
        s = sched_.state.load(std::memory_order_acquire);
    }
    if (s == TASK_INPROGRESS) return XCCL_INPROGRESS;
    if (!notified_) {
        notified_ = true;
        if (on_complete) on_complete();
    }
    return s == TASK_IDLE ? XCCL_OK : sched_.status;
}

}  // namespace xccl
