// Task / event / schedule engine and the two progress queues.
//
// A Task has a state, a progress function and, per event, a list of subscribers. When a task
// fires an event, every subscriber's handler for that event runs. A Schedule is a task that
// completes when all the tasks added to it have completed. Same model as the reference
// (src/core/xccl_schedule.h:8-62, src/core/xccl_schedule.c:5-69), expressed with std::function
// and std::vector instead of fixed tables.
//
// ProgressQueue drives enqueued tasks: the single-thread flavour is a plain list; the
// multi-thread flavour is a pair of fixed CAS slot pools with a spin-locked overflow list
// (reference: src/core/xccl_tasks_queue.c:3-43, src/core/xccl_lock_free_tasks_queue.c:3-121).
#pragma once
#include <atomic>
#include <functional>
#include <list>
#include <memory>
#include <mutex>
#include <vector>

#include "xccl/xccl.h"

namespace xccl {

enum TaskEvent { EVENT_COMPLETED = 0, EVENT_SCHEDULE_STARTED, EVENT_LAST };
enum TaskState { TASK_IDLE = 0, TASK_INPROGRESS, TASK_COMPLETED, TASK_FAILED };

class Schedule;

class Task {
public:
    virtual ~Task() = default;

    using Handler = std::function<void(Task *self, Task *source)>;

    // `listener` runs its handler for `ev` whenever this task fires `ev`.
    void subscribe(TaskEvent ev, Task *listener) { listeners_[ev].push_back(listener); }
    void set_handler(TaskEvent ev, Handler h) { handlers_[ev] = std::move(h); }
    void fire(TaskEvent ev);
    // marks completion, notifies the owning schedule and fires EVENT_COMPLETED
    void complete(xccl_status_t st = XCCL_OK);
    virtual void reset();

    // Called by a progress queue until state leaves TASK_INPROGRESS.
    std::function<xccl_status_t(Task *)> progress;

    std::atomic<int> state{TASK_IDLE};
    xccl_status_t    status   = XCCL_OK;
    Schedule        *schedule = nullptr;

private:
    std::vector<Task *> listeners_[EVENT_LAST];
    Handler             handlers_[EVENT_LAST];
};

class Schedule : public Task {
public:
    void add(Task *t);
    // fires EVENT_SCHEDULE_STARTED; tasks subscribed to it start running
    void start();
    void child_done(Task *t);
    void rearm();
    void reset() override { rearm(); }
    int  n_tasks() const { return (int)tasks_.size(); }
    const std::vector<Task *> &tasks() const { return tasks_; }

private:
    std::vector<Task *> tasks_;
    std::atomic<int>    n_completed_{0};
};

class ProgressQueue {
public:
    virtual ~ProgressQueue() = default;
    virtual void          enqueue(Task *t) = 0;
    virtual xccl_status_t progress()       = 0;
    // lf_slots: slots per pool of the multi-thread flavour
    static std::unique_ptr<ProgressQueue> create(unsigned thread_mode, int lf_slots = 8);
};

}  // namespace xccl
