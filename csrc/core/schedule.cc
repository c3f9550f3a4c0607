#include "schedule.h"

#include <algorithm>
#include <array>
#include <chrono>
#include <deque>
#include <thread>
#include <vector>

#include "log.h"

namespace xccl {

void Task::fire(TaskEvent ev)
{
    // copy: a handler may subscribe further tasks while we iterate
    std::vector<Task *> targets = listeners_[ev];
    for (Task *t : targets) {
        if (t->handlers_[ev]) {
            t->handlers_[ev](t, this);
        }
    }
}

void Task::complete(xccl_status_t st)
{
    status = st;
    state.store(st == XCCL_OK ? TASK_COMPLETED : TASK_FAILED, std::memory_order_release);
    if (schedule != nullptr) {
        schedule->child_done(this);
    }
    fire(EVENT_COMPLETED);
}

void Task::reset()
{
    status = XCCL_OK;
    state.store(TASK_IDLE, std::memory_order_release);
}

void Schedule::add(Task *t)
{
    t->schedule = this;
    tasks_.push_back(t);
}

void Schedule::rearm()
{
    n_completed_.store(0);
    Task::reset();
    for (Task *t : tasks_) {
        t->reset();  // nested schedules re-arm their own tasks
    }
}

void Schedule::start()
{
    state.store(TASK_INPROGRESS, std::memory_order_release);
    if (tasks_.empty()) {
        complete(XCCL_OK);
        return;
    }
    fire(EVENT_SCHEDULE_STARTED);
}

void Schedule::child_done(Task *t)
{
    if (t->status != XCCL_OK && status == XCCL_OK) {
        status = t->status;  // first failure wins; the schedule still drains
    }
    int done = n_completed_.fetch_add(1) + 1;
    if (done == (int)tasks_.size()) {
        Task::complete(status);
    }
}

// ------------------------------------------------------------------ single-thread queue

namespace {

class ListQueue final : public ProgressQueue {
public:
    void enqueue(Task *t) override
    {
        t->state.store(TASK_INPROGRESS, std::memory_order_release);
        tasks_.push_back(t);
    }

    xccl_status_t progress() override
    {
        xccl_status_t result = XCCL_OK;
        // index loop: a completing task may enqueue its successor
        for (size_t i = 0; i < tasks_.size();) {
            Task         *t  = tasks_[i];
            xccl_status_t st = XCCL_OK;
            if (t->state.load(std::memory_order_acquire) == TASK_INPROGRESS && t->progress) {
                st = t->progress(t);
            }
            int s = t->state.load(std::memory_order_acquire);
            if (st < 0 && s == TASK_INPROGRESS) {
                t->complete(st);
                s = TASK_FAILED;
            }
            if (s != TASK_INPROGRESS) {
                if (s == TASK_FAILED) result = t->status;
                tasks_.erase(tasks_.begin() + (long)i);
            } else {
                i++;
            }
        }
        return result;
    }

private:
    std::deque<Task *> tasks_;
};

// ------------------------------------------------------------------ multi-thread queue
// Two pools of `slots` atomic slots (XCCL_LF_TASKS_QUEUE_SIZE, 8 by default: the reference reads the
// same option but keeps its line at 8). Producers CAS a task into the pool that is currently
// "open"; when both the open pool is full the task goes to an overflow list under a spin
// lock. A consumer pops ONE task per call, progresses it outside any lock and re-inserts it
// when it has not finished, so any number of threads may call progress() concurrently.

class LockFreeQueue final : public ProgressQueue {
public:
    explicit LockFreeQueue(int slots)
    {
        for (auto &pool : pools_) {
            pool = std::vector<std::atomic<Task *>>((size_t)std::max(1, slots));
            for (auto &s : pool) s.store(nullptr);
        }
    }

    void enqueue(Task *t) override
    {
        t->state.store(TASK_INPROGRESS, std::memory_order_release);
        insert(t);
    }

    xccl_status_t progress() override
    {
        Task *t = pop();
        if (t == nullptr) {
            return XCCL_OK;
        }
        xccl_status_t st = XCCL_OK;
        if (t->state.load(std::memory_order_acquire) == TASK_INPROGRESS && t->progress) {
            st = t->progress(t);
        }
        int s = t->state.load(std::memory_order_acquire);
        if (st < 0 && s == TASK_INPROGRESS) {
            t->complete(st);
            s = TASK_FAILED;
        }
        if (s == TASK_INPROGRESS) {
            insert(t);
            return XCCL_OK;
        }
        return s == TASK_FAILED ? t->status : XCCL_OK;
    }

private:
    void insert(Task *t)
    {
        int open = open_pool_.load(std::memory_order_acquire);
        for (int k = 0; k < 2; k++) {
            auto &pool = pools_[(open + k) & 1];
            for (auto &slot : pool) {
                Task *expected = nullptr;
                if (slot.load(std::memory_order_relaxed) == nullptr &&
                    slot.compare_exchange_strong(expected, t, std::memory_order_acq_rel)) {
                    return;
                }
            }
        }
        while (lock_.test_and_set(std::memory_order_acquire)) {
        }
        overflow_.push_back(t);
        lock_.clear(std::memory_order_release);
    }

    Task *pop()
    {
        int open = open_pool_.load(std::memory_order_acquire);
        // drain the pool that is NOT receiving new work first, then flip
        for (int k = 1; k <= 2; k++) {
            auto &pool = pools_[(open + k) & 1];
            for (auto &slot : pool) {
                Task *t = slot.load(std::memory_order_relaxed);
                if (t != nullptr && slot.compare_exchange_strong(t, nullptr, std::memory_order_acq_rel)) {
                    return t;
                }
            }
            if (k == 1) {
                open_pool_.compare_exchange_strong(open, open ^ 1, std::memory_order_acq_rel);
            }
        }
        Task *t = nullptr;
        while (lock_.test_and_set(std::memory_order_acquire)) {
        }
        if (!overflow_.empty()) {
            t = overflow_.front();
            overflow_.pop_front();
        }
        lock_.clear(std::memory_order_release);
        return t;
    }

    std::array<std::vector<std::atomic<Task *>>, 2> pools_;
    std::atomic<int>                                open_pool_{0};
    std::atomic_flag                                lock_ = ATOMIC_FLAG_INIT;
    std::deque<Task *>                              overflow_;
};

}  // namespace

std::unique_ptr<ProgressQueue> ProgressQueue::create(unsigned thread_mode, int lf_slots)
{
    if (thread_mode == XCCL_THREAD_MODE_MULTIPLE) {
        return std::make_unique<LockFreeQueue>(lf_slots);
    }
    return std::make_unique<ListQueue>();
}

}  // namespace xccl

// Self-test of a progress queue (tests): `producers` threads enqueue `tasks_per_thread` tasks each, every task needs
// `polls` progress calls to complete, and all threads call progress() until everything has completed or `timeout_s`
// has passed. Returns the number of completed tasks (every task exactly once: a task that is progressed after its
// completion, or twice at the same time, counts as -1000000).
extern "C" long xccl_progress_queue_selftest(unsigned thread_mode, int lf_slots, int producers, int tasks_per_thread,
                                             int polls, double timeout_s)
{
    using namespace xccl;
    struct Counted final : Task {
        std::atomic<int> left{0};
        std::atomic<int> busy{0};
    };
    auto                  queue = ProgressQueue::create(thread_mode, lf_slots);
    const int             total = producers * tasks_per_thread;
    std::vector<Counted>  tasks((size_t)total);
    std::atomic<long>     completed{0}, errors{0};
    for (auto &t : tasks) {
        t.left.store(polls);
        t.progress = [&completed, &errors](Task *self) -> xccl_status_t {
            auto *c = static_cast<Counted *>(self);
            if (c->busy.fetch_add(1) != 0) errors.fetch_add(1);  // two threads in one task at once
            const int left = c->left.fetch_sub(1) - 1;
            if (left < 0) errors.fetch_add(1);                   // progressed after completion
            c->busy.fetch_sub(1);
            if (left == 0) {
                c->complete(XCCL_OK);
                completed.fetch_add(1);
            }
            return XCCL_OK;
        };
    }
    const auto t0 = std::chrono::steady_clock::now();
    auto expired  = [&] { return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s; };
    std::vector<std::thread> threads;
    const int                n_threads = thread_mode == XCCL_THREAD_MODE_MULTIPLE ? producers : 1;
    for (int p = 0; p < n_threads; p++) {
        threads.emplace_back([&, p] {
            const int mine = thread_mode == XCCL_THREAD_MODE_MULTIPLE ? tasks_per_thread : total;
            for (int i = 0; i < mine; i++) {
                queue->enqueue(&tasks[(size_t)(p * tasks_per_thread + i)]);
                queue->progress();
            }
            while (completed.load() < total && !expired()) queue->progress();
        });
    }
    for (auto &t : threads) t.join();
    return errors.load() != 0 ? -1000000 : completed.load();
}
