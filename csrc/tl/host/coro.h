// A minimal resumable-function type. Host collectives are written as straight-line C++20
// coroutines that suspend whenever their outstanding messages are not complete; the request's
// test() resumes them. (The reference hand-codes each algorithm as a switch-based state
// machine, e.g. src/team_lib/ucx/allreduce/allreduce_knomial.c:24-164.)
#pragma once
#include <coroutine>
#include <exception>
#include <utility>

#include "xccl/xccl.h"

namespace xccl {
namespace host {

class Coro {
public:
    struct promise_type {
        xccl_status_t result = XCCL_OK;
        Coro          get_return_object() { return Coro(std::coroutine_handle<promise_type>::from_promise(*this)); }
        std::suspend_always initial_suspend() noexcept { return {}; }
        std::suspend_always final_suspend() noexcept { return {}; }
        void                return_value(xccl_status_t st) { result = st; }
        void                unhandled_exception() { result = XCCL_ERR_NO_MESSAGE; }
    };

    Coro() = default;
    explicit Coro(std::coroutine_handle<promise_type> h) : h_(h) {}
    Coro(Coro &&o) noexcept : h_(std::exchange(o.h_, nullptr)) {}
    Coro &operator=(Coro &&o) noexcept
    {
        if (this != &o) {
            reset();
            h_ = std::exchange(o.h_, nullptr);
        }
        return *this;
    }
    Coro(const Coro &)            = delete;
    Coro &operator=(const Coro &) = delete;
    ~Coro() { reset(); }

    void reset()
    {
        if (h_) h_.destroy();
        h_ = nullptr;
    }
    bool valid() const { return (bool)h_; }
    bool done() const { return !h_ || h_.done(); }
    // Runs until the next suspension point; true when the function has returned.
    bool step()
    {
        if (h_ && !h_.done()) h_.resume();
        return done();
    }
    xccl_status_t result() const { return h_ ? h_.promise().result : XCCL_OK; }

private:
    std::coroutine_handle<promise_type> h_;
};

}  // namespace host
}  // namespace xccl

// Suspend until `cond` holds.
#define XCCL_CO_WAIT(cond)                    \
    while (!(cond)) {                         \
        co_await std::suspend_always{};       \
    }

// Run a nested coroutine to completion; propagates a failure status.
#define XCCL_CO_CALL(expr)                                        \
    do {                                                          \
        ::xccl::host::Coro _sub = (expr);                         \
        while (!_sub.step()) {                                    \
            co_await std::suspend_always{};                       \
        }                                                         \
        if (_sub.result() != XCCL_OK) co_return _sub.result();    \
    } while (0)
