// netsim: C++20 coroutine plumbing for simulated host programs.
//
// The reference's test programs (tests/app/rdma/*.c) and its MPI channel are blocking C code that
// runs on simulated RISC-V cores.  Here a host program is a coroutine: every library call that
// would block (a command written to the NIC, a completion poll, a barrier) is an awaitable that
// suspends the program until a simulator event resumes it, so programs keep the shape of the
// originals while the simulator stays single-threaded and deterministic.
#pragma once
#include <coroutine>
#include <exception>
#include <functional>
#include <memory>
#include <optional>
#include <string>
#include <utility>
#include <vector>

namespace netsim {

struct Unit {};

// One-shot value: a simulator callback sets it, a coroutine awaits it (in either order).
template <class T>
class Future {
 public:
  Future() : s_(std::make_shared<State>()) {}
  void set(T v) const {
    s_->value = std::move(v);
    if (auto h = std::exchange(s_->waiter, nullptr)) h.resume();
  }
  bool ready() const { return s_->value.has_value(); }
  bool await_ready() const { return s_->value.has_value(); }
  void await_suspend(std::coroutine_handle<> h) const { s_->waiter = h; }
  T await_resume() const { return std::move(*s_->value); }

 private:
  struct State {
    std::optional<T> value;
    std::coroutine_handle<> waiter;
  };
  std::shared_ptr<State> s_;
};

namespace detail {
struct FinalAwaiter {
  bool await_ready() noexcept { return false; }
  template <class P>
  std::coroutine_handle<> await_suspend(std::coroutine_handle<P> h) noexcept {
    auto c = h.promise().continuation;
    return c ? c : std::noop_coroutine();
  }
  void await_resume() noexcept {}
};
struct PromiseBase {
  std::coroutine_handle<> continuation;
  std::exception_ptr error;
  std::suspend_always initial_suspend() noexcept { return {}; }
  FinalAwaiter final_suspend() noexcept { return {}; }
  void unhandled_exception() { error = std::current_exception(); }
};
}  // namespace detail

// Lazy coroutine with a result.  `co_await` starts it and resumes the awaiter when it ends.
template <class T = void>
class Co {
 public:
  struct promise_type : detail::PromiseBase {
    std::optional<T> value;
    Co get_return_object() { return Co{std::coroutine_handle<promise_type>::from_promise(*this)}; }
    void return_value(T v) { value = std::move(v); }
  };
  Co(Co&& o) noexcept : h_(std::exchange(o.h_, nullptr)) {}
  Co& operator=(Co&& o) noexcept {
    if (this != &o) {
      if (h_) h_.destroy();
      h_ = std::exchange(o.h_, nullptr);
    }
    return *this;
  }
  Co(const Co&) = delete;
  ~Co() {
    if (h_) h_.destroy();
  }
  bool await_ready() const noexcept { return false; }
  std::coroutine_handle<> await_suspend(std::coroutine_handle<> awaiter) noexcept {
    h_.promise().continuation = awaiter;
    return h_;
  }
  T await_resume() {
    if (h_.promise().error) std::rethrow_exception(h_.promise().error);
    return std::move(*h_.promise().value);
  }

 private:
  explicit Co(std::coroutine_handle<promise_type> h) : h_(h) {}
  std::coroutine_handle<promise_type> h_;
};

template <>
class Co<void> {
 public:
  struct promise_type : detail::PromiseBase {
    Co get_return_object() { return Co{std::coroutine_handle<promise_type>::from_promise(*this)}; }
    void return_void() {}
  };
  Co(Co&& o) noexcept : h_(std::exchange(o.h_, nullptr)) {}
  Co& operator=(Co&& o) noexcept {
    if (this != &o) {
      if (h_) h_.destroy();
      h_ = std::exchange(o.h_, nullptr);
    }
    return *this;
  }
  Co(const Co&) = delete;
  ~Co() {
    if (h_) h_.destroy();
  }
  bool await_ready() const noexcept { return false; }
  std::coroutine_handle<> await_suspend(std::coroutine_handle<> awaiter) noexcept {
    h_.promise().continuation = awaiter;
    return h_;
  }
  void await_resume() {
    if (h_.promise().error) std::rethrow_exception(h_.promise().error);
  }

 private:
  explicit Co(std::coroutine_handle<promise_type> h) : h_(h) {}
  std::coroutine_handle<promise_type> h_;
};

// The programs of one simulation.  A program that is still suspended when the event queue
// drains is a deadlock (a receive that nothing matches, a barrier not everybody joined);
// the set destroys such frames when it goes away, so nothing leaks.
class ProcSet {
 public:
  ProcSet() = default;
  ProcSet(const ProcSet&) = delete;
  ~ProcSet() {
    for (auto h : roots_) h.destroy();
  }
  void spawn(Co<void> program) {
    Root r = run(std::move(program), this);
    roots_.push_back(r.h);
  }
  int started() const { return (int)roots_.size(); }
  int finished() const { return finished_; }
  const std::vector<std::string>& errors() const { return errors_; }

 private:
  struct Root {
    struct promise_type {
      Root get_return_object() { return Root{std::coroutine_handle<promise_type>::from_promise(*this)}; }
      std::suspend_never initial_suspend() noexcept { return {}; }
      std::suspend_always final_suspend() noexcept { return {}; }
      void return_void() {}
      void unhandled_exception() { std::terminate(); }
    };
    std::coroutine_handle<promise_type> h;
  };
  static Root run(Co<void> program, ProcSet* self) {
    try {
      co_await std::move(program);
    } catch (const std::exception& e) {
      self->errors_.push_back(e.what());
    }
    ++self->finished_;
  }
  std::vector<std::coroutine_handle<Root::promise_type>> roots_;
  std::vector<std::string> errors_;
  int finished_ = 0;
};

}  // namespace netsim
