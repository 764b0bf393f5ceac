// Host worker pools.
//
// ThreadPool: N workers over one mutex + condition-variable queue, the same
// shape as the pool the reference actually uses (lib/thread_pool-in.h:47-129).
// A pool of one worker drains its queue in order; the runtime uses such pools ("lanes") where the
// launch order of kernels that wait on peer GPUs must be identical on every rank.
#pragma once
#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace tmpi {

class ThreadPool {
 public:
  explicit ThreadPool(int n) {
    if (n < 1) n = 1;
    for (int i = 0; i < n; ++i) workers_.emplace_back([this] { loop(); });
  }
  ~ThreadPool() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& w : workers_) w.join();
  }
  void enqueue(std::function<void()> fn) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      q_.push_back(std::move(fn));
    }
    cv_.notify_one();
  }
  int size() const { return (int)workers_.size(); }
  // Blocks until the queue is empty and every worker is idle.
  void drain() {
    std::unique_lock<std::mutex> lk(mu_);
    idle_cv_.wait(lk, [this] { return q_.empty() && busy_ == 0; });
  }

 private:
  void loop() {
    for (;;) {
      std::function<void()> fn;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [this] { return stop_ || !q_.empty(); });
        if (stop_ && q_.empty()) return;
        fn = std::move(q_.front());
        q_.pop_front();
        ++busy_;
      }
      fn();
      {
        std::lock_guard<std::mutex> lk(mu_);
        --busy_;
      }
      idle_cv_.notify_all();
    }
  }
  std::mutex mu_;
  std::condition_variable cv_, idle_cv_;
  std::deque<std::function<void()>> q_;
  std::vector<std::thread> workers_;
  int busy_ = 0;
  bool stop_ = false;
};

}  // namespace tmpi
