// Asynchronous-operation handles and the two worker pools.
//
// A handle names one operation in flight.  It completes when its host task
// has returned and, if the task launched GPU work, when the CUDA event the
// task recorded has fired.  Handles are ids into a registry rather than heap
// pointers handed to the scripting layer (the reference returns raw
// SynchronizationHandle* and index-addresses futures in vectors that are
// flushed at 1<<20 entries, lib/resources.cpp:405-481,1173-1242); an unknown
// id is treated as already complete, which keeps the reference's "stale index
// means done" behaviour without the flush.
#include "common.h"
#include "thread_pool.h"
#include <cuda_runtime.h>
#include <atomic>
#include <chrono>
#include <map>
#include <memory>
#include <mutex>

namespace tmpi {
namespace {

struct Handle {
  std::shared_future<int> fut;
  std::atomic<void*> event{nullptr};
  bool lost = false;                      // fault injection: a request whose completion never arrives
};

std::mutex g_mu;
std::map<uint64_t, std::shared_ptr<Handle>> g_handles;
std::atomic<uint64_t> g_next{1};

std::unique_ptr<ThreadPool> g_pools[2];
std::vector<std::unique_ptr<ThreadPool>> g_lanes;
std::mutex g_pool_mu;
thread_local uint64_t t_current_handle = 0;

ThreadPool& pool(int which) {
  std::lock_guard<std::mutex> lk(g_pool_mu);
  if (!g_pools[which]) {
    int n = (int)tunable(which == POOL_COLLECTIVE ? "collective_num_threads" : "parameterserver_num_threads");
    g_pools[which].reset(new ThreadPool(n));
  }
  return *g_pools[which];
}

ThreadPool& lane_pool(int lane) {
  std::lock_guard<std::mutex> lk(g_pool_mu);
  if (lane < 0) lane = 0;
  while ((int)g_lanes.size() <= lane) g_lanes.emplace_back(new ThreadPool(1));
  return *g_lanes[lane];
}

std::shared_ptr<Handle> find(uint64_t id) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_handles.find(id);
  return it == g_handles.end() ? nullptr : it->second;
}

void erase(uint64_t id) {
  std::shared_ptr<Handle> h;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_handles.find(id);
    if (it == g_handles.end()) return;
    h = it->second;
    g_handles.erase(it);
  }
  void* ev = h->event.exchange(nullptr);
  if (ev) cudaEventDestroy((cudaEvent_t)ev);
}

uint64_t submit_to(ThreadPool& p, std::function<int()> fn) {
  uint64_t id = g_next.fetch_add(1);
  auto h = std::make_shared<Handle>();
  auto prom = std::make_shared<std::promise<int>>();
  h->fut = prom->get_future().share();
  {
    std::lock_guard<std::mutex> lk(g_mu);
    g_handles[id] = h;
  }
  p.enqueue([id, prom, fn] {
    t_current_handle = id;
    int st;
    try { st = fn(); } catch (...) { st = TMPI_ERR_STATE; }
    t_current_handle = 0;
    prom->set_value(st);
  });
  return id;
}

}  // namespace

uint64_t submit(int which, std::function<int()> fn) { return submit_to(pool(which), std::move(fn)); }
uint64_t submit_ordered(int lane, std::function<int()> fn) { return submit_to(lane_pool(lane), std::move(fn)); }

void handle_set_event(uint64_t id, void* ev) {
  if (id == 0) id = t_current_handle;
  auto h = find(id);
  if (h) h->event.store(ev);
  else if (ev) cudaEventDestroy((cudaEvent_t)ev);
}

uint64_t make_ready_handle(int status) {
  uint64_t id = g_next.fetch_add(1);
  auto h = std::make_shared<Handle>();
  std::promise<int> p; p.set_value(status);
  h->fut = p.get_future().share();
  std::lock_guard<std::mutex> lk(g_mu);
  g_handles[id] = h;
  return id;
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

int tmpi_handle_wait(uint64_t id, int64_t timeout_ms) {
  auto h = find(id);
  if (!h) return TMPI_OK;  // unknown or already waited: complete
  int64_t budget = timeout_ms >= 0 ? timeout_ms : tunable("handle_wait_budget_ms");
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(budget);
  if (h->fut.wait_until(deadline) != std::future_status::ready)
    return fail(TMPI_ERR_TIMEOUT, "handle %llu: host task still running after %lld ms (looks like a deadlock)",
                (unsigned long long)id, (long long)budget);
  int st = h->fut.get();
  void* ev = h->event.load();
  if (ev && st == TMPI_OK) {
    // poll so that the wait stays bounded even if a peer never arrives
    for (;;) {
      cudaError_t e = cudaEventQuery((cudaEvent_t)ev);
      if (e == cudaSuccess) break;
      if (e != cudaErrorNotReady) { st = fail(TMPI_ERR_CUDA, "event query: %s", cudaGetErrorString(e)); break; }
      if (std::chrono::steady_clock::now() > deadline) {
        return fail(TMPI_ERR_TIMEOUT, "handle %llu: device work still running after %lld ms",
                    (unsigned long long)id, (long long)budget);
      }
      std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
  }
  erase(id);
  return st;
}

int tmpi_handle_done(uint64_t id) {
  auto h = find(id);
  if (!h) return 1;
  if (h->fut.wait_for(std::chrono::seconds(0)) != std::future_status::ready) return 0;
  void* ev = h->event.load();
  if (ev && cudaEventQuery((cudaEvent_t)ev) == cudaErrorNotReady) return 0;
  return 1;
}

int tmpi_handle_stream_wait(uint64_t id, void* stream) {
  auto h = find(id);
  if (!h) return TMPI_OK;
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(tunable("host_wait_budget_ms"));
  if (h->fut.wait_until(deadline) != std::future_status::ready)
    return fail(TMPI_ERR_TIMEOUT, "handle %llu: launch task did not finish", (unsigned long long)id);
  int st = h->fut.get();
  void* ev = h->event.load();
  if (ev && st == TMPI_OK) {
    cudaError_t e = cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)ev, 0);
    if (e != cudaSuccess) st = fail(TMPI_ERR_CUDA, "stream wait: %s", cudaGetErrorString(e));
  }
  return st;
}

int tmpi_sync_all(void) {
  std::vector<uint64_t> ids;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    for (auto& kv : g_handles) ids.push_back(kv.first);
  }
  int st = TMPI_OK;
  for (auto id : ids) {
    auto h = find(id);
    if (h && h->lost) { erase(id); continue; }      // nothing will ever complete it
    int s = tmpi_handle_wait(id, -1);
    if (s != TMPI_OK) st = s;
  }
  return st;
}

// Fault injection on the host: a handle that stands for a request that was dropped on the way - its task never
// reports back.  Waiting on it must end in TMPI_ERR_TIMEOUT within the caller's budget.
uint64_t tmpi_test_lost_handle(void) {
  static std::vector<std::shared_ptr<std::promise<int>>> never;   // kept alive: a destroyed promise would complete the future
  static std::mutex mu;
  uint64_t id = g_next.fetch_add(1);
  auto h = std::make_shared<Handle>();
  auto prom = std::make_shared<std::promise<int>>();
  h->fut = prom->get_future().share();
  h->lost = true;
  {
    std::lock_guard<std::mutex> lk(mu);
    never.push_back(prom);
  }
  std::lock_guard<std::mutex> lk(g_mu);
  g_handles[id] = h;
  return id;
}

int tmpi_handles_in_flight(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  return (int)g_handles.size();
}

uint64_t tmpi_test_sleep_task(int which, int ms, int status) {
  return submit(which, [ms, status] {
    std::this_thread::sleep_for(std::chrono::milliseconds(ms));
    return status;
  });
}

}  // extern "C"
