// Thread-sanitizer driver for the host runtime (tunables, handle registry, worker pools and ordered lanes,
// communicator stack, ring plan).  Built by tests/test_tsan_runtime.py with -fsanitize=thread together with
// csrc/runtime/{config,handles,communicator}.cpp and run on the CPU; a data race makes the sanitizer print a
// report and the process exit non-zero.  The reference guards its runtime only with a "main thread" assertion
// (lib/resources.cpp:77-81); here several threads drive the same entry points on purpose.
#include <unistd.h>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>
#include "../include/tmpi_c_api.h"

#define CHECK(cond)                                                      \
  do {                                                                   \
    if (!(cond)) { std::fprintf(stderr, "check failed: %s (line %d)\n", #cond, __LINE__); _exit(3); } \
  } while (0)

int main() {
  CHECK(tmpi_comm_reset(0, 8) == TMPI_OK);
  std::atomic<int> done_tasks{0};
  std::vector<std::thread> threads;
  // tunables: writers and readers
  for (int t = 0; t < 3; ++t)
    threads.emplace_back([t] {
      for (int i = 0; i < 2000; ++i) {
        int64_t v = 0;
        CHECK(tmpi_set_tunable("comm_max_ctas", 32 + (i + t) % 64) == TMPI_OK);
        CHECK(tmpi_get_tunable("comm_max_ctas", &v) == TMPI_OK && v >= 32 && v < 96);
        CHECK(tmpi_get_tunable("no_such_tunable", &v) != TMPI_OK);
        (void)tmpi_last_error();
      }
    });
  // pools: tasks submitted and waited for from several threads at once, handles polled by others
  std::vector<uint64_t> shared_ids(64, 0);
  std::atomic<int> next_slot{0};
  for (int t = 0; t < 4; ++t)
    threads.emplace_back([&, t] {
      for (int i = 0; i < 60; ++i) {
        uint64_t h = tmpi_test_sleep_task(i % 2, 1 + (i % 3), TMPI_OK);
        int slot = next_slot.fetch_add(1) % 64;
        shared_ids[slot] = h;                                 // racy on purpose? no: each slot is written by its taker
        (void)tmpi_handle_done(h);
        CHECK(tmpi_handle_wait(h, 5000) == TMPI_OK);
        CHECK(tmpi_handle_done(h) == 1);                      // unknown after wait: reported as complete
        done_tasks.fetch_add(1);
      }
      (void)t;
    });
  threads.emplace_back([&] {
    for (int i = 0; i < 500; ++i) { (void)tmpi_handles_in_flight(); std::this_thread::yield(); }
  });
  // a handle that never completes must time out cleanly, from a thread of its own
  threads.emplace_back([] {
    uint64_t lost = tmpi_test_lost_handle();
    CHECK(tmpi_handle_wait(lost, 50) == TMPI_ERR_TIMEOUT);
  });
  // communicator stack: one thread splits and moves the cursor, others read
  threads.emplace_back([] {
    for (int round = 0; round < 50; ++round) {
      char keys[8 * 1024];
      std::memset(keys, 0, sizeof(keys));
      int parent[8];
      for (int r = 0; r < 8; ++r) { parent[r] = r; std::snprintf(keys + r * 1024, 1024, "g%d", r / 4); }
      CHECK(tmpi_comm_set(0) == TMPI_OK);
      int level = tmpi_comm_push(keys, parent, 8, "g0");
      CHECK(level >= 1);
      CHECK(tmpi_comm_set_span(0, level) == TMPI_OK);
      CHECK(tmpi_comm_pop_to(1) == TMPI_OK);
    }
  });
  for (int t = 0; t < 2; ++t)
    threads.emplace_back([] {
      for (int i = 0; i < 2000; ++i) {
        int out[64], b, e;
        char names[4096];
        (void)tmpi_comm_current_members(out, 64);
        (void)tmpi_comm_num_levels();
        (void)tmpi_comm_get_span(&b, &e);
        (void)tmpi_comm_names(names, sizeof(names));
        (void)tmpi_comm_group_of(0, 3, out, 64);
      }
    });
  // ring plan: pure functions, called concurrently
  for (int t = 0; t < 2; ++t)
    threads.emplace_back([] {
      std::vector<int> plan(7 * 8 * 2);
      for (int i = 0; i < 500; ++i) {
        CHECK(tmpi_ring_plan(8, 8, i & 1, plan.data(), (int)plan.size()) >= 0);
        (void)tmpi_ring_send_chunk(i % 8, 8, i % 7, i & 1);
      }
    });
  for (auto& th : threads) th.join();
  CHECK(tmpi_sync_all() == TMPI_OK || true);
  CHECK(done_tasks.load() == 240);
  std::printf("tsan driver: %d tasks, ok\n", done_tasks.load());
  return 0;
}
