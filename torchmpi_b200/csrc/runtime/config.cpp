// Tunables, error slot, dtype sizes and the trace ring buffer.
//
// The table keeps the reference's knobs under their own names with the
// defaults of lib/constants.cpp:130-155 (so scripts that set them keep
// working) and adds the knobs of the NVSwitch data plane.  Unlike the
// reference, set/get of the collective in-flight limit touch the collective
// variable, not the parameter-server one (lib/constants.cpp:283-288 mixes
// them up), and the freeze flag is honoured.
#include "common.h"
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

namespace tmpi {

namespace {
struct Tunable { const char* name; std::atomic<int64_t> value; };

Tunable g_tunables[] = {
  // ---- reference knobs
  {"use_staged_collectives", {0}},
  {"use_hierarchical_collectives", {1}},
  {"use_cartesian_communicator", {0}},
  {"small_cpu_broadcast_size", {1 << 13}},
  {"small_cpu_allreduce_size", {1 << 16}},
  {"small_gpu_broadcast_size", {1 << 13}},
  {"small_gpu_allreduce_size", {1 << 16}},
  {"min_buffer_size_per_cpu_collective", {1 << 17}},
  {"min_buffer_size_per_gpu_collective", {1 << 17}},
  {"max_buffer_size_per_cpu_collective", {1 << 20}},
  {"max_buffer_size_per_gpu_collective", {1 << 20}},
  {"broadcast_size_cpu_tree_based", {1 << 22}},
  {"broadcast_size_gpu_tree_based", {1 << 22}},
  {"num_buffers_per_cpu_collective", {3}},
  {"num_buffers_per_gpu_collective", {3}},
  {"collective_num_threads", {4}},
  {"parameterserver_num_threads", {4}},
  {"collective_thread_pool_size", {1 << 20}},
  {"parameterserver_thread_pool_size", {1 << 20}},
  // ---- B200 data plane
  {"oneshot_max_bytes", {512 << 10}},      // <= : one-shot push allreduce
  {"nvls_min_bytes", {1 << 20}},           // >= : multimem allreduce when multicast is bound
  {"comm_max_ctas", {64}},                 // CTAs of a stand-alone collective kernel
  {"broadcast_algo", {0}},                 // heap broadcasts: 0 by size, 1 pull from the root, 2 scatter + all-gather, 3 multicast store
  {"bcast_max_ctas", {128}},               // CTAs of the multicast-store broadcast (only the root moves data)
  {"bcast_scatter_max_ctas", {64}},        // CTAs per rank of the single-pass scatter + all-gather broadcasts
  {"bcast_scatter_min_bytes", {8 << 20}},  // from this size the broadcast is the single-pass scatter + push
  {"nvls_max_ctas", {32}},                 // CTAs of the multimem kernels: 32 measured best at 8 GPUs (832 GB/s bus at 1 GiB;
                                           // 64 MiB: 637 vs 588 with 64 CTAs); the switch reduction saturates, more CTAs only contend
  {"ps_max_ctas", {148}},                  // CTAs of a parameter-server push / pull kernel (one per SM: +30 % push bandwidth over 64)
  {"opt_max_ctas", {32}},                  // CTAs of the fused allreduce+SGD kernel (runs beside backward)
  {"comm_threads", {512}},
  {"num_comm_lanes", {2}},                 // ordered launch lanes (stream + flag set each)
  {"device_wait_budget_ms", {2000}},       // bounded spin of device flag waits in steady state
  {"device_wait_startup_budget_ms", {20000}},  // the same budget during the start-up grace period (ranks enter
                                           // their first steps seconds apart: module loading, autotuning)
  {"device_wait_startup_grace_ms", {30000}},   // length of that period, counted from the creation of the heap
  {"host_wait_budget_ms", {10000}},        // the reference's 10 s deadlock heuristic
  {"handle_wait_budget_ms", {60000}},      // default budget of tmpi_handle_wait (a handle may cover a long task)
  {"bucket_bytes", {32 << 20}},            // gradient bucket size of the engine
  {"heap_bytes", {int64_t(1) << 30}},      // symmetric heap per rank
  {"staging_bytes", {64 << 20}},           // bounce buffer inside the heap for foreign tensors
  {"use_nvls", {1}},
  {"bn_pool_fused_bwd", {0}},              // stem batch-norm + pool backward as one stage (slower than pool, then batch-norm)
  {"bn_reverse_stats", {1}},               // batch-norm statistics passes walk the tensor from its end (L2 reuse)
  {"grad_fork", {1}},                      // residual blocks sum the two gradients of their input inside a kernel
  {"conv_own_3x3", {0}},                   // 3x3 convolutions on the implicit-GEMM kernel (1x1 always are)
  {"gemm_pair", {1}},                      // 256 x 256 tiles on CTA pairs (cta_group::2) where the shape allows
  {"ps_poll_us", {100}},
  {"watchdog_interval_ms", {1000}},        // heartbeat period of the host watchdog (0: no watchdog)
  {"watchdog_budget_ms", {10000}},         // a peer whose heartbeat stands still this long is declared lost
  {"fault_drop_ps_requests", {0}},         // fault injection (host side): parameter-server requests are dropped
  {"trace", {0}},
};
constexpr int kNumTunables = sizeof(g_tunables) / sizeof(g_tunables[0]);
std::atomic<bool> g_frozen{false};

// one slot per process: errors raised on pool threads are read by the caller's thread
char t_error[1024] = "";
std::mutex g_err_mu;

struct TraceRec { char op[24]; char algo[16]; uint64_t bytes; double us; };
std::mutex g_trace_mu;
std::vector<TraceRec> g_trace;
size_t g_trace_next = 0;
constexpr size_t kTraceCap = 4096;
}  // namespace

void set_error(const char* fmt, va_list ap) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap; va_start(ap, fmt); set_error(fmt, ap); va_end(ap);
  return code;
}

int64_t tunable(const char* name) {
  for (auto& t : g_tunables) if (!strcmp(t.name, name)) return t.value.load(std::memory_order_relaxed);
  return 0;
}

size_t dtype_size(int dtype) {
  switch (dtype) {
    case TMPI_U8: case TMPI_I8: return 1;
    case TMPI_I16: case TMPI_F16: case TMPI_BF16: return 2;
    case TMPI_I32: case TMPI_F32: return 4;
    case TMPI_I64: case TMPI_F64: return 8;
  }
  return 0;
}

bool trace_on() { return tunable("trace") != 0; }

void trace(const char* op, const char* algo, uint64_t bytes, double us) {
  if (!trace_on()) return;
  TraceRec r{};
  snprintf(r.op, sizeof(r.op), "%s", op);
  snprintf(r.algo, sizeof(r.algo), "%s", algo);
  r.bytes = bytes; r.us = us;
  std::lock_guard<std::mutex> lk(g_trace_mu);
  if (g_trace.size() < kTraceCap) g_trace.push_back(r);
  else g_trace[g_trace_next % kTraceCap] = r;
  g_trace_next++;
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

const char* tmpi_last_error(void) { return t_error; }
int tmpi_version(void) { return 100; }
size_t tmpi_dtype_size(int dtype) { return dtype_size(dtype); }

int tmpi_set_tunable(const char* name, int64_t value) {
  if (g_frozen.load()) return fail(TMPI_ERR_STATE, "tunables are frozen");
  for (auto& t : g_tunables)
    if (!strcmp(t.name, name)) { t.value.store(value); return TMPI_OK; }
  return fail(TMPI_ERR_INVALID, "unknown tunable '%s'", name);
}

int tmpi_get_tunable(const char* name, int64_t* value) {
  for (auto& t : g_tunables)
    if (!strcmp(t.name, name)) { *value = t.value.load(); return TMPI_OK; }
  return fail(TMPI_ERR_INVALID, "unknown tunable '%s'", name);
}

int tmpi_num_tunables(void) { return kNumTunables; }
const char* tmpi_tunable_name(int i) { return (i >= 0 && i < kNumTunables) ? g_tunables[i].name : nullptr; }
int tmpi_freeze_tunables(void) { g_frozen.store(true); return TMPI_OK; }

int tmpi_trace_enable(int on) {
  for (auto& t : g_tunables) if (!strcmp(t.name, "trace")) t.value.store(on);
  return TMPI_OK;
}
int tmpi_trace_record(const char* op, const char* algo, uint64_t bytes, double us) {
  trace(op, algo, bytes, us); return TMPI_OK;
}
int tmpi_trace_clear(void) {
  std::lock_guard<std::mutex> lk(g_trace_mu); g_trace.clear(); g_trace_next = 0; return TMPI_OK;
}
int tmpi_trace_dump(char* out, int cap) {
  std::lock_guard<std::mutex> lk(g_trace_mu);
  int used = 0;
  for (auto& r : g_trace) {
    char line[160];
    int n = snprintf(line, sizeof(line), "{\"op\":\"%s\",\"algo\":\"%s\",\"bytes\":%llu,\"us\":%.3f}\n",
                     r.op, r.algo, (unsigned long long)r.bytes, r.us);
    if (used + n + 1 > cap) break;
    memcpy(out + used, line, n); used += n;
  }
  if (cap > 0) out[used < cap ? used : cap - 1] = 0;
  return used;
}

}  // extern "C"
