// Shared internals of the host runtime: error reporting, tunables, pools.
#pragma once
#include <stdint.h>
#include <stdarg.h>
#include <string>
#include <functional>
#include <future>
#include "../include/tmpi_c_api.h"

namespace tmpi {

// Records a message for tmpi_last_error() (thread local) and returns `code`.
int fail(int code, const char* fmt, ...);
void set_error(const char* fmt, va_list ap);

// Tunables are read through this accessor everywhere in the runtime.
int64_t tunable(const char* name);

size_t dtype_size(int dtype);

// ---- pools (collective = 0, parameter server = 1)
enum { POOL_COLLECTIVE = 0, POOL_PS = 1 };
// Runs `fn` on a pool thread; the returned handle completes with fn's status.
uint64_t submit(int pool, std::function<int()> fn);
// Runs `fn` on the dedicated in-order worker of `lane` (launch order across
// ranks must match for kernels that wait on one another).
uint64_t submit_ordered(int lane, std::function<int()> fn);
// Attach a CUDA event (owned by the handle) that marks device completion.
void handle_set_event(uint64_t handle, void* cuda_event);
uint64_t make_ready_handle(int status);

void trace(const char* op, const char* algo, uint64_t bytes, double us);
bool trace_on();

}  // namespace tmpi
