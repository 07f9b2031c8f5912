// Shared helpers of the sc_b200 library: status/error plumbing and small device utilities.
#ifndef SC_COMMON_CUH_
#define SC_COMMON_CUH_

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "sc_b200.h"

namespace sc {

// Message of the last failing call on this host thread (returned by sc_last_error).
void set_error(const char* fmt, ...);

#define SC_FAIL(status, ...)      \
  do {                            \
    ::sc::set_error(__VA_ARGS__); \
    return (status);              \
  } while (0)

#define SC_CUDA_OK(expr)                                                                      \
  do {                                                                                        \
    cudaError_t err__ = (expr);                                                               \
    if (err__ != cudaSuccess) SC_FAIL(SC_CUDA_ERROR, "%s: %s", #expr, cudaGetErrorString(err__)); \
  } while (0)

#define SC_LAUNCH_OK(name)                                                                        \
  do {                                                                                            \
    ::sc::count_launch();                                                                         \
    cudaError_t err__ = cudaGetLastError();                                                       \
    if (err__ != cudaSuccess) SC_FAIL(SC_CUDA_ERROR, "launch %s: %s", name, cudaGetErrorString(err__)); \
  } while (0)

constexpr int kAlign = 8;  // alignment (in slots) of every partition inside a COO buffer

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int bit_width_u32(uint32_t v) {
  int b = 0;
  while (v) { ++b; v >>= 1; }
  return b;
}

// Carves typed, 256-byte aligned regions out of a caller-owned device workspace.
class Workspace {
 public:
  Workspace(void* base, size_t bytes) : base_(static_cast<char*>(base)), bytes_(bytes) {}
  template <typename T>
  T* take(size_t count) {
    size_t off = align_up(used_, 256);
    used_ = off + count * sizeof(T);
    return reinterpret_cast<T*>(base_ + off);  // valid only if ok()
  }
  size_t used() const { return align_up(used_, 256); }
  bool ok() const { return base_ != nullptr && used() <= bytes_; }

 private:
  char* base_;
  size_t bytes_;
  size_t used_ = 0;
};

// Counts kernel launches issued by this library (read with sc_launch_count).
void count_launch(int n = 1);

// Number of SMs of the current device (cached per device).
int sm_count();

// A named stage of a call: an NVTX range on the host thread (free when no tool listens) and, while
// sc_phase_timing(1) is in effect, a pair of CUDA events on `stream` whose distance sc_phase_report
// adds up per name.  Names follow the reference's trace annotations where it has them
// (tsl::profiler::TraceMe in lib/core/input_preprocessing.cc:210-214, 413-417, 632-636;
// @jax.named_call in lib/nn/embedding.py:1047, 1297).
class PhaseScope {
 public:
  PhaseScope(const char* name, cudaStream_t stream);
  ~PhaseScope();
  PhaseScope(const PhaseScope&) = delete;
  PhaseScope& operator=(const PhaseScope&) = delete;

 private:
  cudaStream_t stream_;
  int slot_;
};

}  // namespace sc
#endif  // SC_COMMON_CUH_
