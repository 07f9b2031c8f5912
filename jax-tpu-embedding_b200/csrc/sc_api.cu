// Library-wide entry points: version, status names, last-error text and the host-side
// buffer sizing arithmetic.
#include <stdarg.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <string.h>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "sc_common.cuh"

namespace sc {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
}

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches() { return g_launches.load(std::memory_order_relaxed); }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// ---- phases ------------------------------------------------------------------------------------
namespace {
struct PhaseRecord {
  const char* name;
  cudaEvent_t begin, end;
};
std::mutex g_phase_mutex;
std::vector<PhaseRecord> g_phases;
std::atomic<int> g_phase_timing{0};
}  // namespace

PhaseScope::PhaseScope(const char* name, cudaStream_t stream) : stream_(stream), slot_(-1) {
  nvtxRangePushA(name);
  if (!g_phase_timing.load(std::memory_order_relaxed)) return;
  PhaseRecord r;
  r.name = name;
  if (cudaEventCreate(&r.begin) != cudaSuccess || cudaEventCreate(&r.end) != cudaSuccess) return;
  cudaEventRecord(r.begin, stream);
  std::lock_guard<std::mutex> lock(g_phase_mutex);
  slot_ = (int)g_phases.size();
  g_phases.push_back(r);
}

PhaseScope::~PhaseScope() {
  if (slot_ >= 0) {
    std::lock_guard<std::mutex> lock(g_phase_mutex);
    if (slot_ < (int)g_phases.size()) cudaEventRecord(g_phases[slot_].end, stream_);
  }
  nvtxRangePop();
}

}  // namespace sc

extern "C" int32_t sc_phase_timing(int32_t enable) {
  std::lock_guard<std::mutex> lock(sc::g_phase_mutex);
  for (auto& r : sc::g_phases) { cudaEventDestroy(r.begin); cudaEventDestroy(r.end); }
  sc::g_phases.clear();
  sc::g_phase_timing.store(enable ? 1 : 0);
  return SC_OK;
}

extern "C" int32_t sc_phase_report(char* buffer, int32_t buffer_bytes) {
  if (!buffer || buffer_bytes <= 0) SC_FAIL(SC_INVALID_ARGUMENT, "no buffer for the phase report");
  std::lock_guard<std::mutex> lock(sc::g_phase_mutex);
  std::map<std::string, std::pair<double, int>> total;
  std::vector<std::string> order;
  for (auto& r : sc::g_phases) {
    float ms = 0.f;
    if (cudaEventSynchronize(r.end) == cudaSuccess && cudaEventElapsedTime(&ms, r.begin, r.end) == cudaSuccess) {
      if (!total.count(r.name)) order.push_back(r.name);
      total[r.name].first += ms;
      total[r.name].second += 1;
    }
    cudaEventDestroy(r.begin);
    cudaEventDestroy(r.end);
  }
  cudaGetLastError();
  sc::g_phases.clear();
  std::string out;
  for (auto& name : order) {
    char item[160];
    snprintf(item, sizeof item, "%s%s=%.6f/%d", out.empty() ? "" : ";", name.c_str(), total[name].first, total[name].second);
    out += item;
  }
  strncpy(buffer, out.c_str(), (size_t)buffer_bytes - 1);
  buffer[buffer_bytes - 1] = '\0';
  return SC_OK;
}

extern "C" int32_t sc_version(void) { return 100; }

namespace sc { long long launches(); }
extern "C" int64_t sc_launch_count(void) { return (int64_t)sc::launches(); }

extern "C" const char* sc_status_name(int32_t status) {
  switch (status) {
    case SC_OK: return "OK";
    case SC_INVALID_ARGUMENT: return "INVALID_ARGUMENT";
    case SC_WORKSPACE_TOO_SMALL: return "WORKSPACE_TOO_SMALL";
    case SC_ID_LIMIT_EXCEEDED: return "ID_LIMIT_EXCEEDED";
    case SC_CUDA_ERROR: return "CUDA_ERROR";
    case SC_UNSUPPORTED: return "UNSUPPORTED";
    default: return "UNKNOWN";
  }
}

extern "C" int32_t sc_last_error(char* buffer, int32_t buffer_bytes) {
  if (!buffer || buffer_bytes <= 0) return (int32_t)strlen(sc::g_error);
  strncpy(buffer, sc::g_error, (size_t)buffer_bytes - 1);
  buffer[buffer_bytes - 1] = '\0';
  return (int32_t)strlen(buffer);
}

// ComputeTheoreticalMaxCooBufferSize (input_preprocessing_util.cc:242-254), minibatching off.
extern "C" int64_t sc_compute_theoretical_max_coo_buffer_size(int32_t max_ids_per_partition, int32_t global_device_count,
                                                              int32_t num_sc_per_device) {
  const int64_t num_scs = (int64_t)global_device_count * num_sc_per_device;
  const int64_t rounded = ((int64_t)max_ids_per_partition + sc::kAlign - 1) / sc::kAlign * sc::kAlign;
  return rounded * num_sc_per_device * num_scs;
}

// ComputeCooBufferSizePerDevice + MayBeUpdateBufferSize (input_preprocessing_util.cc:219-312).
extern "C" int64_t sc_compute_coo_buffer_size_per_device(int32_t max_ids_per_partition, int32_t global_device_count,
                                                         int32_t num_sc_per_device, int64_t suggested) {
  const int64_t theoretical = sc_compute_theoretical_max_coo_buffer_size(max_ids_per_partition, global_device_count, num_sc_per_device);
  int64_t v = theoretical;
  if (suggested >= 0) {
    const int64_t m = (int64_t)sc::kAlign * num_sc_per_device;
    v = (suggested + m - 1) / m * m;
    if (v > theoretical) {
      sc::set_error("Suggested Coo Buffer Size is larger than the theoretical max: %lld vs %lld. Adjust the suggested size or the "
                    "max_ids_per_partition values.", (long long)v, (long long)theoretical);
      return -1;
    }
  }
  if (!(v > 0 && v < 2147483647LL)) {
    sc::set_error("Computed Coo Buffer Size (%lld) is out of the valid range (0, INT_MAX).", (long long)v);
    return -1;
  }
  return v;
}

// GetRowPointersSizePerDevice (input_preprocessing_util.h:503-511), minibatching off.
extern "C" int32_t sc_compute_row_pointers_size_per_device(int32_t global_device_count, int32_t num_sc_per_device) {
  const int32_t num_scs = global_device_count * num_sc_per_device;
  return (num_scs > sc::kAlign ? num_scs : sc::kAlign) * num_sc_per_device;
}

// ---- peer-visible device memory (row-sharded tables, one process per GPU) ---------------------
// The reference needs no such calls: the TPU runtime addresses other chips' shards inside the
// custom call (sc/docs/parameters.rst:20-24).  Here every process allocates its shards and
// exchange buffers with sc_peer_alloc, exports a CUDA IPC handle and imports its peers' handles;
// the lookup / update kernels then read remote rows with ordinary loads over NVLink.

extern "C" int32_t sc_peer_alloc(size_t bytes, void** out) {
  if (!out || bytes == 0) SC_FAIL(SC_INVALID_ARGUMENT, "sc_peer_alloc: bad arguments");
  SC_CUDA_OK(cudaMalloc(out, bytes));
  return SC_OK;
}

extern "C" int32_t sc_peer_free(void* ptr) {
  SC_CUDA_OK(cudaFree(ptr));
  return SC_OK;
}

extern "C" int32_t sc_ipc_export(void* ptr, char* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (!ptr || !handle64) SC_FAIL(SC_INVALID_ARGUMENT, "sc_ipc_export: bad arguments");
  cudaIpcMemHandle_t h;
  SC_CUDA_OK(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle64, &h, sizeof h);
  return SC_OK;
}

extern "C" int32_t sc_ipc_import(const char* handle64, void** out) {
  if (!out || !handle64) SC_FAIL(SC_INVALID_ARGUMENT, "sc_ipc_import: bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof h);
  SC_CUDA_OK(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return SC_OK;
}

extern "C" int32_t sc_ipc_release(void* ptr) {
  SC_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return SC_OK;
}
