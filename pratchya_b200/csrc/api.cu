// Error reporting, device queries and small utilities behind the C ABI.
#include "common.cuh"

#include <mutex>

namespace pb {

char* error_buffer() {
  static thread_local char buf[512] = "";
  return buf;
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return status;
}

int sm_count() {
  static std::mutex mu;
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

void* tensor_map_encoder() {
  static void* const fn = [] {      // thread-safe static initialisation
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      return p;
    return static_cast<void*>(nullptr);
  }();
  return fn;
}

}  // namespace pb

extern "C" int pb_version(void) { return 100; }

extern "C" const char* pb_last_error(void) { return pb::error_buffer(); }

extern "C" const char* pb_status_string(int status) {
  switch (status) {
    case PB_OK: return "ok";
    case PB_ERR_NULL_POINTER: return "null pointer";
    case PB_ERR_BAD_SHAPE: return "bad shape";
    case PB_ERR_BAD_GRID: return "bad grid";
    case PB_ERR_BAD_DTYPE: return "bad dtype";
    case PB_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case PB_ERR_CUDA: return "CUDA error";
    case PB_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    case PB_ERR_UNSUPPORTED: return "unsupported";
    case PB_ERR_MISALIGNED: return "misaligned pointer";
    default: return "unknown status";
  }
}

extern "C" int pb_group_geometry(int64_t rows, int64_t cols, int a, int b, int64_t* M, int64_t* K) {
  if (!M || !K) return pb::fail(PB_ERR_NULL_POINTER, "pb_group_geometry: M and K must be non-null");
  pb::Geometry g;
  if (int s = pb::make_geometry(rows, cols, a, b, &g)) return s;
  *M = g.M;
  *K = g.K;
  return PB_OK;
}
