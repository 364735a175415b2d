// Library-wide plumbing: version, status strings, last CUDA error.
#include <string>

#include "common.cuh"

#include <atomic>

namespace tsb {
namespace {
thread_local std::string g_last_error;
std::atomic<long long> g_launches{0};
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
void set_cuda_error(cudaError_t e) {
  g_last_error = cudaGetErrorString(e);
  (void)cudaGetLastError();  // clear the sticky-less error so later calls start clean
}
}  // namespace tsb

extern "C" {

const char* tsb_version(void) { return "tsb200 0.1 (sm_100a)"; }

const char* tsb_status_string(int status) {
  switch (status) {
    case TSB_OK: return "ok";
    case TSB_ERR_BAD_ARG: return "bad argument";
    case TSB_ERR_UNSUPPORTED: return "unsupported dtype or configuration";
    case TSB_ERR_WORKSPACE: return "workspace missing or too small";
    case TSB_ERR_CUDA: return "CUDA runtime error";
    case TSB_ERR_LIMIT: return "size beyond a stated maximum";
  }
  return "unknown status";
}

const char* tsb_last_cuda_error(void) { return tsb::g_last_error.c_str(); }

long long tsb_launch_count(void) { return tsb::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
