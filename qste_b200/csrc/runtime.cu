// Library-wide helpers: status strings, last CUDA error, device queries.
#include <atomic>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace qste {

static thread_local char g_last_error[512] = "";

void set_last_cuda_error(cudaError_t error, const char* where) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", where, cudaGetErrorName(error),
           cudaGetErrorString(error));
}

// the kernel family the calling thread's last forward ran (see qste_b200_last_forward_kernel)
static thread_local const char* g_last_forward = "";
void note_forward_kernel(const char* name) { g_last_forward = name; }

static std::atomic<unsigned long long> g_launches{0};
void note_launches(int count) { g_launches.fetch_add((unsigned long long)count, std::memory_order_relaxed); }

// SMs the persistent GEMMs of the calling thread leave free (see qste_b200_set_reserved_sms);
// -1: not set yet, take QSTE_B200_RESERVED_SMS from the environment
static thread_local int g_reserved_sms = -1;

int reserved_sms() {
  if (g_reserved_sms < 0) {
    const char* text = getenv("QSTE_B200_RESERVED_SMS");
    const int value = text ? atoi(text) : 0;
    g_reserved_sms = value > 0 ? value : 0;
  }
  return g_reserved_sms;
}

int sm_count() {
  static int cached[64];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
  if (cached[device] == 0) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        count <= 0)
      count = 148;
    cached[device] = count;
  }
  return cached[device];
}

int check_arch() {
  static int cached[64];  // 0 unknown, 1 ok, 2 wrong
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) {
    set_last_cuda_error(error, "cudaGetDevice");
    return QSTE_ERR_CUDA;
  }
  if (device < 0 || device >= 64) return QSTE_OK;
  if (cached[device] == 0) {
    int major = 0;
    error = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (error != cudaSuccess) {
      set_last_cuda_error(error, "cudaDeviceGetAttribute");
      return QSTE_ERR_CUDA;
    }
    cached[device] = (major == 10) ? 1 : 2;
  }
  return cached[device] == 1 ? QSTE_OK : QSTE_ERR_ARCH;
}

}  // namespace qste

extern "C" {

int qste_b200_abi_version(void) { return QSTE_B200_ABI_VERSION; }

const char* qste_b200_status_string(int status) {
  switch (status) {
    case QSTE_OK: return "ok";
    case QSTE_ERR_SHAPE: return "shape mismatch or invalid size";
    case QSTE_ERR_DTYPE: return "unknown dtype";
    case QSTE_ERR_ALIGNMENT: return "misaligned pointer";
    case QSTE_ERR_WORKSPACE: return "workspace missing or too small";
    case QSTE_ERR_CUDA: return "CUDA call failed";
    case QSTE_ERR_UNSUPPORTED: return "unsupported argument combination";
    case QSTE_ERR_NULL: return "required pointer is NULL";
    case QSTE_ERR_ARCH: return "device is not compute capability 10.x (B200)";
    case QSTE_ERR_LIMIT: return "size beyond a fixed maximum";
    default: return "unknown status";
  }
}

const char* qste_b200_last_cuda_error(void) { return qste::g_last_error; }

int qste_b200_set_reserved_sms(int count) {
  const int previous = qste::reserved_sms();
  qste::g_reserved_sms = count > 0 ? count : 0;
  return previous;
}

const char* qste_b200_last_forward_kernel(void) { return qste::g_last_forward; }

unsigned long long qste_b200_launch_count(void) { return qste::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
