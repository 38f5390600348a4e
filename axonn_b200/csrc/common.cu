// Host-side error state and the per-device status word shared by all kernels.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace axb {

static thread_local char g_err[1024] = {0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return 0;
  set_error("%s: %s", what, cudaGetErrorString(e));
  return -1;
}

static std::mutex g_status_mu;
static unsigned int* g_status_host[64] = {nullptr};
static unsigned int* g_status_dev[64] = {nullptr};

volatile unsigned int* device_status_word(int device, unsigned int** dev_ptr) {
  std::lock_guard<std::mutex> lock(g_status_mu);
  if (device < 0 || device >= 64) return nullptr;
  if (!g_status_host[device]) {
    unsigned int* h = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&h), 64, cudaHostAllocMapped | cudaHostAllocPortable) !=
        cudaSuccess)
      return nullptr;
    for (int i = 0; i < 16; ++i) h[i] = 0;
    unsigned int* d = nullptr;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), h, 0) != cudaSuccess) return nullptr;
    g_status_host[device] = h;
    g_status_dev[device] = d;
  }
  if (dev_ptr) *dev_ptr = g_status_dev[device];
  return g_status_host[device];
}

// Two minutes: the order of a collective library's watchdog, so that ordinary skew between ranks (a slow
// data loader, a checkpoint write, a first-call compile) never expires a wait.  Tests shorten it.
static unsigned long long g_wait_timeout_ns = 120000000000ull;
unsigned long long wait_timeout_ns() { return g_wait_timeout_ns; }

}  // namespace axb

// Deadline after which a device-side wait (mbarrier, peer flag) gives up and reports through the status word.
extern "C" void axb_set_wait_timeout_ms(unsigned int ms) {
  axb::g_wait_timeout_ns = (ms < 1 ? 1ull : static_cast<unsigned long long>(ms)) * 1000000ull;
}

extern "C" const char* axb_last_error(void) { return axb::g_err; }

extern "C" unsigned int axb_device_status(int device, int clear) {
  volatile unsigned int* w = axb::device_status_word(device, nullptr);
  if (!w) return 0xFFFFFFFFu;
  unsigned int v = w[0];
  if (clear) w[0] = 0;
  return v;
}

// Diagnostic words next to the status word (index 1..15); reading clears when asked.
extern "C" unsigned int axb_debug_word(int device, int index, int clear) {
  volatile unsigned int* w = axb::device_status_word(device, nullptr);
  if (!w || index < 0 || index > 15) return 0;
  unsigned int v = w[index];
  if (clear) w[index] = 0;
  return v;
}
