// Per-device status word. Kernels set it (atomicCAS from 0) when a bounded wait
// expires or a self-check fails; the host polls it after a synchronisation
// point and raises instead of letting a wedged kernel spin.
#include "host_utils.h"

namespace b200 {

static int* g_status[64] = {nullptr};

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_status[dev] = p;
  }
  return g_status[dev];
}

}  // namespace b200

extern "C" {

// Address of the current device's status word (0 when it cannot be created).
void* b200_status_ptr() { return b200::device_status_word(); }

// Synchronises `stream`, returns the status word and clears it.
int b200_read_status(cudaStream_t stream) {
  int* p = b200::device_status_word();
  if (!p) return -1;
  int h = 0;
  B200_CHECK(cudaMemcpyAsync(&h, p, sizeof(int), cudaMemcpyDeviceToHost, stream));
  B200_CHECK(cudaStreamSynchronize(stream));
  if (h != 0) {
    B200_CHECK(cudaMemsetAsync(p, 0, sizeof(int), stream));
    B200_CHECK(cudaStreamSynchronize(stream));
  }
  return h;
}

int b200_sm_count() { return b200::sm_count(); }

// Binds the calling host thread to `dev` in this library's CUDA runtime.
// Threads that PyTorch creates (the autograd engine's workers) have no current
// context for a second runtime instance until one is bound, and the driver's
// tensor-map encoder refuses to run without one.
int b200_ensure_device(int dev) {
  static thread_local int cur = -1;
  if (cur != dev) {
    B200_CHECK(cudaSetDevice(dev));
    B200_CHECK(cudaFree(0));
    cur = dev;
  }
  return 0;
}

}  // extern "C"
