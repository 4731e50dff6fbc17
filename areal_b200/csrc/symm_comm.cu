// Symmetric-memory runtime over NVLink / NVSwitch peer access.
//
// Every rank allocates the same buffers with b200_symm_alloc, exports them with
// CUDA IPC and maps its peers' buffers; kernels then read and write peer memory
// directly with plain loads/stores (no TMA multicast). Synchronisation is a
// flag barrier in symmetric memory: release-stores of an epoch number into
// every peer's flag array and acquire-loads on the own array, with a
// wall-clock bound after which the kernel records kErrPeerFlagTimeout in the
// status word and returns, so a missing peer never wedges the GPU.
//
// On top of it: all-gather (each rank pushes its shard into every peer),
// one-shot all-reduce (each rank pulls and sums all peers; latency-bound
// sizes), reduce-scatter (each rank pulls and sums its slice) and all-to-all
// (each rank pushes chunk p to peer p). They stand in for the NCCL calls of the
// reference (areal/models/fsdp/ulysses.py:153-204,
// areal/utils/functional/vocab_parallel.py:136-158) and are the unfused
// baselines of the fused compute+collective kernels.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "common/host_utils.h"
#include "common/ptx.cuh"

namespace b200 {

constexpr int kMaxPeers = 16;
struct PeerPtrs {
  void* p[kMaxPeers];
};

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Thread t < world signals peer t and waits for peer t's signal.
__device__ __forceinline__ bool flag_barrier(const PeerPtrs& flags, int rank, int world,
                                             uint32_t epoch, int* status) {
  bool ok = true;
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(flags.p[t]) + rank, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[rank]) + t;
    unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > kWaitDeadlineNs) {
        atomicCAS(status, 0, kErrPeerFlagTimeout);
        ok = false;
        break;
      }
    }
  }
  return ok;
}

__global__ void barrier_kernel(PeerPtrs flags, int rank, int world, uint32_t epoch, int* status) {
  flag_barrier(flags, rank, world, epoch, status);
}

// dst buffers: peer p's buffer receives this rank's `bytes` at byte offset dst_off.
__global__ void push_all_kernel(PeerPtrs dst, int world, const uint4* __restrict__ src,
                                long long n16, long long dst_off16) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = src[i];
    for (int p = 0; p < world; ++p) reinterpret_cast<uint4*>(dst.p[p])[dst_off16 + i] = v;
  }
}

// Plan-driven weight push (trainer -> rollout with re-sharding): segment s copies `rows` rows of
// `row16` 16-byte vectors from src (row pitch src_pitch16) into every destination buffer at dst_off16
// (row pitch dst_pitch16). One block per segment piece; the host cuts large segments into pieces so the
// grid fills the machine. A tensor-parallel shard of a column-split weight lands as a strided block
// inside the full matrix, a row-split shard or an expert block as a contiguous range.
struct PushSeg {
  long long src_off16, dst_off16;
  long long src_pitch16, dst_pitch16;
  int rows, row16;
};

__global__ void push_plan_kernel(PeerPtrs dst, int world, const uint4* __restrict__ src,
                                 const PushSeg* __restrict__ segs, int nsegs) {
  for (int s = blockIdx.x; s < nsegs; s += gridDim.x) {
    const PushSeg g = segs[s];
    const long long total = static_cast<long long>(g.rows) * g.row16;
    for (long long i = threadIdx.x; i < total; i += blockDim.x) {
      const long long r = i / g.row16, c = i - r * g.row16;
      const uint4 v = src[g.src_off16 + r * g.src_pitch16 + c];
      const long long at = g.dst_off16 + r * g.dst_pitch16 + c;
      for (int p = 0; p < world; ++p) reinterpret_cast<uint4*>(dst.p[p])[at] = v;
    }
  }
}

// all-to-all: chunk p of src (chunk16 uint4 each) goes to peer p at slot `rank`.
__global__ void a2a_push_kernel(PeerPtrs dst, int world, int rank, const uint4* __restrict__ src,
                                long long chunk16) {
  const long long total = chunk16 * world;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int p = static_cast<int>(i / chunk16);
    const long long j = i - p * chunk16;
    reinterpret_cast<uint4*>(dst.p[p])[static_cast<long long>(rank) * chunk16 + j] = src[i];
  }
}

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// out[i] = sum_p src[p][offset + i]  (pull; fp32 accumulation)
template <typename T>
__global__ void pull_reduce_kernel(PeerPtrs src, int world, long long offset, long long n,
                                   T* __restrict__ out) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float a = 0.f;
    for (int p = 0; p < world; ++p) a += to_f<T>(reinterpret_cast<const T*>(src.p[p])[offset + i]);
    out[i] = from_f<T>(a);
  }
}

// One-shot all-reduce with both barriers inside the kernel (single launch):
// enter barrier → pull+sum → exit barrier. Grid of 1 block for tiny payloads.
__global__ void allreduce_oneshot_kernel(PeerPtrs bufs, PeerPtrs flags, int rank, int world,
                                         uint32_t epoch, long long n, float* __restrict__ out,
                                         int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (!flag_barrier(flags, rank, world, epoch, status)) s_ok = 0;
  __syncthreads();
  if (s_ok) {
    for (long long i = threadIdx.x; i < n; i += blockDim.x) {
      float a = 0.f;
      for (int p = 0; p < world; ++p) a += reinterpret_cast<const float*>(bufs.p[p])[i];
      out[i] = a;
    }
  }
  __syncthreads();
  flag_barrier(flags, rank, world, epoch + 1, status);
}

static inline unsigned grid_for(long long n) {
  long long g = (n + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 4;
  if (g > maxg) g = maxg;
  if (g < 1) g = 1;
  return static_cast<unsigned>(g);
}

static inline bool fill(PeerPtrs& pp, void* const* ptrs, int world) {
  if (world < 1 || world > kMaxPeers) return false;
  for (int i = 0; i < world; ++i) pp.p[i] = ptrs[i];
  return true;
}

}  // namespace b200

extern "C" {

void* b200_symm_alloc(size_t bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, bytes);
  cudaDeviceSynchronize();
  return p;
}
int b200_symm_free(void* p) {
  B200_CHECK(cudaFree(p));
  return 0;
}
int b200_ipc_get_handle(void* ptr, void* out64) {
  cudaIpcMemHandle_t h;
  B200_CHECK(cudaIpcGetMemHandle(&h, ptr));
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(out64, &h, 64);
  return 0;
}
void* b200_ipc_open_handle(const void* in64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, in64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    fprintf(stderr, "[areal_b200] cudaIpcOpenMemHandle failed: %s\n", cudaGetErrorString(e));
    return nullptr;
  }
  return p;
}
int b200_ipc_close_handle(void* p) {
  B200_CHECK(cudaIpcCloseMemHandle(p));
  return 0;
}
// Single-process multi-device use (tests, colocated engines): enable peer access.
int b200_enable_peer_access(int dev, int peer) {
  int can = 0;
  B200_CHECK(cudaDeviceCanAccessPeer(&can, dev, peer));
  if (!can) return -100;
  int cur = 0;
  B200_CHECK(cudaGetDevice(&cur));
  B200_CHECK(cudaSetDevice(dev));
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
    cudaSetDevice(cur);
    return -static_cast<int>(e);
  }
  cudaGetLastError();
  B200_CHECK(cudaSetDevice(cur));
  return 0;
}

int b200_symm_barrier(void* const* peer_flags, int rank, int world, unsigned epoch,
                      cudaStream_t stream) {
  using namespace b200;
  PeerPtrs f;
  if (!fill(f, peer_flags, world)) return -100;
  int* status = device_status_word();
  if (!status) return -3;
  barrier_kernel<<<1, 32, 0, stream>>>(f, rank, world, epoch, status);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// Copies `bytes` (multiple of 16) from src into every peer buffer at dst_offset_bytes.
int b200_push_all(void* const* peer_bufs, int world, const void* src, long long bytes,
                  long long dst_offset_bytes, cudaStream_t stream) {
  using namespace b200;
  PeerPtrs d;
  if (!fill(d, peer_bufs, world)) return -100;
  if ((bytes & 15) || (dst_offset_bytes & 15)) return -101;
  if (bytes == 0) return 0;
  push_all_kernel<<<grid_for(bytes / 16), 256, 0, stream>>>(d, world, (const uint4*)src, bytes / 16,
                                                            dst_offset_bytes / 16);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// segs: device array of `nsegs` PushSeg records (6 x int64-sized fields: src_off16, dst_off16, src_pitch16,
// dst_pitch16, then rows and row16 as two int32). All offsets and pitches in 16-byte units.
int b200_push_plan(void* const* peer_bufs, int world, const void* src, const void* segs, int nsegs,
                   cudaStream_t stream) {
  using namespace b200;
  PeerPtrs d;
  if (!fill(d, peer_bufs, world)) return -100;
  if (nsegs <= 0) return 0;
  const int maxg = sm_count() * 8;
  push_plan_kernel<<<nsegs < maxg ? nsegs : maxg, 512, 0, stream>>>(d, world, (const uint4*)src,
                                                                    (const PushSeg*)segs, nsegs);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_a2a_push(void* const* peer_bufs, int world, int rank, const void* src,
                  long long chunk_bytes, cudaStream_t stream) {
  using namespace b200;
  PeerPtrs d;
  if (!fill(d, peer_bufs, world)) return -100;
  if (chunk_bytes & 15) return -101;
  if (chunk_bytes == 0) return 0;
  a2a_push_kernel<<<grid_for(chunk_bytes / 16 * world), 256, 0, stream>>>(
      d, world, rank, (const uint4*)src, chunk_bytes / 16);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// out[i] = sum over peers of peer[offset + i]; dtype 0 = fp32, 1 = bf16.
int b200_pull_reduce(void* const* peer_bufs, int world, long long offset, long long n, void* out,
                     int dtype, cudaStream_t stream) {
  using namespace b200;
  PeerPtrs s;
  if (!fill(s, peer_bufs, world)) return -100;
  if (n == 0) return 0;
  if (dtype == 0)
    pull_reduce_kernel<float><<<grid_for(n), 256, 0, stream>>>(s, world, offset, n, (float*)out);
  else
    pull_reduce_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, stream>>>(s, world, offset, n,
                                                                      (__nv_bfloat16*)out);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// Uses epochs `epoch` and `epoch + 1`.
int b200_allreduce_oneshot_f32(void* const* peer_bufs, void* const* peer_flags, int rank,
                               int world, unsigned epoch, long long n, float* out,
                               cudaStream_t stream) {
  using namespace b200;
  PeerPtrs b, f;
  if (!fill(b, peer_bufs, world) || !fill(f, peer_flags, world)) return -100;
  int* status = device_status_word();
  if (!status) return -3;
  allreduce_oneshot_kernel<<<1, 256, 0, stream>>>(b, f, rank, world, epoch, n, out, status);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
