// Token embedding: row gather (forward) and scatter-add of the output gradient into the fp32 main
// gradient of the table (backward). Both are pure memory movement: one warp moves one row with
// 16-byte accesses, so a launch runs at the HBM rate of reading and writing T rows.
//
// Ids outside [0, V) yield a zero row in the forward pass and are skipped in the backward pass (the
// vocab-parallel embedding relies on it: a rank looks up only the ids of its own vocabulary slice and
// the slices are summed afterwards).
//
// Role in the reference: torch.nn.Embedding inside the HF / Archon model code
// (areal/experimental/models/archon/qwen3/model/model.py) and Megatron's VocabParallelEmbedding.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/host_utils.h"

namespace b200 {

// H % 8 == 0. ids: int64.
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int T, int H, long long V) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int vec = H >> 3;  // uint4 per row
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < T; t += gridDim.x * warps_per_block) {
    const long long id = ids[t];
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H);
    if (id < 0 || id >= V) {
      for (int i = lane; i < vec; i += 32) dst[i] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * H);
    for (int i = lane; i < vec; i += 32) dst[i] = __ldg(src + i);
  }
}

// grad[id] += dy[t] in fp32. Rows of equal id collide, hence the vector atomic adds (sum order varies
// between runs; callers that need bit-stable sums take the sorted PyTorch path instead).
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dy,
                                     float* __restrict__ grad, int T, int H, long long V) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int vec = H >> 3;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < T; t += gridDim.x * warps_per_block) {
    const long long id = ids[t];
    if (id < 0 || id >= V) continue;
    const uint4* src = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(t) * H);
    float* dst = grad + static_cast<size_t>(id) * H;
    for (int i = lane; i < vec; i += 32) {
      const uint4 u = __ldg(src + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
      const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
      const float2 c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
      float* p = dst + (i << 3);
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a.x), "f"(a.y), "f"(b.x),
                   "f"(b.y)
                   : "memory");
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p + 4), "f"(c.x), "f"(c.y), "f"(d.x),
                   "f"(d.y)
                   : "memory");
    }
  }
}

}  // namespace b200

extern "C" {

int b200_embedding_fwd(const void* ids, const void* table, void* out, int T, int H, long long V,
                       cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return -1;
  const int threads = 256, wpb = threads / 32;
  const int blocks = min((T + wpb - 1) / wpb, 148 * 8);
  b200::embedding_fwd_kernel<<<blocks, threads, 0, stream>>>(
      static_cast<const long long*>(ids), static_cast<const __nv_bfloat16*>(table),
      static_cast<__nv_bfloat16*>(out), T, H, V);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_embedding_bwd(const void* ids, const void* dy, float* grad, int T, int H, long long V,
                       cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return -1;
  const int threads = 256, wpb = threads / 32;
  const int blocks = min((T + wpb - 1) / wpb, 148 * 8);
  b200::embedding_bwd_kernel<<<blocks, threads, 0, stream>>>(
      static_cast<const long long*>(ids), static_cast<const __nv_bfloat16*>(dy), grad, T, H, V);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
