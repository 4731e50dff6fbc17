// Block-scaled fp8 (e4m3) quantisation / dequantisation for sm_100a.
//
//   weights      128 x 128 blocks : scale = amax / 448, one fp32 scale_inv per block
//   activations  1 x 128 groups   : one fp32 scale per (row, 128-column group)
//
// Optional UE8M0 mode rounds every scale up to a power of two (the scale format
// Blackwell block-scaled MMA consumes), which keeps x / scale within range.
// 16-byte vector loads, warp-shuffle amax; each 128x128 block is read once into
// registers (a warp owns 4 rows of the block per step).
//
// Replaces the reference's Triton kernels `_blockwise_cast_to_fp8_triton` and
// `weight_dequant_kernel` (areal/engine/megatron_utils/fp8/kernels.py:13-156).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/host_utils.h"

namespace b200 {

constexpr float kFp8Max = 448.f;

__device__ __forceinline__ float round_scale(float s, int ue8m0) {
  if (!ue8m0) return s;
  // next power of two >= s
  int e;
  const float m = frexpf(s, &e);  // s = m * 2^e, m in [0.5, 1)
  return (m == 0.5f) ? ldexpf(1.f, e - 1) : ldexpf(1.f, e);
}

__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// One CTA (256 threads = 8 warps) per 128x128 block. Thread (warp w, lane l) handles rows
// w*16 .. w*16+15, columns 4*l .. 4*l+3 → 16 x 4 values in registers.
__global__ void __launch_bounds__(256)
quant_block128_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_fp8_e4m3* __restrict__ y,
                      long long ldy, float* __restrict__ scale_inv, int M, int N, int ue8m0) {
  const int bm = blockIdx.y, bn = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = bn * 128 + lane * 4;
  float v[16][4];
  float amax = 0.f;
#pragma unroll
  for (int r = 0; r < 16; ++r) {
    const int row = bm * 128 + warp * 16 + r;
#pragma unroll
    for (int c = 0; c < 4; ++c) v[r][c] = 0.f;
    if (row < M && col < N) {
      if (col + 3 < N && ((ldx & 3) == 0)) {
        const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<long long>(row) * ldx + col);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]);
        v[r][0] = a.x; v[r][1] = a.y; v[r][2] = b.x; v[r][3] = b.y;
      } else {
        for (int c = 0; c < 4 && col + c < N; ++c)
          v[r][c] = __bfloat162float(x[static_cast<long long>(row) * ldx + col + c]);
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) amax = fmaxf(amax, fabsf(v[r][c]));
  }
  __shared__ float s_max[8];
  amax = warp_max_f(amax);
  if (lane == 0) s_max[warp] = amax;
  __syncthreads();
  float bmax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) bmax = fmaxf(bmax, s_max[i]);
  const float scale = round_scale(fmaxf(bmax, 1e-12f) / kFp8Max, ue8m0);
  if (threadIdx.x == 0) scale_inv[static_cast<long long>(bm) * gridDim.x + bn] = scale;
#pragma unroll
  for (int r = 0; r < 16; ++r) {
    const int row = bm * 128 + warp * 16 + r;
    if (row < M && col < N) {
      __nv_fp8_e4m3 q[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) q[c] = __nv_fp8_e4m3(fminf(fmaxf(__fdiv_rn(v[r][c], scale), -kFp8Max), kFp8Max));
      __nv_fp8_e4m3* dst = y + static_cast<long long>(row) * ldy + col;
      if (col + 3 < N && ((ldy & 3) == 0)) {
        *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(q);
      } else {
        for (int c = 0; c < 4 && col + c < N; ++c) dst[c] = q[c];
      }
    }
  }
}

// One warp per (row, 128-column group): lane handles 4 columns.
__global__ void quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                   __nv_fp8_e4m3* __restrict__ y, long long ldy, float* __restrict__ scale,
                                   long long lds, int M, int K, int ue8m0) {
  const int groups = (K + 127) / 128;
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<long long>(M) * groups) return;
  const int row = static_cast<int>(gw / groups), g = static_cast<int>(gw % groups);
  const int col = g * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (col + 3 < K && ((ldx & 3) == 0)) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<long long>(row) * ldx + col);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
    for (int c = 0; c < 4 && col + c < K; ++c) v[c] = __bfloat162float(x[static_cast<long long>(row) * ldx + col + c]);
  }
  const float amax = warp_max_f(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
  const float sc = round_scale(fmaxf(amax, 1e-12f) / kFp8Max, ue8m0);
  if (lane == 0) scale[static_cast<long long>(row) * lds + g] = sc;
  __nv_fp8_e4m3 q[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) q[c] = __nv_fp8_e4m3(fminf(fmaxf(__fdiv_rn(v[c], sc), -kFp8Max), kFp8Max));
  __nv_fp8_e4m3* dst = y + static_cast<long long>(row) * ldy + col;
  if (col + 3 < K && ((ldy & 3) == 0)) {
    *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(q);
  } else {
    for (int c = 0; c < 4 && col + c < K; ++c) dst[c] = q[c];
  }
}

// y = x_fp8 * scale[block]; block_m == 1 selects 1x128 scales ([M, ceil(N/128)]), else 128x128.
__global__ void dequant_kernel(const __nv_fp8_e4m3* __restrict__ x, long long ldx, const float* __restrict__ scale,
                               long long lds, __nv_bfloat16* __restrict__ y, long long ldy, int M, int N,
                               int block_m) {
  const long long total = static_cast<long long>(M) * ((N + 3) / 4);
  const int nq = (N + 3) / 4;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(i / nq), col = static_cast<int>(i % nq) * 4;
    const float s = scale[static_cast<long long>(block_m == 1 ? row : row / 128) * lds + col / 128];
    for (int c = 0; c < 4 && col + c < N; ++c)
      y[static_cast<long long>(row) * ldy + col + c] =
          __float2bfloat16(static_cast<float>(x[static_cast<long long>(row) * ldx + col + c]) * s);
  }
}

}  // namespace b200

extern "C" {

// scale_inv: fp32 [ceil(M/128), ceil(N/128)] (the value to multiply by when dequantising).
int b200_quant_fp8_block128(const void* x, long long ldx, void* y, long long ldy, float* scale_inv, int M,
                            int N, int ue8m0, cudaStream_t stream) {
  using namespace b200;
  if (M == 0 || N == 0) return 0;
  dim3 grid((N + 127) / 128, (M + 127) / 128);
  quant_block128_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (__nv_fp8_e4m3*)y, ldy, scale_inv,
                                                  M, N, ue8m0);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// scale: fp32 [M, lds >= ceil(K/128)].
int b200_quant_fp8_1x128(const void* x, long long ldx, void* y, long long ldy, float* scale, long long lds,
                         int M, int K, int ue8m0, cudaStream_t stream) {
  using namespace b200;
  if (M == 0 || K == 0) return 0;
  const long long warps = static_cast<long long>(M) * ((K + 127) / 128);
  quant_1x128_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)x, ldx, (__nv_fp8_e4m3*)y, ldy, scale, lds, M, K, ue8m0);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_dequant_fp8(const void* x, long long ldx, const float* scale, long long lds, void* y, long long ldy,
                     int M, int N, int block_m, cudaStream_t stream) {
  using namespace b200;
  if (M == 0 || N == 0) return 0;
  long long g = (static_cast<long long>(M) * ((N + 3) / 4) + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 16;
  if (g > maxg) g = maxg;
  dequant_kernel<<<(unsigned)g, 256, 0, stream>>>((const __nv_fp8_e4m3*)x, ldx, scale, lds, (__nv_bfloat16*)y, ldy,
                                                 M, N, block_m);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
