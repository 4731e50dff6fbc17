// Block-scaled fp8 (e4m3) GEMM on tcgen05 for sm_100a.
//
//   C[M,N] (bf16) = sum_kb  sa[m,kb] * sb[n/128,kb] * ( A8[m, kb-block] . B8[n, kb-block]^T )
//
// A8 [M,K] carries 1x128 scales (activations), B8 [N,K] carries 128x128 scales
// (weights) — the recipe of the reference's torchao / DeepGEMM / TransformerEngine
// block-wise paths (areal/experimental/models/archon/fp8.py:134-230,
// areal/engine/megatron_utils/fp8/*). Each 128-wide K block is multiplied on the
// tensor cores (kind::f8f6f4, fp32 accumulate) into one of two TMEM buffers; the
// epilogue warps drain a finished block, apply the two scales and add it to fp32
// accumulators held in registers ("promotion"), while the MMA warp already works
// on the next block in the other buffer. Same warp roles, TMA pipeline and
// bounded waits as the bf16 GEMM.
#include <cuda_fp8.h>

#include "common/host_utils.h"
#include "common/ptx.cuh"

namespace b200 {

constexpr int kF8BM = 128, kF8BN = 256, kF8BK = 128;  // BK in elements == bytes; a tile spans two 128-wide weight scale blocks
constexpr int kF8Stages = 4;
constexpr int kF8ABytes = kF8BM * kF8BK;              // 16 KB
constexpr int kF8BBytes = kF8BN * kF8BK;              // 32 KB
constexpr int kF8StageBytes = kF8ABytes + kF8BBytes;  // the wider tile halves the operand bytes per FLOP:
                                                      // the kernel is bound by the shared-memory fill rate
constexpr int kF8Smem = kF8Stages * kF8StageBytes + 1024 + 256;
constexpr int kF8Threads = 320;  // TMA warp, MMA warp, 8 promotion / epilogue warps

__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const float* __restrict__ sa, long long ldsa, const float* __restrict__ sb,
                      long long ldsb, __nv_bfloat16* __restrict__ C, long long ldc, int M, int N, int K,
                      int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kF8Stages * kF8ABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kF8Stages * kF8StageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kF8Stages;
  uint64_t* tfull = bars + 2 * kF8Stages;
  uint64_t* tempty = bars + 2 * kF8Stages + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * kF8Stages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + kF8BM - 1) / kF8BM, tiles_n = (N + kF8BN - 1) / kF8BN;
  const int kblocks = (K + kF8BK - 1) / kF8BK;
  const long long total = static_cast<long long>(tiles_m) * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kF8Stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 8); }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  auto tile_of = [&](int it, int& m_blk, int& n_blk) -> bool {
    const long long t = static_cast<long long>(it) * gridDim.x + blockIdx.x;
    if (t >= total) return false;
    constexpr int G = 8;
    const int per_group = G * tiles_n;
    const int group = static_cast<int>(t / per_group);
    const int first_m = group * G;
    const int gsize = min(tiles_m - first_m, G);
    const int r = static_cast<int>(t % per_group);
    m_blk = first_m + (r % gsize);
    n_blk = r / gsize;
    return true;
  };

  if (warp == 0) {
    if (elect_one_sync()) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int it = 0; ok; ++it) {
        int m_blk, n_blk;
        if (!tile_of(it, m_blk, n_blk)) break;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[stage], kF8StageBytes);
          tma_load_2d(smem_a + stage * kF8ABytes, &tmA, &full[stage], kb * kF8BK, m_blk * kF8BM);
          tma_load_2d(smem_b + stage * kF8BBytes, &tmB, &full[stage], kb * kF8BK, n_blk * kF8BN);
          if (++stage == kF8Stages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(status, 0, kErrMbarTimeoutProducer);
        unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (elect_one_sync()) {
      constexpr uint32_t idesc = make_idesc(0, 0, 0, 0, kF8BM, kF8BN);  // e4m3 x e4m3 → f32
      int stage = 0; uint32_t phase = 0; bool ok = true;
      long long g = 0;  // running k-block counter: TMEM buffer = g & 1
      for (int it = 0; ok; ++it) {
        int m_blk, n_blk;
        if (!tile_of(it, m_blk, n_blk)) break;
        for (int kb = 0; kb < kblocks; ++kb, ++g) {
          const int buf = static_cast<int>(g & 1);
          const uint32_t bph = static_cast<uint32_t>((g >> 1) & 1);
          if (!mbar_wait(&tempty[buf], bph ^ 1, abort_flag)) { ok = false; break; }
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + stage * kF8ABytes);
          const uint32_t b_addr = smem_u32(smem_b + stage * kF8BBytes);
#pragma unroll
          for (int k = 0; k < kF8BK / 32; ++k)
            umma_f8(tmem_base + buf * kF8BN, make_sdesc_sw128(a_addr + k * 32, 16, 1024),
                    make_sdesc_sw128(b_addr + k * 32, 16, 1024), idesc, k > 0 ? 1u : 0u);
          umma_commit(&empty[stage]);
          umma_commit(&tfull[buf]);
          if (++stage == kF8Stages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(status, 0, kErrMbarTimeoutMma);
      }
    }
  } else {
    // Two warps share every 32-lane quarter of TMEM (a warp may only touch lanes 32 * (warp % 4) ..),
    // each promoting one 64-column half of the tile: the per-K-block drain is the bottleneck of this
    // kernel, so it gets eight warps.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int kCols = kF8BN / 2;
    bool ok = true;
    long long g = 0;
    for (int it = 0; ok; ++it) {
      int m_blk, n_blk;
      if (!tile_of(it, m_blk, n_blk)) break;
      const int row = m_blk * kF8BM + quarter * 32 + lane;
      float acc[kCols];
#pragma unroll
      for (int i = 0; i < kCols; ++i) acc[i] = 0.f;
      for (int kb = 0; kb < kblocks && ok; ++kb, ++g) {
        const int buf = static_cast<int>(g & 1);
        const uint32_t bph = static_cast<uint32_t>((g >> 1) & 1);
        if (!mbar_wait(&tfull[buf], bph, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // this warp's 128 columns lie inside one 128-wide weight scale block
        const int sb_row = min(n_blk * (kF8BN / 128) + half, (N + 127) / 128 - 1);
        const float s = (row < M ? sa[static_cast<long long>(row) * ldsa + kb] : 0.f) *
                        sb[static_cast<long long>(sb_row) * ldsb + kb];
        const uint32_t t_row = tmem_base + buf * kF8BN + half * kCols + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
        for (int c = 0; c < kCols / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 32 + i] += __uint_as_float(r[i]) * s;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[buf]);
      }
      if (ok && row < M) {
        const int col0 = n_blk * kF8BN + half * kCols;
        __nv_bfloat16* out = C + static_cast<long long>(row) * ldc + col0;
        if (col0 + kCols <= N && (ldc & 7) == 0) {
#pragma unroll
          for (int i = 0; i < kCols / 8; ++i) {
            uint4 pk;
            __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int j = 0; j < 4; ++j) pb[j] = __floats2bfloat162_rn(acc[8 * i + 2 * j], acc[8 * i + 2 * j + 1]);
            reinterpret_cast<uint4*>(out)[i] = pk;
          }
        } else {
#pragma unroll
          for (int i = 0; i < kCols; ++i)
            if (col0 + i < N) out[i] = __float2bfloat16(acc[i]);
        }
      }
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicCAS(status, 0, kErrMbarTimeoutEpilogue);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200

extern "C" {

// A8 [M,K] e4m3 with sa [M, ldsa >= ceil(K/128)]; B8 [N,K] e4m3 with sb [ceil(N/128), ldsb >= ceil(K/128)].
// lda / ldb in elements (bytes), multiples of 16.
int b200_gemm_fp8_block(const void* A8, const void* B8, const float* sa, long long ldsa, const float* sb,
                        long long ldsb, void* C, int M, int N, int K, long long lda, long long ldb,
                        long long ldc, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 15) || (ldb & 15)) return -100;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, kF8BM, kF8BK);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, B8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, kF8BN, kF8BK);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CHECK(cudaFuncSetAttribute(gemm_fp8_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kF8Smem));
    attr_set = true;
  }
  const long long tiles = static_cast<long long>((M + kF8BM - 1) / kF8BM) * ((N + kF8BN - 1) / kF8BN);
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  int* status = device_status_word();
  if (!status) return -3;
  gemm_fp8_block_kernel<<<grid, kF8Threads, kF8Smem, stream>>>(tmA, tmB, sa, ldsa, sb, ldsb,
                                                              (__nv_bfloat16*)C, ldc, M, N, K, status);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
