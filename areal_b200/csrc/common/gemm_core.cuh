// Persistent warp-specialised tcgen05 GEMM skeleton for sm_100a.
//
//   D[M,N] = A[M,K] * B[N,K]^T, bf16 operands, fp32 accumulation in TMEM.
//
// Roles (192 threads): warp 0 = TMA producer (one elected lane), warp 1 = MMA
// issuer (one elected lane, also owns the TMEM allocation), warps 2..5 = the
// epilogue (each warp reads its own quarter of the 128 TMEM lanes).
// The accumulator is double-buffered in TMEM (2 x BN fp32 columns), so the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// Operands may be K-major (the reduction index is contiguous in memory) or
// MN-major (the M / N index is contiguous); both come in through TMA with
// 128-byte swizzle, so forward (x W^T), dgrad (dy W) and wgrad (dy^T x) all run
// on the same kernel without a transposed copy.
//
// The epilogue and the tile order are supplied by a policy type `Epi`:
//   struct Epi {
//     __device__ bool tile(int cta, int ncta, int iter, int tiles_m, int tiles_n,
//                          int& m_blk, int& n_blk) const;   // false = done
//     __device__ bool gate(int m_blk, int n_blk, volatile int* abort, int* status) const;  // producer-side
//     __device__ void begin(State&, int m_blk, int n_blk, int row) const;
//     __device__ void chunk(State&, int row, int col0, const float (&v)[32]) const;
//     __device__ void end(State&, int m_blk, int n_blk, int row) const;
//   };
// Optional members for grouped (per-expert) problems; a policy without them gets the defaults:
//     int b_offset(int m_blk)  – added to B's row coordinate (K-major B: rows of the expert's weight
//                                inside a stacked [E*N, K] matrix; MN-major B: its reduction rows)   [0]
//     int a_m0(int m_blk)      – A's M coordinate of the tile                              [m_blk * 128]
//     int k_begin(int m_blk)   – first reduction element of the tile                                [0]
//     int k_blocks(int m_blk)  – number of 64-wide reduction blocks (0 = the tile is all zeros) [K / 64]
#pragma once
#include "ptx.cuh"

namespace b200 {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;

template <int BN>
struct GemmCfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;  // + align slack
  static constexpr int kTmemCols = 2 * BN;  // 512 for BN=256, 256 for BN=128
};

// Grouped raster: consecutive tile ids walk 8 row-blocks before moving to the
// next column block, so CTAs running at the same time share B columns and a
// small set of A rows in L2.
__device__ __forceinline__ bool default_tile(int cta, int ncta, int iter, int tiles_m, int tiles_n,
                                             int& m_blk, int& n_blk) {
  long long t = static_cast<long long>(iter) * ncta + cta;
  long long total = static_cast<long long>(tiles_m) * tiles_n;
  if (t >= total) return false;
  constexpr int G = 8;
  int per_group = G * tiles_n;
  int group = static_cast<int>(t / per_group);
  int first_m = group * G;
  int gsize = min(tiles_m - first_m, G);
  int r = static_cast<int>(t % per_group);
  m_blk = first_m + (r % gsize);
  n_blk = r / gsize;
  return true;
}

// Detection of the optional policy members (the int overload wins when the member exists).
template <class E> __device__ __forceinline__ auto epi_b_offset(const E& e, int m, int) -> decltype(e.b_offset(m)) { return e.b_offset(m); }
template <class E> __device__ __forceinline__ int epi_b_offset(const E&, int, long) { return 0; }
template <class E> __device__ __forceinline__ auto epi_a_m0(const E& e, int m, int) -> decltype(e.a_m0(m)) { return e.a_m0(m); }
template <class E> __device__ __forceinline__ int epi_a_m0(const E&, int m, long) { return m * kBM; }
template <class E> __device__ __forceinline__ auto epi_k_begin(const E& e, int m, int) -> decltype(e.k_begin(m)) { return e.k_begin(m); }
template <class E> __device__ __forceinline__ int epi_k_begin(const E&, int, long) { return 0; }
template <class E> __device__ __forceinline__ auto epi_k_blocks(const E& e, int m, int dflt, int) -> decltype(e.k_blocks(m)) { return e.k_blocks(m); }
template <class E> __device__ __forceinline__ int epi_k_blocks(const E&, int, int dflt, long) { return dflt; }

// k_load(m_blk, kb, ax, ay, bx, abort, status): per-K-block hook of the TMA producer. It may remap the
// K block (operand coordinates ax/ay for A, bx for B; K-major operands only) and wait, bounded, until
// the block's source has arrived; returning false aborts the kernel.
template <class E> __device__ __forceinline__ auto epi_k_load(const E& e, int m, int kb, int& ax, int& ay, int& bx,
                                                              volatile int* ab, int* st, int)
    -> decltype(e.k_load(m, kb, ax, ay, bx, ab, st)) { return e.k_load(m, kb, ax, ay, bx, ab, st); }
template <class E> __device__ __forceinline__ bool epi_k_load(const E&, int, int, int&, int&, int&, volatile int*, int*,
                                                              long) { return true; }

template <int BN, bool A_MN, bool B_MN, class Epi>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    int M, int N, int K, Epi epi, int* status) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * Cfg::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + kBM - 1) / kBM;
  const int tiles_n = (N + BN - 1) / BN;
  const int kblocks = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    if (elect_one_sync()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int it = 0; ok; ++it) {
        int m_blk, n_blk;
        if (!epi.tile(blockIdx.x, gridDim.x, it, tiles_m, tiles_n, m_blk, n_blk)) break;
        // fused all-gather→GEMM: wait (bounded) until the rows of this tile have arrived
        if (!epi.gate(m_blk, n_blk, abort_flag, status)) {
          ok = false;
          break;
        }
        const int kbn = epi_k_blocks(epi, m_blk, kblocks, 0);
        const int k0 = epi_k_begin(epi, m_blk, 0);
        const int a_m0 = epi_a_m0(epi, m_blk, 0);
        const int b_off = epi_b_offset(epi, m_blk, 0);
        for (int kb = 0; kb < kbn; ++kb) {
          int ax = k0 + kb * kBK, ay = a_m0, bx = k0 + kb * kBK;
          if (!epi_k_load(epi, m_blk, kb, ax, ay, bx, abort_flag, status, 0)) {
            ok = false;
            break;
          }
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[stage], Cfg::kStageBytes);
          uint8_t* a_dst = smem_a + stage * Cfg::kABytes;
          uint8_t* b_dst = smem_b + stage * Cfg::kBBytes;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j)
              tma_load_2d(a_dst + j * 8192, &tmA, &full[stage], a_m0 + j * 64, k0 + kb * kBK);
          } else {
            tma_load_2d(a_dst, &tmA, &full[stage], ax, ay);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * 8192, &tmB, &full[stage], n_blk * BN + j * 64, k0 + kb * kBK + b_off);
          } else {
            tma_load_2d(b_dst, &tmB, &full[stage], bx, n_blk * BN + b_off);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(status, 0, kErrMbarTimeoutProducer);
        // Give copies already in flight time to land before the CTA retires.
        unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer --
    if (elect_one_sync()) {
      constexpr uint32_t idesc = make_idesc(1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0, kBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int it = 0; ok; ++it) {
        int m_blk, n_blk;
        if (!epi.tile(blockIdx.x, gridDim.x, it, tiles_m, tiles_n, m_blk, n_blk)) break;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int kbn = epi_k_blocks(epi, m_blk, kblocks, 0);
        for (int kb = 0; kb < kbn; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + stage * Cfg::kABytes);
          const uint32_t b_addr = smem_u32(smem_b + stage * Cfg::kBBytes);
          const uint64_t a_desc =
              A_MN ? make_sdesc_sw128(a_addr, 8192, 1024) : make_sdesc_sw128(a_addr, 16, 1024);
          const uint64_t b_desc =
              B_MN ? make_sdesc_sw128(b_addr, 8192, 1024) : make_sdesc_sw128(b_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // Step 16 reduction elements: 32 bytes inside a K-major swizzle
            // row, 16 rows of 128 bytes in an MN-major tile.
            const uint64_t a_k = a_desc + static_cast<uint64_t>((A_MN ? 2048 : 32) * k >> 4);
            const uint64_t b_k = b_desc + static_cast<uint64_t>((B_MN ? 2048 : 32) * k >> 4);
            umma_f16(d_tmem, a_k, b_k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tfull[acc]);
      }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(status, 0, kErrMbarTimeoutMma);
      }
    }
  } else {
    // ---------------------------------------------------------- epilogue --
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
    typename Epi::State st;
    bool ok = true;
    for (int it = 0; ok; ++it) {
      int m_blk, n_blk;
      if (!epi.tile(blockIdx.x, gridDim.x, it, tiles_m, tiles_n, m_blk, n_blk)) break;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m_blk * kBM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool empty_tile = epi_k_blocks(epi, m_blk, kblocks, 0) == 0;  // nothing was accumulated
      epi.begin(st, m_blk, n_blk, row);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = empty_tile ? 0.f : __uint_as_float(r[i]);
        epi.chunk(st, row, n_blk * BN + c * 32, v);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      epi.end(st, m_blk, n_blk, row);
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
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace b200
