// bf16 GEMM on tcgen05/TMEM for forward, dgrad and wgrad of every linear layer.
//
//   C[M,N] (bf16 or fp32, optionally C += ...) = A * B^T (+ bias[N])
//
// a_mn = 0: A is stored [M,K] row-major (K contiguous);  a_mn = 1: A is stored
// [K,M] row-major (M contiguous). Same for B with N. This covers
//   forward  y  = x W^T      : A = x [T,in]  (K-major), B = W [out,in] (K-major)
//   dgrad    dx = dy W       : A = dy [T,out] (K-major), B = W [out,in] read as [K=out, N=in] (MN-major)
//   wgrad    dW = dy^T x     : A = dy [T,out] read as [K=T, M=out] (MN-major), B = x [T,in] as [K=T, N=in] (MN-major)
// Replaces the cuBLAS calls behind nn.Linear in the reference
// (areal/experimental/models/archon/qwen3/model/model.py:103-293).
#include "common/gemm_core.cuh"
#include "common/host_utils.h"

namespace b200 {

struct StoreEpi {
  void* C;
  const __nv_bfloat16* bias;
  long long ldc;
  int M, N;
  int out_fp32;
  int accumulate;
  struct State {};

  __device__ __forceinline__ bool tile(int cta, int ncta, int it, int tiles_m, int tiles_n,
                                       int& m_blk, int& n_blk) const {
    return default_tile(cta, ncta, it, tiles_m, tiles_n, m_blk, n_blk);
  }
  __device__ __forceinline__ bool gate(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ void begin(State&, int, int, int) const {}
  __device__ __forceinline__ void end(State&, int, int, int) const {}
  __device__ __forceinline__ void chunk(State&, int row, int col0, const float (&v_in)[32]) const {
    if (row >= M || col0 >= N) return;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = v_in[i];
    const bool full = (col0 + 32 <= N);
    if (bias) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (full || col0 + i < N) v[i] += __bfloat162float(bias[col0 + i]);
    }
    if (out_fp32) {
      float* p = reinterpret_cast<float*>(C) + static_cast<long long>(row) * ldc + col0;
      if (full && (ldc & 3) == 0) {
        float4* p4 = reinterpret_cast<float4*>(p);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float4 o = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          if (accumulate) {
            float4 old = p4[i];
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
          }
          p4[i] = o;
        }
      } else {
        for (int i = 0; i < 32; ++i)
          if (col0 + i < N) p[i] = accumulate ? p[i] + v[i] : v[i];
      }
    } else {
      __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(C) + static_cast<long long>(row) * ldc + col0;
      if (full && (ldc & 7) == 0) {
        uint4* p4 = reinterpret_cast<uint4*>(p);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = v[8 * i + j];
          if (accumulate) {
            uint4 old = p4[i];
            const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float2 of = __bfloat1622float2(ob[j]);
              f[2 * j] += of.x;
              f[2 * j + 1] += of.y;
            }
          }
          uint4 o;
          __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int j = 0; j < 4; ++j) ob2[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
          p4[i] = o;
        }
      } else {
        for (int i = 0; i < 32; ++i)
          if (col0 + i < N) {
            float x = v[i];
            if (accumulate) x += __bfloat162float(p[i]);
            p[i] = __float2bfloat16(x);
          }
      }
    }
  }
};

template <int BN, bool A_MN, bool B_MN>
static int launch(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                  long long lda, long long ldb, long long ldc, int out_fp32, int accumulate,
                  cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if (A_MN)
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda * 2, 64, 64);
  else
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda * 2, kBM, 64);
  if (rc) return rc;
  if (B_MN)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb * 2, 64, 64);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb * 2, BN, 64);
  if (rc) return rc;
  StoreEpi epi{C, reinterpret_cast<const __nv_bfloat16*>(bias), ldc, M, N, out_fp32, accumulate};
  auto kern = gemm_tcgen05_kernel<BN, A_MN, B_MN, StoreEpi>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::kSmemBytes));
    attr_set = true;
  }
  long long tiles = static_cast<long long>((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
  int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  if (grid <= 0) return 0;
  int* status = device_status_word();
  if (!status) return -3;
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(tmA, tmB, M, N, K, epi, status);
  B200_CHECK(cudaGetLastError());
  return 0;
}


// ---------------------------------------------------------------- grouped (per-expert) GEMMs --
// Rows live in the padded, expert-sorted layout produced by the MoE sort: tile vm (128 rows)
// belongs to expert tile_expert[vm]; *num_vm tiles are in use (device-side value, so no host
// sync); weights are stacked as [E * rows_per_expert, cols].
struct GroupedEpi {
  StoreEpi st;
  const int* tile_expert;
  const int* num_vm;
  int b_rows_per_expert;  // rows of the stacked B that belong to one expert
  using State = StoreEpi::State;

  __device__ __forceinline__ bool tile(int cta, int ncta, int it, int, int tiles_n, int& m_blk, int& n_blk) const {
    const long long t = static_cast<long long>(it) * ncta + cta;
    if (t >= static_cast<long long>(*num_vm) * tiles_n) return false;
    m_blk = static_cast<int>(t / tiles_n);
    n_blk = static_cast<int>(t % tiles_n);
    return true;
  }
  __device__ __forceinline__ int b_offset(int m_blk) const { return tile_expert[m_blk] * b_rows_per_expert; }
  __device__ __forceinline__ bool gate(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ void begin(State&, int, int, int) const {}
  __device__ __forceinline__ void end(State&, int, int, int) const {}
  __device__ __forceinline__ void chunk(State& s, int row, int col0, const float (&v)[32]) const {
    st.chunk(s, row, col0, v);
  }
};

// dW[e] = dy_e^T x_e: the M dimension runs over the stacked weight rows [E * N], the reduction over
// the (padded, zero-filled) rows of expert e = (m_blk * 128) / N.
struct GroupedWgradEpi {
  StoreEpi st;
  const int* prow0;  // [E + 1] first padded row of every expert
  int n_per_expert;
  using State = StoreEpi::State;

  __device__ __forceinline__ bool tile(int cta, int ncta, int it, int tiles_m, int tiles_n, int& m_blk,
                                       int& n_blk) const {
    return default_tile(cta, ncta, it, tiles_m, tiles_n, m_blk, n_blk);
  }
  __device__ __forceinline__ int expert(int m_blk) const { return (m_blk * kBM) / n_per_expert; }
  __device__ __forceinline__ int a_m0(int m_blk) const { return (m_blk * kBM) % n_per_expert; }
  __device__ __forceinline__ int k_begin(int m_blk) const { return prow0[expert(m_blk)]; }
  __device__ __forceinline__ int k_blocks(int m_blk) const {
    const int e = expert(m_blk);
    return (prow0[e + 1] - prow0[e]) / kBK;
  }
  __device__ __forceinline__ bool gate(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ void begin(State&, int, int, int) const {}
  __device__ __forceinline__ void end(State&, int, int, int) const {}
  __device__ __forceinline__ void chunk(State& s, int row, int col0, const float (&v)[32]) const {
    st.chunk(s, row, col0, v);
  }
};

template <bool B_MN>
static int launch_grouped(const void* A, const void* B, void* C, const int* tile_expert, const int* num_vm,
                          int max_rows, int E, int N, int K, cudaStream_t stream) {
  constexpr int BN = 128;
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, max_rows, K, (long long)K * 2, kBM, 64);
  if (rc) return rc;
  if (B_MN)  // stacked [E*K, N], N contiguous
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (long long)E * K, N, (long long)N * 2, 64, 64);
  else       // stacked [E*N, K], K contiguous
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (long long)E * N, K, (long long)K * 2, BN, 64);
  if (rc) return rc;
  GroupedEpi epi{StoreEpi{C, nullptr, N, max_rows, N, 0, 0}, tile_expert, num_vm, B_MN ? K : N};
  auto kern = gemm_tcgen05_kernel<BN, false, B_MN, GroupedEpi>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set = true;
  }
  const long long tiles = static_cast<long long>((max_rows + kBM - 1) / kBM) * ((N + BN - 1) / BN);
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  if (grid <= 0) return 0;
  int* status = device_status_word();
  if (!status) return -3;
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(tmA, tmB, max_rows, N, K, epi, status);
  B200_CHECK(cudaGetLastError());
  return 0;
}


// ------------------------------------------------------------------------------ split-K --
// Skinny products (a decode step: M <= a few hundred rows against a large weight) have too few
// output tiles to occupy 148 SMs, and each CTA would stream its whole K extent at one SM's share
// of the HBM bandwidth. Split-K gives every (tile, K-slice) pair its own CTA: slice s of tile
// (m, n) is the virtual row block s * tiles_m + m, its partial sums go to an fp32 workspace
// [S, tiles_m * 128, N] and a small kernel adds the slices (+ bias) into the bf16 output.
struct SplitKEpi {
  StoreEpi st;   // writes the fp32 workspace, M = S * tiles_m * 128
  int tiles_m_real, kper, kblocks_total;
  using State = StoreEpi::State;

  __device__ __forceinline__ bool tile(int cta, int ncta, int it, int tiles_m_virtual, int tiles_n, int& m_blk,
                                       int& n_blk) const {
    const long long t = static_cast<long long>(it) * ncta + cta;
    if (t >= static_cast<long long>(tiles_m_virtual) * tiles_n) return false;
    // consecutive CTAs take the K slices of one output tile, then the next column block
    m_blk = static_cast<int>(t % tiles_m_virtual);
    n_blk = static_cast<int>(t / tiles_m_virtual);
    return true;
  }
  __device__ __forceinline__ int a_m0(int mv) const { return (mv % tiles_m_real) * kBM; }
  __device__ __forceinline__ int k_begin(int mv) const { return (mv / tiles_m_real) * kper * kBK; }
  __device__ __forceinline__ int k_blocks(int mv) const {
    const int left = kblocks_total - (mv / tiles_m_real) * kper;
    return left < kper ? (left > 0 ? left : 0) : kper;
  }
  __device__ __forceinline__ bool gate(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ void begin(State&, int, int, int) const {}
  __device__ __forceinline__ void end(State&, int, int, int) const {}
  __device__ __forceinline__ void chunk(State& s, int row, int col0, const float (&v)[32]) const {
    st.chunk(s, row, col0, v);
  }
};

__global__ void splitk_reduce_kernel(const float* __restrict__ ws, const __nv_bfloat16* __restrict__ bias,
                                     __nv_bfloat16* __restrict__ out, long long ldc, int M, int N, int S,
                                     long long slice_stride) {
  const int nq = N >> 2;
  const long long total = static_cast<long long>(M) * nq;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(i / nq), c = static_cast<int>(i % nq) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < S; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(ws + s * slice_stride + static_cast<long long>(row) * N + c);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (bias) {
      acc.x += __bfloat162float(bias[c]); acc.y += __bfloat162float(bias[c + 1]);
      acc.z += __bfloat162float(bias[c + 2]); acc.w += __bfloat162float(bias[c + 3]);
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + static_cast<long long>(row) * ldc + c) = pk;
  }
}

// Split-K reduction fused with the residual add and RMSNorm that follow a projection in a decoder
// block: one warp per row sums the S fp32 slices (+ bias), rounds to bf16 (the projection's output
// precision), adds the bf16 residual stream, stores the new residual (bf16) and the normalised row.
// Every rounding step of the unfused sequence (GEMM → bf16, residual add → bf16, norm) is kept, so
// the results are bit-identical to it. N = 256 * NV at most (a lane owns NV groups of 8 columns).
template <int NV>
__global__ void splitk_reduce_rmsnorm_kernel(const float* __restrict__ ws, const __nv_bfloat16* __restrict__ bias,
                                             const __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ w,
                                             __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ res_out,
                                             int M, int N, int S, long long slice_stride, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = N >> 3;
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); row < M;
       row += static_cast<long long>(gridDim.x) * warps_per_block) {
    float v[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int sl = 0; sl < S; ++sl) {
          const float4* src = reinterpret_cast<const float4*>(ws + sl * slice_stride + row * N + c * 8);
          const float4 a = src[0], b = src[1];
          acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
          acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
        }
        if (bias) {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(bias[c * 8 + j]);
        }
        uint4 rraw = res ? reinterpret_cast<const uint4*>(res + row * N)[c] : make_uint4(0, 0, 0, 0);
        const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rraw);
        uint4 hraw;
        __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&hraw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // projection output in bf16, then the residual add in fp32, then the bf16 residual stream
          const float2 a2 = __bfloat1622float2(__floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]));
          const float2 r2 = __bfloat1622float2(rp[j]);
          hp[j] = res ? __floats2bfloat162_rn(a2.x + r2.x, a2.y + r2.y) : __floats2bfloat162_rn(a2.x, a2.y);
          const float2 h2 = __bfloat1622float2(hp[j]);
          v[i][2 * j] = h2.x;
          v[i][2 * j + 1] = h2.y;
          ss += h2.x * h2.x;  // same accumulation order as the stand-alone RMSNorm kernel
          ss += h2.y * h2.y;
        }
        reinterpret_cast<uint4*>(res_out + row * N)[c] = hraw;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rs = rsqrtf(ss / N + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        const uint4 wraw = reinterpret_cast<const uint4*>(w)[c];
        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wraw);
        uint4 oraw;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 w2 = __bfloat1622float2(wp[j]);
          op[j] = __floats2bfloat162_rn(v[i][2 * j] * rs * w2.x, v[i][2 * j + 1] * rs * w2.y);
        }
        reinterpret_cast<uint4*>(y + row * N)[c] = oraw;
      }
    }
  }
}

}  // namespace b200

extern "C" {

// Row pitches lda/ldb/ldc are in elements. All pitches and base pointers must
// be multiples of 16 bytes (TMA requirement); K, and the contiguous extent of
// an MN-major operand, must be multiples of 8.
int b200_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                   long long lda, long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32,
                   int accumulate, int bn, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -100;
#define DISPATCH(BN_)                                                                              \
  if (!a_mn && !b_mn)                                                                              \
    return launch<BN_, false, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_fp32, accumulate, \
                                     stream);                                                      \
  if (!a_mn && b_mn)                                                                               \
    return launch<BN_, false, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_fp32, accumulate,  \
                                    stream);                                                       \
  if (a_mn && b_mn)                                                                                \
    return launch<BN_, true, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_fp32, accumulate,   \
                                   stream);                                                        \
  return launch<BN_, true, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_fp32, accumulate,    \
                                  stream);
  if (bn == 128) {
    DISPATCH(128)
  }
  DISPATCH(256)
#undef DISPATCH
}

// Grouped forward / dgrad over the padded expert-sorted rows:
//   b_mn == 0:  C[r, :N] = A[r, :K] . W[e(r)]^T   with W stacked [E, N, K]
//   b_mn == 1:  C[r, :N] = A[r, :K] . W[e(r)]     with W stacked [E, K, N]   (K % 64 == 0)
// A is [max_rows, K] and C [max_rows, N], both contiguous bf16; N % 8 == 0, K % 8 == 0.
int b200_gemm_grouped(const void* A, const void* B, void* C, const int* tile_expert, const int* num_vm,
                      int max_rows, int E, int N, int K, int b_mn, cudaStream_t stream) {
  using namespace b200;
  if (max_rows <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 7) || (K & 7) || (b_mn && (K % 64))) return -100;
  return b_mn ? launch_grouped<true>(A, B, C, tile_expert, num_vm, max_rows, E, N, K, stream)
              : launch_grouped<false>(A, B, C, tile_expert, num_vm, max_rows, E, N, K, stream);
}

// Grouped wgrad: dW[e] (+)= dY_e^T X_e with dY [max_rows, N], X [max_rows, K] in the padded layout
// (padding rows zero) and dW stacked [E, N, K] (fp32 when out_fp32). N % 128 == 0, K % 8 == 0.
int b200_gemm_grouped_wgrad(const void* dY, const void* X, void* dW, const int* prow0, int max_rows, int E, int N,
                            int K, int out_fp32, int accumulate, cudaStream_t stream) {
  using namespace b200;
  if (E <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 128) || (K & 7)) return -100;
  constexpr int BN = 128;
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, dY, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, max_rows, N, (long long)N * 2, 64, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, max_rows, K, (long long)K * 2, 64, 64);
  if (rc) return rc;
  const int M = E * N;
  GroupedWgradEpi epi{StoreEpi{dW, nullptr, K, M, K, out_fp32, accumulate}, prow0, N};
  auto kern = gemm_tcgen05_kernel<BN, true, true, GroupedWgradEpi>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set = true;
  }
  const long long tiles = static_cast<long long>(M / kBM) * ((K + BN - 1) / BN);
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  int* status = device_status_word();
  if (!status) return -3;
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(tmA, tmB, M, K, max_rows, epi, status);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// Launches the split-K GEMM proper: fp32 partial tiles into `workspace`. Returns the number of slices
// through *S_out and the slice stride (elements) through *stride_out.
static int launch_splitk_partials(const void* A, const void* B, float* workspace, int M, int N, int K, long long lda,
                                  long long ldb, int splits, int* S_out, long long* stride_out, cudaStream_t stream) {
  using namespace b200;
  constexpr int BN = 128;
  using Cfg = GemmCfg<BN>;
  const int tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + BN - 1) / BN;
  const int kblocks = (K + kBK - 1) / kBK;
  const int kper = (kblocks + splits - 1) / splits;
  const int S = (kblocks + kper - 1) / kper;  // slices that actually hold work
  const int Mv = S * tiles_m * kBM;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda * 2, kBM, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb * 2, BN, 64);
  if (rc) return rc;
  SplitKEpi epi{StoreEpi{workspace, nullptr, N, Mv, N, 1, 0}, tiles_m, kper, kblocks};
  auto kern = gemm_tcgen05_kernel<BN, false, false, SplitKEpi>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set = true;
  }
  const long long tiles = static_cast<long long>(S) * tiles_m * tiles_n;
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  int* status = device_status_word();
  if (!status) return -3;
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(tmA, tmB, Mv, N, K, epi, status);
  B200_CHECK(cudaGetLastError());
  *S_out = S;
  *stride_out = static_cast<long long>(tiles_m) * kBM * N;
  return 0;
}

// C[M,N] (bf16) = A[M,K] . B[N,K]^T (+ bias) with the K extent split over `splits` CTAs per tile.
// workspace: fp32 [splits * ceil(M/128)*128 * N]. N % 4 == 0, ldc % 4 == 0.
int b200_gemm_bf16_splitk(const void* A, const void* B, void* C, const void* bias, float* workspace, int M, int N,
                          int K, long long lda, long long ldb, long long ldc, int splits, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (N & 3) || (ldc & 3) || splits < 1) return -100;
  int S = 0;
  long long stride = 0;
  const int rc = launch_splitk_partials(A, B, workspace, M, N, K, lda, ldb, splits, &S, &stride, stream);
  if (rc) return rc;
  const long long total = static_cast<long long>(M) * (N >> 2);
  long long rg = (total + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 8;
  if (rg > maxg) rg = maxg;
  splitk_reduce_kernel<<<(unsigned)rg, 256, 0, stream>>>(workspace, (const __nv_bfloat16*)bias, (__nv_bfloat16*)C, ldc,
                                                        M, N, S, stride);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// Split-K projection followed, in the reduction kernel, by the residual add and RMSNorm:
//   h = bf16(A . B^T + bias) + residual;  res_out = bf16(h);  y = rmsnorm(res_out) * norm_w
// residual may be null (then res_out = bf16(A . B^T + bias)). y and res_out are contiguous [M, N] bf16;
// N % 8 == 0 and N <= 8192. Two launches instead of three (GEMM, reduce, norm).
int b200_gemm_bf16_splitk_rmsnorm(const void* A, const void* B, const void* bias, float* workspace, int M, int N, int K,
                                  long long lda, long long ldb, int splits, const void* residual, const void* norm_w,
                                  void* y, void* res_out, float eps, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (N & 7) || N > 8192 || splits < 1) return -100;
  int S = 0;
  long long stride = 0;
  const int rc = launch_splitk_partials(A, B, workspace, M, N, K, lda, ldb, splits, &S, &stride, stream);
  if (rc) return rc;
  const int nv = (N / 8 + 31) / 32;
  const int wpb = 8;
  const unsigned grid = static_cast<unsigned>((M + wpb - 1) / wpb);
#define B200_LAUNCH_RN(NV_)                                                                                  \
  splitk_reduce_rmsnorm_kernel<NV_><<<grid, wpb * 32, 0, stream>>>(                                          \
      workspace, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)norm_w,   \
      (__nv_bfloat16*)y, (__nv_bfloat16*)res_out, M, N, S, stride, eps)
  if (nv <= 1) B200_LAUNCH_RN(1);
  else if (nv <= 2) B200_LAUNCH_RN(2);
  else if (nv <= 4) B200_LAUNCH_RN(4);
  else if (nv <= 8) B200_LAUNCH_RN(8);
  else if (nv <= 16) B200_LAUNCH_RN(16);
  else B200_LAUNCH_RN(32);
#undef B200_LAUNCH_RN
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
