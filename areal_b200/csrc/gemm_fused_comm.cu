// Fused compute + collective GEMMs over NVLink peer memory (tcgen05 main loop,
// peer loads/stores in the same kernel; no NCCL, no TMA multicast).
//
// 1. b200_gemm_peer_scatter — GEMM whose epilogue stores each output tile
//    straight into a peer's buffer while later tiles are still being computed:
//      mode 0  GEMM → reduce-scatter (row-parallel linear, K sharded):
//              tile rows owned by rank d = row / rows_per_rank land in
//              stage[d][src = my_rank][row % rows_per_rank][col]; the owner sums
//              the `world` slices with b200_reduce_slices after a flag barrier.
//      mode 1  GEMM → all-to-all (Ulysses QKV projection): output columns are
//              heads; columns of rank d = col / cols_per_rank land in
//              out[d][my_rank * M + row][col % cols_per_rank], i.e. the head
//              slice of every rank's sequence shard is gathered on its owner.
// 2. b200_gemm_gated — all-gather → GEMM / all-to-all → GEMM: operand A is a
//    local buffer that peers fill chunk by chunk (b200_push_chunks raises one
//    flag per source rank when its rows have landed). The TMA producer waits
//    (bounded) on the flag of the rank that owns a tile's rows and visits the
//    local rows first, so transfers overlap the tiles already computable.
//
// These replace the DTensor / NCCL redistributions around Colwise / Rowwise
// linears and the Ulysses all_to_all_single calls of the reference
// (areal/engine/fsdp_utils/parallel.py:219-367, areal/models/fsdp/ulysses.py:153-204).
#include "common/gemm_core.cuh"
#include "common/host_utils.h"

namespace b200 {

constexpr int kMaxPeers = 16;
struct PeerPtrs {
  void* p[kMaxPeers];
};

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

struct PeerScatterEpi {
  PeerPtrs dst;
  int M, N;
  int mode;           // 0 = reduce-scatter staging, 1 = all-to-all (column scatter)
  int rank, world;
  int rows_per_rank;  // mode 0
  int cols_per_rank;  // mode 1
  struct State {};
  __device__ __forceinline__ bool tile(int cta, int ncta, int it, int tiles_m, int tiles_n,
                                       int& m_blk, int& n_blk) const {
    // start every rank on a different destination so the peers' links fill evenly
    if (!default_tile(cta, ncta, it, tiles_m, tiles_n, m_blk, n_blk)) return false;
    if (mode == 0) m_blk = (m_blk + rank * (tiles_m / max(world, 1))) % tiles_m;
    else n_blk = (n_blk + rank * (tiles_n / max(world, 1))) % tiles_n;
    return true;
  }
  __device__ __forceinline__ bool gate(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ void begin(State&, int, int, int) const {}
  __device__ __forceinline__ void end(State&, int, int, int) const {}
  __device__ __forceinline__ void chunk(State&, int row, int col0, const float (&v)[32]) const {
    if (row >= M || col0 >= N) return;
    __nv_bfloat16* base;
    long long off;
    int limit;  // columns of this chunk that belong to the same destination
    if (mode == 0) {
      const int d = row / rows_per_rank;
      base = reinterpret_cast<__nv_bfloat16*>(dst.p[d]);
      off = (static_cast<long long>(rank) * rows_per_rank + (row - d * rows_per_rank)) * N + col0;
      limit = min(32, N - col0);
    } else {
      const int d = col0 / cols_per_rank;
      base = reinterpret_cast<__nv_bfloat16*>(dst.p[d]);
      off = (static_cast<long long>(rank) * M + row) * cols_per_rank + (col0 - d * cols_per_rank);
      limit = min(min(32, N - col0), (d + 1) * cols_per_rank - col0);
    }
    __nv_bfloat16* out = base + off;
    if (limit == 32 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 pk;
        __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int j = 0; j < 4; ++j) pb[j] = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
        reinterpret_cast<uint4*>(out)[i] = pk;
      }
    } else {
      // ragged edge (or a chunk straddling two destinations in mode 1): element-wise
      for (int i = 0; i < 32 && col0 + i < N; ++i) {
        if (mode == 1) {
          const int c = col0 + i, d = c / cols_per_rank;
          reinterpret_cast<__nv_bfloat16*>(dst.p[d])[(static_cast<long long>(rank) * M + row) * cols_per_rank +
                                                     (c - d * cols_per_rank)] = __float2bfloat16(v[i]);
        } else {
          out[i] = __float2bfloat16(v[i]);
        }
      }
    }
  }
};

// out[r][c] = sum_s stage[s][r][c] (+ add[r][c]); stage is this rank's local staging buffer.
__global__ void reduce_slices_kernel(const __nv_bfloat16* __restrict__ stage,
                                     const __nv_bfloat16* __restrict__ add, __nv_bfloat16* __restrict__ out,
                                     int world, long long n) {
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < world; ++s) {
      const uint4 raw = *reinterpret_cast<const uint4*>(stage + static_cast<long long>(s) * n + i);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(pb[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    if (add) {
      const uint4 raw = *reinterpret_cast<const uint4*>(add + i);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(pb[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 pk;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
    for (int j = 0; j < 4; ++j) po[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(out + i) = pk;
  }
}


// Barrier-free GEMM → reduce-scatter. Like PeerScatterEpi mode 0, plus: every epilogue warp that has
// stored its 32 rows of a tile adds 1 to the counter of that row block on the OWNER (release at
// system scope), so the owner's reduction waits per row block instead of behind a whole-group
// barrier, and no barrier precedes the GEMM either: the staging buffer is double-buffered, and a
// rank can only start call i after its reduction of call i-1 has seen every peer's call-(i-1) tiles,
// which those peers emit after finishing their own reduction of call i-2 (stream order) — so the
// half written by call i is no longer being read anywhere.
struct PeerScatterFlagEpi {
  PeerScatterEpi base;
  PeerPtrs counters;  // per rank: uint32 [tiles of rows_per_rank]
  struct State {};
  __device__ __forceinline__ bool tile(int cta, int ncta, int it, int tiles_m, int tiles_n, int& m_blk,
                                       int& n_blk) const {
    return base.tile(cta, ncta, it, tiles_m, tiles_n, m_blk, n_blk);
  }
  __device__ __forceinline__ bool gate(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ void begin(State&, int, int, int) const {}
  __device__ __forceinline__ void chunk(State&, int row, int col0, const float (&v)[32]) const {
    PeerScatterEpi::State s;
    base.chunk(s, row, col0, v);
  }
  __device__ __forceinline__ void end(State&, int m_blk, int, int) const {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) {
      const int row0 = m_blk * kBM;
      if (row0 < base.M) {
        const int d = row0 / base.rows_per_rank;
        uint32_t* cnt = reinterpret_cast<uint32_t*>(counters.p[d]) + (row0 - d * base.rows_per_rank) / kBM;
        __threadfence_system();
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
      }
    }
  }
};

// One block per (local row block, column slab): waits (bounded) until the row block's counter
// reaches `target`, then sums the `world` staged slices (+ add) into out.
__global__ void reduce_slices_flag_kernel(const __nv_bfloat16* __restrict__ stage, const __nv_bfloat16* __restrict__ add,
                                          __nv_bfloat16* __restrict__ out, const uint32_t* __restrict__ counters,
                                          uint32_t target, int world, int rows, int N, int col_slabs, int* status) {
  const int tile = blockIdx.x, slab = blockIdx.y;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    const uint32_t* c = counters + tile;
    int ok = 1;
    if (static_cast<int32_t>(ld_acquire_sys_u32(c) - target) < 0) {
      const unsigned long long t0 = globaltimer_ns();
      uint32_t spins = 0;
      while (static_cast<int32_t>(ld_acquire_sys_u32(c) - target) < 0) {
        if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > kWaitDeadlineNs) {
          atomicCAS(status, 0, kErrPeerFlagTimeout);
          ok = 0;
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  const long long slice = static_cast<long long>(rows) * N;
  const int vec_per_row = N / 8;
  const int v0 = static_cast<int>(static_cast<long long>(vec_per_row) * slab / col_slabs);
  const int v1 = static_cast<int>(static_cast<long long>(vec_per_row) * (slab + 1) / col_slabs);
  const int r0 = tile * kBM, r1 = min(rows, r0 + kBM);
  const int width = v1 - v0;
  for (int i = threadIdx.x; i < (r1 - r0) * width; i += blockDim.x) {
    const long long e = (static_cast<long long>(r0 + i / width) * vec_per_row + v0 + i % width) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < world; ++s) {
      const uint4 raw = *reinterpret_cast<const uint4*>(stage + s * slice + e);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(pb[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    if (add) {
      const uint4 raw = *reinterpret_cast<const uint4*>(add + e);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(pb[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 pk;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
    for (int j = 0; j < 4; ++j) po[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(out + e) = pk;
  }
}

// ---------------------------------------------------------------- gated GEMM --
struct GatedStoreEpi {
  __nv_bfloat16* C;
  long long ldc;
  int M, N;
  const uint32_t* flags;  // local, [world]: flag[s] >= epoch once rank s's rows have landed
  uint32_t epoch;
  int rank, world;
  int tiles_per_rank;  // M-tiles per source rank
  struct State {};
  __device__ __forceinline__ bool tile(int cta, int ncta, int it, int tiles_m, int tiles_n,
                                       int& m_blk, int& n_blk) const {
    // rotate the row blocks so that this rank's own rows (already local) come first,
    // then the peers in ring order
    long long t = static_cast<long long>(it) * ncta + cta;
    const long long total = static_cast<long long>(tiles_m) * tiles_n;
    if (t >= total) return false;
    const int mm = static_cast<int>(t / tiles_n);
    n_blk = static_cast<int>(t % tiles_n);
    m_blk = (mm + rank * tiles_per_rank) % tiles_m;
    return true;
  }
  __device__ __forceinline__ bool gate(int m_blk, int, volatile int* abort_flag, int* status) const {
    const int src = min(m_blk / tiles_per_rank, world - 1);
    if (src == rank) return true;
    const uint32_t* f = flags + src;
    if (static_cast<int32_t>(ld_acquire_sys_u32(f) - epoch) >= 0) {
      asm volatile("fence.proxy.async;" ::: "memory");
      return true;
    }
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys_u32(f) - epoch) < 0) {
      if ((++spins & 0xff) == 0) {
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > kWaitDeadlineNs) {
          atomicCAS(status, 0, kErrPeerFlagTimeout);
          return false;
        }
      }
    }
    // order the TMA (async proxy) reads of the tile after the acquire
    asm volatile("fence.proxy.async;" ::: "memory");
    return true;
  }
  __device__ __forceinline__ void begin(State&, int, int, int) const {}
  __device__ __forceinline__ void end(State&, int, int, int) const {}
  __device__ __forceinline__ void chunk(State&, int row, int col0, const float (&v)[32]) const {
    if (row >= M || col0 >= N) return;
    __nv_bfloat16* out = C + static_cast<long long>(row) * ldc + col0;
    if (col0 + 32 <= N && (ldc & 7) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 pk;
        __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int j = 0; j < 4; ++j) pb[j] = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
        reinterpret_cast<uint4*>(out)[i] = pk;
      }
    } else {
      for (int i = 0; i < 32 && col0 + i < N; ++i) out[i] = __float2bfloat16(v[i]);
    }
  }
};

// Copies this rank's rows into every peer's gather buffer (at row offset rank * rows) and
// then raises flag[rank] = epoch on every peer. One launch; the last block to finish signals.
__global__ void push_chunks_kernel(PeerPtrs bufs, PeerPtrs flags, int world, int rank,
                                   const uint4* __restrict__ src, long long n16, long long dst_off16,
                                   uint32_t epoch, unsigned int* done_counter) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = src[i];
    for (int p = 0; p < world; ++p)
      if (p != rank) reinterpret_cast<uint4*>(bufs.p[p])[dst_off16 + i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;
      __threadfence_system();
      for (int p = 0; p < world; ++p)
        if (p != rank) st_release_sys_u32(reinterpret_cast<uint32_t*>(flags.p[p]) + rank, epoch);
    }
  }
}

template <class Epi>
static int launch_fused(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                        const Epi& epi, cudaStream_t stream) {
  constexpr int BN = 256;
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda * 2, kBM, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb * 2, BN, 64);
  if (rc) return rc;
  auto kern = gemm_tcgen05_kernel<BN, false, false, Epi>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set = true;
  }
  const long long tiles = static_cast<long long>((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  if (grid <= 0) return 0;
  int* status = device_status_word();
  if (!status) return -3;
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(tmA, tmB, M, N, K, epi, status);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace b200

extern "C" {

// C_partial = A[M,K] * B[N,K]^T (both K-major) scattered to peers, see the file header.
// mode 0 needs M % world == 0; mode 1 needs N % world == 0.
int b200_gemm_peer_scatter(const void* A, const void* B, void* const* peer_dst, int world, int rank,
                           int M, int N, int K, long long lda, long long ldb, int mode,
                           cudaStream_t stream) {
  using namespace b200;
  if (world < 1 || world > kMaxPeers) return -100;
  if ((mode == 0 && M % world) || (mode == 1 && N % world)) return -101;
  PeerScatterEpi epi;
  for (int i = 0; i < world; ++i) epi.dst.p[i] = peer_dst[i];
  epi.M = M; epi.N = N; epi.mode = mode; epi.rank = rank; epi.world = world;
  epi.rows_per_rank = M / world;
  epi.cols_per_rank = N / world;
  return launch_fused(A, B, M, N, K, lda, ldb, epi, stream);
}

// out = sum of `world` slices of n elements each (n % 8 == 0), plus optional `add`.
int b200_reduce_slices(const void* stage, const void* add, void* out, int world, long long n,
                       cudaStream_t stream) {
  using namespace b200;
  if (n == 0) return 0;
  if (n & 7) return -101;
  long long g = (n / 8 + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 8;
  if (g > maxg) g = maxg;
  reduce_slices_kernel<<<(unsigned)g, 256, 0, stream>>>((const __nv_bfloat16*)stage, (const __nv_bfloat16*)add,
                                                        (__nv_bfloat16*)out, world, n);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// Pushes `bytes` of src into every other rank's gather buffer at dst_off_bytes and raises the
// per-source flag with `epoch`. done_counter: a zero-initialised device uint32 owned by the caller.
int b200_push_chunks(void* const* peer_bufs, void* const* peer_flags, int world, int rank, const void* src,
                     long long bytes, long long dst_off_bytes, unsigned epoch, void* done_counter,
                     cudaStream_t stream) {
  using namespace b200;
  if (world < 1 || world > kMaxPeers) return -100;
  if ((bytes & 15) || (dst_off_bytes & 15)) return -101;
  PeerPtrs b, f;
  for (int i = 0; i < world; ++i) { b.p[i] = peer_bufs[i]; f.p[i] = peer_flags[i]; }
  long long g = (bytes / 16 + 255) / 256;
  if (g > 64) g = 64;  // a few dozen CTAs saturate NVLink and leave the SMs to the GEMM
  if (g < 1) g = 1;
  push_chunks_kernel<<<(unsigned)g, 256, 0, stream>>>(b, f, world, rank, (const uint4*)src, bytes / 16,
                                                      dst_off_bytes / 16, epoch,
                                                      reinterpret_cast<unsigned int*>(done_counter));
  B200_CHECK(cudaGetLastError());
  return 0;
}

// C[M,N] = A[M,K] * B[N,K]^T where A is the local gather buffer filled by b200_push_chunks.
// flags: local uint32 [world]; M must be a multiple of world * 128.
int b200_gemm_gated(const void* A, const void* B, void* C, const void* flags, unsigned epoch, int world,
                    int rank, int M, int N, int K, long long lda, long long ldb, long long ldc,
                    cudaStream_t stream) {
  using namespace b200;
  if (world < 1 || world > kMaxPeers) return -100;
  if (M % (world * kBM)) return -101;
  GatedStoreEpi epi{reinterpret_cast<__nv_bfloat16*>(C), ldc, M, N, reinterpret_cast<const uint32_t*>(flags),
                    epoch, rank, world, M / world / kBM};
  return launch_fused(A, B, M, N, K, lda, ldb, epi, stream);
}

// Barrier-free GEMM → reduce-scatter, first half: C_partial tiles go to the owners' staging buffers
// (peer_stage[d] = base of the staging half in use) and bump the owners' row-block counters
// (peer_counters[d], uint32 [M / world / 128]). M must be a multiple of world * 128.
int b200_gemm_rs_flagged(const void* A, const void* B, void* const* peer_stage, void* const* peer_counters, int world,
                         int rank, int M, int N, int K, long long lda, long long ldb, cudaStream_t stream) {
  using namespace b200;
  if (world < 1 || world > kMaxPeers) return -100;
  if (M % (world * kBM)) return -101;
  PeerScatterFlagEpi epi;
  for (int i = 0; i < world; ++i) { epi.base.dst.p[i] = peer_stage[i]; epi.counters.p[i] = peer_counters[i]; }
  epi.base.M = M; epi.base.N = N; epi.base.mode = 0; epi.base.rank = rank; epi.base.world = world;
  epi.base.rows_per_rank = M / world;
  epi.base.cols_per_rank = N / world;
  return launch_fused(A, B, M, N, K, lda, ldb, epi, stream);
}

// Second half: out[rows, N] = sum over the `world` staged slices (+ add) once every row block's counter has
// reached `target` (= counter value expected after this call: previous target + world * ceil(N/256) * 4).
int b200_reduce_slices_flagged(const void* stage, const void* add, void* out, const void* counters, unsigned target,
                               int world, int rows, int N, cudaStream_t stream) {
  using namespace b200;
  if (rows == 0) return 0;
  if ((N & 7) || (rows % kBM)) return -101;
  int* status = device_status_word();
  if (!status) return -3;
  const int tiles = rows / kBM;
  int slabs = (2 * sm_count() + tiles - 1) / tiles;
  if (slabs < 1) slabs = 1;
  if (slabs > N / 8) slabs = N / 8;
  dim3 grid(tiles, slabs);
  reduce_slices_flag_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)stage, (const __nv_bfloat16*)add,
                                                      (__nv_bfloat16*)out, (const uint32_t*)counters, target, world,
                                                      rows, N, slabs, status);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
