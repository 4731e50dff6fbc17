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
  // Destination of (row, col) and how many columns from col on share it.
  __device__ __forceinline__ __nv_bfloat16* dest(int row, int col, int& run) const {
    if (mode == 0) {
      const int d = row / rows_per_rank;
      run = N - col;
      return reinterpret_cast<__nv_bfloat16*>(dst.p[d]) +
             (static_cast<long long>(rank) * rows_per_rank + (row - d * rows_per_rank)) * N + col;
    }
    const int d = col / cols_per_rank;
    run = (d + 1) * cols_per_rank - col;
    return reinterpret_cast<__nv_bfloat16*>(dst.p[d]) + (static_cast<long long>(rank) * M + row) * cols_per_rank +
           (col - d * cols_per_rank);
  }

  // A thread owns one accumulator ROW, so storing straight from registers would emit 32 scattered
  // 16-byte writes per instruction — poison for NVLink (and poor for HBM). Each epilogue warp
  // therefore parks two 32-column chunks (its 32 rows x 128 bytes) in shared memory and writes them
  // out row-wise: 8 lanes cover the 128 contiguous bytes of a row, 4 rows per store instruction.
  __device__ __forceinline__ void chunk(State&, int row, int col0, const float (&v)[32]) const {
    __shared__ uint4 s_stage[4][32][8];  // [epilogue warp][row][16-byte piece], pieces XOR-swizzled by row
    const int lane = threadIdx.x & 31, wq = (threadIdx.x >> 5) & 3;
    const int pair = (col0 >> 5) & 1;  // first or second half of the 64-column group
    const int group0 = col0 - pair * 32;
    const bool fast = (group0 + 64 <= N) && ((N & 7) == 0) && (mode == 0 || (cols_per_rank % 64) == 0);
    if (!fast) {  // ragged edge: element-wise, destination per element
      if (row < M)
        for (int i = 0; i < 32 && col0 + i < N; ++i) {
          int run;
          *dest(row, col0 + i, run) = __float2bfloat16(v[i]);
        }
      return;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 pk;
      __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
      for (int j = 0; j < 4; ++j) pb[j] = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
      s_stage[wq][lane][(pair * 4 + i) ^ (lane & 7)] = pk;
    }
    if (pair == 0) return;
    __syncwarp();
    const int row_base = row - lane;  // first row of this warp's 32
    const int piece = lane & 7;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = it * 4 + (lane >> 3);
      if (row_base + r < M) {
        int run;
        __nv_bfloat16* out = dest(row_base + r, group0 + piece * 8, run);
        *reinterpret_cast<uint4*>(out) = s_stage[wq][r][piece ^ (r & 7)];
      }
    }
    __syncwarp();
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


// Barrier-free, single-kernel GEMM → reduce-scatter.
//
// Tiles whose rows belong to a PEER are computed first and stored (coalesced, see PeerScatterEpi) into
// that peer's staging buffer; each epilogue warp then adds 1 to the peer's counter of that
// (row block, column block) with release semantics at system scope. Tiles whose rows this rank OWNS
// come last: their epilogue waits (bounded) until the counter shows that every peer's partial tile
// has landed, adds the staged partials (and an optional residual) to its own accumulator and writes
// the final bf16 result. No barrier, no separate reduction pass: the transfers of the first phase
// overlap the math, and the staging buffer is double-buffered — a rank can only start call i after
// its call i-1 kernel has consumed every peer's call-(i-1) tiles, which those peers emit after
// finishing their own call i-2 kernel (stream order), so the half written by call i is not being
// read anywhere.
struct GemmReduceScatterEpi {
  PeerScatterEpi base;                 // mode 0: destinations and coalesced peer stores
  PeerPtrs counters;                   // per rank: uint32 [row blocks of rows_per_rank][tiles_n]
  const __nv_bfloat16* local_stage;    // this rank's staging half: [world][rows_per_rank][N]
  const uint32_t* local_counters;
  const __nv_bfloat16* add;            // optional [rows_per_rank, N]
  __nv_bfloat16* out;                  // [rows_per_rank, N]
  uint32_t* expected;                  // local, [entries][4]: arrivals each epilogue warp has already consumed
                                       // (kept on the device so calls of different shapes can share the counters)
  int tiles_n, tiles_per_rank;
  int* status;
  struct State { int own; int ok; };

  __device__ __forceinline__ bool tile(int cta, int ncta, int it, int tiles_m, int tiles_n_, int& m_blk,
                                       int& n_blk) const {
    int mm;
    if (!default_tile(cta, ncta, it, tiles_m, tiles_n_, mm, n_blk)) return false;
    // ring order: owner rank+1 first, ..., this rank's own rows last
    const int owner = (base.rank + 1 + mm / tiles_per_rank) % base.world;
    m_blk = owner * tiles_per_rank + mm % tiles_per_rank;
    return true;
  }
  __device__ __forceinline__ bool gate(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ void begin(State& st, int m_blk, int n_blk, int) const {
    st.own = (m_blk / tiles_per_rank) == base.rank;
    st.ok = 1;
    if (!st.own) return;
    int ok = 1;
    if ((threadIdx.x & 31) == 0) {
      const int entry = (m_blk % tiles_per_rank) * tiles_n + n_blk;
      const uint32_t* c = local_counters + entry;
      uint32_t* exp = expected + entry * 4 + ((threadIdx.x >> 5) & 3);
      const uint32_t target = *exp + static_cast<uint32_t>(base.world - 1) * 4u;  // 4 warps per peer tile
      *exp = target;
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
    }
    st.ok = __shfl_sync(0xffffffffu, ok, 0);
  }
  __device__ __forceinline__ void chunk(State& st, int row, int col0, const float (&v_in)[32]) const {
    if (!st.own) {
      PeerScatterEpi::State s;
      base.chunk(s, row, col0, v_in);
      return;
    }
    if (row >= base.M || col0 >= base.N || !st.ok) return;
    const int lr = row - base.rank * base.rows_per_rank;
    const long long off = static_cast<long long>(lr) * base.N + col0;
    const long long slice = static_cast<long long>(base.rows_per_rank) * base.N;
    const bool full = (col0 + 32 <= base.N) && ((base.N & 7) == 0);
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = v_in[i];
    if (full) {
      for (int s = 0; s < base.world; ++s) {
        if (s == base.rank) continue;
        const uint4* p = reinterpret_cast<const uint4*>(local_stage + s * slice + off);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 raw = p[i];
          const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(pb[j]);
            v[8 * i + 2 * j] += f.x;
            v[8 * i + 2 * j + 1] += f.y;
          }
        }
      }
      if (add) {
        const uint4* p = reinterpret_cast<const uint4*>(add + off);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 raw = p[i];
          const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(pb[j]);
            v[8 * i + 2 * j] += f.x;
            v[8 * i + 2 * j + 1] += f.y;
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 pk;
        __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int j = 0; j < 4; ++j) pb[j] = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
        reinterpret_cast<uint4*>(out + off)[i] = pk;
      }
    } else {
      for (int i = 0; i < 32 && col0 + i < base.N; ++i) {
        float x = v[i];
        for (int s = 0; s < base.world; ++s)
          if (s != base.rank) x += __bfloat162float(local_stage[s * slice + off + i]);
        if (add) x += __bfloat162float(add[off + i]);
        out[off + i] = __float2bfloat16(x);
      }
    }
  }
  __device__ __forceinline__ void end(State& st, int m_blk, int n_blk, int) const {
    if (st.own) return;
    __syncwarp();
    if ((threadIdx.x & 31) == 0 && m_blk * kBM < base.M) {
      const int d = m_blk / tiles_per_rank;
      uint32_t* cnt = reinterpret_cast<uint32_t*>(counters.p[d]) + (m_blk % tiles_per_rank) * tiles_n + n_blk;
      __threadfence_system();
      asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
    }
  }
};

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

// all-to-all → GEMM: the reduction dimension is split by source rank. Operand A lives in the local
// gather buffer as `world` chunks [rows, 64 * kb_per_chunk] (chunk s pushed by rank s, this rank's own
// chunk copied locally); K blocks are visited own chunk first, then the peers in ring order, and the
// producer waits (bounded) for a chunk's flag before its first block is loaded.
struct KChunkGatedEpi {
  __nv_bfloat16* C;
  long long ldc;
  int M, N;
  const uint32_t* flags;  // local, [world]
  uint32_t epoch;
  int rank, world;
  int kb_per_chunk;
  int rows;  // rows of one chunk in the gather buffer
  struct State {};
  __device__ __forceinline__ bool tile(int cta, int ncta, int it, int tiles_m, int tiles_n, int& m_blk,
                                       int& n_blk) const {
    return default_tile(cta, ncta, it, tiles_m, tiles_n, m_blk, n_blk);
  }
  __device__ __forceinline__ bool gate(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ bool k_load(int m_blk, int kb, int& ax, int& ay, int& bx, volatile int* abort_flag,
                                         int* status) const {
    const int total = kb_per_chunk * world;
    int kbp = kb + rank * kb_per_chunk;
    if (kbp >= total) kbp -= total;
    const int src = kbp / kb_per_chunk;
    const int kk = kbp - src * kb_per_chunk;
    if (src != rank && kk == 0) {
      const uint32_t* f = flags + src;
      if (static_cast<int32_t>(ld_acquire_sys_u32(f) - epoch) < 0) {
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
      }
      asm volatile("fence.proxy.async;" ::: "memory");  // TMA reads of the chunk come after the acquire
    }
    ax = kk * kBK;
    ay = src * rows + m_blk * kBM;
    bx = kbp * kBK;
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

// All-to-all push: row block d (rows [d * rows, (d+1) * rows) of src [world * rows, row16 * 16 bytes]) goes
// to rank d's gather buffer at chunk slot `rank`; flag[rank] on rank d is raised as soon as ITS block has
// landed (one completion counter per destination). Destinations are served in the order in which their
// GEMMs will ask for this rank's chunk: d = rank-1 first (its K loop visits rank-1, rank, ...: this
// rank's chunk right after its own), then rank-2, and so on.
__global__ void push_a2a_kernel(PeerPtrs bufs, PeerPtrs flags, int world, int rank, const uint4* __restrict__ src,
                                long long block16, uint32_t epoch, unsigned int* done_counters) {
  for (int step = 1; step < world; ++step) {
    const int d = (rank - step + world) % world;
    const uint4* s = src + static_cast<long long>(d) * block16;
    uint4* dst = reinterpret_cast<uint4*>(bufs.p[d]) + static_cast<long long>(rank) * block16;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < block16;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
      dst[i] = s[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int prev = atomicAdd(done_counters + d, 1u);
      if (prev == gridDim.x - 1) {
        done_counters[d] = 0;
        __threadfence_system();
        st_release_sys_u32(reinterpret_cast<uint32_t*>(flags.p[d]) + rank, epoch);
      }
    }
  }
}

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
                        const Epi& epi, cudaStream_t stream, int a_rows = -1, int a_cols = -1) {
  constexpr int BN = 256;
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  // a_rows / a_cols: shape of operand A in memory when it differs from the logical [M, K] (K-chunked A)
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_rows < 0 ? M : a_rows,
                        a_cols < 0 ? K : a_cols, lda * 2, kBM, 64);
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

// All-to-all push for b200_gemm_kchunk_gated: src [world * rows, cols] bf16 row-major (block_bytes =
// rows * cols * 2 per destination, a multiple of 16). done_counters: `world` zero-initialised uint32.
int b200_push_a2a(void* const* peer_bufs, void* const* peer_flags, int world, int rank, const void* src,
                  long long block_bytes, unsigned epoch, void* done_counters, cudaStream_t stream) {
  using namespace b200;
  if (world < 1 || world > kMaxPeers) return -100;
  if (block_bytes & 15) return -101;
  if (world == 1) return 0;
  PeerPtrs b, f;
  for (int i = 0; i < world; ++i) { b.p[i] = peer_bufs[i]; f.p[i] = peer_flags[i]; }
  long long g = (block_bytes / 16 + 255) / 256;
  if (g > 64) g = 64;
  if (g < 1) g = 1;
  push_a2a_kernel<<<(unsigned)g, 256, 0, stream>>>(b, f, world, rank, (const uint4*)src, block_bytes / 16, epoch,
                                                   reinterpret_cast<unsigned int*>(done_counters));
  B200_CHECK(cudaGetLastError());
  return 0;
}

// C[M,N] = sum_s A_s[M,Kc] * B[:, s*Kc:(s+1)*Kc]^T where A_s is chunk s of the local gather buffer
// ([world, M, Kc] bf16, filled by b200_push_a2a and a local copy of this rank's own chunk).
// Kc must be a multiple of 64; flags: local uint32 [world].
int b200_gemm_kchunk_gated(const void* A, const void* B, void* C, const void* flags, unsigned epoch, int world,
                           int rank, int M, int N, int Kc, long long ldb, long long ldc, cudaStream_t stream) {
  using namespace b200;
  if (world < 1 || world > kMaxPeers) return -100;
  if (Kc % kBK) return -101;
  KChunkGatedEpi epi{reinterpret_cast<__nv_bfloat16*>(C), ldc, M, N, reinterpret_cast<const uint32_t*>(flags),
                     epoch, rank, world, Kc / kBK, M};
  return launch_fused(A, B, M, N, Kc * world, Kc, ldb, epi, stream, world * M, Kc);
}

// Single-kernel GEMM → reduce-scatter: out[M/world, N] = rows of sum_ranks(A_r B_r^T) owned by this rank
// (+ add). peer_stage[d] / peer_counters[d]: rank d's staging half ([world][M/world][N] bf16) and counter
// array (uint32 [M/world/128][ceil(N/256)]) of the half in use; local_* are this rank's own; `expected`
// is a zero-initialised local uint32 array with 4 entries per counter that the kernel maintains itself.
// M must be a multiple of world * 128.
int b200_gemm_rs_fused(const void* A, const void* B, void* const* peer_stage, void* const* peer_counters,
                       const void* local_stage, const void* local_counters, void* expected, const void* add,
                       void* out, int world, int rank, int M, int N, int K, long long lda, long long ldb,
                       cudaStream_t stream) {
  using namespace b200;
  if (world < 1 || world > kMaxPeers) return -100;
  if (M % (world * kBM)) return -101;
  int* status = device_status_word();
  if (!status) return -3;
  GemmReduceScatterEpi epi;
  for (int i = 0; i < world; ++i) { epi.base.dst.p[i] = peer_stage[i]; epi.counters.p[i] = peer_counters[i]; }
  epi.base.M = M; epi.base.N = N; epi.base.mode = 0; epi.base.rank = rank; epi.base.world = world;
  epi.base.rows_per_rank = M / world;
  epi.base.cols_per_rank = N / world;
  epi.local_stage = reinterpret_cast<const __nv_bfloat16*>(local_stage);
  epi.local_counters = reinterpret_cast<const uint32_t*>(local_counters);
  epi.add = reinterpret_cast<const __nv_bfloat16*>(add);
  epi.out = reinterpret_cast<__nv_bfloat16*>(out);
  epi.expected = reinterpret_cast<uint32_t*>(expected);
  epi.tiles_n = (N + 255) / 256;
  epi.tiles_per_rank = M / world / kBM;
  epi.status = status;
  return launch_fused(A, B, M, N, K, lda, ldb, epi, stream);
}

}  // extern "C"
