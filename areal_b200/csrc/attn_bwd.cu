// Varlen packed causal FlashAttention backward for sm_100a (tcgen05 + TMEM).
//
// One CTA owns one (128-row key/value block of one sequence, kv head) pair. It
// keeps K_j and V_j resident in shared memory and dK_j / dV_j as fp32
// accumulators in TMEM (2 x 128 columns) while it walks every query block i on
// or below the causal diagonal, for every query head of the GQA group:
//
//   S^T  = K_j Q_i^T            (tcgen05, TMEM cols 256..383)
//   dP^T = V_j dO_i^T           (tcgen05, TMEM cols 384..511)
//   P^T  = exp2(S^T*c - lse_i)  (registers → bf16 → swizzled smem)
//   dV  += P^T dO_i             (tcgen05; dO_i read MN-major from the same tile)
//   dS^T = P^T ∘ (dP^T - Δ_i) * scale
//   dK  += dS^T Q_i             (tcgen05; Q_i read MN-major)
//   dQ_i = dS K_j               (tcgen05 into the S^T columns; both operands MN-major;
//                                then red.global.add.v4.f32 into an fp32 dQ buffer)
//
// Working on the transposed score tile makes each compute thread own (part of)
// one key row, so P^T and dS^T are written row-per-thread as K-major A operands
// and no tile is ever transposed in memory. The kernel is a template on the number
// of compute warps: with 8, warps w and w+4 read the same 32 TMEM lanes and take
// the lower / upper 64 columns of every 128-column tile.
//
// Replaces flash-attn's backward / aten._flash_attention_backward in the
// reference (areal/experimental/models/archon/attention/varlen.py:116).
#include "common/host_utils.h"
#include "common/ptx.cuh"

namespace b200 {

constexpr int kD = 128;
constexpr int kBT = 128;  // rows of every tile (q and kv)
// NCW compute warps (4 or 8) + TMA producer + MMA issuer
template <int NCW> constexpr int bwd_threads() { return NCW * 32 + 64; }

struct AttnBwdTile {
  int kv_start;   // first global token row of this kv block
  int kv_len;     // valid kv rows in the block (<= 128)
  int kv_off;     // offset of the block inside its sequence
  int seq_start;  // first global token row of the sequence
  int seq_len;    // end of the query range (sequence-relative); queries [max(kv_off, q_begin), seq_len) are visited
  int q_begin;    // first sequence position present in the query array (0 unless context-parallel)
  int pad1, pad2;
};

constexpr int kTileBytes = kBT * kD * 2;  // 32 KB
// K, V resident; (Q, dO) x 2 stages; one buffer shared by P^T and dS^T.
constexpr int kAttnBwdSmem = 2 * kTileBytes + 4 * kTileBytes + kTileBytes;  // 224 KB

// Δ[h, t] = sum_d dO[t,h,d] * O[t,h,d]
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                      const __nv_bfloat16* __restrict__ dout,
                                      float* __restrict__ delta, int T, int Hq) {
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<long long>(T) * Hq) return;
  const int t = static_cast<int>(gw / Hq), h = static_cast<int>(gw % Hq);
  const uint2 a = reinterpret_cast<const uint2*>(o + gw * kD)[lane];
  const uint2 b = reinterpret_cast<const uint2*>(dout + gw * kD)[lane];
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o2 = 16; o2 > 0; o2 >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o2);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = s;
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                   long long n) {
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(in + i);
    uint2 pk;
    reinterpret_cast<__nv_bfloat162*>(&pk)[0] = __floats2bfloat162_rn(v.x, v.y);
    reinterpret_cast<__nv_bfloat162*>(&pk)[1] = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(out + i) = pk;
  }
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// TREE: keys carry a subtree end (`key_exit`) that bounds the queries they are visible to. It is a
// template flag because the 4-warp variant sits at the register limit: the extra compare in the
// innermost loop cost the ordinary causal path a third of its speed when it was a run-time test.
template <int NCW, bool TREE>
__global__ void __launch_bounds__(NCW * 32 + 64, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const AttnBwdTile* __restrict__ tiles, const float* __restrict__ lse,
                const float* __restrict__ delta, float* __restrict__ dq_acc,
                __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, int T, int Hq,
                int Hkv, long long lddk, long long lddv, float scale, int* status,
                const int* __restrict__ key_exit) {
  constexpr int kCompute = NCW * 32;     // compute threads
  constexpr int kChunks = 4 / (NCW / 4);  // 32-column chunks of a 128-column tile per compute warp
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bars[16];
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_word;
  __shared__ float s_lse[2][kBT];
  __shared__ float s_delta[2][kBT];
  volatile int* abort_flag = &abort_word;

  uint8_t* sK = smem;
  uint8_t* sV = smem + kTileBytes;
  uint8_t* sQ = smem + 2 * kTileBytes;   // [2 stages]
  uint8_t* sdO = smem + 4 * kTileBytes;  // [2 stages]
  uint8_t* sPS = smem + 6 * kTileBytes;  // P^T, then dS^T
  uint64_t* kv_full = &bars[0];
  uint64_t* qdo_full = &bars[1];   // [2]
  uint64_t* qdo_empty = &bars[3];  // [2]
  uint64_t* s_full = &bars[5];
  uint64_t* dp_full = &bars[6];
  uint64_t* pt_ready = &bars[7];
  uint64_t* pbuf_free = &bars[8];
  uint64_t* dst_ready = &bars[9];
  uint64_t* dq_full = &bars[10];
  uint64_t* dq_read = &bars[11];
  uint64_t* acc_done = &bars[12];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AttnBwdTile tile = tiles[blockIdx.x];
  const int hk = blockIdx.y;
  const int group = Hq / Hkv;
  // query blocks i with rows >= kv_off (causal): first block index containing kv_off
  // q_begin (0 for ordinary batches): first sequence position held by the local query array
  // (context parallelism: this rank owns the positions [q_begin, seq_len) of the sequence)
  const int qb_first = max(tile.kv_off, tile.q_begin) / kBT;
  const int qb_count = (tile.seq_len + kBT - 1) / kBT - qb_first;
  const int n_iter = qb_count * group;  // iteration it -> (head g = it / qb_count, block i = it % qb_count)
  const float scale_log2 = scale * 1.4426950408889634f;

  if (threadIdx.x == 0) {
    abort_word = (smem_u32(smem) & 1023) ? 1 : 0;
    if (abort_word) atomicCAS(status, 0, kErrBounds);
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(pt_ready, kCompute);
    mbar_init(pbuf_free, 1);
    mbar_init(dst_ready, kCompute);
    mbar_init(dq_full, 1);
    mbar_init(dq_read, kCompute);
    mbar_init(acc_done, 1);
    fence_mbar_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmdO);
  }
  if (warp == NCW + 1) {
    tmem_alloc(&tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  const uint32_t tm_dK = tmem_base;
  const uint32_t tm_dV = tmem_base + 128;
  const uint32_t tm_S = tmem_base + 256;   // S^T, later dQ
  const uint32_t tm_dP = tmem_base + 384;  // dP^T
  const bool bad_align = (abort_word != 0);

  if (bad_align) {
  } else if (warp == NCW) {
    // ------------------------------------------------------ TMA producer --
    if (elect_one_sync()) {
      mbar_arrive_expect_tx(kv_full, 2 * kTileBytes);
      tma_load_2d(sK, &tmK, kv_full, hk * kD, tile.kv_start);
      tma_load_2d(sK + kTileBytes / 2, &tmK, kv_full, hk * kD + 64, tile.kv_start);
      tma_load_2d(sV, &tmV, kv_full, hk * kD, tile.kv_start);
      tma_load_2d(sV + kTileBytes / 2, &tmV, kv_full, hk * kD + 64, tile.kv_start);
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int g = it / qb_count, i = qb_first + it % qb_count;
        const int h = hk * group + g;
        const int row = tile.seq_start + i * kBT;
        if (!mbar_wait(&qdo_empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&qdo_full[st], 2 * kTileBytes);
        tma_load_2d(sQ + st * kTileBytes, &tmQ, &qdo_full[st], h * kD, row);
        tma_load_2d(sQ + st * kTileBytes + kTileBytes / 2, &tmQ, &qdo_full[st], h * kD + 64, row);
        tma_load_2d(sdO + st * kTileBytes, &tmdO, &qdo_full[st], h * kD, row);
        tma_load_2d(sdO + st * kTileBytes + kTileBytes / 2, &tmdO, &qdo_full[st], h * kD + 64, row);
      }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(status, 0, kErrMbarTimeoutProducer);
        unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == NCW + 1) {
    // -------------------------------------------------------- MMA issuer --
    if (elect_one_sync()) {
      // all tiles are [128 rows][2 halves of 64 columns], 128B-swizzled.
      // K-major view of a tile (rows = M/N index, columns = reduction):
      //   half hh, k-step kk: base + hh*16K + kk*32, LBO 16, SBO 1024
      // MN-major view (columns = M/N index, rows = reduction):
      //   k-step k (16 rows): base + k*2048, LBO 16K (next 64 columns), SBO 1024
      constexpr uint32_t id_kk = make_idesc(1, 1, 0, 0, kBT, kBT);  // A K-major, B K-major
      constexpr uint32_t id_kmn = make_idesc(1, 1, 0, 1, kBT, kD);  // A K-major, B MN-major
      constexpr uint32_t id_mnmn = make_idesc(1, 1, 1, 1, kBT, kD); // both MN-major
      constexpr uint32_t HALF = kTileBytes / 2;
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), ps_addr = smem_u32(sPS);
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const uint32_t itp = it & 1;
        const uint32_t q_addr = smem_u32(sQ + st * kTileBytes);
        const uint32_t do_addr = smem_u32(sdO + st * kTileBytes);
        if (!mbar_wait(&qdo_full[st], ph, abort_flag)) { ok = false; break; }
        // the S^T columns hold dQ of the previous iteration until it has been read out
        if (it > 0 && !mbar_wait(dq_read, (it - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {  // S^T = K Q^T
          const uint32_t off = (k >> 2) * HALF + (k & 3) * 32;
          umma_f16(tm_S, make_sdesc_sw128(k_addr + off, 16, 1024),
                   make_sdesc_sw128(q_addr + off, 16, 1024), id_kk, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {  // dP^T = V dO^T
          const uint32_t off = (k >> 2) * HALF + (k & 3) * 32;
          umma_f16(tm_dP, make_sdesc_sw128(v_addr + off, 16, 1024),
                   make_sdesc_sw128(do_addr + off, 16, 1024), id_kk, k > 0 ? 1u : 0u);
        }
        umma_commit(dp_full);
        if (!mbar_wait(pt_ready, itp, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kBT / 16; ++k) {  // dV += P^T dO   (reduction over q rows)
          const uint32_t aoff = (k >> 2) * HALF + (k & 3) * 32;
          umma_f16(tm_dV, make_sdesc_sw128(ps_addr + aoff, 16, 1024),
                   make_sdesc_sw128(do_addr + k * 2048, HALF, 1024), id_kmn,
                   (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(pbuf_free);
        if (!mbar_wait(dst_ready, itp, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kBT / 16; ++k) {  // dK += dS^T Q
          const uint32_t aoff = (k >> 2) * HALF + (k & 3) * 32;
          umma_f16(tm_dK, make_sdesc_sw128(ps_addr + aoff, 16, 1024),
                   make_sdesc_sw128(q_addr + k * 2048, HALF, 1024), id_kmn,
                   (it > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < kBT / 16; ++k) {  // dQ = dS K  (reduction over kv rows)
          umma_f16(tm_S, make_sdesc_sw128(ps_addr + k * 2048, HALF, 1024),
                   make_sdesc_sw128(k_addr + k * 2048, HALF, 1024), id_mnmn, k > 0 ? 1u : 0u);
        }
        umma_commit(&qdo_empty[st]);
        umma_commit(dq_full);
      }
      if (ok) umma_commit(acc_done);
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(status, 0, kErrMbarTimeoutMma);
      }
    }
  } else {
    // ---------------------------------------------------- compute warps --
    const int quad = warp & 3;    // TMEM lane quarter this warp may read
    const int cpart = warp >> 2;  // which part of the columns of every 128-column tile this warp handles
    const int r = quad * 32 + lane;  // kv row inside the block == TMEM lane (q row for dQ)
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int kv_pos = tile.kv_off + r;
    const bool kv_valid = r < tile.kv_len;
    // tree attention: this key is visible to the queries of its own subtree only
    const int kv_exit = (TREE && kv_valid) ? key_exit[tile.kv_start + r] : 0x7fffffff;
    uint8_t* psrow = sPS + r * 128;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const uint32_t itp = it & 1;
      const int g = it / qb_count, i = qb_first + it % qb_count;
      const int h = hk * group + g;
      const int q0 = i * kBT;  // offset of the q block inside the sequence
      const int q_rows = min(kBT, tile.seq_len - q0);
      // stage lse / delta of this q block (log2 units for lse)
      if (cpart == 0) {
        const int qi = q0 + r;
        const long long idx = static_cast<long long>(h) * T + tile.seq_start + qi;
        const bool v = r < q_rows;
        s_lse[itp][r] = v ? lse[idx] * 1.4426950408889634f : INFINITY;
        s_delta[itp][r] = v ? delta[idx] : 0.f;
      }
      named_bar_sync(1, kCompute);
      if (!mbar_wait(s_full, itp, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t p_packed[kChunks * 16];  // this warp's columns
      const bool diag = (q0 < tile.kv_off + kBT);  // block touches the causal diagonal
#pragma unroll
      for (int cl = 0; cl < kChunks; ++cl) {
        const int c = cpart * kChunks + cl;
        uint32_t raw[32];
        tmem_ld_32x32(tm_S + lane_addr + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float p2[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int col = c * 32 + 2 * e + u;  // q row inside block
            float p = exp2f(__uint_as_float(raw[2 * e + u]) * scale_log2 - s_lse[itp][col]);
            bool valid = kv_valid && (col < q_rows) && (!diag || (q0 + col >= kv_pos));
            if (TREE) valid = valid && (q0 + col < kv_exit);
            p2[u] = valid ? p : 0.f;
          }
          __nv_bfloat162 pb = __floats2bfloat162_rn(p2[0], p2[1]);
          p_packed[cl * 16 + e] = *reinterpret_cast<uint32_t*>(&pb);
        }
      }
      // the buffer still holds dS^T of the previous iteration until dK/dQ MMAs finished
      if (it > 0) {
        if (!mbar_wait(dq_full, (it - 1) & 1, abort_flag)) { ok = false; break; }
      }
#pragma unroll
      for (int cp = 0; cp < kChunks * 4; ++cp) {  // 16-byte pieces of this warp's part of the row
        uint4 pk = make_uint4(p_packed[cp * 4], p_packed[cp * 4 + 1], p_packed[cp * 4 + 2],
                              p_packed[cp * 4 + 3]);
        const int c = cpart * kChunks * 4 + cp;
        const int half = c >> 3, cc = c & 7;
        *reinterpret_cast<uint4*>(psrow + half * (kTileBytes / 2) + ((cc ^ (r & 7)) << 4)) = pk;
      }
      fence_proxy_async_smem();
      mbar_arrive(pt_ready);
      // read dQ of the previous iteration out of the S^T columns?  No: S^T of this
      // iteration was only issued after dq_read(it-1), so dQ(it-1) is already drained.
      if (!mbar_wait(dp_full, itp, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t ds_packed[kChunks * 16];
#pragma unroll
      for (int cl = 0; cl < kChunks; ++cl) {
        const int c = cpart * kChunks + cl;
        uint32_t raw[32];
        tmem_ld_32x32(tm_dP + lane_addr + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const __nv_bfloat162 pb = *reinterpret_cast<__nv_bfloat162*>(&p_packed[cl * 16 + e]);
          const float2 p = __bfloat1622float2(pb);
          const int col = c * 32 + 2 * e;
          const float d0 = p.x * (__uint_as_float(raw[2 * e]) - s_delta[itp][col]) * scale;
          const float d1 = p.y * (__uint_as_float(raw[2 * e + 1]) - s_delta[itp][col + 1]) * scale;
          __nv_bfloat162 db = __floats2bfloat162_rn(d0, d1);
          ds_packed[cl * 16 + e] = *reinterpret_cast<uint32_t*>(&db);
        }
      }
      if (!mbar_wait(pbuf_free, itp, abort_flag)) { ok = false; break; }
#pragma unroll
      for (int cp = 0; cp < kChunks * 4; ++cp) {
        uint4 pk = make_uint4(ds_packed[cp * 4], ds_packed[cp * 4 + 1], ds_packed[cp * 4 + 2],
                              ds_packed[cp * 4 + 3]);
        const int c = cpart * kChunks * 4 + cp;
        const int half = c >> 3, cc = c & 7;
        *reinterpret_cast<uint4*>(psrow + half * (kTileBytes / 2) + ((cc ^ (r & 7)) << 4)) = pk;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(dst_ready);
      // dQ_i: lane r is now query row q0 + r
      if (!mbar_wait(dq_full, itp, abort_flag)) { ok = false; break; }
      tc_fence_after();
      {
        const bool qv = r < q_rows;
        float* dq_row = dq_acc + (static_cast<long long>(tile.seq_start + q0 + r) * Hq + h) * kD;
#pragma unroll 1
        for (int cl = 0; cl < kChunks; ++cl) {
          const int c = cpart * kChunks + cl;
          uint32_t raw[32];
          tmem_ld_32x32(tm_S + lane_addr + c * 32, raw);
          tmem_ld_wait();
          if (qv) {
#pragma unroll
            for (int e = 0; e < 8; ++e)
              red_add_v4(dq_row + c * 32 + e * 4, __uint_as_float(raw[4 * e]),
                         __uint_as_float(raw[4 * e + 1]), __uint_as_float(raw[4 * e + 2]),
                         __uint_as_float(raw[4 * e + 3]));
          }
        }
      }
      tc_fence_before();
      mbar_arrive(dq_read);
    }
    // epilogue: dK, dV
    if (ok) ok = mbar_wait(acc_done, 0, abort_flag);
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dk_row = dk + static_cast<long long>(tile.kv_start + r) * lddk + hk * kD;
      __nv_bfloat16* dv_row = dv + static_cast<long long>(tile.kv_start + r) * lddv + hk * kD;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = which ? dv_row : dk_row;
        const uint32_t tm = which ? tm_dV : tm_dK;
#pragma unroll 1
        for (int cl = 0; cl < kChunks; ++cl) {
          const int c = cpart * kChunks + cl;
          uint32_t raw[32];
          if (n_iter > 0) {
            tmem_ld_32x32(tm + lane_addr + c * 32, raw);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) raw[e] = 0;
          }
          if (kv_valid) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              uint4 pk;
              __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
              for (int u = 0; u < 4; ++u)
                pb[u] = __floats2bfloat162_rn(__uint_as_float(raw[e * 8 + 2 * u]),
                                              __uint_as_float(raw[e * 8 + 2 * u + 1]));
              reinterpret_cast<uint4*>(dst + c * 32)[e] = pk;
            }
          }
        }
      }
    } else if (lane == 0) {
      *abort_flag = 1;
      atomicCAS(status, 0, kErrMbarTimeoutEpilogue);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == NCW + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200

extern "C" {

// q, o, dout: [T, Hq*128] contiguous bf16; k, v with pitches ldk/ldv; lse and
// delta_ws are [Hq, T] fp32; dq_acc is a zero-initialised fp32 [T, Hq*128]
// workspace; dq (bf16, pitch lddq) receives its rounded value; dk/dv are bf16
// with pitches lddk/lddv (they may point into a fused dqkv buffer).
int b200_attn_bwd_ex(const void* q, const void* k, const void* v, const void* o, const void* dout,
                     const float* lse, float* delta_ws, float* dq_acc, void* dq, void* dk, void* dv,
                     const void* tiles, int n_tiles, int T, int Tkv, int Hq, int Hkv, long long ldk,
                     long long ldv, long long lddk, long long lddv, float softmax_scale,
                     const int* key_exit, cudaStream_t stream);

int b200_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                  const float* lse, float* delta_ws, float* dq_acc, void* dq, void* dk, void* dv,
                  const void* tiles, int n_tiles, int T, int Hq, int Hkv, long long ldk,
                  long long ldv, long long lddk, long long lddv, float softmax_scale,
                  cudaStream_t stream) {
  return b200_attn_bwd_ex(q, k, v, o, dout, lse, delta_ws, dq_acc, dq, dk, dv, tiles, n_tiles, T, 0, Hq, Hkv, ldk,
                          ldv, lddk, lddv, softmax_scale, nullptr, stream);
}

// Extended form, see b200_attn_fwd_ex: k, v, dk, dv have Tkv rows; key_exit enables the tree mask.
int b200_attn_bwd_ex(const void* q, const void* k, const void* v, const void* o, const void* dout,
                     const float* lse, float* delta_ws, float* dq_acc, void* dq, void* dk, void* dv,
                     const void* tiles, int n_tiles, int T, int Tkv, int Hq, int Hkv, long long ldk,
                     long long ldv, long long lddk, long long lddv, float softmax_scale,
                     const int* key_exit, cudaStream_t stream) {
  using namespace b200;
  if (n_tiles == 0 || T == 0) return 0;
  if (Tkv <= 0) Tkv = T;
  if (Hq % Hkv) return -100;
  {
    const long long warps = static_cast<long long>(T) * Hq;
    attn_bwd_delta_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta_ws, T, Hq);
  }
  CUtensorMap tmQ, tmK, tmV, tmdO;
  int rc = make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)Hq * kD,
                        (uint64_t)Hq * kD * 2, kBT, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tmdO, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)Hq * kD,
                    (uint64_t)Hq * kD * 2, kBT, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tkv, (uint64_t)Hkv * kD, ldk * 2,
                    kBT, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tkv, (uint64_t)Hkv * kD, ldv * 2,
                    kBT, 64);
  if (rc) return rc;
  static bool attr_set = false;
  static int compute_warps = 8;
  if (!attr_set) {
    B200_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kAttnBwdSmem));
    B200_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kAttnBwdSmem));
    B200_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kAttnBwdSmem));
    B200_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kAttnBwdSmem));
    // 8 compute warps by default (measured 472 vs 403 TFLOP/s); AREAL_B200_ATTN_BWD_WARPS=4 selects the
    // variant in which one warp handles all 128 columns of its rows
    const char* e = getenv("AREAL_B200_ATTN_BWD_WARPS");
    if (e && atoi(e) == 4) compute_warps = 4;
    attr_set = true;
  }
  int* status = device_status_word();
  if (!status) return -3;
  dim3 grid(n_tiles, Hkv);
#define B200_ATTN_BWD_LAUNCH(NCW, TREE)                                                                   \
  attn_bwd_kernel<NCW, TREE><<<grid, bwd_threads<NCW>(), kAttnBwdSmem, stream>>>(                         \
      tmQ, tmK, tmV, tmdO, reinterpret_cast<const AttnBwdTile*>(tiles), lse, delta_ws, dq_acc,            \
      (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, T, Hq, Hkv, lddk, lddv, softmax_scale, status, key_exit)
  const bool tree = key_exit != nullptr;
  if (compute_warps == 8) {
    if (tree) B200_ATTN_BWD_LAUNCH(8, true); else B200_ATTN_BWD_LAUNCH(8, false);
  } else {
    if (tree) B200_ATTN_BWD_LAUNCH(4, true); else B200_ATTN_BWD_LAUNCH(4, false);
  }
#undef B200_ATTN_BWD_LAUNCH
  B200_CHECK(cudaGetLastError());
  if (dq) {
    const long long n = static_cast<long long>(T) * Hq * kD;
    long long g = (n / 4 + 255) / 256;
    const long long maxg = static_cast<long long>(sm_count()) * 16;
    if (g > maxg) g = maxg;
    f32_to_bf16_kernel<<<(unsigned)g, 256, 0, stream>>>(dq_acc, (__nv_bfloat16*)dq, n);
    B200_CHECK(cudaGetLastError());
  }
  return 0;
}

}  // extern "C"
