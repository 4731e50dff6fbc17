// Varlen packed causal FlashAttention forward for sm_100a (tcgen05 + TMEM).
//
//   q [T, Hq, 128], k/v [T, Hkv, 128] (bf16, row pitch given), cu_seqlens → o [T, Hq, 128], lse [Hq, T]
//
// One CTA handles one (128-row query tile of one sequence, query head) pair and
// walks the key/value blocks (64 rows each) up to the causal diagonal.
// S = Q K^T and O += P V both run on tcgen05 with fp32 accumulators in TMEM:
// S is double-buffered (2 x 64 columns) and O takes 128 columns, 256 columns
// per CTA, so two CTAs share an SM and one CTA's tensor work overlaps the
// other's softmax. The 128 softmax threads each own one query row (TMEM lane),
// so row max / row sum need no shuffles. O is rescaled in TMEM only when a
// row's running max grows by more than 2^8 (lazy rescaling).
//
// K/V tiles arrive by TMA (no multicast) into 128B-swizzled shared memory; V is
// consumed as an MN-major B operand straight from its natural [kv, d] layout,
// P is written by the softmax threads as a K-major swizzled A operand.
//
// Replaces flash-attn / aten._flash_attention_forward in the reference
// (areal/models/transformers/ulyssess_patch.py:57,
//  areal/experimental/models/archon/attention/varlen.py:49).
#include "common/host_utils.h"
#include "common/ptx.cuh"

namespace b200 {

constexpr int kD = 128;
constexpr int kQT = 128;  // query rows per CTA
constexpr int kKT = 64;   // kv rows per block
constexpr int kAttnThreads = 192;

struct AttnTile {
  int q_start;   // first global token row of the query tile
  int q_len;     // valid query rows (<= 128)
  int kv_start;  // first global token row of the sequence
  int kv_len;    // keys visible to the last row of the tile (causal extent)
  int q_off;     // offset of the tile's first row inside its sequence
  int pad0, pad1, pad2;
};

constexpr int kSmemQ = kQT * kD * 2;           // 32 KB
constexpr int kSmemK = kKT * kD * 2;           // 16 KB per stage
constexpr int kSmemV = kKT * kD * 2;           // 16 KB per stage
constexpr int kSmemP = kQT * kKT * 2;          // 16 KB
constexpr int kAttnFwdSmem = kSmemQ + 2 * kSmemK + 2 * kSmemV + kSmemP;  // 112 KB

__global__ void __launch_bounds__(kAttnThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnTile* __restrict__ tiles,
                __nv_bfloat16* __restrict__ o, float* __restrict__ lse, int T, int Hq, int Hkv,
                float scale_log2, int* status, const int* __restrict__ key_exit) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bars[16];
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;

  uint8_t* sQ = smem;
  uint8_t* sK = smem + kSmemQ;
  uint8_t* sV = sK + 2 * kSmemK;
  uint8_t* sP = sV + 2 * kSmemV;
  uint64_t* q_full = &bars[0];
  uint64_t* k_full = &bars[1];   // [2]
  uint64_t* k_empty = &bars[3];  // [2]
  uint64_t* v_full = &bars[5];   // [2]
  uint64_t* v_empty = &bars[7];  // [2]
  uint64_t* s_full = &bars[9];   // [2]
  uint64_t* p_ready = &bars[11];
  uint64_t* pv_done = &bars[12];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AttnTile tile = tiles[blockIdx.x];
  const int h = blockIdx.y;
  const int hk = h / (Hq / Hkv);
  const int nblk = (tile.kv_len + kKT - 1) / kKT;

  if (threadIdx.x == 0) {
    if (smem_u32(smem) & 1023) {
      atomicCAS(status, 0, kErrBounds);
      abort_word = 1;
    } else {
      abort_word = 0;
    }
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(p_ready, 128);
    mbar_init(pv_done, 1);
    fence_mbar_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  if (warp == 5) {
    tmem_alloc(&tmem_holder, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  const uint32_t tmem_O = tmem_base + 128;
  const bool bad_align = (abort_word != 0);

  if (bad_align) {
    // fall through to teardown
  } else if (warp == 4) {
    // ------------------------------------------------------ TMA producer --
    if (elect_one_sync()) {
      mbar_arrive_expect_tx(q_full, kSmemQ);
      tma_load_2d(sQ, &tmQ, q_full, h * kD, tile.q_start);
      tma_load_2d(sQ + kSmemQ / 2, &tmQ, q_full, h * kD + 64, tile.q_start);
      bool ok = true;
      for (int j = 0; j < nblk && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int row = tile.kv_start + j * kKT;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&k_full[st], kSmemK);
        tma_load_2d(sK + st * kSmemK, &tmK, &k_full[st], hk * kD, row);
        tma_load_2d(sK + st * kSmemK + kSmemK / 2, &tmK, &k_full[st], hk * kD + 64, row);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&v_full[st], kSmemV);
        tma_load_2d(sV + st * kSmemV, &tmV, &v_full[st], hk * kD, row);
        tma_load_2d(sV + st * kSmemV + kSmemV / 2, &tmV, &v_full[st], hk * kD + 64, row);
      }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(status, 0, kErrMbarTimeoutProducer);
        unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------- MMA issuer --
    if (elect_one_sync()) {
      constexpr uint32_t idesc_s = make_idesc(1, 1, 0, 0, kQT, kKT);
      constexpr uint32_t idesc_o = make_idesc(1, 1, 0, 1, kQT, kD);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      const uint32_t q_addr = smem_u32(sQ);
      const uint32_t p_addr = smem_u32(sP);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, abort_flag)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + st * kSmemK);
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          const uint32_t half = k >> 2, kk = k & 3;
          const uint64_t a = make_sdesc_sw128(q_addr + half * (kSmemQ / 2) + kk * 32, 16, 1024);
          const uint64_t b = make_sdesc_sw128(k_addr + half * (kSmemK / 2) + kk * 32, 16, 1024);
          umma_f16(tmem_base + st * kKT, a, b, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[st]);
        return true;
      };
      if (ok && nblk > 0) ok = issue_s(0);
      for (int j = 0; j < nblk && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < nblk) {
          // S buffer (j+1)&1 was consumed by the softmax of block j-1, which
          // has signalled p_ready for j-1 (waited on below in the previous turn).
          if (!issue_s(j + 1)) { ok = false; break; }
        }
        if (!mbar_wait(p_ready, j & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(&v_full[st], ph, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + st * kSmemV);
#pragma unroll
        for (int k = 0; k < kKT / 16; ++k) {
          const uint64_t a = make_sdesc_sw128(p_addr + k * 32, 16, 1024);
          const uint64_t b = make_sdesc_sw128(v_addr + k * 2048, kSmemV / 2, 1024);
          umma_f16(tmem_O, a, b, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(pv_done);
      }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(status, 0, kErrMbarTimeoutMma);
      }
    }
  } else {
    // ----------------------------------------------------------- softmax --
    const int r = warp * 32 + lane;  // query row inside the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const int q_pos = tile.q_off + r;  // position inside the sequence
    float m_used = -INFINITY;
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk && ok; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[st], ph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      float s[kKT];
      {
        uint32_t raw[32];
        tmem_ld_32x32(tmem_base + lane_addr + st * kKT, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(raw[i]);
        tmem_ld_32x32(tmem_base + lane_addr + st * kKT + 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[32 + i] = __uint_as_float(raw[i]);
      }
      const int kv0 = j * kKT;
      float mx = -INFINITY;
      const bool need_mask = (kv0 + kKT - 1 > tile.q_off) || (kv0 + kKT > tile.kv_len);
      if (key_exit != nullptr) {
        // tree (trie-packed) attention: tokens are in depth-first order, key kv is an ancestor of
        // query q_pos iff kv <= q_pos < exit[kv] (exit = end of the key's subtree)
        const int* ex = key_exit + tile.kv_start + kv0;
#pragma unroll
        for (int i = 0; i < kKT; ++i) {
          const int kv = kv0 + i;
          const bool valid = (kv <= q_pos) && (kv < tile.kv_len) && (q_pos < __ldg(ex + i));
          s[i] = valid ? s[i] * scale_log2 : -INFINITY;
          mx = fmaxf(mx, s[i]);
        }
      } else if (need_mask) {
#pragma unroll
        for (int i = 0; i < kKT; ++i) {
          const int kv = kv0 + i;
          const bool valid = (kv <= q_pos) && (kv < tile.kv_len);
          s[i] = valid ? s[i] * scale_log2 : -INFINITY;
          mx = fmaxf(mx, s[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < kKT; ++i) {
          s[i] *= scale_log2;
          mx = fmaxf(mx, s[i]);
        }
      }
      // the previous P V product must be complete before O is rescaled or P overwritten
      if (j > 0) {
        if (!mbar_wait(pv_done, (j - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
      }
      const float m_new = fmaxf(m_used, mx);
      const bool grow = (m_new > m_used + 8.f) || (m_used == -INFINITY && m_new > -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_new);
        l *= alpha;
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < kD / 32; ++c) {
            uint32_t raw[32];
            tmem_ld_32x32(tmem_O + lane_addr + c * 32, raw);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * alpha);
            tmem_st_32x32(tmem_O + lane_addr + c * 32, raw);
          }
          tmem_st_wait();
        }
        m_used = m_new;
      }
      const float mref = (m_used == -INFINITY) ? 0.f : m_used;
      float rs = 0.f;
      uint8_t* prow = sP + r * 128;
#pragma unroll
      for (int c = 0; c < kKT / 8; ++c) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          p[i] = exp2f(s[c * 8 + i] - mref);
        }
        uint4 pk;
        __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          pb[i] = __floats2bfloat162_rn(p[2 * i], p[2 * i + 1]);
          // accumulate the row sum from the rounded values the tensor core will see
          float2 back = __bfloat1622float2(pb[i]);
          rs += back.x + back.y;
        }
        *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = pk;
      }
      l += rs;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    if (ok && nblk > 0) {
      ok = mbar_wait(pv_done, (nblk - 1) & 1, abort_flag);
      tc_fence_after();
    }
    if (ok) {
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const bool row_valid = r < tile.q_len;
      __nv_bfloat16* orow = o + (static_cast<long long>(tile.q_start + r) * Hq + h) * kD;
#pragma unroll 1
      for (int c = 0; c < kD / 32; ++c) {
        uint32_t raw[32];
        if (nblk > 0) {
          tmem_ld_32x32(tmem_O + lane_addr + c * 32, raw);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) raw[i] = 0;
        }
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 pk;
            __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              pb[e] = __floats2bfloat162_rn(__uint_as_float(raw[i * 8 + 2 * e]) * inv_l,
                                            __uint_as_float(raw[i * 8 + 2 * e + 1]) * inv_l);
            reinterpret_cast<uint4*>(orow + c * 32)[i] = pk;
          }
        }
      }
      if (row_valid)
        lse[static_cast<long long>(h) * T + tile.q_start + r] =
            (l > 0.f) ? (m_used * 0.6931471805599453f + logf(l)) : -INFINITY;
    } else if (lane == 0) {
      *abort_flag = 1;
      atomicCAS(status, 0, kErrMbarTimeoutEpilogue);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace b200

extern "C" {

// q: [T, Hq*128] contiguous; k, v: rows of Hkv*128 bf16 with pitches ldk / ldv
// (elements; multiples of 8, so k and v may be views into a fused qkv buffer).
// tiles: device array of n_tiles AttnTile records (see attention.py).
// Extended form: `Tkv` rows in k / v (context parallelism: local queries against gathered keys;
// 0 = same as T) and `key_exit` (int [Tkv], sequence-relative end of every key's subtree; enables
// the ancestor mask of tree attention, null = plain causal).
int b200_attn_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse,
                     const void* tiles, int n_tiles, int T, int Tkv, int Hq, int Hkv, long long ldq,
                     long long ldk, long long ldv, float softmax_scale, const int* key_exit,
                     cudaStream_t stream);

int b200_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                  const void* tiles, int n_tiles, int T, int Hq, int Hkv, long long ldq,
                  long long ldk, long long ldv, float softmax_scale, cudaStream_t stream) {
  return b200_attn_fwd_ex(q, k, v, o, lse, tiles, n_tiles, T, 0, Hq, Hkv, ldq, ldk, ldv, softmax_scale, nullptr,
                          stream);
}

int b200_attn_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse,
                     const void* tiles, int n_tiles, int T, int Tkv, int Hq, int Hkv, long long ldq,
                     long long ldk, long long ldv, float softmax_scale, const int* key_exit,
                     cudaStream_t stream) {
  using namespace b200;
  if (n_tiles == 0 || T == 0) return 0;
  if (Tkv <= 0) Tkv = T;
  if (Hq % Hkv) return -100;
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)Hq * kD,
                        ldq * 2, kQT, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tkv, (uint64_t)Hkv * kD, ldk * 2,
                    kKT, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tkv, (uint64_t)Hkv * kD, ldv * 2,
                    kKT, 64);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CHECK(cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kAttnFwdSmem));
    attr_set = true;
  }
  int* status = device_status_word();
  if (!status) return -3;
  dim3 grid(n_tiles, Hq);
  attn_fwd_kernel<<<grid, kAttnThreads, kAttnFwdSmem, stream>>>(
      tmQ, tmK, tmV, reinterpret_cast<const AttnTile*>(tiles), (__nv_bfloat16*)o, lse, T, Hq, Hkv,
      softmax_scale * 1.4426950408889634f, status, key_exit);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
