// Fused LM-head GEMM + log-softmax statistics (vocab-parallel ready) on tcgen05.
//
// Forward: logits = X W^T / temperature are produced tile by tile in TMEM and
// consumed in the epilogue; only four floats per (row, vocab split) leave the
// SM: running max, sum of exp, sum of exp*logit (for the entropy) and the
// label's logit when the label falls inside the split. A combine kernel merges
// the splits of all vocab shards (local splits and, under tensor parallelism,
// the other ranks' partials) into logprob, entropy, logZ and E[logit].
// The [T, V] logits are never written.
//
// Backward: the same GEMM recomputes a [rows, V_local] block of logits and its
// epilogue writes d logits (bf16) for that row chunk,
//   dz = (g_logp * (onehot - p) + g_ent * p * (E[y] - y)) / temperature,
// which two plain GEMMs then turn into dX and dW. Only one row chunk of dz is
// ever resident.
//
// Replaces the reference's chunked log_softmax over materialised logits and its
// 3-4 all-reduces (areal/utils/functional/vocab_parallel.py:84-372).
#include "common/gemm_core.cuh"
#include "common/host_utils.h"

namespace b200 {

struct LmStatsEpi {
  float* partials;          // [nsplit, T, 4] : m, l, sx, target
  // vocab-parallel: the records go straight into every tensor-parallel peer's buffer
  // ([n_peers * nsplit, T, 4], this rank's records at slot_base) instead of `partials`
  float* peers[8];
  int n_peers;
  int slot_base;
  const int* labels;        // [T] global vocab ids
  int T, N;                 // rows, local vocab size
  int vocab_start;          // global id of local column 0
  int nb_per;               // n-blocks per split
  int nsplit;
  float inv_temp;
  struct State {
    float m, l, sx, t;
  };
  __device__ __forceinline__ bool tile(int cta, int ncta, int it, int tiles_m, int tiles_n,
                                       int& m_blk, int& n_blk) const {
    const int item_local = it / nb_per;
    const int j = it - item_local * nb_per;
    const long long w = static_cast<long long>(item_local) * ncta + cta;
    if (w >= static_cast<long long>(tiles_m) * nsplit) return false;
    m_blk = static_cast<int>(w % tiles_m);
    n_blk = static_cast<int>(w / tiles_m) * nb_per + j;
    return true;
  }
  __device__ __forceinline__ bool gate(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ void begin(State& s, int, int n_blk, int) const {
    if (n_blk % nb_per == 0) {
      s.m = -INFINITY;
      s.l = 0.f;
      s.sx = 0.f;
      s.t = 0.f;
    }
  }
  __device__ __forceinline__ void chunk(State& s, int row, int col0, const float (&v)[32]) const {
    if (row >= T || col0 >= N) return;
    const int label = labels[row] - vocab_start;
    float x[32];
    float cm = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      x[i] = (col0 + i < N) ? v[i] * inv_temp : -INFINITY;
      cm = fmaxf(cm, x[i]);
    }
    if (label >= col0 && label < col0 + 32) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i == label) s.t = x[i];
    }
    const float m_new = fmaxf(s.m, cm);
    const float sc = (s.m == -INFINITY) ? 0.f : __expf(s.m - m_new);
    float l = 0.f, sx = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float e = __expf(x[i] - m_new);  // exp(-inf) = 0 for masked columns
      l += e;
      sx += (x[i] == -INFINITY) ? 0.f : e * x[i];
    }
    s.l = s.l * sc + l;
    s.sx = s.sx * sc + sx;
    s.m = m_new;
  }
  __device__ __forceinline__ void end(State& s, int, int n_blk, int row) const {
    if ((n_blk + 1) % nb_per == 0 && row < T) {
      const int split = n_blk / nb_per;
      const float4 rec = make_float4(s.m, s.l, s.sx, s.t);
      if (n_peers == 0) {
        reinterpret_cast<float4*>(partials)[static_cast<long long>(split) * T + row] = rec;
      } else {
        const long long at = static_cast<long long>(slot_base + split) * T + row;
        for (int p = 0; p < n_peers; ++p) reinterpret_cast<float4*>(peers[p])[at] = rec;
      }
    }
  }
};

// Merges `nparts` partial records per row. partials: [nparts, T, 4].
// has_target: row's label lies in exactly one part (its t is non-zero there;
// the others wrote 0) so the target logit is the sum.
__global__ void lm_combine_kernel(const float* __restrict__ partials, int nparts, int T,
                                  float* __restrict__ logp, float* __restrict__ entropy,
                                  float* __restrict__ logz, float* __restrict__ ey) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= T) return;
  float M = -INFINITY;
  for (int p = 0; p < nparts; ++p)
    M = fmaxf(M, partials[(static_cast<long long>(p) * T + row) * 4]);
  float L = 0.f, SX = 0.f, t = 0.f;
  for (int p = 0; p < nparts; ++p) {
    const float4 r = reinterpret_cast<const float4*>(partials)[static_cast<long long>(p) * T + row];
    const float sc = (r.x == -INFINITY) ? 0.f : __expf(r.x - M);
    L += r.y * sc;
    SX += r.z * sc;
    t += r.w;
  }
  const float lz = M + logf(L);
  const float e = SX / L;
  if (logp) logp[row] = t - lz;
  if (entropy) entropy[row] = lz - e;
  if (logz) logz[row] = lz;
  if (ey) ey[row] = e;
}

struct LmDlogitsEpi {
  __nv_bfloat16* dz;  // [rows, ldz]
  const int* labels;
  const float* g_logp;  // [T] (may be null → 0)
  const float* g_ent;   // [T] (may be null → 0)
  const float* logz;    // [T]
  const float* ey;      // [T]
  long long ldz;
  int T, N, vocab_start;
  float inv_temp;
  struct State {
    float gl, ge, lz, e;
    int label;
  };
  __device__ __forceinline__ bool tile(int cta, int ncta, int it, int tiles_m, int tiles_n,
                                       int& m_blk, int& n_blk) const {
    return default_tile(cta, ncta, it, tiles_m, tiles_n, m_blk, n_blk);
  }
  __device__ __forceinline__ bool gate(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ void begin(State& s, int, int, int row) const {
    if (row < T) {
      s.gl = g_logp ? g_logp[row] : 0.f;
      s.ge = g_ent ? g_ent[row] : 0.f;
      s.lz = logz[row];
      s.e = ey[row];
      s.label = labels[row] - vocab_start;
    }
  }
  __device__ __forceinline__ void end(State&, int, int, int) const {}
  __device__ __forceinline__ void chunk(State& s, int row, int col0, const float (&v)[32]) const {
    if (row >= T || col0 >= N) return;
    float d[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float y = v[i] * inv_temp;
      const float p = __expf(y - s.lz);
      const float onehot = (col0 + i == s.label) ? 1.f : 0.f;
      d[i] = (s.gl * (onehot - p) + s.ge * p * (s.e - y)) * inv_temp;
    }
    __nv_bfloat16* out = dz + static_cast<long long>(row) * ldz + col0;
    if (col0 + 32 <= N && (ldz & 7) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 pk;
        __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int j = 0; j < 4; ++j) pb[j] = __floats2bfloat162_rn(d[8 * i + 2 * j], d[8 * i + 2 * j + 1]);
        reinterpret_cast<uint4*>(out)[i] = pk;
      }
    } else {
      for (int i = 0; i < 32; ++i)
        if (col0 + i < N) out[i] = __float2bfloat16(d[i]);
    }
  }
};


// ------------------------------------------------------------------ fused sampling (rollout decode)
//
// The decode step's LM head draws the next token inside the GEMM epilogue, so the [B, V] logits are
// never written either. Sampling from softmax(x / temperature) uses the Gumbel-max identity:
// argmax_i (x_i / T + g_i) with g_i = -log(-log u_i) i.i.d. is a draw from the softmax. Each
// (row, vocab split) emits its running max, its sum of exponentials, and the best perturbed score with
// the index and the (scaled) logit that achieved it; the combine kernel picks the best split and
// returns log p(token) = x_token / T - logZ under the unfiltered distribution. temperature <= 0 means
// greedy (no noise, logprob under T = 1). The noise comes from Philox4x32-7 keyed by a seed, with the
// counter (column / 4, row, step): the step counter lives in device memory and the combine kernel
// advances it, so a captured CUDA graph draws fresh noise on every replay.
__device__ __forceinline__ uint4 philox4x32_7(uint4 c, uint2 k) {
#pragma unroll
  for (int i = 0; i < 7; ++i) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
    c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
    k.x += 0x9E3779B9u;
    k.y += 0xBB67AE85u;
  }
  return c;
}

// Standard Gumbel variate from 32 random bits. w is uniform on a 2^-23 grid strictly inside (0, 1);
// E = -log(1 - w) is Exp(1): by its series where w is small (the approximate log loses all relative
// accuracy next to 1), by the fast log elsewhere.
__device__ __forceinline__ float gumbel_from_bits(uint32_t r) {
  const float w = (static_cast<float>(r >> 9) + 0.5f) * 1.1920928955078125e-07f;
  const float e_small = w * (1.f + w * (0.5f + w * (0.33333334f + 0.25f * w)));
  const float e = (w < 0.015625f) ? e_small : -__logf(1.f - w);
  return -__logf(e);
}

struct LmSampleRec {
  float m, l, best, bx;
};

struct LmSampleEpi {
  LmSampleRec* partials;      // [nsplit, T]
  int* part_idx;              // [nsplit, T]
  const float* temperature;   // [T]
  const unsigned long long* rng;  // [0] seed, [1] step counter
  int T, N;
  int nb_per, nsplit;
  struct State {
    float m, l, best, bx, inv_t;
    int bi;
    uint32_t noisy, k0, k1, c2, c3;
  };
  __device__ __forceinline__ bool tile(int cta, int ncta, int it, int tiles_m, int tiles_n,
                                       int& m_blk, int& n_blk) const {
    const int item_local = it / nb_per;
    const int j = it - item_local * nb_per;
    const long long w = static_cast<long long>(item_local) * ncta + cta;
    if (w >= static_cast<long long>(tiles_m) * nsplit) return false;
    m_blk = static_cast<int>(w % tiles_m);
    n_blk = static_cast<int>(w / tiles_m) * nb_per + j;
    return true;  // blocks past the last column of a short final split load zeros and are skipped by chunk()
  }
  __device__ __forceinline__ bool gate(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ void begin(State& s, int, int n_blk, int row) const {
    if (n_blk % nb_per == 0) {
      s.m = -INFINITY;
      s.l = 0.f;
      s.best = -INFINITY;
      s.bx = 0.f;
      s.bi = 0x7fffffff;
      const float t = (row < T) ? temperature[row] : 1.f;
      s.noisy = (t > 0.f) ? 1u : 0u;
      s.inv_t = s.noisy ? 1.f / t : 1.f;
      const unsigned long long seed = rng[0], step = rng[1];
      s.k0 = static_cast<uint32_t>(seed);
      s.k1 = static_cast<uint32_t>(seed >> 32);
      s.c2 = static_cast<uint32_t>(step);
      s.c3 = static_cast<uint32_t>(step >> 32);
    }
  }
  __device__ __forceinline__ void chunk(State& s, int row, int col0, const float (&v)[32]) const {
    if (row >= T || col0 >= N) return;
    float x[32];
    float cm = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      x[i] = (col0 + i < N) ? v[i] * s.inv_t : -INFINITY;
      cm = fmaxf(cm, x[i]);
    }
    const float m_new = fmaxf(s.m, cm);
    const float sc = (s.m == -INFINITY) ? 0.f : __expf(s.m - m_new);
    float l = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) l += __expf(x[i] - m_new);  // exp(-inf) = 0 for masked columns
    s.l = s.l * sc + l;
    s.m = m_new;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t r[4] = {0u, 0u, 0u, 0u};
      if (s.noisy) {
        const uint4 q = philox4x32_7(make_uint4(static_cast<uint32_t>((col0 >> 2) + j), static_cast<uint32_t>(row),
                                                s.c2, s.c3), make_uint2(s.k0, s.k1));
        r[0] = q.x; r[1] = q.y; r[2] = q.z; r[3] = q.w;
      }
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int i = 4 * j + t;
        const float score = s.noisy ? x[i] + gumbel_from_bits(r[t]) : x[i];
        if (score > s.best) {  // strict: the smallest index wins a tie
          s.best = score;
          s.bx = x[i];
          s.bi = col0 + i;
        }
      }
    }
  }
  __device__ __forceinline__ void end(State& s, int, int n_blk, int row) const {
    if ((n_blk + 1) % nb_per == 0 && row < T) {
      const long long at = static_cast<long long>(n_blk / nb_per) * T + row;
      partials[at] = LmSampleRec{s.m, s.l, s.best, s.bx};
      part_idx[at] = s.bi;
    }
  }
};

// One warp per row: the lanes stride over the vocab splits, then merge (max, sum-exp) pairs and the best
// perturbed score by shuffles (ties go to the lower split, i.e. the smaller token id).
__global__ void lm_sample_combine_kernel(const LmSampleRec* __restrict__ partials, const int* __restrict__ part_idx,
                                         int nparts, int T, int* __restrict__ tokens, float* __restrict__ logprobs,
                                         unsigned long long* rng) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row < T) {
    float m = -INFINITY, l = 0.f, best = -INFINITY, bx = 0.f;
    int bp = 0x7fffffff;
    for (int p = lane; p < nparts; p += 32) {
      const LmSampleRec r = partials[static_cast<long long>(p) * T + row];
      if (r.m != -INFINITY) {
        const float mn = fmaxf(m, r.m);
        l = l * ((m == -INFINITY) ? 0.f : __expf(m - mn)) + r.l * __expf(r.m - mn);
        m = mn;
      }
      if (r.best > best) {
        best = r.best;
        bx = r.bx;
        bp = p;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), l2 = __shfl_xor_sync(0xffffffffu, l, o);
      const float b2 = __shfl_xor_sync(0xffffffffu, best, o), x2 = __shfl_xor_sync(0xffffffffu, bx, o);
      const int p2 = __shfl_xor_sync(0xffffffffu, bp, o);
      const float mn = fmaxf(m, m2);
      const float s1 = (m == -INFINITY) ? 0.f : __expf(m - mn), s2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
      l = l * s1 + l2 * s2;
      m = mn;
      if (b2 > best || (b2 == best && p2 < bp)) {
        best = b2;
        bx = x2;
        bp = p2;
      }
    }
    if (lane == 0) {
      tokens[row] = (bp == 0x7fffffff) ? 0 : part_idx[static_cast<long long>(bp) * T + row];
      logprobs[row] = bx - (m + logf(l));
    }
  }
  // every block of the GEMM that read the counter has finished (stream order): advance it for the next step
  if (blockIdx.x == 0 && threadIdx.x == 0) rng[1] += 1ull;
}

template <class Epi>
static int launch_lm(const void* X, const void* W, int T, int V, int H, long long ldx,
                     long long ldw, const Epi& epi, long long work_items, cudaStream_t stream) {
  constexpr int BN = 256;
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, H, ldx * 2, kBM, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, V, H, ldw * 2, BN, 64);
  if (rc) return rc;
  auto kern = gemm_tcgen05_kernel<BN, false, false, Epi>;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::kSmemBytes));
    attr_set = true;
  }
  int grid = static_cast<int>(work_items < sm_count() ? work_items : sm_count());
  if (grid <= 0) return 0;
  int* status = device_status_word();
  if (!status) return -3;
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(tmA, tmB, T, V, H, epi, status);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace b200

extern "C" {

// Number of vocab splits the forward uses for (T, V): enough work items to
// fill the SMs without making the partial buffer large.
int b200_lm_head_nsplit(int T, int V) {
  const int tiles_m = (T + 127) / 128;
  const int tiles_n = (V + 255) / 256;
  int want = (2 * b200::sm_count() + tiles_m - 1) / tiles_m;
  if (want < 1) want = 1;
  if (want > tiles_n) want = tiles_n;
  const int nb_per = (tiles_n + want - 1) / want;
  return (tiles_n + nb_per - 1) / nb_per;
}

// partials: fp32 [nsplit, T, 4] with nsplit = b200_lm_head_nsplit(T, V).
int b200_lm_head_stats(const void* X, const void* W, const int* labels, float* partials, int T,
                       int V, int H, long long ldx, long long ldw, int vocab_start,
                       float inv_temp, cudaStream_t stream) {
  using namespace b200;
  if (T == 0 || V == 0) return 0;
  const int tiles_m = (T + 127) / 128;
  const int tiles_n = (V + 255) / 256;
  const int nsplit = b200_lm_head_nsplit(T, V);
  const int nb_per = (tiles_n + nsplit - 1) / nsplit;
  LmStatsEpi epi{partials, {}, 0, 0, labels, T, V, vocab_start, nb_per, nsplit, inv_temp};
  return launch_lm(X, W, T, V, H, ldx, ldw, epi, static_cast<long long>(tiles_m) * nsplit,
                   stream);
}

// Vocab-parallel form: the epilogue stores this rank's records into every peer's buffer
// (peer_partials[p]: fp32 [n_peers * nsplit, T, 4] on rank p, this rank's slots starting at
// rank * nsplit), so the all-gather of the softmax statistics happens inside the GEMM kernel. A barrier
// among the ranks must separate this launch from b200_lm_head_combine over the local buffer.
int b200_lm_head_stats_peers(const void* X, const void* W, const int* labels, void* const* peer_partials,
                             int n_peers, int rank, int T, int V, int H, long long ldx, long long ldw,
                             int vocab_start, float inv_temp, cudaStream_t stream) {
  using namespace b200;
  if (n_peers < 1 || n_peers > 8) return -100;
  if (T == 0 || V == 0) return 0;
  const int tiles_m = (T + 127) / 128;
  const int tiles_n = (V + 255) / 256;
  const int nsplit = b200_lm_head_nsplit(T, V);
  const int nb_per = (tiles_n + nsplit - 1) / nsplit;
  LmStatsEpi epi{nullptr, {}, n_peers, rank * nsplit, labels, T, V, vocab_start, nb_per, nsplit, inv_temp};
  for (int p = 0; p < n_peers; ++p) epi.peers[p] = reinterpret_cast<float*>(peer_partials[p]);
  return launch_lm(X, W, T, V, H, ldx, ldw, epi, static_cast<long long>(tiles_m) * nsplit, stream);
}

// Vocab splits of the fused sampling head for (B, V): the split length (in 256-column blocks) that
// minimises the busiest CTA's number of tiles; ties go to the shorter split (more CTAs share the tail).
int b200_lm_head_sample_nb_per(int B, int V) {
  const int tiles_m = (B + 127) / 128;
  const int tiles_n = (V + 255) / 256;
  const int sms = b200::sm_count();
  long long best_cost = -1;
  int best = 1;
  for (int nb = 1; nb <= tiles_n && nb <= 64; ++nb) {
    const long long nsplit = (tiles_n + nb - 1) / nb;
    const long long items = nsplit * tiles_m;
    const long long cost = ((items + sms - 1) / sms) * nb;
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = nb;
    }
  }
  return best;
}

int b200_lm_head_sample_nsplit(int B, int V) {
  const int tiles_n = (V + 255) / 256;
  const int nb = b200_lm_head_sample_nb_per(B, V);
  return (tiles_n + nb - 1) / nb;
}

// Next-token sampling fused into the LM head: tokens[b] ~ softmax(X[b] W^T / temperature[b]) (argmax when
// temperature[b] <= 0) and logprobs[b] = log of that probability (under T = 1 for greedy rows).
// partials: 16 * nsplit * B bytes, part_idx: 4 * nsplit * B bytes with nsplit = b200_lm_head_sample_nsplit(B, V);
// rng: two 64-bit words on the device (seed, step counter), the counter is advanced by one.
int b200_lm_head_sample(const void* X, const void* W, const float* temperature, void* partials, int* part_idx,
                        unsigned long long* rng, int* tokens, float* logprobs, int B, int V, int H,
                        long long ldx, long long ldw, cudaStream_t stream) {
  using namespace b200;
  if (B == 0 || V == 0) return 0;
  const int tiles_m = (B + 127) / 128;
  const int nb_per = b200_lm_head_sample_nb_per(B, V);
  const int nsplit = b200_lm_head_sample_nsplit(B, V);
  LmSampleEpi epi{reinterpret_cast<LmSampleRec*>(partials), part_idx, temperature, rng, B, V, nb_per, nsplit};
  int rc = launch_lm(X, W, B, V, H, ldx, ldw, epi, static_cast<long long>(tiles_m) * nsplit, stream);
  if (rc) return rc;
  lm_sample_combine_kernel<<<(B + 3) / 4, 128, 0, stream>>>(reinterpret_cast<const LmSampleRec*>(partials),
                                                                part_idx, nsplit, B, tokens, logprobs, rng);
  B200_CHECK(cudaGetLastError());
  return 0;
}


int b200_lm_head_combine(const float* partials, int nparts, int T, float* logp, float* entropy,
                         float* logz, float* ey, cudaStream_t stream) {
  if (T == 0) return 0;
  b200::lm_combine_kernel<<<(T + 255) / 256, 256, 0, stream>>>(partials, nparts, T, logp, entropy,
                                                               logz, ey);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// Writes dz [T, V] (bf16, pitch ldz) for the rows of X given.
int b200_lm_head_dlogits(const void* X, const void* W, const int* labels, const float* g_logp,
                         const float* g_ent, const float* logz, const float* ey, void* dz, int T,
                         int V, int H, long long ldx, long long ldw, long long ldz,
                         int vocab_start, float inv_temp, cudaStream_t stream) {
  using namespace b200;
  if (T == 0 || V == 0) return 0;
  LmDlogitsEpi epi{reinterpret_cast<__nv_bfloat16*>(dz), labels, g_logp, g_ent, logz, ey, ldz, T, V,
                   vocab_start, inv_temp};
  const long long tiles = static_cast<long long>((T + 127) / 128) * ((V + 255) / 256);
  return launch_lm(X, W, T, V, H, ldx, ldw, epi, tiles, stream);
}

}  // extern "C"
