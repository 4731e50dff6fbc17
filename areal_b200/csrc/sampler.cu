// Fused sampling for the rollout engine: temperature, optional top-k / top-p,
// inverse-CDF sampling from one uniform per row, and the log-probability of the
// drawn token under the temperature-scaled (unfiltered) distribution, which is
// what the trainer later compares with its own recomputed logprob.
//
// One CTA per row of fp32 logits [B, V]. Pass 1: online max / sum-exp.
// Optional: bisection on a logit threshold for top-k (count) and top-p (mass).
// Pass 2: per-thread chunk masses → block scan → locate the token whose CDF
// interval contains u * Z. The second pass hits L2.
//
// Stands in for the sampler of the external inference server the reference
// drives (areal/engine/sglang_remote.py:43-127 sampling_params, return_logprob).
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "common/host_utils.h"

namespace b200 {

constexpr int kSampThreads = 512;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_add(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide reductions over kSampThreads threads (result broadcast to all).
__device__ __forceinline__ float block_max(float v, float* sm) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  float r = (lane < kSampThreads / 32) ? sm[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}
__device__ __forceinline__ float block_add(float v, float* sm) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_add(v);
  __syncthreads();
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  float r = (lane < kSampThreads / 32) ? sm[lane] : 0.f;
  r = warp_add(r);
  return r;
}

// uniforms: [B] in (0,1). temperature <= 0 means greedy. top_k <= 0 or >= V
// disables top-k; top_p >= 1 disables top-p.
__global__ void __launch_bounds__(kSampThreads)
sample_kernel(const float* __restrict__ logits, long long ld, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ uniforms,
              int* __restrict__ tokens, float* __restrict__ logprobs) {
  __shared__ float sm[kSampThreads / 32 + 1];
  __shared__ float s_scan[kSampThreads];
  __shared__ int s_pick;
  const int row = blockIdx.x;
  const float* x = logits + static_cast<long long>(row) * ld;
  const float temp = temperature[row];
  const bool greedy = !(temp > 0.f);
  const float inv_t = greedy ? 1.f : 1.f / temp;
  const int tid = threadIdx.x;
  // contiguous chunk per thread so the scan order is the vocabulary order
  const int per = (V + kSampThreads - 1) / kSampThreads;
  const int c0 = min(V, tid * per), c1 = min(V, c0 + per);

  // pass 1: max (and argmax for greedy)
  float mx = -INFINITY;
  int amax = 0x7fffffff;
  for (int i = c0; i < c1; ++i) {
    const float v = x[i] * inv_t;
    if (v > mx) {
      mx = v;
      amax = i;
    }
  }
  const float M = block_max(mx, sm);
  float se = 0.f;
  for (int i = c0; i < c1; ++i) se += __expf(x[i] * inv_t - M);
  const float Z = block_add(se, sm);
  const float logZ = M + logf(Z);

  if (greedy) {
    // smallest index among the maxima
    int cand = (mx == M) ? amax : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __shared__ int s_cand[kSampThreads / 32];
    if ((tid & 31) == 0) s_cand[tid >> 5] = cand;
    __syncthreads();
    if (tid == 0) {
      int best = 0x7fffffff;
      for (int w = 0; w < kSampThreads / 32; ++w) best = min(best, s_cand[w]);
      tokens[row] = best;
      logprobs[row] = x[best] * inv_t - logZ;
    }
    return;
  }

  // threshold (in the shifted domain y = x/T - M, y <= 0): keep y >= thr
  float thr = -INFINITY;
  const int k = top_k ? top_k[row] : 0;
  const float p = top_p ? top_p[row] : 1.f;
  if (k > 0 && k < V) {
    // largest thr with count(y >= thr) >= k
    float lo = -60.f, hi = 0.f;  // count(>=lo) is (nearly) everything, count(>=hi) >= 1
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (lo + hi);
      float cnt = 0.f;
      for (int i = c0; i < c1; ++i) cnt += (x[i] * inv_t - M >= mid) ? 1.f : 0.f;
      cnt = block_add(cnt, sm);
      if (cnt >= static_cast<float>(k)) lo = mid; else hi = mid;
    }
    thr = fmaxf(thr, lo);
  }
  if (p < 1.f) {
    // largest thr with mass(y >= thr) >= p * Z
    float lo = -60.f, hi = 0.f;
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (lo + hi);
      float mass = 0.f;
      for (int i = c0; i < c1; ++i) {
        const float y = x[i] * inv_t - M;
        mass += (y >= mid) ? __expf(y) : 0.f;
      }
      mass = block_add(mass, sm);
      if (mass >= p * Z) lo = mid; else hi = mid;
    }
    thr = fmaxf(thr, lo);
  }

  // pass 2: chunk masses over the kept set, scan, locate
  float cm = 0.f;
  for (int i = c0; i < c1; ++i) {
    const float y = x[i] * inv_t - M;
    cm += (y >= thr) ? __expf(y) : 0.f;
  }
  s_scan[tid] = cm;
  if (tid == 0) s_pick = -1;
  __syncthreads();
  // inclusive scan (Hillis-Steele over 512 entries)
  for (int off = 1; off < kSampThreads; off <<= 1) {
    const float add = (tid >= off) ? s_scan[tid - off] : 0.f;
    __syncthreads();
    s_scan[tid] += add;
    __syncthreads();
  }
  const float total = s_scan[kSampThreads - 1];
  const float target = uniforms[row] * total;
  const float before = (tid == 0) ? 0.f : s_scan[tid - 1];
  const float after = s_scan[tid];
  // the owning thread is the first whose inclusive prefix reaches the target
  if (cm > 0.f && before <= target && target < after) {
    float run = before;
    int pick = -1, last_kept = -1;
    for (int i = c0; i < c1; ++i) {
      const float y = x[i] * inv_t - M;
      if (y >= thr) {
        last_kept = i;
        run += __expf(y);
        if (run > target) {
          pick = i;
          break;
        }
      }
    }
    if (pick < 0) pick = last_kept;
    atomicMax(&s_pick, pick);
  }
  __syncthreads();
  if (tid == 0) {
    int pick = s_pick;
    if (pick < 0) {
      // numerical corner (target == total): fall back to the most likely token
      pick = 0;
      float best = -INFINITY;
      for (int i = 0; i < V; ++i)
        if (x[i] > best) {
          best = x[i];
          pick = i;
        }
    }
    tokens[row] = pick;
    logprobs[row] = x[pick] * inv_t - logZ;
  }
}

}  // namespace b200

extern "C" {

int b200_sample(const float* logits, long long ld, int B, int V, const float* temperature,
                const int* top_k, const float* top_p, const float* uniforms, int* tokens,
                float* logprobs, cudaStream_t stream) {
  if (B == 0) return 0;
  b200::sample_kernel<<<B, b200::kSampThreads, 0, stream>>>(logits, ld, V, temperature, top_k,
                                                            top_p, uniforms, tokens, logprobs);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
