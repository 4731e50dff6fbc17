// PPO / GRPO numerics kernels: decoupled clipped policy loss (forward value and
// d loss / d logprob in one pass), group-normalised advantages, and the GAE
// reverse scan over packed sequences.
//
// Semantics follow the reference implementation:
//   loss   areal/utils/functional/functional.py:429-559 (ratio, clip, dual clip,
//          behaviour importance weight with an upper cap, fixed denominator)
//   norm   areal/utils/data.py:1378-1595 (group mean / std, unbiased std, eps)
//   GAE    areal/trainer/ppo/actor.py:214-235
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "common/host_utils.h"

namespace b200 {

struct PpoLossParams {
  float eps_clip;
  float eps_clip_higher;  // < 0: same as eps_clip
  float c_clip;           // <= 1: dual clip disabled
  float behav_cap;        // <= 0: no cap on exp(prox - behave)
  float inv_denom;        // 1 / max(count(loss_mask), 1) fixed before any rejection
  int use_decoupled;      // bit 0: the ratio's denominator is the proximal policy (else the behaviour policy);
                          // bit 1: multiply by the behaviour importance weight exp(prox - behave)
};

// stats[0] = sum loss, [1] = # clipped tokens, [2] = # dual-clipped tokens,
// [3] = sum importance weight over masked tokens, [4] = sum |ratio-1|,
// [5] = # tokens dropped by the behaviour cap.
__global__ void ppo_loss_kernel(const float* __restrict__ logp, const float* __restrict__ prox,
                                const float* __restrict__ behav, const float* __restrict__ adv,
                                const uint8_t* __restrict__ mask, float* __restrict__ dlogp,
                                float* __restrict__ stats, long long n, PpoLossParams p) {
  float acc[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g = 0.f;
    if (mask[i]) {
      const float lp = logp[i];
      const float px = (p.use_decoupled & 1) ? prox[i] : behav[i];
      const float A = adv[i];
      const float ratio = __expf(lp - px);
      const float hi = 1.f + (p.eps_clip_higher >= 0.f ? p.eps_clip_higher : p.eps_clip);
      const float lo = 1.f - p.eps_clip;
      const float clipped = fminf(fmaxf(ratio, lo), hi);
      const float l1 = -A * ratio;
      const float l2 = -A * clipped;
      float L = fmaxf(l1, l2);
      // d/d logp: ratio' = ratio; the clipped branch has zero slope when active
      const bool clip_active = (l2 > l1);
      float dL = clip_active ? 0.f : -A * ratio;
      bool dual = false;
      if (p.c_clip > 1.f && A < 0.f) {
        const float l3 = -A * p.c_clip;  // sign(A) * c * A with A < 0
        if (l3 < L) {
          L = l3;
          dL = 0.f;
          dual = true;
        }
      }
      float w = 1.f;
      bool dropped = false;
      if (p.use_decoupled & 2) {
        w = __expf(px - behav[i]);
        if (p.behav_cap > 0.f && w > p.behav_cap) {
          w = 0.f;
          dropped = true;
        }
      }
      acc[0] += L * w * p.inv_denom;
      g = dL * w * p.inv_denom;
      acc[1] += clip_active ? 1.f : 0.f;
      acc[2] += dual ? 1.f : 0.f;
      acc[3] += w;
      acc[4] += fabsf(ratio - 1.f);
      acc[5] += dropped ? 1.f : 0.f;
    }
    dlogp[i] = g;
  }
  __shared__ float red[6][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int k = 0; k < 6; ++k) {
    float v = acc[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[k][warp] = v;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
#pragma unroll
    for (int k = 0; k < 6; ++k) {
      float v = lane < nw ? red[k][lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) atomicAdd(&stats[k], v);
    }
  }
}

// One warp per group of `group_size` consecutive sequences.
// out[i] = (r[i] - mean_g) / (std_g + eps); std over the group (unbiased if
// requested); leave-one-out mean optional. mean_level / std_level: 1 = group, 0 = none.
__global__ void group_norm_kernel(const float* __restrict__ r, float* __restrict__ out, int n_groups,
                                  int group_size, int mean_group, int std_group, int leave1out,
                                  int unbiased, float eps) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= n_groups) return;
  const float* rg = r + static_cast<long long>(gw) * group_size;
  double s = 0.0, ss = 0.0;
  for (int i = lane; i < group_size; i += 32) {
    s += rg[i];
    ss += static_cast<double>(rg[i]) * rg[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
  }
  const double mean = s / group_size;
  double var = ss / group_size - mean * mean;
  if (var < 0) var = 0;
  if (unbiased && group_size > 1) var *= static_cast<double>(group_size) / (group_size - 1);
  const float sd = static_cast<float>(sqrt(var));
  for (int i = lane; i < group_size; i += 32) {
    float m = 0.f;
    if (mean_group) {
      m = (leave1out && group_size > 1) ? static_cast<float>((s - rg[i]) / (group_size - 1))
                                        : static_cast<float>(mean);
    }
    float v = rg[i] - m;
    if (std_group) v /= (sd + eps);
    out[static_cast<long long>(gw) * group_size + i] = v;
  }
}

// GAE over packed sequences; one thread per sequence walks it backwards.
// rewards / values / mask are [T] packed; values may be null (treated as 0);
// no_eos[b] != 0 marks sequences truncated at the length limit.
__global__ void gae_kernel(const float* __restrict__ rewards, const float* __restrict__ values,
                           const uint8_t* __restrict__ mask, const int* __restrict__ cu_seqlens,
                           const uint8_t* __restrict__ no_eos, float* __restrict__ adv,
                           float* __restrict__ ret, int n_seqs, float gamma, float lam) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_seqs) return;
  const int s = cu_seqlens[b], e = cu_seqlens[b + 1];
  if (e <= s) return;
  float last_gae = 0.f;
  // bootstrap from the last value only when the sequence was cut off without EOS
  float next_v = (values && no_eos && no_eos[b]) ? values[e - 1] : 0.f;
  adv[e - 1] = 0.f;
  ret[e - 1] = values ? values[e - 1] : 0.f;
  for (int t = e - 2; t >= s; --t) {
    const float v = values ? values[t] : 0.f;
    const float delta = rewards[t] + gamma * next_v - v;
    const float a = delta + gamma * lam * last_gae;
    // positions outside the loss mask carry the running values through
    if (mask[t]) {
      last_gae = a;
      next_v = v;
    }
    adv[t] = last_gae;
    ret[t] = last_gae + v;
  }
}

}  // namespace b200

extern "C" {

int b200_ppo_loss(const float* logp, const float* prox, const float* behav, const float* adv,
                  const uint8_t* mask, float* dlogp, float* stats, long long n, float eps_clip,
                  float eps_clip_higher, float c_clip, float behav_cap, float inv_denom,
                  int use_decoupled, cudaStream_t stream) {
  using namespace b200;
  B200_CHECK(cudaMemsetAsync(stats, 0, 6 * sizeof(float), stream));
  if (n == 0) return 0;
  PpoLossParams p{eps_clip, eps_clip_higher, c_clip, behav_cap, inv_denom, use_decoupled};
  long long grid = (n + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 8;
  if (grid > maxg) grid = maxg;
  ppo_loss_kernel<<<(unsigned)grid, 256, 0, stream>>>(logp, prox, behav, adv, mask, dlogp, stats, n,
                                                      p);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_group_norm(const float* r, float* out, int n_groups, int group_size, int mean_group,
                    int std_group, int leave1out, int unbiased, float eps, cudaStream_t stream) {
  if (n_groups == 0) return 0;
  const int tpb = 128;
  const int grid = (n_groups * 32 + tpb - 1) / tpb;
  b200::group_norm_kernel<<<grid, tpb, 0, stream>>>(r, out, n_groups, group_size, mean_group,
                                                    std_group, leave1out, unbiased, eps);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_gae(const float* rewards, const float* values, const uint8_t* mask, const int* cu_seqlens,
             const uint8_t* no_eos, float* adv, float* ret, int n_seqs, float gamma, float lam,
             cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  b200::gae_kernel<<<(n_seqs + 127) / 128, 128, 0, stream>>>(rewards, values, mask, cu_seqlens,
                                                             no_eos, adv, ret, n_seqs, gamma, lam);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
