// Linear-attention building blocks for hybrid models (Qwen3.5 GatedDeltaNet, Bailing lightning
// attention) on packed variable-length sequences:
//
//   * causal depthwise conv1d (+ optional SiLU), forward and backward;
//   * gated delta rule and simple gated linear attention, forward, in the recurrent form with the
//     [Dk, Dv] state of a (sequence, head) pair resident in shared memory for the whole sequence.
//
// Counterparts of the external kernels the reference calls: causal_conv1d_fn
// (areal/experimental/models/archon/qwen3_5/model/model.py:244), fla chunk_gated_delta_rule (:291)
// and fla chunk_simple_gla (areal/models/mcore/lightning_attention.py:304).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "common/host_utils.h"

namespace b200 {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float dsilu_f(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

// seq_of[t] = index of the sequence that owns token t; cu[seq] = its first token.
// y[t,c] = act(bias[c] + sum_j w[c,j] * x[t - (K-1) + j, c]) over tokens of the same sequence.
__global__ void conv1d_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                  const float* __restrict__ bias, const int* __restrict__ seq_of,
                                  const int* __restrict__ cu, __nv_bfloat16* __restrict__ y, int T, int C, int K, int act) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(T) * C) return;
  const int t = static_cast<int>(i / C), c = static_cast<int>(i % C);
  const int s0 = cu[seq_of[t]];
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < K; ++j) {
    const int tt = t - (K - 1) + j;
    if (tt >= s0) acc += w[c * K + j] * __bfloat162float(x[static_cast<long long>(tt) * C + c]);
  }
  y[i] = __float2bfloat16(act ? silu_f(acc) : acc);
}

// dx[t,c] = sum_j w[c,j] * g[t + (K-1) - j, c] (same sequence), g = dy * act'(pre);
// dw[c,j] += sum_t g[t,c] * x[t - (K-1) + j, c]; dbias[c] += sum_t g[t,c].
// Block = 32 channels x 8 token lanes; each block owns a token range and reduces its dw / dbias
// contribution in shared memory before one atomic per (c, j).
__global__ void conv1d_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                  const float* __restrict__ w, const float* __restrict__ bias,
                                  const int* __restrict__ seq_of, const int* __restrict__ cu,
                                  __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, float* __restrict__ dbias,
                                  int T, int C, int K, int act, int tokens_per_block) {
  const int c = blockIdx.x * 32 + (threadIdx.x & 31);
  const int tl = threadIdx.x >> 5;  // 0..7
  const int t_begin = blockIdx.y * tokens_per_block;
  const int t_end = min(T, t_begin + tokens_per_block);
  __shared__ float s_dw[8][32][8];  // [token lane][channel][j], K <= 7 plus bias slot
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (c < C) {
    auto g_at = [&](int t) -> float {  // gradient at the conv output (before the activation)
      float g = __bfloat162float(dy[static_cast<long long>(t) * C + c]);
      if (act) {
        const int s0 = cu[seq_of[t]];
        float pre = bias ? bias[c] : 0.f;
        for (int j = 0; j < K; ++j) {
          const int tt = t - (K - 1) + j;
          if (tt >= s0) pre += w[c * K + j] * __bfloat162float(x[static_cast<long long>(tt) * C + c]);
        }
        g *= dsilu_f(pre);
      }
      return g;
    };
    for (int t = t_begin + tl; t < t_end; t += 8) {
      const int sid = seq_of[t];
      const int s0 = cu[sid], s1 = cu[sid + 1];
      float d = 0.f;
      for (int j = 0; j < K; ++j) {
        const int tt = t + (K - 1) - j;  // outputs that read x[t] through tap j
        if (tt < s1) d += w[c * K + j] * g_at(tt);
      }
      dx[static_cast<long long>(t) * C + c] = __float2bfloat16(d);
      const float g = g_at(t);
      for (int j = 0; j < K; ++j) {
        const int tt = t - (K - 1) + j;
        if (tt >= s0) acc[j] += g * __bfloat162float(x[static_cast<long long>(tt) * C + c]);
      }
      acc[7] += g;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) s_dw[tl][threadIdx.x & 31][j] = acc[j];
  __syncthreads();
  if (tl == 0 && c < C) {
    for (int j = 0; j < 8; ++j) {
      float s = 0.f;
      for (int l = 0; l < 8; ++l) s += s_dw[l][threadIdx.x][j];
      if (j < K) atomicAdd(&dw[c * K + j], s);
      else if (j == 7 && dbias) atomicAdd(&dbias[c], s);
    }
  }
}

// Recurrent linear attention, one CTA per (sequence, head); state S [DK, DV] fp32 in shared memory.
//   mode 0 (simple GLA):        S = a_t * S + k_t v_t^T
//   mode 1 (gated delta rule):  S = a_t * S;  u = S^T k_t;  S += b_t * k_t (v_t - u)^T
//   o_t = scale * S^T q_t
// q, k: [T, H, DK]; v, o: [T, H, DV]; a (decay, already exp'ed, in (0, 1]) and b: [T, H] fp32.
// Thread j < DV owns column j of S (DK registers-worth of shared memory reads per step).
template <int DK>
__global__ void linear_attn_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                       const __nv_bfloat16* __restrict__ v, const float* __restrict__ a,
                                       const float* __restrict__ b, const int* __restrict__ cu,
                                       __nv_bfloat16* __restrict__ o, float* __restrict__ final_state, int H, int DV,
                                       float scale, int mode) {
  extern __shared__ float sm[];  // S [DK][DV] then k_t [DK], q_t [DK]
  float* S = sm;
  float* ks = sm + DK * DV;
  float* qs = ks + DK;
  const int seq = blockIdx.x, h = blockIdx.y;
  const int t0 = cu[seq], t1 = cu[seq + 1];
  const int j = threadIdx.x;  // column of S / output dim
  for (int i = threadIdx.x; i < DK * DV; i += blockDim.x) S[i] = 0.f;
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const long long qk_off = (static_cast<long long>(t) * H + h) * DK;
    for (int i = threadIdx.x; i < DK; i += blockDim.x) {
      ks[i] = __bfloat162float(k[qk_off + i]);
      qs[i] = __bfloat162float(q[qk_off + i]);
    }
    __syncthreads();
    if (j < DV) {
      const float at = a[static_cast<long long>(t) * H + h];
      const float vt = __bfloat162float(v[(static_cast<long long>(t) * H + h) * DV + j]);
      float out = 0.f;
      if (mode == 0) {
#pragma unroll 8
        for (int i = 0; i < DK; ++i) {
          const float s = at * S[i * DV + j] + ks[i] * vt;
          S[i * DV + j] = s;
          out += s * qs[i];
        }
      } else {
        const float bt = b[static_cast<long long>(t) * H + h];
        float u = 0.f;
#pragma unroll 8
        for (int i = 0; i < DK; ++i) u += at * S[i * DV + j] * ks[i];
        const float d = bt * (vt - u);
#pragma unroll 8
        for (int i = 0; i < DK; ++i) {
          const float s = at * S[i * DV + j] + ks[i] * d;
          S[i * DV + j] = s;
          out += s * qs[i];
        }
      }
      o[(static_cast<long long>(t) * H + h) * DV + j] = __float2bfloat16(out * scale);
    }
    __syncthreads();
  }
  if (final_state)
    for (int i = threadIdx.x; i < DK * DV; i += blockDim.x)
      final_state[(static_cast<long long>(seq) * H + h) * DK * DV + i] = S[i];
}

}  // namespace b200

extern "C" {

int b200_causal_conv1d_fwd(const void* x, const float* w, const float* bias, const int* seq_of, const int* cu, void* y,
                           int T, int C, int K, int act, cudaStream_t stream) {
  using namespace b200;
  if (K < 1 || K > 7) return -100;
  if (T == 0) return 0;
  const long long n = static_cast<long long>(T) * C;
  conv1d_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)x, w, bias, seq_of, cu,
                                                                     (__nv_bfloat16*)y, T, C, K, act);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// dw [C, K] and dbias [C] (may be null) are accumulated into: zero them first for plain gradients.
int b200_causal_conv1d_bwd(const void* x, const void* dy, const float* w, const float* bias, const int* seq_of,
                           const int* cu, void* dx, float* dw, float* dbias, int T, int C, int K, int act,
                           cudaStream_t stream) {
  using namespace b200;
  if (K < 1 || K > 7) return -100;
  if (T == 0) return 0;
  const int tpb = 256;
  dim3 grid((C + 31) / 32, (T + tpb - 1) / tpb);
  conv1d_bwd_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, w, bias, seq_of, cu,
                                              (__nv_bfloat16*)dx, dw, dbias, T, C, K, act, tpb);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// final_state: fp32 [n_seq, H, DK, DV] or null. DK in {64, 128}; DV <= 256.
int b200_linear_attn_fwd(const void* q, const void* k, const void* v, const float* a, const float* b, const int* cu,
                         void* o, float* final_state, int n_seq, int H, int DK, int DV, float scale, int mode,
                         cudaStream_t stream) {
  using namespace b200;
  if (n_seq == 0) return 0;
  if (DV > 256 || (mode == 1 && b == nullptr)) return -100;
  const size_t smem = (static_cast<size_t>(DK) * DV + 2 * DK) * sizeof(float);
  dim3 grid(n_seq, H);
  const int threads = ((DV + 31) / 32) * 32;
#define LA(DK_)                                                                                                  \
  cudaFuncSetAttribute(linear_attn_fwd_kernel<DK_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
  linear_attn_fwd_kernel<DK_><<<grid, threads, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, \
                                                               (const __nv_bfloat16*)v, a, b, cu,               \
                                                               (__nv_bfloat16*)o, final_state, H, DV, scale, mode)
  if (DK == 64) { LA(64); }
  else if (DK == 128) { LA(128); }
  else return -101;
#undef LA
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
