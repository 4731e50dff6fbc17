// Flat-buffer optimizer kernels for the sharded (ZeRO-style) train engine.
//
// The engine keeps fp32 main gradients in one flat buffer per rank and fp32
// master weights + Adam moments for the rank's shard only. A step is
//   1. reduce_scatter_sumsq : shard = scale * sum_p grads_p[shard range]   (peer loads over NVLink)
//                             + sum of squares of the reduced shard       (for the global norm)
//   2. (tiny all-reduce of the per-rank sums of squares)
//   3. adamw_bcast          : clip by the global norm, AdamW on the shard,
//                             cast to bf16 and store the new weights into
//                             every rank's parameter buffer (peer stores).
// so the reduce-scatter, the fp32 cast/scale, grad-norm, clipping, AdamW and
// the parameter all-gather are two kernels with no intermediate buffers.
// A non-finite norm skips the update (the reference skips the step likewise,
// areal/engine/fsdp_engine.py:682-713).
//
// Replaces FSDP2's NCCL reduce-scatter / all-gather plus torch's fused AdamW
// and multi_tensor_l2norm (areal/engine/fsdp_utils/grad.py:89-281).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/host_utils.h"

namespace b200 {

constexpr int kMaxPeers = 16;
struct PeerPtrs {
  void* p[kMaxPeers];
};

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float red[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  v = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  }
  return v;
}

// out[i] = scale * sum_p peers[p][offset + i], i in [0, n); sumsq += sum out[i]^2.
__global__ void reduce_scatter_sumsq_kernel(PeerPtrs peers, int n_peers, long long offset,
                                            long long n, float scale, float* __restrict__ out,
                                            float* __restrict__ sumsq) {
  float ss = 0.f;
  const long long n4 = n >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int p = 0; p < n_peers; ++p) {
      const float4 v = reinterpret_cast<const float4*>(
          reinterpret_cast<const float*>(peers.p[p]) + offset)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    reinterpret_cast<float4*>(out)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  for (long long i = (n4 << 2) + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
       i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float a = 0.f;
    for (int p = 0; p < n_peers; ++p) a += reinterpret_cast<const float*>(peers.p[p])[offset + i];
    a *= scale;
    out[i] = a;
    ss += a * a;
  }
  ss = block_sum(ss);
  if (threadIdx.x == 0) atomicAdd(sumsq, ss);
}

struct AdamParams {
  float lr, beta1, beta2, eps, weight_decay;
  float bias_corr1, bias_corr2;  // 1 - beta^t
  float max_norm;                // <= 0: no clipping
};

// AdamW on a shard; the updated weights are written (bf16) at `offset` into
// each of the n_peers parameter buffers. norm_sq points to the global squared
// gradient norm (already summed over ranks).
__global__ void adamw_bcast_kernel(float* __restrict__ master, float* __restrict__ m,
                                   float* __restrict__ v, const float* __restrict__ grad,
                                   PeerPtrs params, int n_peers, long long offset, long long n,
                                   const float* __restrict__ norm_sq, AdamParams hp,
                                   int* __restrict__ skipped) {
  const float nsq = norm_sq ? *norm_sq : 0.f;
  if (!isfinite(nsq)) {
    if (blockIdx.x == 0 && threadIdx.x == 0 && skipped) *skipped = 1;
    return;
  }
  float coef = 1.f;
  if (hp.max_norm > 0.f) coef = fminf(1.f, hp.max_norm / (sqrtf(nsq) + 1e-6f));
  const float step = hp.lr / hp.bias_corr1;
  const float inv_bc2_sqrt = rsqrtf(hp.bias_corr2);
  const long long n4 = n >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 w4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    const float4 g4 = reinterpret_cast<const float4*>(grad)[i];
    float* w = &w4.x; float* mm = &m4.x; float* vv = &v4.x; const float* g = &g4.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = g[k] * coef;
      mm[k] = hp.beta1 * mm[k] + (1.f - hp.beta1) * gk;
      vv[k] = hp.beta2 * vv[k] + (1.f - hp.beta2) * gk * gk;
      const float denom = sqrtf(vv[k]) * inv_bc2_sqrt + hp.eps;
      w[k] = w[k] * (1.f - hp.lr * hp.weight_decay) - step * mm[k] / denom;
    }
    reinterpret_cast<float4*>(master)[i] = w4;
    reinterpret_cast<float4*>(m)[i] = m4;
    reinterpret_cast<float4*>(v)[i] = v4;
    uint2 pk;
    reinterpret_cast<__nv_bfloat162*>(&pk)[0] = __floats2bfloat162_rn(w4.x, w4.y);
    reinterpret_cast<__nv_bfloat162*>(&pk)[1] = __floats2bfloat162_rn(w4.z, w4.w);
    for (int p = 0; p < n_peers; ++p)
      reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(params.p[p]) + offset)[i] = pk;
  }
  for (long long i = (n4 << 2) + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
       i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float gk = grad[i] * coef;
    const float mk = hp.beta1 * m[i] + (1.f - hp.beta1) * gk;
    const float vk = hp.beta2 * v[i] + (1.f - hp.beta2) * gk * gk;
    const float denom = sqrtf(vk) * inv_bc2_sqrt + hp.eps;
    const float wk = master[i] * (1.f - hp.lr * hp.weight_decay) - step * mk / denom;
    m[i] = mk; v[i] = vk; master[i] = wk;
    for (int p = 0; p < n_peers; ++p)
      reinterpret_cast<__nv_bfloat16*>(params.p[p])[offset + i] = __float2bfloat16(wk);
  }
}

// AdamW with bf16 moments and no fp32 master copy: the weight shard is read from this rank's own
// bf16 parameter buffer and the rounding error of every update is carried in a bf16 Kahan
// compensation buffer (6 bytes of state per parameter instead of 12).
//   c += update;  w' = bf16(w + c);  c += w - w'
__global__ void adamw_bf16_bcast_kernel(const __nv_bfloat16* w_local,
                                        __nv_bfloat16* __restrict__ comp, __nv_bfloat16* __restrict__ m,
                                        __nv_bfloat16* __restrict__ v, const float* __restrict__ grad,
                                        PeerPtrs params, int n_peers, long long offset, long long n,
                                        const float* __restrict__ norm_sq, AdamParams hp,
                                        int* __restrict__ skipped) {
  const float nsq = norm_sq ? *norm_sq : 0.f;
  if (!isfinite(nsq)) {
    if (blockIdx.x == 0 && threadIdx.x == 0 && skipped) *skipped = 1;
    return;
  }
  float coef = 1.f;
  if (hp.max_norm > 0.f) coef = fminf(1.f, hp.max_norm / (sqrtf(nsq) + 1e-6f));
  const float step = hp.lr / hp.bias_corr1;
  const float inv_bc2_sqrt = rsqrtf(hp.bias_corr2);
  auto update = [&](float w, float gk, float& mk, float& vk, float& c) -> __nv_bfloat16 {
    gk *= coef;
    mk = hp.beta1 * mk + (1.f - hp.beta1) * gk;
    vk = hp.beta2 * vk + (1.f - hp.beta2) * gk * gk;
    const float denom = sqrtf(vk) * inv_bc2_sqrt + hp.eps;
    c = c - hp.lr * hp.weight_decay * w - step * mk / denom;
    const __nv_bfloat16 wn = __float2bfloat16(w + c);
    c += w - __bfloat162float(wn);
    return wn;
  };
  // 8 elements per thread: one 16-byte access per bf16 array, two per fp32 gradient (offset and the
  // shard's base pointers are 16-byte aligned: offset is a multiple of 8 elements in this path)
  const long long n8 = ((offset & 7) == 0) ? (n >> 3) : 0;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 w8 = reinterpret_cast<const uint4*>(w_local)[i];
    uint4 m8 = reinterpret_cast<uint4*>(m)[i];
    uint4 v8 = reinterpret_cast<uint4*>(v)[i];
    uint4 c8 = reinterpret_cast<uint4*>(comp)[i];
    const float4 g0 = reinterpret_cast<const float4*>(grad)[2 * i];
    const float4 g1 = reinterpret_cast<const float4*>(grad)[2 * i + 1];
    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    __nv_bfloat16* wb = reinterpret_cast<__nv_bfloat16*>(&w8);
    __nv_bfloat16* mb = reinterpret_cast<__nv_bfloat16*>(&m8);
    __nv_bfloat16* vb = reinterpret_cast<__nv_bfloat16*>(&v8);
    __nv_bfloat16* cb = reinterpret_cast<__nv_bfloat16*>(&c8);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float mk = __bfloat162float(mb[k]), vk = __bfloat162float(vb[k]), c = __bfloat162float(cb[k]);
      wb[k] = update(__bfloat162float(wb[k]), g[k], mk, vk, c);
      mb[k] = __float2bfloat16(mk);
      vb[k] = __float2bfloat16(vk);
      cb[k] = __float2bfloat16(c);
    }
    reinterpret_cast<uint4*>(m)[i] = m8;
    reinterpret_cast<uint4*>(v)[i] = v8;
    reinterpret_cast<uint4*>(comp)[i] = c8;
    for (int p = 0; p < n_peers; ++p)
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[p]) + offset)[i] = w8;
  }
  for (long long i = (n8 << 3) + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float mk = __bfloat162float(m[i]), vk = __bfloat162float(v[i]), c = __bfloat162float(comp[i]);
    const __nv_bfloat16 wn = update(__bfloat162float(w_local[i]), grad[i], mk, vk, c);
    m[i] = __float2bfloat16(mk);
    v[i] = __float2bfloat16(vk);
    comp[i] = __float2bfloat16(c);
    for (int p = 0; p < n_peers; ++p)
      reinterpret_cast<__nv_bfloat16*>(params.p[p])[offset + i] = wn;
  }
}

// Plain SGD with (coupled) weight decay on the fp32 master shard.
__global__ void sgd_bcast_kernel(float* __restrict__ master, const float* __restrict__ grad,
                                 PeerPtrs params, int n_peers, long long offset, long long n,
                                 const float* __restrict__ norm_sq, AdamParams hp,
                                 int* __restrict__ skipped) {
  const float nsq = norm_sq ? *norm_sq : 0.f;
  if (!isfinite(nsq)) {
    if (blockIdx.x == 0 && threadIdx.x == 0 && skipped) *skipped = 1;
    return;
  }
  float coef = 1.f;
  if (hp.max_norm > 0.f) coef = fminf(1.f, hp.max_norm / (sqrtf(nsq) + 1e-6f));
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float w = master[i];
    const float wn = w - hp.lr * (grad[i] * coef + hp.weight_decay * w);
    master[i] = wn;
    for (int p = 0; p < n_peers; ++p)
      reinterpret_cast<__nv_bfloat16*>(params.p[p])[offset + i] = __float2bfloat16(wn);
  }
}

__global__ void sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  float ss = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    ss += x[i] * x[i];
  ss = block_sum(ss);
  if (threadIdx.x == 0) atomicAdd(out, ss);
}

__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out,
                                   long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = __bfloat162float(in[i]);
}

static inline unsigned grid_for(long long n, int per_thread) {
  long long g = (n / per_thread + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 8;
  if (g > maxg) g = maxg;
  if (g < 1) g = 1;
  return static_cast<unsigned>(g);
}

}  // namespace b200

extern "C" {

// peer_grads: host array of n_peers device pointers (fp32 flat gradient
// buffers, this rank's own included). offset and n are in elements and offset
// must be a multiple of 4. sumsq is a device float that is added to.
int b200_reduce_scatter_sumsq(void* const* peer_grads, int n_peers, long long offset, long long n,
                              float scale, float* out, float* sumsq, cudaStream_t stream) {
  using namespace b200;
  if (n_peers < 1 || n_peers > kMaxPeers) return -100;
  if (offset & 3) return -101;
  if (n == 0) return 0;
  PeerPtrs pp;
  for (int i = 0; i < n_peers; ++i) pp.p[i] = peer_grads[i];
  reduce_scatter_sumsq_kernel<<<grid_for(n, 4), 256, 0, stream>>>(pp, n_peers, offset, n, scale,
                                                                  out, sumsq);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_adamw_bcast(float* master, float* m, float* v, const float* grad, void* const* peer_params,
                     int n_peers, long long offset, long long n, const float* norm_sq, float lr,
                     float beta1, float beta2, float eps, float weight_decay, float bias_corr1,
                     float bias_corr2, float max_norm, int* skipped, cudaStream_t stream) {
  using namespace b200;
  if (n_peers < 1 || n_peers > kMaxPeers) return -100;
  if (offset & 3) return -101;
  if (n == 0) return 0;
  PeerPtrs pp;
  for (int i = 0; i < n_peers; ++i) pp.p[i] = peer_params[i];
  AdamParams hp{lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, max_norm};
  adamw_bcast_kernel<<<grid_for(n, 4), 256, 0, stream>>>(master, m, v, grad, pp, n_peers, offset, n,
                                                         norm_sq, hp, skipped);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// mode 1: bf16 moments + Kahan compensation (w_local: this rank's bf16 weight shard; comp/m/v bf16).
int b200_adamw_bf16_bcast(const void* w_local, void* comp, void* m, void* v, const float* grad,
                          void* const* peer_params, int n_peers, long long offset, long long n,
                          const float* norm_sq, float lr, float beta1, float beta2, float eps,
                          float weight_decay, float bias_corr1, float bias_corr2, float max_norm,
                          int* skipped, cudaStream_t stream) {
  using namespace b200;
  if (n_peers < 1 || n_peers > kMaxPeers) return -100;
  if (n == 0) return 0;
  PeerPtrs pp;
  for (int i = 0; i < n_peers; ++i) pp.p[i] = peer_params[i];
  AdamParams hp{lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, max_norm};
  adamw_bf16_bcast_kernel<<<grid_for(n, 8), 256, 0, stream>>>(
      (const __nv_bfloat16*)w_local, (__nv_bfloat16*)comp, (__nv_bfloat16*)m, (__nv_bfloat16*)v, grad, pp,
      n_peers, offset, n, norm_sq, hp, skipped);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_sgd_bcast(float* master, const float* grad, void* const* peer_params, int n_peers,
                   long long offset, long long n, const float* norm_sq, float lr, float weight_decay,
                   float max_norm, int* skipped, cudaStream_t stream) {
  using namespace b200;
  if (n_peers < 1 || n_peers > kMaxPeers) return -100;
  if (n == 0) return 0;
  PeerPtrs pp;
  for (int i = 0; i < n_peers; ++i) pp.p[i] = peer_params[i];
  AdamParams hp{lr, 0.f, 0.f, 0.f, weight_decay, 1.f, 1.f, max_norm};
  sgd_bcast_kernel<<<grid_for(n, 2), 256, 0, stream>>>(master, grad, pp, n_peers, offset, n, norm_sq, hp,
                                                       skipped);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_sumsq_f32(const float* x, long long n, float* out, cudaStream_t stream) {
  using namespace b200;
  if (n == 0) return 0;
  sumsq_kernel<<<grid_for(n, 1), 256, 0, stream>>>(x, n, out);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_bf16_to_f32(const void* in, float* out, long long n, cudaStream_t stream) {
  using namespace b200;
  if (n == 0) return 0;
  bf16_to_f32_kernel<<<grid_for(n, 1), 256, 0, stream>>>((const __nv_bfloat16*)in, out, n);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
