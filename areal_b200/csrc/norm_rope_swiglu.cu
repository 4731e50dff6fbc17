// Memory-bound transformer glue for sm_100a: RMSNorm (+ fused residual add),
// per-head q/k RMSNorm fused with rotary embedding, and SwiGLU, each with its
// backward. All kernels move 16-byte vectors, keep a row in registers between
// the reduction and the write, and accumulate in fp32.
//
// Replaces the eager / Inductor-fused RMSNorm, rotate_half RoPE and SiLU*mul of
// the reference models (areal/experimental/models/archon/qwen3/model/model.py:75-101,
// 103-293; qwen2/model/rope.py).
#include <cstdio>
#include <mutex>

#include "norm_static_scratch.h"
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/host_utils.h"

namespace b200 {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct alignas(16) BF8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void bf8_to_float(const BF8& b, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(b.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ BF8 float_to_bf8(const float* f) {
  BF8 b;
#pragma unroll
  for (int i = 0; i < 4; ++i) b.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return b;
}

// ------------------------------------------------------------------ RMSNorm --
// One warp per row; a lane holds NV 16-byte vectors (8 bf16 each), so the row
// (H = 256 * NV elements at most) is read once.
template <int NV>
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ res,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd,
                                   int T, int H, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
       row < T; row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const BF8* xr = reinterpret_cast<const BF8*>(x + row * H);
    const BF8* rr = res ? reinterpret_cast<const BF8*>(res + row * H) : nullptr;
    float v[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        bf8_to_float(xr[c], v[i]);
        if (rr) {
          float r[8];
          bf8_to_float(rr[c], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += r[j];
          // the residual stream is kept in bf16: normalise what is stored
          BF8 h = float_to_bf8(v[i]);
          reinterpret_cast<BF8*>(res_out + row * H)[c] = h;
          bf8_to_float(h, v[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / H + eps);
    if (lane == 0 && rstd) rstd[row] = rs;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        float wv[8];
        bf8_to_float(reinterpret_cast<const BF8*>(w)[c], wv);
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rs * wv[j];
        reinterpret_cast<BF8*>(y + row * H)[c] = float_to_bf8(o);
      }
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres); dw partial per block.
template <int NV>
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                   const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w,
                                   const float* __restrict__ rstd,
                                   const __nv_bfloat16* __restrict__ dres,
                                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial,
                                   int T, int H) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nvec = H >> 3;
  float dwacc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  float wv[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) bf8_to_float(reinterpret_cast<const BF8*>(w)[c], wv[i]);
  }
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_block + warp; row < T;
       row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const float rs = rstd[row];
    float g[NV][8], xh[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        bf8_to_float(reinterpret_cast<const BF8*>(dy + row * H)[c], g[i]);
        bf8_to_float(reinterpret_cast<const BF8*>(x + row * H)[c], xh[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rs;
          dwacc[i][j] += g[i][j] * xh[i][j];
          g[i][j] *= wv[i][j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    dot = warp_sum(dot) / H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (g[i][j] - xh[i][j] * dot);
        if (dres) {
          float r[8];
          bf8_to_float(reinterpret_cast<const BF8*>(dres + row * H)[c], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        reinterpret_cast<BF8*>(dx + row * H)[c] = float_to_bf8(o);
      }
    }
  }
  // reduce the per-warp dw accumulators across the block through shared memory
  extern __shared__ float sm[];  // [warps][H]
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec)
#pragma unroll
      for (int j = 0; j < 8; ++j) sm[warp * H + c * 8 + j] = dwacc[i][j];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float s = 0.f;
    for (int wi = 0; wi < warps_per_block; ++wi) s += sm[wi * H + c];
    dw_partial[static_cast<long long>(blockIdx.x) * H + c] = s;
  }
}

__global__ void colsum_partials_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                       int nblocks, int H, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[static_cast<long long>(b) * H + c];
  out[c] = accumulate ? out[c] + s : s;
}

// ------------------------------------------------------- q/k norm + RoPE ----
// qkv: [T, (Hq + 2*Hkv) * D] bf16 (q heads, then k heads, then v heads).
// One warp per (token, head) over the q and k heads; D == 128 (lane owns the
// pairs j = 2*lane, 2*lane+1 and their partners j + 64).
__global__ void qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv,
                                       const __nv_bfloat16* __restrict__ qw,
                                       const __nv_bfloat16* __restrict__ kw,
                                       const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t,
                                       const int* __restrict__ pos, __nv_bfloat16* __restrict__ q_out,
                                       __nv_bfloat16* __restrict__ k_out, float* __restrict__ rstd_out,
                                       int T, int Hq, int Hkv, float eps, int has_norm) {
  constexpr int D = 128;
  const int lane = threadIdx.x & 31;
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int heads = Hq + Hkv;
  if (gw >= static_cast<long long>(T) * heads) return;
  const int t = static_cast<int>(gw / heads);
  const int h = static_cast<int>(gw % heads);
  const long long row_stride = static_cast<long long>(Hq + 2 * Hkv) * D;
  const __nv_bfloat16* src = qkv + t * row_stride + static_cast<long long>(h) * D;
  const bool is_q = h < Hq;
  const __nv_bfloat16* w = is_q ? qw : kw;
  __nv_bfloat16* dst = is_q ? q_out + (static_cast<long long>(t) * Hq + h) * D
                            : k_out + (static_cast<long long>(t) * Hkv + (h - Hq)) * D;
  float2 a = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src)[lane]);
  float2 b = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src + 64)[lane]);
  if (has_norm) {
    float ss = warp_sum(a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y);
    const float rs = rsqrtf(ss / D + eps);
    if (lane == 0) rstd_out[gw] = rs;
    float2 wa = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(w)[lane]);
    float2 wb = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(w + 64)[lane]);
    // match the reference's rounding: the normalised value is cast to bf16 before RoPE
    a.x = __bfloat162float(__float2bfloat16(a.x * rs * wa.x));
    a.y = __bfloat162float(__float2bfloat16(a.y * rs * wa.y));
    b.x = __bfloat162float(__float2bfloat16(b.x * rs * wb.x));
    b.y = __bfloat162float(__float2bfloat16(b.y * rs * wb.y));
  }
  const int p = pos[t];
  const float2 c = reinterpret_cast<const float2*>(cos_t + static_cast<long long>(p) * 64)[lane];
  const float2 s = reinterpret_cast<const float2*>(sin_t + static_cast<long long>(p) * 64)[lane];
  float2 oa, ob;
  oa.x = a.x * c.x - b.x * s.x;
  oa.y = a.y * c.y - b.y * s.y;
  ob.x = b.x * c.x + a.x * s.x;
  ob.y = b.y * c.y + a.y * s.y;
  reinterpret_cast<__nv_bfloat162*>(dst)[lane] = __floats2bfloat162_rn(oa.x, oa.y);
  reinterpret_cast<__nv_bfloat162*>(dst + 64)[lane] = __floats2bfloat162_rn(ob.x, ob.y);
}

// Decode / prefill form of the kernel above: q is written out as before, k goes straight into the
// paged K cache and v is copied into the paged V cache (`[page, kv head, slot in page, D]`), so the
// separate cache-write launch disappears. One warp per (token, head) over q, k AND v heads.
// slot_mapping[t] = page * block_size + offset, negative to skip the token's cache write.
__global__ void qknorm_rope_kvwrite_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ qw,
                                           const __nv_bfloat16* __restrict__ kw, const float* __restrict__ cos_t,
                                           const float* __restrict__ sin_t, const int* __restrict__ pos,
                                           __nv_bfloat16* __restrict__ q_out,
                                           const long long* __restrict__ slot_mapping,
                                           __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                           int T, int Hq, int Hkv, int block_size, float eps, int has_norm) {
  constexpr int D = 128;
  const int lane = threadIdx.x & 31;
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int heads = Hq + 2 * Hkv;
  if (gw >= static_cast<long long>(T) * heads) return;
  const int t = static_cast<int>(gw / heads);
  const int h = static_cast<int>(gw % heads);
  const __nv_bfloat16* src = qkv + (static_cast<long long>(t) * heads + h) * D;
  const bool is_q = h < Hq;
  const bool is_v = h >= Hq + Hkv;
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out + (static_cast<long long>(t) * Hq + h) * D;
  } else {
    const long long slot = slot_mapping[t];
    if (slot < 0) return;
    const long long blk = slot / block_size, off = slot % block_size;
    const int hk = is_v ? h - Hq - Hkv : h - Hq;
    dst = (is_v ? v_cache : k_cache) + ((blk * Hkv + hk) * block_size + off) * D;
  }
  if (is_v) {
    reinterpret_cast<uint2*>(dst)[lane] = reinterpret_cast<const uint2*>(src)[lane];
    return;
  }
  const __nv_bfloat16* w = is_q ? qw : kw;
  float2 a = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src)[lane]);
  float2 b = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src + 64)[lane]);
  if (has_norm) {
    float ss = warp_sum(a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y);
    const float rs = rsqrtf(ss / D + eps);
    float2 wa = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(w)[lane]);
    float2 wb = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(w + 64)[lane]);
    a.x = __bfloat162float(__float2bfloat16(a.x * rs * wa.x));
    a.y = __bfloat162float(__float2bfloat16(a.y * rs * wa.y));
    b.x = __bfloat162float(__float2bfloat16(b.x * rs * wb.x));
    b.y = __bfloat162float(__float2bfloat16(b.y * rs * wb.y));
  }
  const int p = pos[t];
  const float2 c = reinterpret_cast<const float2*>(cos_t + static_cast<long long>(p) * 64)[lane];
  const float2 s = reinterpret_cast<const float2*>(sin_t + static_cast<long long>(p) * 64)[lane];
  float2 oa, ob;
  oa.x = a.x * c.x - b.x * s.x;
  oa.y = a.y * c.y - b.y * s.y;
  ob.x = b.x * c.x + a.x * s.x;
  ob.y = b.y * c.y + a.y * s.y;
  reinterpret_cast<__nv_bfloat162*>(dst)[lane] = __floats2bfloat162_rn(oa.x, oa.y);
  reinterpret_cast<__nv_bfloat162*>(dst + 64)[lane] = __floats2bfloat162_rn(ob.x, ob.y);
}

// Backward: un-rotate dq/dk, then per-head RMSNorm backward; writes into the
// q and k slots of dqkv and accumulates dqw / dkw [D] with atomics (fp32).
__global__ void qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dq,
                                       const __nv_bfloat16* __restrict__ dk,
                                       const __nv_bfloat16* __restrict__ qkv,
                                       const __nv_bfloat16* __restrict__ qw,
                                       const __nv_bfloat16* __restrict__ kw,
                                       const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t,
                                       const int* __restrict__ pos, const float* __restrict__ rstd,
                                       __nv_bfloat16* __restrict__ dqkv, float* __restrict__ dqw,
                                       float* __restrict__ dkw, int T, int Hq, int Hkv, int has_norm) {
  constexpr int D = 128;
  __shared__ float s_dw[2][D];
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) (&s_dw[0][0])[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int heads = Hq + Hkv;
  if (gw < static_cast<long long>(T) * heads) {
    const int t = static_cast<int>(gw / heads);
    const int h = static_cast<int>(gw % heads);
    const bool is_q = h < Hq;
    const long long row_stride = static_cast<long long>(Hq + 2 * Hkv) * D;
    const __nv_bfloat16* g = is_q ? dq + (static_cast<long long>(t) * Hq + h) * D
                                  : dk + (static_cast<long long>(t) * Hkv + (h - Hq)) * D;
    float2 ga = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(g)[lane]);
    float2 gb = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(g + 64)[lane]);
    const int p = pos[t];
    const float2 c = reinterpret_cast<const float2*>(cos_t + static_cast<long long>(p) * 64)[lane];
    const float2 s = reinterpret_cast<const float2*>(sin_t + static_cast<long long>(p) * 64)[lane];
    // transpose of the rotation
    float2 da, db;
    da.x = ga.x * c.x + gb.x * s.x;
    da.y = ga.y * c.y + gb.y * s.y;
    db.x = gb.x * c.x - ga.x * s.x;
    db.y = gb.y * c.y - ga.y * s.y;
    __nv_bfloat16* out = dqkv + t * row_stride + static_cast<long long>(h) * D;
    if (has_norm) {
      const __nv_bfloat16* src = qkv + t * row_stride + static_cast<long long>(h) * D;
      const __nv_bfloat16* w = is_q ? qw : kw;
      float2 xa = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src)[lane]);
      float2 xb = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src + 64)[lane]);
      float2 wa = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(w)[lane]);
      float2 wb = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(w + 64)[lane]);
      const float rs = rstd[gw];
      xa.x *= rs; xa.y *= rs; xb.x *= rs; xb.y *= rs;
      float* sw = s_dw[is_q ? 0 : 1];
      atomicAdd(&sw[2 * lane], da.x * xa.x);
      atomicAdd(&sw[2 * lane + 1], da.y * xa.y);
      atomicAdd(&sw[64 + 2 * lane], db.x * xb.x);
      atomicAdd(&sw[64 + 2 * lane + 1], db.y * xb.y);
      da.x *= wa.x; da.y *= wa.y; db.x *= wb.x; db.y *= wb.y;
      float dot = warp_sum(da.x * xa.x + da.y * xa.y + db.x * xb.x + db.y * xb.y) / D;
      da.x = rs * (da.x - xa.x * dot);
      da.y = rs * (da.y - xa.y * dot);
      db.x = rs * (db.x - xb.x * dot);
      db.y = rs * (db.y - xb.y * dot);
    }
    reinterpret_cast<__nv_bfloat162*>(out)[lane] = __floats2bfloat162_rn(da.x, da.y);
    reinterpret_cast<__nv_bfloat162*>(out + 64)[lane] = __floats2bfloat162_rn(db.x, db.y);
  }
  if (has_norm) {
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      if (s_dw[0][i] != 0.f) atomicAdd(&dqw[i], s_dw[0][i]);
      if (s_dw[1][i] != 0.f) atomicAdd(&dkw[i], s_dw[1][i]);
    }
  }
}

// ------------------------------------------------------------------- SwiGLU --
// gu: [T, 2*I] (gate = first I columns, up = last I columns); out: [T, I].
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ out, long long T, int I) {
  const int nvec = I >> 3;
  const long long total = T * nvec;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / nvec;
    const int c = static_cast<int>(i % nvec);
    float g[8], u[8], o[8];
    bf8_to_float(reinterpret_cast<const BF8*>(gu + t * 2 * I)[c], g);
    bf8_to_float(reinterpret_cast<const BF8*>(gu + t * 2 * I + I)[c], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    reinterpret_cast<BF8*>(out + t * I)[c] = float_to_bf8(o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                  const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int I) {
  const int nvec = I >> 3;
  const long long total = T * nvec;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / nvec;
    const int c = static_cast<int>(i % nvec);
    float g[8], u[8], d[8], dg[8], du[8];
    bf8_to_float(reinterpret_cast<const BF8*>(gu + t * 2 * I)[c], g);
    bf8_to_float(reinterpret_cast<const BF8*>(gu + t * 2 * I + I)[c], u);
    bf8_to_float(reinterpret_cast<const BF8*>(dy + t * I)[c], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (sg * (1.f + g[j] * (1.f - sg)));
    }
    reinterpret_cast<BF8*>(dgu + t * 2 * I)[c] = float_to_bf8(dg);
    reinterpret_cast<BF8*>(dgu + t * 2 * I + I)[c] = float_to_bf8(du);
  }
}

template <typename F>
static int dispatch_nv(int H, F&& f) {
  const int nv = (H / 8 + 31) / 32;
  if (nv <= 1) return f(std::integral_constant<int, 1>{});
  if (nv <= 2) return f(std::integral_constant<int, 2>{});
  if (nv <= 4) return f(std::integral_constant<int, 4>{});
  if (nv <= 8) return f(std::integral_constant<int, 8>{});
  if (nv <= 16) return f(std::integral_constant<int, 16>{});
  if (nv <= 32) return f(std::integral_constant<int, 32>{});
  return -101;
}

}  // namespace b200

extern "C" {

// H must be a multiple of 8 and at most 8192. res/res_out/rstd may be null.
int b200_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out,
                     float* rstd, int T, int H, float eps, cudaStream_t stream) {
  using namespace b200;
  if (T == 0) return 0;
  if (H % 8) return -100;
  const int wpb = 4;
  int grid = (T + wpb - 1) / wpb;
  const int maxg = sm_count() * 16;
  if (grid > maxg) grid = maxg;
  int rc = dispatch_nv(H, [&](auto nv) {
    rmsnorm_fwd_kernel<decltype(nv)::value><<<grid, wpb * 32, 0, stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w,
        (__nv_bfloat16*)y, (__nv_bfloat16*)res_out, rstd, T, H, eps);
    return 0;
  });
  if (rc) return rc;
  B200_CHECK(cudaGetLastError());
  return 0;
}

// dw_partial: scratch of at least b200_rmsnorm_bwd_blocks(T) * H floats.
int b200_rmsnorm_bwd_blocks(int T) {
  int grid = (T + 3) / 4;
  const int maxg = b200::sm_count() * 2;
  return grid > maxg ? maxg : grid;
}
int b200_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                     const void* dres, void* dx, float* dw_partial, float* dw, int dw_accumulate,
                     int T, int H, cudaStream_t stream) {
  using namespace b200;
  if (T == 0) return 0;
  if (H % 8) return -100;
  const int wpb = 4;
  const int grid = b200_rmsnorm_bwd_blocks(T);
  const size_t smem = static_cast<size_t>(wpb) * H * sizeof(float);
  int rc = dispatch_nv(H, [&](auto nv) {
    auto k = rmsnorm_bwd_kernel<decltype(nv)::value>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<grid, wpb * 32, smem, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                        (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,
                                        (__nv_bfloat16*)dx, dw_partial, T, H);
    return 0;
  });
  if (rc) return rc;
  colsum_partials_kernel<<<(H + 255) / 256, 256, 0, stream>>>(dw_partial, dw, grid, H,
                                                              dw_accumulate);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_qknorm_rope_fwd(const void* qkv, const void* qw, const void* kw, const float* cos_t,
                         const float* sin_t, const int* pos, void* q_out, void* k_out,
                         float* rstd, int T, int Hq, int Hkv, int D, float eps, int has_norm,
                         cudaStream_t stream) {
  using namespace b200;
  if (D != 128) return -100;
  if (T == 0) return 0;
  const long long warps = static_cast<long long>(T) * (Hq + Hkv);
  const int tpb = 256;
  const long long grid = (warps * 32 + tpb - 1) / tpb;
  qknorm_rope_fwd_kernel<<<(unsigned)grid, tpb, 0, stream>>>(
      (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, cos_t, sin_t,
      pos, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, rstd, T, Hq, Hkv, eps, has_norm);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// q/k norm + RoPE of a fused qkv projection whose k and v go straight into the paged KV caches
// ([num_blocks, Hkv, block_size, 128] bf16) at slot_mapping[t] (int64; negative = skip).
int b200_qknorm_rope_kvwrite(const void* qkv, const void* qw, const void* kw, const float* cos_t,
                             const float* sin_t, const int* pos, void* q_out, const long long* slot_mapping,
                             void* k_cache, void* v_cache, int T, int Hq, int Hkv, int D, int block_size,
                             float eps, int has_norm, cudaStream_t stream) {
  using namespace b200;
  if (D != 128) return -100;
  if (T == 0) return 0;
  const long long warps = static_cast<long long>(T) * (Hq + 2 * Hkv);
  const int tpb = 256;
  const long long grid = (warps * 32 + tpb - 1) / tpb;
  qknorm_rope_kvwrite_kernel<<<(unsigned)grid, tpb, 0, stream>>>(
      (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, cos_t, sin_t, pos,
      (__nv_bfloat16*)q_out, slot_mapping, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, T, Hq, Hkv,
      block_size, eps, has_norm);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// dqw/dkw are fp32 [D] accumulators (added to, not overwritten).
int b200_qknorm_rope_bwd(const void* dq, const void* dk, const void* qkv, const void* qw,
                         const void* kw, const float* cos_t, const float* sin_t, const int* pos,
                         const float* rstd, void* dqkv, float* dqw, float* dkw, int T, int Hq,
                         int Hkv, int D, int has_norm, cudaStream_t stream) {
  using namespace b200;
  if (D != 128) return -100;
  if (T == 0) return 0;
  const long long warps = static_cast<long long>(T) * (Hq + Hkv);
  const int tpb = 256;
  const long long grid = (warps * 32 + tpb - 1) / tpb;
  qknorm_rope_bwd_kernel<<<(unsigned)grid, tpb, 0, stream>>>(
      (const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)qkv,
      (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, cos_t, sin_t, pos, rstd,
      (__nv_bfloat16*)dqkv, dqw, dkw, T, Hq, Hkv, has_norm);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_swiglu_fwd(const void* gu, void* out, long long T, int I, cudaStream_t stream) {
  using namespace b200;
  if (T == 0) return 0;
  if (I % 8) return -100;
  long long total = T * (I / 8);
  long long grid = (total + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 16;
  if (grid > maxg) grid = maxg;
  swiglu_fwd_kernel<<<(unsigned)grid, 256, 0, stream>>>((const __nv_bfloat16*)gu,
                                                        (__nv_bfloat16*)out, T, I);
  B200_CHECK(cudaGetLastError());
  return 0;
}
int b200_swiglu_bwd(const void* dy, const void* gu, void* dgu, long long T, int I,
                    cudaStream_t stream) {
  using namespace b200;
  if (T == 0) return 0;
  if (I % 8) return -100;
  long long total = T * (I / 8);
  long long grid = (total + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 16;
  if (grid > maxg) grid = maxg;
  swiglu_bwd_kernel<<<(unsigned)grid, 256, 0, stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, T, I);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"

// ------------------------------------------ RMSNorm backward, built-in scratch ----
// See norm_static_scratch.h. The partial sums of dw go to a file-scope device array
// whose address is looked up once per device; nothing here allocates.
namespace b200 {
static __device__ __align__(256) float g_rmsnorm_bwd_scratch[static_cast<size_t>(B200_RMSNORM_STATIC_MAX_BLOCKS) *
                                                             B200_RMSNORM_STATIC_MAX_H];
constexpr int kMaxDevices = 64;
static std::mutex g_scratch_mu;
static float* g_scratch_ptr[kMaxDevices] = {};
}  // namespace b200

extern "C" int b200_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd,
                                       const void* dres, void* dx, float* dw, int dw_accumulate, int T, int H,
                                       cudaStream_t stream) {
  using namespace b200;
  if (T == 0) return 0;
  if (H % 8) return -100;
  const int grid = b200_rmsnorm_bwd_blocks(T);
  if (H > B200_RMSNORM_STATIC_MAX_H || grid > B200_RMSNORM_STATIC_MAX_BLOCKS) {
    fprintf(stderr,
            "b200_rmsnorm_bwd_static: H=%d (max %d) or %d blocks (max %d) exceeds the built-in scratch; "
            "use b200_rmsnorm_bwd with a caller-provided buffer\n",
            H, B200_RMSNORM_STATIC_MAX_H, grid, B200_RMSNORM_STATIC_MAX_BLOCKS);
    return B200_ERR_STATIC_SCRATCH_TOO_SMALL;
  }
  int dev = 0;
  B200_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return -3;
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (!g_scratch_ptr[dev]) {
      // the array's name is only meaningful in device code; ask the runtime for its address on
      // the current device
      float* p = nullptr;
      B200_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rmsnorm_bwd_scratch));
      g_scratch_ptr[dev] = p;
    }
    scratch = g_scratch_ptr[dev];
  }
  const int wpb = 4;
  const size_t smem = static_cast<size_t>(wpb) * H * sizeof(float);
  int rc = dispatch_nv(H, [&](auto nv) {
    auto k = rmsnorm_bwd_kernel<decltype(nv)::value>;
    if (smem > 48 * 1024)
      B200_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k<<<grid, wpb * 32, smem, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                        rstd, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, scratch, T, H);
    B200_CHECK(cudaGetLastError());
    return 0;
  });
  if (rc) return rc;
  colsum_partials_kernel<<<(H + 255) / 256, 256, 0, stream>>>(scratch, dw, grid, H, dw_accumulate);
  B200_CHECK(cudaGetLastError());
  return 0;
}
