// Rollout-engine kernels: paged-KV cache write and single-token (decode)
// attention over a paged cache with GQA and split-KV (flash-decoding).
//
// Cache layout: k_cache / v_cache [num_blocks, block_size, Hkv, 128] bf16.
// A sequence's pages are listed in block_table[seq, max_blocks].
// Decode attention is memory-bound (each K/V byte is used once per query head
// of the group), so it runs on CUDA cores: one CTA per (sequence, kv head,
// split); a group of 8 lanes owns one cached token (16 dims each, two 16-byte
// loads), a warp covers 4 tokens per step, all query heads of the GQA group
// share the loaded K/V. Partial (max, sum, acc) results of the splits are
// merged by a second small kernel.
//
// These replace the external inference server's decode path in the reference
// (SGLang / vLLM paged attention; areal/engine/sglang_remote.py).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "common/host_utils.h"

namespace b200 {

constexpr int kHD = 128;
constexpr int kMaxGroup = 8;

// slot_mapping[t] = block * block_size + offset (or < 0 to skip the token)
__global__ void kv_cache_write_kernel(const __nv_bfloat16* __restrict__ k,
                                      const __nv_bfloat16* __restrict__ v, long long ldk,
                                      long long ldv, const long long* __restrict__ slot_mapping,
                                      __nv_bfloat16* __restrict__ k_cache,
                                      __nv_bfloat16* __restrict__ v_cache, int T, int Hkv) {
  const int vec_per_tok = Hkv * kHD / 8;
  const long long total = static_cast<long long>(T) * vec_per_tok;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / vec_per_tok);
    const int c = static_cast<int>(i % vec_per_tok);
    const long long slot = slot_mapping[t];
    if (slot < 0) continue;
    reinterpret_cast<uint4*>(k_cache + slot * Hkv * kHD)[c] =
        reinterpret_cast<const uint4*>(k + t * ldk)[c];
    reinterpret_cast<uint4*>(v_cache + slot * Hkv * kHD)[c] =
        reinterpret_cast<const uint4*>(v + t * ldv)[c];
  }
}

// q: [B, Hq, 128]; partial outputs: o_part [B, Hq, nsplit, 128] fp32, ml_part [B, Hq, nsplit, 2].
//
// Bandwidth: K/V rows stream into shared memory through a 4-stage cp.async
// pipeline (32 tokens = 16 KB per stage, 64 KB per CTA, 3 CTAs per SM), so
// ~190 KB per SM are in flight regardless of register pressure. The softmax
// running max is only raised when a score exceeds it by 2^8 (lazy rescaling),
// which removes the per-token rescale multiplies from the common path.
constexpr int kTok = 32;      // tokens per pipeline stage
constexpr int kStagesD = 4;
constexpr int kRowB = 256;    // bytes of one K (or V) row of one kv head
constexpr int kStageB = 2 * kTok * kRowB;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                   static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(gsrc)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int G>
__global__ void __launch_bounds__(128, (G <= 2 ? 3 : (G <= 4 ? 2 : 1)))
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                    const int* __restrict__ seq_lens, float* __restrict__ o_part,
                    float* __restrict__ ml_part, int Hq, int Hkv, int block_size, int max_blocks,
                    int nsplit, float scale_log2) {
  extern __shared__ __align__(16) uint8_t dsm[];  // kStagesD stages of [K 32x256B | V 32x256B]
  const int b = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int L = seq_lens[b];
  const int per = (L + nsplit - 1) / nsplit;
  const int t_begin = split * per;
  const int t_end = min(L, t_begin + per);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane >> 3;  // token slot inside a warp step (0..3)
  const int dl = lane & 7;    // owns dims [16*dl, 16*dl+16)
  const int n_tiles = (max(t_end - t_begin, 0) + kTok - 1) / kTok;
  const int* bt = block_table + static_cast<long long>(b) * max_blocks;

  // each thread copies 4 K chunks and 4 V chunks (16 B) per stage: chunk c = tid + 128*i,
  // token = c / 16, piece = c % 16
  auto issue = [&](int tile) {
    if (tile < n_tiles) {
      uint8_t* st = dsm + (tile % kStagesD) * kStageB;
      const int t0 = t_begin + tile * kTok;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + 128 * i;
        const int tok = c >> 4, piece = c & 15;
        const int t = t0 + tok;
        if (t < t_end) {
          const int blk = __ldg(bt + t / block_size);
          const long long slot = static_cast<long long>(blk) * block_size + (t % block_size);
          const uint8_t* kp = reinterpret_cast<const uint8_t*>(k_cache + (slot * Hkv + hk) * kHD) + piece * 16;
          const uint8_t* vp = reinterpret_cast<const uint8_t*>(v_cache + (slot * Hkv + hk) * kHD) + piece * 16;
          cp_async16(st + tok * kRowB + piece * 16, kp);
          cp_async16(st + kTok * kRowB + tok * kRowB + piece * 16, vp);
        }
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int sgi = 0; sgi < kStagesD - 1; ++sgi) issue(sgi);

  float qv[G][16];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const __nv_bfloat16* qp = q + (static_cast<long long>(b) * Hq + hk * G + g) * kHD + dl * 16;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 f = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(qp)[i]);
      qv[g][2 * i] = f.x * scale_log2;
      qv[g][2 * i + 1] = f.y * scale_log2;
    }
  }
  float m[G], l[G], acc[G][16];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[g][i] = 0.f;
  }

  for (int tile = 0; tile < n_tiles; ++tile) {
    issue(tile + kStagesD - 1);
    cp_async_wait<kStagesD - 1>();
    __syncthreads();
    const uint8_t* st = dsm + (tile % kStagesD) * kStageB;
    const int t0 = t_begin + tile * kTok;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int tok = warp * 8 + it * 4 + sub;
      const bool valid = t0 + tok < t_end;
      const uint4* kp = reinterpret_cast<const uint4*>(st + tok * kRowB + dl * 32);
      const uint4* vp = reinterpret_cast<const uint4*>(st + kTok * kRowB + tok * kRowB + dl * 32);
      uint4 kr[2], vr[2];
      kr[0] = kp[0]; kr[1] = kp[1];
      vr[0] = vp[0]; vr[1] = vp[1];
      const __nv_bfloat162* kb = reinterpret_cast<const __nv_bfloat162*>(kr);
      const __nv_bfloat162* vb = reinterpret_cast<const __nv_bfloat162*>(vr);
      float kf[16], vf[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 a = __bfloat1622float2(kb[i]);
        const float2 c = __bfloat1622float2(vb[i]);
        kf[2 * i] = a.x; kf[2 * i + 1] = a.y;
        vf[2 * i] = c.x; vf[2 * i + 1] = c.y;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) s += qv[g][i] * kf[i];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (valid) {
          if (s > m[g] + 8.f) {  // raise the reference max only when needed (also the first token)
            const float sc = exp2f(m[g] - s);
            l[g] *= sc;
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[g][i] *= sc;
            m[g] = s;
          }
          const float p = exp2f(s - m[g]);
          l[g] += p;
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[g][i] += p * vf[i];
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  // merge the 4 token slots of the warp (lanes with equal dl), then the 4 warps
  __shared__ float s_m[4][G], s_l[4][G], s_acc[4][G][kHD];
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int off = 8; off <= 16; off <<= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], off);
      const float lo = __shfl_xor_sync(0xffffffffu, l[g], off);
      const float mn = fmaxf(m[g], mo);
      const float a = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mn);
      const float bsc = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
      l[g] = l[g] * a + lo * bsc;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[g][i], off);
        acc[g][i] = acc[g][i] * a + ao * bsc;
      }
      m[g] = mn;
    }
    if (sub == 0) {
      if (dl == 0) { s_m[warp][g] = m[g]; s_l[warp][g] = l[g]; }
#pragma unroll
      for (int i = 0; i < 16; ++i) s_acc[warp][g][dl * 16 + i] = acc[g][i];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * kHD; idx += blockDim.x) {
    const int g = idx / kHD, d = idx % kHD;
    float mn = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mn = fmaxf(mn, s_m[w][g]);
    float lt = 0.f, at = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float sc = (s_m[w][g] == -INFINITY) ? 0.f : exp2f(s_m[w][g] - mn);
      lt += s_l[w][g] * sc;
      at += s_acc[w][g][d] * sc;
    }
    const long long o = ((static_cast<long long>(b) * Hq + hk * G + g) * nsplit + split);
    o_part[o * kHD + d] = at;
    if (d == 0) {
      ml_part[o * 2] = mn;
      ml_part[o * 2 + 1] = lt;
    }
  }
}

__global__ void paged_decode_merge_kernel(const float* __restrict__ o_part,
                                          const float* __restrict__ ml_part,
                                          __nv_bfloat16* __restrict__ out, int nsplit) {
  const long long bh = blockIdx.x;  // (b * Hq + h)
  const int d = threadIdx.x;        // 128 threads
  float mn = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mn = fmaxf(mn, ml_part[(bh * nsplit + s) * 2]);
  float lt = 0.f, at = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = ml_part[(bh * nsplit + s) * 2];
    const float sc = (ms == -INFINITY) ? 0.f : exp2f(ms - mn);
    lt += ml_part[(bh * nsplit + s) * 2 + 1] * sc;
    at += o_part[(bh * nsplit + s) * kHD + d] * sc;
  }
  out[bh * kHD + d] = __float2bfloat16(lt > 0.f ? at / lt : 0.f);
}

}  // namespace b200

extern "C" {

int b200_kv_cache_write(const void* k, const void* v, long long ldk, long long ldv,
                        const long long* slot_mapping, void* k_cache, void* v_cache, int T,
                        int Hkv, int D, cudaStream_t stream) {
  using namespace b200;
  if (D != kHD) return -100;
  if (T == 0) return 0;
  const long long total = static_cast<long long>(T) * Hkv * kHD / 8;
  long long grid = (total + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 8;
  if (grid > maxg) grid = maxg;
  kv_cache_write_kernel<<<(unsigned)grid, 256, 0, stream>>>(
      (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, ldk, ldv, slot_mapping,
      (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, T, Hkv);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// o_part: fp32 [B, Hq, nsplit, 128]; ml_part: fp32 [B, Hq, nsplit, 2].
int b200_paged_decode(const void* q, const void* k_cache, const void* v_cache,
                      const int* block_table, const int* seq_lens, void* out, float* o_part,
                      float* ml_part, int B, int Hq, int Hkv, int D, int block_size,
                      int max_blocks, int nsplit, float softmax_scale, cudaStream_t stream) {
  using namespace b200;
  if (D != kHD || Hq % Hkv) return -100;
  if (B == 0) return 0;
  const int G = Hq / Hkv;
  const float sl2 = softmax_scale * 1.4426950408889634f;
  dim3 grid(B, Hkv, nsplit);
#define LAUNCH(G_)                                                                             \
  cudaFuncSetAttribute(paged_decode_kernel<G_>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                       kStagesD * kStageB);                                                     \
  paged_decode_kernel<G_><<<grid, 128, kStagesD * kStageB, stream>>>(                                           \
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,   \
      block_table, seq_lens, o_part, ml_part, Hq, Hkv, block_size, max_blocks, nsplit, sl2)
  switch (G) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 4: LAUNCH(4); break;
    case 7: LAUNCH(7); break;
    case 8: LAUNCH(8); break;
    default: return -101;
  }
#undef LAUNCH
  B200_CHECK(cudaGetLastError());
  paged_decode_merge_kernel<<<B * Hq, kHD, 0, stream>>>(o_part, ml_part, (__nv_bfloat16*)out,
                                                        nsplit);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
