// Rollout-engine kernels: paged-KV cache write and single-token (decode)
// attention over a paged cache with GQA and split-KV (flash-decoding).
//
// Cache layout: k_cache / v_cache [num_blocks, Hkv, block_size, 128] bf16, so
// the tokens of one (page, kv head) are contiguous. A sequence's pages are
// listed in block_table[seq, max_blocks]. Decode attention is memory-bound
// (each K/V byte is used once per query head of the group): one CTA per
// (sequence, kv head, split) streams its K/V slabs with TMA; partial
// (max, sum, acc) results of the splits are merged by a second small kernel.
//
// These replace the external inference server's decode path in the reference
// (SGLang / vLLM paged attention; areal/engine/sglang_remote.py).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "common/host_utils.h"
#include "common/ptx.cuh"

namespace b200 {

constexpr int kHD = 128;
constexpr int kMaxGroup = 8;

// slot_mapping[t] = block * block_size + offset (or < 0 to skip the token)
__global__ void kv_cache_write_kernel(const __nv_bfloat16* __restrict__ k,
                                      const __nv_bfloat16* __restrict__ v, long long ldk,
                                      long long ldv, const long long* __restrict__ slot_mapping,
                                      __nv_bfloat16* __restrict__ k_cache,
                                      __nv_bfloat16* __restrict__ v_cache, int T, int Hkv, int block_size) {
  const int vec_per_tok = Hkv * kHD / 8;
  const long long total = static_cast<long long>(T) * vec_per_tok;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / vec_per_tok);
    const int c = static_cast<int>(i % vec_per_tok);
    const long long slot = slot_mapping[t];
    if (slot < 0) continue;
    const long long blk = slot / block_size, off = slot % block_size;
    const int h = c / (kHD / 8), piece = c % (kHD / 8);
    const long long dst = ((blk * Hkv + h) * block_size + off) * (kHD / 8) + piece;
    reinterpret_cast<uint4*>(k_cache)[dst] = reinterpret_cast<const uint4*>(k + t * ldk)[c];
    reinterpret_cast<uint4*>(v_cache)[dst] = reinterpret_cast<const uint4*>(v + t * ldv)[c];
  }
}

// q: [B, Hq, 128]; partial outputs: o_part [B, Hq, nsplit, 128] fp32, ml_part [B, Hq, nsplit, 2].
//
// One CTA per (sequence, kv head, split), four warps, and every warp is its own
// pipeline: it owns a ring of kSlots 16-token slabs (K and V, 8 KB per slab) that
// lane 0 fills with TMA (128-byte swizzle, so ldmatrix is conflict-free) and
// consumes them in order; there is no CTA-wide barrier in the main loop. With the
// cache laid out [page, kv head, token, dim] a slab is one contiguous 4 KB read
// for K and one for V. The query heads of the GQA group form the (zero-padded)
// 16 rows of an m16n8k16 tensor-core tile: S = Q K^T and O += P V cost ~7 warp
// instructions per cached token, so the kernel stays bound by HBM, not by issue
// slots. The running max is raised lazily (only when a score exceeds it by 2^8).
constexpr int kSlab = 16;
constexpr int kSlots = 3;
constexpr int kWarpsD = 4;
constexpr int kHalfB = kSlab * 128;        // one 64-dim half of a slab: 16 rows x 128 B
constexpr int kSlabB = 4 * kHalfB;         // K lo | K hi | V lo | V hi
constexpr int kDecodeSmem = kWarpsD * kSlots * kSlabB + 1024 + 256;

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D += A(16x16, row) * B(16x8, col), bf16 inputs, fp32 accumulate
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int G>
__global__ void __launch_bounds__(kWarpsD * 32, 2)
paged_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const __nv_bfloat16* __restrict__ q, const int* __restrict__ block_table,
                    const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out,
                    float* __restrict__ o_part, float* __restrict__ ml_part, int Hq, int Hkv, int block_size,
                    int max_blocks, int nsplit, float scale_log2, int* status) {
  extern __shared__ uint8_t dsm_raw[];
  uint8_t* dsm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dsm_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(dsm + kWarpsD * kSlots * kSlabB);  // [warp][slot]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kWarpsD * kSlots);

  const int b = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = seq_lens[b];
  const int slabs_total = (L + kSlab - 1) / kSlab;
  const int per = (slabs_total + nsplit - 1) / nsplit;
  const int s_begin = split * per;
  const int s_end = min(slabs_total, s_begin + per);
  const int spp = block_size / kSlab;  // slabs per page
  const int* bt = block_table + static_cast<long long>(b) * max_blocks;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kWarpsD * kSlots; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  __syncthreads();

  uint8_t* ring = dsm + warp * kSlots * kSlabB;
  uint64_t* full = bars + warp * kSlots;
  const int my_first = s_begin + warp;
  const int my_count = my_first < s_end ? (s_end - my_first + kWarpsD - 1) / kWarpsD : 0;

  auto issue = [&](int j) {  // lane 0 only
    const int sl = my_first + j * kWarpsD;
    const int page = __ldg(bt + sl / spp);
    const int y = (page * Hkv + hk) * block_size + (sl % spp) * kSlab;
    uint8_t* dst = ring + (j % kSlots) * kSlabB;
    uint64_t* bar = &full[j % kSlots];
    mbar_arrive_expect_tx(bar, kSlabB);
    tma_load_2d(dst, &tmK, bar, 0, y);
    tma_load_2d(dst + kHalfB, &tmK, bar, 64, y);
    tma_load_2d(dst + 2 * kHalfB, &tmV, bar, 0, y);
    tma_load_2d(dst + 3 * kHalfB, &tmV, bar, 64, y);
  };
  if (lane == 0)
    for (int j = 0; j < kSlots && j < my_count; ++j) issue(j);

  // query fragments: row = lane / 4 is the head inside the group (rows >= G are zero)
  const int row = lane >> 2, cq = (lane & 3) * 2;
  uint32_t qa0[8], qa2[8];
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    qa0[kk] = 0u; qa2[kk] = 0u;
    if (row < G) {
      const __nv_bfloat16* qp = q + (static_cast<long long>(b) * Hq + hk * G + row) * kHD + kk * 16 + cq;
      qa0[kk] = *reinterpret_cast<const uint32_t*>(qp);
      qa2[kk] = *reinterpret_cast<const uint32_t*>(qp + 8);
    }
  }
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
  float m = -INFINITY, l = 0.f;

  // per-lane ldmatrix row: matrix id = lane / 8, row in matrix = lane % 8
  const int lm = lane >> 3, lr = lane & 7;
  bool ok = true;
  for (int j = 0; j < my_count; ++j) {
    const int slot = j % kSlots;
    if (!mbar_wait(&full[slot], (j / kSlots) & 1, abort_flag)) { ok = false; break; }
    const uint32_t kbase = smem_u32(ring + slot * kSlabB);
    const uint32_t vbase = kbase + 2 * kHalfB;
    float s[2][4];
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[t][c] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      // matrices: (tokens 0-7, dims k..k+7), (0-7, k+8..), (8-15, k..), (8-15, k+8..)
      const int tok = ((lm >> 1) << 3) + lr;
      const int chunk = ((kk & 3) << 1) + (lm & 1);
      const uint32_t addr = kbase + (kk >> 2) * kHalfB + tok * 128 + ((chunk ^ (tok & 7)) << 4);
      uint32_t b00, b01, b10, b11;
      ldsm_x4(addr, b00, b01, b10, b11);
      mma_16816(s[0], qa0[kk], 0u, qa2[kk], 0u, b00, b01);
      mma_16816(s[1], qa0[kk], 0u, qa2[kk], 0u, b10, b11);
    }
    // scale, mask the tail, row max over the 16 tokens (columns live in the 4 lanes of a quad)
    const int tok0 = (my_first + j * kWarpsD) * kSlab + cq;
    float sv[4] = {s[0][0] * scale_log2, s[0][1] * scale_log2, s[1][0] * scale_log2, s[1][1] * scale_log2};
    if (tok0 >= L) sv[0] = -INFINITY;
    if (tok0 + 1 >= L) sv[1] = -INFINITY;
    if (tok0 + 8 >= L) sv[2] = -INFINITY;
    if (tok0 + 9 >= L) sv[3] = -INFINITY;
    float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const bool raise = mx > m + 8.f;
    if (__any_sync(0xffffffffu, raise)) {
      const float mn = raise ? mx : m;
      const float sc = (m == -INFINITY) ? 0.f : exp2f(m - mn);
      l *= sc;
#pragma unroll
      for (int i = 0; i < 16; ++i) { o[i][0] *= sc; o[i][1] *= sc; }
      m = mn;
    }
    const float p0 = exp2f(sv[0] - m), p1 = exp2f(sv[1] - m), p2 = exp2f(sv[2] - m), p3 = exp2f(sv[3] - m);
    l += (p0 + p1) + (p2 + p3);
    const uint32_t pa0 = pack_bf16x2(p0, p1), pa2 = pack_bf16x2(p2, p3);
#pragma unroll
    for (int nd = 0; nd < 8; ++nd) {
      // matrices: (tokens 0-7, dims d..d+7), (8-15, d..), (0-7, d+8..), (8-15, d+8..), transposed on load
      const int tok = ((lm & 1) << 3) + lr;
      const int dchunk = (nd << 1) + (lm >> 1);
      const uint32_t addr = vbase + (dchunk >> 3) * kHalfB + tok * 128 + (((dchunk & 7) ^ (tok & 7)) << 4);
      uint32_t v00, v01, v10, v11;
      ldsm_x4_t(addr, v00, v01, v10, v11);
      mma_16816(o[2 * nd], pa0, 0u, pa2, 0u, v00, v01);
      mma_16816(o[2 * nd + 1], pa0, 0u, pa2, 0u, v10, v11);
    }
    __syncwarp();
    if (lane == 0 && j + kSlots < my_count) {
      fence_proxy_async_smem();  // the slab was read through the generic proxy; TMA writes through the async one
      issue(j + kSlots);
    }
  }
  if (!ok) {
    *abort_flag = 1;
    if (lane == 0) atomicCAS(status, 0, kErrMbarTimeoutEpilogue);
    const unsigned long long t0 = globaltimer_ns();  // let copies already in flight land before the CTA retires
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  __syncthreads();  // every warp is done with its ring: reuse it for the cross-warp merge
  float* s_o = reinterpret_cast<float*>(dsm);                 // [warp][G][128]
  float* s_ml = s_o + kWarpsD * G * kHD;                      // [warp][G][2]
  if (row < G) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      s_o[(warp * G + row) * kHD + i * 8 + cq] = o[i][0];
      s_o[(warp * G + row) * kHD + i * 8 + cq + 1] = o[i][1];
    }
    if ((lane & 3) == 0) {
      s_ml[(warp * G + row) * 2] = m;
      s_ml[(warp * G + row) * 2 + 1] = l;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * kHD; idx += blockDim.x) {
    const int g = idx / kHD, d = idx % kHD;
    float mn = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarpsD; ++w) mn = fmaxf(mn, s_ml[(w * G + g) * 2]);
    float lt = 0.f, at = 0.f;
#pragma unroll
    for (int w = 0; w < kWarpsD; ++w) {
      const float mw = s_ml[(w * G + g) * 2];
      const float sc = (mw == -INFINITY) ? 0.f : exp2f(mw - mn);
      lt += s_ml[(w * G + g) * 2 + 1] * sc;
      at += s_o[(w * G + g) * kHD + d] * sc;
    }
    const long long bh = static_cast<long long>(b) * Hq + hk * G + g;
    if (nsplit == 1) {
      out[bh * kHD + d] = __float2bfloat16(lt > 0.f ? at / lt : 0.f);
    } else {
      const long long oidx = bh * nsplit + split;
      o_part[oidx * kHD + d] = at;
      if (d == 0) {
        ml_part[oidx * 2] = mn;
        ml_part[oidx * 2 + 1] = lt;
      }
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
                        int Hkv, int D, int block_size, cudaStream_t stream) {
  using namespace b200;
  if (D != kHD) return -100;
  if (T == 0) return 0;
  const long long total = static_cast<long long>(T) * Hkv * kHD / 8;
  long long grid = (total + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 8;
  if (grid > maxg) grid = maxg;
  kv_cache_write_kernel<<<(unsigned)grid, 256, 0, stream>>>(
      (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, ldk, ldv, slot_mapping,
      (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, T, Hkv, block_size);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// k_cache / v_cache: [num_blocks, Hkv, block_size, 128] bf16, block_size a multiple of 16.
// o_part: fp32 [B, Hq, nsplit, 128]; ml_part: fp32 [B, Hq, nsplit, 2] (unused when nsplit == 1).
int b200_paged_decode(const void* q, const void* k_cache, const void* v_cache,
                      const int* block_table, const int* seq_lens, void* out, float* o_part,
                      float* ml_part, int B, int Hq, int Hkv, int D, int block_size, int num_blocks,
                      int max_blocks, int nsplit, float softmax_scale, cudaStream_t stream) {
  using namespace b200;
  if (D != kHD || Hq % Hkv || block_size % kSlab) return -100;
  if (B == 0) return 0;
  const int G = Hq / Hkv;
  const float sl2 = softmax_scale * 1.4426950408889634f;
  CUtensorMap tmK, tmV;
  const uint64_t rows = static_cast<uint64_t>(num_blocks) * Hkv * block_size;
  int rc = make_tmap_2d(&tmK, k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, kHD, kHD * 2, kSlab, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, v_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, kHD, kHD * 2, kSlab, 64);
  if (rc) return rc;
  int* status = device_status_word();
  if (!status) return -3;
  dim3 grid(B, Hkv, nsplit);
#define LAUNCH(G_)                                                                                        \
  cudaFuncSetAttribute(paged_decode_kernel<G_>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmem); \
  paged_decode_kernel<G_><<<grid, kWarpsD * 32, kDecodeSmem, stream>>>(                                   \
      tmK, tmV, (const __nv_bfloat16*)q, block_table, seq_lens, (__nv_bfloat16*)out, o_part, ml_part, Hq, \
      Hkv, block_size, max_blocks, nsplit, sl2, status)
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
  if (nsplit > 1) {
    paged_decode_merge_kernel<<<B * Hq, kHD, 0, stream>>>(o_part, ml_part, (__nv_bfloat16*)out, nsplit);
    B200_CHECK(cudaGetLastError());
  }
  return 0;
}

}  // extern "C"
