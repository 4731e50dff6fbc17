// Mixture-of-experts routing for sm_100a: softmax + top-k, a stable counting sort of
// the [T*k] (token, choice) copies by expert into a layout whose per-expert segments
// are padded to 128 rows (one GEMM row tile never straddles two experts and the
// padded rows are zero, so they drop out of every reduction), the gather into that
// layout and the weighted combine back. Everything stays on the device: the tile
// table that the grouped GEMM walks is produced here, no host round-trip.
//
// Semantics follow the reference's token reorderer and router
// (areal/experimental/models/archon/moe/{router,token_reorderer,utils}.py,
// kernel areal/experimental/models/archon/moe/kernels.py `_fill_indices_kernel`):
// copies are ordered by expert, ties by flat index t*k + j.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "common/host_utils.h"

namespace b200 {

constexpr int kMaxE = 1024;
constexpr int kChunk = 256;  // flat entries per warp in the sort

// One warp per token. logits [T, E] fp32 → idx [T, k] int32, w [T, k] fp32.
// score = softmax over all experts; the k largest are kept (ties: lowest index) and
// optionally renormalised to sum to one.
template <int PER>  // experts per lane = ceil(E / 32)
__global__ void moe_route_kernel(const float* __restrict__ logits, int* __restrict__ idx, float* __restrict__ w,
                                 int T, int E, int k, int renorm) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? logits[t * E + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = (lane + 32 * i < E) ? expf(v[i] - mx) : -1.f;  // -1 marks "not available"
    if (v[i] > 0.f) sum += v[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  float picked_sum = 0.f;
  float my_w = 0.f;
  int my_e = 0;
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (v[i] > best) { best = v[i]; be = lane + 32 * i; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (lane + 32 * i == be) v[i] = -1.f;
    picked_sum += best * inv;
    if (lane == j) { my_w = best * inv; my_e = be; }
  }
  if (lane < k) {
    idx[t * k + lane] = my_e;
    w[t * k + lane] = renorm ? my_w / picked_sum : my_w;
  }
}

// Pass A: per-chunk expert histograms. One warp per chunk of kChunk flat entries.
__global__ void moe_hist_kernel(const int* __restrict__ idx, int n, int E, int* __restrict__ chunk_hist) {
  extern __shared__ int sh[];  // [warps][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * (blockDim.x >> 5) + warp;
  int* h = sh + warp * E;
  for (int e = lane; e < E; e += 32) h[e] = 0;
  __syncwarp();
  const int base = chunk * kChunk;
  for (int i = lane; i < kChunk; i += 32)
    if (base + i < n) atomicAdd(&h[idx[base + i]], 1);
  __syncwarp();
  if (base < n)
    for (int e = lane; e < E; e += 32) chunk_hist[static_cast<long long>(chunk) * E + e] = h[e];
}

// Pass B: one block, thread e owns expert e. chunk_hist becomes the exclusive prefix over chunks;
// counts, padded segment starts, the tile → expert table and the tile count follow.
__global__ void moe_scan_kernel(int* __restrict__ chunk_hist, int nchunks, int E, int* __restrict__ counts,
                                int* __restrict__ prow0, int* __restrict__ tile_expert, int* __restrict__ num_vm) {
  __shared__ int s_tiles[kMaxE + 1];
  const int e = threadIdx.x;
  int run = 0;
  if (e < E) {
    for (int c = 0; c < nchunks; ++c) {
      const long long o = static_cast<long long>(c) * E + e;
      const int v = chunk_hist[o];
      chunk_hist[o] = run;
      run += v;
    }
    counts[e] = run;
    s_tiles[e] = (run + 127) >> 7;
  }
  __syncthreads();
  if (threadIdx.x == 0) {  // E <= 1024: a serial scan is a few hundred cycles
    int acc = 0;
    for (int i = 0; i < E; ++i) {
      const int tl = s_tiles[i];
      s_tiles[i] = acc;
      acc += tl;
    }
    s_tiles[E] = acc;
    *num_vm = acc;
  }
  __syncthreads();
  if (e < E) {
    prow0[e] = s_tiles[e] << 7;
    for (int vm = s_tiles[e]; vm < s_tiles[e + 1]; ++vm) tile_expert[vm] = e;
  }
  if (e == 0) prow0[E] = s_tiles[E] << 7;
}

// Pass C: stable placement. dest[i] = padded row of flat entry i; src_of[row] = i (rows of padding keep -1).
__global__ void moe_place_kernel(const int* __restrict__ idx, int n, int E, const int* __restrict__ chunk_base,
                                 const int* __restrict__ prow0, int* __restrict__ dest, int* __restrict__ src_of) {
  extern __shared__ int sh[];  // [warps][E] running counters
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * (blockDim.x >> 5) + warp;
  int* run = sh + warp * E;
  for (int e = lane; e < E; e += 32) run[e] = 0;
  __syncwarp();
  const int base = chunk * kChunk;
  if (base >= n) return;
  for (int it = 0; it < kChunk / 32; ++it) {
    const int i = base + it * 32 + lane;
    const bool valid = i < n;
    const int e = valid ? idx[i] : -1 - lane;  // invalid lanes match nobody
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (valid) {
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int pos = prow0[e] + chunk_base[static_cast<long long>(chunk) * E + e] + run[e] + rank;
      dest[i] = pos;
      src_of[pos] = i;
    }
    __syncwarp();
    if (valid && lane == (__ffs(peers) - 1)) run[e] += __popc(peers);
    __syncwarp();
  }
}

// out[r] = scale[src] * x[src / k] for padded row r (zeros for padding rows); rows beyond num_vm*128 untouched.
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ src_of,
                                  const float* __restrict__ scale, const int* __restrict__ num_vm, int k, int H,
                                  __nv_bfloat16* __restrict__ out) {
  const int rows = *num_vm * 128;
  const int vec = H >> 3;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const int src = src_of[r];
    uint4* o = reinterpret_cast<uint4*>(out + static_cast<long long>(r) * H);
    if (src < 0) {
      for (int c = lane; c < vec; c += 32) o[c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const uint4* in = reinterpret_cast<const uint4*>(x + static_cast<long long>(src / k) * ldx);
    if (scale == nullptr) {
      for (int c = lane; c < vec; c += 32) o[c] = in[c];
    } else {
      const float s = scale[src];
      for (int c = lane; c < vec; c += 32) {
        uint4 v = in[c];
        __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(b[j]);
          b[j] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
        o[c] = v;
      }
    }
  }
}

// out[t] = sum_j w[t,j] * y[dest[t*k+j]] (w == nullptr: plain sum). One warp per token, fp32 accumulation.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ dest,
                                   const float* __restrict__ w, int T, int k, int H, __nv_bfloat16* __restrict__ out) {
  const int vec = H >> 3;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    for (int c = lane; c < vec; c += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
        const int r = dest[t * k + j];
        const float s = w ? w[t * k + j] : 1.f;
        const uint4 v = reinterpret_cast<const uint4*>(y + static_cast<long long>(r) * H)[c];
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __bfloat1622float2(b[q]);
          acc[2 * q] += s * f.x;
          acc[2 * q + 1] += s * f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) ob[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H)[c] = o;
    }
  }
}

// dw[t,j] = <dout[t], y[dest[t*k+j]]>. One warp per (t, j).
__global__ void moe_combine_dw_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                                      const int* __restrict__ dest, int n, int k, int H, float* __restrict__ dw) {
  const int vec = H >> 3;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
    const uint4* a = reinterpret_cast<const uint4*>(dout + static_cast<long long>(i / k) * H);
    const uint4* b = reinterpret_cast<const uint4*>(y + static_cast<long long>(dest[i]) * H);
    float s = 0.f;
    for (int c = lane; c < vec; c += 32) {
      const uint4 va = a[c], vb = b[c];
      const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&va);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&vb);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fa = __bfloat1622float2(pa[q]), fb = __bfloat1622float2(pb[q]);
        s += fa.x * fb.x + fa.y * fb.y;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) dw[i] = s;
  }
}


// ------------------------------------------------------------------ expert parallelism --
// Experts are split over P ranks (rank d owns experts [d*E/P, (d+1)*E/P)). Each rank sorts its own
// (token, choice) copies by GLOBAL expert; after the ranks have exchanged their per-expert counts
// every rank can compute, without talking to the host, where each of its copies lands in the
// owner's padded expert-sorted buffer: owner segment of the expert, then source-rank order, then
// the source's stable order. The dispatch kernel stores rows straight into the owners' buffers over
// NVLink, the owners run the grouped GEMMs in place, and the combine kernel pulls the result rows
// back from the owners (weighted sum per token). No intermediate send / receive staging, no
// host-side `tolist()` of the counts as in the reference
// (areal/experimental/models/archon/expert_parallel.py:70-262).

// One block, thread e owns global expert e. counts_all: [P, E].
__global__ void ep_plan_kernel(const int* __restrict__ counts_all, int me, int P, int E, int* __restrict__ send_base,
                               int* __restrict__ prow0_loc, int* __restrict__ total_loc,
                               int* __restrict__ tile_expert_loc, int* __restrict__ num_vm) {
  __shared__ int s_total[kMaxE], s_before[kMaxE], s_start[kMaxE + 1];
  const int e = threadIdx.x;
  const int el = E / P;
  if (e < E) {
    int tot = 0, before = 0;
    for (int s = 0; s < P; ++s) {
      const int c = counts_all[s * E + e];
      if (s < me) before += c;
      tot += c;
    }
    s_total[e] = tot;
    s_before[e] = before;
  }
  __syncthreads();
  if (threadIdx.x < P) {  // thread d scans the experts of owner d
    const int d = threadIdx.x;
    int acc = 0;
    for (int i = 0; i < el; ++i) {
      const int ge = d * el + i;
      s_start[ge] = acc;
      acc += ((s_total[ge] + 127) >> 7) << 7;
    }
    if (d == me) {
      prow0_loc[el] = acc;
      *num_vm = acc >> 7;
    }
  }
  __syncthreads();
  if (e < E) {
    send_base[e] = s_start[e] + s_before[e];
    if (e / el == me) {
      const int l = e - me * el;
      prow0_loc[l] = s_start[e];
      total_loc[l] = s_total[e];
      const int t0 = s_start[e] >> 7, t1 = t0 + ((s_total[e] + 127) >> 7);
      for (int vm = t0; vm < t1; ++vm) tile_expert_loc[vm] = l;
    }
  }
}

// One warp per local copy i = t*k + j: store x[t] into the owner's buffer, remember the row.
__global__ void ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ idx,
                                   const float* __restrict__ w, const int* __restrict__ dest_src,
                                   const int* __restrict__ prow0_src, const int* __restrict__ send_base, int n, int k,
                                   int H, int el, int cap, void* const* __restrict__ peer_x,
                                   float* const* __restrict__ peer_w, int* __restrict__ copy_row, int* status) {
  const int vec = H >> 3;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
    const int e = idx[i];
    const int d = e / el;
    const int row = send_base[e] + (dest_src[i] - prow0_src[e]);
    if (row >= cap) {  // the owner's buffer is too small for this routing: drop the copy, flag it
      if (lane == 0) {
        copy_row[i] = -1;
        atomicCAS(status, 0, 5 /* kErrBounds */);
      }
      continue;
    }
    const uint4* in = reinterpret_cast<const uint4*>(x + static_cast<long long>(i / k) * ldx);
    uint4* out = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(peer_x[d]) + static_cast<long long>(row) * H);
    for (int c = lane; c < vec; c += 32) out[c] = in[c];
    if (lane == 0) {
      copy_row[i] = row;
      if (w) peer_w[d][row] = w[i];
    }
  }
}

// Owner side: zero the padding rows of every local expert segment (peers only write real rows).
__global__ void ep_zero_pad_kernel(__nv_bfloat16* __restrict__ xbuf, float* __restrict__ row_w,
                                   const int* __restrict__ prow0_loc, const int* __restrict__ total_loc, int el, int H) {
  const int l = blockIdx.x;
  if (l >= el) return;
  const int r0 = prow0_loc[l] + total_loc[l], r1 = prow0_loc[l + 1];
  const int vec = H >> 3;
  for (int r = r0 + (threadIdx.x >> 5); r < r1; r += blockDim.x >> 5) {
    uint4* o = reinterpret_cast<uint4*>(xbuf + static_cast<long long>(r) * H);
    for (int c = threadIdx.x & 31; c < vec; c += 32) o[c] = make_uint4(0, 0, 0, 0);
    if ((threadIdx.x & 31) == 0 && row_w) row_w[r] = 0.f;
  }
}

// out[t] = sum_j w[t,j] * y_owner(t,j)[row(t,j)], rows read from the owners' buffers over NVLink.
__global__ void ep_combine_kernel(void* const* __restrict__ peer_y, const int* __restrict__ idx,
                                  const int* __restrict__ copy_row, const float* __restrict__ w, int T, int k, int H,
                                  int el, __nv_bfloat16* __restrict__ out) {
  const int vec = H >> 3;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    for (int c = lane; c < vec; c += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
        const int r = copy_row[t * k + j];
        if (r < 0) continue;
        const int d = idx[t * k + j] / el;
        const float s = w ? w[t * k + j] : 1.f;
        const uint4 v = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(peer_y[d]) +
                                                       static_cast<long long>(r) * H)[c];
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __bfloat1622float2(b[q]);
          acc[2 * q] += s * f.x;
          acc[2 * q + 1] += s * f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) ob[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H)[c] = o;
    }
  }
}

// vals[i] = peer_s(owner of copy i)[row(i)]
__global__ void ep_pull_scalar_kernel(float* const* __restrict__ peer_s, const int* __restrict__ idx,
                                      const int* __restrict__ copy_row, int n, int el, float* __restrict__ vals) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = copy_row[i];
  vals[i] = r < 0 ? 0.f : peer_s[idx[i] / el][r];
}

// s[r] = <a[r], b[r]> and (optionally) a[r] *= scale[r], for the rows in use (num_vm * 128).
__global__ void rowdot_scale_kernel(__nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                    const float* __restrict__ scale, const int* __restrict__ num_vm, int H,
                                    float* __restrict__ s_out) {
  const int rows = *num_vm * 128;
  const int vec = H >> 3;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    uint4* pa = reinterpret_cast<uint4*>(a + static_cast<long long>(r) * H);
    const uint4* pb = reinterpret_cast<const uint4*>(b + static_cast<long long>(r) * H);
    const float sc = scale ? scale[r] : 1.f;
    float s = 0.f;
    for (int c = lane; c < vec; c += 32) {
      uint4 va = pa[c];
      const uint4 vb = pb[c];
      __nv_bfloat162* xa = reinterpret_cast<__nv_bfloat162*>(&va);
      const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&vb);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fa = __bfloat1622float2(xa[q]), fb = __bfloat1622float2(xb[q]);
        s += fa.x * fb.x + fa.y * fb.y;
        xa[q] = __floats2bfloat162_rn(fa.x * sc, fa.y * sc);
      }
      if (scale) pa[c] = va;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0 && s_out) s_out[r] = s;
  }
}

}  // namespace b200

extern "C" {

int b200_moe_route(const float* logits, int* idx, float* w, int T, int E, int k, int renorm, cudaStream_t stream) {
  using namespace b200;
  if (T == 0) return 0;
  if (E > 256 || k > 32 || k > E) return -100;
  const unsigned grid = (static_cast<long long>(T) * 32 + 255) / 256;
  const int per = (E + 31) / 32;
#define RT(P) moe_route_kernel<P><<<grid, 256, 0, stream>>>(logits, idx, w, T, E, k, renorm)
  if (per <= 1) RT(1); else if (per <= 2) RT(2); else if (per <= 4) RT(4); else RT(8);
#undef RT
  B200_CHECK(cudaGetLastError());
  return 0;
}

// Workspace (ints): chunk_hist [ceil(n/256) * E]. Outputs: counts [E], prow0 [E+1], tile_expert [max_vm],
// num_vm [1], dest [n], src_of [max_vm * 128] with max_vm >= n/128 + E. idx values must lie in [0, E).
int b200_moe_sort(const int* idx, int n, int E, int* chunk_hist, int* counts, int* prow0, int* tile_expert,
                  int* num_vm, int* dest, int* src_of, int max_vm, cudaStream_t stream) {
  using namespace b200;
  if (E > kMaxE) return -100;
  if (max_vm < (n + 127) / 128 + E) return -101;
  const int nchunks = (n + kChunk - 1) / kChunk;
  const int wpb = 4;
  const int grid = (nchunks + wpb - 1) / wpb;
  const size_t sh = static_cast<size_t>(wpb) * E * sizeof(int);
  B200_CHECK(cudaMemsetAsync(src_of, 0xFF, static_cast<size_t>(max_vm) * 128 * sizeof(int), stream));
  if (n > 0) moe_hist_kernel<<<grid, wpb * 32, sh, stream>>>(idx, n, E, chunk_hist);
  moe_scan_kernel<<<1, ((E + 31) / 32) * 32, 0, stream>>>(chunk_hist, nchunks, E, counts, prow0, tile_expert, num_vm);
  if (n > 0) moe_place_kernel<<<grid, wpb * 32, sh, stream>>>(idx, n, E, chunk_hist, prow0, dest, src_of);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_moe_gather(const void* x, long long ldx, const int* src_of, const float* scale, const int* num_vm, int k,
                    int H, void* out, int max_rows, cudaStream_t stream) {
  using namespace b200;
  if (H % 8) return -100;
  if (max_rows == 0) return 0;
  long long grid = (static_cast<long long>(max_rows) * 32 + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 16;
  if (grid > maxg) grid = maxg;
  moe_gather_kernel<<<(unsigned)grid, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, src_of, scale, num_vm, k, H,
                                                       (__nv_bfloat16*)out);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_moe_combine(const void* y, const int* dest, const float* w, int T, int k, int H, void* out,
                     cudaStream_t stream) {
  using namespace b200;
  if (H % 8) return -100;
  if (T == 0) return 0;
  long long grid = (static_cast<long long>(T) * 32 + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 16;
  if (grid > maxg) grid = maxg;
  moe_combine_kernel<<<(unsigned)grid, 256, 0, stream>>>((const __nv_bfloat16*)y, dest, w, T, k, H,
                                                        (__nv_bfloat16*)out);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_moe_combine_dw(const void* dout, const void* y, const int* dest, int n, int k, int H, float* dw,
                        cudaStream_t stream) {
  using namespace b200;
  if (H % 8) return -100;
  if (n == 0) return 0;
  long long grid = (static_cast<long long>(n) * 32 + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 16;
  if (grid > maxg) grid = maxg;
  moe_combine_dw_kernel<<<(unsigned)grid, 256, 0, stream>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)y, dest,
                                                           n, k, H, dw);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_ep_plan(const int* counts_all, int me, int P, int E, int* send_base, int* prow0_loc, int* total_loc,
                 int* tile_expert_loc, int* num_vm, cudaStream_t stream) {
  using namespace b200;
  if (E > kMaxE || E % P || P > E) return -100;
  ep_plan_kernel<<<1, ((E + 31) / 32) * 32, 0, stream>>>(counts_all, me, P, E, send_base, prow0_loc, total_loc,
                                                         tile_expert_loc, num_vm);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// peer_x / peer_w: device arrays of P pointers (the owners' row buffers [cap, H] bf16 and row weights [cap]).
int b200_ep_dispatch(const void* x, long long ldx, const int* idx, const float* w, const int* dest_src,
                     const int* prow0_src, const int* send_base, int n, int k, int H, int experts_per_rank, int cap,
                     void* const* peer_x, float* const* peer_w, int* copy_row, cudaStream_t stream) {
  using namespace b200;
  if (H % 8) return -100;
  if (n == 0) return 0;
  int* status = device_status_word();
  if (!status) return -3;
  long long grid = (static_cast<long long>(n) * 32 + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 16;
  if (grid > maxg) grid = maxg;
  ep_dispatch_kernel<<<(unsigned)grid, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, idx, w, dest_src, prow0_src,
                                                        send_base, n, k, H, experts_per_rank, cap, peer_x, peer_w,
                                                        copy_row, status);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_ep_zero_pad(void* xbuf, float* row_w, const int* prow0_loc, const int* total_loc, int experts_per_rank, int H,
                     cudaStream_t stream) {
  using namespace b200;
  ep_zero_pad_kernel<<<experts_per_rank, 256, 0, stream>>>((__nv_bfloat16*)xbuf, row_w, prow0_loc, total_loc,
                                                           experts_per_rank, H);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_ep_combine(void* const* peer_y, const int* idx, const int* copy_row, const float* w, int T, int k, int H,
                    int experts_per_rank, void* out, cudaStream_t stream) {
  using namespace b200;
  if (H % 8) return -100;
  if (T == 0) return 0;
  long long grid = (static_cast<long long>(T) * 32 + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 16;
  if (grid > maxg) grid = maxg;
  ep_combine_kernel<<<(unsigned)grid, 256, 0, stream>>>(peer_y, idx, copy_row, w, T, k, H, experts_per_rank,
                                                       (__nv_bfloat16*)out);
  B200_CHECK(cudaGetLastError());
  return 0;
}

int b200_ep_pull_scalar(float* const* peer_s, const int* idx, const int* copy_row, int n, int experts_per_rank,
                        float* vals, cudaStream_t stream) {
  using namespace b200;
  if (n == 0) return 0;
  ep_pull_scalar_kernel<<<(n + 255) / 256, 256, 0, stream>>>(peer_s, idx, copy_row, n, experts_per_rank, vals);
  B200_CHECK(cudaGetLastError());
  return 0;
}

// s_out[r] = <a[r], b[r]> (s_out may be null), then a[r] *= scale[r] (scale may be null), rows < *num_vm * 128.
int b200_rowdot_scale(void* a, const void* b, const float* scale, const int* num_vm, int max_rows, int H, float* s_out,
                      cudaStream_t stream) {
  using namespace b200;
  if (H % 8) return -100;
  if (max_rows == 0) return 0;
  long long grid = (static_cast<long long>(max_rows) * 32 + 255) / 256;
  const long long maxg = static_cast<long long>(sm_count()) * 16;
  if (grid > maxg) grid = maxg;
  rowdot_scale_kernel<<<(unsigned)grid, 256, 0, stream>>>((__nv_bfloat16*)a, (const __nv_bfloat16*)b, scale, num_vm, H,
                                                         s_out);
  B200_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
