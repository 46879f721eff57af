// Mixture-of-experts routing and token movement (no host synchronisation anywhere):
//   route   : sigmoid scores, selection bias, group-limited top-k, normalised weights, expert histogram
//   plan    : histogram -> expert offsets aligned to the GEMM's 128-row tile + per-tile expert table
//   permute : token rows -> expert-sorted rows (slot claimed with one atomic per (token, k))
//   combine : weighted sum of each token's k expert outputs in fp32
// The grouped GEMM in gemm_tcgen05.cu consumes `tile_expert` from `plan`.
// Role in the reference: the router and the grouped expert forward of telefuser/ops/moe.py (torch top-k + per-expert
// loops / grouped library GEMMs) and the expert-specialised GEMM glue under tf-kernel/csrc/expert_specialization/.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "tfb_api.h"
#include "tfb_common.cuh"
#include "tfb_host.h"

namespace tfb {

constexpr int MOE_MAX_EXPERTS = 1024;

// One warp per token. Expert e lives in lane e % 32, slot e / 32.
template <int SLOTS>
__global__ void moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int G,
                                 int topk_groups, int K, float scale, int use_softmax, int* __restrict__ ids,
                                 float* __restrict__ weights, int* __restrict__ counts) {
  extern __shared__ float sm[];  // per warp: sel[E]
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int warps_per_block = blockDim.x >> 5;
  float* sel_s = sm + wib * E;
  const int per_group = E / G;
  for (int t = blockIdx.x * warps_per_block + wib; t < T; t += gridDim.x * warps_per_block) {
    float score[SLOTS], sel[SLOTS];
    const float* lr = logits + static_cast<long>(t) * E;
    float mx = -INFINITY;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
      const int e = s * 32 + lane;
      score[s] = e < E ? lr[e] : -INFINITY;
      mx = fmaxf(mx, score[s]);
    }
    if (use_softmax) {
      mx = warp_max(mx);
      float sum = 0.f;
#pragma unroll
      for (int s = 0; s < SLOTS; ++s) {
        score[s] = (s * 32 + lane) < E ? expf(score[s] - mx) : 0.f;
        sum += score[s];
      }
      sum = warp_sum(sum);
#pragma unroll
      for (int s = 0; s < SLOTS; ++s) score[s] = __fdiv_rn(score[s], sum);
    } else {
#pragma unroll
      for (int s = 0; s < SLOTS; ++s) score[s] = __fdiv_rn(1.f, 1.f + expf(-score[s]));
    }
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
      const int e = s * 32 + lane;
      sel[s] = e < E ? score[s] + (bias ? bias[e] : 0.f) : -INFINITY;
      if (e < E) sel_s[e] = sel[s];
    }
    __syncwarp();
    // Group scores: sum of the two largest selection scores of each group (lane g handles group g).
    uint32_t group_mask = 0xffffffffu;
    if (G > 1 && topk_groups < G) {
      float gv = -INFINITY;
      if (lane < G) {
        float a = -INFINITY, b = -INFINITY;
        for (int i = 0; i < per_group; ++i) {
          const float v = sel_s[lane * per_group + i];
          if (v > a) {
            b = a;
            a = v;
          } else if (v > b) {
            b = v;
          }
        }
        gv = per_group > 1 ? a + b : a;
      }
      group_mask = 0;
      for (int r = 0; r < topk_groups; ++r) {
        float best = gv;
        int arg = lane;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
          if (ob > best || (ob == best && oa < arg)) {
            best = ob;
            arg = oa;
          }
        }
        group_mask |= 1u << arg;
        if (lane == arg) gv = -INFINITY;
      }
#pragma unroll
      for (int s = 0; s < SLOTS; ++s) {
        const int e = s * 32 + lane;
        if (e < E && !((group_mask >> (e / per_group)) & 1u)) sel[s] = -INFINITY;
      }
    }
    // Top-k by repeated warp arg-max (ties -> lower expert id).
    float wsum = 0.f, my_w = 0.f;
    int my_id = 0;
    for (int r = 0; r < K; ++r) {
      float best = -INFINITY;
      int arg = 0x7fffffff;
#pragma unroll
      for (int s = 0; s < SLOTS; ++s) {
        const int e = s * 32 + lane;
        if (e < E && (sel[s] > best || (sel[s] == best && e < arg))) {
          best = sel[s];
          arg = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) {
          best = ob;
          arg = oa;
        }
      }
      // owner lane reports the unbiased score and retires the expert
      float sc = 0.f;
#pragma unroll
      for (int s = 0; s < SLOTS; ++s) {
        if (s * 32 + lane == arg) {
          sc = score[s];
          sel[s] = -INFINITY;
        }
      }
      sc = __shfl_sync(0xffffffffu, sc, arg & 31);
      wsum += sc;
      if (lane == r) {
        my_w = sc;
        my_id = arg;
      }
    }
    if (lane < K) {
      const float denom = fmaxf(wsum, 1.1920929e-07f);
      ids[static_cast<long>(t) * K + lane] = my_id;
      weights[static_cast<long>(t) * K + lane] = __fdiv_rn(my_w, denom) * scale;
      if (counts) atomicAdd(&counts[my_id], 1);
    }
    __syncwarp();
  }
}

// One block. offsets[e] = first row of expert e (multiple of `align`), offsets[E] = padded total.
// tile_expert[m] for m < max_tiles: expert owning rows [m*align, (m+1)*align) or -1.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int align, int* __restrict__ offsets,
                                int* __restrict__ tile_expert, int max_tiles) {
  __shared__ int s_off[MOE_MAX_EXPERTS + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = acc;
      acc += (counts[e] + align - 1) / align * align;
    }
    s_off[E] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = s_off[e];
  for (int m = threadIdx.x; m < max_tiles; m += blockDim.x) {
    const int row = m * align;
    int owner = -1;
    if (row < s_off[E]) {
      int lo = 0, hi = E - 1;  // last e with s_off[e] <= row
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid - 1;
      }
      owner = lo;
    }
    tile_expert[m] = owner;
  }
}

// One warp per (token, k): claims a slot in its expert's segment and copies the token row.
// `cursor` (int[E]) is scratch and must be zero on entry. An expert id outside [0, E) claims nothing: its
// row_map entry becomes -1 (skipped by the combine) and the status word records a bad-shape error.
__global__ void moe_permute_kernel(const uint4* __restrict__ x, int row_vecs, const int* __restrict__ ids,
                                   const int* __restrict__ offsets, int* __restrict__ cursor, long TK, int K, int E,
                                   uint4* __restrict__ xp, int* __restrict__ row_map, int* status) {
  const int lane = threadIdx.x & 31;
  const long warp = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const long nwarps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  for (long i = warp; i < TK; i += nwarps) {
    int pos = -1;
    if (lane == 0) {
      const int e = ids[i];
      if (e >= 0 && e < E) {
        pos = offsets[e] + atomicAdd(&cursor[e], 1);
      } else if (status) {
        atomicCAS(status, 0, TFB_ERR_BAD_SHAPE | (70 << 8));
      }
      row_map[i] = pos;
    }
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (pos < 0) continue;
    const uint4* src = x + (i / K) * row_vecs;
    uint4* dst = xp + static_cast<long>(pos) * row_vecs;
    for (int c = lane; c < row_vecs; c += 32) dst[c] = src[c];
  }
}

// out[t] = (residual[t]) + sum_k w[t,k] * y[row_map[t*K+k]]   (fp32 accumulate, bf16 in/out)
__global__ void moe_combine_kernel(const uint4* __restrict__ y, int row_vecs, const int* __restrict__ row_map,
                                   const float* __restrict__ w, int T, int K, const uint4* __restrict__ residual,
                                   uint4* __restrict__ out) {
  const long total = static_cast<long>(T) * row_vecs;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = i / row_vecs;
    const int c = static_cast<int>(i - t * row_vecs);
    float acc[8];
    if (residual) {
      const uint4 r = residual[i];
      const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(rp[k]);
        acc[2 * k] = f.x;
        acc[2 * k + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    }
    for (int k = 0; k < K; ++k) {
      const float wk = w[t * K + k];
      const int src_row = row_map[t * K + k];
      if (src_row < 0) continue;  // an expert id that the permute refused
      const uint4 v = y[static_cast<long>(src_row) * row_vecs + c];
      const __nv_bfloat162* vp = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(vp[j]);
        acc[2 * j] = fmaf(f.x, wk, acc[2 * j]);
        acc[2 * j + 1] = fmaf(f.y, wk, acc[2 * j + 1]);
      }
    }
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) op[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
    out[i] = o;
  }
}

static inline int moe_grid(long items, int per_block = 256, int max_blocks = 148 * 16) {
  long b = (items + per_block - 1) / per_block;
  return static_cast<int>(b < 1 ? 1 : (b > max_blocks ? max_blocks : b));
}

}  // namespace tfb

using namespace tfb;

extern "C" int tfb_moe_route(const float* logits, const float* bias, int T, int E, int num_groups, int topk_groups,
                             int K, float scale, int use_softmax, int* ids, float* weights, int* counts,
                             void* stream) {
  if (T <= 0) return TFB_OK;
  if (E < 1 || E > MOE_MAX_EXPERTS || K < 1 || K > 32 || K > E || num_groups < 1 || num_groups > 32 ||
      E % num_groups || topk_groups < 1 || topk_groups > num_groups)
    return TFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (counts) cudaMemsetAsync(counts, 0, sizeof(int) * E, st);
  const int warps = 8;
  const size_t smem = static_cast<size_t>(warps) * E * sizeof(float);
  const int grid = moe_grid(static_cast<long>(T) * 32, warps * 32);
  const int slots = (E + 31) / 32;
#define TFB_ROUTE(S_)                                                                                              \
  moe_route_kernel<S_><<<grid, warps * 32, smem, st>>>(logits, bias, T, E, num_groups, topk_groups, K, scale,      \
                                                       use_softmax, ids, weights, counts)
  if (slots <= 1) TFB_ROUTE(1);
  else if (slots <= 2) TFB_ROUTE(2);
  else if (slots <= 4) TFB_ROUTE(4);
  else if (slots <= 8) TFB_ROUTE(8);
  else if (slots <= 16) TFB_ROUTE(16);
  else TFB_ROUTE(32);
#undef TFB_ROUTE
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

extern "C" int tfb_moe_plan(const int* counts, int E, int align, int* offsets, int* tile_expert, int max_tiles,
                            void* stream) {
  if (E < 1 || E > MOE_MAX_EXPERTS || align < 1 || max_tiles < 0) return TFB_ERR_BAD_SHAPE;
  moe_plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts, E, align, offsets, tile_expert, max_tiles);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

// `cursor`: int[E] scratch supplied by the caller; zeroed here before the kernel runs.
extern "C" int tfb_moe_permute(const void* x, int hidden, const int* ids, const int* offsets, int* cursor, int E,
                               long T, int K, void* x_perm, int* row_map, void* stream) {
  if (T <= 0) return TFB_OK;
  if (hidden % 8 || E < 1 || K < 1 || !cursor) return TFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaMemsetAsync(cursor, 0, sizeof(int) * E, st);
  moe_permute_kernel<<<moe_grid(T * K * 32), 256, 0, st>>>(static_cast<const uint4*>(x), hidden / 8, ids, offsets,
                                                           cursor, T * K, K, E, static_cast<uint4*>(x_perm), row_map,
                                                           status_word());
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------------------------
// Variant of tfb_moe_permute that allocates nothing: the per-expert cursor lives in a fixed array in
// device memory instead of a caller-supplied buffer. See the declaration in tfb_api.h.
constexpr int MOE_STATIC_MAX_EXPERTS = 1024;  // 4 KB of scratch per device
static __device__ __align__(256) int g_moe_static_cursor[MOE_STATIC_MAX_EXPERTS];
constexpr int MOE_STATIC_MAX_DEVICES = 64;
static int* g_moe_static_cursor_ptr[MOE_STATIC_MAX_DEVICES] = {nullptr};

extern "C" int tfb_moe_permute_static(const void* x, int hidden, const int* ids, const int* offsets, int E, long T,
                                      int K, void* x_perm, int* row_map, void* stream) {
  if (T <= 0) return TFB_OK;
  if (hidden % 8 || E < 1 || K < 1) return TFB_ERR_BAD_SHAPE;
  if (E > MOE_STATIC_MAX_EXPERTS) {
    fprintf(stderr, "tfb_moe_permute_static: %d experts exceed the static scratch limit of %d; use tfb_moe_permute\n",
            E, MOE_STATIC_MAX_EXPERTS);
    return TFB_ERR_TOO_LARGE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MOE_STATIC_MAX_DEVICES) return TFB_ERR_LAUNCH;
  if (!g_moe_static_cursor_ptr[dev]) {
    // One-time set-up per device: address of this device's copy of the array.
    int* p = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_moe_static_cursor);
    if (err != cudaSuccess || !p) {
      fprintf(stderr, "tfb_moe_permute_static: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(err));
      return TFB_ERR_LAUNCH;
    }
    g_moe_static_cursor_ptr[dev] = p;
  }
  int* cursor = g_moe_static_cursor_ptr[dev];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The first E cursors must be zero when the kernel starts: cleared here, in stream order.
  if (cudaMemsetAsync(cursor, 0, sizeof(int) * E, st) != cudaSuccess) return TFB_ERR_LAUNCH;
  moe_permute_kernel<<<moe_grid(T * K * 32), 256, 0, st>>>(static_cast<const uint4*>(x), hidden / 8, ids, offsets,
                                                           cursor, T * K, K, E, static_cast<uint4*>(x_perm), row_map,
                                                           status_word());
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

extern "C" int tfb_moe_combine(const void* y, int hidden, const int* row_map, const float* weights, int T, int K,
                               const void* residual, void* out, void* stream) {
  if (T <= 0) return TFB_OK;
  if (hidden % 8 || K < 1) return TFB_ERR_BAD_SHAPE;
  moe_combine_kernel<<<moe_grid(static_cast<long>(T) * (hidden / 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(y), hidden / 8, row_map, weights, T, K, static_cast<const uint4*>(residual),
      static_cast<uint4*>(out));
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

// =============================================================================================
// Expert parallelism over peer-mapped memory: experts are split evenly over P ranks (rank o owns
// experts [o*E_loc, (o+1)*E_loc)). Dispatch = the permute kernel storing token rows straight into
// the owner's receive buffer; combine = the weighted sum loading expert outputs straight from the
// owners' output buffers. No all-to-all, no staging copies.
namespace tfb {

struct MoePeers {
  void* p[8];
};

// counts_all: int[P][E] (row s = histogram of rank s's tokens). One block.
//   dst_base[e]   : first row, in the owner's receive buffer, for THIS rank's tokens of expert e
//   tile_expert[m]: local expert id owning rows [m*align, (m+1)*align) of THIS rank's receive buffer, or -1
__global__ void moe_ep_plan_kernel(const int* __restrict__ counts_all, int P, int E, int E_loc, int my_rank, int align,
                                   int* __restrict__ dst_base, int* __restrict__ tile_expert, int max_tiles) {
  __shared__ int seg_off[MOE_MAX_EXPERTS + 1];  // per owner: aligned start of each of its local experts
  __shared__ int before_me[MOE_MAX_EXPERTS];    // rows of lower ranks inside the expert's segment
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int b = 0;
    for (int s = 0; s < my_rank; ++s) b += counts_all[s * E + e];
    before_me[e] = b;
  }
  __syncthreads();
  if (threadIdx.x < P) {  // thread o lays out owner o's buffer
    const int o = threadIdx.x;
    int acc = 0;
    for (int l = 0; l < E_loc; ++l) {
      const int e = o * E_loc + l;
      int tot = 0;
      for (int s = 0; s < P; ++s) tot += counts_all[s * E + e];
      seg_off[e] = acc;
      acc += (tot + align - 1) / align * align;
    }
    if (o == my_rank) seg_off[E] = acc;  // padded total of my own buffer
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) dst_base[e] = seg_off[e] + before_me[e];
  const int base = my_rank * E_loc;
  for (int m = threadIdx.x; m < max_tiles; m += blockDim.x) {
    const int row = m * align;
    int owner = -1;
    if (row < seg_off[E]) {
      int lo = 0, hi = E_loc - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (seg_off[base + mid] <= row) lo = mid; else hi = mid - 1;
      }
      owner = lo;
    }
    tile_expert[m] = owner;
  }
}

// One warp per (token, k). row_map[i] = (owner << 26) | row.
__global__ void moe_ep_dispatch_kernel(const uint4* __restrict__ x, int row_vecs, const int* __restrict__ ids,
                                       const int* __restrict__ dst_base, int* __restrict__ cursor, long TK, int K,
                                       int E_loc, MoePeers recv, int* __restrict__ row_map) {
  const int lane = threadIdx.x & 31;
  const long warp = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const long nwarps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  for (long i = warp; i < TK; i += nwarps) {
    int pos = 0, owner = 0;
    if (lane == 0) {
      const int e = ids[i];
      owner = e / E_loc;
      pos = dst_base[e] + atomicAdd(&cursor[e], 1);
      row_map[i] = (owner << 26) | pos;
    }
    pos = __shfl_sync(0xffffffffu, pos, 0);
    owner = __shfl_sync(0xffffffffu, owner, 0);
    const uint4* src = x + (i / K) * row_vecs;
    uint4* dst = static_cast<uint4*>(recv.p[owner]) + static_cast<long>(pos) * row_vecs;
    for (int c = lane; c < row_vecs; c += 32) dst[c] = src[c];
  }
}

__global__ void moe_ep_combine_kernel(MoePeers ybuf, int row_vecs, const int* __restrict__ row_map,
                                      const float* __restrict__ w, int T, int K, const uint4* __restrict__ residual,
                                      uint4* __restrict__ out) {
  const long total = static_cast<long>(T) * row_vecs;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = i / row_vecs;
    const int c = static_cast<int>(i - t * row_vecs);
    float acc[8];
    if (residual) {
      const uint4 r = residual[i];
      const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(rp[k]);
        acc[2 * k] = f.x, acc[2 * k + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    }
    for (int k = 0; k < K; ++k) {
      const float wk = w[t * K + k];
      if (wk == 0.f) continue;
      const int rm = row_map[t * K + k];
      const uint4 v = static_cast<const uint4*>(ybuf.p[rm >> 26])[static_cast<long>(rm & 0x3ffffff) * row_vecs + c];
      const __nv_bfloat162* vp = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(vp[j]);
        acc[2 * j] = fmaf(f.x, wk, acc[2 * j]);
        acc[2 * j + 1] = fmaf(f.y, wk, acc[2 * j + 1]);
      }
    }
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) op[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
    out[i] = o;
  }
}

}  // namespace tfb

extern "C" int tfb_moe_ep_plan(const int* counts_all, int P, int E, int my_rank, int align, int* dst_base,
                               int* tile_expert, int max_tiles, void* stream) {
  if (P < 1 || P > 8 || E < 1 || E > MOE_MAX_EXPERTS || E % P || my_rank < 0 || my_rank >= P || align < 1)
    return TFB_ERR_BAD_SHAPE;
  moe_ep_plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts_all, P, E, E / P, my_rank, align, dst_base,
                                                                     tile_expert, max_tiles);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

// recv: HOST array of P device pointers (every rank's receive buffer). cursor: int[E] scratch (zeroed here).
extern "C" int tfb_moe_ep_dispatch(const void* x, int hidden, const int* ids, const int* dst_base, int* cursor, int E,
                                   int P, long T, int K, void* const* recv, int* row_map, void* stream) {
  if (T <= 0) return TFB_OK;
  if (hidden % 8 || P < 1 || P > 8 || E % P || K < 1) return TFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MoePeers r;
  for (int i = 0; i < 8; ++i) r.p[i] = i < P ? recv[i] : nullptr;
  cudaMemsetAsync(cursor, 0, sizeof(int) * E, st);
  moe_ep_dispatch_kernel<<<moe_grid(T * K * 32), 256, 0, st>>>(static_cast<const uint4*>(x), hidden / 8, ids, dst_base,
                                                               cursor, T * K, K, E / P, r, row_map);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

// ybuf: HOST array of P device pointers (every rank's expert-output buffer).
extern "C" int tfb_moe_ep_combine(void* const* ybuf, int P, int hidden, const int* row_map, const float* weights, int T,
                                  int K, const void* residual, void* out, void* stream) {
  if (T <= 0) return TFB_OK;
  if (hidden % 8 || P < 1 || P > 8 || K < 1) return TFB_ERR_BAD_SHAPE;
  MoePeers y;
  for (int i = 0; i < 8; ++i) y.p[i] = i < P ? ybuf[i] : nullptr;
  moe_ep_combine_kernel<<<moe_grid(static_cast<long>(T) * (hidden / 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      y, hidden / 8, row_map, weights, T, K, static_cast<const uint4*>(residual), static_cast<uint4*>(out));
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}
