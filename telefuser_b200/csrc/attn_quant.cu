// Int8 quantisation of attention operands (head_dim 128).
//   k_stats       : per (batch, head, channel) sum of K over tokens and per (batch, head) max |K|, one pass
//   quant_q_int8  : per (token, head) scale = max|q| / 127, q8 = round(q / scale)
//   quant_k_int8  : k8 = round((k - mean_k) / k_scale) with one scale per (batch, head)
// Subtracting the per-channel mean of K over the tokens leaves softmax(Q.K^T) unchanged (it shifts every score of
// a query row by the same amount) and removes the common offset that would otherwise eat most of the 8-bit range.
// The roles of tf-kernel/csrc/sageattn2/fused/fused.cu:66-333 (per-block int8 quantisers, K mean subtraction).
#include "tfb_api.h"
#include "tfb_common.cuh"
#include "tfb_host.h"

namespace tfb {

__device__ __forceinline__ void unpack8_bf16(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = bf16_lo(w[i]);
    f[2 * i + 1] = bf16_hi(w[i]);
  }
}

// grid (token chunks, B), 256 threads. Each thread owns vector columns tid, tid + 256, ... of the H*128-wide row and
// walks the chunk's tokens, so that a warp always reads 512 consecutive bytes of one token.
__global__ void __launch_bounds__(256) k_stats_kernel(const uint4* __restrict__ k, long ld_vec, long bs_vec, int S,
                                                      int row_vecs, int rows_per_block, float* __restrict__ sums,
                                                      unsigned int* __restrict__ amax_bits, int H) {
  const int b = blockIdx.y;
  const int s0 = blockIdx.x * rows_per_block;
  const int s1 = min(S, s0 + rows_per_block);
  const uint4* base = k + b * bs_vec;
  for (int v = threadIdx.x; v < row_vecs; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float mx = 0.f;
    for (int s = s0; s < s1; ++s) {
      float f[8];
      unpack8_bf16(base[static_cast<long>(s) * ld_vec + v], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        acc[e] += f[e];
        mx = fmaxf(mx, fabsf(f[e]));
      }
    }
    float* dst = sums + (static_cast<long>(b) * row_vecs + v) * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) atomicAdd(dst + e, acc[e]);
    atomicMax(amax_bits + b * H + v / 16, __float_as_uint(mx));  // non-negative floats order like their bit patterns
  }
}

__device__ __forceinline__ uint2 pack_int8x8(const float (&f)[8], float inv) {
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    int q[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = __float2int_rn(f[h * 4 + e] * inv);
      q[e] = max(-127, min(127, r)) & 0xff;
    }
    w[h] = static_cast<uint32_t>(q[0]) | (static_cast<uint32_t>(q[1]) << 8) | (static_cast<uint32_t>(q[2]) << 16) |
           (static_cast<uint32_t>(q[3]) << 24);
  }
  return make_uint2(w[0], w[1]);
}

// One half-warp (16 lanes x 8 elements) per (token, head). items = B * S * H.
// IS_K: subtract mean[b, h, :] and use the head's scale; else per-(token, head) scale written to scale_out[b, h, s].
template <bool IS_K>
__global__ void __launch_bounds__(256) quant_qk_int8_kernel(const uint4* __restrict__ x, long ld_vec, long bs_vec,
                                                            uint2* __restrict__ out, long items, int S, int H,
                                                            const float* __restrict__ mean,
                                                            const float* __restrict__ k_scale,
                                                            float* __restrict__ scale_out) {
  const int lane16 = threadIdx.x & 15;
  const long half_warps = (static_cast<long>(gridDim.x) * blockDim.x) >> 4;
  const long items_pad = (items + 1) & ~1L;  // both halves of a warp stay in the loop for the shuffles
  for (long i = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 4; i < items_pad; i += half_warps) {
    const bool valid = i < items;
    const long ii = valid ? i : 0;
    const int h = static_cast<int>(ii % H);
    const long bs_i = ii / H;
    const int s = static_cast<int>(bs_i % S);
    const int b = static_cast<int>(bs_i / S);
    float f[8];
    unpack8_bf16(x[b * bs_vec + static_cast<long>(s) * ld_vec + h * 16 + lane16], f);
    float inv;
    if (IS_K) {
      const float4* mp = reinterpret_cast<const float4*>(mean + (static_cast<long>(b) * H + h) * 128 + lane16 * 8);
      const float4 m0 = __ldg(mp), m1 = __ldg(mp + 1);
      f[0] -= m0.x, f[1] -= m0.y, f[2] -= m0.z, f[3] -= m0.w;
      f[4] -= m1.x, f[5] -= m1.y, f[6] -= m1.z, f[7] -= m1.w;
      inv = 1.f / __ldg(k_scale + b * H + h);
    } else {
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float sc = fmaxf(amax * (1.f / 127.f), 1e-12f);
      inv = 1.f / sc;
      if (valid && lane16 == 0) scale_out[(static_cast<long>(b) * H + h) * S + s] = sc;
    }
    if (valid) out[(static_cast<long>(b) * S + s) * (H * 16) + h * 16 + lane16] = pack_int8x8(f, inv);
  }
}

static inline int quant_grid(long work_items, int per_block) {
  long blocks = (work_items + per_block - 1) / per_block;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

}  // namespace tfb

using namespace tfb;

// k: bf16 [B, S, H, 128] (token stride ld, batch stride bs, in elements). sums fp32 [B, H*128] and amax fp32 [B, H]
// are zeroed here and accumulated with atomics (amax as the bit pattern of a non-negative float).
extern "C" int tfb_attn_k_stats(const void* k, long ld, long bs, int B, int S, int H, float* sums, float* amax,
                                void* stream) {
  if (B <= 0 || S <= 0 || H <= 0 || ld % 8 || bs % 8 || (reinterpret_cast<uintptr_t>(k) & 15)) return TFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaMemsetAsync(sums, 0, sizeof(float) * B * H * 128, st);
  cudaMemsetAsync(amax, 0, sizeof(float) * B * H, st);
  const int rows_per_block = 64;
  dim3 grid((S + rows_per_block - 1) / rows_per_block, B);
  k_stats_kernel<<<grid, 256, 0, st>>>(static_cast<const uint4*>(k), ld / 8, bs / 8, S, H * 16, rows_per_block, sums,
                                       reinterpret_cast<unsigned int*>(amax), H);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

// x: bf16 [B, S, H, 128] strided as above -> out int8 [B, S, H, 128] contiguous.
//   is_k = 0: per-(token, head) scales written to scale_out fp32 [B, H, S].
//   is_k = 1: out = round((x - mean[b, h, :]) / k_scale[b, h]); mean fp32 [B, H, 128], k_scale fp32 [B, H].
extern "C" int tfb_attn_quant_int8(const void* x, long ld, long bs, void* out, int B, int S, int H, int is_k,
                                   const float* mean, const float* k_scale, float* scale_out, void* stream) {
  if (B <= 0 || S <= 0 || H <= 0 || ld % 8 || bs % 8) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) return TFB_ERR_BAD_SHAPE;
  if (is_k ? (!mean || !k_scale || (reinterpret_cast<uintptr_t>(mean) & 15)) : !scale_out) return TFB_ERR_BAD_SHAPE;
  const long items = static_cast<long>(B) * S * H;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = quant_grid(items * 16, 256);
  if (is_k)
    quant_qk_int8_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint4*>(x), ld / 8, bs / 8,
                                                     static_cast<uint2*>(out), items, S, H, mean, k_scale, nullptr);
  else
    quant_qk_int8_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint4*>(x), ld / 8, bs / 8,
                                                      static_cast<uint2*>(out), items, S, H, nullptr, nullptr, scale_out);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}
