// Memory-bound fused ops of the DiT block, written for HBM3e streaming:
// 16-byte vector loads/stores, one pass over the activations, fp32 math.
//
//  * layernorm_modulate : LN (optional affine) -> y*(1+scale)+shift
//      (reference: LayerNorm + modulate, telefuser/ops/normalization.py:116-265,
//       Triton kernels telefuser/kernel/triton/scale_shift.py)
//  * rmsnorm_rope       : RMSNorm over H*D + interleaved-pair 3-D RoPE, in place
//      (reference: RMSNorm telefuser/ops/normalization.py:39-113 followed by
//       apply_rotary_emb telefuser/ops/rotary.py:105-135)
//  * gated_residual     : x + gate*y   (GateModule, telefuser/models/wan_video_dit.py:343-348)
//  * act_mul            : silu/gelu(x[:d]) * x[d:]   (telefuser/ops/activations.py:46-81)
//  * cfg_euler_step     : guidance + flow-matching Euler update in one pass
//      (telefuser/pipelines/wan_video/single_dit_denoising.py:131-158 and
//       telefuser/schedulers/flow_match.py:309-333)
//  * quant_mxfp8        : e4m3 + UE8M0/32 row-wise quantiser
#include "tfb_api.h"
#include "tfb_common.cuh"
#include "tfb_host.h"

namespace tfb {

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  f[0] = bf16_lo(u.x);
  f[1] = bf16_hi(u.x);
  f[2] = bf16_lo(u.y);
  f[3] = bf16_hi(u.y);
  f[4] = bf16_lo(u.z);
  f[5] = bf16_hi(u.z);
  f[6] = bf16_lo(u.w);
  f[7] = bf16_hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) t += red[i];
  return t;
}

// ---------------------------------------------------------------------------
// LayerNorm (+affine) (+modulate). One CTA of 256 threads walks LN_ROWS consecutive rows; NV uint4 per thread and
// row. The per-column factors (affine weight / bias, 1 + scale, shift) are folded into one multiplier and one
// addend per column, held in registers and rebuilt only when the modulation row changes: a row then costs its own
// 2 x C x 2 bytes of traffic instead of dragging 8 x C bytes of fp32 table through L1 with it. The next row is
// loaded (still packed) before the current one is reduced, so each thread keeps two rows of loads in flight.
// ---------------------------------------------------------------------------
constexpr int LN_ROWS = 16;
template <int NV>
__global__ void __launch_bounds__(256, NV >= 4 ? 1 : 2) layernorm_modulate_kernel(
    const __nv_bfloat16* __restrict__ x, long ldx, __nv_bfloat16* __restrict__ out, long ldo, int rows, int C,
    float eps, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
    const float* __restrict__ shift, const float* __restrict__ scale, long ldmod, int rows_per_mod) {
  __shared__ float red[2][16];
  const int row0 = blockIdx.x * LN_ROWS;
  const int row_end = min(rows, row0 + LN_ROWS);
  const int nvec = C >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float mul[NV][8], add[NV][8];
  long cached_mod = -1;
  uint4 nxt[NV];
  {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row0 * ldx);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * 256;
      nxt[i] = vi < nvec ? xr[vi] : make_uint4(0, 0, 0, 0);
    }
  }
  for (int row = row0; row < row_end; ++row) {
    float v[NV][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      unpack8(nxt[i], v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        s += v[i][e];
        ss = fmaf(v[i][e], v[i][e], ss);
      }
    }
    if (row + 1 < row_end) {
      const uint4* xr = reinterpret_cast<const uint4*>(x + (row + 1) * ldx);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = threadIdx.x + i * 256;
        nxt[i] = vi < nvec ? xr[vi] : make_uint4(0, 0, 0, 0);
      }
    }
    const long mod = row / rows_per_mod;
    if (mod != cached_mod) {
      cached_mod = mod;
      const long mrow = mod * ldmod;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = threadIdx.x + i * 256;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          mul[i][e] = 1.f;
          add[i][e] = 0.f;
        }
        if (vi < nvec) {
          if (w) unpack8(__ldg(reinterpret_cast<const uint4*>(w) + vi), mul[i]);
          if (b) unpack8(__ldg(reinterpret_cast<const uint4*>(b) + vi), add[i]);
          if (scale) {
            const float4* sp = reinterpret_cast<const float4*>(scale + mrow) + vi * 2;
            const float4 s0 = __ldg(sp), s1 = __ldg(sp + 1);
            const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {  // (y w + b)(1 + sc) = y (w (1 + sc)) + b (1 + sc)
              mul[i][e] *= (1.f + sc[e]);
              add[i][e] *= (1.f + sc[e]);
            }
          }
          if (shift) {
            const float4* sp = reinterpret_cast<const float4*>(shift + mrow) + vi * 2;
            const float4 s0 = __ldg(sp), s1 = __ldg(sp + 1);
            const float sh[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) add[i][e] += sh[e];
          }
        }
      }
    }
    // Mean and variance from one pass over the registers and ONE block reduction (sum and sum of squares side by
    // side; the scratch alternates between rows, so a row costs a single barrier). fp32 sums of bf16 data;
    // var = E[x^2] - mean^2, floored at 0.
    s = warp_sum(s);
    ss = warp_sum(ss);
    float* rd = red[(row - row0) & 1];
    if (lane == 0) {
      rd[warp] = s;
      rd[8 + warp] = ss;
    }
    __syncthreads();
    s = ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      s += rd[i];
      ss += rd[8 + i];
    }
    const float mean = s / C;
    const float rstd = rsqrtf(fmaxf(ss / C - mean * mean, 0.f) + eps);
    uint4* orow = reinterpret_cast<uint4*>(out + row * ldo);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * 256;
      if (vi < nvec) {
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = fmaf((v[i][e] - mean) * rstd, mul[i][e], add[i][e]);
        orow[vi] = pack8(y);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// RMSNorm over C = H*D + RoPE (interleaved pairs), in place.
// grid = (rows, nmat); 256 threads.
// ---------------------------------------------------------------------------
template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_rope_kernel(__nv_bfloat16* __restrict__ x, long ldx, long mat_stride,
                                                           int rows, int H, int D, float eps,
                                                           const __nv_bfloat16* __restrict__ w0,
                                                           const __nv_bfloat16* __restrict__ w1,
                                                           const float* __restrict__ cs, const float* __restrict__ sn) {
  __shared__ float red[8];
  const int row = blockIdx.x;
  const int mat = blockIdx.y;
  const int C = H * D;
  const int nvec = C >> 3;
  uint4* xr = reinterpret_cast<uint4*>(x + row * ldx + mat * mat_stride);
  const __nv_bfloat16* w = mat == 0 ? w0 : w1;
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      unpack8(xr[vi], v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  const float rstd = rsqrtf(block_sum<256>(ss, red) / C + eps);
  const int halfD = D >> 1;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      float y[8];
      float wf[8];
      if (w) {
        unpack8(__ldg(reinterpret_cast<const uint4*>(w) + vi), wf);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) wf[e] = 1.f;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = v[i][e] * rstd * wf[e];
      if (cs) {
        const int d0 = (vi * 8) % D;  // head-local element index, multiple of 8
        const float4 c4 = __ldg(reinterpret_cast<const float4*>(cs + static_cast<long>(row) * halfD + (d0 >> 1)));
        const float4 s4 = __ldg(reinterpret_cast<const float4*>(sn + static_cast<long>(row) * halfD + (d0 >> 1)));
        const float cc[4] = {c4.x, c4.y, c4.z, c4.w};
        const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float a = y[2 * p], bq = y[2 * p + 1];
          y[2 * p] = a * cc[p] - bq * sv[p];
          y[2 * p + 1] = a * sv[p] + bq * cc[p];
        }
      }
      xr[vi] = pack8(y);
    }
  }
}

// ---------------------------------------------------------------------------
// x + gate * y
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gated_residual_kernel(const uint4* __restrict__ x, const uint4* __restrict__ y,
                                                             uint4* __restrict__ out, long nvec_total, int vec_per_row,
                                                             const float* __restrict__ gate, long ldg,
                                                             int rows_per_gate) {
  for (long i = blockIdx.x * 256L + threadIdx.x; i < nvec_total; i += static_cast<long>(gridDim.x) * 256L) {
    float xf[8], yf[8];
    unpack8(x[i], xf);
    unpack8(y[i], yf);
    if (gate) {
      const long row = i / vec_per_row;
      const int vi = static_cast<int>(i - row * vec_per_row);
      const float4* gp = reinterpret_cast<const float4*>(gate + (row / rows_per_gate) * ldg) + vi * 2;
      const float4 g0 = __ldg(gp), g1 = __ldg(gp + 1);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) xf[e] += g[e] * yf[e];
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) xf[e] += yf[e];
    }
    out[i] = pack8(xf);
  }
}

// ---------------------------------------------------------------------------
// Row softmax in place: x[r, :] = softmax(scale * x[r, :]) over C columns (bf16 storage, fp32 maths). One CTA per
// row: an online max / sum pass, then the exponentials (the second read of the row comes from L1 / L2). Used by the
// unfused attention of heads wider than 128 (single-head VAE attention: scores GEMM -> this -> P.V GEMM).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) softmax_rows_kernel(__nv_bfloat16* __restrict__ x, long ldx, int C, float scale) {
  __shared__ float red_m[8], red_s[8];
  uint4* xr = reinterpret_cast<uint4*>(x + blockIdx.x * ldx);
  const int nvec = C >> 3;
  const float k = scale * 1.4426950408889634f;  // exponentials in base 2
  float m = -INFINITY, sum = 0.f;
  for (int vi = threadIdx.x; vi < nvec; vi += 256) {
    float f[8];
    unpack8(xr[vi], f);
    float cm = f[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) cm = fmaxf(cm, f[e]);
    cm *= k;  // k > 0 is required by the launcher, so the scaled maximum is the maximum of the scaled values
    if (cm > m) {
      sum *= fast_exp2(m - cm);
      m = cm;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) sum += fast_exp2(fmaf(f[e], k, -m));
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float wm = warp_max(m);
  sum = warp_sum(m == -INFINITY ? 0.f : sum * fast_exp2(m - wm));
  if (lane == 0) {
    red_m[warp] = wm;
    red_s[warp] = sum;
  }
  __syncthreads();
  float bm = red_m[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) bm = fmaxf(bm, red_m[i]);
  float bs = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) bs += red_m[i] == -INFINITY ? 0.f : red_s[i] * fast_exp2(red_m[i] - bm);
  const float inv = 1.f / bs;
  for (int vi = threadIdx.x; vi < nvec; vi += 256) {
    float f[8];
    unpack8(xr[vi], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = fast_exp2(fmaf(f[e], k, -bm)) * inv;
    xr[vi] = pack8(f);
  }
}

// ---------------------------------------------------------------------------
// act(x[:, :d]) * x[:, d:]
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) act_mul_kernel(const __nv_bfloat16* __restrict__ x,
                                                      __nv_bfloat16* __restrict__ out, long rows, int d, int act) {
  const int vec_per_row = d >> 3;
  const long total = rows * vec_per_row;
  for (long i = blockIdx.x * 256L + threadIdx.x; i < total; i += static_cast<long>(gridDim.x) * 256L) {
    const long row = i / vec_per_row;
    const int vi = static_cast<int>(i - row * vec_per_row);
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * 2L * d);
    float a[8], g[8];
    unpack8(xr[vi], a);
    unpack8(xr[vi + vec_per_row], g);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float t;
      if (act == 0)
        t = silu(a[e]);
      else if (act == 1)
        t = gelu_tanh(a[e]);
      else
        t = 0.5f * a[e] * (1.f + erff(a[e] * 0.70710678118654752f));
      a[e] = t * g[e];
    }
    reinterpret_cast<uint4*>(out + row * static_cast<long>(d))[vi] = pack8(a);
  }
}

// ---------------------------------------------------------------------------
// CFG combine + Euler step
// ---------------------------------------------------------------------------
template <bool BF16>
__global__ void __launch_bounds__(256) cfg_euler_kernel(const float* __restrict__ x, const void* __restrict__ cond,
                                                        const void* __restrict__ uncond, float s, float dsigma,
                                                        float* __restrict__ x_out, float* __restrict__ v_out, long n) {
  for (long i = blockIdx.x * 256L + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * 256L) {
    float c, u;
    if (BF16) {
      c = __bfloat162float(static_cast<const __nv_bfloat16*>(cond)[i]);
      u = uncond ? __bfloat162float(static_cast<const __nv_bfloat16*>(uncond)[i]) : c;
    } else {
      c = static_cast<const float*>(cond)[i];
      u = uncond ? static_cast<const float*>(uncond)[i] : c;
    }
    const float v = u + s * (c - u);
    if (v_out) v_out[i] = v;
    x_out[i] = x[i] + v * dsigma;
  }
}

// ---------------------------------------------------------------------------
// MXFP8 row-wise quantiser: one warp per 32-element block group; each lane
// owns 8 elements -> 4 lanes per 32-block.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quant_mxfp8_kernel(const __nv_bfloat16* __restrict__ x, long ldx,
                                                          uint8_t* __restrict__ q, uint8_t* __restrict__ sf, long rows,
                                                          int C, int tiled) {
  const int vec_per_row = C >> 3;
  const long total = rows * vec_per_row;
  const long total_pad = (total + 31) & ~31L;  // whole warps stay in the loop for the shuffles
  for (long i = blockIdx.x * 256L + threadIdx.x; i < total_pad; i += static_cast<long>(gridDim.x) * 256L) {
    const bool valid = i < total;
    const long row = valid ? i / vec_per_row : 0;
    const int vi = valid ? static_cast<int>(i - row * vec_per_row) : 0;
    float f[8];
    if (valid) {
      unpack8(reinterpret_cast<const uint4*>(x + row * ldx)[vi], f);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
    // 4 consecutive lanes form one 32-element block (vec_per_row is a multiple of 4).
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    // scale = 2^ceil(log2(amax / 448)), stored as biased exponent (UE8M0).
    int ebits = 0;
    if (amax > 0.f) {
      const float r = amax * (1.f / 448.f);
      const uint32_t rb = __float_as_uint(r);
      ebits = static_cast<int>((rb >> 23) & 0xff) + ((rb & 0x7fffff) ? 1 : 0);
      ebits = ebits < 1 ? 1 : (ebits > 253 ? 253 : ebits);
    } else {
      ebits = 127;
    }
    const float inv = __uint_as_float(static_cast<uint32_t>(254 - ebits) << 23);  // 2^-(ebits-127)
    uint32_t packed[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint16_t lo, hi;
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(f[h * 4 + 1] * inv), "f"(f[h * 4] * inv));
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(f[h * 4 + 3] * inv), "f"(f[h * 4 + 2] * inv));
      packed[h] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
    if (!valid) continue;
    reinterpret_cast<uint2*>(q + row * static_cast<long>(C))[vi] = make_uint2(packed[0], packed[1]);
    if ((vi & 3) == 0) {
      const int blk = vi >> 2;  // index of the 32-element block in the row
      if (tiled) {
        // Order read by the block-scaled MMA (gemm_mxfp8.cu): 512-byte tiles of 128 rows x 4 blocks.
        const long tile = (row >> 7) * (C >> 7) + (blk >> 2);
        sf[tile * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (blk & 3)] = static_cast<uint8_t>(ebits);
      } else {
        sf[row * (C >> 5) + blk] = static_cast<uint8_t>(ebits);
      }
    }
  }
}

static inline int grid_for(long work_items, int per_block = 256, int max_blocks = 148 * 16) {
  long b = (work_items + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return static_cast<int>(b);
}

}  // namespace tfb

using namespace tfb;

extern "C" int tfb_layernorm_modulate(const void* x, long ldx, void* out, long ldo, int rows, int C, float eps,
                                      const void* w, const void* b, const float* shift, const float* scale,
                                      long ldmod, int rows_per_mod, void* stream) {
  if (rows <= 0) return TFB_OK;
  if (C % 8 || C > 8192 || ldx % 8 || ldo % 8 || (ldmod % 4)) return TFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nv = (C / 8 + 255) / 256;
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(out);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
  const __nv_bfloat16* bp = static_cast<const __nv_bfloat16*>(b);
  if (rows_per_mod <= 0) rows_per_mod = 1;
#define TFB_LN_LAUNCH(NV_)                                                                                        \
  layernorm_modulate_kernel<NV_><<<(rows + LN_ROWS - 1) / LN_ROWS, 256, 0, st>>>(xp, ldx, op, ldo, rows, C, eps, wp, bp, shift, scale, ldmod, \
                                                       rows_per_mod)
  switch (nv) {
    case 1: TFB_LN_LAUNCH(1); break;
    case 2: TFB_LN_LAUNCH(2); break;
    case 3: TFB_LN_LAUNCH(3); break;
    default: TFB_LN_LAUNCH(4); break;
  }
#undef TFB_LN_LAUNCH
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

extern "C" int tfb_rmsnorm_rope(void* x, long ldx, long mat_stride, int nmat, int rows, int H, int D, float eps,
                                const void* w0, const void* w1, const float* cos, const float* sin, void* stream) {
  if (rows <= 0) return TFB_OK;
  const int C = H * D;
  if (C % 8 || C > 8192 || ldx % 8 || mat_stride % 8 || D % 8 || nmat < 1 || nmat > 2) return TFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nv = (C / 8 + 255) / 256;
  dim3 grid(rows, nmat);
  __nv_bfloat16* xp = static_cast<__nv_bfloat16*>(x);
  const __nv_bfloat16* w0p = static_cast<const __nv_bfloat16*>(w0);
  const __nv_bfloat16* w1p = static_cast<const __nv_bfloat16*>(w1);
#define TFB_RMS_LAUNCH(NV_) \
  rmsnorm_rope_kernel<NV_><<<grid, 256, 0, st>>>(xp, ldx, mat_stride, rows, H, D, eps, w0p, w1p, cos, sin)
  switch (nv) {
    case 1: TFB_RMS_LAUNCH(1); break;
    case 2: TFB_RMS_LAUNCH(2); break;
    case 3: TFB_RMS_LAUNCH(3); break;
    default: TFB_RMS_LAUNCH(4); break;
  }
#undef TFB_RMS_LAUNCH
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

extern "C" int tfb_gated_residual(const void* x, const void* y, void* out, int rows, int C, const float* gate,
                                  long ldg, int rows_per_gate, void* stream) {
  if (rows <= 0) return TFB_OK;
  if (C % 8 || (gate && ldg % 4)) return TFB_ERR_BAD_SHAPE;
  const long nvec = static_cast<long>(rows) * (C / 8);
  gated_residual_kernel<<<grid_for(nvec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), static_cast<const uint4*>(y), static_cast<uint4*>(out), nvec, C / 8, gate, ldg,
      rows_per_gate > 0 ? rows_per_gate : 1);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

extern "C" int tfb_softmax_rows(void* x, long ldx, int rows, int C, float scale, void* stream) {
  if (rows <= 0) return TFB_OK;
  if (C < 8 || C % 8 || ldx % 8 || !(scale > 0.f) || (reinterpret_cast<uintptr_t>(x) & 15)) return TFB_ERR_BAD_SHAPE;
  softmax_rows_kernel<<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<__nv_bfloat16*>(x), ldx, C, scale);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

extern "C" int tfb_act_mul(const void* x, void* out, int rows, int d, int act, void* stream) {
  if (rows <= 0) return TFB_OK;
  if (d % 8) return TFB_ERR_BAD_SHAPE;
  const long nvec = static_cast<long>(rows) * (d / 8);
  act_mul_kernel<<<grid_for(nvec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), rows, d, act);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

extern "C" int tfb_cfg_euler_step(const float* x, const void* cond, const void* uncond, int pred_is_bf16,
                                  float cfg_scale, float dsigma, float* x_out, float* v_out, long n, void* stream) {
  if (n <= 0) return TFB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (pred_is_bf16)
    cfg_euler_kernel<true><<<grid_for(n), 256, 0, st>>>(x, cond, uncond, cfg_scale, dsigma, x_out, v_out, n);
  else
    cfg_euler_kernel<false><<<grid_for(n), 256, 0, st>>>(x, cond, uncond, cfg_scale, dsigma, x_out, v_out, n);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

// tiled = 0: sf is [rows, C/32]; tiled = 1: sf is [ceil(rows/128)][C/128][512] in the order the block-scaled
// MMA reads (C a multiple of 128; bytes of rows past `rows` are left as they are).
extern "C" int tfb_quant_mxfp8(const void* x, long ldx, void* q, void* sf, int rows, int C, int tiled, void* stream) {
  if (rows <= 0) return TFB_OK;
  if (C % 32 || ldx % 8 || (tiled && C % 128)) return TFB_ERR_BAD_SHAPE;
  const long nvec = static_cast<long>(rows) * (C / 8);
  // Blocks must cover whole groups of 4 lanes: total is a multiple of 4 and
  // the grid-stride step (gridDim*256) keeps lane groups aligned.
  quant_mxfp8_kernel<<<grid_for(nvec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), rows, C, tiled);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------
// NF4 weights -> bf16. A code is a 4-bit index into 16 fixed levels (quantiles of a standard normal scaled to [-1, 1]);
// every `block` consecutive values share one fp32 absmax. Two codes per byte, the first in the high nibble.
// ---------------------------------------------------------------------------
__constant__ float kNF4Levels[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                     -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                     0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                                     0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

__global__ void __launch_bounds__(256) nf4_dequant_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ absmax,
                                                          __nv_bfloat16* __restrict__ out, long n_vec, int block) {
  __shared__ float lv[16];
  if (threadIdx.x < 16) lv[threadIdx.x] = kNF4Levels[threadIdx.x];
  __syncthreads();
  // one vector = 8 bytes = 16 values, which never straddles a block (block is a multiple of 16)
  for (long i = blockIdx.x * 256L + threadIdx.x; i < n_vec; i += static_cast<long>(gridDim.x) * 256L) {
    const uint2 raw = reinterpret_cast<const uint2*>(packed)[i];
    const float s = absmax[(i * 16) / block];
    const uint32_t w[2] = {raw.x, raw.y};
    uint32_t o[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t byte = (w[h] >> (8 * b)) & 0xffu;
        const __nv_bfloat162 v = __floats2bfloat162_rn(lv[byte >> 4] * s, lv[byte & 15u] * s);
        o[h * 4 + b] = *reinterpret_cast<const uint32_t*>(&v);
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + i * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

extern "C" int tfb_nf4_dequant(const void* packed, const float* absmax, void* out, long numel, int block, void* stream) {
  if (numel <= 0 || (numel & 15) || block < 16 || (block & 15)) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(packed) & 7) || (reinterpret_cast<uintptr_t>(out) & 15)) return TFB_ERR_BAD_SHAPE;
  const long n_vec = numel >> 4;
  nf4_dequant_kernel<<<grid_for(n_vec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(packed), absmax, static_cast<__nv_bfloat16*>(out), n_vec, block);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}
