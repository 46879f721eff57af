// RMSNorm-based block glue of sandwich-norm DiTs (RMSNorm before and after every sub-layer, tanh gates):
//   rmsnorm_modulate      : out = (w * x * rstd) * (1 + scale) + shift
//   rmsnorm_gate_residual : out = res + tanh(gate) * (w * y * rstd)
//   headnorm_rope         : per-head RMSNorm of q and k (weight [D]) + interleaved-pair RoPE, in place
// Row kernels use one CTA of 256 threads per token row (C <= 8192); the head kernel one warp per
// (token, head). bf16 activations, fp32 statistics, fp32 modulation / gate tables.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tfb_api.h"
#include "tfb_common.cuh"

namespace tfb {

__device__ __forceinline__ void r_unpack8(const uint4& u, float (&f)[8]) {
  f[0] = bf16_lo(u.x), f[1] = bf16_hi(u.x), f[2] = bf16_lo(u.y), f[3] = bf16_hi(u.y);
  f[4] = bf16_lo(u.z), f[5] = bf16_hi(u.z), f[6] = bf16_lo(u.w), f[7] = bf16_hi(u.w);
}
__device__ __forceinline__ uint4 r_pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]), u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]), u.w = pack_bf16x2(f[6], f[7]);
  return u;
}
__device__ __forceinline__ float r_block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) t += red[i];
  return t;
}
__device__ __forceinline__ void load_f8(const float* p, float (&f)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
}

// MODE 0: modulate (aux0 = shift, aux1 = scale; either may be null)
// MODE 1: gated residual (res + tanh?(gate) * normed; aux0 = gate or null, res required)
template <int NV, int MODE>
__global__ void __launch_bounds__(256) rmsnorm_row_kernel(const __nv_bfloat16* __restrict__ x, long ldx,
                                                          const __nv_bfloat16* __restrict__ res, long ldr,
                                                          __nv_bfloat16* __restrict__ out, long ldo, int C, float eps,
                                                          const float* __restrict__ w, const float* __restrict__ aux0,
                                                          const float* __restrict__ aux1, long ldaux, int rows_per_aux,
                                                          int tanh_gate) {
  __shared__ float red[8];
  const long row = blockIdx.x;
  const int nvec = C >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      r_unpack8(xr[vi], v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  const float rstd = rsqrtf(r_block_sum(ss, red) / C + eps);
  const long arow = (row / rows_per_aux) * ldaux;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      float wf[8], y[8];
      if (w) {
        load_f8(w + vi * 8, wf);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) wf[e] = 1.f;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = v[i][e] * rstd * wf[e];
      if (MODE == 0) {
        if (aux1) {
          float sc[8];
          load_f8(aux1 + arow + vi * 8, sc);
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] *= 1.f + sc[e];
        }
        if (aux0) {
          float sh[8];
          load_f8(aux0 + arow + vi * 8, sh);
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] += sh[e];
        }
      } else {
        float r[8];
        r_unpack8(reinterpret_cast<const uint4*>(res + row * ldr)[vi], r);
        if (aux0) {
          float g[8];
          load_f8(aux0 + arow + vi * 8, g);
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] = r[e] + (tanh_gate ? tanhf(g[e]) : g[e]) * y[e];
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] += r[e];
        }
      }
      reinterpret_cast<uint4*>(out + row * ldo)[vi] = r_pack8(y);
    }
  }
}

// One warp per (row, head, matrix); PL = D / 32 elements per lane (2, 4, 6 or 8), pairs stay in a lane.
template <int PL>
__global__ void headnorm_rope_kernel(__nv_bfloat16* __restrict__ x, long ldx, long mat_stride, int nmat, long rows,
                                     int H, float eps, const float* __restrict__ w0, const float* __restrict__ w1,
                                     const float* __restrict__ cs, const float* __restrict__ sn) {
  constexpr int D = PL * 32;
  const int lane = threadIdx.x & 31;
  const long warp = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const long nwarps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  const long total = rows * H * nmat;
  for (long i = warp; i < total; i += nwarps) {
    const int mat = static_cast<int>(i % nmat);
    const long rh = i / nmat;
    const int h = static_cast<int>(rh % H);
    const long row = rh / H;
    __nv_bfloat16* p = x + row * ldx + mat * mat_stride + h * D + lane * PL;
    float v[PL];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < PL; e += 2) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + e));
      v[e] = f.x, v[e + 1] = f.y;
      ss += f.x * f.x + f.y * f.y;
    }
    const float rstd = rsqrtf(warp_sum(ss) / D + eps);
    const float* w = mat == 0 ? w0 : w1;
#pragma unroll
    for (int e = 0; e < PL; ++e) v[e] *= rstd * (w ? __ldg(w + lane * PL + e) : 1.f);
    if (cs) {
      const long t = row * (D / 2) + lane * (PL / 2);
#pragma unroll
      for (int e = 0; e < PL; e += 2) {
        const float c = __ldg(cs + t + e / 2), s = __ldg(sn + t + e / 2);
        const float a = v[e], b = v[e + 1];
        v[e] = a * c - b * s;
        v[e + 1] = a * s + b * c;
      }
    }
#pragma unroll
    for (int e = 0; e < PL; e += 2) *reinterpret_cast<__nv_bfloat162*>(p + e) = __floats2bfloat162_rn(v[e], v[e + 1]);
  }
}

// Per-token 8-bit quantisation for the W8A8 GEMMs. FP8: q = e4m3(x / s), s = max(row amax / 448, 1e-12);
// INT8: q = round(x / s) in [-127, 127], s = max(row amax / 127, 1e-12). One CTA per row. With NV > 0 the row
// (up to 2048 * NV elements) stays in registers between the amax pass and the conversion, so it is read from
// memory once; NV == 0 is the any-width form that reads the row twice (the second read hits L1 / L2).
template <bool INT8>
__device__ __forceinline__ uint2 quant8_pack(const float (&f)[8], float inv) {
  if (INT8) {
    uint32_t b[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      int v;
      asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(v) : "f"(fminf(fmaxf(f[e] * inv, -127.f), 127.f)));
      b[e] = static_cast<uint32_t>(v) & 0xffu;
    }
    return make_uint2(b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24), b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24));
  }
  uint16_t h[4];
#pragma unroll
  for (int e = 0; e < 4; ++e)
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h[e]) : "f"(f[2 * e + 1] * inv), "f"(f[2 * e] * inv));
  return make_uint2(static_cast<uint32_t>(h[0]) | (static_cast<uint32_t>(h[1]) << 16),
                    static_cast<uint32_t>(h[2]) | (static_cast<uint32_t>(h[3]) << 16));
}

template <int NV, bool INT8>
__global__ void __launch_bounds__(256) quant_fp8_row_kernel(const __nv_bfloat16* __restrict__ x, long ldx,
                                                            uint8_t* __restrict__ q, long ldq,
                                                            float* __restrict__ scale, int C) {
  __shared__ float red[8];
  const long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  const int nvec = C >> 3;
  constexpr int NR = NV > 0 ? NV : 1;
  uint4 held[NR];
  float amax = 0.f;
  if (NV > 0) {
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int vi = threadIdx.x + i * 256;
      held[i] = vi < nvec ? xr[vi] : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      float f[8];
      r_unpack8(held[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
    }
  } else {
    for (int vi = threadIdx.x; vi < nvec; vi += 256) {
      float f[8];
      r_unpack8(xr[vi], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
    }
  }
  amax = warp_max(amax);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float s = fmaxf(amax * (INT8 ? 1.f / 127.f : 1.f / 448.f), 1e-12f);
  const float inv = __fdiv_rn(1.f, s);
  if (threadIdx.x == 0) scale[row] = s;
  uint2* qr = reinterpret_cast<uint2*>(q + row * ldq);
  if (NV > 0) {
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int vi = threadIdx.x + i * 256;
      if (vi < nvec) {
        float f[8];
        r_unpack8(held[i], f);
        qr[vi] = quant8_pack<INT8>(f, inv);
      }
    }
  } else {
    for (int vi = threadIdx.x; vi < nvec; vi += 256) {
      float f[8];
      r_unpack8(xr[vi], f);
      qr[vi] = quant8_pack<INT8>(f, inv);
    }
  }
}

// Per-tensor FP8 quantisation: one scale for the whole tensor. Pass 1 reduces |x| to a single maximum (the bit
// pattern of a non-negative float orders like an unsigned integer, so atomicMax on the bits is exact); pass 2
// converts with s = max(amax / 448, 1e-12) read from device memory, so a static (calibrated) scale skips pass 1.
__global__ void __launch_bounds__(256) absmax_kernel(const __nv_bfloat16* __restrict__ x, long n8, long n,
                                                     unsigned* __restrict__ amax_bits) {
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  float amax = 0.f;
  for (long i = blockIdx.x * 256L + threadIdx.x; i < n8; i += gridDim.x * 256L) {
    float f[8];
    r_unpack8(xv[i], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
  }
  if (blockIdx.x == 0)
    for (long i = n8 * 8 + threadIdx.x; i < n; i += 256) amax = fmaxf(amax, fabsf(__bfloat162float(x[i])));
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0 && amax > 0.f) atomicMax(amax_bits, __float_as_uint(amax));
}
__global__ void __launch_bounds__(256) quant_fp8_tensor_kernel(const __nv_bfloat16* __restrict__ x, long n8, long n,
                                                               uint8_t* __restrict__ q, float* __restrict__ scale,
                                                               const unsigned* __restrict__ amax_bits) {
  float s;
  if (amax_bits) {
    s = fmaxf(__uint_as_float(*amax_bits) * (1.f / 448.f), 1e-12f);
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale = s;
  } else {
    s = *scale;
  }
  const float inv = __fdiv_rn(1.f, s);
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  uint2* qv = reinterpret_cast<uint2*>(q);
  for (long i = blockIdx.x * 256L + threadIdx.x; i < n8; i += gridDim.x * 256L) {
    float f[8];
    r_unpack8(xv[i], f);
    qv[i] = quant8_pack<false>(f, inv);
  }
  if (blockIdx.x == 0)
    for (long i = n8 * 8 + threadIdx.x; i < n; i += 256) {
      uint16_t h;
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h) : "f"(0.f), "f"(__bfloat162float(x[i]) * inv));
      q[i] = static_cast<uint8_t>(h & 0xff);
    }
}

}  // namespace tfb

using namespace tfb;

template <bool INT8>
static int launch_quant_row8(const void* x, long ldx, void* q, long ldq, float* scale, int rows, int C, void* stream) {
  if (rows <= 0) return TFB_OK;
  if (C % 8 || ldx % 8 || ldq % 8) return TFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  uint8_t* qp = static_cast<uint8_t*>(q);
  const int nv = (C / 8 + 255) / 256;
#define TFB_Q8(NV_) quant_fp8_row_kernel<NV_, INT8><<<rows, 256, 0, st>>>(xp, ldx, qp, ldq, scale, C)
  switch (nv) {
    case 1: TFB_Q8(1); break;
    case 2: TFB_Q8(2); break;
    case 3: TFB_Q8(3); break;
    case 4: TFB_Q8(4); break;
    case 5: case 6: TFB_Q8(6); break;
    case 7: case 8: TFB_Q8(8); break;
    default: TFB_Q8(0); break;
  }
#undef TFB_Q8
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

extern "C" int tfb_quant_fp8_rowwise(const void* x, long ldx, void* q, long ldq, float* scale, int rows, int C,
                                     void* stream) {
  return launch_quant_row8<false>(x, ldx, q, ldq, scale, rows, C, stream);
}

// Per-token int8 quantisation (symmetric, [-127, 127]); the reference's per-token int8 path
// (tf-kernel/csrc/gemm/per_token_group_quant_8bit.cu with a whole-row group).
extern "C" int tfb_quant_int8_rowwise(const void* x, long ldx, void* q, long ldq, float* scale, int rows, int C,
                                      void* stream) {
  return launch_quant_row8<true>(x, ldx, q, ldq, scale, rows, C, stream);
}

// Per-tensor FP8 quantisation of n contiguous bf16 values. `scale` (device, one float) receives the scale; with
// is_static != 0 it is read instead (a calibrated scale) and no reduction runs. `scratch` is one device word used
// for the reduction (cleared here, stream-ordered). Role of tf-kernel/csrc/gemm/per_tensor_quant_fp8.cu.
extern "C" int tfb_quant_fp8_per_tensor(const void* x, void* q, float* scale, unsigned* scratch, long n, int is_static,
                                        void* stream) {
  if (n <= 0) return TFB_OK;
  if (!scale || (!is_static && !scratch)) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7)) return TFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const long n8 = n / 8;
  long blocks = (n8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  if (!is_static) {
    if (cudaMemsetAsync(scratch, 0, sizeof(unsigned), st) != cudaSuccess) return TFB_ERR_LAUNCH;
    absmax_kernel<<<blocks, 256, 0, st>>>(xp, n8, n, scratch);
  }
  quant_fp8_tensor_kernel<<<blocks, 256, 0, st>>>(xp, n8, n, static_cast<uint8_t*>(q), scale,
                                                  is_static ? nullptr : scratch);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

template <int MODE>
static int launch_rms_row(const void* x, long ldx, const void* res, long ldr, void* out, long ldo, int rows, int C,
                          float eps, const float* w, const float* a0, const float* a1, long ldaux, int rows_per_aux,
                          int tanh_gate, void* stream) {
  if (rows <= 0) return TFB_OK;
  if (C % 8 || C > 8192 || ldx % 8 || ldo % 8 || ldaux % 4 || (MODE == 1 && (!res || ldr % 8))) return TFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nv = (C / 8 + 255) / 256;
  if (rows_per_aux <= 0) rows_per_aux = 1;
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* rp = static_cast<const __nv_bfloat16*>(res);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(out);
#define TFB_RMS_ROW(NV_)                                                                                         \
  rmsnorm_row_kernel<NV_, MODE><<<rows, 256, 0, st>>>(xp, ldx, rp, ldr, op, ldo, C, eps, w, a0, a1, ldaux,         \
                                                      rows_per_aux, tanh_gate)
  switch (nv) {
    case 1: TFB_RMS_ROW(1); break;
    case 2: TFB_RMS_ROW(2); break;
    case 3: TFB_RMS_ROW(3); break;
    default: TFB_RMS_ROW(4); break;
  }
#undef TFB_RMS_ROW
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

extern "C" int tfb_rmsnorm_modulate(const void* x, long ldx, void* out, long ldo, int rows, int C, float eps,
                                    const float* w, const float* shift, const float* scale, long ldmod,
                                    int rows_per_mod, void* stream) {
  return launch_rms_row<0>(x, ldx, nullptr, 0, out, ldo, rows, C, eps, w, shift, scale, ldmod, rows_per_mod, 0, stream);
}

extern "C" int tfb_rmsnorm_gate_residual(const void* y, long ldy, const void* res, long ldr, void* out, long ldo,
                                         int rows, int C, float eps, const float* w, const float* gate, long ldg,
                                         int rows_per_gate, int tanh_gate, void* stream) {
  return launch_rms_row<1>(y, ldy, res, ldr, out, ldo, rows, C, eps, w, gate, nullptr, ldg, rows_per_gate, tanh_gate,
                           stream);
}

extern "C" int tfb_headnorm_rope(void* x, long ldx, long mat_stride, int nmat, long rows, int H, int D, float eps,
                                 const float* w0, const float* w1, const float* cos, const float* sin, void* stream) {
  if (rows <= 0) return TFB_OK;
  if (D % 64 || D > 256 || ldx % 2 || mat_stride % 2 || nmat < 1 || nmat > 2 || H < 1) return TFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long warps = rows * H * nmat;
  long blocks = (warps + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  __nv_bfloat16* xp = static_cast<__nv_bfloat16*>(x);
  switch (D / 32) {
    case 2: headnorm_rope_kernel<2><<<blocks, 256, 0, st>>>(xp, ldx, mat_stride, nmat, rows, H, eps, w0, w1, cos, sin); break;
    case 4: headnorm_rope_kernel<4><<<blocks, 256, 0, st>>>(xp, ldx, mat_stride, nmat, rows, H, eps, w0, w1, cos, sin); break;
    case 6: headnorm_rope_kernel<6><<<blocks, 256, 0, st>>>(xp, ldx, mat_stride, nmat, rows, H, eps, w0, w1, cos, sin); break;
    default: headnorm_rope_kernel<8><<<blocks, 256, 0, st>>>(xp, ldx, mat_stride, nmat, rows, H, eps, w0, w1, cos, sin); break;
  }
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}
