// Memory-bound glue of the video VAE on channels-last tensors (a "row" is the C channels of one pixel):
//   pixel_norm_act     : y = act(x / max(|x|_2, 1e-12) * sqrt(C) * gamma[c]), act = SiLU or identity
//   upsample2x_nearest : [N, H, W, C] -> [N, 2H, 2W, C], out(h, w) = in(h / 2, w / 2)
// One read and one write per element each; the reference's VAE spends several full passes on the same work
// (F.normalize, the gamma product, SiLU and an fp32 round trip for the upsample:
// telefuser/models/wan_video_vae.py:118-217).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tfb_api.h"
#include "tfb_common.cuh"

namespace tfb {

// A group of G lanes owns one pixel; lane l of the group holds vectors l, l + G, ... (NV of them, 8 channels each),
// so a warp-wide load touches 32 / G consecutive pixels' worth of contiguous bytes. C = 8 * G * NV.
template <int G, int NV, bool SILU>
__global__ void __launch_bounds__(256) pixel_norm_act_kernel(const uint4* __restrict__ x, uint4* __restrict__ out,
                                                             long pixels, const float* __restrict__ gamma, float scale) {
  const int lane_g = threadIdx.x % G;
  const long group = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) / G;
  const long groups = (static_cast<long>(gridDim.x) * blockDim.x) / G;
  float gm[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const float4* gp = reinterpret_cast<const float4*>(gamma + (lane_g + i * G) * 8);
    const float4 a = __ldg(gp), b = __ldg(gp + 1);
    gm[i][0] = a.x * scale, gm[i][1] = a.y * scale, gm[i][2] = a.z * scale, gm[i][3] = a.w * scale;
    gm[i][4] = b.x * scale, gm[i][5] = b.y * scale, gm[i][6] = b.z * scale, gm[i][7] = b.w * scale;
  }
  const long pixels_pad = (pixels + (32 / G) - 1) / (32 / G) * (32 / G);  // whole warps stay in the loop
  for (long pix = group; pix < pixels_pad; pix += groups) {
    const bool valid = pix < pixels;
    const uint4* row = x + (valid ? pix : 0) * (G * NV);
    float v[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const uint4 u = row[lane_g + i * G];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[i][2 * e] = bf16_lo(w[e]);
        v[i][2 * e + 1] = bf16_hi(w[e]);
        ss = fmaf(v[i][2 * e], v[i][2 * e], ss);
        ss = fmaf(v[i][2 * e + 1], v[i][2 * e + 1], ss);
      }
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.f / fmaxf(sqrtf(ss), 1e-12f);
    if (!valid) continue;
    uint4* orow = out + pix * (G * NV);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float y[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        y[e] = v[i][e] * inv * gm[i][e];
        if (SILU) y[e] = y[e] / (1.f + __expf(-y[e]));
      }
      uint4 o;
      o.x = pack_bf16x2(y[0], y[1]), o.y = pack_bf16x2(y[2], y[3]);
      o.z = pack_bf16x2(y[4], y[5]), o.w = pack_bf16x2(y[6], y[7]);
      orow[lane_g + i * G] = o;
    }
  }
}

__global__ void __launch_bounds__(256) upsample2x_kernel(const uint4* __restrict__ x, uint4* __restrict__ out, long N,
                                                         int H, int W, int cvec) {
  const long total = N * (2L * H) * (2L * W) * cvec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % cvec);
    long r = i / cvec;
    const int w = static_cast<int>(r % (2 * W));
    r /= 2 * W;
    const int h = static_cast<int>(r % (2 * H));
    const long n = r / (2 * H);
    out[i] = x[((n * H + (h >> 1)) * W + (w >> 1)) * cvec + c];
  }
}

static inline int vae_grid(long threads_wanted) {
  long b = (threads_wanted + 255) / 256;
  return static_cast<int>(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace tfb

using namespace tfb;

// x, out: bf16 [pixels, C] contiguous; gamma fp32 [C]. C / 8 must be G * NV with G a power of two <= 32 and NV <= 4:
// 16, 32, 64, 96, 128, 192, 256, 384, 512, ... (the widths of the Wan VAEs).
extern "C" int tfb_pixel_norm_act(const void* x, void* out, long pixels, int C, const float* gamma, int silu,
                                  void* stream) {
  if (pixels <= 0) return TFB_OK;
  if (C % 8 || (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(gamma)) & 15)
    return TFB_ERR_BAD_SHAPE;
  const int vecs = C / 8;
  int G = 1;
  while (G < 32 && vecs % (G * 2) == 0) G *= 2;
  const int NV = vecs / G;
  if (NV > 4) return TFB_ERR_BAD_SHAPE;
  const float scale = sqrtf(static_cast<float>(C));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = vae_grid(pixels * G);
  const uint4* xp = static_cast<const uint4*>(x);
  uint4* op = static_cast<uint4*>(out);
#define TFB_PNA(G_, NV_)                                                                                         \
  if (G == G_ && NV == NV_) {                                                                                    \
    if (silu)                                                                                                    \
      pixel_norm_act_kernel<G_, NV_, true><<<grid, 256, 0, st>>>(xp, op, pixels, gamma, scale);                   \
    else                                                                                                         \
      pixel_norm_act_kernel<G_, NV_, false><<<grid, 256, 0, st>>>(xp, op, pixels, gamma, scale);                  \
    return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;                                          \
  }
  TFB_PNA(2, 1) TFB_PNA(4, 1) TFB_PNA(8, 1) TFB_PNA(16, 1) TFB_PNA(32, 1) TFB_PNA(32, 2) TFB_PNA(4, 3) TFB_PNA(8, 3)
  TFB_PNA(16, 3) TFB_PNA(32, 3) TFB_PNA(1, 1) TFB_PNA(1, 3) TFB_PNA(2, 3) TFB_PNA(32, 4)
#undef TFB_PNA
  return TFB_ERR_BAD_SHAPE;
}

// x bf16 [N, H, W, C] -> out [N, 2H, 2W, C], C % 8 == 0.
extern "C" int tfb_upsample2x_nearest(const void* x, void* out, long N, int H, int W, int C, void* stream) {
  if (N <= 0 || H <= 0 || W <= 0) return TFB_OK;
  if (C % 8 || (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) return TFB_ERR_BAD_SHAPE;
  const long total = N * 4L * H * W * (C / 8);
  upsample2x_kernel<<<vae_grid(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), static_cast<uint4*>(out), N, H, W, C / 8);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}
