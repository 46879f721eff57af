// Memory-bound kernels of the streaming / caching paths: rolling KV-cache shift + append, fp8 KV
// quantisation, log-sum-exp merge of partial attention results, Taylor feature-cache update / apply,
// Pluecker ray maps folded to the latent grid, decoded frames -> uint8 HWC.
// All are single-pass, 16-byte vectorised where the layout allows, grid-stride over 148 x 16 CTAs.
// Role in the reference: the torch-op KV-cache roll of the LingBot-World DiT (telefuser/models/lingbot_world_fast_dit.py),
// the fp8 KV cache of LiveAct (telefuser/cache/kv_cache.py), the Taylor cache arithmetic of
// telefuser/feature_cache/ada_taylor_cache/ada_taylor_cache.py, the Pluecker control maths of telefuser/pipelines/lingbot_world_fast/ and the
// Triton LSE-merge kernel its ring attention imports (`fused_merge_attn_states`, telefuser/distributed/ring.py:25).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tfb_api.h"
#include "tfb_common.cuh"

namespace tfb {

static inline int so_grid(long items, int per_block = 256, int max_blocks = 148 * 16) {
  long b = (items + per_block - 1) / per_block;
  return static_cast<int>(b < 1 ? 1 : (b > max_blocks ? max_blocks : b));
}

// ---------------------------------------------------------------------------------------------
// Rolling KV cache. Rows are tokens of `row_vecs` uint4 (H*D bf16 / 8). One launch copies the token
// range [src_tok, src_tok+ntok) of every batch entry to dst_tok for K and V at once. The launcher
// splits an overlapping left shift into stream-ordered launches whose source and destination ranges
// are disjoint (the shift distance is at least one chunk, so there are few of them).
__global__ void kv_copy_rows_kernel(uint4* __restrict__ kc, uint4* __restrict__ vc, const uint4* __restrict__ ks,
                                    const uint4* __restrict__ vs, long cache_bs, long src_bs, long src_ld,
                                    int dst_tok, int src_tok, int ntok, int row_vecs, int B) {
  const long per_b = static_cast<long>(ntok) * row_vecs;
  const long total = per_b * B;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int b = static_cast<int>(i / per_b);
    const long r = i - b * per_b;
    const int t = static_cast<int>(r / row_vecs);
    const int c = static_cast<int>(r - static_cast<long>(t) * row_vecs);
    const long d = b * cache_bs + (static_cast<long>(dst_tok) + t) * row_vecs + c;
    const long s = b * src_bs + (static_cast<long>(src_tok) + t) * src_ld + c;
    kc[d] = ks[s];
    vc[d] = vs[s];
  }
}

// ---------------------------------------------------------------------------------------------
// fp8 KV quantisation: one warp per (token, head) row of D bf16; scale = amax / 448 (floor 1e-12).
__global__ void fp8_kv_quant_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                    float* __restrict__ scale, long rows, int D) {
  const int lane = threadIdx.x & 31;
  const long warp = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const long nwarps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  const int per_lane = D / 32;  // 2, 4 or 8
  for (long r = warp; r < rows; r += nwarps) {
    const __nv_bfloat16* xr = x + r * D + lane * per_lane;
    float f[8];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (i < per_lane) {
        f[i] = __bfloat162float(xr[i]);
        amax = fmaxf(amax, fabsf(f[i]));
      }
    }
    amax = warp_max(amax);
    const float s = fmaxf(amax * (1.f / 448.f), 1e-12f);
    // The oracle divides in the input dtype: x / bf16(s).
    const float sb = __bfloat162float(__float2bfloat16(s));
    uint8_t* qr = q + r * D + lane * per_lane;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (i < per_lane) {
        const float v = __bfloat162float(__float2bfloat16(__fdiv_rn(f[i], sb)));
        qr[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
      }
    }
    if (lane == 0) scale[r] = s;
  }
}

// ---------------------------------------------------------------------------------------------
// Merge of two partial attention results: o* [B,S,H,D] bf16, lse* [B,H,S] fp32 (natural log).
__global__ void merge_attn_states_kernel(const uint4* __restrict__ o1, const float* __restrict__ l1,
                                         const uint4* __restrict__ o2, const float* __restrict__ l2,
                                         uint4* __restrict__ out, float* __restrict__ lse_out, int B, int S, int H,
                                         int dvec) {
  const long total = static_cast<long>(B) * S * H * dvec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % dvec);
    const long row = i / dvec;  // (b, s, h)
    const int h = static_cast<int>(row % H);
    const long bs = row / H;
    const int s = static_cast<int>(bs % S);
    const int b = static_cast<int>(bs / S);
    const long li = (static_cast<long>(b) * H + h) * S + s;
    const float a = l1[li], bb = l2[li];
    const float m = fmaxf(a, bb);
    const float w1 = __expf(a - m), w2 = __expf(bb - m);
    const float inv = 1.f / (w1 + w2);
    const uint4 u = o1[i], v = o2[i];
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    const __nv_bfloat162* vp = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint4 r;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = __bfloat1622float2(up[k]), y = __bfloat1622float2(vp[k]);
      rp[k] = __floats2bfloat162_rn((x.x * w1 + y.x * w2) * inv, (x.y * w1 + y.y * w2) * inv);
    }
    out[i] = r;
    if (c == 0 && lse_out) lse_out[li] = m + __logf(w1 + w2);
  }
}

// ---------------------------------------------------------------------------------------------
// Taylor feature cache. Terms t[0..order) are bf16 buffers of n elements.
//   update: r = out - ori;  new[0] = r;  new[i+1] = (new[i] - old[i]) / window   (in place on t[i])
//   apply : y = x + sum_i t[i] * coef[i]
struct TaylorPtrs {
  __nv_bfloat16* t[4];
};

__global__ void taylor_update_kernel(const uint4* __restrict__ out, const uint4* __restrict__ ori, TaylorPtrs p,
                                     int n_old, int n_new, float window, long nvec) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const uint4 a = out[i], b = ori[i];
    const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
    float cur[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = __bfloat1622float2(ap[k]), y = __bfloat1622float2(bp[k]);
      // the oracle forms the residual in bf16
      cur[2 * k] = __bfloat162float(__float2bfloat16(x.x - y.x));
      cur[2 * k + 1] = __bfloat162float(__float2bfloat16(x.y - y.y));
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      if (t >= n_new) break;
      uint4* tp = reinterpret_cast<uint4*>(p.t[t]) + i;
      float old[8];
      const bool has_old = t < n_old && t + 1 < n_new;
      if (has_old) {
        const uint4 o = *tp;
        const __nv_bfloat162* op = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 x = __bfloat1622float2(op[k]);
          old[2 * k] = x.x;
          old[2 * k + 1] = x.y;
        }
      }
      uint4 w;
      __nv_bfloat162* wp = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
      for (int k = 0; k < 4; ++k) wp[k] = __floats2bfloat162_rn(cur[2 * k], cur[2 * k + 1]);
      *tp = w;
      if (!has_old) break;
#pragma unroll
      for (int k = 0; k < 8; ++k)
        cur[k] = __bfloat162float(
            __float2bfloat16(__fdiv_rn(__bfloat162float(__float2bfloat16(cur[k] - old[k])), window)));
    }
  }
}

__global__ void taylor_apply_kernel(const uint4* __restrict__ x, TaylorPtrs p, float c0, float c1, float c2, float c3,
                                    int nterms, uint4* __restrict__ y, long nvec) {
  const float coef[4] = {c0, c1, c2, c3};
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      if (t >= nterms) break;
      const uint4 v = reinterpret_cast<const uint4*>(p.t[t])[i];
      const __nv_bfloat162* vp = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(vp[k]);
        acc[2 * k] = fmaf(f.x, coef[t], acc[2 * k]);
        acc[2 * k + 1] = fmaf(f.y, coef[t], acc[2 * k + 1]);
      }
    }
    const uint4 xv = x[i];
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
    uint4 r;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(xp[k]);
      rp[k] = __floats2bfloat162_rn(f.x + acc[2 * k], f.y + acc[2 * k + 1]);
    }
    y[i] = r;
  }
}

// ---------------------------------------------------------------------------------------------
// Pluecker ray maps folded to the latent grid.
//   c2w  : fp32 [F, 4, 4] camera-to-world;  ks: fp32 [F, 4] = fx, fy, cx, cy (pixels of the HxW image)
//   extra: optional fp32 [F, n_extra] per-frame channels appended after the ray channels (actions)
//   out  : fp32 [(C) * c1 * c2, F, h, w], C = (only_d ? 3 : 6) + n_extra, channel = (c * c1 + i1) * c2 + i2,
//          pixel (y*c1 + i1, x*c2 + i2), centre at +0.5
__global__ void plucker_fold_kernel(const float* __restrict__ c2w, const float* __restrict__ ks,
                                    const float* __restrict__ extra, int n_extra, float* __restrict__ out, int F, int h,
                                    int w, int c1, int c2, int only_d) {
  const long total = static_cast<long>(F) * h * c1 * w * c2;
  const long plane = static_cast<long>(F) * h * w;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    // decompose with x fastest so that stores of one (channel, i1, i2) are coalesced
    long r = i;
    const int x = static_cast<int>(r % w);
    r /= w;
    const int y = static_cast<int>(r % h);
    r /= h;
    const int f = static_cast<int>(r % F);
    r /= F;
    const int i2 = static_cast<int>(r % c2);
    const int i1 = static_cast<int>(r / c2);
    const float* M = c2w + f * 16;
    const float fx = ks[f * 4], fy = ks[f * 4 + 1], cx = ks[f * 4 + 2], cy = ks[f * 4 + 3];
    const float px = static_cast<float>(x * c2 + i2) + 0.5f, py = static_cast<float>(y * c1 + i1) + 0.5f;
    float d0 = __fdiv_rn(px - cx, fx), d1 = __fdiv_rn(py - cy, fy), d2 = 1.f;
    const float nrm = __fsqrt_rn(d0 * d0 + d1 * d1 + d2 * d2);
    d0 = __fdiv_rn(d0, nrm);
    d1 = __fdiv_rn(d1, nrm);
    d2 = __fdiv_rn(d2, nrm);
    float v[6];
    v[0] = M[3];
    v[1] = M[7];
    v[2] = M[11];
    v[3] = d0 * M[0] + d1 * M[1] + d2 * M[2];
    v[4] = d0 * M[4] + d1 * M[5] + d2 * M[6];
    v[5] = d0 * M[8] + d1 * M[9] + d2 * M[10];
    const long pix = (static_cast<long>(f) * h + y) * w + x;
    const int sub = i1 * c2 + i2, nsub = c1 * c2;
    const int nray = only_d ? 3 : 6;
    for (int c = 0; c < nray; ++c) out[(static_cast<long>(c) * nsub + sub) * plane + pix] = v[only_d ? c + 3 : c];
    for (int e = 0; e < n_extra; ++e)
      out[(static_cast<long>(nray + e) * nsub + sub) * plane + pix] = extra[f * n_extra + e];
  }
}

// ---------------------------------------------------------------------------------------------
// Decoded frames [3, T, H, W] in [-1, 1] -> uint8 [T, H, W, 3]; 4 pixels per thread (W % 4 == 0).
template <typename T>
__device__ __forceinline__ void load4(const T* p, float* f);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float* f) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
  const float2 a = __bfloat1622float2(b[0]), c = __bfloat1622float2(b[1]);
  f[0] = a.x, f[1] = a.y, f[2] = c.x, f[3] = c.y;
}

template <typename T>
__global__ void frames_to_u8_kernel(const T* __restrict__ in, uint8_t* __restrict__ out, long plane /* T*H*W */) {
  const long nq = plane / 4;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nq;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float c[3][4];
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) load4<T>(in + ch * plane + i * 4, c[ch]);
    uint8_t b[12];
#pragma unroll
    for (int p = 0; p < 4; ++p)
#pragma unroll
      for (int ch = 0; ch < 3; ++ch) {
        const float v = fminf(fmaxf((c[ch][p] + 1.f) * 127.5f, 0.f), 255.f);
        b[p * 3 + ch] = static_cast<uint8_t>(__float2int_rn(v));
      }
    uint32_t* o = reinterpret_cast<uint32_t*>(out + i * 12);
    o[0] = b[0] | (b[1] << 8) | (b[2] << 16) | (static_cast<uint32_t>(b[3]) << 24);
    o[1] = b[4] | (b[5] << 8) | (b[6] << 16) | (static_cast<uint32_t>(b[7]) << 24);
    o[2] = b[8] | (b[9] << 8) | (b[10] << 16) | (static_cast<uint32_t>(b[11]) << 24);
  }
}

}  // namespace tfb

using namespace tfb;

#define TFB_LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH)

extern "C" int tfb_kv_cache_roll_append(void* k_cache, void* v_cache, long cache_bs, const void* new_k,
                                        const void* new_v, long new_ld, long new_bs, int B, int row_elems, int sink,
                                        int evicted, int keep, int local_start, int n_new, void* stream) {
  if (row_elems % 8 || cache_bs % 8 || new_ld % 8 || new_bs % 8 || evicted < 0 || keep < 0 || n_new < 0 || B < 1)
    return TFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rv = row_elems / 8;
  uint4* kc = static_cast<uint4*>(k_cache);
  uint4* vc = static_cast<uint4*>(v_cache);
  if (evicted > 0 && keep > 0) {
    // Left shift by `evicted` tokens in pieces of at most `evicted` tokens: each piece reads
    // [dst+evicted, dst+evicted+len) and writes [dst, dst+len), which never overlap, and pieces run
    // in stream order from the left, so a piece's source is never overwritten before it is read.
    for (int done = 0; done < keep; done += evicted) {
      const int len = keep - done < evicted ? keep - done : evicted;
      kv_copy_rows_kernel<<<so_grid(static_cast<long>(len) * rv * B), 256, 0, st>>>(
          kc, vc, kc, vc, cache_bs / 8, cache_bs / 8, rv, sink + done, sink + done + evicted, len, rv, B);
    }
  }
  if (n_new > 0)
    kv_copy_rows_kernel<<<so_grid(static_cast<long>(n_new) * rv * B), 256, 0, st>>>(
        kc, vc, static_cast<const uint4*>(new_k), static_cast<const uint4*>(new_v), cache_bs / 8, new_bs / 8,
        new_ld / 8, local_start, 0, n_new, rv, B);
  return TFB_LAUNCH_OK();
}

extern "C" int tfb_fp8_kv_quant(const void* x, void* q, float* scale, long rows, int D, void* stream) {
  if (rows <= 0) return TFB_OK;
  if (D % 32 || D > 256) return TFB_ERR_BAD_SHAPE;
  fp8_kv_quant_kernel<<<so_grid(rows * 32), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scale, rows, D);
  return TFB_LAUNCH_OK();
}

extern "C" int tfb_merge_attn_states(const void* o1, const float* lse1, const void* o2, const float* lse2, void* out,
                                     float* lse_out, int B, int S, int H, int D, void* stream) {
  if (D % 8) return TFB_ERR_BAD_SHAPE;
  const long total = static_cast<long>(B) * S * H * (D / 8);
  if (total <= 0) return TFB_OK;
  merge_attn_states_kernel<<<so_grid(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(o1), lse1, static_cast<const uint4*>(o2), lse2, static_cast<uint4*>(out), lse_out, B, S,
      H, D / 8);
  return TFB_LAUNCH_OK();
}

extern "C" int tfb_taylor_update(const void* out, const void* ori, void* t0, void* t1, void* t2, void* t3, int n_old,
                                 int n_new, float window, long n, void* stream) {
  if (n % 8 || n_new < 1 || n_new > 4 || n_old < 0 || n_old > 4) return TFB_ERR_BAD_SHAPE;
  TaylorPtrs p;
  p.t[0] = static_cast<__nv_bfloat16*>(t0), p.t[1] = static_cast<__nv_bfloat16*>(t1);
  p.t[2] = static_cast<__nv_bfloat16*>(t2), p.t[3] = static_cast<__nv_bfloat16*>(t3);
  taylor_update_kernel<<<so_grid(n / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(out), static_cast<const uint4*>(ori), p, n_old, n_new, window, n / 8);
  return TFB_LAUNCH_OK();
}

extern "C" int tfb_taylor_apply(const void* x, const void* t0, const void* t1, const void* t2, const void* t3,
                                float c0, float c1, float c2, float c3, int nterms, void* y, long n, void* stream) {
  if (n % 8 || nterms < 1 || nterms > 4) return TFB_ERR_BAD_SHAPE;
  TaylorPtrs p;
  p.t[0] = static_cast<__nv_bfloat16*>(const_cast<void*>(t0)), p.t[1] = static_cast<__nv_bfloat16*>(const_cast<void*>(t1));
  p.t[2] = static_cast<__nv_bfloat16*>(const_cast<void*>(t2)), p.t[3] = static_cast<__nv_bfloat16*>(const_cast<void*>(t3));
  taylor_apply_kernel<<<so_grid(n / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), p, c0, c1, c2, c3, nterms, static_cast<uint4*>(y), n / 8);
  return TFB_LAUNCH_OK();
}

extern "C" int tfb_plucker_fold(const float* c2w, const float* ks, const float* extra, int n_extra, float* out, int F,
                                int h, int w, int c1, int c2, int only_d, void* stream) {
  if (F < 1 || h < 1 || w < 1 || c1 < 1 || c2 < 1 || n_extra < 0 || (n_extra > 0 && !extra)) return TFB_ERR_BAD_SHAPE;
  const long total = static_cast<long>(F) * h * c1 * w * c2;
  plucker_fold_kernel<<<so_grid(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(c2w, ks, extra, n_extra, out, F,
                                                                                     h, w, c1, c2, only_d);
  return TFB_LAUNCH_OK();
}

extern "C" int tfb_frames_to_u8(const void* frames, int is_bf16, void* out, int T, int H, int W, void* stream) {
  const long plane = static_cast<long>(T) * H * W;
  if (plane <= 0) return TFB_OK;
  if (W % 4) return TFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    frames_to_u8_kernel<__nv_bfloat16><<<so_grid(plane / 4), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(frames),
                                                                           static_cast<uint8_t*>(out), plane);
  else
    frames_to_u8_kernel<float><<<so_grid(plane / 4), 256, 0, st>>>(static_cast<const float*>(frames),
                                                                   static_cast<uint8_t*>(out), plane);
  return TFB_LAUNCH_OK();
}
