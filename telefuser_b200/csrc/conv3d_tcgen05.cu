// Causal 3-D convolution (stride 1) as an implicit GEMM on tcgen05, channels-last.
//
//   x    [B, T, H, W, Cin]  bf16      prev [B, Tp, H, W, Cin] (optional: the frames before x, from the last chunk)
//   w    [Cout, kt*kh*kw, Cin] bf16   out  [B, T, H, W, Cout] = conv(x) + bias (+ residual)
//
// An output tile is 128 pixels of one frame (8 rows x 16 columns) by BN output channels. The reduction runs over
// filter taps x blocks of 64 input channels; for one tap the A operand of the MMA is simply the same 8 x 16 pixel
// box of the input shifted by the tap's offset, which a 5-D tiled TMA load delivers in exactly the K-major,
// 128B-swizzled form the tensor core reads (128 rows = pixels, 64 channels = 128 bytes per row). Coordinates that
// fall outside the tensor are filled with zeros by the TMA unit, so spatial zero padding and the causal padding in
// time cost nothing: no padded copy of the input is ever made. Frames before t = 0 come from `prev` through a
// second tensor map when the caller streams chunk by chunk (no concatenation either).
//
// Roles (192 threads): warp 0 producer (TMA), warp 1 MMA issuer + TMEM owner, warps 2..5 epilogue (bias, residual,
// bf16 stores straight to the pixel's row). Persistent over tiles, accumulator double-buffered in TMEM.
// Replaces the cuDNN convolutions of the reference's VAE (telefuser/models/wan_video_vae.py:92-115, 396-501).
#include "tfb_api.h"
#include "tfb_common.cuh"
#include "tfb_host.h"

namespace tfb {

constexpr int CONV_TH = 8, CONV_TW = 16;  // pixel tile: 8 rows x 16 columns = 128 GEMM rows

struct ConvParams {
  int B, T, H, W, Cin, Cout;
  int kt, kh, kw;
  int pad_t, pad_h, pad_w;  // zeros (or `prev` frames) in front of t = 0; symmetric spatial padding
  int prev_T;               // frames in `prev` (0: none)
  __nv_bfloat16* out;
  const __nv_bfloat16* bias;   // [Cout] or null
  const __nv_bfloat16* resid;  // same layout as out, or null
  int tiles_h, tiles_w, m_tiles, n_tiles;
  int* status;
};

template <int BN>
struct ConvCfg {
  static constexpr int BK = 64;  // input channels per pipeline stage
  static constexpr int STAGES = 6;
  static constexpr int A_BYTES = 128 * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512));
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
  static_assert(B_BYTES % 1024 == 0, "stages must keep the 1024-byte alignment of swizzled tiles");
};

__device__ __forceinline__ void tma_load_5d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2,
                                            int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
      "r"(c3), "r"(c4)
      : "memory");
}

template <int BN>
__global__ void __launch_bounds__(192, 1)
    conv3d_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmPrev,
                  const __grid_constant__ CUtensorMap tmW, const ConvParams p) {
  using Cfg = ConvCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  AbortCtx ctx{abort_flag, p.status};
  const int cta = blockIdx.x, n_cta = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.m_tiles * p.n_tiles;
  const int taps = p.kt * p.kh * p.kw;
  const int c_blocks = (p.Cin + Cfg::BK - 1) / Cfg::BK;
  const int k_iters = taps * c_blocks;
  // Tile t -> (output-channel block, batch, frame, first row, first column); channel blocks vary fastest so that the
  // CTAs running together share input boxes in L2.
  auto map_tile = [&](int t, int& n_blk, int& b, int& f, int& h0, int& w0) {
    n_blk = t % p.n_tiles;
    int m = t / p.n_tiles;
    w0 = (m % p.tiles_w) * CONV_TW;
    m /= p.tiles_w;
    h0 = (m % p.tiles_h) * CONV_TH;
    m /= p.tiles_h;
    f = m % p.T;
    b = m / p.T;
  };

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmX);
      tma_prefetch_desc(&tmW);
      if (p.prev_T > 0) tma_prefetch_desc(&tmPrev);
      uint32_t it = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += n_cta) {
        int n_blk, b, f, h0, w0;
        map_tile(t, n_blk, b, f, h0, w0);
        for (int tap = 0; tap < taps && ok; ++tap) {
          const int dt = tap / (p.kh * p.kw);
          const int dh = (tap / p.kw) % p.kh;
          const int dw = tap % p.kw;
          int t_in = f + dt - p.pad_t;
          const CUtensorMap* src = &tmX;
          if (t_in < 0 && p.prev_T > 0) {  // a frame of the previous chunk (or, further back still, zeros)
            src = &tmPrev;
            t_in += p.prev_T;
          }
          const int h_in = h0 + dh - p.pad_h, w_in = w0 + dw - p.pad_w;
          for (int cb = 0; cb < c_blocks; ++cb, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            if (!mbar_wait(&empty[s], ph ^ 1, ctx, 51)) {
              ok = false;
              break;
            }
            uint8_t* a_dst = smem + s * Cfg::STAGE_BYTES;
            uint8_t* b_dst = a_dst + Cfg::A_BYTES;
            mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
            tma_load_5d(a_dst, src, &full[s], cb * Cfg::BK, w_in, h_in, t_in, b);
            tma_load_3d(b_dst, &tmW, &full[s], cb * Cfg::BK, tap, n_blk * BN);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc = make_idesc(128, BN, 1, 1, 0, 0);
    uint32_t it = 0, tile_iter = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += n_cta) {
      const uint32_t acc = tile_iter & 1;
      const uint32_t accph = (tile_iter >> 1) & 1;
      ++tile_iter;
      if (!mbar_wait_warp(&tempty[acc], accph ^ 1, ctx, 52)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int ki = 0; ki < k_iters; ++ki, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait_warp(&full[s], ph, ctx, 53)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < Cfg::BK / 16; ++kk)
            umma_f16_ss(d_tmem, make_desc_k_sw128(a_addr + kk * 32), make_desc_k_sw128(b_addr + kk * 32), idesc,
                        (ki | kk) != 0 ? 1u : 0u);
          umma_commit(&empty[s]);
          if (ki == k_iters - 1) umma_commit(&tfull[acc]);
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3;
    uint32_t tile_iter = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += n_cta) {
      int n_blk, b, f, h0, w0;
      map_tile(t, n_blk, b, f, h0, w0);
      const uint32_t acc = tile_iter & 1;
      const uint32_t accph = (tile_iter >> 1) & 1;
      ++tile_iter;
      if (!mbar_wait_warp(&tfull[acc], accph, ctx, 54)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int r = q * 32 + lane;  // GEMM row = pixel of the tile
      const int h = h0 + r / CONV_TW, w = w0 + r % CONV_TW;
      const bool row_ok = h < p.H && w < p.W;
      const size_t pix = ((static_cast<size_t>(b) * p.T + f) * p.H + (row_ok ? h : 0)) * p.W + (row_ok ? w : 0);
      __nv_bfloat16* out_row = p.out + pix * p.Cout;
      const __nv_bfloat16* res_row = p.resid ? p.resid + pix * p.Cout : nullptr;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v32[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32, v32);
        tmem_ld_wait();
        const int col0 = n_blk * BN + c * 32;
        if (!row_ok || col0 >= p.Cout) continue;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(v32[i]);
        if (col0 + 32 <= p.Cout) {
          if (p.bias) {
            const uint4* bp = reinterpret_cast<const uint4*>(p.bias + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 bb = __ldg(bp + j);
              const uint32_t wv[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                v[j * 8 + e * 2] += bf16_lo(wv[e]);
                v[j * 8 + e * 2 + 1] += bf16_hi(wv[e]);
              }
            }
          }
          if (res_row) {
            const uint4* rp = reinterpret_cast<const uint4*>(res_row + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 bb = rp[j];
              const uint32_t wv[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                v[j * 8 + e * 2] += bf16_lo(wv[e]);
                v[j * 8 + e * 2 + 1] += bf16_hi(wv[e]);
              }
            }
          }
          uint4* op = reinterpret_cast<uint4*>(out_row + col0);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16x2(v[j * 8], v[j * 8 + 1]);
            o.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
            o.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
            o.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
            op[j] = o;
          }
        } else {
          for (int i = 0; i < 32; ++i) {  // ragged channel edge (e.g. the 3 output channels of the last layer)
            const int col = col0 + i;
            if (col >= p.Cout) break;
            float xv = v[i];
            if (p.bias) xv += __bfloat162float(p.bias[col]);
            if (res_row) xv += __bfloat162float(res_row[col]);
            out_row[col] = __float2bfloat16(xv);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  if (*abort_flag) __nanosleep(200000);  // let copies in flight land before the CTA exits
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

template <int BN>
static int launch_conv(const CUtensorMap& tmX, const CUtensorMap& tmPrev, const void* w, ConvParams p, cudaStream_t st) {
  using Cfg = ConvCfg<BN>;
  CUtensorMap tmW;
  {
    const int taps = p.kt * p.kh * p.kw;
    uint64_t dims[3] = {static_cast<uint64_t>(p.Cin), static_cast<uint64_t>(taps), static_cast<uint64_t>(p.Cout)};
    uint64_t str[2] = {static_cast<uint64_t>(p.Cin) * 2, static_cast<uint64_t>(taps) * p.Cin * 2};
    uint32_t box[3] = {64u, 1u, static_cast<uint32_t>(BN)};
    if (int e = make_tmap(&tmW, w, TM_BF16, 3, dims, str, box, TM_SW_128)) return e;
  }
  p.n_tiles = (p.Cout + BN - 1) / BN;
  static bool attr_set[TFB_MAX_DEVICES] = {false};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&conv3d_kernel<BN>), Cfg::SMEM_BYTES, attr_set)) return rc;
  const long tiles = static_cast<long>(p.m_tiles) * p.n_tiles;
  const int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
  conv3d_kernel<BN><<<grid, 192, Cfg::SMEM_BYTES, st>>>(tmX, tmPrev, tmW, p);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

static int make_act_tmap(CUtensorMap* m, const void* base, int B, int T, int H, int W, int C) {
  uint64_t dims[5] = {static_cast<uint64_t>(C), static_cast<uint64_t>(W), static_cast<uint64_t>(H),
                      static_cast<uint64_t>(T), static_cast<uint64_t>(B)};
  uint64_t str[4] = {static_cast<uint64_t>(C) * 2, static_cast<uint64_t>(W) * C * 2,
                     static_cast<uint64_t>(H) * W * C * 2, static_cast<uint64_t>(T) * H * W * C * 2};
  uint32_t box[5] = {64u, CONV_TW, CONV_TH, 1u, 1u};
  return make_tmap(m, base, TM_BF16, 5, dims, str, box, TM_SW_128);
}

}  // namespace tfb

using namespace tfb;

// x [B, T, H, W, Cin], prev [B, prev_T, H, W, Cin] or null, w [Cout, kt*kh*kw, Cin], out / resid [B, T, H, W, Cout];
// all bf16, contiguous. Cin and Cout multiples of 8. pad_t frames of padding in front (the first prev_T of them read
// from `prev`, the rest zeros); pad_h / pad_w on both sides. The output has the input's T, H and W, so
// pad_t = kt - 1, pad_h = (kh - 1) / 2, pad_w = (kw - 1) / 2 for a "same" causal convolution.
extern "C" int tfb_conv3d_causal(const void* x, const void* prev, int prev_T, const void* w, const void* bias,
                                 const void* resid, void* out, int B, int T, int H, int W, int Cin, int Cout, int kt,
                                 int kh, int kw, int pad_t, int pad_h, int pad_w, void* stream) {
  if (B <= 0 || T <= 0 || H <= 0 || W <= 0) return TFB_OK;
  if (Cin < 8 || Cin % 8 || Cout < 1 || (Cout % 8 && Cout > 32) || kt < 1 || kh < 1 || kw < 1 || kt * kh * kw > 125)
    return TFB_ERR_BAD_SHAPE;
  if (pad_t < 0 || pad_h < 0 || pad_w < 0 || prev_T < 0 || prev_T > pad_t || (prev_T > 0 && !prev)) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(prev) | reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(resid)) & 15)
    return TFB_ERR_BAD_SHAPE;
  CUtensorMap tmX, tmPrev;
  if (int e = make_act_tmap(&tmX, x, B, T, H, W, Cin)) return e;
  if (int e = make_act_tmap(&tmPrev, prev_T > 0 ? prev : x, B, prev_T > 0 ? prev_T : T, H, W, Cin)) return e;
  ConvParams p;
  p.B = B, p.T = T, p.H = H, p.W = W, p.Cin = Cin, p.Cout = Cout;
  p.kt = kt, p.kh = kh, p.kw = kw;
  p.pad_t = pad_t, p.pad_h = pad_h, p.pad_w = pad_w;
  p.prev_T = prev_T;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.resid = static_cast<const __nv_bfloat16*>(resid);
  p.tiles_h = (H + CONV_TH - 1) / CONV_TH;
  p.tiles_w = (W + CONV_TW - 1) / CONV_TW;
  const long m_tiles = static_cast<long>(B) * T * p.tiles_h * p.tiles_w;
  if (m_tiles * ((Cout + 31) / 32) > 0x7fffffffL) return TFB_ERR_TOO_LARGE;
  p.m_tiles = static_cast<int>(m_tiles);
  p.n_tiles = 0;
  p.status = status_word();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (Cout <= 32) return launch_conv<32>(tmX, tmPrev, w, p, st);
  if (Cout % 128 == 0 || Cout > 192) return launch_conv<128>(tmX, tmPrev, w, p, st);
  if (Cout % 96 == 0) return launch_conv<96>(tmX, tmPrev, w, p, st);
  return launch_conv<128>(tmX, tmPrev, w, p, st);
}
