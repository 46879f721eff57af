// Flash-attention forward for sm_100a (bf16, head_dim 128, non-causal).
//
// One CTA = one 128-row query tile of one (batch, head). Warp roles:
//   warp 0      TMA loader: Q once, K/V tiles through 2-stage rings
//   warp 1      tcgen05.mma issuer (S = Q K^T into TMEM, O += P V into TMEM)
//   warps 2..5  softmax: one query row per thread (TMEM lane == row), online
//               softmax in the log2 domain with lazy accumulator rescaling,
//               P handed to the PV MMA either through TMEM (aliasing the S
//               columns) or through a swizzled shared-memory tile.
// S is double buffered in TMEM so Q K^T of tile j+1 overlaps softmax of tile j.
//
// Replaces the library attention back-ends that the reference dispatches to
// (telefuser/ops/attention/attention_impl.py:112-315).
#include <math.h>

#include "attn_common.cuh"
#include "tfb_api.h"

namespace tfb {

constexpr int ATT_KV_STAGES = 2;

template <bool P_TMEM>
struct AttnSmem {
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = ATT_TILE_BYTES;
  static constexpr int V_OFF = K_OFF + ATT_KV_STAGES * ATT_TILE_BYTES;
  static constexpr int P_OFF = V_OFF + ATT_KV_STAGES * ATT_TILE_BYTES;
  static constexpr int BAR_OFF = P_OFF + (P_TMEM ? 0 : ATT_TILE_BYTES);
  static constexpr int BYTES = BAR_OFF + 256 + 1024;
};

template <bool P_TMEM>
__global__ void __launch_bounds__(192, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using L = AttnSmem<P_TMEM>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* k_empty = bars + 3;  // [2]
  uint64_t* v_full = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;  // [2]
  uint64_t* s_full = bars + 9;   // [2]
  uint64_t* p_ready = bars + 11;
  uint64_t* pv_done = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q_tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n_kv = (p.Skv + ATT_BN - 1) / ATT_BN;
  AbortCtx ctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
    }
    mbar_init(p_ready, 128);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    // ------------------------------ TMA loader ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, ATT_TILE_BYTES);
      tma_load_3d(smem + L::Q_OFF, &tmQ, q_full, h * ATT_D, q_tile * ATT_BM, b);
      tma_load_3d(smem + L::Q_OFF + ATT_BOX_BYTES, &tmQ, q_full, h * ATT_D + 64, q_tile * ATT_BM, b);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[s], ph ^ 1, ctx, 10)) break;
        uint8_t* kd = smem + L::K_OFF + s * ATT_TILE_BYTES;
        mbar_expect_tx(&k_full[s], ATT_TILE_BYTES);
        tma_load_3d(kd, &tmK, &k_full[s], h * ATT_D, j * ATT_BN, b);
        tma_load_3d(kd + ATT_BOX_BYTES, &tmK, &k_full[s], h * ATT_D + 64, j * ATT_BN, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1, ctx, 11)) break;
        uint8_t* vd = smem + L::V_OFF + s * ATT_TILE_BYTES;
        mbar_expect_tx(&v_full[s], ATT_TILE_BYTES);
        tma_load_3d(vd, &tmV, &v_full[s], h * ATT_D, j * ATT_BN, b);
        tma_load_3d(vd + ATT_BOX_BYTES, &tmV, &v_full[s], h * ATT_D + 64, j * ATT_BN, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    constexpr uint32_t idesc_qk = make_idesc(128, 128, 1, 1, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc(128, 128, 1, 1, 0, 1);  // B (= V) is MN-major
    const uint32_t q_addr = smem_u32(smem + L::Q_OFF);
    auto issue_qk = [&](int j) {
      const int s = j & 1;
      const uint32_t k_addr = smem_u32(smem + L::K_OFF + s * ATT_TILE_BYTES);
      const uint32_t d_tmem = tmem_base + s * 128;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk >> 2) * ATT_BOX_BYTES + (kk & 3) * 32;
        umma_f16_ss(d_tmem, make_desc_k_sw128(q_addr + off), make_desc_k_sw128(k_addr + off), idesc_qk,
                    kk ? 1u : 0u);
      }
      umma_commit(&k_empty[s]);
      umma_commit(&s_full[s]);
    };
    bool ok = mbar_wait_warp(q_full, 0, ctx, 20) && mbar_wait_warp(&k_full[0], 0, ctx, 21);
    if (ok) {
      tc_fence_after();
      if (lane == 0) issue_qk(0);
      __syncwarp();
    }
    for (int j = 0; j < n_kv && ok; ++j) {
      if (j + 1 < n_kv) {
        const int s1 = (j + 1) & 1;
        if (!mbar_wait_warp(&k_full[s1], ((j + 1) >> 1) & 1, ctx, 22)) break;
        tc_fence_after();
        if (lane == 0) issue_qk(j + 1);
        __syncwarp();
      }
      if (!mbar_wait_warp(p_ready, j & 1, ctx, 23)) break;
      if (!mbar_wait_warp(&v_full[j & 1], (j >> 1) & 1, ctx, 24)) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t v_addr = smem_u32(smem + L::V_OFF + (j & 1) * ATT_TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t bd = make_desc_mn_sw128(v_addr + kk * 2048, ATT_BOX_BYTES);
          const uint32_t acc = (j | kk) ? 1u : 0u;
          if (P_TMEM) {
            umma_f16_ts(tmem_o, tmem_base + (j & 1) * 128 + kk * 8, bd, idesc_pv, acc);
          } else {
            const uint32_t p_addr = smem_u32(smem + L::P_OFF) + (kk >> 2) * ATT_BOX_BYTES + (kk & 3) * 32;
            umma_f16_ss(tmem_o, make_desc_k_sw128(p_addr), bd, idesc_pv, acc);
          }
        }
        umma_commit(&v_empty[j & 1]);
        umma_commit(pv_done);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------ softmax ------------------------------
    const int qq = warp & 3;
    const int row = qq * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(qq * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int sb = j & 1;
      if (!mbar_wait_warp(&s_full[sb], (j >> 1) & 1, ctx, 30)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(tmem_base + lane_addr + sb * 128 + c * 32, s[c]);
      tmem_ld_wait();
      const int kv_valid = p.Skv - j * ATT_BN;
      if (kv_valid < ATT_BN) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i >= kv_valid) s[c][i] = 0xff800000u;  // -inf
      }
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(s[c][i]));
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      bool waited_pv = false;
      if (j == 0) {
        m_used = m_new;
      } else {
        const bool need = (m_new - m_used) > ATT_RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, need)) {
          if (!mbar_wait_warp(pv_done, (j - 1) & 1, ctx, 31)) {
            ok = false;
            break;
          }
          waited_pv = true;
          tc_fence_after();
          const float alpha = fast_exp2(m_used - m_new);
          m_used = m_new;
          l *= alpha;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_o + lane_addr + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_o + lane_addr + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      const float neg_m = -m_used;
      float psum = 0.f;
      uint32_t pk[64];
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(s[c][i]), p.scale_log2, neg_m));
          const float p1 = fast_exp2(fmaf(__uint_as_float(s[c][i + 1]), p.scale_log2, neg_m));
          psum += p0 + p1;
          pk[c * 16 + (i >> 1)] = pack_bf16x2(p0, p1);
        }
      l += psum;
      if (P_TMEM) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t t[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) t[i] = pk[c * 16 + i];
          tmem_st_32x16(tmem_base + lane_addr + sb * 128 + c * 16, t);
        }
        tmem_st_wait();
        tc_fence_before();
      } else {
        if (j > 0 && !waited_pv) {
          if (!mbar_wait_warp(pv_done, (j - 1) & 1, ctx, 32)) {
            ok = false;
            break;
          }
        }
        uint8_t* pbase = smem + L::P_OFF;
#pragma unroll
        for (int ch = 0; ch < 16; ++ch) {
          // 16-byte chunk ch of this row: kv columns ch*8 .. ch*8+7
          const int box = ch >> 3, cin = ch & 7;
          uint4 val = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
          *reinterpret_cast<uint4*>(pbase + box * ATT_BOX_BYTES + row * 128 + ((cin ^ (row & 7)) << 4)) = val;
        }
        fence_proxy_async_smem();
        tc_fence_before();
      }
      mbar_arrive(p_ready);
    }
    if (ok) ok = mbar_wait_warp(pv_done, (n_kv - 1) & 1, ctx, 33);
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      const int grow = q_tile * ATT_BM + row;
      const bool row_ok = grow < p.Sq;
      __nv_bfloat16* orow = p.out + static_cast<long>(b) * p.bso + static_cast<long>(grow) * p.ldo + h * ATT_D;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_o + lane_addr + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[v4 * 8 + 0]) * inv_l, __uint_as_float(o[v4 * 8 + 1]) * inv_l);
            w.y = pack_bf16x2(__uint_as_float(o[v4 * 8 + 2]) * inv_l, __uint_as_float(o[v4 * 8 + 3]) * inv_l);
            w.z = pack_bf16x2(__uint_as_float(o[v4 * 8 + 4]) * inv_l, __uint_as_float(o[v4 * 8 + 5]) * inv_l);
            w.w = pack_bf16x2(__uint_as_float(o[v4 * 8 + 6]) * inv_l, __uint_as_float(o[v4 * 8 + 7]) * inv_l);
            reinterpret_cast<uint4*>(orow + c * 32)[v4] = w;
          }
        }
      }
      if (p.lse && row_ok)
        p.lse[(static_cast<long>(b) * p.H + h) * p.Sq + grow] = m_used * 0.6931471805599453f + logf(l);
    }
  }

  if (*abort_flag) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

template <bool P_TMEM>
static int launch_attn(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, int B,
                       cudaStream_t st) {
  using L = AttnSmem<P_TMEM>;
  static bool attr_set[16] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 15;
  if (!attr_set[dev]) {
    cudaFuncSetAttribute(attn_fwd_kernel<P_TMEM>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES);
    attr_set[dev] = true;
  }
  dim3 grid((p.Sq + ATT_BM - 1) / ATT_BM, p.H, B);
  attn_fwd_kernel<P_TMEM><<<grid, 192, L::BYTES, st>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------
// Descriptor self-test (single CTA, 128 threads): D[128,128] = A[128,128] @ B^T
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1)
    umma_probe_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ Bm,
                      float* __restrict__ D, int mode, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_s = smem;
  uint8_t* b_s = smem + ATT_TILE_BYTES;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 2 * ATT_TILE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = threadIdx.x;
  AbortCtx ctx{abort_flag, status};
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;

  // A: [128 rows][128 k] -> K-major swizzled boxes (modes 0,1) or TMEM (mode 2).
  if (mode != 2) {
    for (int ch = 0; ch < 16; ++ch) {
      const uint4 v = *reinterpret_cast<const uint4*>(A + row * 128 + ch * 8);
      const int box = ch >> 3, cin = ch & 7;
      *reinterpret_cast<uint4*>(a_s + box * ATT_BOX_BYTES + row * 128 + ((cin ^ (row & 7)) << 4)) = v;
    }
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t t[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) t[i] = *reinterpret_cast<const uint32_t*>(A + row * 128 + c * 32 + i * 2);
      tmem_st_32x16(tmem_base + lane_addr + 128 + c * 16, t);
    }
    tmem_st_wait();
  }
  // B: mode 0/2: given [N=128][K=128] -> K-major boxes; mode 1: given [K=128][N=128] -> MN-major boxes.
  for (int ch = 0; ch < 16; ++ch) {
    const uint4 v = *reinterpret_cast<const uint4*>(Bm + row * 128 + ch * 8);
    const int box = ch >> 3, cin = ch & 7;
    *reinterpret_cast<uint4*>(b_s + box * ATT_BOX_BYTES + row * 128 + ((cin ^ (row & 7)) << 4)) = v;
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0 && lane == 0) {
    const uint32_t a_addr = smem_u32(a_s), b_addr = smem_u32(b_s);
    const uint32_t idesc = make_idesc(128, 128, 1, 1, 0, mode == 1 ? 1 : 0);
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t koff = (kk >> 2) * ATT_BOX_BYTES + (kk & 3) * 32;
      const uint64_t bd = mode == 1 ? make_desc_mn_sw128(b_addr + kk * 2048, ATT_BOX_BYTES)
                                    : make_desc_k_sw128(b_addr + koff);
      if (mode == 2)
        umma_f16_ts(tmem_base, tmem_base + 128 + kk * 8, bd, idesc, kk ? 1u : 0u);
      else
        umma_f16_ss(tmem_base, make_desc_k_sw128(a_addr + koff), bd, idesc, kk ? 1u : 0u);
    }
    umma_commit(bar);
  }
  __syncwarp();
  if (mbar_wait(bar, 0, ctx, 40)) {
    tc_fence_after();
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t o[32];
      tmem_ld_32x32(tmem_base + lane_addr + c * 32, o);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) D[row * 128 + c * 32 + i] = __uint_as_float(o[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 256);
}

}  // namespace tfb

using namespace tfb;

static int attn_fwd_impl(const void* q, long ldq, long bsq, const void* k, long ldk, long bsk, const void* v,
                         long ldv, long bsv, void* out, long ldo, long bso, float* lse, int B, int H, int Sq, int Skv,
                         float scale, int variant, const int* blk_idx, const int* blk_cnt, int max_blocks,
                         void* stream) {
  if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0) return TFB_ERR_BAD_SHAPE;
  if ((ldq | ldk | ldv | ldo | bsq | bsk | bsv | bso) % 8) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return TFB_ERR_BAD_SHAPE;
  CUtensorMap tq, tk, tv;
  int e;
  if ((e = make_qkv_tmap(&tq, q, ldq, bsq, B, Sq, H))) return e;
  if ((e = make_qkv_tmap(&tk, k, ldk, bsk, B, Skv, H))) return e;
  if ((e = make_qkv_tmap(&tv, v, ldv, bsv, B, Skv, H))) return e;
  AttnParams p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.bso = bso;
  p.lse = lse;
  p.H = H;
  p.Sq = Sq;
  p.Skv = Skv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_word();
  p.poly = (variant >= 20 && variant <= 22) ? variant - 20 : 0;
  p.n_peers = 0;
  p.rows_per_rank = 1;
  p.head_off = 0;
  p.blk_idx = blk_idx;
  p.blk_cnt = blk_cnt;
  p.max_blocks = max_blocks;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (blk_idx) return launch_attn2(tq, tk, tv, p, B, st);
  if (variant == 1) return launch_attn<false>(tq, tk, tv, p, B, st);
  if (variant == 3) return launch_attn<true>(tq, tk, tv, p, B, st);
  return launch_attn2(tq, tk, tv, p, B, st);
}

extern "C" int tfb_attn_fwd(const void* q, long ldq, long bsq, const void* k, long ldk, long bsk, const void* v,
                            long ldv, long bsv, void* out, long ldo, long bso, float* lse, int B, int H, int Sq,
                            int Skv, float scale, int variant, void* stream) {
  return attn_fwd_impl(q, ldq, bsq, k, ldk, bsk, v, ldv, bsv, out, ldo, bso, lse, B, H, Sq, Skv, scale, variant, nullptr,
                       nullptr, 0, stream);
}

// Block-sparse attention: blk_idx int32 [B, H, ceil(Sq/256), max_blocks] lists the 128-key blocks every
// 256-row query group attends to, blk_cnt int32 [B, H, ceil(Sq/256)] how many of them are valid.
extern "C" int tfb_attn_fwd_sparse(const void* q, long ldq, long bsq, const void* k, long ldk, long bsk, const void* v,
                                   long ldv, long bsv, void* out, long ldo, long bso, float* lse, int B, int H, int Sq,
                                   int Skv, float scale, const int* blk_idx, const int* blk_cnt, int max_blocks,
                                   void* stream) {
  if (!blk_idx || !blk_cnt || max_blocks < 1) return TFB_ERR_BAD_SHAPE;
  return attn_fwd_impl(q, ldq, bsq, k, ldk, bsk, v, ldv, bsv, out, ldo, bso, lse, B, H, Sq, Skv, scale, 0, blk_idx,
                       blk_cnt, max_blocks, stream);
}

// Attention whose epilogue performs the sequence-parallel "gather heads" exchange: this rank holds
// H local heads of all Sq tokens; output row g goes to rank g / rows_per_rank, into its buffer
// peer_out[rank] laid out [B, rows_per_rank, H_total*128] (row stride ldo, batch stride bso), at head
// head_off + h. peer_out: HOST array of n_peers device pointers (this rank's own buffer included).
extern "C" int tfb_attn_fwd_peer(const void* q, long ldq, long bsq, const void* k, long ldk, long bsk, const void* v,
                                 long ldv, long bsv, void* const* peer_out, int n_peers, int rows_per_rank,
                                 int head_off, long ldo, long bso, int B, int H, int Sq, int Skv, float scale,
                                 void* stream) {
  if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0 || n_peers < 1 || n_peers > 8 || rows_per_rank < 1) return TFB_ERR_BAD_SHAPE;
  if (static_cast<long>(rows_per_rank) * n_peers < Sq) return TFB_ERR_BAD_SHAPE;
  if ((ldq | ldk | ldv | ldo | bsq | bsk | bsv | bso) % 8) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15)
    return TFB_ERR_BAD_SHAPE;
  CUtensorMap tq, tk, tv;
  int e;
  if ((e = make_qkv_tmap(&tq, q, ldq, bsq, B, Sq, H))) return e;
  if ((e = make_qkv_tmap(&tk, k, ldk, bsk, B, Skv, H))) return e;
  if ((e = make_qkv_tmap(&tv, v, ldv, bsv, B, Skv, H))) return e;
  AttnParams p;
  p.out = nullptr;
  p.ldo = ldo;
  p.bso = bso;
  p.lse = nullptr;
  p.H = H;
  p.Sq = Sq;
  p.Skv = Skv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_word();
  p.poly = 0;
  for (int i = 0; i < 8; ++i) {
    p.peer_out[i] = i < n_peers ? static_cast<__nv_bfloat16*>(peer_out[i]) : nullptr;
    if (i < n_peers && (reinterpret_cast<uintptr_t>(peer_out[i]) & 15)) return TFB_ERR_BAD_SHAPE;
  }
  p.n_peers = n_peers;
  p.rows_per_rank = rows_per_rank;
  p.head_off = head_off;
  p.blk_idx = nullptr;
  p.blk_cnt = nullptr;
  p.max_blocks = 0;
  return launch_attn2(tq, tk, tv, p, B, static_cast<cudaStream_t>(stream));
}

extern "C" int tfb_umma_probe(const void* A, const void* B, float* D, int N, int K, int mode, void* stream) {
  if (N != 128 || K != 128 || mode < 0 || mode > 2) return TFB_ERR_BAD_SHAPE;
  const int smem_bytes = 2 * ATT_TILE_BYTES + 1024 + 64;
  static bool attr_set[16] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 15;
  if (!attr_set[dev]) {
    cudaFuncSetAttribute(umma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    attr_set[dev] = true;
  }
  umma_probe_kernel<<<1, 128, smem_bytes, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(B), D, mode, status_word());
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}
