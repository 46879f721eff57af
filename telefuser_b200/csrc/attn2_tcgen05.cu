// Flash-attention forward for sm_100a, two query tiles per CTA (bf16, head_dim 128).
//
// One CTA owns 256 query rows of one (batch, head) as two independent 128-row
// tiles that share every K/V tile. 384 threads (warps 10, 11 only donate registers):
//   warps 0..3  softmax group 0 (query tile 0; TMEM lane == row)
//   warps 4..7  softmax group 1 (query tile 1)
//   warp  8     TMA loader: both Q tiles once, then K0 V0 K1 V1 ... through a 4-slot ring
//   warp  9     tcgen05.mma issuer and TMEM owner
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each. P (bf16) is
// written over the first 64 columns of its S tile and fed to the P.V MMA from
// TMEM, so no shared-memory bandwidth is spent on P. While one group runs its
// softmax the tensor core works on the other group's tile, which keeps the
// MMA pipe and the exp2 pipe busy at the same time.
//
// The row maximum used for exp2 is only raised when it grew by more than 2^8;
// the accumulator rescale (a TMEM round trip) is therefore rare. Replaces the
// attention back-ends dispatched in telefuser/ops/attention/attention_impl.py:112-315.
#include <math.h>

#include "attn_common.cuh"

namespace tfb {

constexpr int A2_KV_SLOTS = 4;
constexpr int A2_Q_OFF = 0;
constexpr int A2_KV_OFF = 2 * ATT_TILE_BYTES;
constexpr int A2_BAR_OFF = A2_KV_OFF + A2_KV_SLOTS * ATT_TILE_BYTES;
constexpr int A2_SMEM_BYTES = A2_BAR_OFF + 256 + 1024;

// POLY: share of exp2 evaluated on the FMA pipe instead of MUFU (0 none, 1 a quarter, 2 half).
// PEER: the epilogue stores each output row into the buffer of the rank that owns the token.
// SPARSE: block-sparse attention. Each CTA (256 query rows of one head) visits only the 128-key blocks
//         listed for it in p.blk_idx (p.blk_cnt of them); everything else is the dense pipeline.
template <int POLY, bool PEER = false, bool SPARSE = false>
__global__ void __launch_bounds__(384, 1)
    attn2_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A2_BAR_OFF);
  uint64_t* q_full = bars + 0;     // [2]
  uint64_t* kv_full = bars + 2;    // [4]
  uint64_t* kv_empty = bars + 6;   // [4]
  uint64_t* s_full = bars + 10;    // [2]
  uint64_t* p_ready = bars + 12;   // [2]
  uint64_t* o_final = bars + 14;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q_pair = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const long list_row = (static_cast<long>(b) * p.H + h) * gridDim.x + q_pair;
  const int* blk_list = SPARSE ? p.blk_idx + list_row * p.max_blocks : nullptr;
  const int n_kv = SPARSE ? __ldg(p.blk_cnt + list_row) : (p.Skv + ATT_BN - 1) / ATT_BN;
  AbortCtx ctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_ready[s], 128);
      mbar_init(&o_final[s], 1);
    }
    for (int s = 0; s < A2_KV_SLOTS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Register budget: the two softmax groups take registers from the loader /
  // MMA group (warps 8..11; 10 and 11 only take part in this hand-over).
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  if (warp == 8) {
    // ------------------------------ TMA loader ------------------------------
    if (lane == 0 && n_kv > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      for (int st = 0; st < 2; ++st) {
        uint8_t* qd = smem + A2_Q_OFF + st * ATT_TILE_BYTES;
        const int q0 = (q_pair * 2 + st) * ATT_BM;
        mbar_expect_tx(&q_full[st], ATT_TILE_BYTES);
        tma_load_3d(qd, &tmQ, &q_full[st], h * ATT_D, q0, b);
        tma_load_3d(qd + ATT_BOX_BYTES, &tmQ, &q_full[st], h * ATT_D + 64, q0, b);
      }
      for (int n = 0; n < 2 * n_kv; ++n) {
        const int slot = n & (A2_KV_SLOTS - 1);
        const uint32_t ph = (n / A2_KV_SLOTS) & 1;
        if (!mbar_wait(&kv_empty[slot], ph ^ 1, ctx, 10)) break;
        uint8_t* dst = smem + A2_KV_OFF + slot * ATT_TILE_BYTES;
        const CUtensorMap* tm = (n & 1) ? &tmV : &tmK;
        const int j = SPARSE ? __ldg(blk_list + (n >> 1)) : (n >> 1);
        mbar_expect_tx(&kv_full[slot], ATT_TILE_BYTES);
        tma_load_3d(dst, tm, &kv_full[slot], h * ATT_D, j * ATT_BN, b);
        tma_load_3d(dst + ATT_BOX_BYTES, tm, &kv_full[slot], h * ATT_D + 64, j * ATT_BN, b);
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ------------------------------ MMA issuer ------------------------------
    constexpr uint32_t idesc_qk = make_idesc(128, 128, 1, 1, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc(128, 128, 1, 1, 0, 1);  // B (= V) is MN-major
    auto slot_addr = [&](int n) { return smem_u32(smem + A2_KV_OFF + (n & (A2_KV_SLOTS - 1)) * ATT_TILE_BYTES); };
    auto issue_qk = [&](int st, int j) {
      const uint32_t q_addr = smem_u32(smem + A2_Q_OFF + st * ATT_TILE_BYTES);
      const uint32_t k_addr = slot_addr(2 * j);
      const uint32_t d_tmem = tmem_base + st * 128;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk >> 2) * ATT_BOX_BYTES + (kk & 3) * 32;
        umma_f16_ss(d_tmem, make_desc_k_sw128(q_addr + off), make_desc_k_sw128(k_addr + off), idesc_qk,
                    kk ? 1u : 0u);
      }
    };
    auto issue_pv = [&](int st, int j) {
      const uint32_t v_addr = slot_addr(2 * j + 1);
      const uint32_t o_tmem = tmem_base + 256 + st * 128;
      const uint32_t p_tmem = tmem_base + st * 128;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_f16_ts(o_tmem, p_tmem + kk * 8, make_desc_mn_sw128(v_addr + kk * 2048, ATT_BOX_BYTES), idesc_pv,
                    (j | kk) ? 1u : 0u);
    };
    bool ok = n_kv > 0 && mbar_wait_warp(&q_full[0], 0, ctx, 20) && mbar_wait_warp(&q_full[1], 0, ctx, 21) &&
              mbar_wait_warp(&kv_full[0], 0, ctx, 22);
    if (ok) {
      tc_fence_after();
      if (lane == 0) {
        issue_qk(0, 0);
        umma_commit(&s_full[0]);
        issue_qk(1, 0);
        umma_commit(&s_full[1]);
        umma_commit(&kv_empty[0]);
      }
      __syncwarp();
    }
    for (int j = 0; j < n_kv && ok; ++j) {
      const bool has_next = j + 1 < n_kv;
      const int nv = 2 * j + 1, nk = 2 * j + 2;
      if (!mbar_wait_warp(&kv_full[nv & (A2_KV_SLOTS - 1)], (nv / A2_KV_SLOTS) & 1, ctx, 23)) break;
      if (has_next && !mbar_wait_warp(&kv_full[nk & (A2_KV_SLOTS - 1)], (nk / A2_KV_SLOTS) & 1, ctx, 24)) break;
      for (int st = 0; st < 2 && ok; ++st) {
        if (!mbar_wait_warp(&p_ready[st], j & 1, ctx, 25)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          issue_pv(st, j);
          if (has_next) {
            issue_qk(st, j + 1);
            umma_commit(&s_full[st]);
          } else {
            umma_commit(&o_final[st]);
          }
        }
        __syncwarp();
      }
      if (ok && lane == 0) {
        umma_commit(&kv_empty[nv & (A2_KV_SLOTS - 1)]);
        if (has_next) umma_commit(&kv_empty[nk & (A2_KV_SLOTS - 1)]);
      }
      __syncwarp();
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // ------------------------------ softmax groups ------------------------------
    const int st = warp >> 2;
    const int qq = warp & 3;
    const int row = qq * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(qq * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_addr + st * 128;
    const uint32_t tmem_o = tmem_base + lane_addr + 256 + st * 128;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait_warp(&s_full[st], j & 1, ctx, 30)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(tmem_s + c * 32, s[c]);
      tmem_ld_wait();
      const int kv_valid = p.Skv - (SPARSE ? __ldg(blk_list + j) : j) * ATT_BN;
      if (kv_valid < ATT_BN) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i >= kv_valid) s[c][i] = 0xff800000u;  // -inf
      }
      // Row maximum: 8 independent chains of 3-input max.
      float mx8[8];
#pragma unroll
      for (int a = 0; a < 8; ++a) mx8[a] = __uint_as_float(s[a >> 1][a & 1]);
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 2; i < 32; i += 4) {
          mx8[c * 2] = fmax3(mx8[c * 2], __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
          if (i + 3 < 32)
            mx8[c * 2 + 1] = fmax3(mx8[c * 2 + 1], __uint_as_float(s[c][i + 2]), __uint_as_float(s[c][i + 3]));
        }
      const float mx = fmax3(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]));
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      if (j == 0) {
        m_used = m_new;
      } else {
        const bool need = (m_new - m_used) > ATT_RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, need)) {
          // All MMAs issued before S(j) have completed, so O is stable here.
          const float alpha = fast_exp2(m_used - m_new);
          m_used = m_new;
          l *= alpha;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_o + c * 32, o);
          }
        }
      }
      // p = 2^(s*scale - m): packed fp32x2 FMAs, exp2 split between the MUFU
      // pipe and a cubic on the FMA pipe, packed row-sum accumulation.
      const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
      const uint64_t negm2 = f2_pack(-m_used, -m_used);
      uint64_t ps[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t t[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const uint64_t x2 = f2_fma(f2_pack(__uint_as_float(s[c][2 * k]), __uint_as_float(s[c][2 * k + 1])), scale2,
                                     negm2);
          float p0, p1;
          if ((POLY == 1 && (k & 3) == 3) || (POLY == 2 && (k & 1))) {  // FMA-pipe exp2 share
            exp2_poly_pair(x2, p0, p1);
          } else {
            float x0, x1;
            f2_unpack(x2, x0, x1);
            p0 = fast_exp2(x0);
            p1 = fast_exp2(x1);
          }
          ps[k & 3] = f2_add(ps[k & 3], f2_pack(p0, p1));
          t[k] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x16(tmem_s + c * 16, t);
      }
      {
        float a0, a1, b0, b1;
        f2_unpack(f2_add(ps[0], ps[1]), a0, a1);
        f2_unpack(f2_add(ps[2], ps[3]), b0, b1);
        l += (a0 + a1) + (b0 + b1);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_ready[st]);
    }
    if (SPARSE && n_kv == 0) {  // no key block listed for these rows: zero output, lse = -inf
      const int grow = (q_pair * 2 + st) * ATT_BM + row;
      if (grow < p.Sq) {
        uint4* orow = reinterpret_cast<uint4*>(p.out + static_cast<long>(b) * p.bso + static_cast<long>(grow) * p.ldo +
                                               h * ATT_D);
        for (int i = 0; i < ATT_D / 8; ++i) orow[i] = make_uint4(0, 0, 0, 0);
        if (p.lse) p.lse[(static_cast<long>(b) * p.H + h) * p.Sq + grow] = -INFINITY;
      }
      ok = false;
    }
    if (ok) ok = mbar_wait_warp(&o_final[st], 0, ctx, 33);
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      const int grow = (q_pair * 2 + st) * ATT_BM + row;
      const bool row_ok = grow < p.Sq;
      __nv_bfloat16* orow;
      if (PEER) {
        const int dst = row_ok ? grow / p.rows_per_rank : 0;
        orow = p.peer_out[dst] + static_cast<long>(b) * p.bso +
               static_cast<long>(grow - dst * p.rows_per_rank) * p.ldo + (p.head_off + h) * ATT_D;
      } else {
        orow = p.out + static_cast<long>(b) * p.bso + static_cast<long>(grow) * p.ldo + h * ATT_D;
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_o + c * 32, o);
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
  if (warp == 9) tmem_dealloc(tmem_base, 512);
}

template <int POLY>
static int launch_attn2_impl(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
                             int B, cudaStream_t st) {
  static bool attr_set[TFB_MAX_DEVICES] = {false};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&attn2_fwd_kernel<POLY>), A2_SMEM_BYTES, attr_set)) return rc;
  dim3 grid((p.Sq + 2 * ATT_BM - 1) / (2 * ATT_BM), p.H, B);
  attn2_fwd_kernel<POLY><<<grid, 384, A2_SMEM_BYTES, st>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

static int launch_attn2_peer(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
                             int B, cudaStream_t st) {
  static bool attr_set[TFB_MAX_DEVICES] = {false};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&attn2_fwd_kernel<0, true>), A2_SMEM_BYTES, attr_set)) return rc;
  dim3 grid((p.Sq + 2 * ATT_BM - 1) / (2 * ATT_BM), p.H, B);
  attn2_fwd_kernel<0, true><<<grid, 384, A2_SMEM_BYTES, st>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

static int launch_attn2_sparse(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
                               int B, cudaStream_t st) {
  static bool attr_set[TFB_MAX_DEVICES] = {false};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&attn2_fwd_kernel<0, false, true>), A2_SMEM_BYTES, attr_set)) return rc;
  dim3 grid((p.Sq + 2 * ATT_BM - 1) / (2 * ATT_BM), p.H, B);
  attn2_fwd_kernel<0, false, true><<<grid, 384, A2_SMEM_BYTES, st>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

int launch_attn2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, int B,
                 cudaStream_t st) {
  if (p.blk_idx) return launch_attn2_sparse(tq, tk, tv, p, B, st);
  if (p.n_peers > 0) return launch_attn2_peer(tq, tk, tv, p, B, st);
  switch (p.poly) {
    case 0: return launch_attn2_impl<0>(tq, tk, tv, p, B, st);
    case 2: return launch_attn2_impl<2>(tq, tk, tv, p, B, st);
    default: return launch_attn2_impl<1>(tq, tk, tv, p, B, st);
  }
}

}  // namespace tfb
