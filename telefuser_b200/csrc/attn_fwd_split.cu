// Flash-attention forward for sm_100a with every query row shared by two threads
// (bf16, head_dim 64 or 128, optional causal mask, optional peer-store epilogue, optional block sparsity;
// optionally Q.K^T on int8 operands with per-token / per-head scales, P.V staying in bf16).
//
// One CTA owns 256 query rows of one (batch, head) as two independent 128-row tiles that share every
// K/V tile. 640 threads:
//   warps 0..7   softmax group 0 (query tile 0): warp w works on TMEM lanes 32*(w&3).. and on the key
//                columns [64*((w>>2)&1), +64) of the 128-column score tile, so a row's exponentials are
//                spread over two warps of the same scheduler partition and the per-tile latency of the
//                load -> max -> exp2 -> store chain is half of the one-thread-per-row form
//   warps 8..15  softmax group 1 (query tile 1)
//   warp  16     TMA loader: both Q tiles once, then K0 V0 K1 V1 ... through a 4-slot ring
//   warp  17     tcgen05.mma issuer and TMEM owner
//   warps 18,19  only donate registers (setmaxnreg works on whole warpgroups)
// Register budget: the CTA is launched with 640 x 96 registers and `setmaxnreg` only moves registers inside that
// allocation (an increase waits until other warps of the CTA have released enough, for ever if they never do), so
// the split must balance: 512 x 112 + 128 x 32 = 640 x 96.
// TMEM (512 columns): S0 | S1 | O0 | O1. P (bf16) is written over the first 64 columns of its S tile
// and fed to the P.V MMA from TMEM. The two threads of a row exchange their partial row maxima through
// shared memory and a 64-thread mbarrier (bounded wait) once per K/V tile; that exchange also orders the
// second thread's P store after the first thread's S load of the columns it overwrites.
//
// The row maximum used for exp2 is only raised when it grew by more than 2^8, so the accumulator
// rescale (a TMEM round trip) is rare. Replaces the attention back-ends dispatched in
// telefuser/ops/attention/attention_impl.py:112-315.
#include <math.h>

#include "attn_common.cuh"

namespace tfb {

// QK8: Q and K arrive as int8 (one 16 KB box of [128 rows][128 bytes] per tile), S = Q.K^T is accumulated in
// int32 by `tcgen05.mma.kind::i8` and scaled per row in the softmax; V and P stay bf16.
template <int HD, bool QK8 = false>
struct SplitCfg {
  static constexpr int TILE_BYTES = 128 * HD * 2;  // one 128-row bf16 tile of Q, K or V (a ring slot)
  static constexpr int QK_TILE_BYTES = QK8 ? 128 * HD : TILE_BYTES;  // bytes of a Q or K tile
  static constexpr int BOXES = HD / 64;            // 16 KB boxes of [128 rows][64 columns] per bf16 tile
  static constexpr int QK_BOXES = QK8 ? 1 : BOXES;
  static constexpr int KV_SLOTS = 4;
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = 2 * TILE_BYTES;
  static constexpr int MX_OFF = KV_OFF + KV_SLOTS * TILE_BYTES;  // float [2 parity][2 tiles][2 halves][128]
  static constexpr int BAR_OFF = MX_OFF + 2 * 2 * 2 * 128 * 4;
  static constexpr int SMEM_BYTES = BAR_OFF + 512 + 1024;
  static constexpr int O_COL = 256;        // first accumulator column in TMEM
  static constexpr int OC = HD / 2;        // accumulator columns per thread
};

constexpr int SPLIT_THREADS = 640, SPLIT_LAUNCH_REGS = 96, SPLIT_SOFTMAX_REGS = 112, SPLIT_OTHER_REGS = 32;
static_assert(512 * SPLIT_SOFTMAX_REGS + 128 * SPLIT_OTHER_REGS <= SPLIT_THREADS * SPLIT_LAUNCH_REGS,
              "setmaxnreg.inc would wait for registers that no warp of the CTA ever releases");
static_assert(SPLIT_LAUNCH_REGS == (65536 / SPLIT_THREADS) / 8 * 8, "launch registers follow from the launch bound");

template <int HD, int POLY, bool PEER, bool SPARSE, bool CAUSAL, bool QK8 = false>
__global__ void __launch_bounds__(640, 1)
    attn_split_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using C = SplitCfg<HD, QK8>;
  static_assert(!QK8 || HD == 128, "the int8 score path is built for head_dim 128");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* mx_buf = reinterpret_cast<float*>(smem + C::MX_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::BAR_OFF);
  uint64_t* q_full = bars + 0;     // [2]
  uint64_t* kv_full = bars + 2;    // [4]
  uint64_t* kv_empty = bars + 6;   // [4]
  uint64_t* s_full = bars + 10;    // [2]
  uint64_t* p_ready = bars + 12;   // [2]
  uint64_t* o_final = bars + 14;   // [2]
  uint64_t* pair_bar = bars + 16;  // [8]: (tile, lane quarter)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q_pair = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const long list_row = (static_cast<long>(b) * p.H + h) * gridDim.x + q_pair;
  const int* blk_list = SPARSE ? p.blk_idx + list_row * p.max_blocks : nullptr;
  const int causal_off = p.Skv - p.Sq;  // key j is visible to query row i when j <= i + causal_off
  int n_kv = SPARSE ? __ldg(p.blk_cnt + list_row) : (p.Skv + ATT_BN - 1) / ATT_BN;
  if (CAUSAL) {
    const int last_row = min(p.Sq, (q_pair + 1) * 2 * ATT_BM) - 1;
    n_kv = min(n_kv, (last_row + causal_off) / ATT_BN + 1);
  }
  AbortCtx ctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_ready[s], 256);
      mbar_init(&o_final[s], 1);
    }
    for (int s = 0; s < C::KV_SLOTS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int s = 0; s < 8; ++s) mbar_init(&pair_bar[s], 64);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 17) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 16) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 32;");
    if (warp == 16) {
      // ------------------------------ TMA loader ------------------------------
      if (lane == 0 && n_kv > 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        for (int st = 0; st < 2; ++st) {
          uint8_t* qd = smem + C::Q_OFF + st * C::TILE_BYTES;
          const int q0 = (q_pair * 2 + st) * ATT_BM;
          mbar_expect_tx(&q_full[st], C::QK_TILE_BYTES);
#pragma unroll
          for (int x = 0; x < C::QK_BOXES; ++x)
            tma_load_3d(qd + x * ATT_BOX_BYTES, &tmQ, &q_full[st], h * HD + x * 64, q0, b);
        }
        for (int n = 0; n < 2 * n_kv; ++n) {
          const int slot = n & (C::KV_SLOTS - 1);
          const uint32_t ph = (n / C::KV_SLOTS) & 1;
          if (!mbar_wait(&kv_empty[slot], ph ^ 1, ctx, 10)) break;
          uint8_t* dst = smem + C::KV_OFF + slot * C::TILE_BYTES;
          const CUtensorMap* tm = (n & 1) ? &tmV : &tmK;
          const int j = SPARSE ? __ldg(blk_list + (n >> 1)) : (n >> 1);
          if (QK8 && !(n & 1)) {  // int8 K: one box of 128 bytes per row
            mbar_expect_tx(&kv_full[slot], C::QK_TILE_BYTES);
            tma_load_3d(dst, tm, &kv_full[slot], h * HD, j * ATT_BN, b);
          } else {
            mbar_expect_tx(&kv_full[slot], C::TILE_BYTES);
#pragma unroll
            for (int x = 0; x < C::BOXES; ++x)
              tma_load_3d(dst + x * ATT_BOX_BYTES, tm, &kv_full[slot], h * HD + x * 64, j * ATT_BN, b);
          }
        }
      }
      __syncwarp();
    } else if (warp == 17) {
      // ------------------------------ MMA issuer ------------------------------
      constexpr uint32_t idesc_qk = QK8 ? make_idesc_i8(128, 128) : make_idesc(128, 128, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(128, HD, 1, 1, 0, 1);  // B (= V) is MN-major
      auto slot_addr = [&](int n) { return smem_u32(smem + C::KV_OFF + (n & (C::KV_SLOTS - 1)) * C::TILE_BYTES); };
      auto issue_qk = [&](int st, int j) {
        const uint32_t q_addr = smem_u32(smem + C::Q_OFF + st * C::TILE_BYTES);
        const uint32_t k_addr = slot_addr(2 * j);
        const uint32_t d_tmem = tmem_base + st * 128;
        if (QK8) {  // 32 int8 elements (32 bytes of the 128-byte row) per instruction
#pragma unroll
          for (int kk = 0; kk < HD / 32; ++kk)
            umma_i8_ss(d_tmem, make_desc_k_sw128(q_addr + kk * 32), make_desc_k_sw128(k_addr + kk * 32), idesc_qk,
                       kk ? 1u : 0u);
        } else {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t off = (kk >> 2) * ATT_BOX_BYTES + (kk & 3) * 32;
            umma_f16_ss(d_tmem, make_desc_k_sw128(q_addr + off), make_desc_k_sw128(k_addr + off), idesc_qk,
                        kk ? 1u : 0u);
          }
        }
      };
      auto issue_pv = [&](int st, int j) {
        const uint32_t v_addr = slot_addr(2 * j + 1);
        const uint32_t o_tmem = tmem_base + C::O_COL + st * HD;
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
        if (!mbar_wait_warp(&kv_full[nv & (C::KV_SLOTS - 1)], (nv / C::KV_SLOTS) & 1, ctx, 23)) break;
        if (has_next && !mbar_wait_warp(&kv_full[nk & (C::KV_SLOTS - 1)], (nk / C::KV_SLOTS) & 1, ctx, 24)) break;
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
          umma_commit(&kv_empty[nv & (C::KV_SLOTS - 1)]);
          if (has_next) umma_commit(&kv_empty[nk & (C::KV_SLOTS - 1)]);
        }
        __syncwarp();
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 112;");
    // ------------------------------ softmax groups ------------------------------
    const int st = warp >> 3;
    const int half = (warp >> 2) & 1;
    const int qq = warp & 3;
    const int row = qq * 32 + lane;
    const int grow = (q_pair * 2 + st) * ATT_BM + row;  // query row in the sequence
    const uint32_t lane_addr = static_cast<uint32_t>(qq * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_addr + st * 128 + half * 64;      // my 64 score columns
    const uint32_t tmem_p = tmem_base + lane_addr + st * 128 + half * 32;      // my 32 packed P columns
    const uint32_t tmem_o = tmem_base + lane_addr + C::O_COL + st * HD + half * C::OC;
    uint64_t* my_pair = &pair_bar[st * 4 + qq];
    float* mx_mine = mx_buf + ((st * 2 + half) * 128 + row);
    float* mx_other = mx_buf + ((st * 2 + (half ^ 1)) * 128 + row);
    constexpr int MX_PARITY_STRIDE = 2 * 2 * 128;
    float m_used = -INFINITY, l = 0.f;
    // Score scale of this row in the log2 domain. Int8 scores carry the row's Q scale and the head's K scale.
    float row_scale = p.scale_log2;
    if (QK8) {
      const long bh = static_cast<long>(b) * p.H + h;
      row_scale *= __ldg(p.k_scale + bh) * (grow < p.Sq ? __ldg(p.q_scale + bh * p.Sq + grow) : 0.f);
    }
    bool ok = true;
    int j = 0;
    for (; j < n_kv; ++j) {
      if (!mbar_wait_warp(&s_full[st], j & 1, ctx, 30)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s[2][32];
      tmem_ld_32x32(tmem_s, s[0]);
      tmem_ld_32x32(tmem_s + 32, s[1]);
      tmem_ld_wait();
      if (QK8) {
        // int32 -> fp32 without the conversion pipe: |s| <= 128 * 127^2 < 2^22, so adding the bit pattern of
        // 1.5 * 2^23 gives the float 1.5 * 2^23 + s exactly, and the subtraction is exact too.
        const uint64_t neg_magic2 = f2_pack(-12582912.f, -12582912.f);
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t f2 = f2_add(f2_pack(__uint_as_float(s[c][i] + 0x4B400000u), __uint_as_float(s[c][i + 1] + 0x4B400000u)),
                                       neg_magic2);
            float lo, hi;
            f2_unpack(f2, lo, hi);
            s[c][i] = __float_as_uint(lo);
            s[c][i + 1] = __float_as_uint(hi);
          }
      }
      const int key0 = (SPARSE ? __ldg(blk_list + j) : j) * ATT_BN + half * 64;  // key index of my first column
      int kv_valid = p.Skv - key0;
      if (CAUSAL) kv_valid = min(kv_valid, grow + causal_off - key0 + 1);
      if (kv_valid < 64) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i >= kv_valid) s[c][i] = 0xff800000u;  // -inf
      }
      // Partial row maximum over my 64 columns: 4 independent chains of 3-input max.
      float mx4[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) mx4[a] = __uint_as_float(s[a >> 1][a & 1]);
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 2; i < 32; i += 4) {
          mx4[c * 2] = fmax3(mx4[c * 2], __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
          if (i + 3 < 32)
            mx4[c * 2 + 1] = fmax3(mx4[c * 2 + 1], __uint_as_float(s[c][i + 2]), __uint_as_float(s[c][i + 3]));
        }
      const float mx_part = fmaxf(fmax3(mx4[0], mx4[1], mx4[2]), mx4[3]);
      // Exchange with the thread that holds the other 64 columns of this row.
      mx_mine[(j & 1) * MX_PARITY_STRIDE] = mx_part;
      tc_fence_before();
      mbar_arrive(my_pair);
      if (!mbar_wait_warp(my_pair, j & 1, ctx, 31)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const float mx = fmaxf(mx_part, mx_other[(j & 1) * MX_PARITY_STRIDE]);
      // A fully masked row keeps m at a finite floor so that exp2(-inf - m) is 0, not NaN.
      const float m_new = fmaxf(fmaxf(m_used, mx * row_scale), -1e30f);
      if (j == 0) {
        m_used = m_new;
      } else {
        const bool need = (m_new - m_used) > ATT_RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, need)) {
          // All MMAs issued before S(j) have completed, so O is stable here.
          const float alpha = fast_exp2(m_used - m_new);
          m_used = m_new;
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < C::OC / 32; ++c) {  // one 32-column chunk at a time: the score registers stay live
            uint32_t o[32];
            tmem_ld_32x32(tmem_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_o + c * 32, o);
          }
        }
      }
      // p = 2^(s*scale - m): packed fp32x2 FMAs, exp2 split between the MUFU pipe and a cubic on the
      // FMA pipe, packed row-sum accumulation.
      const uint64_t scale2 = f2_pack(row_scale, row_scale);
      const uint64_t negm2 = f2_pack(-m_used, -m_used);
      uint64_t ps[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int c = 0; c < 2; ++c) {
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
        tmem_st_32x16(tmem_p + c * 16, t);
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
      if (grow < p.Sq) {
        uint4* orow = reinterpret_cast<uint4*>(p.out + static_cast<long>(b) * p.bso + static_cast<long>(grow) * p.ldo +
                                               h * HD + half * C::OC);
        for (int i = 0; i < C::OC / 8; ++i) orow[i] = make_uint4(0, 0, 0, 0);
        if (p.lse && half == 0) p.lse[(static_cast<long>(b) * p.H + h) * p.Sq + grow] = -INFINITY;
      }
      ok = false;
    }
    // Row sum of the two halves (one more round of the pair exchange).
    if (ok) {
      mx_mine[(j & 1) * MX_PARITY_STRIDE] = l;
      mbar_arrive(my_pair);
      ok = mbar_wait_warp(my_pair, j & 1, ctx, 32);
      if (ok) l += mx_other[(j & 1) * MX_PARITY_STRIDE];
    }
    if (ok) ok = mbar_wait_warp(&o_final[st], 0, ctx, 33);
    if (ok) {
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = grow < p.Sq;
      __nv_bfloat16* orow;
      if (PEER) {
        const int dst = row_ok ? grow / p.rows_per_rank : 0;
        orow = p.peer_out[dst] + static_cast<long>(b) * p.bso +
               static_cast<long>(grow - dst * p.rows_per_rank) * p.ldo + (p.head_off + h) * HD;
      } else {
        orow = p.out + static_cast<long>(b) * p.bso + static_cast<long>(grow) * p.ldo + h * HD;
      }
      orow += half * C::OC;
#pragma unroll
      for (int c = 0; c < C::OC / 32; ++c) {
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
      if (p.lse && row_ok && half == 0)
        p.lse[(static_cast<long>(b) * p.H + h) * p.Sq + grow] =
            l > 0.f ? m_used * 0.6931471805599453f + logf(l) : -INFINITY;
    }
  }

  if (*abort_flag) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  if (warp == 17) tmem_dealloc(tmem_base, 512);
}

template <int HD, int POLY, bool PEER, bool SPARSE, bool CAUSAL, bool QK8 = false>
static int launch_split_impl(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
                             int B, cudaStream_t st) {
  static bool attr_set[TFB_MAX_DEVICES] = {false};
  auto* kern = attn_split_kernel<HD, POLY, PEER, SPARSE, CAUSAL, QK8>;
  constexpr int SMEM = SplitCfg<HD, QK8>::SMEM_BYTES;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), SMEM, attr_set)) return rc;
  dim3 grid((p.Sq + 2 * ATT_BM - 1) / (2 * ATT_BM), p.H, B);
  kern<<<grid, 640, SMEM, st>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

int launch_attn_split(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, int B,
                      cudaStream_t st) {
  if (p.q_scale) {  // int8 scores
    if (p.head_dim != 128 || p.blk_idx || p.n_peers > 0 || !p.k_scale) return TFB_ERR_BAD_SHAPE;
    return p.causal ? launch_split_impl<128, 0, false, false, true, true>(tq, tk, tv, p, B, st)
                    : launch_split_impl<128, 0, false, false, false, true>(tq, tk, tv, p, B, st);
  }
  if (p.head_dim == 64) {
    if (p.blk_idx || p.n_peers > 0) return TFB_ERR_BAD_SHAPE;
    return p.causal ? launch_split_impl<64, 0, false, false, true>(tq, tk, tv, p, B, st)
                    : launch_split_impl<64, 0, false, false, false>(tq, tk, tv, p, B, st);
  }
  if (p.blk_idx) return launch_split_impl<128, 0, false, true, false>(tq, tk, tv, p, B, st);
  if (p.n_peers > 0) return launch_split_impl<128, 0, true, false, false>(tq, tk, tv, p, B, st);
  if (p.causal) return launch_split_impl<128, 0, false, false, true>(tq, tk, tv, p, B, st);
  switch (p.poly) {
    case 1: return launch_split_impl<128, 1, false, false, false>(tq, tk, tv, p, B, st);
    case 2: return launch_split_impl<128, 2, false, false, false>(tq, tk, tv, p, B, st);
    default: return launch_split_impl<128, 0, false, false, false>(tq, tk, tv, p, B, st);
  }
}

}  // namespace tfb
