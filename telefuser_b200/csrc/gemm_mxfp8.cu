// Block-scaled MXFP8 GEMM for sm_100a:
//   out[M,N] = epilogue( sum_kb  (A_kb * 2^(sfa-127)) @ (B_kb * 2^(sfb-127))^T )
// A [M,K] and B [N,K] are e4m3 bytes; every 32 consecutive K elements of a row share one UE8M0 scale.
// The scaling happens inside the tensor core (`tcgen05.mma.kind::mxf8f6f4.block_scale`): per 128-deep
// k-block the producer brings A, B (TMA, 128B swizzle) and the two 512-byte scale-factor tiles (bulk copies)
// into one pipeline stage; the MMA warp copies the scale tiles shared memory -> TMEM with `tcgen05.cp`
// and issues four K=32 MMAs whose descriptors select the scale byte of their 32-element block.
//
// Scale factors are stored in the tile order the hardware reads: for rows [128*i, +128) and k-blocks
// [4*j, +4) (= 128 K elements) one 512-byte tile at ((i * K/128) + j) * 512, inside which row r and k-block
// b sit at (r % 32) * 16 + (r / 32) * 4 + b. The quantiser (elementwise.cu, tiled mode) writes that order
// directly, so neither operand's scales are ever re-laid-out.
//
// The tile is 128 x 192: one K=32 MMA then reads 4 KB of A and 6 KB of B per 96 tensor-core clocks, which stays under
// the shared-memory read rate (a 128 x 128 tile needs the full rate and measured half the throughput), and two
// accumulators (384 columns) leave TMEM room for double-buffered scale columns. A 192-row B tile starts on a 64-row
// boundary of the 128-row scale tiles: the producer always brings the two scale tiles that cover it and the MMA's
// scale address skips two columns (64 rows) for odd tiles.
//
// Roles (192 threads): warp 0 producer, warp 1 MMA issuer + TMEM owner, warps 2..5 epilogue.
// Replaces the reference's block-scaled FP8 GEMM (tf-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:41-198)
// with the micro-scaling format that sm_100a multiplies natively.
#include "tfb_api.h"
#include "tfb_common.cuh"
#include "tfb_host.h"

namespace tfb {

struct MxGemmParams {
  int M, N, K;
  __nv_bfloat16* out;
  int ldo;
  const uint8_t* sfa;  // tiled UE8M0 scales of A: [ceil(M/128)][K/128][512]
  const uint8_t* sfb;  // tiled UE8M0 scales of B: [ceil(N/128)][K/128][512]
  const __nv_bfloat16* bias;
  const __nv_bfloat16* resid;
  int ldr;
  const float* gate;
  int ldg, rows_per_gate;
  int epi;
  int m_tiles, n_tiles;
  int sfb_tiles;  // 128-row scale tiles of B: ceil(N / 128)
  int* status;
};

struct MxCfg {
  static constexpr int BM = 128, BN = 192, BK = 128;  // BK in elements = bytes
  static constexpr int STAGES = 5;
  static constexpr int A_BYTES = BM * BK;
  static constexpr int B_BYTES = BN * BK;
  static constexpr int SF_BYTES = 512;        // one scale tile: 128 rows x 4 k-blocks
  static constexpr int SF_REGION = 2048;      // A tile, two B tiles, padding that keeps stages 1024-byte aligned
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SF_REGION;  // 42 KB
  static constexpr int ACC_COLS = 2 * BN;     // double-buffered accumulator
  static constexpr int SFA_COL = ACC_COLS;    // 2 x 4 columns (alternating by k-block)
  static constexpr int SFB_COL = ACC_COLS + 8;  // 2 x 8 columns
  static constexpr int TMEM_COLS = 512;
  static_assert(SFB_COL + 16 <= TMEM_COLS && STAGE_BYTES % 1024 == 0, "TMEM / shared-memory budget");
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

__device__ __forceinline__ void mx_bulk_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, replicated into the four 32-lane quarters.
__device__ __forceinline__ void tmem_cp_sf(uint32_t tmem_col, uint32_t smem_addr) {
  const uint64_t desc = make_smem_desc(smem_addr, 0, 128, 0);  // no swizzle, 8-row groups 128 bytes apart
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(desc) : "memory");
}

__global__ void __launch_bounds__(192, 1)
    gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const MxGemmParams p) {
  using Cfg = MxCfg;
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
  const int k_blocks = p.K / Cfg::BK;
  // Tiles are walked in bands of 8 M tiles so that the CTAs running at the same time share both a few A row
  // blocks and a few B row blocks in L2.
  auto map_tile = [&](int t, int& m_blk, int& n_blk) {
    constexpr int BAND = 8;
    const int per_band = BAND * p.n_tiles;
    const int band = t / per_band;
    const int rows_in_band = min(BAND, p.m_tiles - band * BAND);
    const int r = t - band * per_band;
    m_blk = band * BAND + r % rows_in_band;
    n_blk = r / rows_in_band;
  };

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += n_cta) {
        int m_blk, n_blk;
        map_tile(t, m_blk, n_blk);
        const uint8_t* sfa = p.sfa + static_cast<size_t>(m_blk) * k_blocks * Cfg::SF_BYTES;
        // rows [192 n, 192 n + 192) live in scale tiles floor(3 n / 2) and the next one
        const int sfb_tile = (3 * n_blk) >> 1;
        const bool two_b = sfb_tile + 1 < p.sfb_tiles;
        const uint8_t* sfb = p.sfb + static_cast<size_t>(sfb_tile) * k_blocks * Cfg::SF_BYTES;
        const uint8_t* sfb2 = sfb + static_cast<size_t>(k_blocks) * Cfg::SF_BYTES;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, ctx, 41)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * Cfg::STAGE_BYTES;
          uint8_t* b_dst = a_dst + Cfg::A_BYTES;
          uint8_t* sf_dst = b_dst + Cfg::B_BYTES;
          mbar_expect_tx(&full[s], Cfg::A_BYTES + Cfg::B_BYTES + (two_b ? 3 : 2) * Cfg::SF_BYTES);
          tma_load_2d(a_dst, &tmA, &full[s], kb * Cfg::BK, m_blk * Cfg::BM);
          tma_load_2d(b_dst, &tmB, &full[s], kb * Cfg::BK, n_blk * Cfg::BN);
          mx_bulk_load(sf_dst, sfa + static_cast<size_t>(kb) * Cfg::SF_BYTES, Cfg::SF_BYTES, &full[s]);
          mx_bulk_load(sf_dst + Cfg::SF_BYTES, sfb + static_cast<size_t>(kb) * Cfg::SF_BYTES, Cfg::SF_BYTES,
                       &full[s]);
          if (two_b)  // past the last scale tile only columns beyond N would use it; those are never stored
            mx_bulk_load(sf_dst + 2 * Cfg::SF_BYTES, sfb2 + static_cast<size_t>(kb) * Cfg::SF_BYTES, Cfg::SF_BYTES,
                         &full[s]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    uint32_t it = 0, tile_iter = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += n_cta) {
      int m_blk, n_blk;
      map_tile(t, m_blk, n_blk);
      const uint32_t sfb_shift = (n_blk & 1) * 2;  // odd tiles start 64 rows into their first scale tile
      const uint32_t acc = tile_iter & 1;
      const uint32_t accph = (tile_iter >> 1) & 1;
      ++tile_iter;
      if (!mbar_wait_warp(&tempty[acc], accph ^ 1, ctx, 42)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * Cfg::BN;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait_warp(&full[s], ph, ctx, 43)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
          const uint32_t sf_addr = b_addr + Cfg::B_BYTES;
          // tcgen05.cp and tcgen05.mma of one thread run in issue order; the scale columns alternate between two
          // sets so that a copy never has to wait for the previous k-block's MMAs to drain.
          const uint32_t sfa_tmem = tmem_base + Cfg::SFA_COL + (kb & 1) * 4;
          const uint32_t sfb_tmem = tmem_base + Cfg::SFB_COL + (kb & 1) * 8;
          tmem_cp_sf(sfa_tmem, sf_addr);
          tmem_cp_sf(sfb_tmem, sf_addr + Cfg::SF_BYTES);
          tmem_cp_sf(sfb_tmem + 4, sf_addr + 2 * Cfg::SF_BYTES);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t idesc = make_idesc_mx(128, Cfg::BN, 0, 0, kk, kk);
            umma_mxf8_ss(d_tmem, make_desc_k_sw128(a_addr + kk * 32), make_desc_k_sw128(b_addr + kk * 32), idesc,
                         sfa_tmem, sfb_tmem + sfb_shift, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          if (kb == k_blocks - 1) umma_commit(&tfull[acc]);
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
      int m_blk, n_blk;
      map_tile(t, m_blk, n_blk);
      const uint32_t acc = tile_iter & 1;
      const uint32_t accph = (tile_iter >> 1) & 1;
      ++tile_iter;
      if (!mbar_wait_warp(&tfull[acc], accph, ctx, 44)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m_blk * Cfg::BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      __nv_bfloat16* out_row = p.out + static_cast<size_t>(row) * p.ldo;
      const float* gate_row =
          p.gate ? p.gate + static_cast<size_t>(row_ok ? row / p.rows_per_gate : 0) * p.ldg : nullptr;
#pragma unroll 1
      for (int c = 0; c < Cfg::BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * Cfg::BN + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_blk * Cfg::BN + c * 32;
        if (!row_ok || col0 >= p.N) continue;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        if (col0 + 32 <= p.N) {
          if (p.bias) {
            const uint4* bp = reinterpret_cast<const uint4*>(p.bias + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 b = __ldg(bp + j);
              const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                v[j * 8 + e * 2] += bf16_lo(w[e]);
                v[j * 8 + e * 2 + 1] += bf16_hi(w[e]);
              }
            }
          }
          if (p.epi == TFB_EPI_GELU) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
          }
          if (gate_row) {
            const float4* gp = reinterpret_cast<const float4*>(gate_row + col0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 g = __ldg(gp + j);
              v[j * 4] *= g.x;
              v[j * 4 + 1] *= g.y;
              v[j * 4 + 2] *= g.z;
              v[j * 4 + 3] *= g.w;
            }
          }
          if (p.resid) {
            const uint4* rp = reinterpret_cast<const uint4*>(p.resid + static_cast<size_t>(row) * p.ldr + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 b = rp[j];
              const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                v[j * 8 + e * 2] += bf16_lo(w[e]);
                v[j * 8 + e * 2 + 1] += bf16_hi(w[e]);
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
          for (int i = 0; i < 32; ++i) {  // ragged N edge
            const int col = col0 + i;
            if (col >= p.N) break;
            float x = v[i];
            if (p.bias) x += __bfloat162float(p.bias[col]);
            if (p.epi == TFB_EPI_GELU) x = gelu_tanh(x);
            if (gate_row) x *= gate_row[col];
            if (p.resid) x += __bfloat162float(p.resid[static_cast<size_t>(row) * p.ldr + col]);
            out_row[col] = __float2bfloat16(x);
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

}  // namespace tfb

using namespace tfb;

// A [M, K] e4m3 (row stride lda bytes), B [N, K] e4m3 (row stride ldb bytes), K a multiple of 128;
// sfa / sfb: tiled UE8M0 scales (see the head of this file) covering ceil(M/128)*128 and ceil(N/128)*128 rows.
extern "C" int tfb_gemm_mxfp8(const void* A, int lda, const void* sfa, const void* B, int ldb, const void* sfb,
                              void* out, int ldo, int M, int N, int K, const void* bias, int epi, const void* resid,
                              int ldr, const float* gate, int ldg, int rows_per_gate, void* stream) {
  if (M <= 0 || N <= 0) return TFB_OK;
  if (K < 128 || K % 128 || N % 8 || ldo % 8 || lda % 16 || ldb % 16 || !sfa || !sfb) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(sfa) | reinterpret_cast<uintptr_t>(sfb)) & 15)
    return TFB_ERR_BAD_SHAPE;
  if (resid && ((ldr % 8) || (reinterpret_cast<uintptr_t>(resid) & 15))) return TFB_ERR_BAD_SHAPE;
  if (gate && ((ldg % 4) || rows_per_gate < 1 || (reinterpret_cast<uintptr_t>(gate) & 15))) return TFB_ERR_BAD_SHAPE;
  if (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) return TFB_ERR_BAD_SHAPE;
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda)};
    uint32_t box[2] = {128u, 128u};
    if (int e = make_tmap(&tmA, A, TM_U8, 2, dims, str, box, TM_SW_128)) return e;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    uint64_t str[1] = {static_cast<uint64_t>(ldb)};
    uint32_t box[2] = {128u, static_cast<uint32_t>(MxCfg::BN)};
    if (int e = make_tmap(&tmB, B, TM_U8, 2, dims, str, box, TM_SW_128)) return e;
  }
  MxGemmParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.resid = static_cast<const __nv_bfloat16*>(resid);
  p.ldr = ldr;
  p.gate = gate;
  p.ldg = ldg;
  p.rows_per_gate = rows_per_gate < 1 ? 1 : rows_per_gate;
  p.epi = epi;
  p.m_tiles = (M + 127) / 128;
  p.n_tiles = (N + MxCfg::BN - 1) / MxCfg::BN;
  p.sfb_tiles = (N + 127) / 128;
  p.status = status_word();
  static bool attr_set[TFB_MAX_DEVICES] = {false};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&gemm_mxfp8_kernel), MxCfg::SMEM_BYTES, attr_set))
    return rc;
  const int tiles = p.m_tiles * p.n_tiles;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_mxfp8_kernel<<<grid, 192, MxCfg::SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}
