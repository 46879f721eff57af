// Persistent, warp-specialised bf16 GEMM for sm_100a:
//   out[M,N] = epilogue(A[M,K] @ B[N,K]^T)      (nn.Linear weight layout)
// TMA (128B swizzle) -> shared-memory ring -> tcgen05.mma (UMMA 128 x BN x 16)
// -> fp32 accumulators in TMEM (double buffered) -> tcgen05.ld epilogue.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM
// owner, warps 2..5 = epilogue (one TMEM lane quarter each).
//
// Epilogue functors fused here (replacing separate elementwise passes of the
// reference's DiT block, telefuser/models/wan_video_dit.py:351-407):
//   bias add, GELU-tanh, residual add, gate * y + residual.
#include "tfb_api.h"
#include "tfb_common.cuh"
#include "tfb_host.h"

namespace tfb {

struct GemmParams {
  int M, N, K;
  __nv_bfloat16* out;
  int ldo;
  const __nv_bfloat16* bias;   // [N] or null
  const __nv_bfloat16* resid;  // [M, ldr] or null
  int ldr;
  const float* gate;  // row r reads gate[(r / rows_per_gate) * ldg + col]; null == 1
  int ldg;
  int rows_per_gate;
  int epi;
  int m_tiles, n_tiles;
  int* status;
  // Grouped mode (mixture of experts): M tile m uses weight rows [tile_expert[m] * N, +N) of B, which
  // then has E * N rows; tiles whose entry is negative (padding past the last expert) are skipped.
  const int* tile_expert;
  // FP8 (e4m3) operands: out = act((A @ B^T) * a_scale[row] * b_scale[col] + bias); null for bf16.
  const float* a_scale;
  const float* b_scale;
  // With the 8-bit template: operands are signed int8 (tcgen05 kind::i8, int32 accumulators) instead of e4m3.
  int int8;
  // Distributed modes (tensor parallel group of n_seg ranks, M = n_seg * seg_rows, one segment per rank;
  // n_seg == 0 otherwise). Tiles never straddle segments: segment s owns M tiles [s*seg_tiles, +seg_tiles).
  // Tile order is rotated by seg_rot tiles so that every rank starts with its own segment.
  int n_seg, seg_rows, seg_tiles, seg_rot;
  // GEMM -> reduce-scatter: the partial tile of segment s is stored into rank s's slab buffer
  // peer_out[s] at rows [src_rank*seg_rows, +seg_rows) (plain peer stores from the epilogue).
  __nv_bfloat16* peer_out[8];
  int src_rank;
  // all-gather -> GEMM: n_copiers CTAs of this launch copy segment s of A from peer_a[s] (contiguous
  // seg_bytes, bulk copies staged through shared memory, each byte crosses NVLink once) into
  // a_gather + s*seg_bytes, which tmA covers; sync[1+s] counts the copiers done with segment s and the
  // TMA producers of the compute CTAs wait (bounded) for it before their first load from that segment.
  const uint8_t* peer_a[8];
  uint8_t* a_gather;
  long long seg_bytes;
  int n_copiers;
  int* sync;  // [0] role ticket, [1 + s] arrivals for segment s; zeroed before the launch
};

template <int BN>
struct GemmCfg {
  static constexpr int BM = 128;
  static constexpr int BK = 64;
  static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

// Untiled bulk copies (16-byte aligned addresses and sizes), global -> shared with mbarrier completion and
// shared -> global in a bulk group; plain per-CTA forms only.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store_1d(void* dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(reinterpret_cast<uint64_t>(dst)),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ unsigned long long gtimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Copier CTA of the all-gather -> GEMM mode: one thread moves this CTA's share of every segment (16 KB
// chunks cid, cid + C, ...) peer -> shared memory -> local gathered A with bulk copies, keeping LOOK loads
// in flight over a ring of NSLOT slots, and publishes each finished segment with a release add.
template <int RING_BYTES>
__device__ void ag_copier(const GemmParams& p, uint8_t* smem, uint64_t* bars, const AbortCtx& ctx, int cid) {
  constexpr int SLOT = 16384;
  constexpr int NSLOT = RING_BYTES / SLOT >= 12 ? 12 : RING_BYTES / SLOT;
  constexpr int LOOK = NSLOT - 4;
  const int C = p.n_copiers;
  const long long n_chunks = (p.seg_bytes + SLOT - 1) / SLOT;
  if (cid >= n_chunks) {  // nothing to move: still counted as done for every segment
    for (int s = 0; s < p.n_seg; ++s) red_release_gpu_add(p.sync + 1 + s, 1);
    return;
  }
  for (int i = 0; i < NSLOT; ++i) mbar_init(&bars[i], 1);
  mbar_fence_init();
  // (order index, chunk) iterators: segments are visited own first, then rank + 1, ...
  int l_oi = 0, s_oi = 0;
  long long l_c = cid, s_c = cid;
  uint32_t kl = 0, ks = 0;
  auto chunk_bytes = [&](long long c) -> uint32_t {
    const long long left = p.seg_bytes - c * SLOT;
    return static_cast<uint32_t>(left < SLOT ? left : SLOT);
  };
  auto issue_load = [&]() {
    if (l_oi >= p.n_seg) return;
    const int seg = (p.src_rank + l_oi) % p.n_seg;
    const int slot = kl % NSLOT;
    if (kl >= static_cast<uint32_t>(NSLOT)) asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
    const uint32_t nb = chunk_bytes(l_c);
    mbar_expect_tx(&bars[slot], nb);
    bulk_load_1d(smem + slot * SLOT, p.peer_a[seg] + l_c * SLOT, nb, &bars[slot]);
    ++kl;
    l_c += C;
    if (l_c >= n_chunks) {
      l_c = cid;
      ++l_oi;
    }
  };
  for (int i = 0; i < LOOK; ++i) issue_load();
  bool ok = true;
  while (s_oi < p.n_seg && ok) {
    const int seg = (p.src_rank + s_oi) % p.n_seg;
    const int slot = ks % NSLOT;
    if (!mbar_wait(&bars[slot], (ks / NSLOT) & 1, ctx, 6)) {
      ok = false;
      break;
    }
    bulk_store_1d(p.a_gather + seg * p.seg_bytes + s_c * SLOT, smem + slot * SLOT, chunk_bytes(s_c));
    tma_store_commit();
    ++ks;
    s_c += C;
    const bool seg_done = s_c >= n_chunks;
    if (seg_done) {
      s_c = cid;
      ++s_oi;
    }
    issue_load();
    if (seg_done) {
      tma_store_wait_all();
      fence_proxy_async_all();
      red_release_gpu_add(p.sync + 1 + seg, 1);
    }
  }
  tma_store_wait_all();
  if (!ok) __nanosleep(200000);  // loads in flight land before the CTA's shared memory goes away
}

// FP8: operands are e4m3 bytes. A stage row is still 128 bytes (128 elements instead of 64), so the
// shared-memory layout, descriptors and the K-step of 32 bytes are those of the bf16 kernel; only the
// MMA kind (K = 32 per instruction), the element count per stage and the epilogue scales differ.
// DIST: the M tiles are grouped in per-rank segments (see GemmParams) for the fused collective modes.
template <int BN, bool FP8 = false, bool DIST = false>
__global__ void __launch_bounds__(192, 1)
    gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int BKE = FP8 ? 2 * Cfg::BK : Cfg::BK;  // K elements per stage
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

  // CTA index among the compute CTAs and their count. With copiers, roles go by arrival ticket so that
  // the copiers are CTAs that are certainly running when a compute CTA starts to wait for them.
  int cta = blockIdx.x, n_cta = gridDim.x;
  if (DIST && p.n_copiers > 0) {
    if (threadIdx.x == 0) {
      *abort_flag = 0;
      *tmem_slot = static_cast<uint32_t>(atomicAdd(p.sync, 1));
    }
    __syncthreads();
    const int ticket = static_cast<int>(*tmem_slot);
    __syncthreads();
    if (ticket < p.n_copiers) {
      if (threadIdx.x == 0) ag_copier<STAGES * Cfg::STAGE_BYTES>(p, smem, bars, ctx, ticket);
      return;
    }
    cta = ticket - p.n_copiers;
    n_cta = gridDim.x - p.n_copiers;
  }
  // Tile t -> (M tile, N tile, segment, tile within the segment, first A row).
  auto map_tile = [&](int t, int& m_blk, int& n_blk, int& seg, int& lt, int& a_row) {
    if (!DIST && !p.tile_expert) {
      // Bands of 8 M tiles, walked M-fastest: the ~148 tiles in flight cover 8 row blocks of A and ~18 row blocks
      // of B instead of 7 x all of B, so both operands of a wave stay in L2 and A is fetched from DRAM once.
      constexpr int BAND = 8;
      const int per_band = BAND * p.n_tiles;
      const int band = t / per_band;
      const int rows_in_band = min(BAND, p.m_tiles - band * BAND);
      const int r = t - band * per_band;
      m_blk = band * BAND + r % rows_in_band;
      n_blk = r / rows_in_band;
    } else {
      m_blk = t / p.n_tiles;
      n_blk = t % p.n_tiles;
    }
    if (DIST) {
      m_blk = (m_blk + p.seg_rot) % p.m_tiles;
      seg = m_blk / p.seg_tiles;
      lt = m_blk % p.seg_tiles;
      a_row = seg * p.seg_rows + lt * Cfg::BM;
    } else {
      seg = 0;
      lt = m_blk;
      a_row = m_blk * Cfg::BM;
    }
  };

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
  const int k_blocks = (p.K + BKE - 1) / BKE;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      uint32_t seg_ready = 0;
      for (int t = cta; t < num_tiles && ok; t += n_cta) {
        int m_blk, n_blk, seg, lt, a_row;
        map_tile(t, m_blk, n_blk, seg, lt, a_row);
        int b_row = n_blk * BN;
        if (p.tile_expert) {
          const int e = __ldg(p.tile_expert + m_blk);
          if (e < 0) continue;
          b_row += e * p.N;
        }
        if (DIST && p.n_copiers > 0 && !(seg_ready >> seg & 1u)) {
          // Bounded wait for the copiers to land this segment of A in local memory.
          const unsigned long long t0 = gtimer_ns();
          while (ld_acquire_gpu(p.sync + 1 + seg) < p.n_copiers) {
            if (*abort_flag || gtimer_ns() - t0 > 2000000000ull) {
              *abort_flag = 1;
              if (p.status) atomicCAS(p.status, 0, TFB_ERR_TIMEOUT | (5 << 8));
              ok = false;
              break;
            }
            __nanosleep(100);
          }
          if (!ok) break;
          fence_proxy_async_all();
          seg_ready |= 1u << seg;
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, ctx, 1)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * Cfg::STAGE_BYTES;
          uint8_t* b_dst = a_dst + Cfg::A_BYTES;
          mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, &full[s], kb * BKE, a_row);
          tma_load_2d(b_dst, &tmB, &full[s], kb * BKE, b_row);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc = FP8 ? make_idesc(128, BN, 0, 0, 0, 0) : make_idesc(128, BN, 1, 1, 0, 0);
    constexpr uint32_t idesc_i8 = make_idesc_i8(128, BN);
    const bool int8 = FP8 && p.int8;
    uint32_t it = 0;
    uint32_t tile_iter = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += n_cta) {
      if (p.tile_expert && __ldg(p.tile_expert + t / p.n_tiles) < 0) continue;
      const uint32_t acc = tile_iter & 1;
      const uint32_t accph = (tile_iter >> 1) & 1;
      ++tile_iter;
      if (!mbar_wait_warp(&tempty[acc], accph ^ 1, ctx, 2)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait_warp(&full[s], ph, ctx, 3)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < Cfg::BK / 16; ++kk) {
            const uint64_t ad = make_desc_k_sw128(a_addr + kk * 32);
            const uint64_t bd = make_desc_k_sw128(b_addr + kk * 32);
            if (FP8 && int8)
              umma_i8_ss(d_tmem, ad, bd, idesc_i8, (kb | kk) != 0 ? 1u : 0u);
            else if (FP8)
              umma_f8_ss(d_tmem, ad, bd, idesc, (kb | kk) != 0 ? 1u : 0u);
            else
              umma_f16_ss(d_tmem, ad, bd, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          if (kb == k_blocks - 1) umma_commit(&tfull[acc]);
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------- Epilogue ----------------
    const int q = warp & 3;
    uint32_t tile_iter = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += n_cta) {
      int m_blk, n_blk, seg, lt, a_row;
      map_tile(t, m_blk, n_blk, seg, lt, a_row);
      if (p.tile_expert && __ldg(p.tile_expert + m_blk) < 0) continue;
      const uint32_t acc = tile_iter & 1;
      const uint32_t accph = (tile_iter >> 1) & 1;
      ++tile_iter;
      if (!mbar_wait_warp(&tfull[acc], accph, ctx, 4)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = a_row + q * 32 + lane;
      const bool row_ok = DIST ? (lt * Cfg::BM + q * 32 + lane < p.seg_rows) : (row < p.M);
      // Row of the destination: the local output, or the slab of the rank that owns this segment.
      __nv_bfloat16* out_row = p.out + static_cast<size_t>(row) * p.ldo;
      if (DIST && p.peer_out[0])
        out_row = p.peer_out[seg] + (static_cast<size_t>(p.src_rank) * p.seg_rows + (row - seg * p.seg_rows)) * p.ldo;
      const float* gate_row =
          p.gate ? p.gate + static_cast<size_t>(row_ok ? row / p.rows_per_gate : 0) * p.ldg : nullptr;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32;
        tmem_ld_32x32(taddr, r);
        tmem_ld_wait();
        const int col0 = n_blk * BN + c * 32;
        if (row_ok && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          const bool full_chunk = col0 + 32 <= p.N;
          if (FP8 && p.int8) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = static_cast<float>(static_cast<int>(r[i]));
          }
          if (FP8) {
            const float as = __ldg(p.a_scale + row);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= as * ((full_chunk || col0 + i < p.N) ? __ldg(p.b_scale + col0 + i) : 0.f);
          }
          if (full_chunk) {
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
            // Ragged N edge: scalar path.
            for (int i = 0; i < 32; ++i) {
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  // Teardown: everyone meets, then the allocating warp frees TMEM.
  if (*abort_flag) __nanosleep(200000);  // let copies in flight land before the CTA exits
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

template <int BN, bool FP8 = false, bool DIST = false>
static int launch_gemm(const CUtensorMap& tmA, const void* B, int ldb, GemmParams p, cudaStream_t stream,
                       long b_rows = 0) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmB;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(p.K), static_cast<uint64_t>(b_rows > 0 ? b_rows : p.N)};
    uint64_t str[1] = {static_cast<uint64_t>(ldb) * (FP8 ? 1 : 2)};
    uint32_t box[2] = {FP8 ? 128u : 64u, static_cast<uint32_t>(BN)};
    int e = make_tmap(&tmB, B, FP8 ? TM_U8 : TM_BF16, 2, dims, str, box, TM_SW_128);
    if (e) return e;
  }
  p.m_tiles = DIST ? p.n_seg * p.seg_tiles : (p.M + 127) / 128;
  p.n_tiles = (p.N + BN - 1) / BN;
  static bool attr_set[TFB_MAX_DEVICES] = {false};
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&gemm_bf16_kernel<BN, FP8, DIST>), Cfg::SMEM_BYTES, attr_set)) return rc;
  const int tiles = p.m_tiles * p.n_tiles;
  const int copiers = DIST ? p.n_copiers : 0;
  const int compute = tiles < sm_count() - copiers ? tiles : sm_count() - copiers;
  const int grid = compute + copiers;
  gemm_bf16_kernel<BN, FP8, DIST><<<grid, 192, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

}  // namespace tfb

extern "C" int tfb_gemm_bf16(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N,
                             int K, const void* bias, int epi, const void* resid, int ldr, const float* gate,
                             int ldg, int rows_per_gate, int force_bn, void* stream) {
  using namespace tfb;
  if (M <= 0 || N <= 0 || K <= 0) return TFB_ERR_BAD_SHAPE;
  if ((K % 8) || (lda % 8) || (ldb % 8) || (ldo % 8) || (N % 8)) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out)) & 15)
    return TFB_ERR_BAD_SHAPE;
  if (resid && ((ldr % 8) || (reinterpret_cast<uintptr_t>(resid) & 15))) return TFB_ERR_BAD_SHAPE;
  if (gate && ((ldg % 4) || (reinterpret_cast<uintptr_t>(gate) & 15))) return TFB_ERR_BAD_SHAPE;
  if (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) return TFB_ERR_BAD_SHAPE;
  GemmParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.resid = static_cast<const __nv_bfloat16*>(resid);
  p.ldr = ldr;
  p.gate = gate;
  p.ldg = ldg;
  p.rows_per_gate = rows_per_gate > 0 ? rows_per_gate : 1;
  p.epi = epi;
  p.status = status_word();
  p.tile_expert = nullptr;
  p.a_scale = p.b_scale = nullptr;
  p.int8 = 0;
  p.n_seg = 0;
  p.n_copiers = 0;
  CUtensorMap tmA;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {64, 128};
    int e = make_tmap(&tmA, A, TM_BF16, 2, dims, str, box, TM_SW_128);
    if (e) return e;
  }
  int bn = force_bn;
  if (bn != 256 && bn != 128 && bn != 64) {
    const long m_tiles = (M + 127) / 128;
    const int sms = sm_count();
    if (N % 256 == 0 && m_tiles * (N / 256) >= sms)
      bn = 256;
    else if (N >= 128 && m_tiles * ((N + 127) / 128) >= sms / 2)
      bn = 128;
    else
      bn = N >= 128 ? 128 : 64;
    if (N < 128) bn = 64;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (bn) {
    case 256: return launch_gemm<256>(tmA, B, ldb, p, st);
    case 128: return launch_gemm<128>(tmA, B, ldb, p, st);
    default: return launch_gemm<64>(tmA, B, ldb, p, st);
  }
}

// Grouped GEMM for expert layers: rows of A are tokens sorted by expert, every expert's segment
// starts on a multiple of 128 rows; M tile m multiplies with expert tile_expert[m]'s weights
// B[e] = rows [e*N, (e+1)*N) of B (bf16 [E*N, K]). `M` is the padded row count (upper bound).
extern "C" int tfb_gemm_bf16_grouped(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N,
                                     int K, int num_experts, const int* tile_expert, int epi, void* stream) {
  using namespace tfb;
  if (M <= 0 || N <= 0 || K <= 0 || num_experts <= 0 || !tile_expert) return TFB_ERR_BAD_SHAPE;
  if ((K % 8) || (lda % 8) || (ldb % 8) || (ldo % 8) || (N % 64) || (M % 128)) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out)) & 15)
    return TFB_ERR_BAD_SHAPE;
  GemmParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.bias = nullptr;
  p.resid = nullptr;
  p.ldr = 0;
  p.gate = nullptr;
  p.ldg = 0;
  p.rows_per_gate = 1;
  p.epi = epi;
  p.status = status_word();
  p.tile_expert = tile_expert;
  p.a_scale = p.b_scale = nullptr;
  p.int8 = 0;
  p.n_seg = 0;
  p.n_copiers = 0;
  CUtensorMap tmA;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {64, 128};
    int e = make_tmap(&tmA, A, TM_BF16, 2, dims, str, box, TM_SW_128);
    if (e) return e;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long b_rows = static_cast<long>(num_experts) * N;
  if (N % 256 == 0) return launch_gemm<256>(tmA, B, ldb, p, st, b_rows);
  if (N % 128 == 0) return launch_gemm<128>(tmA, B, ldb, p, st, b_rows);
  return launch_gemm<64>(tmA, B, ldb, p, st, b_rows);
}

// W8A8 GEMM: A e4m3 [M, K] with one fp32 scale per row (per-token), B e4m3 [N, K] with one fp32 scale
// per row (per-output-channel); out bf16 = epilogue((A @ B^T) * a_scale[m] * b_scale[n]).
static int gemm_8bit(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N, int K,
                     const float* a_scale, const float* b_scale, const void* bias, int epi, const void* resid, int ldr,
                     const float* gate, int ldg, int rows_per_gate, int int8, void* stream) {
  using namespace tfb;
  if (M <= 0 || N <= 0 || K <= 0 || !a_scale || !b_scale) return TFB_ERR_BAD_SHAPE;
  if ((K % 16) || (lda % 16) || (ldb % 16) || (ldo % 8) || (N % 8)) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out)) & 15)
    return TFB_ERR_BAD_SHAPE;
  if (resid && ((ldr % 8) || (reinterpret_cast<uintptr_t>(resid) & 15))) return TFB_ERR_BAD_SHAPE;
  if (gate && ((ldg % 4) || (reinterpret_cast<uintptr_t>(gate) & 15))) return TFB_ERR_BAD_SHAPE;
  if (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) return TFB_ERR_BAD_SHAPE;
  GemmParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.resid = static_cast<const __nv_bfloat16*>(resid);
  p.ldr = ldr;
  p.gate = gate;
  p.ldg = ldg;
  p.rows_per_gate = rows_per_gate > 0 ? rows_per_gate : 1;
  p.epi = epi;
  p.status = status_word();
  p.tile_expert = nullptr;
  p.a_scale = a_scale;
  p.b_scale = b_scale;
  p.int8 = int8;
  p.n_seg = 0;
  p.n_copiers = 0;
  CUtensorMap tmA;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda)};
    uint32_t box[2] = {128, 128};
    int e = make_tmap(&tmA, A, TM_U8, 2, dims, str, box, TM_SW_128);
    if (e) return e;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long m_tiles = (M + 127) / 128;
  if (N % 256 == 0 && m_tiles * (N / 256) >= sm_count()) return launch_gemm<256, true>(tmA, B, ldb, p, st);
  if (N >= 128) return launch_gemm<128, true>(tmA, B, ldb, p, st);
  return launch_gemm<64, true>(tmA, B, ldb, p, st);
}

// W8A8 with e4m3 operands: out = epilogue((A @ B^T) * a_scale[row] * b_scale[col]).
extern "C" int tfb_gemm_fp8(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N, int K,
                            const float* a_scale, const float* b_scale, const void* bias, int epi, const void* resid,
                            int ldr, const float* gate, int ldg, int rows_per_gate, void* stream) {
  return gemm_8bit(A, lda, B, ldb, out, ldo, M, N, K, a_scale, b_scale, bias, epi, resid, ldr, gate, ldg, rows_per_gate, 0,
                   stream);
}

// W8A8 with signed 8-bit integer operands (tcgen05 kind::i8, exact int32 accumulation), same scales and epilogue.
// Takes the place of the reference's int8 scaled GEMM (tf-kernel/csrc/gemm/int8_gemm_kernel.cu).
extern "C" int tfb_gemm_int8(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N, int K,
                             const float* a_scale, const float* b_scale, const void* bias, int epi, const void* resid,
                             int ldr, const float* gate, int ldg, int rows_per_gate, void* stream) {
  return gemm_8bit(A, lda, B, ldb, out, ldo, M, N, K, a_scale, b_scale, bias, epi, resid, ldr, gate, ldg, rows_per_gate, 1,
                   stream);
}

namespace tfb {
static void dist_defaults(GemmParams& p, int n_seg, int rank, int seg_rows, int N, int K) {
  p.M = n_seg * seg_rows;
  p.N = N;
  p.K = K;
  p.bias = nullptr;
  p.resid = nullptr;
  p.ldr = 0;
  p.gate = nullptr;
  p.ldg = 0;
  p.rows_per_gate = 1;
  p.epi = 0;
  p.status = status_word();
  p.tile_expert = nullptr;
  p.a_scale = p.b_scale = nullptr;
  p.int8 = 0;
  p.n_seg = n_seg;
  p.seg_rows = seg_rows;
  p.seg_tiles = (seg_rows + 127) / 128;
  p.seg_rot = rank * p.seg_tiles;
  p.src_rank = rank;
  p.n_copiers = 0;
  p.sync = nullptr;
  p.a_gather = nullptr;
  p.seg_bytes = 0;
  for (int i = 0; i < 8; ++i) {
    p.peer_out[i] = nullptr;
    p.peer_a[i] = nullptr;
  }
}
}  // namespace tfb

// GEMM -> reduce-scatter over peer memory. A [n_seg*seg_rows, K] holds this rank's K-shard of the
// activations, B [N, K] its K-shard of the weight. The partial product of row segment s is stored by the
// epilogue straight into rank s's slab buffer peer_out[s] ([n_seg, seg_rows, ldo] bf16) at slab `rank`.
// After a barrier every rank sums its n_seg slabs (tfb_slab_reduce).
extern "C" int tfb_gemm_bf16_rs(const void* A, int lda, const void* B, int ldb, void* const* peer_out, int ldo,
                                int n_seg, int rank, int seg_rows, int N, int K, const void* bias, void* stream) {
  using namespace tfb;
  if (n_seg < 1 || n_seg > 8 || rank < 0 || rank >= n_seg || seg_rows <= 0 || N <= 0 || K <= 0 || !peer_out)
    return TFB_ERR_BAD_SHAPE;
  if ((K % 8) || (lda % 8) || (ldb % 8) || (ldo % 8) || (N % 8)) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) return TFB_ERR_BAD_SHAPE;
  GemmParams p;
  dist_defaults(p, n_seg, rank, seg_rows, N, K);
  p.out = nullptr;
  p.ldo = ldo;
  if (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) return TFB_ERR_BAD_SHAPE;
  p.bias = static_cast<const __nv_bfloat16*>(bias);  // added to this rank's partial: give it to one rank only
  for (int i = 0; i < n_seg; ++i) {
    if (!peer_out[i] || (reinterpret_cast<uintptr_t>(peer_out[i]) & 15)) return TFB_ERR_BAD_SHAPE;
    p.peer_out[i] = static_cast<__nv_bfloat16*>(peer_out[i]);
  }
  CUtensorMap tmA;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(p.M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {64, 128};
    int e = make_tmap(&tmA, A, TM_BF16, 2, dims, str, box, TM_SW_128);
    if (e) return e;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long tiles256 = static_cast<long>(n_seg) * p.seg_tiles * (N / 256);
  if (N % 256 == 0 && tiles256 >= sm_count()) return launch_gemm<256, false, true>(tmA, B, ldb, p, st);
  return launch_gemm<128, false, true>(tmA, B, ldb, p, st);
}

// all-gather -> GEMM over peer memory. Every rank holds seg_rows rows of A (contiguous [seg_rows, K]
// bf16, peer_a[s] on rank s); B [N, K] is this rank's weight shard. `n_copiers` CTAs of the launch pull
// the segments into a_gather ([n_seg*seg_rows, K], local) while the other CTAs multiply the segments
// that have landed; out [n_seg*seg_rows, ldo] = act(A_full @ B^T + bias). `sync` is 16 ints of local
// scratch. The caller guarantees (barrier) that every peer's shard is complete before the launch and
// not overwritten before all ranks have finished theirs.
extern "C" int tfb_gemm_bf16_ag(void* const* peer_a, void* a_gather, int* sync, int n_copiers, const void* B, int ldb,
                                void* out, int ldo, int n_seg, int rank, int seg_rows, int N, int K, const void* bias,
                                int epi, void* stream) {
  using namespace tfb;
  if (n_seg < 1 || n_seg > 8 || rank < 0 || rank >= n_seg || seg_rows <= 0 || N <= 0 || K <= 0) return TFB_ERR_BAD_SHAPE;
  if (!peer_a || !a_gather || !sync || n_copiers < 1 || n_copiers > 32) return TFB_ERR_BAD_SHAPE;
  if ((K % 8) || (ldb % 8) || (ldo % 8) || (N % 8)) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(a_gather) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out)) & 15)
    return TFB_ERR_BAD_SHAPE;
  if (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) return TFB_ERR_BAD_SHAPE;
  GemmParams p;
  dist_defaults(p, n_seg, rank, seg_rows, N, K);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.epi = epi;
  p.seg_bytes = static_cast<long long>(seg_rows) * K * 2;
  p.a_gather = static_cast<uint8_t*>(a_gather);
  p.n_copiers = n_copiers;
  p.sync = sync;
  for (int i = 0; i < n_seg; ++i) {
    if (!peer_a[i] || (reinterpret_cast<uintptr_t>(peer_a[i]) & 15)) return TFB_ERR_BAD_SHAPE;
    p.peer_a[i] = static_cast<const uint8_t*>(peer_a[i]);
  }
  CUtensorMap tmA;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(p.M)};
    uint64_t str[1] = {static_cast<uint64_t>(K) * 2};
    uint32_t box[2] = {64, 128};
    int e = make_tmap(&tmA, a_gather, TM_BF16, 2, dims, str, box, TM_SW_128);
    if (e) return e;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(sync, 0, 16 * sizeof(int), st) != cudaSuccess) return TFB_ERR_LAUNCH;
  const long tiles256 = static_cast<long>(n_seg) * p.seg_tiles * (N / 256);
  if (N % 256 == 0 && tiles256 >= sm_count()) return launch_gemm<256, false, true>(tmA, B, ldb, p, st);
  return launch_gemm<128, false, true>(tmA, B, ldb, p, st);
}
