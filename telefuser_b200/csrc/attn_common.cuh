// Shared declarations of the attention kernels.
#pragma once
#include "tfb_common.cuh"
#include "tfb_host.h"

namespace tfb {

struct AttnParams {
  __nv_bfloat16* out;
  long ldo, bso;
  float* lse;
  int H, Sq, Skv;
  float scale_log2;
  int* status;
  int poly;  // share of exp2 evaluated on the FMA pipe: 0 none, 1 a quarter, 2 half
  // Sequence-parallel output scatter (Ulysses "gather heads" folded into the epilogue): query row g of
  // this rank's head slice belongs to rank g / rows_per_rank and is stored straight into that rank's
  // buffer [B, rows_per_rank, H_total * 128] (row stride ldo, batch stride bso) at head head_off + h
  // with plain peer stores. n_peers == 0: ordinary local output.
  __nv_bfloat16* peer_out[8];
  int n_peers, rows_per_rank, head_off;
  // Block-sparse attention: for the CTA of (batch b, head h, query pair qp) the 128-key blocks to visit
  // are blk_idx[((b*H + h)*n_qp + qp) * max_blocks + i], i < blk_cnt[(b*H + h)*n_qp + qp]; null = dense.
  const int* blk_idx;
  const int* blk_cnt;
  int max_blocks;
  int head_dim;  // 64 or 128
  int causal;    // key j visible to query row i when j <= i + (Skv - Sq)
  // Int8 scores: q / k operands are int8, q_scale fp32 [B, H, Sq] (one per query token and head) and k_scale
  // fp32 [B, H] (one per head) restore their magnitudes; both null for bf16 operands.
  const float* q_scale;
  const float* k_scale;
};

constexpr int ATT_BM = 128, ATT_BN = 128, ATT_D = 128;
constexpr int ATT_TILE_BYTES = 128 * 128 * 2;  // 32 KB: two 16 KB boxes of [128 rows][64 cols]
constexpr int ATT_BOX_BYTES = 16384;
constexpr float ATT_RESCALE_THRESHOLD = 8.0f;

// 3-D tensor map over [B][S][H*128] int8 with a [1][128][128] box and 128B swizzle (ld / bs in elements = bytes).
inline int make_qk8_tmap(CUtensorMap* m, const void* base, long ld, long bs, int B, int S, int H) {
  uint64_t dims[3] = {static_cast<uint64_t>(H) * 128, static_cast<uint64_t>(S), static_cast<uint64_t>(B)};
  uint64_t str[2] = {static_cast<uint64_t>(ld), static_cast<uint64_t>(bs)};
  uint32_t box[3] = {128, 128, 1};
  return make_tmap(m, base, TM_U8, 3, dims, str, box, TM_SW_128);
}

// 3-D tensor map over [B][S][H*head_dim] bf16 with a [1][128][64] box and 128B swizzle.
inline int make_qkv_tmap(CUtensorMap* m, const void* base, long ld, long bs, int B, int S, int H, int head_dim = ATT_D) {
  uint64_t dims[3] = {static_cast<uint64_t>(H) * head_dim, static_cast<uint64_t>(S), static_cast<uint64_t>(B)};
  uint64_t str[2] = {static_cast<uint64_t>(ld) * 2, static_cast<uint64_t>(bs) * 2};
  uint32_t box[3] = {64, 128, 1};
  return make_tmap(m, base, TM_BF16, 3, dims, str, box, TM_SW_128);
}

// Two query tiles per CTA, each row split over two threads (attn_fwd_split.cu).
int launch_attn_split(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, int B,
                      cudaStream_t st);
// Two query tiles per CTA, one thread per row (attn2_tcgen05.cu): head_dim 128, no causal mask.
int launch_attn2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, int B,
                 cudaStream_t st);

}  // namespace tfb
