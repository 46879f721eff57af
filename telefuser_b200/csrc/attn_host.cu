// C entry points of the attention kernels: argument checks, tensor maps, kernel selection.
//
// `variant` selects the kernel for benchmarks and regression tests: 30 / 31 / 32 = two threads per query row with
// none / a quarter / half of the exponentials on the FMA pipe, 20 / 21 / 22 = one thread per query row (head_dim
// 128, no causal mask) with those shares. 0 = default: all exponentials on the MUFU pipe (the polynomial shares
// measured slower in both kernels), and for plain dense head_dim-128 attention the kernel by key count: one thread
// per row below 48k keys (987 vs 933 TFLOP/s at 16k keys x 12 heads), two threads per row from there on (1066 -
// 1076 vs 1016 - 1039 TFLOP/s at 75,600 keys x 5 heads).
// Role in the reference: the attention dispatch of telefuser/ops/attention/attention_impl.py:213-300 (SDPA, cuDNN,
// FlashAttention and SageAttention back ends behind one call).
#include "attn_common.cuh"
#include "tfb_api.h"

using namespace tfb;

static int attn_fwd_impl(const void* q, long ldq, long bsq, const void* k, long ldk, long bsk, const void* v,
                         long ldv, long bsv, void* out, long ldo, long bso, float* lse, int B, int H, int Sq, int Skv,
                         int D, int causal, float scale, int variant, const int* blk_idx, const int* blk_cnt,
                         int max_blocks, void* stream) {
  if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0 || (D != 64 && D != 128)) return TFB_ERR_BAD_SHAPE;
  if (causal && Skv < Sq) return TFB_ERR_BAD_SHAPE;
  if ((ldq | ldk | ldv | ldo | bsq | bsk | bsv | bso) % 8) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return TFB_ERR_BAD_SHAPE;
  CUtensorMap tq, tk, tv;
  int e;
  if ((e = make_qkv_tmap(&tq, q, ldq, bsq, B, Sq, H, D))) return e;
  if ((e = make_qkv_tmap(&tk, k, ldk, bsk, B, Skv, H, D))) return e;
  if ((e = make_qkv_tmap(&tv, v, ldv, bsv, B, Skv, H, D))) return e;
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
  p.poly = (variant >= 20 && variant <= 22) ? variant - 20 : (variant >= 30 && variant <= 32) ? variant - 30 : 0;
  if (variant == 0 && D == 128 && !causal && !blk_idx && Skv < 49152) variant = 20;
  for (int i = 0; i < 8; ++i) p.peer_out[i] = nullptr;
  p.n_peers = 0;
  p.rows_per_rank = 1;
  p.head_off = 0;
  p.blk_idx = blk_idx;
  p.blk_cnt = blk_cnt;
  p.max_blocks = max_blocks;
  p.head_dim = D;
  p.causal = causal;
  p.q_scale = nullptr;
  p.k_scale = nullptr;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (variant >= 20 && variant <= 22) {
    if (D != 128 || causal) return TFB_ERR_BAD_SHAPE;
    return launch_attn2(tq, tk, tv, p, B, st);
  }
  return launch_attn_split(tq, tk, tv, p, B, st);
}

extern "C" int tfb_attn_fwd(const void* q, long ldq, long bsq, const void* k, long ldk, long bsk, const void* v,
                            long ldv, long bsv, void* out, long ldo, long bso, float* lse, int B, int H, int Sq,
                            int Skv, int D, int causal, float scale, int variant, void* stream) {
  return attn_fwd_impl(q, ldq, bsq, k, ldk, bsk, v, ldv, bsv, out, ldo, bso, lse, B, H, Sq, Skv, D, causal, scale,
                       variant, nullptr, nullptr, 0, stream);
}

// Block-sparse attention: blk_idx int32 [B, H, ceil(Sq/256), max_blocks] lists the 128-key blocks every
// 256-row query group attends to, blk_cnt int32 [B, H, ceil(Sq/256)] how many of them are valid.
extern "C" int tfb_attn_fwd_sparse(const void* q, long ldq, long bsq, const void* k, long ldk, long bsk, const void* v,
                                   long ldv, long bsv, void* out, long ldo, long bso, float* lse, int B, int H, int Sq,
                                   int Skv, float scale, const int* blk_idx, const int* blk_cnt, int max_blocks,
                                   int variant, void* stream) {
  if (!blk_idx || !blk_cnt || max_blocks < 1) return TFB_ERR_BAD_SHAPE;
  return attn_fwd_impl(q, ldq, bsq, k, ldk, bsk, v, ldv, bsv, out, ldo, bso, lse, B, H, Sq, Skv, 128, 0, scale,
                       variant, blk_idx, blk_cnt, max_blocks, stream);
}

// Attention whose epilogue performs the sequence-parallel "gather heads" exchange: this rank holds
// H local heads of all Sq tokens; output row g goes to rank g / rows_per_rank, into its buffer
// peer_out[rank] laid out [B, rows_per_rank, H_total*128] (row stride ldo, batch stride bso), at head
// head_off + h. peer_out: HOST array of n_peers device pointers (this rank's own buffer included).
extern "C" int tfb_attn_fwd_peer(const void* q, long ldq, long bsq, const void* k, long ldk, long bsk, const void* v,
                                 long ldv, long bsv, void* const* peer_out, int n_peers, int rows_per_rank,
                                 int head_off, long ldo, long bso, int B, int H, int Sq, int Skv, float scale,
                                 int variant, void* stream) {
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
  p.head_dim = 128;
  p.causal = 0;
  p.q_scale = nullptr;
  p.k_scale = nullptr;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return (variant >= 20 && variant <= 22) ? launch_attn2(tq, tk, tv, p, B, st) : launch_attn_split(tq, tk, tv, p, B, st);
}

// Attention with int8 scores (the role of the reference's SageAttention "qk int8, pv fp16" kernels): q8 / k8 are
// int8 [B, S, H, 128] (strides in bytes = elements), q_scale fp32 [B, H, Sq], k_scale fp32 [B, H]; v and out are
// bf16. softmax((q8 . k8) * q_scale * k_scale * scale) @ v, the product accumulated in int32 by the tensor core.
extern "C" int tfb_attn_fwd_qk8(const void* q8, long ldq, long bsq, const void* k8, long ldk, long bsk, const void* v,
                                long ldv, long bsv, const float* q_scale, const float* k_scale, void* out, long ldo,
                                long bso, int B, int H, int Sq, int Skv, int causal, float scale, void* stream) {
  if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0 || !q_scale || !k_scale) return TFB_ERR_BAD_SHAPE;
  if (causal && Skv < Sq) return TFB_ERR_BAD_SHAPE;
  if ((ldq | ldk | bsq | bsk) % 16 || (ldv | ldo | bsv | bso) % 8) return TFB_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q8) | reinterpret_cast<uintptr_t>(k8) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return TFB_ERR_BAD_SHAPE;
  CUtensorMap tq, tk, tv;
  int e;
  if ((e = make_qk8_tmap(&tq, q8, ldq, bsq, B, Sq, H))) return e;
  if ((e = make_qk8_tmap(&tk, k8, ldk, bsk, B, Skv, H))) return e;
  if ((e = make_qkv_tmap(&tv, v, ldv, bsv, B, Skv, H, 128))) return e;
  AttnParams p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.bso = bso;
  p.lse = nullptr;
  p.H = H;
  p.Sq = Sq;
  p.Skv = Skv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_word();
  p.poly = 1;
  for (int i = 0; i < 8; ++i) p.peer_out[i] = nullptr;
  p.n_peers = 0;
  p.rows_per_rank = 1;
  p.head_off = 0;
  p.blk_idx = nullptr;
  p.blk_cnt = nullptr;
  p.max_blocks = 0;
  p.head_dim = 128;
  p.causal = causal;
  p.q_scale = q_scale;
  p.k_scale = k_scale;
  return launch_attn_split(tq, tk, tv, p, B, static_cast<cudaStream_t>(stream));
}
