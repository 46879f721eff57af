// C ABI of libtfb200: hand-written sm_100a kernels of telefuser_b200.
// All pointers are device pointers unless stated; `stream` is a cudaStream_t.
// Every function returns 0 on success or a TFB_ERR_* code (tfb_common.cuh).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// GEMM epilogue activation selector.
enum { TFB_EPI_NONE = 0, TFB_EPI_GELU = 1 };

int tfb_abi_version();
int tfb_sm_count();
// Reads and clears the per-device status word written by bounded waits (synchronises the device).
int tfb_last_status();
// Non-blocking form for serving loops: tfb_status_post enqueues a copy of the status word into pinned host
// memory on `stream`; tfb_status_peek returns the last copy that has landed, without touching the device.
int tfb_status_post(void* stream);
int tfb_status_peek();
// Upper bound of every wait on another rank (flag barriers), in milliseconds; 4000 by default.
int tfb_set_peer_wait_ms(int ms);

// out[M,N] = resid + gate * act(A[M,K] @ B[N,K]^T + bias)   (bf16 in/out, fp32 accumulate)
//   bias  : bf16 [N] or null
//   resid : bf16 [M, ldr] or null (may alias out)
//   gate  : fp32, row r uses gate[(r / rows_per_gate) * ldg + col], or null (== 1)
//   force_bn: 0 = auto, else 64/128/256 (N tile)
int tfb_gemm_bf16(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N, int K,
                  const void* bias, int epi, const void* resid, int ldr, const float* gate, int ldg,
                  int rows_per_gate, int force_bn, void* stream);

// Flash attention forward, bf16, head_dim D = 64 or 128 (tcgen05 + TMEM).
//   q   : [B, Sq, H, D] with row stride ldq (elements between tokens), batch stride bsq
//   k,v : [B, Skv, H, D] likewise
//   out : [B, Sq, H, D] bf16, row stride ldo
//   lse : optional fp32 [B, H, Sq] (natural log), or null
//   causal: key j is visible to query row i when j <= i + (Skv - Sq); needs Skv >= Sq
//   variant: 0 = default; see attn_host.cu for the benchmark selectors
int tfb_attn_fwd(const void* q, long ldq, long bsq, const void* k, long ldk, long bsk, const void* v, long ldv,
                 long bsv, void* out, long ldo, long bso, float* lse, int B, int H, int Sq, int Skv, int D, int causal,
                 float scale, int variant, void* stream);

// Block-sparse variant: blk_idx int32 [B, H, ceil(Sq/256), max_blocks] lists the 128-key blocks each
// group of 256 query rows attends to (ascending), blk_cnt int32 [B, H, ceil(Sq/256)] how many are valid;
// a group with no block gets zero output.
int tfb_attn_fwd_sparse(const void* q, long ldq, long bsq, const void* k, long ldk, long bsk, const void* v, long ldv,
                        long bsv, void* out, long ldo, long bso, float* lse, int B, int H, int Sq, int Skv, float scale,
                        const int* blk_idx, const int* blk_cnt, int max_blocks, int variant, void* stream);

// Attention with int8 scores: softmax((q8 . k8) * q_scale[b,h,i] * k_scale[b,h] * scale) @ v. q8 / k8 int8
// [B, S, H, 128] (strides in elements), v / out bf16, q_scale fp32 [B, H, Sq], k_scale fp32 [B, H].
int tfb_attn_fwd_qk8(const void* q8, long ldq, long bsq, const void* k8, long ldk, long bsk, const void* v, long ldv,
                     long bsv, const float* q_scale, const float* k_scale, void* out, long ldo, long bso, int B, int H,
                     int Sq, int Skv, int causal, float scale, void* stream);
// Operand preparation for it (attn_quant.cu): per-channel sums and per-head max |k| of K; int8 quantisation of Q
// (per token and head) and of mean-centred K (per head).
int tfb_attn_k_stats(const void* k, long ld, long bs, int B, int S, int H, float* sums, float* amax, void* stream);
int tfb_attn_quant_int8(const void* x, long ld, long bs, void* out, int B, int S, int H, int is_k, const float* mean,
                        const float* k_scale, float* scale_out, void* stream);

// Causal 3-D convolution, stride 1, channels-last, as an implicit GEMM (conv3d_tcgen05.cu). x [B,T,H,W,Cin],
// prev [B,prev_T,H,W,Cin] or null (frames in front of x), w [Cout, kt*kh*kw, Cin], out / resid [B,T,H,W,Cout], bf16.
// pad_t frames of padding in front (the first prev_T of them from `prev`), pad_h / pad_w on both sides.
int tfb_conv3d_causal(const void* x, const void* prev, int prev_T, const void* w, const void* bias, const void* resid,
                      void* out, int B, int T, int H, int W, int Cin, int Cout, int kt, int kh, int kw, int pad_t,
                      int pad_h, int pad_w, void* stream);

// VAE glue on channels-last rows (vae_ops.cu): per-pixel L2 normalisation * sqrt(C) * gamma with optional SiLU, and
// nearest-neighbour 2x spatial upsampling.
int tfb_pixel_norm_act(const void* x, void* out, long pixels, int C, const float* gamma, int silu, void* stream);
int tfb_upsample2x_nearest(const void* x, void* out, long N, int H, int W, int C, void* stream);

// LayerNorm over the last dim (C), optional affine (bf16 w/b), then optional
// modulation y = y * (1 + scale) + shift with fp32 scale/shift taken from row
// (r / rows_per_mod) * ldmod of `shift` / `scale`.
int tfb_layernorm_modulate(const void* x, long ldx, void* out, long ldo, int rows, int C, float eps, const void* w,
                           const void* b, const float* shift, const float* scale, long ldmod, int rows_per_mod,
                           void* stream);

// In-place RMSNorm over C = H*D (weight bf16 [C]) followed by optional
// interleaved-pair RoPE with per-token cos/sin fp32 [rows, D/2].
// Processes `nmat` matrices that start `mat_stride` elements apart inside the
// same rows (e.g. the q and k parts of a fused qkv buffer); weights are
// w0 / w1 for matrix 0 / 1.
int tfb_rmsnorm_rope(void* x, long ldx, long mat_stride, int nmat, int rows, int H, int D, float eps,
                     const void* w0, const void* w1, const float* cos, const float* sin, void* stream);

// out = x + gate * y   (bf16 x,y,out; fp32 gate rows as in the GEMM epilogue; gate null == 1)
int tfb_gated_residual(const void* x, const void* y, void* out, int rows, int C, const float* gate, long ldg,
                       int rows_per_gate, void* stream);

// x[r, :] = softmax(scale * x[r, :]) in place over C columns (bf16, fp32 maths); C % 8 == 0, scale > 0.
int tfb_softmax_rows(void* x, long ldx, int rows, int C, float scale, void* stream);
// act(x[:, :d]) * x[:, d:]   with act = 0 silu, 1 gelu-tanh, 2 gelu-erf.   x: [rows, 2d] bf16
int tfb_act_mul(const void* x, void* out, int rows, int d, int act, void* stream);

// Classifier-free guidance + flow-matching Euler step in one pass (fp32 latents):
//   v = uncond + s * (cond - uncond);  x_out = x + v * dsigma;  optional v_out
// cond/uncond are bf16 or fp32 (pred_is_bf16).
int tfb_cfg_euler_step(const float* x, const void* cond, const void* uncond, int pred_is_bf16, float cfg_scale,
                       float dsigma, float* x_out, float* v_out, long n, void* stream);

// Per-row MXFP8 quantisation: e4m3 payload + UE8M0 scale per 32 elements.
//   x: bf16 [rows, C];  q: uint8 [rows, C];  sf: uint8 [rows, C/32] (row-major, tiled = 0) or the tiled order
//   of tfb_gemm_mxfp8 (tiled = 1, C a multiple of 128, buffer of ceil(rows/128) * (C/128) * 512 bytes)
int tfb_quant_mxfp8(const void* x, long ldx, void* q, void* sf, int rows, int C, int tiled, void* stream);

// Block-scaled MXFP8 GEMM: out[M,N] = resid + gate * act(deq(A) @ deq(B)^T + bias), A [M,K] / B [N,K] e4m3 bytes
// (row strides lda / ldb in bytes, K a multiple of 128), sfa / sfb their UE8M0 scales per 32 K-elements in 512-byte
// tiles: rows [128*i, +128) x k-blocks [4*j, +4) at ((i * K/128) + j) * 512, row r / block b at
// (r%32)*16 + (r/32)*4 + b. The scale buffers cover whole 128-row tiles. Epilogue arguments as tfb_gemm_bf16.
int tfb_gemm_mxfp8(const void* A, int lda, const void* sfa, const void* B, int ldb, const void* sfb, void* out,
                   int ldo, int M, int N, int K, const void* bias, int epi, const void* resid, int ldr,
                   const float* gate, int ldg, int rows_per_gate, void* stream);
// NF4 codes (two per byte, first in the high nibble) with one fp32 absmax per `block` values -> bf16; numel % 16 == 0.
int tfb_nf4_dequant(const void* packed, const float* absmax, void* out, long numel, int block, void* stream);

// Grouped bf16 GEMM for expert layers. A: [M, K] token rows sorted by expert, each expert's segment
// starting on a multiple of 128 rows (M = padded row count, multiple of 128); B: [E*N, K]; M tile m
// uses expert tile_expert[m] (device int[M/128]; negative = skip the tile). N % 64 == 0.
int tfb_gemm_bf16_grouped(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N, int K,
                          int num_experts, const int* tile_expert, int epi, void* stream);

// ---- mixture-of-experts routing and token movement (moe.cu) ----
// logits fp32 [T, E] -> ids int32 [T, K], weights fp32 [T, K]; optional counts int32 [E] (zeroed here,
// then incremented once per selected (token, k)). Scores: sigmoid (use_softmax 0) or softmax over E.
// Selection uses score + bias (bias fp32 [E] or null), restricted to the `topk_groups` expert groups
// with the largest sum of their two best selection scores; weights are the unbiased scores of the
// selected experts, normalised to sum 1, times `scale`. E <= 1024, K <= 32, num_groups <= 32.
int tfb_moe_route(const float* logits, const float* bias, int T, int E, int num_groups, int topk_groups, int K,
                  float scale, int use_softmax, int* ids, float* weights, int* counts, void* stream);
// counts int32 [E] -> offsets int32 [E+1] (segment starts, multiples of `align`; offsets[E] = padded
// total) and tile_expert int32 [max_tiles] (owner of rows [m*align, (m+1)*align) or -1).
int tfb_moe_plan(const int* counts, int E, int align, int* offsets, int* tile_expert, int max_tiles, void* stream);
// x bf16 [T, hidden] -> x_perm bf16 [padded rows, hidden] in expert order; row_map int32 [T*K] gives
// the row of each (token, k). `cursor` is int32 [E] scratch owned by the caller (zeroed here).
int tfb_moe_permute(const void* x, int hidden, const int* ids, const int* offsets, int* cursor, int E, long T, int K,
                    void* x_perm, int* row_map, void* stream);
// Same operation as tfb_moe_permute, for callers that must not allocate: it takes no scratch buffer
// and calls no allocating routine. This entry point has no counterpart in the reference; it is an
// addition of this library. The per-expert cursor lives in a fixed device array of 1024 ints (4 KB)
// per device, so E <= 1024; a larger E is rejected with TFB_ERR_TOO_LARGE and a message on stderr
// (use tfb_moe_permute then). The first E cursors must be zero when the kernel starts; the call
// clears them itself with an asynchronous memset on `stream` before the kernel.
// The scratch is shared by every call on a device: two calls that overlap in time (different streams
// or host threads, same device) race on it and must be serialised by the caller. The first call on
// each device looks up the array's address (one-time set-up); make that first call before any
// stream capture begins.
int tfb_moe_permute_static(const void* x, int hidden, const int* ids, const int* offsets, int E, long T, int K,
                           void* x_perm, int* row_map, void* stream);
// out[t] = residual[t] (or 0) + sum_k weights[t,k] * y[row_map[t*K+k]]   (bf16, fp32 accumulate)
int tfb_moe_combine(const void* y, int hidden, const int* row_map, const float* weights, int T, int K,
                    const void* residual, void* out, void* stream);

// ---- W8A8 FP8 linear: per-token activation scales x per-output-channel weight scales ----
// out bf16 [M, N] = epilogue((A e4m3 [M,K] @ B e4m3 [N,K]^T) * a_scale[m] * b_scale[n]); same epilogue
// options as tfb_gemm_bf16 (bias, GELU, gate, residual). K % 16 == 0.
int tfb_gemm_fp8(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N, int K,
                 const float* a_scale, const float* b_scale, const void* bias, int epi, const void* resid, int ldr,
                 const float* gate, int ldg, int rows_per_gate, void* stream);
// x bf16 [rows, C] -> q e4m3 [rows, C] + scale fp32 [rows] (= max(amax/448, 1e-12)).
int tfb_quant_fp8_rowwise(const void* x, long ldx, void* q, long ldq, float* scale, int rows, int C, void* stream);
// The same GEMM on signed 8-bit integers (exact int32 accumulation): A int8 [M,K], B int8 [N,K].
int tfb_gemm_int8(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N, int K,
                  const float* a_scale, const float* b_scale, const void* bias, int epi, const void* resid, int ldr,
                  const float* gate, int ldg, int rows_per_gate, void* stream);
// x bf16 [rows, C] -> q int8 [rows, C] in [-127, 127] + scale fp32 [rows] (= max(amax/127, 1e-12)).
int tfb_quant_int8_rowwise(const void* x, long ldx, void* q, long ldq, float* scale, int rows, int C, void* stream);
// n contiguous bf16 values -> e4m3 with ONE scale (device float). is_static: read *scale (calibrated) instead of
// reducing the tensor's amax; otherwise *scale = max(amax/448, 1e-12) is written. scratch: one device word.
int tfb_quant_fp8_per_tensor(const void* x, void* q, float* scale, unsigned* scratch, long n, int is_static,
                             void* stream);

// ---- RMSNorm block glue of sandwich-norm DiTs (rms_ops.cu); norm weights and tables are fp32 ----
// out = (w * x * rstd) * (1 + scale) + shift; w / shift / scale may be null; table row = row / rows_per_mod.
int tfb_rmsnorm_modulate(const void* x, long ldx, void* out, long ldo, int rows, int C, float eps, const float* w,
                         const float* shift, const float* scale, long ldmod, int rows_per_mod, void* stream);
// out = res + g * (w * y * rstd), g = tanh(gate) if tanh_gate else gate (gate null: g = 1).
int tfb_rmsnorm_gate_residual(const void* y, long ldy, const void* res, long ldr, void* out, long ldo, int rows, int C,
                              float eps, const float* w, const float* gate, long ldg, int rows_per_gate,
                              int tanh_gate, void* stream);
// In place: per-head RMSNorm (weight fp32 [D], w0 for matrix 0, w1 for matrix 1) then interleaved-pair
// RoPE with per-token cos/sin fp32 [rows, D/2] (null: no rotation). D in {64, 128, 192, 256}.
int tfb_headnorm_rope(void* x, long ldx, long mat_stride, int nmat, long rows, int H, int D, float eps,
                      const float* w0, const float* w1, const float* cos, const float* sin, void* stream);

// ---- peer-mapped buffers (ipc.cu): allocate (zero-filled) + export a 64-byte IPC handle; map a peer's ----
int tfb_ipc_alloc(long bytes, void** ptr, void* handle64);
int tfb_ipc_open(const void* handle64, void** ptr);
int tfb_ipc_close(void* ptr);
int tfb_ipc_free(void* ptr);

// ---- peer-memory kernels over NVLink (peer_ops.cu, attn_tcgen05.cu); pointer tables are HOST arrays ----
// All-rank barrier on flag arrays in peer-mapped memory: flags[r] = rank r's int[slots*8], zero at start;
// `epoch` must grow by one per call on a slot (same sequence on every rank). The wait is bounded (4 s);
// on expiry the status word is set and the kernel returns.
int tfb_peer_barrier(void* const* flags, int my_rank, int n, int slot, int epoch, void* stream);
// Sequence-sharded q/k/v [B, S_loc, H, D] (strides lds/bss in elements) -> head-sharded slabs
// [B, S_loc*P, H/P, D] of every rank, written with peer stores. dsts[t*P + r] = rank r's slab of tensor t.
int tfb_ulysses_scatter(void* const* srcs, const long* lds, const long* bss, void* const* dsts, int ntensors, int B,
                        int S_loc, int H, int D, int P, int my_rank, void* stream);
// rows [row0, row0+rows) of every rank's buffer dsts[r] <- src (byte strides; row bytes % 16 == 0).
int tfb_peer_push_rows(const void* src, long ld_bytes, void* const* dsts, int P, long row0, long rows,
                       int row_bytes, long dst_ld_bytes, void* stream);
// GEMM -> reduce-scatter: epilogue tiles of row segment s go to rank s's slab buffer peer_out[s]
// ([n_seg, seg_rows, ldo] bf16) at slab `rank`; every rank then sums its slabs with tfb_slab_reduce.
int tfb_gemm_bf16_rs(const void* A, int lda, const void* B, int ldb, void* const* peer_out, int ldo, int n_seg,
                     int rank, int seg_rows, int N, int K, const void* bias, void* stream);
// all-gather -> GEMM: n_copiers CTAs pull the row shards peer_a[s] ([seg_rows, K] contiguous) into the local
// a_gather while the other CTAs multiply the shards that have landed. sync: 16 ints of local scratch.
int tfb_gemm_bf16_ag(void* const* peer_a, void* a_gather, int* sync, int n_copiers, const void* B, int ldb, void* out,
                     int ldo, int n_seg, int rank, int seg_rows, int N, int K, const void* bias, int epi, void* stream);
// out row r = resid[r] + gate[(gate_row0 + r) / rows_per_gate] * (sum_p slabs[p][r] + bias) at row dst_row0 + r of
// each of the n_dst destinations (1: local result of a reduce-scatter; P peers: all-reduce).
int tfb_slab_reduce(const void* slabs, int P, long rows, int N, long ld, const void* bias, const void* resid, long ldr,
                    const float* gate, long ldg, int rows_per_gate, long gate_row0, void* const* dsts, int n_dst,
                    long ldd, long dst_row0, void* stream);
// Attention over this rank's head slice whose epilogue stores each output row into the buffer of the
// rank that owns the token (see attn_host.cu).
int tfb_attn_fwd_peer(const void* q, long ldq, long bsq, const void* k, long ldk, long bsk, const void* v, long ldv,
                      long bsv, void* const* peer_out, int n_peers, int rows_per_rank, int head_off, long ldo, long bso,
                      int B, int H, int Sq, int Skv, float scale, int variant, void* stream);

// ---- expert parallelism over peer-mapped memory (moe.cu); rank o owns experts [o*E/P, (o+1)*E/P) ----
// counts_all int32 [P, E] (row s = histogram of rank s) -> dst_base int32 [E] (first row of this rank's
// tokens of expert e inside the owner's receive buffer) and tile_expert int32 [max_tiles] (local expert
// id per 128-row tile of THIS rank's receive buffer, -1 past the end).
int tfb_moe_ep_plan(const int* counts_all, int P, int E, int my_rank, int align, int* dst_base, int* tile_expert,
                    int max_tiles, void* stream);
// Token rows -> the owners' receive buffers by peer stores; row_map[t*K+k] = (owner << 26) | row.
int tfb_moe_ep_dispatch(const void* x, int hidden, const int* ids, const int* dst_base, int* cursor, int E, int P,
                        long T, int K, void* const* recv, int* row_map, void* stream);
// out[t] = residual[t] (or 0) + sum_k weights[t,k] * ybuf[owner][row]   (peer loads, fp32 accumulate)
int tfb_moe_ep_combine(void* const* ybuf, int P, int hidden, const int* row_map, const float* weights, int T, int K,
                       const void* residual, void* out, void* stream);

// ---- streaming / caching kernels (stream_ops.cu) ----
// Rolling KV cache [B, kv_size, row_elems] bf16 (batch stride cache_bs elements): optional left shift
// of `keep` tokens by `evicted` positions starting at token `sink` + `evicted`, then append of n_new
// tokens at local_start from new_k/new_v (token stride new_ld, batch stride new_bs elements).
int tfb_kv_cache_roll_append(void* k_cache, void* v_cache, long cache_bs, const void* new_k, const void* new_v,
                             long new_ld, long new_bs, int B, int row_elems, int sink, int evicted, int keep,
                             int local_start, int n_new, void* stream);
// x bf16 [rows, D] -> q e4m3 [rows, D], scale fp32 [rows] = max(amax/448, 1e-12).  D in {32..256}, D % 32 == 0.
int tfb_fp8_kv_quant(const void* x, void* q, float* scale, long rows, int D, void* stream);
// Log-sum-exp merge of two partial attention results (o* bf16 [B,S,H,D], lse* fp32 [B,H,S]).
int tfb_merge_attn_states(const void* o1, const float* lse1, const void* o2, const float* lse2, void* out,
                          float* lse_out, int B, int S, int H, int D, void* stream);
// Taylor feature cache on bf16 buffers of n elements (n % 8 == 0), terms t0..t3:
//   update (in place): t0 <- out - ori; t[i+1] <- (new t[i] - old t[i]) / window for i+1 < n_new, i < n_old
//   apply: y = x + sum_{i<nterms} t[i] * c[i]
int tfb_taylor_update(const void* out, const void* ori, void* t0, void* t1, void* t2, void* t3, int n_old, int n_new,
                      float window, long n, void* stream);
int tfb_taylor_apply(const void* x, const void* t0, const void* t1, const void* t2, const void* t3, float c0, float c1,
                     float c2, float c3, int nterms, void* y, long n, void* stream);
// Pluecker ray maps folded to the latent grid: c2w fp32 [F,4,4], ks fp32 [F,4] (fx,fy,cx,cy), optional
// extra fp32 [F,n_extra] per-frame channels -> out fp32 [C*c1*c2, F, h, w], C = (only_d ? 3 : 6) + n_extra.
int tfb_plucker_fold(const float* c2w, const float* ks, const float* extra, int n_extra, float* out, int F, int h,
                     int w, int c1, int c2, int only_d, void* stream);
// frames [3, T, H, W] (fp32 or bf16) in [-1, 1] -> uint8 [T, H, W, 3].  W % 4 == 0.
int tfb_frames_to_u8(const void* frames, int is_bf16, void* out, int T, int H, int W, void* stream);

#ifdef __cplusplus
}
#endif
