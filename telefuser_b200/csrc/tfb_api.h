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
// Reads and clears the per-device status word written by bounded waits.
int tfb_last_status();

// out[M,N] = resid + gate * act(A[M,K] @ B[N,K]^T + bias)   (bf16 in/out, fp32 accumulate)
//   bias  : bf16 [N] or null
//   resid : bf16 [M, ldr] or null (may alias out)
//   gate  : fp32, row r uses gate[(r / rows_per_gate) * ldg + col], or null (== 1)
//   force_bn: 0 = auto, else 64/128/256 (N tile)
int tfb_gemm_bf16(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N, int K,
                  const void* bias, int epi, const void* resid, int ldr, const float* gate, int ldg,
                  int rows_per_gate, int force_bn, void* stream);

// Flash attention forward, bf16, head_dim 128 (tcgen05 + TMEM).
//   q   : [B, Sq, H, 128] with row stride ldq (elements between tokens), batch stride bsq
//   k,v : [B, Skv, H, 128] likewise
//   out : [B, Sq, H, 128] bf16, row stride ldo
//   lse : optional fp32 [B, H, Sq] (natural log), or null
//   variant: 0 = default
int tfb_attn_fwd(const void* q, long ldq, long bsq, const void* k, long ldk, long bsk, const void* v, long ldv,
                 long bsv, void* out, long ldo, long bso, float* lse, int B, int H, int Sq, int Skv, float scale,
                 int variant, void* stream);

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

// act(x[:, :d]) * x[:, d:]   with act = 0 silu, 1 gelu-tanh, 2 gelu-erf.   x: [rows, 2d] bf16
int tfb_act_mul(const void* x, void* out, int rows, int d, int act, void* stream);

// Classifier-free guidance + flow-matching Euler step in one pass (fp32 latents):
//   v = uncond + s * (cond - uncond);  x_out = x + v * dsigma;  optional v_out
// cond/uncond are bf16 or fp32 (pred_is_bf16).
int tfb_cfg_euler_step(const float* x, const void* cond, const void* uncond, int pred_is_bf16, float cfg_scale,
                       float dsigma, float* x_out, float* v_out, long n, void* stream);

// Per-row MXFP8 quantisation: e4m3 payload + UE8M0 scale per 32 elements.
//   x: bf16 [rows, C];  q: uint8 [rows, C];  sf: uint8 [rows, C/32] (row-major)
int tfb_quant_mxfp8(const void* x, long ldx, void* q, void* sf, int rows, int C, void* stream);

// Descriptor self-test: one CTA computes D[128,N] = A[128,K] @ B^T with the
// operand modes used by the attention kernel. mode 0: A,B K-major from smem;
// mode 1: B MN-major from smem (B given as [K,N]); mode 2: A from TMEM.
int tfb_umma_probe(const void* A, const void* B, float* D, int N, int K, int mode, void* stream);

#ifdef __cplusplus
}
#endif
