// Kernels that move data between GPUs of one node through peer-mapped (symmetric) memory with plain
// loads and stores over NVLink: no collective library on the path, no intermediate pack / unpack
// buffers, plain per-CTA accesses only. Every wait on a peer is bounded by wall time and reports through the
// status word instead of spinning forever.
//   peer_barrier        : all ranks signal each other and wait (epoch counters, never reset)
//   ulysses_scatter     : sequence-sharded q/k/v -> head-sharded slabs of every peer in ONE pass
//   peer_push_rows      : this rank's row block -> the same rows of every peer's full buffer (all-gather)
// Role in the reference: the NCCL all-to-all / all-gather calls of telefuser/distributed/ulysses_comm.py:53-124 and
// telefuser/distributed/parallel_shard.py (sequence shard / unshard); there the collective library moves the data.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tfb_api.h"
#include "tfb_common.cuh"
#include "tfb_host.h"

namespace tfb {

constexpr int PEER_MAX = 8;

struct PeerPtrs {
  void* p[PEER_MAX];
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// flags[r] is rank r's flag array (int[PEER_MAX] per slot). Thread t < n: tells rank t that this
// rank reached `epoch`, then waits until rank t told us the same.
__global__ void peer_barrier_kernel(PeerPtrs flags, int my_rank, int n, int slot, int epoch, int* status,
                                    unsigned long long wait_ns) {
  const int t = threadIdx.x;
  if (t < n) {
    __threadfence_system();
    st_release_sys(static_cast<int*>(flags.p[t]) + slot * PEER_MAX + my_rank, epoch);
    const int* mine = static_cast<const int*>(flags.p[my_rank]) + slot * PEER_MAX + t;
    const unsigned long long t0 = globaltimer_ns();
    while (ld_acquire_sys(mine) < epoch) {
      if (globaltimer_ns() - t0 > wait_ns) {
        if (status) atomicCAS(status, 0, TFB_ERR_TIMEOUT | (60 << 8));
        break;
      }
      __nanosleep(200);
    }
    __threadfence_system();
  }
}

// src tensors: [B, S_loc, H, D] bf16 (token stride ld, batch stride bs, D contiguous, heads adjacent).
// dst of rank r: [B, S_loc * P, H / P, D] contiguous. blockIdx.y selects the tensor (q, k, v).
struct ScatterArgs {
  const uint4* src[3];
  PeerPtrs dst[3];
  long ld_vec[3], bs_vec[3];
};

__global__ void ulysses_scatter_kernel(ScatterArgs a, int B, int S_loc, int H, int dvec, int P, int my_rank) {
  const int which = blockIdx.y;
  const uint4* __restrict__ src = a.src[which];
  const long ld = a.ld_vec[which], bs = a.bs_vec[which];
  const int Hp = H / P;
  const long row_vecs = static_cast<long>(H) * dvec;
  const long total = static_cast<long>(B) * S_loc * row_vecs;
  const long S_tot = static_cast<long>(S_loc) * P;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % row_vecs);  // (h, vec) inside the token row
    const long bs_i = i / row_vecs;
    const int s = static_cast<int>(bs_i % S_loc);
    const int b = static_cast<int>(bs_i / S_loc);
    const int h = c / dvec;
    const int r = h / Hp;
    const uint4 v = src[b * bs + static_cast<long>(s) * ld + c];
    uint4* dst = static_cast<uint4*>(a.dst[which].p[r]);
    dst[((b * S_tot + static_cast<long>(my_rank) * S_loc + s) * Hp) * dvec + (c - r * Hp * dvec)] = v;
  }
}

// Every rank's buffer: [rows_total, row_vecs]; this rank owns rows [row0, row0 + rows).
__global__ void peer_push_rows_kernel(const uint4* __restrict__ src, long ld_vec, PeerPtrs dst, int P, long row0,
                                      long rows, int row_vecs, long dst_ld_vec) {
  const long total = rows * row_vecs;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / row_vecs;
    const int c = static_cast<int>(i - r * row_vecs);
    const uint4 v = src[r * ld_vec + c];
    for (int p = 0; p < P; ++p) static_cast<uint4*>(dst.p[p])[(row0 + r) * dst_ld_vec + c] = v;
  }
}

// Second half of GEMM -> reduce-scatter / all-reduce: sums the P partial slabs that the GEMM epilogues of
// all ranks stored into this rank's buffer (fp32 accumulation), applies bias / gate / residual once, and
// writes the rows to n_dst destinations (1 = local reduce-scatter result, P = every peer's full output).
struct SlabReduceArgs {
  const uint4* slabs;  // [P, rows, ld_vec]
  long ld_vec, slab_vecs;
  const __nv_bfloat16* bias;
  const uint4* resid;
  long ldr_vec;
  const float* gate;  // row r reads gate[((gate_row0 + r) / rows_per_gate) * ldg + col]
  long ldg;
  long gate_row0;
  int rows_per_gate;
  PeerPtrs dst;
  int n_dst;
  long ldd_vec, dst_row0;
};

__global__ void slab_reduce_kernel(SlabReduceArgs a, int P, long rows, int row_vecs) {
  const long total = rows * row_vecs;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / row_vecs;
    const int c = static_cast<int>(i - r * row_vecs);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < P; ++p) {
      const uint4 v = a.slabs[p * a.slab_vecs + r * a.ld_vec + c];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] += bf16_lo(w[e]);
        acc[2 * e + 1] += bf16_hi(w[e]);
      }
    }
    if (a.bias) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += __bfloat162float(a.bias[c * 8 + e]);
    }
    if (a.gate) {
      const float* g = a.gate + ((a.gate_row0 + r) / a.rows_per_gate) * a.ldg + c * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] *= g[e];
    }
    if (a.resid) {
      const uint4 v = a.resid[r * a.ldr_vec + c];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] += bf16_lo(w[e]);
        acc[2 * e + 1] += bf16_hi(w[e]);
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    for (int d = 0; d < a.n_dst; ++d) static_cast<uint4*>(a.dst.p[d])[(a.dst_row0 + r) * a.ldd_vec + c] = o;
  }
}

static inline int peer_grid(long items, int per_block = 256, int max_blocks = 148 * 8) {
  long b = (items + per_block - 1) / per_block;
  return static_cast<int>(b < 1 ? 1 : (b > max_blocks ? max_blocks : b));
}

}  // namespace tfb

using namespace tfb;

// flags: HOST array of n device pointers, entry r = rank r's flag array (int[slots * 8], zero at start).
extern "C" int tfb_peer_barrier(void* const* flags, int my_rank, int n, int slot, int epoch, void* stream) {
  if (n < 1 || n > PEER_MAX || my_rank < 0 || my_rank >= n || slot < 0 || epoch < 1) return TFB_ERR_BAD_SHAPE;
  PeerPtrs f;
  for (int i = 0; i < PEER_MAX; ++i) f.p[i] = i < n ? flags[i] : nullptr;
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, my_rank, n, slot, epoch, status_word(),
                                                                       peer_wait_ns());
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

// srcs / lds / bss: 3 entries (q, k, v); dsts: HOST array of 3 * P device pointers, dsts[t * P + r] = rank r's
// slab for tensor t. ntensors in 1..3.
extern "C" int tfb_ulysses_scatter(void* const* srcs, const long* lds, const long* bss, void* const* dsts, int ntensors,
                                   int B, int S_loc, int H, int D, int P, int my_rank, void* stream) {
  if (ntensors < 1 || ntensors > 3 || P < 1 || P > PEER_MAX || H % P || D % 8 || B < 1 || S_loc < 1)
    return TFB_ERR_BAD_SHAPE;
  ScatterArgs a;
  for (int t = 0; t < 3; ++t) {
    const int u = t < ntensors ? t : 0;
    if (lds[u] % 8 || bss[u] % 8 || (reinterpret_cast<uintptr_t>(srcs[u]) & 15)) return TFB_ERR_BAD_SHAPE;
    a.src[t] = static_cast<const uint4*>(srcs[u]);
    a.ld_vec[t] = lds[u] / 8;
    a.bs_vec[t] = bss[u] / 8;
    for (int r = 0; r < PEER_MAX; ++r) a.dst[t].p[r] = r < P ? dsts[u * P + r] : nullptr;
  }
  const long total = static_cast<long>(B) * S_loc * H * (D / 8);
  dim3 grid(peer_grid(total), ntensors);
  ulysses_scatter_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a, B, S_loc, H, D / 8, P, my_rank);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

extern "C" int tfb_peer_push_rows(const void* src, long ld, void* const* dsts, int P, long row0, long rows,
                                  int row_elems_bytes, long dst_ld_bytes, void* stream) {
  if (P < 1 || P > PEER_MAX || rows < 0 || row_elems_bytes % 16 || dst_ld_bytes % 16 || ld % 16) return TFB_ERR_BAD_SHAPE;
  if (rows == 0) return TFB_OK;
  PeerPtrs d;
  for (int r = 0; r < PEER_MAX; ++r) d.p[r] = r < P ? dsts[r] : nullptr;
  peer_push_rows_kernel<<<peer_grid(rows * (row_elems_bytes / 16)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), ld / 16, d, P, row0, rows, row_elems_bytes / 16, dst_ld_bytes / 16);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

// slabs: local bf16 [P, rows, ld]; out row r = resid[r] + gate[(gate_row0 + r) / rows_per_gate] * (sum_p slabs[p][r] + bias),
// stored at row dst_row0 + r of each of the n_dst destinations (HOST array of device pointers, leading dim ldd).
extern "C" int tfb_slab_reduce(const void* slabs, int P, long rows, int N, long ld, const void* bias, const void* resid,
                               long ldr, const float* gate, long ldg, int rows_per_gate, long gate_row0,
                               void* const* dsts, int n_dst, long ldd, long dst_row0, void* stream) {
  if (P < 1 || P > PEER_MAX || n_dst < 1 || n_dst > PEER_MAX || rows < 0 || N % 8 || ld % 8 || ldd % 8) return TFB_ERR_BAD_SHAPE;
  if (resid && ldr % 8) return TFB_ERR_BAD_SHAPE;
  if (gate && (ldg % 4 || rows_per_gate < 1)) return TFB_ERR_BAD_SHAPE;
  if (rows == 0) return TFB_OK;
  SlabReduceArgs a;
  a.slabs = static_cast<const uint4*>(slabs);
  a.ld_vec = ld / 8;
  a.slab_vecs = rows * (ld / 8);
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.resid = static_cast<const uint4*>(resid);
  a.ldr_vec = ldr / 8;
  a.gate = gate;
  a.ldg = ldg;
  a.gate_row0 = gate_row0;
  a.rows_per_gate = rows_per_gate > 0 ? rows_per_gate : 1;
  for (int r = 0; r < PEER_MAX; ++r) a.dst.p[r] = r < n_dst ? dsts[r] : nullptr;
  a.n_dst = n_dst;
  a.ldd_vec = ldd / 8;
  a.dst_row0 = dst_row0;
  slab_reduce_kernel<<<peer_grid(rows * (N / 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(a, P, rows, N / 8);
  return cudaGetLastError() == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}
