// Host utilities: tensor maps via the driver entry point, SM count, status word.
#include "tfb_host.h"

#include <atomic>
#include <mutex>

#include "tfb_common.cuh"

namespace tfb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap(CUtensorMap* out, const void* base, int dtype, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, int swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return TFB_ERR_NO_DRIVER;
  CUtensorMapDataType dt;
  switch (dtype) {
    case TM_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case TM_U8: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    case TM_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    case TM_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    default: return TFB_ERR_TMAP;
  }
  CUtensorMapSwizzle sw;
  switch (swizzle) {
    case TM_SW_NONE: sw = CU_TENSOR_MAP_SWIZZLE_NONE; break;
    case TM_SW_32: sw = CU_TENSOR_MAP_SWIZZLE_32B; break;
    case TM_SW_64: sw = CU_TENSOR_MAP_SWIZZLE_64B; break;
    default: sw = CU_TENSOR_MAP_SWIZZLE_128B; break;
  }
  cuuint64_t gdims[5];
  cuuint64_t gstr[5];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  CUresult r = fn(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstr, gbox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TFB_OK : TFB_ERR_TMAP;
}

int device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= TFB_MAX_DEVICES) return -1;
  return dev;
}

int ensure_dynamic_smem(const void* func, int bytes, bool* done_per_device) {
  const int dev = device_slot();
  if (dev < 0) return TFB_ERR_TOO_LARGE;
  if (!done_per_device[dev]) {
    if (cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
      return TFB_ERR_LAUNCH;
    done_per_device[dev] = true;
  }
  return TFB_OK;
}

int sm_count() {
  static int cached[TFB_MAX_DEVICES] = {0};
  int dev = device_slot();
  if (dev < 0) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

static std::atomic<unsigned long long> g_peer_wait_ns{4000000000ull};

unsigned long long peer_wait_ns() { return g_peer_wait_ns.load(std::memory_order_relaxed); }

// Pinned host copy of the status word per device: filled by stream-ordered copies (tfb_status_post) and read
// without touching the device (tfb_status_peek).
static volatile int* host_status_copy(int dev) {
  static int* copies[TFB_MAX_DEVICES] = {nullptr};
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  if (!copies[dev]) {
    int* p = nullptr;
    if (cudaHostAlloc(&p, sizeof(int), cudaHostAllocDefault) != cudaSuccess) return nullptr;
    *p = 0;
    copies[dev] = p;
  }
  return copies[dev];
}

int* status_word() {
  static int* words[TFB_MAX_DEVICES] = {nullptr};
  static std::mutex mu;
  const int dev = device_slot();
  if (dev < 0) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (!words[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(int));
    words[dev] = p;
  }
  return words[dev];
}

}  // namespace tfb

// Reads and clears the status word of the current device. Synchronises the
// device: call it from tests and error paths, not from a hot loop.
extern "C" int tfb_last_status() {
  int* p = tfb::status_word();
  if (!p) return tfb::TFB_ERR_LAUNCH;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return tfb::TFB_ERR_LAUNCH;
  if (v != 0) cudaMemset(p, 0, sizeof(int));
  const int dev = tfb::device_slot();
  volatile int* h = dev >= 0 ? tfb::host_status_copy(dev) : nullptr;
  if (h) *h = 0;
  return v;
}

// Enqueues a copy of the status word into pinned host memory on `stream` (no synchronisation). The value
// becomes visible to tfb_status_peek() once the stream has reached this point.
extern "C" int tfb_status_post(void* stream) {
  int* p = tfb::status_word();
  const int dev = tfb::device_slot();
  if (!p || dev < 0) return tfb::TFB_ERR_LAUNCH;
  volatile int* h = tfb::host_status_copy(dev);
  if (!h) return tfb::TFB_ERR_LAUNCH;
  return cudaMemcpyAsync(const_cast<int*>(h), p, sizeof(int), cudaMemcpyDeviceToHost,
                         static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? tfb::TFB_OK
             : tfb::TFB_ERR_LAUNCH;
}

// Last posted value of the status word of the current device; never blocks, never touches the device.
extern "C" int tfb_status_peek() {
  const int dev = tfb::device_slot();
  if (dev < 0) return 0;
  volatile int* h = tfb::host_status_copy(dev);
  return h ? *h : 0;
}

// Upper bound of every wait on a peer (flag barrier, gathered-segment wait), in milliseconds (100 .. 600000).
extern "C" int tfb_set_peer_wait_ms(int ms) {
  if (ms < 100 || ms > 600000) return tfb::TFB_ERR_BAD_SHAPE;
  tfb::g_peer_wait_ns.store(static_cast<unsigned long long>(ms) * 1000000ull, std::memory_order_relaxed);
  return tfb::TFB_OK;
}

extern "C" int tfb_sm_count() { return tfb::sm_count(); }

extern "C" int tfb_abi_version() { return 1; }
