// Host utilities: tensor maps via the driver entry point, SM count, status word.
#include "tfb_host.h"

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

int sm_count() {
  static int cached[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

int* status_word() {
  static int* words[16] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
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
  return v;
}

extern "C" int tfb_sm_count() { return tfb::sm_count(); }

extern "C" int tfb_abi_version() { return 1; }
