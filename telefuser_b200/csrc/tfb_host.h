// Host-side helpers shared by the launchers: tensor-map construction through
// the driver entry point (no link-time dependency on libcuda), SM count cache,
// and the per-launch status buffer.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tfb {

// Element kinds for tensor maps.
enum TmapDtype : int { TM_BF16 = 0, TM_U8 = 1, TM_F32 = 2, TM_F16 = 3 };
// Swizzle kinds.
enum TmapSwizzle : int { TM_SW_NONE = 0, TM_SW_32 = 1, TM_SW_64 = 2, TM_SW_128 = 3 };

// Builds a tiled tensor map over a row-major tensor of `rank` dims.
// dims[0] is the innermost (contiguous) extent; strides_bytes[i] is the byte
// stride of dim i+1 (rank-1 entries). box[i] is the tile extent per dim.
// Returns 0 on success, a TFB_ERR_* code otherwise.
int make_tmap(CUtensorMap* out, const void* base, int dtype, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, int swizzle);

// Per-device tables in the launchers have this many entries; a device ordinal beyond it is refused.
constexpr int TFB_MAX_DEVICES = 64;
// Current device ordinal, or -1 when it does not fit the per-device tables.
int device_slot();
// Raises a kernel's dynamic shared-memory limit once per device; `done_per_device` has TFB_MAX_DEVICES entries.
int ensure_dynamic_smem(const void* func, int bytes, bool* done_per_device);

int sm_count();

// Limit of a wait on another rank (set by tfb_set_peer_wait_ms, 4 s by default).
unsigned long long peer_wait_ns();

// Device int used by kernels to report bounded-wait expiry. One per device,
// allocated on first use; reset by the launcher before each launch that uses
// it and read back by tfb_last_status().
int* status_word();

}  // namespace tfb
