// Host-side helpers shared by all translation units of the native library: tensor-map (TMA
// descriptor) encoding through the driver entry point, the per-device status word that bounded
// waits report into, and device properties.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define PT_API extern "C" __attribute__((visibility("default")))

namespace pt {

// Status word (device memory, one per device) that kernels write on a bounded-wait timeout.
int* device_status_word();
// Number of SMs of the current device (cached).
int sm_count();

enum TmDtype { TM_BF16 = 0, TM_F32 = 1, TM_U8 = 2, TM_F16 = 3, TM_I32 = 4 };
enum TmSwizzle { TM_SW_NONE = 0, TM_SW_32 = 1, TM_SW_64 = 2, TM_SW_128 = 3 };

// Encode a 2-D tiled tensor map over a row-major [rows, cols] tensor whose row pitch is
// `ld_elems` elements; box = [box_rows, box_cols]. Returns 0 on success.
int encode_tmap_2d(CUtensorMap* out, const void* base, TmDtype dt, uint64_t rows, uint64_t cols,
                   uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols, TmSwizzle sw);
// 3-D variant: [d2, rows, cols] with pitches ld_elems (rows) and ld2_elems (d2).
int encode_tmap_3d(CUtensorMap* out, const void* base, TmDtype dt, uint64_t d2, uint64_t rows,
                   uint64_t cols, uint64_t ld_elems, uint64_t ld2_elems, uint32_t box_d2,
                   uint32_t box_rows, uint32_t box_cols, TmSwizzle sw);

}  // namespace pt
