// host_common.h - host-side helpers shared by the kernel launchers: the per-device status
// word that bounded waits report into, TMA tensor-map encoding through the driver entry point
// (no link-time dependency on libcuda), and cached device properties.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "cai_kernels.h"

namespace cai {

// Error codes returned by the extern "C" launchers (0 = ok, negative = host-side failure).
enum : int {
    CAI_K_OK = 0,
    CAI_K_BAD_ARG = -2,
    CAI_K_CUDA = -6,
};

// Device pointer to this device's status word block (64 ints, zero on creation). Allocated once
// per device on first use; kernels receive it as an argument.
int* status_words(int device);
int current_device();
int sm_count(int device);

// Encode a 2-D bf16 (or other 2-byte / 1-byte / 4-byte) row-major tensor map with a 128-byte
// swizzle. `cols` is the contiguous extent, `ld` the row pitch in elements.
// Returns false if the driver rejected the arguments (alignment, pitch).
bool encode_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                    uint32_t box_cols, uint32_t box_rows, int elem_bytes, bool swizzle128 = true);
// 3-D variant: dims (cols, rows, batch) with pitches in elements.
bool encode_tmap_3d(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t batch,
                    uint64_t ld_row, uint64_t ld_batch, uint32_t box_cols, uint32_t box_rows,
                    int elem_bytes);

const char* last_error();
void set_last_error(const char* fmt, ...);

}  // namespace cai
