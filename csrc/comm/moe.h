// moe.h - launchers of the expert-parallel exchange kernels (moe.cu): internal C++ forms used by the
// executor, and C forms that take the member arena bases as an array (tests, other runtimes).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../kernels/cai_kernels.h"

namespace cai {
struct PeerTable;
}

int cai_moe_dispatch(const cai::PeerTable& pt, const void* rows, const int* idx, const int* pos, const float* scale,
                     const int* counts, unsigned long long slab_off, unsigned long long cnt_off, int T, int H, int k, int E,
                     int cap, const uint32_t* epoch_base, uint32_t seq, unsigned int* done_counter, cudaStream_t st);
int cai_moe_combine(const cai::PeerTable& pt, const void* base, void* out, const int* idx, const int* pos, const float* w,
                    unsigned long long slab_off, const void* dot_with, float* dw, int T, int H, int k, int E, int cap,
                    int announce, const uint32_t* epoch_base, uint32_t seq, cudaStream_t st);

/* Router: softmax over E experts, top-k, weights renormalised over the chosen k. logits f32 [T,E];
 * idx/pos int32 [T,k], w f32 [T,k]; counts int32 [E] is zeroed, then holds how many tokens chose
 * each expert; pos is the token's slot in the expert's slab, -1 when the slab (cap rows) is full. */
CAI_API int cai_moe_route_fwd(const float* logits, int* idx, float* w, int* pos, int* counts, int T, int E, int k, int cap,
                              void* stream);
CAI_API int cai_moe_route_bwd(const float* logits, const int* idx, const float* dw, const int* pos, void* dlogits, int T, int E,
                              int k, void* stream);
/* Size of the signal block (epoch counters) that every member arena carries at sig_off. */
CAI_API unsigned long long cai_signal_block_bytes(void);
/* Exchange kernels with explicit member bases (bases[rank] is the local arena). sig_off is the
 * arena offset of the signal block, epoch_base a device word, scratch a zeroed device uint32. */
CAI_API int cai_moe_dispatch_c(void* const* bases, int rank, int size, unsigned long long sig_off, const void* rows,
                               const int* idx, const int* pos, const float* scale, const int* counts,
                               unsigned long long slab_off, unsigned long long cnt_off, int T, int H, int k, int E, int cap,
                               const uint32_t* epoch_base, uint32_t seq, unsigned int* scratch, void* stream);
CAI_API int cai_moe_combine_c(void* const* bases, int rank, int size, unsigned long long sig_off, const void* base, void* out,
                              const int* idx, const int* pos, const float* w, unsigned long long slab_off, const void* dot_with,
                              float* dw, int T, int H, int k, int E, int cap, int announce, const uint32_t* epoch_base,
                              uint32_t seq, void* stream);
