/* rmsnorm_bwd_static.h - RMSNorm backward for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference project; it exists for users of this
 * library whose own constraints rule out device allocation at the call site: runtimes that hand a
 * fixed memory budget to each component at start-up and forbid cudaMalloc afterwards, latency-bound
 * loops in which an allocator call (and the synchronisation it can imply) is not acceptable, and
 * plug-ins loaded into a host process whose allocator they may not call into. cai_rmsnorm_bwd() needs a caller-provided scratch
 * buffer for the per-CTA partial sums of the gain gradient; here that scratch lives in a
 * fixed-size array inside the library image instead, so the call itself allocates nothing.
 *
 * Limits and rules:
 *  - H <= CAI_RMSNORM_STATIC_MAX_H (and a multiple of 8); larger H is rejected with an error
 *    (return value < 0, text in cai_last_error()). Any number of rows is accepted.
 *  - The scratch array (CAI_RMSNORM_STATIC_PARTS x CAI_RMSNORM_STATIC_MAX_H floats, 4 MiB) is
 *    held by every GPU that loads the library until the process exits.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress) once;
 *    make that first call before any stream capture starts on that device.
 *  - All calls share the one array. It keeps whatever the previous call left in it; every call
 *    overwrites the part it reads before reading it, so nothing needs clearing, but two calls
 *    that overlap on the GPU (different streams) race on it. Serialise them.
 *  - The same kernels run as in cai_rmsnorm_bwd(); only the number of partial rows, and with it
 *    the summation order of dg, can differ, so results agree to rounding, not bit for bit. */
#ifndef CAI_RMSNORM_BWD_STATIC_H
#define CAI_RMSNORM_BWD_STATIC_H

#include "cai_kernels.h"

#define CAI_RMSNORM_STATIC_MAX_H 4096
#define CAI_RMSNORM_STATIC_PARTS 256

/* dx (+)= d(rmsnorm)/dx * dy and dg (+)= sum over rows, like cai_rmsnorm_bwd(), without a scratch
 * argument and without any allocation. x, dy, dx are bf16 [rows, H]; g is bf16 [H]; rstd is f32
 * [rows] as saved by cai_rmsnorm_fwd(); dg is f32 [H]. */
CAI_API int cai_rmsnorm_bwd_static(const void* x, const void* g, const float* rstd, const void* dy, void* dx, float* dg,
                                   int rows, int H, int dx_accumulate, int dg_accumulate, void* stream);

#endif /* CAI_RMSNORM_BWD_STATIC_H */
