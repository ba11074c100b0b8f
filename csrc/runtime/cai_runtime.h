/* cai_runtime.h - C ABI of the device runtime (part of libcai_kernels.so).
 *
 * An executor owns six CUDA streams, an event pool and the parsed version-2 plan of one rank;
 * the arena it runs in is allocated by the caller (one allocation, carved by the plan). */
#ifndef CAI_RUNTIME_H
#define CAI_RUNTIME_H

#include <stddef.h>
#include <stdint.h>

#include "../kernels/cai_kernels.h"

#ifdef __cplusplus
namespace cai {
struct ExecOp;
struct NcclId { char bytes[128]; };
}  // namespace cai
struct cai_exec;
typedef int (*cai_fused_hook_t)(void* ctx, cai_exec* ex, const cai::ExecOp* op, int stream_id, void* cuda_stream);
#else
typedef struct cai_exec cai_exec;
typedef int (*cai_fused_hook_t)(void* ctx, cai_exec* ex, const void* op, int stream_id, void* cuda_stream);
#endif

typedef struct {
    uint32_t op_index;
    uint16_t kind;
    uint16_t stream;
    double start_s;
    double end_s;
    uint64_t bytes;
    uint64_t flops;
} cai_exec_trace_rec;

/* caller_streams: NULL, or six CUDA stream handles (NULL entries are created and owned by the executor). */
CAI_API int cai_exec_create(cai_exec** out, const void* plan_bytes, size_t nbytes, void* arena_base,
                            void* const* caller_streams);
CAI_API void cai_exec_destroy(cai_exec* ex);
CAI_API int cai_nccl_unique_id(const char* libpath, void* id128);
CAI_API int cai_exec_init_comm(cai_exec* ex, const char* libpath, int group_kind, const void* id128,
                               const void* id128_second, int nranks, int rank);
CAI_API int cai_exec_set_peers(cai_exec* ex, int group_kind, int n, void* const* bases, int rank);
CAI_API void cai_exec_set_ag_copy_ctas(cai_exec* ex, int n);
CAI_API int cai_ipc_export(void* ptr, void* handle64, unsigned long long* offset);
CAI_API int cai_ipc_open(const void* handle64, unsigned long long offset, void** out);
CAI_API int cai_ipc_close(void* mapped, unsigned long long offset);
CAI_API void* cai_exec_stream(cai_exec* ex, int stream_id);
CAI_API void* cai_exec_tensor_ptr(cai_exec* ex, int tensor);
CAI_API long long cai_exec_tensor_ld(cai_exec* ex, int tensor);
CAI_API unsigned long long cai_exec_tensor_bytes(cai_exec* ex, int tensor);
CAI_API int cai_exec_group_rank(cai_exec* ex, int kind);
CAI_API int cai_exec_group_size(cai_exec* ex, int kind);
CAI_API unsigned long long cai_exec_launches(cai_exec* ex);
CAI_API void cai_exec_set_fused_hook(cai_exec* ex, cai_fused_hook_t hook, void* ctx);
CAI_API void cai_exec_set_sm_limit(cai_exec* ex, int sms);
CAI_API float* cai_exec_hyper(cai_exec* ex);
CAI_API int cai_exec_step(cai_exec* ex, int step, float lr);
CAI_API int cai_exec_sync(cai_exec* ex);
CAI_API int cai_exec_use_graph(cai_exec* ex, int on);
CAI_API int cai_exec_trace_enable(cai_exec* ex, int on);
/* One NVTX range per op, named by its kernel, around the launches of a replay (stream replays only; a captured
 * graph keeps the ranges of the capture). */
CAI_API int cai_exec_nvtx_enable(cai_exec* ex, int on);
CAI_API int cai_exec_trace_read(cai_exec* ex, cai_exec_trace_rec* out, int cap);
/* Debug mode (also CAI_DEBUG_BOUNDS=1 in the environment): before each launch of a replay, the extent every operand
 * needs (from the record's rows / columns / pitch) is checked against the plan's tensor table; a mismatch fails the
 * step with the op's index instead of letting a kernel write past its tensor. */
CAI_API int cai_exec_set_debug(cai_exec* ex, int on);

#endif /* CAI_RUNTIME_H */
