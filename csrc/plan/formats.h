// formats.h - binary layouts shared by the offline compiler and the runtimes.
//
// The on-disk layouts (topology.bin, plan.rankNNNNNN.bin) are byte-compatible with the
// reference project so that its configs produce identical files and hashes here
// (include/cai_tensor.h, include/cai_plan.h, include/cai_topology.h, src/cai_model.h:14-47 of the
// reference). Version 2 of the plan file appends an execution section (real tensors, kernel
// records) after the version-1 payload; a version-1 reader that ignores trailing bytes still sees
// a valid schedule.
#pragma once

#include <cstddef>
#include <cstdint>

namespace cai {

// ---- status codes (public API) -------------------------------------------------------
enum Status : int {
    OK = 0,
    ERR_IO = -1,
    ERR_INVALID = -2,
    ERR_OOM = -3,
    ERR_TOPOLOGY = -4,
    ERR_PLAN = -5,
    ERR_BACKEND = -6,
    ERR_DEPENDENCY = -7,
    ERR_BUDGET = -8,
};

// ---- element types / tensor classes --------------------------------------------------
enum DType : uint16_t { DT_FP32 = 0, DT_BF16, DT_FP16, DT_FP8_E4M3, DT_FP8_E5M2, DT_INT32, DT_UINT8, DT_COUNT };

enum TensorClass : uint16_t {
    TC_PARAM = 0,    // sharded weights, resident
    TC_GRAD,         // sharded gradients, resident
    TC_OPTSTATE,     // optimizer moments and fp32 master weights, resident
    TC_ACTIVATION,   // saved activations
    TC_COMM,         // staging for collectives / pipeline hand-off (symmetric memory on device)
    TC_WORKSPACE,    // reusable scratch
    TC_COUNT
};

struct TensorDesc {          // 24 bytes
    uint64_t offset;         // byte offset in the arena (class-local until relocated)
    uint64_t nbytes;
    uint32_t shape_id;
    uint16_t dtype;
    uint16_t tclass;
};
static_assert(sizeof(TensorDesc) == 24, "TensorDesc layout");

// ---- schedule ---------------------------------------------------------------------------
enum Stream : uint16_t { ST_COMPUTE_HI = 0, ST_COMPUTE_LO, ST_COMM_TP, ST_COMM_PP, ST_COMM_DP, ST_IO, ST_COUNT };

enum OpKind : uint16_t {
    OP_GEMM = 0,
    OP_ATTENTION_FWD,
    OP_ATTENTION_BWD,
    OP_RMSNORM,
    OP_SWIGLU,
    OP_ELEMENTWISE,
    OP_REDUCE_SCATTER,
    OP_ALL_GATHER,
    OP_ALL_REDUCE,
    OP_ALL_TO_ALL,
    OP_PIPE_SEND,
    OP_PIPE_RECV,
    OP_OPTIMIZER,
    OP_EVENT_RECORD,
    OP_EVENT_WAIT,
    OP_COUNT_V1,
    // ---- version-2 kinds: fused compute+collective ops, one kernel each
    OP_GEMM_RS = OP_COUNT_V1,  // row-parallel GEMM whose epilogue reduce-scatters over the TP group
    OP_AG_GEMM,                // all-gather of the sequence-sharded activation fused into a GEMM
    OP_RS_ADAMW,               // gradient reduce-scatter + scale + sharded AdamW
    OP_FSDP_AG_GEMM,           // parameter all-gather fused into the first consuming GEMM
    OP_MOE_DISPATCH_GEMM,      // token dispatch all-to-all + permute + expert up-projection
    OP_MOE_GEMM_COMBINE,       // expert down-projection + weighted combine all-to-all
    OP_COUNT
};

struct Op {                  // 32 bytes
    uint64_t flops;
    uint64_t bytes;
    uint32_t aux0;           // comm group id, or event id for record/wait
    uint32_t aux1;           // microbatch id
    uint16_t kind;
    uint16_t stream_id;
    uint32_t exec;           // v1: zero padding. v2: index+1 into the exec table (0 = none)
};
static_assert(sizeof(Op) == 32, "Op layout");

enum GroupKind : uint16_t { GROUP_TP = 0, GROUP_DP, GROUP_PP, GROUP_EP, GROUP_COUNT, GROUP_CP = GROUP_COUNT };

struct CommGroup {           // 16 bytes
    uint32_t group_id;
    uint16_t kind;
    uint16_t intra_rack;
    uint32_t size;
    uint32_t color;
};
static_assert(sizeof(CommGroup) == 16, "CommGroup layout");

constexpr uint32_t kPlanMagic = 0x50494143u;  // 'CAIP'
constexpr uint32_t kTopoMagic = 0x504F5443u;  // 'CTOP'
constexpr uint32_t kExecMagic = 0x58494143u;  // 'CAIX' - start of the version-2 execution section

struct PlanHeader {          // 128 bytes
    uint32_t magic;
    uint32_t version;
    uint64_t plan_hash;
    uint64_t topology_hash;
    uint32_t global_rank, world_size, pipeline_stage, num_stages;
    uint32_t tp, dp, ep, cp;
    uint32_t microbatch, grad_accum, num_microbatches, seq_len;
    uint32_t hidden_size, layers_in_stage, num_tensors, num_groups;
    uint32_t num_ops, num_events;
    uint64_t arena_bytes;
    uint64_t global_tokens_per_step;
    uint64_t flops_per_token_useful;
    uint32_t vpp;
    uint32_t reserved;
};
static_assert(sizeof(PlanHeader) == 128, "PlanHeader layout");

// ---- topology -------------------------------------------------------------------------
struct PhysId {              // 12 bytes
    uint32_t global_rank;
    uint16_t rack_id;
    uint8_t tray_id, gpu_in_tray, gpu_in_rack, nic_id, rail_id, reserved;
};
static_assert(sizeof(PhysId) == 12, "PhysId layout");

struct Topology {            // 64 bytes
    uint32_t gpus_per_rack, trays_per_rack, gpus_per_tray, num_racks;
    uint32_t world_size, spare_gpus;
    uint64_t intra_rack_bw, inter_rack_bw, hbm_bw;
    double gpu_flops_bf16;
    uint64_t gpu_mem_bytes;
};
static_assert(sizeof(Topology) == 64, "Topology layout");

// ---- model + parallelism spec (hashed into plan_hash; layout is part of the format) ----
struct ModelSpec {           // 96 bytes
    uint32_t hidden_size, ffn_hidden, num_layers, num_heads, num_kv_heads, head_dim, vocab_size, seq_len;
    int32_t is_moe;
    uint32_t num_experts, moe_top_k;
    uint16_t param_dtype, optim_dtype;
    uint32_t optim_states;
    int32_t master_weights, recompute;
    uint32_t tp, pp, ep, cp, vpp, microbatch, grad_accum;
    uint64_t mem_budget;
};
static_assert(sizeof(ModelSpec) == 96, "ModelSpec layout");

// Training hyper-parameters and execution options that the reference does not have. They are
// NOT part of plan_hash (so hashes stay comparable with the reference) but are stored in the
// version-2 execution section.
struct TrainSpec {
    float lr = 1e-3f, beta1 = 0.9f, beta2 = 0.999f, adam_eps = 1e-8f, weight_decay = 0.01f;
    float rope_theta = 10000.f, norm_eps = 1e-6f, init_std = 0.02f;
    uint32_t seed = 0;
    uint32_t tie_embeddings = 1;
    uint32_t zero_stage = 1;      // 1 = optimizer state sharded over dp (fused path), 2 = fp32 gradients sharded too, 3 = bf16 parameters sharded too
    uint32_t fp8_block = 128;
    uint32_t comm_mode = 1;       // 0 = NCCL-only baseline ops, 1 = fused compute+collective kernels
    uint32_t ce_chunk = 4096;     // rows of logits materialised at a time (the head's weight gradient is read-modify-written once per chunk)
    uint32_t moe_capacity_factor_x100 = 200;
    uint32_t wgrad_overlap = 1;   // tp > 1: weight-gradient GEMMs run on compute_lo next to the backward's critical path
    // Microbatches of a step are independent until the optimizer. With pp = 1 the schedule may launch `mb_group`
    // of them together (their sequences side by side in one activation set): the same tokens, loss and gradients
    // with 1/mb_group as many kernel launches and collective hand-shakes. 0 = chosen by the compiler (dense models
    // without a pipeline or parameter sharding: the largest power of two that divides grad_accum and keeps a launch
    // at or under 16384 tokens; otherwise 1).
    uint32_t mb_group = 0;
    uint32_t fuse_swiglu = 1;     // 1: SwiGLU forward inside the gate/up GEMM epilogue; 2: also its backward inside the down-gradient GEMM
    uint32_t dp_buckets = 1;      // dp > 1, fused: gradient reduce-scatter + AdamW per layer bucket, overlapped with backward
    uint32_t wait_limit_ms = 0;   // bounded device-side waits: 0 = the library default (about a second)
    uint32_t reserved[4] = {0, 0, 0, 0};
};
static_assert(sizeof(TrainSpec) == 96, "TrainSpec layout");

struct Config {
    ModelSpec model;
    Topology topo;
    TrainSpec train;
};

// ---- version-2 execution section --------------------------------------------------------
enum KernelId : uint16_t {
    K_NONE = 0,
    K_EMBED_FWD, K_EMBED_BWD,
    K_RMSNORM_FWD, K_RMSNORM_BWD,
    K_GEMM,
    K_ROPE,
    K_ATTN_FWD, K_ATTN_BWD,
    K_SWIGLU_FWD, K_SWIGLU_BWD,
    K_CROSS_ENTROPY,
    K_ADAMW,
    K_ZERO,
    K_NCCL_ALL_REDUCE, K_NCCL_REDUCE_SCATTER, K_NCCL_ALL_GATHER, K_NCCL_ALL_TO_ALL, K_NCCL_SEND, K_NCCL_RECV,
    K_GEMM_RS, K_AG_GEMM, K_RS_ADAMW, K_FSDP_AG_GEMM, K_MOE_ROUTE, K_MOE_DISPATCH_GEMM, K_MOE_GEMM_COMBINE,
    K_LOAD_TOKENS,
    K_ADD,
    K_CROSS_ENTROPY_TP,
    K_QUANT_FP8,             // flags 0: rows 1x128 (activations), 1: blocks 128x128 (+ transposed copy) (weights)
    K_GEMM_FP8,              // e4m3 block-scaled GEMM
    K_COUNT
};

struct ExecOp {              // 64 bytes
    uint16_t kernel;         // KernelId
    uint16_t flags;          // kernel specific (GEMM: bit0 transA, bit1 transB, bits 4-7 epilogue)
    int32_t t[8];            // tensor ids, -1 = unused
    int32_t i[5];            // integer parameters
    float f[2];              // float parameters
};
static_assert(sizeof(ExecOp) == 64, "ExecOp layout");

struct ExecHeader {          // 32 bytes + TrainSpec
    uint32_t magic;          // kExecMagic
    uint32_t num_exec;
    uint32_t num_named;      // entries of the name table (parameters, for checkpoints / init)
    uint32_t act_slots;      // microbatch slots the activation segment holds
    uint64_t param_elems;    // elements of this rank's parameter shard
    uint64_t reserved;
};
static_assert(sizeof(ExecHeader) == 32, "ExecHeader layout");

struct NamedTensor {         // 64 bytes: lets the runtime initialise / checkpoint parameters by name
    char name[40];
    int32_t tensor;          // tensor id of the bf16 parameter
    int32_t grad;            // tensor id of the fp32 gradient
    int32_t master;          // offset of the parameter in the flat space, in units of 512 elements
    uint32_t rows, cols;
    float init_std;          // 0 = initialise to ones (norm gains)
};
static_assert(sizeof(NamedTensor) == 64, "NamedTensor layout");

}  // namespace cai
