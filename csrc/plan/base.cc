// base.cc - logging, FNV-1a, raw IO, formatters, name tables, topology math.
// Behaviour mirrors the reference's src/common.c and src/topology.c so that files and hashes
// stay interchangeable.
#include <sys/stat.h>

#include <strings.h>

#include <cstdarg>
#include <cstdlib>
#include <cstring>

#include "plan.h"

namespace cai {

// Default INFO, as in the reference (src/common.c:9-22). CAI_LOG_LEVEL (error | warn | info | debug, or 0..3) sets the
// starting level of a process; log_set_level() / cai_log_set_level() override it.
static int g_level = -1;
static int level_from_env() {
    const char* e = std::getenv("CAI_LOG_LEVEL");
    if (!e || !*e) return LOG_INFO;
    static const char* names[] = {"error", "warn", "info", "debug"};
    for (int i = 0; i < 4; ++i)
        if (!strcasecmp(e, names[i])) return i;
    if (e[0] >= '0' && e[0] <= '3' && !e[1]) return e[0] - '0';
    return LOG_INFO;
}
void log_set_level(LogLevel lv) { g_level = lv; }
void logf(LogLevel lv, const char* fmt, ...) {
    if (g_level < 0) g_level = level_from_env();
    if (lv > g_level) return;
    static const char* tags[] = {"ERROR", "WARN", "INFO", "DEBUG"};
    std::fprintf(stderr, "[cai %s] ", tags[lv]);
    va_list ap;
    va_start(ap, fmt);
    std::vfprintf(stderr, fmt, ap);
    va_end(ap);
    std::fputc('\n', stderr);
}

uint64_t fnv1a(const void* data, size_t len, uint64_t seed) {
    auto* p = static_cast<const unsigned char*>(data);
    uint64_t h = seed;
    for (size_t i = 0; i < len; ++i) h = (h ^ p[i]) * 1099511628211ull;
    return h;
}

bool write_all(FILE* f, const void* buf, size_t n) { return n == 0 || std::fwrite(buf, 1, n, f) == n; }
bool read_all(FILE* f, void* buf, size_t n) { return n == 0 || std::fread(buf, 1, n, f) == n; }

std::string fmt_bytes(uint64_t bytes) {
    static const char* unit[] = {"B", "KiB", "MiB", "GiB", "TiB", "PiB"};
    double v = static_cast<double>(bytes);
    int u = 0;
    for (; v >= 1024.0 && u < 5; ++u) v /= 1024.0;
    char buf[48];
    std::snprintf(buf, sizeof buf, "%.2f %s", v, unit[u]);
    return buf;
}

std::string fmt_count(double v) {
    static const char* unit[] = {"", "K", "M", "B", "T", "P", "E"};
    int u = 0;
    for (; v >= 1000.0 && u < 6; ++u) v /= 1000.0;
    char buf[48];
    if (v >= 1000.0) std::snprintf(buf, sizeof buf, "%.2e", v * 1e18);
    else std::snprintf(buf, sizeof buf, "%.2f%s", v, unit[u]);
    return buf;
}

bool mkdir_p(const std::string& path) {
    std::string cur;
    for (size_t i = 0; i <= path.size(); ++i) {
        if (i == path.size() || path[i] == '/') {
            if (!cur.empty()) ::mkdir(cur.c_str(), 0755);
        }
        if (i < path.size()) cur.push_back(path[i]);
    }
    struct stat st;
    return ::stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}

const char* status_str(int s) {
    switch (s) {
        case OK: return "ok";
        case ERR_IO: return "io error";
        case ERR_INVALID: return "invalid argument";
        case ERR_OOM: return "out of memory";
        case ERR_TOPOLOGY: return "topology error";
        case ERR_PLAN: return "plan error";
        case ERR_BACKEND: return "backend error";
        case ERR_DEPENDENCY: return "dependency violation";
        case ERR_BUDGET: return "memory budget exceeded";
        default: return "unknown error";
    }
}

size_t dtype_size(uint16_t dt) {
    static const size_t sz[DT_COUNT] = {4, 2, 2, 1, 1, 4, 1};
    return dt < DT_COUNT ? sz[dt] : 0;
}
const char* dtype_name(uint16_t dt) {
    static const char* n[DT_COUNT] = {"fp32", "bf16", "fp16", "fp8e4m3", "fp8e5m2", "int32", "uint8"};
    return dt < DT_COUNT ? n[dt] : "?";
}
const char* tclass_name(uint16_t c) {
    static const char* n[TC_COUNT] = {"param", "grad", "optstate", "activation", "comm", "workspace"};
    return c < TC_COUNT ? n[c] : "?";
}
const char* stream_name(uint16_t s) {
    static const char* n[ST_COUNT] = {"compute_hi", "compute_lo", "comm_tp", "comm_pp", "comm_dp", "io"};
    return s < ST_COUNT ? n[s] : "?";
}
const char* op_name(uint16_t k) {
    static const char* n[OP_COUNT] = {"gemm", "attn_fwd", "attn_bwd", "rmsnorm", "swiglu", "elementwise",
                                      "reduce_scatter", "all_gather", "all_reduce", "all_to_all", "pipe_send",
                                      "pipe_recv", "optimizer", "event_record", "event_wait",
                                      "gemm_rs", "ag_gemm", "rs_adamw", "fsdp_ag_gemm", "moe_dispatch_gemm",
                                      "moe_gemm_combine"};
    return k < OP_COUNT ? n[k] : "?";
}
const char* kernel_name(uint16_t k) {
    static const char* n[K_COUNT] = {"none", "embed_fwd", "embed_bwd", "rmsnorm_fwd", "rmsnorm_bwd", "gemm", "rope",
                                     "attn_fwd", "attn_bwd", "swiglu_fwd", "swiglu_bwd", "cross_entropy", "adamw",
                                     "zero", "nccl_all_reduce", "nccl_reduce_scatter", "nccl_all_gather",
                                     "nccl_all_to_all", "nccl_send", "nccl_recv", "gemm_rs", "ag_gemm", "rs_adamw",
                                     "fsdp_ag_gemm", "moe_route", "moe_dispatch_gemm", "moe_gemm_combine",
                                     "load_tokens", "add", "cross_entropy_tp", "quant_fp8", "gemm_fp8"};
    return k < K_COUNT ? n[k] : "?";
}
bool op_is_comm(uint16_t k) {
    switch (k) {
        case OP_REDUCE_SCATTER: case OP_ALL_GATHER: case OP_ALL_REDUCE: case OP_ALL_TO_ALL:
        case OP_PIPE_SEND: case OP_PIPE_RECV: return true;
        default: return false;
    }
}
bool op_is_compute(uint16_t k) {
    switch (k) {
        case OP_GEMM: case OP_ATTENTION_FWD: case OP_ATTENTION_BWD: case OP_RMSNORM: case OP_SWIGLU:
        case OP_ELEMENTWISE: case OP_OPTIMIZER:
        // fused compute+collective kernels occupy SMs and are costed as compute plus their bytes
        case OP_GEMM_RS: case OP_AG_GEMM: case OP_RS_ADAMW: case OP_FSDP_AG_GEMM:
        case OP_MOE_DISPATCH_GEMM: case OP_MOE_GEMM_COMBINE: return true;
        default: return false;
    }
}

// ---- topology -------------------------------------------------------------------------
void topology_default(Topology* t) {
    std::memset(t, 0, sizeof *t);
    t->gpus_per_rack = 72;
    t->trays_per_rack = 18;
    t->gpus_per_tray = 4;
    t->num_racks = 1;
    t->intra_rack_bw = 1800ull * 1000000000ull;
    t->inter_rack_bw = 100ull * 1000000000ull;
    t->hbm_bw = 8000ull * 1000000000ull;
    t->gpu_flops_bf16 = 2.5e15;
    t->gpu_mem_bytes = 288ull * 1000000000ull;
}

static int fail(std::string* err, int code, const char* fmt, ...) {
    if (err) {
        char buf[256];
        va_list ap;
        va_start(ap, fmt);
        std::vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        *err = buf;
    }
    return code;
}

int topology_finalize(Topology* t, std::string* err) {
    if (!t->gpus_per_rack || !t->num_racks)
        return fail(err, ERR_TOPOLOGY, "gpus_per_rack and num_racks must be > 0");
    if (!t->gpus_per_tray) t->gpus_per_tray = 4;
    if (!t->trays_per_rack) t->trays_per_rack = t->gpus_per_rack / t->gpus_per_tray;
    if (t->trays_per_rack * t->gpus_per_tray != t->gpus_per_rack)
        return fail(err, ERR_TOPOLOGY, "trays_per_rack(%u)*gpus_per_tray(%u) != gpus_per_rack(%u)",
                    t->trays_per_rack, t->gpus_per_tray, t->gpus_per_rack);
    const uint64_t total = static_cast<uint64_t>(t->gpus_per_rack) * t->num_racks;
    if (t->spare_gpus >= total)
        return fail(err, ERR_TOPOLOGY, "spare_gpus(%u) >= total gpus(%llu)", t->spare_gpus,
                    static_cast<unsigned long long>(total));
    const uint64_t usable = total - t->spare_gpus;
    if (usable > 0xFFFFFFFFull)
        return fail(err, ERR_TOPOLOGY, "world_size %llu exceeds 32-bit rank space",
                    static_cast<unsigned long long>(usable));
    t->world_size = static_cast<uint32_t>(usable);
    if (!(t->gpu_flops_bf16 > 0) || !t->hbm_bw || !t->intra_rack_bw || !t->inter_rack_bw)
        return fail(err, ERR_TOPOLOGY, "bandwidth/flops fields must be > 0");
    return OK;
}

PhysId phys_of_rank(const Topology& t, uint32_t rank) {
    PhysId p{};
    p.global_rank = rank;
    p.rack_id = static_cast<uint16_t>(rank / t.gpus_per_rack);
    p.gpu_in_rack = static_cast<uint8_t>(rank % t.gpus_per_rack);
    p.tray_id = static_cast<uint8_t>(p.gpu_in_rack / t.gpus_per_tray);
    p.gpu_in_tray = static_cast<uint8_t>(p.gpu_in_rack % t.gpus_per_tray);
    p.nic_id = p.gpu_in_rack;
    p.rail_id = p.gpu_in_tray;
    return p;
}
uint32_t rank_of(const Topology& t, uint16_t rack, uint8_t tray, uint8_t gpu) {
    return rack * t.gpus_per_rack + tray * t.gpus_per_tray + gpu;
}
bool same_rack(const Topology& t, uint32_t a, uint32_t b) { return a / t.gpus_per_rack == b / t.gpus_per_rack; }

int spare_rank(const Topology& t, uint32_t failed, uint32_t* out) {
    const uint64_t total = static_cast<uint64_t>(t.gpus_per_rack) * t.num_racks;
    if (t.world_size >= total || failed >= t.world_size) return ERR_INVALID;
    const uint32_t bad_rack = failed / t.gpus_per_rack;
    for (uint64_t s = t.world_size; s < total; ++s)
        if (s / t.gpus_per_rack != bad_rack) {
            *out = static_cast<uint32_t>(s);
            return OK;
        }
    *out = t.world_size;  // every spare sits in the failed rack: take the first one
    return OK;
}

int topology_write(const std::string& path, const Topology& t) {
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) return ERR_IO;
    const uint32_t magic = kTopoMagic;
    const bool ok = write_all(f, &magic, 4) && write_all(f, &t, sizeof t);
    return (std::fclose(f) == 0 && ok) ? OK : ERR_IO;
}
int topology_read(const std::string& path, Topology* t) {
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return ERR_IO;
    uint32_t magic = 0;
    int rc = OK;
    if (!read_all(f, &magic, 4)) rc = ERR_IO;
    else if (magic != kTopoMagic) rc = ERR_TOPOLOGY;
    else if (!read_all(f, t, sizeof *t)) rc = ERR_IO;
    std::fclose(f);
    return rc;
}
uint64_t topology_hash(const Topology& t) { return fnv1a(&t, sizeof t); }

}  // namespace cai
