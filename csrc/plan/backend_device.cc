// backend_device.cc - the executing backend of the C runtime: the plan runs on a GPU.
//
// libcai_host.so stays free of CUDA: the kernel library (libcai_kernels.so, next to this library) is
// opened with dlopen when this backend is asked for, and everything below goes through its C ABI
// (csrc/runtime/cai_runtime.h): allocate the arena, create the executor over the plan's bytes,
// initialise parameters, copy a synthetic batch in, enqueue the step, read the loss and the measured
// per-op timeline back. This is the role the reference sketches for its CUDA backend
// (src/backend_cuda.c:13-30: "cuInit, load kernels, streams/events, NCCL comms, time each op") and
// never fills in.
//
// Scope: plans of a single rank (world_size 1). Multi-rank jobs need NCCL ids and peer arenas
// exchanged between processes, which the Python launcher (python -m cai_b200.trainer) does.
#include <dlfcn.h>

#include <algorithm>

#include <cmath>
#include <cstdio>
#include <cstring>

#include "backend.h"

namespace cai {
namespace {

struct TraceRec {   // cai_exec_trace_rec of cai_runtime.h
    uint32_t op_index; uint16_t kind, stream; double start_s, end_s; uint64_t bytes, flops;
};

struct Api {
    void* lib = nullptr;
    int (*dev_count)() = nullptr;
    int (*dev_set)(int) = nullptr;
    int (*dev_malloc)(void**, unsigned long long) = nullptr;
    int (*dev_free)(void*) = nullptr;
    int (*dev_memset)(void*, int, unsigned long long) = nullptr;
    int (*dev_h2d)(void*, const void*, unsigned long long) = nullptr;
    int (*dev_d2h)(void*, const void*, unsigned long long) = nullptr;
    int (*dev_h2d_async)(void*, const void*, unsigned long long, void*) = nullptr;
    int (*host_alloc)(void**, unsigned long long) = nullptr;
    int (*host_free)(void*) = nullptr;
    int (*exec_create)(void**, const void*, size_t, void*, void* const*) = nullptr;
    void (*exec_destroy)(void*) = nullptr;
    void* (*exec_stream)(void*, int) = nullptr;
    void* (*exec_tensor_ptr)(void*, int) = nullptr;
    int (*exec_step)(void*, int, float) = nullptr;
    int (*exec_sync)(void*) = nullptr;
    int (*exec_trace_enable)(void*, int) = nullptr;
    int (*exec_trace_read)(void*, TraceRec*, int) = nullptr;
    int (*rope_table)(float*, int, int, float, void*) = nullptr;
    int (*status_read)(int) = nullptr;
    const char* (*last_error)() = nullptr;
};

struct DeviceImpl {
    Api api;
    void* arena_raw = nullptr;
    uint8_t* arena = nullptr;
    void* ex = nullptr;
    Plan plan;                 // tensor / name tables of the bound plan
    int t_tokens = -1, t_targets = -1, t_loss = -1, t_rope = -1, t_param = -1, t_master = -1, t_m = -1, t_v = -1;
    int32_t* host_batch = nullptr;   // pinned: tokens then targets
    uint64_t batch_elems = 0;
};

std::string own_directory() {
    Dl_info info;
    if (dladdr(reinterpret_cast<void*>(&own_directory), &info) && info.dli_fname) {
        std::string p = info.dli_fname;
        const size_t s = p.find_last_of('/');
        return s == std::string::npos ? "." : p.substr(0, s);
    }
    return ".";
}

bool load_api(Api* a, std::string* why) {
    const char* env = std::getenv("CAI_KERNEL_LIB");
    const std::string path = env && *env ? env : own_directory() + "/libcai_kernels.so";
    a->lib = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!a->lib) {
        *why = std::string("cannot open the kernel library: ") + dlerror();
        return false;
    }
    bool ok = true;
    auto sym = [&](auto& fn, const char* name) {
        fn = reinterpret_cast<std::decay_t<decltype(fn)>>(dlsym(a->lib, name));
        if (!fn) {
            *why = std::string("kernel library lacks ") + name;
            ok = false;
        }
    };
    sym(a->dev_count, "cai_dev_count"); sym(a->dev_set, "cai_dev_set"); sym(a->dev_malloc, "cai_dev_malloc");
    sym(a->dev_free, "cai_dev_free"); sym(a->dev_memset, "cai_dev_memset"); sym(a->dev_h2d, "cai_dev_h2d");
    sym(a->dev_d2h, "cai_dev_d2h"); sym(a->dev_h2d_async, "cai_dev_h2d_async"); sym(a->host_alloc, "cai_dev_host_alloc");
    sym(a->host_free, "cai_dev_host_free"); sym(a->exec_create, "cai_exec_create"); sym(a->exec_destroy, "cai_exec_destroy");
    sym(a->exec_stream, "cai_exec_stream"); sym(a->exec_tensor_ptr, "cai_exec_tensor_ptr"); sym(a->exec_step, "cai_exec_step");
    sym(a->exec_sync, "cai_exec_sync"); sym(a->exec_trace_enable, "cai_exec_trace_enable");
    sym(a->exec_trace_read, "cai_exec_trace_read"); sym(a->rope_table, "cai_rope_table"); sym(a->status_read, "cai_status_read");
    sym(a->last_error, "cai_last_error");
    return ok;
}

// xorshift64 + Box-Muller, the generator family of the fp64 oracle (csrc/ref/refmodel.cc)
struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed ? seed : 0x9E3779B97F4A7C15ull) {}
    uint64_t next() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return s; }
    double uniform() { return ((next() >> 11) + 1.0) / 9007199254740994.0; }
    double normal() { return std::sqrt(-2.0 * std::log(uniform())) * std::cos(6.283185307179586 * uniform()); }
};

uint16_t to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);   // round to nearest even
    return static_cast<uint16_t>(u >> 16);
}

int find_named(const Plan& p, const char* name) {
    for (const NamedTensor& nt : p.named)
        if (!std::strcmp(nt.name, name)) return nt.tensor;
    return -1;
}

DeviceImpl* D(Backend* be) { return static_cast<DeviceImpl*>(be->impl); }

int fail(DeviceImpl* d, const char* what) {
    logf(LOG_ERROR, "device backend: %s failed: %s", what, d->api.last_error ? d->api.last_error() : "?");
    return ERR_BACKEND;
}

void release(DeviceImpl* d) {
    if (d->ex) d->api.exec_destroy(d->ex);
    d->ex = nullptr;
    if (d->arena_raw) d->api.dev_free(d->arena_raw);
    d->arena_raw = nullptr;
    if (d->host_batch) d->api.host_free(d->host_batch);
    d->host_batch = nullptr;
}

int dev_load_plan(Backend* be, const Plan& plan, const std::string& path, uint32_t rank, uint32_t world) {
    DeviceImpl* d = D(be);
    release(d);
    if (plan.hdr.version != 2) {
        logf(LOG_ERROR, "device backend: '%s' is a cost-only (version 1) plan; compile it with --exec", path.c_str());
        return ERR_PLAN;
    }
    if (world != 1 || plan.hdr.world_size != 1) {
        logf(LOG_ERROR, "device backend of the C runtime drives single-rank plans (world_size %u); multi-rank jobs start "
                        "through `python -m cai_b200.trainer`, which exchanges NCCL ids and peer arenas", plan.hdr.world_size);
        return ERR_INVALID;
    }
    (void)rank;
    d->plan = plan;
    std::vector<uint8_t> raw;
    {
        FILE* f = std::fopen(path.c_str(), "rb");
        if (!f) return ERR_IO;
        std::fseek(f, 0, SEEK_END);
        const long n = std::ftell(f);
        std::fseek(f, 0, SEEK_SET);
        raw.resize(n > 0 ? static_cast<size_t>(n) : 0);
        const bool ok = n > 0 && std::fread(raw.data(), 1, raw.size(), f) == raw.size();
        std::fclose(f);
        if (!ok) return ERR_IO;
    }
    const Api& a = d->api;
    const uint64_t bytes = plan.hdr.arena_bytes + 2048;
    if (a.dev_malloc(&d->arena_raw, bytes) != 0) return fail(d, "arena allocation");
    if (a.dev_memset(d->arena_raw, 0, bytes) != 0) return fail(d, "arena clear");
    d->arena = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(d->arena_raw) + 1023) & ~uintptr_t(1023));
    if (a.exec_create(&d->ex, raw.data(), raw.size(), d->arena, nullptr) != 0) return fail(d, "executor creation");
    d->t_tokens = find_named(plan, "@tokens"); d->t_targets = find_named(plan, "@targets");
    d->t_loss = find_named(plan, "@loss"); d->t_rope = find_named(plan, "@rope_table");
    d->t_param = find_named(plan, "@flat_param"); d->t_master = find_named(plan, "@flat_master");
    d->t_m = find_named(plan, "@flat_m"); d->t_v = find_named(plan, "@flat_v");
    if (d->t_tokens < 0 || d->t_targets < 0 || d->t_loss < 0 || d->t_rope < 0 || d->t_master < 0) {
        logf(LOG_ERROR, "device backend: plan lacks its runtime buffers");
        return ERR_PLAN;
    }
    const ModelSpec& m = plan.model;
    if (a.rope_table(static_cast<float*>(a.exec_tensor_ptr(d->ex, d->t_rope)), m.seq_len, m.head_dim, plan.train.rope_theta,
                     a.exec_stream(d->ex, 0)) != 0)
        return fail(d, "rope table");
    // Parameters: N(0, init_std) for matrices, ones for norm gains; the fp32 master copy holds the value, the
    // bf16 tensor its rounding. One generator per tensor, seeded from its name, so a layout change does not
    // reshuffle the model.
    float* master = static_cast<float*>(a.exec_tensor_ptr(d->ex, d->t_master));
    std::vector<float> w32;
    std::vector<uint16_t> w16;
    for (const NamedTensor& nt : plan.named) {
        if (nt.init_std < 0) continue;
        const uint64_t n = static_cast<uint64_t>(nt.rows) * nt.cols;
        w32.resize(n);
        w16.resize(n);
        if (nt.init_std == 0.f) {
            std::fill(w32.begin(), w32.end(), 1.0f);
        } else {
            Rng rng(fnv1a(nt.name, std::strlen(nt.name), kFnvInit) ^ (static_cast<uint64_t>(plan.train.seed) + 1));
            for (uint64_t i = 0; i < n; ++i) w32[i] = static_cast<float>(rng.normal() * nt.init_std);
        }
        for (uint64_t i = 0; i < n; ++i) w16[i] = to_bf16(w32[i]);
        if (a.dev_h2d(a.exec_tensor_ptr(d->ex, nt.tensor), w16.data(), n * 2) != 0 ||
            a.dev_h2d(master + static_cast<uint64_t>(nt.master) * 512, w32.data(), n * 4) != 0)
            return fail(d, "parameter upload");
    }
    d->batch_elems = static_cast<uint64_t>(plan.hdr.num_microbatches) * m.microbatch * m.seq_len;
    if (a.host_alloc(reinterpret_cast<void**>(&d->host_batch), d->batch_elems * 2 * sizeof(int32_t)) != 0)
        return fail(d, "pinned batch buffer");
    a.exec_trace_enable(d->ex, 1);   // every step is timed op by op: the statistics are measurements
    if (a.exec_sync(d->ex) != 0) return fail(d, "set-up synchronisation");
    logf(LOG_INFO, "device backend: arena %.2f GiB on the GPU, %zu parameters tensors initialised",
         plan.hdr.arena_bytes / (1024.0 * 1024.0 * 1024.0), plan.named.size());
    return OK;
}

int dev_run_step(Backend* be, uint32_t step_1based, uint64_t seed, bool want_trace, StepResult* out) {
    DeviceImpl* d = D(be);
    if (!d->ex) return ERR_PLAN;
    const Api& a = d->api;
    const ModelSpec& m = d->plan.model;
    // uniform-random sequences of seq_len + 1 tokens: inputs are the first seq_len, targets the last seq_len
    Rng rng(seed);
    const uint64_t rows = d->batch_elems / m.seq_len;
    int32_t* tok = d->host_batch;
    int32_t* tgt = d->host_batch + d->batch_elems;
    for (uint64_t r = 0; r < rows; ++r) {
        int32_t prev = static_cast<int32_t>(rng.next() % m.vocab_size);
        for (uint32_t t = 0; t < m.seq_len; ++t) {
            const int32_t next = static_cast<int32_t>(rng.next() % m.vocab_size);
            tok[r * m.seq_len + t] = prev;
            tgt[r * m.seq_len + t] = next;
            prev = next;
        }
    }
    void* s0 = a.exec_stream(d->ex, 0);
    if (a.dev_h2d_async(a.exec_tensor_ptr(d->ex, d->t_tokens), tok, d->batch_elems * 4, s0) != 0 ||
        a.dev_h2d_async(a.exec_tensor_ptr(d->ex, d->t_targets), tgt, d->batch_elems * 4, s0) != 0)
        return fail(d, "batch upload");
    if (a.exec_step(d->ex, static_cast<int>(step_1based), d->plan.train.lr) != 0) return fail(d, "step launch");
    if (a.exec_sync(d->ex) != 0) return fail(d, "step synchronisation");
    const int st = a.status_read(1);
    if (st != 0) {
        logf(LOG_ERROR, "device backend: a kernel gave up on a bounded wait (device status %d)", st);
        return ERR_BACKEND;
    }
    float loss[8] = {0};
    if (a.dev_d2h(loss, a.exec_tensor_ptr(d->ex, d->t_loss), sizeof loss) != 0) return fail(d, "loss read");
    out->loss = loss[0];
    out->has_loss = true;
    std::vector<TraceRec> recs(d->plan.ops.size());
    const int n = a.exec_trace_read(d->ex, recs.data(), static_cast<int>(recs.size()));
    double t0 = 1e300, t1 = 0.0;
    std::vector<std::pair<double, double>> hi;
    for (int i = 0; i < n; ++i) {
        const TraceRec& r = recs[i];
        t0 = std::min(t0, r.start_s);
        t1 = std::max(t1, r.end_s);
        if (r.stream < ST_COUNT) out->stream_busy[r.stream] += std::max(0.0, r.end_s - r.start_s);
        if (r.stream == ST_COMPUTE_HI) hi.emplace_back(r.start_s, r.end_s);
        if (want_trace) out->trace.push_back({r.op_index, r.kind, r.stream, r.start_s, r.end_s, r.bytes, r.flops});
    }
    out->step_time_s = n ? t1 - t0 : 0.0;
    std::sort(hi.begin(), hi.end());
    double covered = 0.0, cs = 0.0, ce = -1.0;
    for (const auto& iv : hi) {
        if (ce < 0 || iv.first > ce) {
            if (ce >= 0) covered += ce - cs;
            cs = iv.first;
            ce = iv.second;
        } else {
            ce = std::max(ce, iv.second);
        }
    }
    if (ce >= 0) covered += ce - cs;
    out->hi_idle_ratio = out->step_time_s > 0 ? 1.0 - covered / out->step_time_s : 0.0;
    return OK;
}

const char* const kSections[4] = {"param", "master", "m", "v"};

int dev_snapshot(Backend* be, std::vector<std::string>* names, std::vector<std::vector<uint8_t>>* data) {
    DeviceImpl* d = D(be);
    if (!d->ex) return ERR_PLAN;
    const int ids[4] = {d->t_param, d->t_master, d->t_m, d->t_v};
    for (int k = 0; k < 4; ++k) {
        if (ids[k] < 0) continue;
        const uint64_t n = d->plan.tensors[ids[k]].nbytes;
        std::vector<uint8_t> buf(n);
        if (d->api.dev_d2h(buf.data(), d->api.exec_tensor_ptr(d->ex, ids[k]), n) != 0) return fail(d, "state download");
        names->push_back(kSections[k]);
        data->push_back(std::move(buf));
    }
    return OK;
}

int dev_restore(Backend* be, const std::string& name, const void* data, uint64_t nbytes) {
    DeviceImpl* d = D(be);
    if (!d->ex) return ERR_PLAN;
    const int ids[4] = {d->t_param, d->t_master, d->t_m, d->t_v};
    for (int k = 0; k < 4; ++k)
        if (name == kSections[k] && ids[k] >= 0) {
            if (d->plan.tensors[ids[k]].nbytes != nbytes) return ERR_PLAN;
            return d->api.dev_h2d(d->api.exec_tensor_ptr(d->ex, ids[k]), data, nbytes) == 0 ? OK : fail(d, "state upload");
        }
    return OK;   // sections this backend does not know are skipped
}

int dev_sync(Backend* be) { return D(be)->ex && D(be)->api.exec_sync(D(be)->ex) != 0 ? ERR_BACKEND : OK; }

void dev_destroy(Backend* be) {
    DeviceImpl* d = D(be);
    release(d);
    // the library stays loaded: its CUDA context and static state are process-wide
    delete d;
    delete be;
}

}  // namespace

Backend* backend_device_create(uint32_t local_rank, std::string* why) {
    auto d = new DeviceImpl();
    if (!load_api(&d->api, why)) {
        delete d;
        return nullptr;
    }
    const int n = d->api.dev_count();
    if (n <= 0 || static_cast<int>(local_rank) >= n || d->api.dev_set(static_cast<int>(local_rank)) != 0) {
        *why = n <= 0 ? "no CUDA device is visible" : "local rank has no device";
        delete d;
        return nullptr;
    }
    auto be = new Backend();
    be->name = "device";
    be->impl = d;
    be->op_seconds = nullptr;
    be->load_plan = dev_load_plan;
    be->run_step = dev_run_step;
    be->snapshot = dev_snapshot;
    be->restore = dev_restore;
    be->sync = dev_sync;
    be->destroy = dev_destroy;
    return be;
}

}  // namespace cai
