// optable.cc - rank coordinates, communicator groups, the version-1 (cost-only) op table and
// plan file IO.
//
// The version-1 table reproduces the reference's schedule language op for op
// (src/model.c:365-752): same issue order, same flops / bytes, same event numbering, so the
// files it writes are byte-identical and the analytic replay gives the same numbers.
#include <algorithm>
#include <cstdarg>
#include <cstring>

#include "plan.h"

namespace cai {

// ------------------------------------------------------------------ coordinates and groups
// Rank layout: tensor-parallel innermost, then context, pipeline, data parallel.
uint32_t rank_stage(const Decomp& d, uint32_t rank) {
    return static_cast<uint32_t>((rank / (static_cast<uint64_t>(d.tp) * d.cp)) % d.pp);
}

// One communicator of one rank, computed without touching the heap: whole-world checks call this once per rank and kind
// (hundreds of thousands of ranks), so it does only the arithmetic its kind needs.
bool rank_group(const Decomp& d, const Topology& topo, bool is_moe, uint16_t kind, uint32_t rank, CommGroup* out) {
    const uint32_t replica = d.tp * d.pp * d.cp;
    CommGroup c{};
    c.kind = kind;
    switch (kind) {
        case GROUP_TP: {
            const uint32_t tp_first = rank - rank % d.tp;
            c.group_id = 0;
            c.size = d.tp;
            c.color = tp_first;
            c.intra_rack = same_rack(topo, tp_first, tp_first + d.tp - 1) ? 1 : 0;
            break;
        }
        case GROUP_DP: {
            const uint32_t within = rank % replica;
            c.group_id = 1;
            c.size = d.dp;
            c.color = within;
            c.intra_rack = d.dp > 1 && same_rack(topo, within, within + (d.dp - 1) * replica) ? 1 : 0;
            break;
        }
        case GROUP_PP: {
            // The reference always prices pipeline and expert groups at the inter-rack rate
            // (src/model.c:581,589); kept so version-1 plans stay byte-identical.
            const uint32_t tp_id = rank % d.tp, cp_id = (rank / d.tp) % d.cp, dp_id = rank / replica;
            c.group_id = 2;
            c.size = d.pp;
            c.color = dp_id * (d.tp * d.cp) + cp_id * d.tp + tp_id;
            break;
        }
        case GROUP_EP: {
            if (!(is_moe && d.ep > 1)) return false;
            const uint32_t within = rank % replica, dp_id = rank / replica;
            c.group_id = 3;
            c.size = d.ep;
            c.color = within + (dp_id / d.ep) * d.ep * replica;
            break;
        }
        default: return false;
    }
    *out = c;
    return true;
}

std::vector<CommGroup> rank_groups(const Decomp& d, const Topology& topo, bool is_moe, uint32_t rank) {
    std::vector<CommGroup> g;
    g.reserve(4);
    CommGroup c;
    for (uint16_t kind : {GROUP_TP, GROUP_DP, GROUP_PP, GROUP_EP})
        if (rank_group(d, topo, is_moe, kind, rank, &c)) g.push_back(c);
    return g;
}

std::vector<uint32_t> group_members(const Decomp& d, bool is_moe, uint16_t kind, uint32_t rank) {
    const uint32_t replica = d.tp * d.pp * d.cp;
    const uint32_t tp_id = rank % d.tp;
    const uint32_t dp_id = rank / replica;
    const uint32_t within = rank % replica;
    std::vector<uint32_t> m;
    switch (kind) {
        case GROUP_TP:
            for (uint32_t i = 0; i < d.tp; ++i) m.push_back(rank - tp_id + i);
            break;
        case GROUP_DP:
            for (uint32_t i = 0; i < d.dp; ++i) m.push_back(within + i * replica);
            break;
        case GROUP_PP: {
            const uint32_t stage = rank_stage(d, rank);
            const uint32_t base = rank - stage * d.tp * d.cp;
            for (uint32_t s = 0; s < d.pp; ++s) m.push_back(base + s * d.tp * d.cp);
            break;
        }
        case GROUP_EP:
            if (is_moe && d.ep > 1) {
                const uint32_t first_dp = (dp_id / d.ep) * d.ep;
                for (uint32_t i = 0; i < d.ep; ++i) m.push_back(within + (first_dp + i) * replica);
            }
            break;
        default: break;
    }
    return m;
}

// ------------------------------------------------------------------ version-1 emitter
namespace {

struct Emitter {
    std::vector<Op> ops;
    uint32_t next_event = 0;

    void compute(uint16_t kind, uint16_t stream, double flops, uint16_t mb) {
        Op o{};
        o.kind = kind;
        o.stream_id = stream;
        o.flops = static_cast<uint64_t>(flops < 0 ? 0 : flops);
        o.aux1 = mb;
        ops.push_back(o);
    }
    void comm(uint16_t kind, uint16_t stream, double bytes, uint32_t group, uint16_t mb) {
        Op o{};
        o.kind = kind;
        o.stream_id = stream;
        o.bytes = static_cast<uint64_t>(bytes < 0 ? 0 : bytes);
        o.aux0 = group;
        o.aux1 = mb;
        ops.push_back(o);
    }
    uint32_t record(uint16_t stream, uint16_t mb) {
        Op o{};
        o.kind = OP_EVENT_RECORD;
        o.stream_id = stream;
        o.aux0 = next_event;
        o.aux1 = mb;
        ops.push_back(o);
        return next_event++;
    }
    void wait(uint16_t stream, uint32_t ev, uint16_t mb) {
        Op o{};
        o.kind = OP_EVENT_WAIT;
        o.stream_id = stream;
        o.aux0 = ev;
        o.aux1 = mb;
        ops.push_back(o);
    }
    // record on `from`, make each of `to` wait for it
    void sync(uint16_t from, std::initializer_list<uint16_t> to, uint16_t mb) {
        const uint32_t e = record(from, mb);
        for (uint16_t s : to) wait(s, e, mb);
    }
};

struct Costs {
    double norm, qkv, attn, o, mlp_up, mlp_down, swiglu, logits, loss, recompute, opt;
    double tp_msg, pipe_msg, layer_w, a2a;
    uint32_t tp, dp, ep, stage, layers, last_stage;
    bool moe;
};

void tp_all_reduce(Emitter& e, const Costs& c, uint16_t mb, bool also_lo) {
    e.sync(ST_COMPUTE_HI, {ST_COMM_TP}, mb);
    e.comm(OP_ALL_REDUCE, ST_COMM_TP, c.tp_msg, GROUP_TP, mb);
    if (also_lo) e.sync(ST_COMM_TP, {ST_COMPUTE_HI, ST_COMPUTE_LO}, mb);
    else e.sync(ST_COMM_TP, {ST_COMPUTE_HI}, mb);
}

void expert_all_to_all(Emitter& e, const Costs& c, uint16_t mb) {
    e.comm(OP_ALL_TO_ALL, ST_COMM_DP, c.a2a, GROUP_EP, mb);
    e.sync(ST_COMM_DP, {ST_COMPUTE_HI}, mb);
}

void layer_forward(Emitter& e, const Costs& c, uint16_t mb) {
    if (c.dp > 1) {
        // FSDP weight gather overlaps the first norm
        e.comm(OP_ALL_GATHER, ST_COMM_DP, c.layer_w, GROUP_DP, mb);
        const uint32_t ev = e.record(ST_COMM_DP, mb);
        e.compute(OP_RMSNORM, ST_COMPUTE_LO, c.norm, mb);
        e.wait(ST_COMPUTE_HI, ev, mb);
    } else {
        e.compute(OP_RMSNORM, ST_COMPUTE_LO, c.norm, mb);
    }
    e.compute(OP_GEMM, ST_COMPUTE_HI, c.qkv, mb);
    e.compute(OP_ATTENTION_FWD, ST_COMPUTE_HI, c.attn, mb);
    e.compute(OP_GEMM, ST_COMPUTE_HI, c.o, mb);
    if (c.tp > 1) tp_all_reduce(e, c, mb, true);
    e.compute(OP_RMSNORM, ST_COMPUTE_LO, c.norm, mb);
    const bool a2a = c.moe && c.ep > 1;
    if (a2a) expert_all_to_all(e, c, mb);
    e.compute(OP_GEMM, ST_COMPUTE_HI, c.mlp_up, mb);
    e.compute(OP_SWIGLU, ST_COMPUTE_LO, c.swiglu, mb);
    e.compute(OP_GEMM, ST_COMPUTE_HI, c.mlp_down, mb);
    if (a2a) expert_all_to_all(e, c, mb);
    if (c.tp > 1) tp_all_reduce(e, c, mb, false);
}

void layer_backward(Emitter& e, const Costs& c, uint16_t mb) {
    if (c.recompute > 0) e.compute(OP_GEMM, ST_COMPUTE_HI, c.recompute, mb);
    e.compute(OP_GEMM, ST_COMPUTE_HI, 2.0 * c.mlp_down, mb);
    e.compute(OP_GEMM, ST_COMPUTE_HI, 2.0 * c.mlp_up, mb);
    e.compute(OP_ATTENTION_BWD, ST_COMPUTE_HI, 2.0 * c.attn, mb);
    e.compute(OP_GEMM, ST_COMPUTE_HI, 2.0 * (c.qkv + c.o), mb);
    if (c.tp > 1) tp_all_reduce(e, c, mb, false);
    if (c.dp > 1) e.comm(OP_REDUCE_SCATTER, ST_COMM_DP, c.layer_w, GROUP_DP, mb);
}

void microbatch_forward(Emitter& e, const Costs& c, uint16_t mb) {
    if (c.stage > 0) {
        e.comm(OP_PIPE_RECV, ST_COMM_PP, c.pipe_msg, GROUP_PP, mb);
        e.sync(ST_COMM_PP, {ST_COMPUTE_HI, ST_COMPUTE_LO}, mb);
    }
    for (uint32_t l = 0; l < c.layers; ++l) layer_forward(e, c, mb);
    if (c.stage < c.last_stage) {
        e.sync(ST_COMPUTE_HI, {ST_COMM_PP}, mb);
        e.comm(OP_PIPE_SEND, ST_COMM_PP, c.pipe_msg, GROUP_PP, mb);
    } else {
        e.compute(OP_GEMM, ST_COMPUTE_HI, c.logits, mb);
        e.compute(OP_ELEMENTWISE, ST_COMPUTE_LO, c.loss, mb);
    }
}

void microbatch_backward(Emitter& e, const Costs& c, uint16_t mb) {
    if (c.stage == c.last_stage) {
        e.compute(OP_ELEMENTWISE, ST_COMPUTE_LO, c.loss, mb);
        e.compute(OP_GEMM, ST_COMPUTE_HI, 2.0 * c.logits, mb);
    } else {
        e.comm(OP_PIPE_RECV, ST_COMM_PP, c.pipe_msg, GROUP_PP, mb);
        e.sync(ST_COMM_PP, {ST_COMPUTE_HI}, mb);
    }
    for (uint32_t l = 0; l < c.layers; ++l) layer_backward(e, c, mb);
    if (c.stage > 0) {
        e.sync(ST_COMPUTE_HI, {ST_COMM_PP}, mb);
        e.comm(OP_PIPE_SEND, ST_COMM_PP, c.pipe_msg, GROUP_PP, mb);
    }
}

int failf(std::string* err, int code, const char* fmt, ...) {
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

}  // namespace

// Fills every header field that does not depend on the op table. Shared by v1 and v2.
int fill_plan_header(const Config& cfg, const Decomp& d, uint32_t rank, uint64_t ph, uint64_t th, uint32_t version,
                     Topology* topo_out, PlanHeader* h, std::string* err) {
    const ModelSpec& m = cfg.model;
    Topology topo = cfg.topo;
    if (int rc = topology_finalize(&topo, err); rc != OK) return rc;
    if (rank >= topo.world_size) return failf(err, ERR_INVALID, "rank %u >= world_size %u", rank, topo.world_size);
    const uint32_t stage = rank_stage(d, rank);
    const uint32_t base = m.num_layers / d.pp, rem = m.num_layers % d.pp;
    std::memset(h, 0, sizeof *h);
    h->magic = kPlanMagic;
    h->version = version;
    h->plan_hash = ph;
    h->topology_hash = th;
    h->global_rank = rank;
    h->world_size = topo.world_size;
    h->pipeline_stage = stage;
    h->num_stages = d.pp;
    h->tp = d.tp; h->dp = d.dp; h->ep = d.ep; h->cp = d.cp;
    h->microbatch = m.microbatch;
    h->grad_accum = m.grad_accum;
    h->num_microbatches = d.num_microbatches;
    h->seq_len = m.seq_len;
    h->hidden_size = m.hidden_size;
    h->layers_in_stage = base + (stage < rem ? 1 : 0);
    h->vpp = d.vpp ? d.vpp : 1;
    h->global_tokens_per_step = d.global_tokens;
    h->flops_per_token_useful = static_cast<uint64_t>(d.flops_per_token_useful);
    if (topo_out) *topo_out = topo;
    return OK;
}

int build_plan_v1(const Config& cfg, const Decomp& d, uint32_t rank, uint64_t ph, uint64_t th, Plan* out,
                  std::string* err) {
    const ModelSpec& m = cfg.model;
    Topology topo;
    *out = Plan{};
    if (int rc = fill_plan_header(cfg, d, rank, ph, th, 1, &topo, &out->hdr, err); rc != OK) return rc;
    PlanHeader& h = out->hdr;
    out->groups = rank_groups(d, topo, m.is_moe != 0, rank);

    Costs c{};
    c.tp = d.tp; c.dp = d.dp; c.ep = d.ep;
    c.stage = h.pipeline_stage; c.layers = h.layers_in_stage; c.last_stage = d.pp - 1;
    c.moe = m.is_moe != 0;
    const double pb = static_cast<double>(dtype_size(m.param_dtype));
    const double T = static_cast<double>(m.microbatch) * m.seq_len;
    const double hq = static_cast<double>(m.num_heads) * m.head_dim;
    const double hkv = static_cast<double>(m.num_kv_heads) * m.head_dim;
    const double tpf = d.tp;
    const double topk = c.moe ? m.moe_top_k : 1;
    c.qkv = 2.0 * T * m.hidden_size * (hq + 2.0 * hkv) / tpf;
    c.o = 2.0 * T * hq * m.hidden_size / tpf;
    c.attn = 2.0 * T * hq * m.seq_len / tpf;
    const double mlp_full = 2.0 * 3.0 * m.hidden_size * m.ffn_hidden * T * topk;
    const double mlp = c.moe ? mlp_full / (tpf * d.ep) : mlp_full / tpf;
    c.mlp_up = mlp * 2.0 / 3.0;
    c.mlp_down = mlp / 3.0;
    c.norm = 5.0 * T * m.hidden_size / tpf;
    c.swiglu = 4.0 * T * m.ffn_hidden * topk / tpf;
    c.logits = 2.0 * T * m.hidden_size * m.vocab_size / tpf;
    c.loss = 5.0 * T * m.vocab_size / tpf;
    c.recompute = m.recompute ? (c.qkv + c.o + c.mlp_up + c.mlp_down) : 0.0;
    c.opt = static_cast<double>(d.mem_param) / (pb > 0 ? pb : 1) * 18.0;
    const double act_bytes = T * m.hidden_size * pb;
    c.tp_msg = act_bytes / d.cp;
    c.pipe_msg = act_bytes / (tpf * d.cp);
    c.layer_w = static_cast<double>(layer_params_total(m)) / tpf / (c.moe ? d.ep : 1) * pb;
    c.a2a = c.moe ? T * m.moe_top_k * m.hidden_size * pb / tpf : 0.0;

    // The forward (and the backward) op sequence of a stage is the same for every microbatch but for the microbatch id
    // and the numbers of its events, which count up in emission order: each is emitted once and stamped per tick.
    Emitter fwd, bwd, e;
    microbatch_forward(fwd, c, 0);
    microbatch_backward(bwd, c, 0);
    const std::vector<Tick> ticks = schedule_1f1b(c.stage, d.pp, d.num_microbatches);
    size_t total = 8;
    for (const Tick& t : ticks) total += t.kind == 0 ? fwd.ops.size() : bwd.ops.size();
    e.ops.reserve(total);
    for (const Tick& t : ticks) {
        const Emitter& src = t.kind == 0 ? fwd : bwd;
        const size_t at = e.ops.size();
        e.ops.insert(e.ops.end(), src.ops.begin(), src.ops.end());
        for (size_t i = at; i < e.ops.size(); ++i) {
            Op& o = e.ops[i];
            o.aux1 = t.microbatch;
            if (o.kind == OP_EVENT_RECORD || o.kind == OP_EVENT_WAIT) o.aux0 += e.next_event;
        }
        e.next_event += src.next_event;
    }
    if (d.dp > 1) e.sync(ST_COMM_DP, {ST_COMPUTE_LO}, 0);
    e.compute(OP_OPTIMIZER, ST_COMPUTE_LO, c.opt, 0);

    // one descriptor per class, for memory accounting
    const uint64_t want[TC_COUNT] = {d.mem_param, d.mem_grad, d.mem_opt, d.mem_act, d.mem_comm, d.mem_ws};
    Arena arena;
    arena_layout(&arena, want);
    out->tensors.assign(TC_COUNT, TensorDesc{});
    for (uint16_t k = 0; k < TC_COUNT; ++k) {
        TensorDesc& t = out->tensors[k];
        t.nbytes = want[k];
        t.dtype = k == TC_OPTSTATE ? m.optim_dtype : m.param_dtype;
        t.tclass = k;
        t.shape_id = k;
    }
    arena_relocate(arena, out->tensors.data(), TC_COUNT);

    out->ops = std::move(e.ops);
    h.num_tensors = TC_COUNT;
    h.num_groups = static_cast<uint32_t>(out->groups.size());
    h.num_ops = static_cast<uint32_t>(out->ops.size());
    h.num_events = e.next_event;
    h.arena_bytes = arena.total;
    return OK;
}

// ------------------------------------------------------------------ plan files
void plan_class_bytes(const Plan& p, uint64_t out[TC_COUNT]) {
    uint64_t lo[TC_COUNT], hi[TC_COUNT];
    for (int c = 0; c < TC_COUNT; ++c) {
        lo[c] = ~0ull;
        hi[c] = 0;
    }
    for (const TensorDesc& t : p.tensors) {
        if (t.tclass >= TC_COUNT || t.nbytes == 0) continue;
        lo[t.tclass] = std::min(lo[t.tclass], t.offset);
        hi[t.tclass] = std::max(hi[t.tclass], t.offset + t.nbytes);
    }
    for (int c = 0; c < TC_COUNT; ++c) out[c] = hi[c] > lo[c] ? hi[c] - lo[c] : 0;
}

int plan_write(const std::string& path, const Plan& p) {
    if (p.hdr.magic != kPlanMagic) return ERR_INVALID;
    const std::string tmp = path + ".tmp";
    FILE* f = std::fopen(tmp.c_str(), "wb");
    if (!f) return ERR_IO;
    bool ok = write_all(f, &p.hdr, sizeof p.hdr) &&
              write_all(f, p.tensors.data(), p.tensors.size() * sizeof(TensorDesc)) &&
              write_all(f, p.groups.data(), p.groups.size() * sizeof(CommGroup)) &&
              write_all(f, p.ops.data(), p.ops.size() * sizeof(Op));
    if (ok && p.hdr.version >= 2) {
        ExecHeader xh = p.xhdr;
        xh.magic = kExecMagic;
        xh.num_exec = static_cast<uint32_t>(p.exec.size());
        xh.num_named = static_cast<uint32_t>(p.named.size());
        ok = write_all(f, &xh, sizeof xh) && write_all(f, &p.train, sizeof p.train) &&
             write_all(f, &p.model, sizeof p.model) &&
             write_all(f, p.exec.data(), p.exec.size() * sizeof(ExecOp)) &&
             write_all(f, p.named.data(), p.named.size() * sizeof(NamedTensor)) &&
             write_all(f, p.shapes.data(), p.shapes.size() * sizeof(uint32_t));
    }
    ok = (std::fclose(f) == 0) && ok;
    if (!ok || std::rename(tmp.c_str(), path.c_str()) != 0) {
        std::remove(tmp.c_str());
        return ERR_IO;
    }
    return OK;
}

int plan_read(const std::string& path, Plan* p) {
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return ERR_IO;
    *p = Plan{};
    int rc = OK;
    auto rd = [&](void* dst, size_t n) { return read_all(f, dst, n); };
    if (!rd(&p->hdr, sizeof p->hdr)) rc = ERR_IO;
    else if (p->hdr.magic != kPlanMagic || (p->hdr.version != 1 && p->hdr.version != 2)) rc = ERR_PLAN;
    if (rc == OK) {
        p->tensors.resize(p->hdr.num_tensors);
        p->groups.resize(p->hdr.num_groups);
        p->ops.resize(p->hdr.num_ops);
        if (!rd(p->tensors.data(), p->tensors.size() * sizeof(TensorDesc)) ||
            !rd(p->groups.data(), p->groups.size() * sizeof(CommGroup)) ||
            !rd(p->ops.data(), p->ops.size() * sizeof(Op)))
            rc = ERR_IO;
    }
    if (rc == OK && p->hdr.version >= 2) {
        if (!rd(&p->xhdr, sizeof p->xhdr) || p->xhdr.magic != kExecMagic) rc = ERR_PLAN;
        else {
            p->exec.resize(p->xhdr.num_exec);
            p->named.resize(p->xhdr.num_named);
            p->shapes.resize(static_cast<size_t>(p->hdr.num_tensors) * 4);
            if (!rd(&p->train, sizeof p->train) || !rd(&p->model, sizeof p->model) ||
                !rd(p->exec.data(), p->exec.size() * sizeof(ExecOp)) ||
                !rd(p->named.data(), p->named.size() * sizeof(NamedTensor)) ||
                !rd(p->shapes.data(), p->shapes.size() * sizeof(uint32_t)))
                rc = ERR_IO;
        }
    }
    std::fclose(f);
    if (rc != OK) *p = Plan{};
    return rc;
}

void plan_arena_breakdown(const Plan& p, uint64_t out_bytes[TC_COUNT]) {
    std::fill(out_bytes, out_bytes + TC_COUNT, 0);
    for (const TensorDesc& t : p.tensors)
        if (t.tclass < TC_COUNT) out_bytes[t.tclass] += t.nbytes;
}

}  // namespace cai
