// pipeline_sim.cc - joint replay of all stages of one pipeline.
//
// The single-plan replayer (runtime_sim.cc) walks one rank's op table and, like the reference
// (src/runtime.c:191-194), corrects for pipeline fill and drain with the closed formula step = busy / (1 - bubble).
// This file replays the plans of every stage of a pipeline together instead. The ops of all stages form one directed
// graph: the order of ops on a stream, the record / wait edges, and the messages between neighbouring stages (the k-th
// send of a stage towards a neighbour belongs to the neighbour's k-th receive from it). In executable plans a message is
// ONE node that starts when both sides are ready and occupies both streams for the transfer time, because an NCCL
// send returns only when the matching receive runs; in the reference's cost-only schedule sends do not wait (see
// below). The finish time of every op is a longest path, computed in one topological sweep. Fill, drain, uneven stages
// (the last one also runs the LM head and the loss) and transfer times then show up in the step time by themselves,
// and a schedule whose sends and receives cannot all meet leaves a cycle, which is reported as a deadlock.
//
// Host issue order is not modelled (the host is assumed to run ahead of the device, as in the single-plan replay).
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>

#include "backend.h"
#include "cai.h"
#include "plan.h"

namespace cai {

namespace {

struct Node {
    double dur = 0.0, start = 0.0;
    uint32_t indeg = 0;
    uint32_t stage = 0, op = 0;   // where it came from (the sending side for a transfer)
    uint16_t kind = 0, stream = 0;
    bool visible = false;         // appears in a timeline
};

struct Graph {
    std::vector<Node> nodes;
    std::vector<std::pair<uint32_t, uint32_t>> edges;  // from -> to
    uint32_t add(double dur) {
        Node n;
        n.dur = dur;
        nodes.push_back(n);
        return static_cast<uint32_t>(nodes.size() - 1);
    }
    void edge(int64_t from, uint32_t to) {
        if (from < 0) return;
        edges.emplace_back(static_cast<uint32_t>(from), to);
        nodes[to].indeg++;
    }
};

// Which neighbour a point-to-point op talks to. Executable plans name the peer stage; cost-only plans follow the 1F1B
// tick list: forward ticks receive from the stage below and send to the stage above, backward ticks the other way.
std::vector<int> p2p_peers(const Plan& p) {
    std::vector<int> peer(p.ops.size(), -1);
    const uint32_t s = p.hdr.pipeline_stage, last = p.hdr.num_stages - 1;
    if (p.hdr.version >= 2) {
        for (size_t i = 0; i < p.ops.size(); ++i) {
            const Op& o = p.ops[i];
            if ((o.kind == OP_PIPE_SEND || o.kind == OP_PIPE_RECV) && o.exec && o.exec <= p.exec.size())
                peer[i] = p.exec[o.exec - 1].i[4];
        }
        return peer;
    }
    const std::vector<Tick> ticks = schedule_1f1b(s, p.hdr.num_stages, p.hdr.num_microbatches);
    const uint32_t per_tick = (s > 0 ? 1u : 0u) + (s < last ? 1u : 0u);
    uint32_t seen = 0;
    for (size_t i = 0; i < p.ops.size() && per_tick; ++i) {
        const Op& o = p.ops[i];
        if (o.kind != OP_PIPE_SEND && o.kind != OP_PIPE_RECV) continue;
        const uint32_t t = seen++ / per_tick;
        if (t >= ticks.size()) break;
        const bool fwd = ticks[t].kind == 0;
        const bool up = (o.kind == OP_PIPE_SEND) == fwd;   // forward sends and backward receives involve the stage above
        peer[i] = up ? static_cast<int>(s) + 1 : static_cast<int>(s) - 1;
    }
    return peer;
}

}  // namespace

int replay_pipeline(const std::vector<const Plan*>& stages, const Topology& topo, Backend* be, PipelineResult* out,
                    std::string* err) {
    auto fail = [&](int code, const std::string& why) {
        if (err) *err = why;
        return code;
    };
    const uint32_t S = static_cast<uint32_t>(stages.size());
    if (!S) return fail(ERR_INVALID, "no stages");
    for (uint32_t s = 0; s < S; ++s) {
        const PlanHeader& h = stages[s]->hdr;
        if (h.num_stages != S || h.pipeline_stage != s)
            return fail(ERR_PLAN, "plan " + std::to_string(s) + " is stage " + std::to_string(h.pipeline_stage) + " of " +
                                      std::to_string(h.num_stages) + ", expected stage " + std::to_string(s) + " of " + std::to_string(S));
        if (h.plan_hash != stages[0]->hdr.plan_hash || h.topology_hash != stages[0]->hdr.topology_hash)
            return fail(ERR_PLAN, "the stages were compiled from different configurations (hash mismatch)");
    }
    Graph g;
    // Executable plans talk through NCCL, whose send returns when the matching receive runs: one shared node. The
    // cost-only schedule of the reference puts both directions on one in-order stream and relies on sends that do not
    // wait for the receiver (with a rendezvous its warm-up sends and the first gradient send of the stage above would
    // wait for each other): there a send costs its own stream its duration, and the receive starts once the receiver
    // is ready and the sender has started.
    const bool rendezvous = stages[0]->hdr.version >= 2;
    struct Msg { int64_t node = -1, send_pred = -1, recv_node = -1; bool has_send = false; };
    std::map<std::pair<int, int>, std::vector<Msg>> channel;      // (from stage, to stage) -> messages in issue order
    std::map<std::pair<int, int>, uint32_t> sent, received;
    out->stages.assign(S, PipelineResult::Stage{});
    std::vector<std::vector<int64_t>> tails(S, std::vector<int64_t>(ST_COUNT, -1));

    for (uint32_t s = 0; s < S; ++s) {
        const Plan& p = *stages[s];
        const std::vector<int> peer = p2p_peers(p);
        if (be->load_plan)      // a backend that prices by kernel record binds the stage's exec table first
            if (int rc = be->load_plan(be, p, std::string(), p.hdr.global_rank, p.hdr.world_size); rc != OK) return fail(rc, "backend refused the plan of stage " + std::to_string(s));
        std::vector<int64_t> event(p.hdr.num_events ? p.hdr.num_events : 1, -1);
        std::vector<int64_t>& last = tails[s];
        const CommGroup* by_id[16] = {};
        for (const CommGroup& c : p.groups)
            if (c.group_id < 16) by_id[c.group_id] = &c;
        PipelineResult::Stage& st = out->stages[s];
        for (uint32_t i = 0; i < p.ops.size(); ++i) {
            const Op& op = p.ops[i];
            if (op.stream_id >= ST_COUNT) return fail(ERR_PLAN, "op on an unknown stream");
            const uint16_t q = op.stream_id;
            if (op.kind == OP_EVENT_RECORD) {
                if (op.aux0 >= event.size()) return fail(ERR_PLAN, "event id out of range");
                event[op.aux0] = last[q];
                continue;
            }
            if (op.kind == OP_EVENT_WAIT) {
                if (op.aux0 >= event.size()) return fail(ERR_DEPENDENCY, "wait on an unknown event");
                if (event[op.aux0] < 0) continue;            // nothing was in flight on the recording stream
                const uint32_t w = g.add(0.0);
                g.edge(last[q], w);
                g.edge(event[op.aux0], w);
                last[q] = w;
                continue;
            }
            const CommGroup* grp = nullptr;
            if (op_is_comm(op.kind) || op.kind >= OP_COUNT_V1) {
                grp = op.aux0 < 16 ? by_id[op.aux0] : nullptr;
                if (!grp && op_is_comm(op.kind)) return fail(ERR_PLAN, "communication op without its group");
            }
            const double dur = be->op_seconds(be, topo, op, grp);
            st.stream_busy[q] += dur;
            if (be->op_sm_share) st.sm_work_s += dur * be->op_sm_share(be, topo, op, grp);
            auto fresh = [&](double d) {
                const uint32_t n = g.add(d);
                Node& t = g.nodes[n];
                t.stage = s; t.op = i; t.kind = op.kind; t.stream = q; t.visible = true;
                return n;
            };
            uint32_t n;
            if ((op.kind == OP_PIPE_SEND || op.kind == OP_PIPE_RECV) && S > 1) {
                const int other = peer[i];
                if (other < 0 || other >= static_cast<int>(S) || (other != static_cast<int>(s) + 1 && other + 1 != static_cast<int>(s)))
                    return fail(ERR_PLAN, "stage " + std::to_string(s) + ": point-to-point op " + std::to_string(i) + " names no neighbouring stage");
                const bool send = op.kind == OP_PIPE_SEND;
                const std::pair<int, int> key = send ? std::make_pair(static_cast<int>(s), other) : std::make_pair(other, static_cast<int>(s));
                const uint32_t k = (send ? sent[key] : received[key])++;
                std::vector<Msg>& ch = channel[key];
                if (k >= ch.size()) ch.resize(k + 1);
                Msg& m = ch[k];
                if (rendezvous) {
                    if (m.node < 0) m.node = fresh(dur);
                    n = static_cast<uint32_t>(m.node);
                    Node& t = g.nodes[n];
                    t.dur = std::max(t.dur, dur);
                    if (send) { t.stage = s; t.op = i; t.kind = op.kind; t.stream = q; }   // timelines show it on the sender
                } else {
                    n = fresh(dur);
                    if (send) { m.has_send = true; m.send_pred = last[q]; }
                    else m.recv_node = n;
                }
            } else {
                n = fresh(dur);
            }
            g.edge(last[q], n);
            last[q] = n;
        }
    }
    for (const auto& kv : channel) {
        const uint32_t a = sent.count(kv.first) ? sent[kv.first] : 0, b = received.count(kv.first) ? received[kv.first] : 0;
        if (a != b)
            return fail(ERR_DEPENDENCY, "stage " + std::to_string(kv.first.first) + " sends " + std::to_string(a) + " messages to stage " +
                                            std::to_string(kv.first.second) + ", which receives " + std::to_string(b));
        if (!rendezvous)
            for (const Msg& m : kv.second)
                if (m.has_send && m.recv_node >= 0) g.edge(m.send_pred, static_cast<uint32_t>(m.recv_node));
    }

    // longest paths in one topological sweep (Kahn)
    const uint32_t N = static_cast<uint32_t>(g.nodes.size());
    std::vector<uint32_t> head(N + 1, 0), succ(g.edges.size());
    for (const auto& e : g.edges) head[e.first + 1]++;
    for (uint32_t i = 0; i < N; ++i) head[i + 1] += head[i];
    {
        std::vector<uint32_t> fill(head.begin(), head.end() - 1);
        for (const auto& e : g.edges) succ[fill[e.first]++] = e.second;
    }
    std::vector<uint32_t> ready;
    ready.reserve(N);
    for (uint32_t i = 0; i < N; ++i)
        if (!g.nodes[i].indeg) ready.push_back(i);
    uint32_t done = 0;
    while (done < ready.size()) {
        const uint32_t n = ready[done++];
        const double fin = g.nodes[n].start + g.nodes[n].dur;
        for (uint32_t e = head[n]; e < head[n + 1]; ++e) {
            Node& t = g.nodes[succ[e]];
            t.start = std::max(t.start, fin);
            if (--t.indeg == 0) ready.push_back(succ[e]);
        }
    }
    if (done != N) {
        // name one op that never became ready: it sits on a cycle of sends and receives waiting for each other
        for (uint32_t i = 0; i < N; ++i)
            if (g.nodes[i].indeg && g.nodes[i].visible)
                return fail(ERR_DEPENDENCY, "deadlock: stage " + std::to_string(g.nodes[i].stage) + " op " + std::to_string(g.nodes[i].op) + " (" +
                                                op_name(g.nodes[i].kind) + ") can never start; sends and receives of neighbouring stages wait for each other");
        return fail(ERR_DEPENDENCY, "deadlock between the stages");
    }

    out->step_time_s = 0.0;
    for (uint32_t s = 0; s < S; ++s) {
        PipelineResult::Stage& st = out->stages[s];
        for (int q = 0; q < ST_COUNT; ++q)
            if (tails[s][q] >= 0) st.finish_s = std::max(st.finish_s, g.nodes[tails[s][q]].start + g.nodes[tails[s][q]].dur);
        // streams overlap only as far as their kernels leave SMs to each other (backends that know the share): a stage
        // cannot finish before the SM time of all its kernels has been served
        out->step_time_s = std::max(out->step_time_s, std::max(st.finish_s, st.sm_work_s));
    }
    for (PipelineResult::Stage& st : out->stages)
        st.idle_hi = out->step_time_s > 0 ? 1.0 - std::min(1.0, st.stream_busy[ST_COMPUTE_HI] / out->step_time_s) : 0.0;
    const PlanHeader& h = stages[0]->hdr;
    out->bubble_formula = pipeline_bubble_interleaved(h.num_stages, h.num_microbatches, h.vpp ? h.vpp : 1);
    out->tokens_per_s = out->step_time_s > 0 ? h.global_tokens_per_step / out->step_time_s : 0.0;
    const double useful = static_cast<double>(h.global_tokens_per_step) * static_cast<double>(h.flops_per_token_useful) / h.world_size;
    out->mfu = out->step_time_s > 0 ? useful / (topo.gpu_flops_bf16 * out->step_time_s) : 0.0;
    out->trace.clear();
    if (out->want_trace) {
        out->trace.reserve(N);
        for (const Node& n : g.nodes)
            if (n.visible) out->trace.push_back({n.stage, {n.op, n.kind, n.stream, n.start, n.start + n.dur, stages[n.stage]->ops[n.op].bytes, stages[n.stage]->ops[n.op].flops}});
    }
    return OK;
}

}  // namespace cai

using namespace cai;

extern "C" int cai_pipeline_replay(const char* const* plan_paths, uint32_t n_stages, const char* topology_path, uint32_t backend,
                                   const char* calibration_path, const char* trace_json_path, cai_pipeline_stats_t* out,
                                   char* err, size_t errlen) {
    auto fail = [&](int code, const std::string& why) {
        if (err && errlen) std::snprintf(err, errlen, "%s", why.c_str());
        return code;
    };
    if (!plan_paths || !n_stages || !topology_path || !out) return fail(ERR_INVALID, "missing argument");
    if (n_stages > CAI_MAX_PIPELINE_STAGES) return fail(ERR_INVALID, "more stages than the result structure holds");
    Topology topo;
    std::string why;
    if (int rc = topology_read(topology_path, &topo); rc != OK) return fail(rc, std::string("cannot read topology ") + topology_path);
    if (topology_finalize(&topo, &why) != OK) return fail(ERR_TOPOLOGY, why);
    std::vector<Plan> plans(n_stages);
    std::vector<const Plan*> ptrs;
    for (uint32_t s = 0; s < n_stages; ++s) {
        if (int rc = plan_read(plan_paths[s], &plans[s]); rc != OK) return fail(rc, std::string("cannot read plan ") + plan_paths[s]);
        if (plans[s].hdr.topology_hash != topology_hash(topo)) return fail(ERR_TOPOLOGY, std::string(plan_paths[s]) + " was compiled for a different topology");
        ptrs.push_back(&plans[s]);
    }
    struct Closer { void operator()(Backend* b) const { if (b) b->destroy(b); } };
    std::unique_ptr<Backend, Closer> be;
    if (backend == CAI_BACKEND_CALIBRATED) {
        be.reset(backend_calibrated_create(calibration_path, &why));
        if (!be) return fail(ERR_BACKEND, "calibrated backend: " + why);
    } else if (backend == CAI_BACKEND_ANALYTIC || backend == CAI_BACKEND_DEFAULT) {
        be.reset(backend_analytic_create());
    } else {
        return fail(ERR_INVALID, "the joint replay needs a pricing backend (analytic or calibrated)");
    }
    PipelineResult r;
    r.want_trace = trace_json_path != nullptr;
    if (int rc = replay_pipeline(ptrs, topo, be.get(), &r, &why); rc != OK) return fail(rc, why);
    std::memset(out, 0, sizeof *out);
    out->n_stages = n_stages;
    out->step_time_s = r.step_time_s;
    out->bubble_formula = r.bubble_formula;
    out->tokens_per_s = r.tokens_per_s;
    out->mfu = r.mfu;
    double busiest = 0.0;
    for (uint32_t s = 0; s < n_stages; ++s) {
        out->stage_finish_s[s] = r.stages[s].finish_s;
        out->stage_busy_hi_s[s] = r.stages[s].stream_busy[ST_COMPUTE_HI];
        out->stage_idle_hi[s] = r.stages[s].idle_hi;
        out->stage_sm_busy_s[s] = r.stages[s].sm_work_s;
        busiest = std::max(busiest, r.stages[s].stream_busy[ST_COMPUTE_HI]);
    }
    // share of the step the busiest stage's main compute stream stands still: what fill, drain and transfers cost
    out->bubble_replayed = r.step_time_s > 0 ? 1.0 - std::min(1.0, busiest / r.step_time_s) : 0.0;
    if (trace_json_path) {
        FILE* f = std::fopen(trace_json_path, "w");
        if (!f) return fail(ERR_IO, std::string("cannot write ") + trace_json_path);
        std::fprintf(f, "{\"displayTimeUnit\": \"ms\", \"traceEvents\": [\n");
        for (uint32_t s = 0; s < n_stages; ++s) {
            std::fprintf(f, "{\"ph\": \"M\", \"pid\": %u, \"name\": \"process_name\", \"args\": {\"name\": \"stage %u (rank %u)\"}},\n", s, s,
                         plans[s].hdr.global_rank);
            for (int q = 0; q < ST_COUNT; ++q)
                std::fprintf(f, "{\"ph\": \"M\", \"pid\": %u, \"tid\": %d, \"name\": \"thread_name\", \"args\": {\"name\": \"%s\"}},\n", s, q,
                             stream_name(static_cast<uint16_t>(q)));
        }
        for (size_t i = 0; i < r.trace.size(); ++i) {
            const cai_trace_rec_t& t = r.trace[i].rec;
            std::fprintf(f, "{\"ph\": \"X\", \"pid\": %u, \"tid\": %u, \"name\": \"%s\", \"ts\": %.4f, \"dur\": %.4f, "
                            "\"args\": {\"op\": %u, \"microbatch\": %u, \"bytes\": %llu, \"flops\": %llu}}%s\n",
                         r.trace[i].stage, t.stream, op_name(t.kind), t.start_s * 1e6, (t.end_s - t.start_s) * 1e6, t.op_index,
                         plans[r.trace[i].stage].ops[t.op_index].aux1, (unsigned long long)t.bytes, (unsigned long long)t.flops,
                         i + 1 < r.trace.size() ? "," : "");
        }
        std::fprintf(f, "]}\n");
        std::fclose(f);
    }
    return OK;
}
