// backend_calibrated.cc - a pricing backend whose costs are fitted to measurements on B200s.
//
// The analytic backend keeps the reference's model (FLOPs over the datasheet peak, bytes over the link figure:
// src/backend_cpu.c:28-49), which is what its published predictions are made of. This backend prices the same
// executable plans with what the kernels of this repository were measured to do, so that a configuration can be
// judged without a GPU: the replayer (runtime_sim.cc) walks the op table over the six stream clocks as before, and
// additionally keeps the step from being shorter than the GPU-filling work of all streams together (two kernels that
// each fill the GPU do not speed each other up by sitting on different streams).
//
// Model per kernel (constants: `Calibration`, overridable from a key = value file; sources in the comments there):
//   GEMM            launch + waves * (tile overhead + tile FLOPs / per-SM rate), 128 x 256 (or 128 x 128) tiles on 148 SMs,
//                   a lower rate for transposed-A products (weight gradients)
//   attention       per-CTA critical path: steps = max(all steps / SMs, longest CTA) * time per 128 x 128 step
//   pointwise       per-kernel fixed cost + operand bytes * per-kernel microseconds per MB
//   fused TP ops    launch + max(GEMM on the SMs left beside the copy CTAs, wire bytes / measured rate under all-to-all
//                   load for the group size) (+ the own-row tail of the reduce-scatter)
//   NCCL, p2p       latency + bytes / rate
// Needs a version-2 plan (kernel records and shapes); version-1 plans fall back to the analytic cost.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>

#include "backend.h"

namespace cai {
namespace {

struct PointCost {
    double fixed_us;
    double us_per_mb;
};

struct Calibration {
    int sms = 148;
    // GEMM, fitted to the per-op CUDA-event times of the headline config inside a step on one GPU (fifteen shapes,
    // fit error <= 13 %): [0] A not transposed, [1] A transposed (weight-gradient form)
    double gemm_launch_us = 12.0;
    double gemm_tile_us[2] = {0.5, 4.0};
    double gemm_sm_flops[2] = {7.9e12, 6.9e12};
    // fp8 block-scaled GEMM: 1708 against 1361 TFLOP/s at 8192^3
    double fp8_speedup = 1.25;
    // attention, microseconds per 128 x 128 step of one CTA (16 / 8 heads, seq 4096, batches 1 and 4)
    double attn_fwd_step_us = 1.64, attn_fwd_fixed_us = 20.0;
    double attn_dkdv_step_us = 3.08, attn_dq_step_us = 2.75, attn_bwd_fixed_us = 10.0;
    // fused tensor-parallel kernels: bytes a GPU moves per second while every member pulls and pushes at once
    // (steady-state chains on 2 / 4 / 8 GPUs), copy CTAs of the all-gather form, tail of the reduce-scatter form
    double link_rate[4] = {0.60e12, 0.60e12, 0.45e12, 0.35e12};  // group size 1-2, 2, 4, 8
    int ag_copy_ctas = 16;
    double rs_tail_us = 35.0;
    double fused_launch_us = 15.0;
    double fused_min_share = 0.6;
    // NCCL collectives and p2p next to compute
    double nccl_latency_us = 20.0;
    double nccl_rate = 0.60e12;   // bytes per GPU and second of ring collectives of 17-120 MB (NCCL arms of the chains)
    // pointwise kernels (two points each: one GPU and eight GPUs of the headline config)
    PointCost point_default = {8.0, 0.20};
    PointCost rmsnorm_fwd = {9.3, 0.143}, rmsnorm_bwd = {30.0, 0.327}, rope = {7.9, 0.262}, swiglu = {7.6, 0.158},
              adamw = {10.0, 0.238}, cross_entropy = {10.0, 0.20}, embed = {15.0, 0.60};
};

bool set_key(Calibration* c, const std::string& k, double v) {
    struct Entry { const char* name; double* dst; };
    Entry table[] = {
        {"gemm_launch_us", &c->gemm_launch_us}, {"gemm_tile_us", &c->gemm_tile_us[0]}, {"gemm_tile_us_ta", &c->gemm_tile_us[1]},
        {"gemm_sm_flops", &c->gemm_sm_flops[0]}, {"gemm_sm_flops_ta", &c->gemm_sm_flops[1]}, {"fp8_speedup", &c->fp8_speedup},
        {"attn_fwd_step_us", &c->attn_fwd_step_us}, {"attn_fwd_fixed_us", &c->attn_fwd_fixed_us},
        {"attn_dkdv_step_us", &c->attn_dkdv_step_us}, {"attn_dq_step_us", &c->attn_dq_step_us},
        {"attn_bwd_fixed_us", &c->attn_bwd_fixed_us}, {"link_rate_2", &c->link_rate[1]}, {"link_rate_4", &c->link_rate[2]},
        {"link_rate_8", &c->link_rate[3]}, {"rs_tail_us", &c->rs_tail_us}, {"fused_launch_us", &c->fused_launch_us},
        {"nccl_latency_us", &c->nccl_latency_us}, {"nccl_rate", &c->nccl_rate}, {"fused_min_share", &c->fused_min_share},
    };
    for (const Entry& e : table)
        if (k == e.name) {
            *e.dst = v;
            return true;
        }
    struct PEntry { const char* name; PointCost* dst; };
    PEntry points[] = {{"pointwise", &c->point_default}, {"rmsnorm_fwd", &c->rmsnorm_fwd}, {"rmsnorm_bwd", &c->rmsnorm_bwd},
                       {"rope", &c->rope}, {"swiglu", &c->swiglu}, {"adamw", &c->adamw}, {"cross_entropy", &c->cross_entropy},
                       {"embed", &c->embed}};
    for (const PEntry& e : points) {   // <kernel>_fixed_us, <kernel>_us_per_mb
        const std::string n = e.name;
        if (k == n + "_fixed_us") { e.dst->fixed_us = v; return true; }
        if (k == n + "_us_per_mb") { e.dst->us_per_mb = v; return true; }
    }
    if (k == "sms") { c->sms = static_cast<int>(v); return true; }
    if (k == "ag_copy_ctas") { c->ag_copy_ctas = static_cast<int>(v); return true; }
    return false;
}

struct CalibratedImpl {
    Calibration c;
    std::vector<ExecOp> exec;
    std::vector<TensorDesc> tensors;
    uint32_t capacity_x100 = 200;
};

double gemm_seconds(const Calibration& c, double M, double N, double K, bool ta, int sms, double* share) {
    const int cls = ta ? 1 : 0;
    const double bn = (static_cast<long long>(N) % 256 == 0) ? 256.0 : 128.0;
    const double tiles = std::ceil(M / 128.0) * std::ceil(N / bn);
    const double waves = std::max(1.0, std::ceil(tiles / sms));
    if (share) *share = std::min(1.0, tiles / (waves * c.sms));
    return (c.gemm_launch_us + waves * (c.gemm_tile_us[cls] + 2.0 * 128.0 * bn * K / c.gemm_sm_flops[cls] * 1e6)) * 1e-6;
}

double operand_mb(const CalibratedImpl& im, const ExecOp& x) {
    double b = 0.0;
    for (int t : x.t)
        if (t >= 0 && static_cast<size_t>(t) < im.tensors.size()) b += static_cast<double>(im.tensors[t].nbytes);
    return b / 1e6;
}

double link_rate(const Calibration& c, uint32_t n) { return c.link_rate[n <= 2 ? 1 : n <= 4 ? 2 : 3]; }

// Seconds and the share of the GPU's SMs the op keeps busy while it runs.
double price(const CalibratedImpl& im, const Topology& topo, const Op& op, const CommGroup* g, double* share) {
    const Calibration& c = im.c;
    *share = 1.0;
    if (!op.exec || op.exec > im.exec.size()) {
        *share = op_is_compute(op.kind) ? 1.0 : 0.0;
        return analytic_op_seconds(topo, op, g);
    }
    const ExecOp& x = im.exec[op.exec - 1];
    const uint32_t n = g ? g->size : 1;
    auto point = [&](const PointCost& pc) { return (pc.fixed_us + operand_mb(im, x) * pc.us_per_mb) * 1e-6; };
    switch (x.kernel) {
    case K_GEMM: {
        double M = x.i[0], N = x.i[1], K = x.i[2];
        if (x.flags & 0x100) {
            // grouped expert GEMM: one launch over all local experts' slabs (op.flops counts every slab row); tiles past a
            // slab's token count are skipped, and with balanced routing a slab is filled to 1 / capacity factor
            const double experts = std::max(1.0, std::round(static_cast<double>(op.flops) / (2.0 * M * N * K)));
            const double live = std::min(1.0, 100.0 / std::max(100u, im.capacity_x100));
            if (x.i[4] == 2050) K *= live;   // weight-gradient form: the ragged dimension is K
            else M *= live;
            if (x.i[4] == 2050) return experts * gemm_seconds(c, M, N, K, x.flags & 1, c.sms, share);
            M *= experts;
        }
        return gemm_seconds(c, M, N, K, x.flags & 1, c.sms, share);
    }
    case K_GEMM_FP8:
        return gemm_seconds(c, x.i[0], x.i[1], x.i[2], false, c.sms, share) / c.fp8_speedup;
    case K_AG_GEMM: case K_GEMM_RS: {
        const bool ag = x.kernel != K_GEMM_RS;
        const double compute = gemm_seconds(c, x.i[0], x.i[1], x.i[2], x.flags & 1, ag ? c.sms - c.ag_copy_ctas : c.sms, nullptr);
        const double wire = n > 1 ? (n - 1.0) / n * static_cast<double>(op.bytes) / link_rate(c, n) : 0.0;
        const double tail = (x.kernel == K_GEMM_RS && n > 1) ? c.rs_tail_us * 1e-6 : 0.0;
        const double dur = c.fused_launch_us * 1e-6 + std::max(compute, wire) + tail;
        // a transfer-bound call leaves issue slots and memory bandwidth to kernels of other streams while it waits
        *share = compute >= wire ? 1.0 : std::max(c.fused_min_share, compute / wire);
        return dur;
    }
    case K_ATTN_FWD: case K_ATTN_BWD: {
        const double B = x.i[0], S = x.i[1], nh = x.i[2], nkv = std::max(1, x.i[3]);
        const double nq = S / 128.0, tri = nq * (nq + 1.0) / 2.0, rep = nh / nkv;
        if (x.kernel == K_ATTN_FWD) {
            const double steps = std::max(B * nh * tri / c.sms, nq);
            *share = std::min(1.0, B * nh * nq / c.sms);
            return (c.attn_fwd_fixed_us + steps * c.attn_fwd_step_us) * 1e-6;
        }
        // parts (flags): bit 0 delta, bit 1 dK / dV, bit 2 dQ; 0 means all three
        const int parts = (x.flags & 7) ? (x.flags & 7) : 7;
        double t = c.attn_bwd_fixed_us;
        if (parts & 2) {
            // one CTA per (kv tile, kv group) sweeping the group's heads, or per query head when that grid fits the SMs
            const bool split = rep > 1 && B * nkv * nq < c.sms && B * nh * nq <= c.sms;
            const double longest = (split ? 1.0 : rep) * nq;
            t += std::max(B * nh * tri / c.sms, longest) * c.attn_dkdv_step_us;
        }
        if (parts & 4) t += std::max(B * nh * tri / c.sms, nq) * c.attn_dq_step_us;
        *share = std::min(1.0, B * nh * nq / c.sms);
        return t * 1e-6;
    }
    case K_RMSNORM_FWD: return point(c.rmsnorm_fwd);
    case K_RMSNORM_BWD: return point(c.rmsnorm_bwd);
    case K_ROPE: return point(c.rope);
    case K_SWIGLU_FWD: case K_SWIGLU_BWD: return point(c.swiglu);
    case K_ADAMW: return point(c.adamw);
    case K_CROSS_ENTROPY: case K_CROSS_ENTROPY_TP: return point(c.cross_entropy);
    case K_EMBED_FWD: case K_EMBED_BWD: return point(c.embed);
    case K_FSDP_AG_GEMM: {
        // ZeRO-3 parameter gather of one group (op.bytes = what crosses the links); flag 1: the copy CTAs ride in the
        // first GEMM that reads the group, which measured slower than the transfer alone (482 us against 406 us of
        // all-gather + GEMM at 2 GPUs for a 50 MB group), priced here as twice the transfer
        const double wire = static_cast<double>(op.bytes) / link_rate(c, n);
        *share = 0.2;
        return c.fused_launch_us * 1e-6 + ((x.flags & 1) ? 2.0 : 1.0) * wire;
    }
    case K_RS_ADAMW: {
        // reduce-scatter + AdamW (+ parameter all-gather) over the data-parallel group. op.flops = 18 per element of
        // the owned slice: the slice's optimizer traffic, and (n - 1) x 6 bytes per owned element over the links
        // (fp32 gradients in, bf16 parameters out). 1.72 ms for 256 Mi parameters on 2 GPUs.
        const double owned = static_cast<double>(op.flops) / 18.0;
        const double opt = (c.adamw.fixed_us + owned * 18.0 / 1e6 * c.adamw.us_per_mb) * 1e-6;
        const double wire = n > 1 ? (n - 1.0) * owned * 6.0 / link_rate(c, n) : 0.0;
        *share = 0.45;  // launched on a slice of the SMs beside the backward
        return c.fused_launch_us * 1e-6 + std::max(opt, wire) + 0.5 * std::min(opt, wire);
    }
    case K_NCCL_ALL_REDUCE: case K_NCCL_REDUCE_SCATTER: case K_NCCL_ALL_GATHER: case K_NCCL_ALL_TO_ALL:
    case K_NCCL_SEND: case K_NCCL_RECV: {
        *share = 0.15;  // NCCL's own CTAs
        // op.bytes: the whole tensor for an all-reduce, this rank's shard for the others
        double wire = static_cast<double>(op.bytes);
        if (x.kernel == K_NCCL_ALL_REDUCE) wire *= n > 1 ? 2.0 * (n - 1.0) / n : 0.0;
        else if (x.kernel != K_NCCL_SEND && x.kernel != K_NCCL_RECV) wire *= n > 1 ? n - 1.0 : 0.0;
        return c.nccl_latency_us * 1e-6 + wire / c.nccl_rate;
    }
    case K_MOE_DISPATCH_GEMM: case K_MOE_GEMM_COMBINE: {
        const double wire = n > 1 ? (n - 1.0) / n * static_cast<double>(op.bytes) / link_rate(c, n) : 0.0;
        return c.fused_launch_us * 1e-6 + std::max(point(c.point_default), wire);
    }
    default:
        *share = 0.5;
        return point(c.point_default);
    }
}

double calibrated_op_seconds(Backend* be, const Topology& topo, const Op& op, const CommGroup* g) {
    double share;
    return price(*static_cast<CalibratedImpl*>(be->impl), topo, op, g, &share);
}

double calibrated_sm_share(Backend* be, const Topology& topo, const Op& op, const CommGroup* g) {
    double share = 0.0;
    price(*static_cast<CalibratedImpl*>(be->impl), topo, op, g, &share);
    return share;
}

int calibrated_load_plan(Backend* be, const Plan& plan, const std::string&, uint32_t, uint32_t) {
    auto* im = static_cast<CalibratedImpl*>(be->impl);
    im->exec = plan.exec;
    im->tensors = plan.tensors;
    im->capacity_x100 = plan.train.moe_capacity_factor_x100 ? plan.train.moe_capacity_factor_x100 : 200;
    return OK;
}

void calibrated_destroy(Backend* be) {
    delete static_cast<CalibratedImpl*>(be->impl);
    delete be;
}

}  // namespace

Backend* backend_calibrated_create(const char* calibration_path, std::string* why) {
    auto im = new CalibratedImpl();
    if (calibration_path && *calibration_path) {
        std::ifstream f(calibration_path);
        if (!f) {
            if (why) *why = std::string("cannot read calibration file ") + calibration_path;
            delete im;
            return nullptr;
        }
        std::string line;
        int lineno = 0;
        while (std::getline(f, line)) {
            ++lineno;
            const size_t hash = line.find('#');
            if (hash != std::string::npos) line.resize(hash);
            const size_t eq = line.find('=');
            if (eq == std::string::npos) continue;
            auto trim = [](std::string s) {
                const size_t a = s.find_first_not_of(" \t\r"), b = s.find_last_not_of(" \t\r");
                return a == std::string::npos ? std::string() : s.substr(a, b - a + 1);
            };
            const std::string k = trim(line.substr(0, eq)), v = trim(line.substr(eq + 1));
            char* end = nullptr;
            const double val = std::strtod(v.c_str(), &end);
            if (k.empty() || end == v.c_str() || !set_key(&im->c, k, val)) {
                if (why) {
                    std::ostringstream o;
                    o << calibration_path << ":" << lineno << ": unknown key or bad value '" << k << "'";
                    *why = o.str();
                }
                delete im;
                return nullptr;
            }
        }
    }
    auto be = new Backend();
    be->name = "calibrated";
    be->impl = im;
    be->op_seconds = calibrated_op_seconds;
    be->op_sm_share = calibrated_sm_share;
    be->load_plan = calibrated_load_plan;
    be->run_step = nullptr;
    be->snapshot = nullptr;
    be->restore = nullptr;
    be->sync = nullptr;
    be->destroy = calibrated_destroy;
    return be;
}

}  // namespace cai
