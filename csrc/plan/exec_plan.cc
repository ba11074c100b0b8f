// exec_plan.cc - the version-2 plan: an executable schedule for one rank.
//
// Where the reference's op table only carries costs (src/model.c:441-539), this builder lays out
// every tensor of the rank in the static arena and emits, in 1F1B order over the six streams, one
// record per kernel launch with its operands. It also closes the gaps the reference schedule
// has for real execution: norm / SwiGLU / embedding backward ops exist, dependent pointwise ops run
// on the stream of their producer instead of racing on compute_lo, and every cross-stream edge
// has a record/wait pair (verify_hazards proves it).
//
// Parallel layout of a dense decoder under tensor parallelism (Megatron with sequence
// parallelism): the residual stream is sharded by rows ([T/tp, H] per rank); QKV and gate/up are
// column-parallel (all-gather of the normalised rows feeds the GEMM), the attention output and
// down projections are row-parallel (GEMM feeds a reduce-scatter that also adds the residual).
// In comm mode "fused" those pairs are single kernels (OP_AG_GEMM / OP_GEMM_RS); in mode
// "baseline" they are NCCL collectives next to plain GEMMs.
#include <algorithm>
#include <array>
#include <cmath>
#include <cstdarg>
#include <cstring>
#include <map>

#include "../comm/signals.h"
#include "plan.h"

namespace cai {

int fill_plan_header(const Config& cfg, const Decomp& d, uint32_t rank, uint64_t ph, uint64_t th, uint32_t version,
                     Topology* topo_out, PlanHeader* h, std::string* err);

namespace {

constexpr uint64_t kTensorAlign = 1024;
constexpr uint64_t kSegmentGuardBytes = 1024;
constexpr uint32_t kFlatAlignElems = 512;  // parameters start on multiples of this many elements

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

ExecOp xop(uint16_t kernel, uint16_t flags = 0) {
    ExecOp x{};
    x.kernel = kernel;
    x.flags = flags;
    for (int& t : x.t) t = -1;
    return x;
}

struct Param {
    int w = -1, g = -1;      // bf16 weight, fp32 gradient
    uint32_t rows = 0, cols = 0;
};

struct LayerParams { Param g1, wqkv, wo, g2, wgu, wd, wr; };  // MoE: wgu / wd stack the local experts, wr is the router

// Saved activations of one layer for one in-flight microbatch.
struct LayerActs {
    int x, rstd1, xn1, qkv, ao, lse, hmid, rstd2, xn2, gu, act;
    // mixture-of-experts layers: router state and the expert slabs (gu / act above are slabs too)
    int logits = -1, ridx = -1, rw = -1, rpos = -1, counts = -1, cnt_recv = -1, xs = -1, ys = -1;
};

struct Builder {
    const Config& cfg;
    const Decomp& d;
    Plan* p;
    uint32_t rank, stage, tp_id;
    bool first_stage, last_stage, fused, tied;
    uint64_t cursor[TC_COUNT] = {0, 0, 0, 0, 0, 0};
    uint64_t flat_elems = 0;       // elements in the flat parameter space so far
    uint32_t next_event = 0;
    uint32_t next_seq = 0;         // sequence number of the next fused compute+collective op
    int flat_param = -1, flat_grad = -1, flat_master = -1, flat_m = -1, flat_v = -1;
    // fp8 (param_dtype = fp8e4m3, tp = 1): e4m3 copies of the linear weights (plain and transposed, one fp32
    // scale per 128x128 block) and a scratch for the 1x128-quantised activation that feeds a GEMM
    struct Fp8Weight { int q = -1, s = -1, qt = -1, st = -1; };
    bool fp8 = false;
    std::map<int, Fp8Weight> fp8w;   // keyed by the bf16 weight tensor
    int fp8_xq = -1, fp8_sx = -1;

    // local dimensions
    uint32_t H, hd, nh_l, nkv_l, Hq_l, Cqkv, F_l, V_l, T, Tl, seq, mbsz, tp, layers;

    Builder(const Config& c, const Decomp& dd, Plan* pl, uint32_t r) : cfg(c), d(dd), p(pl), rank(r) {}

    // ---- tensors
    int tensor_at(uint16_t tclass, uint16_t dtype, uint64_t offset, uint32_t rows, uint32_t cols, uint32_t ld) {
        TensorDesc t{};
        t.offset = offset;
        t.nbytes = static_cast<uint64_t>(rows) * ld * dtype_size(dtype);
        t.shape_id = static_cast<uint32_t>(p->tensors.size());
        t.dtype = dtype;
        t.tclass = tclass;
        p->tensors.push_back(t);
        p->shapes.insert(p->shapes.end(), {rows, cols, ld, 1u});
        return static_cast<int>(p->tensors.size()) - 1;
    }
    int tensor(uint16_t tclass, uint16_t dtype, uint32_t rows, uint32_t cols) {
        cursor[tclass] = align_up(cursor[tclass], kTensorAlign);
        const int id = tensor_at(tclass, dtype, cursor[tclass], rows, cols, cols);
        cursor[tclass] += p->tensors[id].nbytes;
        return id;
    }
    // rows [row0, row0+rows) of an existing tensor
    int view(int parent, uint32_t row0, uint32_t rows) {
        const TensorDesc& pt = p->tensors[parent];
        const uint32_t cols = p->shapes[parent * 4 + 1], ld = p->shapes[parent * 4 + 2];
        return tensor_at(pt.tclass, pt.dtype, pt.offset + static_cast<uint64_t>(row0) * ld * dtype_size(pt.dtype), rows,
                         cols, ld);
    }
    // columns [col0, col0+cols) of every row of an existing tensor
    int colview(int parent, uint32_t col0, uint32_t cols) {
        const TensorDesc& pt = p->tensors[parent];
        const uint32_t rows = p->shapes[parent * 4], ld = p->shapes[parent * 4 + 2];
        const uint64_t es = dtype_size(pt.dtype);
        const int id = tensor_at(pt.tclass, pt.dtype, pt.offset + col0 * es, rows, cols, ld);
        p->tensors[id].nbytes = (static_cast<uint64_t>(rows - 1) * ld + cols) * es;
        return id;
    }
    uint32_t rows_of(int t) const { return p->shapes[t * 4]; }
    uint32_t cols_of(int t) const { return p->shapes[t * 4 + 1]; }

    // A parameter occupies the same element range in the bf16 weight, fp32 gradient, master,
    // m and v buffers, so a single AdamW launch covers the whole flat space.
    Param param(const char* name, uint32_t rows, uint32_t cols, float init_std) {
        flat_elems = align_up(flat_elems, kFlatAlignElems);
        Param q;
        q.rows = rows;
        q.cols = cols;
        q.w = tensor_at(TC_PARAM, DT_BF16, flat_elems * 2, rows, cols, cols);
        q.g = tensor_at(TC_GRAD, DT_FP32, flat_elems * 4, rows, cols, cols);
        NamedTensor nt{};
        std::snprintf(nt.name, sizeof nt.name, "%s", name);
        nt.tensor = q.w;
        nt.grad = q.g;
        nt.master = static_cast<int32_t>(flat_elems >> 9);  // flat offset in units of kFlatAlignElems
        nt.rows = rows;
        nt.cols = cols;
        nt.init_std = init_std;
        p->named.push_back(nt);
        flat_elems += static_cast<uint64_t>(rows) * cols;
        return q;
    }

    // ---- ops
    void push(uint16_t kind, uint16_t stream, double flops, double bytes, uint32_t aux0, uint16_t mb, const ExecOp* x) {
        Op o{};
        o.kind = kind;
        o.stream_id = stream;
        o.flops = static_cast<uint64_t>(flops < 0 ? 0 : flops);
        o.bytes = static_cast<uint64_t>(bytes < 0 ? 0 : bytes);
        o.aux0 = aux0;
        o.aux1 = mb;
        if (x) {
            p->exec.push_back(*x);
            o.exec = static_cast<uint32_t>(p->exec.size());
        }
        p->ops.push_back(o);
    }
    uint32_t record(uint16_t stream, uint16_t mb) {
        push(OP_EVENT_RECORD, stream, 0, 0, next_event, mb, nullptr);
        return next_event++;
    }
    void wait(uint16_t stream, uint32_t ev, uint16_t mb) { push(OP_EVENT_WAIT, stream, 0, 0, ev, mb, nullptr); }
    void sync(uint16_t from, uint16_t to, uint16_t mb) {
        if (from == to) return;
        wait(to, record(from, mb), mb);
    }

    // C[M,N] = A * B^T style product; trans flags as in the kernel library.
    void gemm(uint16_t stream, int A, int B, int C, int R, uint32_t M, uint32_t N, uint32_t K, bool ta, bool tb, int epi,
              uint16_t mb) {
        ExecOp x = xop(K_GEMM, static_cast<uint16_t>((ta ? 1 : 0) | (tb ? 2 : 0) | (epi << 4)));
        x.t[0] = A; x.t[1] = B; x.t[2] = C; x.t[3] = R;
        x.i[0] = M; x.i[1] = N; x.i[2] = K;
        x.f[0] = 1.0f;
        push(OP_GEMM, stream, 2.0 * M * N * K, 0, 0, mb, &x);
    }
    // Linear layer product with tp = 1: C[T,N] = a[T,K] * W[N,K]^T (tb: a[T,K] * W[K,N]) (+ residual R).
    // With fp8 weights the activation is quantised per row and 128 columns and the e4m3 tensor-core GEMM runs.
    void linear(int a, int W, int C, int R, uint32_t N, uint32_t K, bool tb, uint16_t mb, int epi = -1) {
        auto it = fp8w.find(W);
        if (!fp8 || it == fp8w.end() || K % 128 || epi > 3) {
            gemm(ST_COMPUTE_HI, a, W, C, R, T, N, K, false, tb, epi >= 0 ? epi : (R >= 0 ? 3 : 0), mb);
            return;
        }
        const Fp8Weight& w = it->second;
        const int xq = tensor_at(TC_WORKSPACE, DT_FP8_E4M3, p->tensors[fp8_xq].offset, T, K, K);
        const int sx = tensor_at(TC_WORKSPACE, DT_FP32, p->tensors[fp8_sx].offset, T, K / 128, K / 128);
        ExecOp qx = xop(K_QUANT_FP8, 0);
        qx.t[0] = a; qx.t[1] = xq; qx.t[2] = sx;
        qx.i[0] = T; qx.i[1] = K;
        push(OP_ELEMENTWISE, ST_COMPUTE_HI, 2.0 * T * K, 3.0 * T * K, 0, mb, &qx);
        ExecOp x = xop(K_GEMM_FP8, static_cast<uint16_t>((R >= 0 ? 3 : 0) << 4));
        x.t[0] = xq; x.t[1] = tb ? w.qt : w.q; x.t[2] = C; x.t[3] = R; x.t[4] = sx; x.t[5] = tb ? w.st : w.s;
        x.i[0] = T; x.i[1] = N; x.i[2] = K;
        push(OP_GEMM, ST_COMPUTE_HI, 2.0 * T * N * K, 0, 0, mb, &x);
    }
    // e4m3 copies of a weight [rows, cols]: blocks of 128x128 share a scale; the transposed copy serves the input gradient
    void quant_weight(int W, uint16_t mb) {
        const Fp8Weight& w = fp8w.at(W);
        ExecOp e = xop(K_QUANT_FP8, 1);
        e.t[0] = W; e.t[1] = w.q; e.t[2] = w.s; e.t[3] = w.qt; e.t[4] = w.st;
        e.i[0] = rows_of(W); e.i[1] = cols_of(W);
        push(OP_ELEMENTWISE, ST_COMPUTE_HI, 0, 4.0 * rows_of(W) * cols_of(W), 0, mb, &e);
    }
    // GEMM over a ragged expert slab: `counts` holds the live rows of each `seg_rows`-row sub-slab.
    // seg_mode 1 segments M (forward / input gradient), 2 segments K (weight gradient).
    void gemm_seg(int A, int B, int C, uint32_t M, uint32_t N, uint32_t K, bool ta, bool tb, int epi, int counts,
                  uint32_t seg_rows, int seg_mode, uint16_t mb) {
        ExecOp x = xop(K_GEMM, static_cast<uint16_t>((ta ? 1 : 0) | (tb ? 2 : 0) | (epi << 4)));
        x.t[0] = A; x.t[1] = B; x.t[2] = C; x.t[4] = counts;
        x.i[0] = M; x.i[1] = N; x.i[2] = K; x.i[3] = seg_rows; x.i[4] = seg_mode;
        x.f[0] = 1.0f;
        push(OP_GEMM, ST_COMPUTE_HI, 2.0 * M * N * K, 0, 0, mb, &x);
    }
    // `groups` products of one shape in a single launch (the local experts): A, B, C are the stacked tensors,
    // M / N / K the per-group sizes; the runtime derives each group's row offsets from the operand forms.
    void gemm_grouped(int A, int B, int C, uint32_t M, uint32_t N, uint32_t K, bool ta, bool tb, int epi, int counts,
                      uint32_t seg_rows, int seg_mode, uint32_t groups, uint16_t mb) {
        ExecOp x = xop(K_GEMM, static_cast<uint16_t>((ta ? 1 : 0) | (tb ? 2 : 0) | (epi << 4) | 0x100));
        x.t[0] = A; x.t[1] = B; x.t[2] = C; x.t[4] = counts;
        x.i[0] = M; x.i[1] = N; x.i[2] = K; x.i[3] = seg_rows; x.i[4] = seg_mode | static_cast<int32_t>(groups << 8);
        x.f[0] = 1.0f;
        push(OP_GEMM, ST_COMPUTE_HI, 2.0 * M * N * K * groups, 0, 0, mb, &x);
    }
    void rmsnorm_fwd(int x, int g, int y, int rstd, uint32_t rows, uint16_t mb) {
        ExecOp e = xop(K_RMSNORM_FWD);
        e.t[0] = x; e.t[1] = g; e.t[2] = y; e.t[3] = rstd;
        e.i[0] = rows; e.i[1] = H;
        e.f[0] = cfg.train.norm_eps;
        push(OP_RMSNORM, ST_COMPUTE_HI, 5.0 * rows * H, 0, 0, mb, &e);
    }
    void rmsnorm_bwd(int x, int g, int rstd, int dy, int dx, int dg, int scratch, uint32_t rows, bool dx_acc, bool dg_acc,
                     uint16_t mb) {
        ExecOp e = xop(K_RMSNORM_BWD);
        e.t[0] = x; e.t[1] = g; e.t[2] = rstd; e.t[3] = dy; e.t[4] = dx; e.t[5] = dg; e.t[6] = scratch;
        e.i[0] = rows; e.i[1] = H; e.i[2] = dx_acc; e.i[3] = dg_acc;
        push(OP_RMSNORM, ST_COMPUTE_HI, 10.0 * rows * H, 0, 0, mb, &e);
    }
    void nccl(uint16_t kernel, uint16_t opkind, uint16_t stream, int src, int dst, uint64_t count, uint16_t dtype,
              uint16_t group, int peer, uint16_t mb) {
        ExecOp e = xop(kernel);
        e.t[0] = src; e.t[1] = dst;
        e.i[0] = static_cast<int32_t>(count & 0xFFFFFFFFu);
        e.i[1] = static_cast<int32_t>(count >> 32);
        e.i[2] = dtype; e.i[3] = group; e.i[4] = peer;
        push(opkind, stream, 0, static_cast<double>(count) * dtype_size(dtype), group, mb, &e);
    }

    // y[T, N] = gather_rows(x_local[Tl, K]) * W[N, K]^T  (column-parallel linear, forward), or
    // with tb: y[T, N] = gather_rows(x_local) * W[K, N] (input gradient of a row-parallel linear).
    // x_full receives the gathered rows (kept for the weight gradient).
    // epi / aux select a fused epilogue of the product (CAI_EPI_SWIGLU: aux receives the activation;
    // CAI_EPI_SWIGLU_BWD: aux is the saved [gate | up] tensor and y receives [dgate | dup]).
    void col_parallel(int x_local, int x_full, int W, int y, uint32_t N, uint32_t K, bool tb, uint16_t mb, int epi = 0,
                      int aux = -1) {
        if (tp == 1) {
            linear(x_local, W, y, aux, N, K, tb, mb, epi);
            return;
        }
        if (fused && !fp8) {
            ExecOp e = xop(K_AG_GEMM, static_cast<uint16_t>((tb ? 2 : 0) | (epi << 4)));
            e.t[0] = x_local; e.t[1] = W; e.t[2] = y; e.t[3] = x_full; e.t[5] = aux;
            e.i[0] = T; e.i[1] = N; e.i[2] = K; e.i[3] = GROUP_TP; e.i[4] = static_cast<int32_t>(next_seq++);
            e.f[0] = 1.0f;
            push(OP_AG_GEMM, ST_COMPUTE_HI, 2.0 * T * N * K, static_cast<double>(T) * K * 2, GROUP_TP, mb, &e);
            return;
        }
        sync(ST_COMPUTE_HI, ST_COMM_TP, mb);
        nccl(K_NCCL_ALL_GATHER, OP_ALL_GATHER, ST_COMM_TP, x_local, x_full, static_cast<uint64_t>(Tl) * K, DT_BF16,
             GROUP_TP, -1, mb);
        sync(ST_COMM_TP, ST_COMPUTE_HI, mb);
        // e4m3 weights: the gathered rows are quantised and the block-scaled product runs (there is no e4m3 form of
        // the all-gather + GEMM kernel, so the collective stays a call of its own beside it)
        if (fp8) linear(x_full, W, y, aux, N, K, tb, mb, epi);
        else gemm(ST_COMPUTE_HI, x_full, W, y, aux, T, N, K, false, tb, epi, mb);
    }
    // out_local[Tl, N] = residual + reduce_scatter_rows(a[T, K] * W[N, K]^T) (row-parallel linear,
    // forward), or with tb the input gradient of a column-parallel linear (residual may be -1).
    void row_parallel(int a, int W, int residual, int out_local, int partial, int rs_tmp, uint32_t N, uint32_t K, bool tb,
                      uint16_t mb) {
        if (tp == 1) {
            linear(a, W, out_local, residual, N, K, tb, mb);
            return;
        }
        if (fused && !fp8) {
            ExecOp e = xop(K_GEMM_RS, static_cast<uint16_t>(tb ? 2 : 0));
            e.t[0] = a; e.t[1] = W; e.t[2] = out_local; e.t[3] = residual; e.t[4] = partial;
            e.i[0] = T; e.i[1] = N; e.i[2] = K; e.i[3] = GROUP_TP; e.i[4] = static_cast<int32_t>(next_seq++);
            e.f[0] = 1.0f;
            push(OP_GEMM_RS, ST_COMPUTE_HI, 2.0 * T * N * K, static_cast<double>(T) * N * 2, GROUP_TP, mb, &e);
            return;
        }
        if (fp8) linear(a, W, partial, -1, N, K, tb, mb);
        else gemm(ST_COMPUTE_HI, a, W, partial, -1, T, N, K, false, tb, 0, mb);
        sync(ST_COMPUTE_HI, ST_COMM_TP, mb);
        nccl(K_NCCL_REDUCE_SCATTER, OP_REDUCE_SCATTER, ST_COMM_TP, partial, residual >= 0 ? rs_tmp : out_local,
             static_cast<uint64_t>(Tl) * N, DT_BF16, GROUP_TP, -1, mb);
        sync(ST_COMM_TP, ST_COMPUTE_HI, mb);
        if (residual >= 0) {
            ExecOp e = xop(K_ADD);
            e.t[0] = residual; e.t[1] = rs_tmp; e.t[2] = out_local;
            e.i[0] = static_cast<int32_t>(static_cast<uint64_t>(Tl) * N);
            push(OP_ELEMENTWISE, ST_COMPUTE_HI, static_cast<double>(Tl) * N, 0, 0, mb, &e);
        }
    }
};

}  // namespace

void exec_operands(const ExecOp& x, std::vector<int>* reads, std::vector<int>* writes) {
    reads->clear();
    writes->clear();
    auto R = [&](int i) { if (x.t[i] >= 0) reads->push_back(x.t[i]); };
    auto W = [&](int i) { if (x.t[i] >= 0) writes->push_back(x.t[i]); };
    switch (x.kernel) {
        case K_EMBED_FWD: R(0); R(1); W(2); break;
        case K_EMBED_BWD: R(0); R(1); R(2); W(2); break;
        case K_RMSNORM_FWD: R(0); R(1); W(2); W(3); break;
        case K_RMSNORM_BWD: R(0); R(1); R(2); R(3); if (x.i[2]) R(4); W(4); if (x.i[3]) R(5); W(5); W(6); break;
        case K_GEMM: {
            const int epi = (x.flags >> 4) & 0xF;
            R(0); R(1); if (epi == 2) R(2); R(4); W(2);
            if (epi == 4) W(3); else R(3);   // fused SwiGLU writes the activation into its second tensor
            break;
        }
        case K_ROPE: R(0); R(1); W(0); break;
        case K_ATTN_FWD: R(0); W(1); W(2); break;
        case K_ATTN_BWD:
            R(0); R(1); R(2); R(3);
            if (x.flags == 0 || (x.flags & 1)) W(4); else R(4);
            if (x.flags == 0) W(5);
            else if (x.flags & 6) W(6);
            break;
        case K_SWIGLU_FWD: R(0); W(1); break;
        case K_SWIGLU_BWD: R(0); R(1); W(2); break;
        case K_CROSS_ENTROPY: case K_CROSS_ENTROPY_TP: R(0); R(1); R(2); W(0); W(2); W(3); break;
        case K_ADAMW: R(0); R(1); R(2); R(3); W(0); W(1); W(2); W(4); break;
        case K_ZERO: W(0); break;
        case K_ADD: R(0); R(1); W(2); break;
        case K_NCCL_ALL_REDUCE: R(0); W(1); break;
        case K_NCCL_REDUCE_SCATTER: case K_NCCL_ALL_GATHER: case K_NCCL_ALL_TO_ALL: R(0); W(1); break;
        case K_NCCL_SEND: R(0); break;
        case K_NCCL_RECV: W(1); break;
        case K_AG_GEMM:
            R(0); R(1); W(2); W(3);
            if (((x.flags >> 4) & 0xF) == 4) W(5); else R(5);
            break;
        case K_GEMM_RS: R(0); R(1); R(3); W(2); W(4); break;
        case K_RS_ADAMW: R(0); R(1); R(2); R(3); R(5); W(0); W(1); W(2); W(4); W(5); break;   // t[5]: gradient accumulator of the shard
        case K_FSDP_AG_GEMM: if (x.t[2] >= 0) R(2); else R(0); W(1); break;   // t[2]: the slice of the local shard that is read
        case K_QUANT_FP8: R(0); W(1); W(2); W(3); W(4); break;
        case K_GEMM_FP8: R(0); R(1); R(3); R(4); R(5); W(2); break;
        case K_MOE_ROUTE:
            if (x.flags & 1) { R(0); R(1); R(2); R(3); W(4); } else { R(0); W(1); W(2); W(3); W(4); }
            break;
        case K_MOE_DISPATCH_GEMM: R(0); R(1); R(2); R(3); R(4); W(5); W(6); break;
        case K_MOE_GEMM_COMBINE: R(0); R(2); R(3); R(4); R(5); R(6); W(1); W(7); break;
        default:
            for (int i = 0; i < 8; ++i) { R(i); }
            break;
    }
}

int build_plan_v2(const Config& cfg, const Decomp& d, uint32_t rank, uint64_t ph, uint64_t th, Plan* out,
                  std::string* err) {
    const ModelSpec& m = cfg.model;
    *out = Plan{};
    Topology topo;
    if (int rc = fill_plan_header(cfg, d, rank, ph, th, 2, &topo, &out->hdr, err); rc != OK) return rc;
    PlanHeader& h = out->hdr;
    out->groups = rank_groups(d, topo, m.is_moe != 0, rank);
    out->train = cfg.train;
    out->model = m;

    const bool moe = m.is_moe != 0;
    if (moe) {
        // Under tensor parallelism the experts are spread over the tp x ep ranks of a replica block (every rank routes
        // the rows of the sequence it owns), so that group must fit one peer table.
        if (d.tp * std::max(1u, d.ep) > static_cast<uint32_t>(kMaxPeers) || m.num_experts % (d.tp * std::max(1u, d.ep)))
            return failf(err, ERR_INVALID, "MoE plans need tp x ep <= %d and experts %% (tp x ep) == 0 (got tp=%u ep=%u)", kMaxPeers, d.tp, d.ep);
        if (d.ep != 1 && d.ep != d.dp) return failf(err, ERR_INVALID, "MoE plans need ep = 1 or ep = dp (got ep=%u dp=%u)", d.ep, d.dp);
        if (m.num_experts % 32 || m.num_experts > 256 || m.moe_top_k < 1 || m.moe_top_k > 8 || m.num_experts % d.ep)
            return failf(err, ERR_INVALID, "MoE plans need experts %% 32 == 0 (<= 256), top_k <= 8, experts %% ep == 0");
        if (!cfg.train.comm_mode) return failf(err, ERR_INVALID, "MoE plans exist only for comm = fused (in-kernel dispatch/combine)");
    }
    // ZeRO-3: the bf16 parameters are sharded over the data-parallel group like the optimizer state and
    // gathered layer by layer (the gather is fused into the first GEMM that reads the layer's weights). Beside tensor
    // parallelism every rank shards ITS slice of the weights over the ranks that hold the same slice; the gathers are
    // then kernels of their own (the first consumer is an all-gather + GEMM kernel, which has no copy role for weights)
    // and gradients stay whole (the per-layer buckets that shard them exist for tp = 1).
    const bool zero3 = cfg.train.zero_stage >= 3 && d.dp > 1 && cfg.train.comm_mode != 0 && !moe;
    if (cfg.train.zero_stage >= 3 && d.dp > 1 && !zero3)
        return failf(err, ERR_INVALID, "zero_stage = 3 needs comm = fused and a dense model");
    // ZeRO-2: parameters stay whole on every rank (as with zero_stage = 1), but the fp32 gradients are sharded like under
    // ZeRO-3: a layer's weight gradients of one microbatch land in one of two alternating layer-sized buffers and the
    // layer's bucket kernel sums the members' buffers into the owners' shard-sized accumulators. Needs the per-layer
    // buckets, which exist for tp = 1.
    const bool zero2 = cfg.train.zero_stage == 2 && d.dp > 1 && !moe && cfg.train.comm_mode != 0 && d.tp == 1 && cfg.train.dp_buckets != 0;
    if (cfg.train.zero_stage == 2 && d.dp > 1 && !zero2)
        return failf(err, ERR_INVALID, "zero_stage = 2 needs comm = fused, tp = 1, per-layer buckets (dp_buckets = 1) and a dense model");
    // fp8 parameters: forward and input-gradient GEMMs of the linear layers run in e4m3 with block scales
    // (tp = 1, dense); weight gradients, attention, the LM head and everything else stay bf16.
    if (m.param_dtype == DT_FP8_E4M3 && moe)
        return failf(err, ERR_INVALID, "param_dtype = fp8e4m3 has an executable schedule for dense models only; "
                                       "use bf16 for mixture-of-experts models instead of a silent change of precision");
    const bool fp8 = m.param_dtype == DT_FP8_E4M3;
    if (d.cp != 1) return failf(err, ERR_INVALID, "context parallelism (cp>1) has no executable schedule");
    if (d.vpp > 1)
        return failf(err, ERR_INVALID, "vpp = %u: there is no interleaved executable schedule (the key changes the bubble formula of "
                     "cost-only plans only, as in the reference); use vpp = 1", d.vpp);
    if (m.head_dim != 128) return failf(err, ERR_INVALID, "executable plans need head_dim = 128 (got %u)", m.head_dim);
    if (m.num_heads % d.tp || m.num_kv_heads % d.tp || m.ffn_hidden % d.tp || m.vocab_size % d.tp)
        return failf(err, ERR_INVALID, "tp=%u must divide heads, kv heads, ffn and vocab", d.tp);
    if ((m.microbatch * m.seq_len) % d.tp || m.seq_len % 128)
        return failf(err, ERR_INVALID, "tokens per microbatch must divide by tp and seq_len by 128");
    // Microbatches launched together (TrainSpec::mb_group). A pipeline keeps the configured granularity (fewer,
    // larger microbatches would widen its bubble); the per-tile signal slots of the fused TP kernels bound the rows.
    uint32_t mb_group = cfg.train.mb_group;
    auto rows_fit = [&](uint32_t g) {
        const uint64_t rows = static_cast<uint64_t>(g) * m.microbatch * m.seq_len;
        return rows / 128 <= kSigLocalSlots && !(d.tp > 1 && (rows / d.tp / 128) * ((m.hidden_size + 127) / 128) > kSigTileSlots);
    };
    if (mb_group == 0) {
        // as many as divide grad_accum and keep a launch at or under 16384 tokens (a launch that size fills the GPU
        // and amortises the hand-shakes of the fused kernels; activation memory grows with it)
        mb_group = 1;
        if (d.pp == 1 && !moe && cfg.train.zero_stage < 3)
            for (uint32_t g = 2; g <= d.num_microbatches; g *= 2)
                if (d.num_microbatches % g == 0 && static_cast<uint64_t>(g) * m.microbatch * m.seq_len <= 16384 && rows_fit(g)) mb_group = g;
    }
    if (mb_group > 1) {
        if (d.pp != 1) return failf(err, ERR_INVALID, "mb_group > 1 needs pp = 1 (got pp=%u)", d.pp);
        if (d.num_microbatches % mb_group) return failf(err, ERR_INVALID, "mb_group=%u must divide grad_accum=%u", mb_group, d.num_microbatches);
        if (!rows_fit(mb_group))
            return failf(err, ERR_INVALID, "mb_group=%u: %llu rows per launch exceed the signal slots of the fused kernels", mb_group,
                         static_cast<unsigned long long>(mb_group) * m.microbatch * m.seq_len);
    }
    if ((m.vocab_size / d.tp) % 8 || m.hidden_size % 8 || (m.ffn_hidden / d.tp) % 8)
        return failf(err, ERR_INVALID, "local hidden / ffn / vocab sizes must be multiples of 8");

    Builder b(cfg, d, out, rank);
    b.stage = h.pipeline_stage;
    b.tp_id = rank % d.tp;
    b.first_stage = b.stage == 0;
    b.last_stage = b.stage == d.pp - 1;
    b.fused = cfg.train.comm_mode != 0;
    b.tied = cfg.train.tie_embeddings && d.pp == 1;
    b.tp = d.tp;
    b.H = m.hidden_size; b.hd = m.head_dim;
    b.nh_l = m.num_heads / d.tp; b.nkv_l = m.num_kv_heads / d.tp;
    b.Hq_l = b.nh_l * b.hd;
    b.Cqkv = (b.nh_l + 2 * b.nkv_l) * b.hd;
    b.F_l = m.ffn_hidden / d.tp;
    b.V_l = m.vocab_size / d.tp;
    b.seq = m.seq_len; b.mbsz = m.microbatch * mb_group;
    b.T = b.mbsz * m.seq_len;
    b.Tl = b.T / d.tp;
    b.layers = h.layers_in_stage;
    const uint32_t H = b.H, T = b.T, Tl = b.Tl, tp = b.tp, ga = d.num_microbatches / mb_group;   // launches per step
    const float istd = cfg.train.init_std;

    // ---------------- parameters (flat space)
    Param embed, head, gf;
    if (b.first_stage || (b.last_stage && b.tied)) embed = b.param("embed", b.V_l, H, istd);
    std::vector<LayerParams> L(b.layers);
    const uint32_t base_layer = [&] {
        uint32_t base = m.num_layers / d.pp, rem = m.num_layers % d.pp, s = b.stage;
        return s * base + std::min(s, rem);
    }();
    // Under ZeRO-3 the small vectors (norm gains) and the embedding form one group that is gathered once
    // per step; every layer's matrices form a group of their own, contiguous in the flat space.
    uint64_t misc_hi = 0;
    std::vector<std::pair<uint64_t, uint64_t>> layer_range(b.layers);
    auto lname = [&](char* nm, uint32_t l, const char* suffix) {
        std::snprintf(nm, 40, "L%u.%s", base_layer + l, suffix);
        return nm;
    };
    if (zero3 || zero2) {      // the small tensors first, then every layer's matrices as one contiguous group
        char nm[40];
        for (uint32_t l = 0; l < b.layers; ++l) {
            L[l].g1 = b.param(lname(nm, l, "g1"), 1, H, 0.f);
            L[l].g2 = b.param(lname(nm, l, "g2"), 1, H, 0.f);
        }
        if (b.last_stage) {
            gf = b.param("gf", 1, H, 0.f);
            if (!b.tied) head = b.param("lm_head", b.V_l, H, istd);
            else head = embed;
        }
        misc_hi = align_up(b.flat_elems, kFlatAlignElems);
        for (uint32_t l = 0; l < b.layers; ++l) {
            layer_range[l].first = align_up(b.flat_elems, kFlatAlignElems);
            L[l].wqkv = b.param(lname(nm, l, "wqkv"), b.Cqkv, H, istd);
            L[l].wo = b.param(lname(nm, l, "wo"), H, b.Hq_l, istd);
            L[l].wgu = b.param(lname(nm, l, "wgu"), 2 * b.F_l, H, istd);
            L[l].wd = b.param(lname(nm, l, "wd"), H, b.F_l, istd);
            layer_range[l].second = align_up(b.flat_elems, kFlatAlignElems);
        }
    } else {
        for (uint32_t l = 0; l < b.layers; ++l) {
            char nm[40];
            auto name = [&](const char* suffix) {
                std::snprintf(nm, sizeof nm, "L%u.%s", base_layer + l, suffix);
                return nm;
            };
            layer_range[l].first = align_up(b.flat_elems, kFlatAlignElems);
            L[l].g1 = b.param(name("g1"), 1, H, 0.f);
            L[l].wqkv = b.param(name("wqkv"), b.Cqkv, H, istd);
            L[l].wo = b.param(name("wo"), H, b.Hq_l, istd);
            L[l].g2 = b.param(name("g2"), 1, H, 0.f);
            if (moe) {
                L[l].wr = b.param(name("wr"), m.num_experts, H, istd);
            } else {
                L[l].wgu = b.param(name("wgu"), 2 * b.F_l, H, istd);
                L[l].wd = b.param(name("wd"), H, b.F_l, istd);
            }
            layer_range[l].second = align_up(b.flat_elems, kFlatAlignElems);
        }
        if (b.last_stage) {
            gf = b.param("gf", 1, H, 0.f);
            if (!b.tied) head = b.param("lm_head", b.V_l, H, istd);
            else head = embed;
        }
    }
    // Expert weights come last in the flat space: everything before them is replicated over the
    // data-parallel group (gradients are reduced), the experts of an expert-parallel group are not.
    const uint32_t xg = moe ? d.tp * std::max(1u, d.ep) : 1;   // members of the expert group: tp x ep
    const uint32_t E_l = moe ? m.num_experts / xg : 0;
    const uint64_t n_replicated = moe && d.ep > 1 ? align_up(b.flat_elems, kFlatAlignElems) : 0;
    if (moe)
        for (uint32_t l = 0; l < b.layers; ++l) {
            char nm[40];
            std::snprintf(nm, sizeof nm, "L%u.experts.wgu", base_layer + l);
            L[l].wgu = b.param(nm, E_l * 2 * m.ffn_hidden, H, istd);
            std::snprintf(nm, sizeof nm, "L%u.experts.wd", base_layer + l);
            L[l].wd = b.param(nm, E_l * H, m.ffn_hidden, istd);
        }
    const uint64_t n_flat = align_up(b.flat_elems, kFlatAlignElems);
    if (n_flat > 0x7FFFFFFFFFFFull) return failf(err, ERR_INVALID, "parameter space too large");
    b.flat_param = b.tensor_at(TC_PARAM, DT_BF16, 0, 1, static_cast<uint32_t>(std::min<uint64_t>(n_flat, 0xFFFFFFFFu)), 0);
    b.flat_grad = b.tensor_at(TC_GRAD, DT_FP32, 0, 1, static_cast<uint32_t>(std::min<uint64_t>(n_flat, 0xFFFFFFFFu)), 0);
    out->tensors[b.flat_param].nbytes = n_flat * 2;
    out->tensors[b.flat_grad].nbytes = n_flat * 4;
    b.cursor[TC_PARAM] = n_flat * 2;
    b.cursor[TC_GRAD] = n_flat * 4;
    // optimizer state: master | m | v, each n_flat fp32 (sharded 1/dp when the optimizer is sharded)
    // sharded 1/dp only when the fused reduce-scatter + AdamW kernel owns the update; the NCCL baseline
    // all-reduces the gradients and every replica updates everything
    // Expert weights of an expert-parallel group are not replicated: their optimizer state is local and
    // sits behind the (possibly sharded) state of the replicated parameters.
    const uint64_t n_rep = n_replicated ? n_replicated : n_flat;
    const uint64_t n_exp = n_flat - n_rep;
    const uint64_t n_shard = (d.dp > 1 && b.fused) ? align_up((n_rep + d.dp - 1) / d.dp, kFlatAlignElems) : n_rep;
    const uint64_t n_opt = n_shard + n_exp;
    b.flat_master = b.tensor_at(TC_OPTSTATE, DT_FP32, 0, 1, 0, 0);
    b.flat_m = b.tensor_at(TC_OPTSTATE, DT_FP32, n_opt * 4, 1, 0, 0);
    b.flat_v = b.tensor_at(TC_OPTSTATE, DT_FP32, n_opt * 8, 1, 0, 0);
    for (int t : {b.flat_master, b.flat_m, b.flat_v}) out->tensors[t].nbytes = n_opt * 4;
    b.cursor[TC_OPTSTATE] = n_opt * 12;
    out->xhdr.param_elems = n_flat;
    out->xhdr.reserved = n_opt;
    const uint64_t hdr_n_rep = n_rep, hdr_n_shard = n_shard;
    int stage_misc = -1, stage_layer[2] = {-1, -1};
    if (zero3) {
        // the parameter class holds this rank's shard, the resident group and two layer-sized staging buffers
        out->tensors[b.flat_param].nbytes = n_shard * 2;
        b.cursor[TC_PARAM] = n_shard * 2;
        uint64_t max_layer = 0;
        for (const auto& r : layer_range) max_layer = std::max(max_layer, r.second - r.first);
        auto stage = [&](uint64_t elems) {
            b.cursor[TC_PARAM] = align_up(b.cursor[TC_PARAM], kTensorAlign);
            const int id = b.tensor_at(TC_PARAM, DT_BF16, b.cursor[TC_PARAM], 1, static_cast<uint32_t>(std::min<uint64_t>(elems, 0xFFFFFFFFu)), 0);
            out->tensors[id].nbytes = elems * 2;
            b.cursor[TC_PARAM] += elems * 2;
            return id;
        };
        stage_misc = stage(misc_hi);
        stage_layer[0] = stage(max_layer);
        stage_layer[1] = b.layers > 1 ? stage(max_layer) : stage_layer[0];
        // every parameter tensor now names its place in a staging buffer instead of the flat space
        auto relocate = [&](const Param& q) {
            if (q.w < 0) return;
            const uint64_t flat_off = out->tensors[q.w].offset / 2;
            uint64_t base = out->tensors[stage_misc].offset, lo = 0;
            if (flat_off >= misc_hi)
                for (uint32_t l = 0; l < b.layers; ++l)
                    if (flat_off >= layer_range[l].first && flat_off < layer_range[l].second) {
                        base = out->tensors[stage_layer[l & 1]].offset;
                        lo = layer_range[l].first;
                    }
            out->tensors[q.w].offset = base + (flat_off - lo) * 2;
        };
        relocate(embed);
        if (!b.tied) relocate(head); else head = embed;
        relocate(gf);
        for (LayerParams& w : L) for (const Param* q : {&w.g1, &w.wqkv, &w.wo, &w.g2, &w.wgu, &w.wd}) relocate(*q);
    }
    // ZeRO-3 with per-layer buckets: gradients are sharded too. A layer's weight gradients of ONE microbatch land in
    // one of two alternating layer-sized fp32 buffers; the layer's bucket kernel (every microbatch) sums the
    // members' buffers for the elements this rank owns into a shard-sized accumulator, and on the last microbatch
    // goes on to AdamW. Only the small resident group (embedding, gains, head) keeps full-size gradients.
    const bool shard_grads = (zero3 || zero2) && cfg.train.dp_buckets != 0 && b.layers > 0 && d.tp == 1;
    int grad_stage[2] = {-1, -1}, grad_acc = -1;
    if (shard_grads) {
        uint64_t max_layer = 0;
        for (const auto& r : layer_range) max_layer = std::max(max_layer, r.second - r.first);
        out->tensors[b.flat_grad].nbytes = misc_hi * 4;
        b.cursor[TC_GRAD] = misc_hi * 4;
        auto gbuf = [&](uint64_t elems) {
            b.cursor[TC_GRAD] = align_up(b.cursor[TC_GRAD], kTensorAlign);
            const int id = b.tensor_at(TC_GRAD, DT_FP32, b.cursor[TC_GRAD], 1, 0, 0);
            out->tensors[id].nbytes = elems * 4;
            b.cursor[TC_GRAD] += elems * 4;
            return id;
        };
        grad_stage[0] = gbuf(max_layer);
        grad_stage[1] = b.layers > 1 ? gbuf(max_layer) : grad_stage[0];
        grad_acc = gbuf(n_shard);
        for (uint32_t l = 0; l < b.layers; ++l)
            for (const Param* q : {&L[l].wqkv, &L[l].wo, &L[l].wgu, &L[l].wd}) {
                const uint64_t flat_off = out->tensors[q->g].offset / 4;
                out->tensors[q->g].offset = out->tensors[grad_stage[l & 1]].offset + (flat_off - layer_range[l].first) * 4;
            }
    }
    // Emits the gather of one parameter group. `fuse` marks a record that the runtime merges into the
    // GEMM that follows it (the gather runs in that kernel's copy CTAs); otherwise it is a kernel of its own.
    int resident[2] = {-1, -1};
    auto gather_group = [&](int layer, bool reverse, bool fuse, uint16_t mb) {
        if (!zero3) return;
        uint64_t lo = 0, hi = misc_hi;
        int dst = stage_misc;
        if (layer >= 0) {
            if (resident[layer & 1] == layer) return;   // still there from the forward pass
            resident[layer & 1] = layer;
            lo = layer_range[layer].first; hi = layer_range[layer].second;
            dst = stage_layer[layer & 1];
        }
        ExecOp e = xop(K_FSDP_AG_GEMM, static_cast<uint16_t>((fuse ? 1 : 0) | (reverse ? 2 : 0)));
        e.t[0] = b.flat_param; e.t[1] = dst;
        {
            // the part of the local shard the peers (and this rank) read for this group: what the hazard analysis
            // orders against the optimizer's writes into the shard
            const uint64_t r = rank / (d.tp * d.pp * d.cp) % std::max(1u, d.dp);
            const uint64_t a0 = std::max<uint64_t>(lo, r * n_shard), a1 = std::min<uint64_t>(hi, (r + 1) * n_shard);
            const uint64_t off = a0 < a1 ? a0 - r * n_shard : 0;
            e.t[2] = b.tensor_at(TC_PARAM, DT_BF16, out->tensors[b.flat_param].offset + off * 2, 1, 0, 0);
            out->tensors[e.t[2]].nbytes = a0 < a1 ? (a1 - a0) * 2 : 0;
        }
        e.i[0] = static_cast<int32_t>(lo >> 9); e.i[1] = static_cast<int32_t>(hi >> 9); e.i[2] = 0;
        e.i[3] = GROUP_DP; e.i[4] = static_cast<int32_t>(b.next_seq++);
        b.push(OP_ALL_GATHER, ST_COMPUTE_HI, 0, static_cast<double>(hi - lo) * 2 * (d.dp - 1) / d.dp, GROUP_DP, mb, &e);
    };
    // fp8 copies of the linear weights: one set per layer, or a single set under ZeRO-3 (quantised right after
    // the layer's gather, which then is a kernel of its own instead of riding in the first GEMM)
    b.fp8 = fp8;
    int fp8_resident = -1;
    if (fp8) {
        const uint32_t max_k = std::max({H, b.Hq_l, b.F_l, b.Cqkv, 2 * b.F_l});
        b.fp8_xq = b.tensor(TC_WORKSPACE, DT_FP8_E4M3, T, max_k);
        b.fp8_sx = b.tensor(TC_WORKSPACE, DT_FP32, T, (max_k + 127) / 128);
        const uint32_t sets = zero3 ? 1 : b.layers;
        std::vector<std::array<Builder::Fp8Weight, 4>> set(sets);
        for (uint32_t i = 0; i < sets; ++i) {
            const Param* ws[4] = {&L[i].wqkv, &L[i].wo, &L[i].wgu, &L[i].wd};
            for (int k = 0; k < 4; ++k) {
                const uint32_t r = ws[k]->rows, c = ws[k]->cols;
                Builder::Fp8Weight& f = set[i][k];
                f.q = b.tensor(TC_PARAM, DT_FP8_E4M3, r, c);
                f.qt = b.tensor(TC_PARAM, DT_FP8_E4M3, c, r);
                f.s = b.tensor(TC_PARAM, DT_FP32, (r + 127) / 128, (c + 127) / 128);
                f.st = b.tensor(TC_PARAM, DT_FP32, (c + 127) / 128, (r + 127) / 128);
            }
        }
        for (uint32_t l = 0; l < b.layers; ++l) {
            const Param* ws[4] = {&L[l].wqkv, &L[l].wo, &L[l].wgu, &L[l].wd};
            for (int k = 0; k < 4; ++k) b.fp8w[ws[k]->w] = set[zero3 ? 0 : l][k];
        }
    }
    auto quant_layer = [&](uint32_t l, uint16_t mb) {
        for (const Param* q : {&L[l].wqkv, &L[l].wo, &L[l].wgu, &L[l].wd}) b.quant_weight(q->w, mb);
    };
    // makes layer l's weights usable: ZeRO-3 gather (fused into the next GEMM unless fp8 needs them quantised first)
    auto prepare_layer = [&](int l, bool reverse, uint16_t mb) {
        gather_group(l, reverse, !fp8 && d.tp == 1, mb);
        if (fp8 && zero3 && fp8_resident != l) {
            quant_layer(static_cast<uint32_t>(l), mb);
            fp8_resident = l;
        }
    };

    // ---------------- inputs, workspace
    const int tokens = b.tensor(TC_COMM, DT_INT32, ga, T);
    const int targets = b.tensor(TC_COMM, DT_INT32, ga, T);
    const int loss_acc = b.tensor(TC_WORKSPACE, DT_FP32, 1, 8);
    const int signals = b.tensor(TC_COMM, DT_UINT8, 1, kSigBytes);  // epoch counters of the fused kernels
    const int rope_tab = b.tensor(TC_WORKSPACE, DT_FP32, b.seq, b.hd);  // [seq, hd/2] float2
    const uint32_t norm_parts = std::min<uint32_t>(std::max(Tl, 1u), 4 * 160);
    const int norm_scratch = b.tensor(TC_WORKSPACE, DT_FP32, norm_parts, H);
    const int dstream = b.tensor(TC_WORKSPACE, DT_BF16, Tl, H);     // gradient of the residual stream
    const int dxn = b.tensor(TC_WORKSPACE, DT_BF16, Tl, H);         // gradient of a norm output (local rows)
    const int dfull = tp > 1 ? b.tensor(TC_WORKSPACE, DT_BF16, T, H) : -1;  // gathered gradient rows
    // With tensor parallelism the kernels of the backward's critical path are small or wait on peers, so the
    // weight-gradient GEMMs (nothing downstream in the layer needs them) go to compute_lo and fill idle SMs,
    // most of all under the attention backward. The attention half of a layer then gathers into its own buffer.
    const bool overlap_wgrad = tp > 1 && !moe && cfg.train.wgrad_overlap != 0;
    // SwiGLU (forward and backward) rides in the epilogues of the gate/up and down-gradient products
    const bool fuse_swiglu = cfg.train.fuse_swiglu != 0 && !moe && !fp8 && b.F_l % 128 == 0;
    // The backward form is opt-in (fuse_swiglu = 2): its epilogue reads gate / up row by row next to the stores and
    // is slower than the product it rides on (measured 53 ms against 23 + 11 ms per step for the two kernels)
    const bool fuse_swiglu_bwd = fuse_swiglu && cfg.train.fuse_swiglu >= 2;
    const int dfull_attn = overlap_wgrad ? b.tensor(TC_WORKSPACE, DT_BF16, T, H) : dfull;
    const int dqkv = b.tensor(TC_WORKSPACE, DT_BF16, T, b.Cqkv);
    const int dao = b.tensor(TC_WORKSPACE, DT_BF16, T, b.Hq_l);
    const int dgu = b.tensor(TC_WORKSPACE, DT_BF16, T, 2 * b.F_l);
    const int dact = b.tensor(TC_WORKSPACE, DT_BF16, T, b.F_l);
    const int delta = b.tensor(TC_WORKSPACE, DT_FP32, b.nh_l, T);
    const int partial = tp > 1 ? b.tensor(TC_COMM, DT_BF16, T, H) : -1;     // row-parallel partial sums / staging
    const int rs_tmp = tp > 1 ? b.tensor(TC_WORKSPACE, DT_BF16, Tl, H) : -1;
    const int xn_local = tp > 1 ? b.tensor(TC_COMM, DT_BF16, Tl, H) : -1;   // norm output peers gather from
    const uint32_t chunk = std::min<uint32_t>(cfg.train.ce_chunk ? cfg.train.ce_chunk : 1024, T);
    int logits = -1, hf = -1, hf_full = -1, rstdf = -1, xf = -1, dhf_full = -1;
    if (b.last_stage) logits = b.tensor(TC_WORKSPACE, DT_BF16, chunk, b.V_l);
    const int ce_scratch = (b.last_stage && tp > 1) ? b.tensor(TC_WORKSPACE, DT_FP32, 2, chunk) : -1;
    if (b.last_stage && tp > 1) dhf_full = dfull;

    // Mixture of experts: every member keeps, per local expert and per source member, a slab of
    // `moe_cap` rows (capacity factor x the even share); tokens beyond a slab's capacity skip that expert.
    const uint32_t moe_cap = moe ? static_cast<uint32_t>(align_up(
        static_cast<uint64_t>(std::max(1.0, cfg.train.moe_capacity_factor_x100 / 100.0) * Tl * m.moe_top_k / m.num_experts + 0.999), 128)) : 0;
    const uint32_t moe_rows = moe ? E_l * xg * moe_cap : 0;   // every member routes its own Tl rows of the sequence
    int dy_s = -1, dact_s = -1, dgu_s = -1, dx_s = -1, dw_r = -1, dlogits = -1;
    if (moe) {
        dy_s = b.tensor(TC_COMM, DT_BF16, moe_rows, H);        // gradient rows pushed by the token owners
        dx_s = b.tensor(TC_COMM, DT_BF16, moe_rows, H);        // input gradients pulled back by the token owners
        dact_s = b.tensor(TC_WORKSPACE, DT_BF16, moe_rows, m.ffn_hidden);
        dgu_s = b.tensor(TC_WORKSPACE, DT_BF16, moe_rows, 2 * m.ffn_hidden);
        dw_r = b.tensor(TC_WORKSPACE, DT_FP32, Tl, m.moe_top_k);
        dlogits = b.tensor(TC_WORKSPACE, DT_BF16, Tl, m.num_experts);
    }
    auto moe_dispatch = [&](int rows, int scale, const LayerActs& a, int slab, uint16_t mb) {
        ExecOp e = xop(K_MOE_DISPATCH_GEMM);
        e.t[0] = rows; e.t[1] = a.ridx; e.t[2] = a.rpos; e.t[3] = scale; e.t[4] = a.counts; e.t[5] = slab; e.t[6] = a.cnt_recv;
        e.i[0] = m.moe_top_k; e.i[1] = m.num_experts; e.i[2] = moe_cap; e.i[3] = GROUP_EP; e.i[4] = static_cast<int32_t>(b.next_seq++);
        b.push(OP_MOE_DISPATCH_GEMM, ST_COMPUTE_HI, 0, 2.0 * Tl * m.moe_top_k * H, GROUP_EP, mb, &e);
    };
    // mode 0: out = base + sum_s w_s * slab row ; mode 1: plain sum ; mode 2: dw[t, s] = <dot_with[t], slab row>
    auto moe_combine = [&](int base, int outt, int weights, const LayerActs& a, int slab, int dot_with, int dw, bool announce,
                           uint16_t mb) {
        ExecOp e = xop(K_MOE_GEMM_COMBINE, announce ? 1 : 0);
        e.t[0] = base; e.t[1] = outt; e.t[2] = a.ridx; e.t[3] = a.rpos; e.t[4] = weights; e.t[5] = slab; e.t[6] = dot_with; e.t[7] = dw;
        e.i[0] = m.moe_top_k; e.i[1] = m.num_experts; e.i[2] = moe_cap; e.i[3] = GROUP_EP; e.i[4] = static_cast<int32_t>(b.next_seq++);
        b.push(OP_MOE_GEMM_COMBINE, ST_COMPUTE_HI, 2.0 * Tl * m.moe_top_k * H, 2.0 * Tl * m.moe_top_k * H, GROUP_EP, mb, &e);
    };
    // ---------------- activations: one set per in-flight microbatch
    const uint32_t slots = std::max<uint32_t>(1, std::min<uint32_t>(d.pp - b.stage, ga));
    out->xhdr.act_slots = slots;
    std::vector<std::vector<LayerActs>> A(slots, std::vector<LayerActs>(b.layers));
    std::vector<int> x_out(slots), hf_s(slots), hff_s(slots), rstdf_s(slots);
    // Full activation recompute keeps, per in-flight microbatch and layer, only the layer's input;
    // everything else lives once per stage and is rebuilt by re-running the layer's forward right
    // before its backward (all of it on the one compute stream, so the shared set is never contended).
    const bool recompute = m.recompute != 0;
    auto alloc_layer_rest = [&](LayerActs& a) {
        a.rstd1 = b.tensor(TC_ACTIVATION, DT_FP32, 1, Tl);
        a.xn1 = b.tensor(TC_ACTIVATION, DT_BF16, T, H);       // gathered rows (== local when tp = 1)
        a.qkv = b.tensor(TC_ACTIVATION, DT_BF16, T, b.Cqkv);
        a.ao = b.tensor(TC_ACTIVATION, DT_BF16, T, b.Hq_l);
        a.lse = b.tensor(TC_ACTIVATION, DT_FP32, b.nh_l, T);
        a.hmid = b.tensor(TC_ACTIVATION, DT_BF16, Tl, H);
        a.rstd2 = b.tensor(TC_ACTIVATION, DT_FP32, 1, Tl);
        a.xn2 = b.tensor(TC_ACTIVATION, DT_BF16, moe ? Tl : T, H);   // MoE: the router and the dispatch work on the local rows
        if (!moe) {
            a.gu = b.tensor(TC_ACTIVATION, DT_BF16, T, 2 * b.F_l);
            a.act = b.tensor(TC_ACTIVATION, DT_BF16, T, b.F_l);
        } else {
            a.logits = b.tensor(TC_ACTIVATION, DT_FP32, Tl, m.num_experts);
            a.ridx = b.tensor(TC_ACTIVATION, DT_INT32, Tl, m.moe_top_k);
            a.rw = b.tensor(TC_ACTIVATION, DT_FP32, Tl, m.moe_top_k);
            a.rpos = b.tensor(TC_ACTIVATION, DT_INT32, Tl, m.moe_top_k);
            a.counts = b.tensor(TC_ACTIVATION, DT_INT32, 1, m.num_experts);
            a.cnt_recv = b.tensor(TC_COMM, DT_INT32, 1, E_l * xg);       // written by the sending members
            a.xs = b.tensor(TC_COMM, DT_BF16, moe_rows, H);              // expert inputs, written by the senders
            a.gu = b.tensor(TC_ACTIVATION, DT_BF16, moe_rows, 2 * m.ffn_hidden);
            a.act = b.tensor(TC_ACTIVATION, DT_BF16, moe_rows, m.ffn_hidden);
            a.ys = b.tensor(TC_COMM, DT_BF16, moe_rows, H);              // expert outputs, read by the token owners
        }
    };
    LayerActs shared_acts;
    int x_scratch = -1;
    if (recompute) {
        alloc_layer_rest(shared_acts);
        x_scratch = b.tensor(TC_ACTIVATION, DT_BF16, Tl, H);   // output of a re-run layer (already consumed downstream)
    }
    for (uint32_t s = 0; s < slots; ++s) {
        for (uint32_t l = 0; l < b.layers; ++l) {
            LayerActs& a = A[s][l];
            if (recompute) a = shared_acts;
            a.x = b.tensor(TC_ACTIVATION, DT_BF16, Tl, H);
            if (!recompute) alloc_layer_rest(a);
        }
        x_out[s] = b.tensor(TC_ACTIVATION, DT_BF16, Tl, H);       // output of the stage's last layer
        if (b.last_stage) {
            rstdf_s[s] = b.tensor(TC_ACTIVATION, DT_FP32, 1, Tl);
            hf_s[s] = tp > 1 ? b.tensor(TC_ACTIVATION, DT_BF16, Tl, H) : -1;
            hff_s[s] = b.tensor(TC_ACTIVATION, DT_BF16, T, H);    // normalised final hidden, all rows
        }
    }
    (void)hf; (void)hf_full; (void)rstdf; (void)xf;

    // pipeline hand-off buffers
    const int pipe_in = !b.first_stage ? b.tensor(TC_COMM, DT_BF16, Tl, H) : -1;
    const int pipe_gin = !b.last_stage ? b.tensor(TC_COMM, DT_BF16, Tl, H) : -1;
    const uint32_t pp_prev = b.stage > 0 ? b.stage - 1 : 0, pp_next = b.stage + 1;

    const double grad_scale = 1.0 / (static_cast<double>(T) * ga);

    // ---- data-parallel gradient buckets (fused mode): reduce-scatter + AdamW (+ parameter all-gather) of a range of
    // the flat space as ONE kernel on comm_dp. With dp_buckets every layer is a bucket, launched in the last
    // microbatch's backward right after the layer's weight gradients, so it overlaps the layers below it.
    const uint32_t dp_rank = rank / (d.tp * d.pp * d.cp) % std::max(1u, d.dp);
    const bool dp_buckets = d.dp > 1 && b.fused && cfg.train.dp_buckets != 0 && tp == 1;
    // layer >= 0 with sharded gradients: the bucket reads the layer's staging buffers; `last` = the step's last
    // microbatch (the update follows the reduction), `first` = its first (the accumulator is overwritten)
    auto emit_bucket = [&](uint64_t lo, uint64_t hi, int max_ctas, uint16_t mb, int layer = -1, bool first = true, bool last = true) {
        if (hi > hdr_n_rep) hi = hdr_n_rep;
        if (lo >= hi) return;
        auto sub = [&](int flat, uint16_t tclass, uint16_t dt, uint64_t elem_off, uint64_t elems) {
            const int id = b.tensor_at(tclass, dt, out->tensors[flat].offset + elem_off * dtype_size(dt), 1, 0, 0);
            out->tensors[id].nbytes = elems * dtype_size(dt);
            return id;
        };
        // what this rank's kernel touches: everybody's gradients of the bucket are read by the owners; the owner
        // updates its part of master / m / v; parameters change in the bucket on every member (replicated) or in
        // the owner's shard (ZeRO-3)
        const bool staged = shard_grads && layer >= 0;
        const uint64_t own_lo = std::max<uint64_t>(lo, static_cast<uint64_t>(dp_rank) * hdr_n_shard);
        const uint64_t own_hi = std::min<uint64_t>(hi, static_cast<uint64_t>(dp_rank + 1) * hdr_n_shard);
        // flags: 1 parameters sharded (write my shard only), 2 a bucket (bounds in i[0..1]), 4 gradients staged per layer,
        // 8 reduce into the accumulator only (not the last microbatch), 16 overwrite the accumulator (first microbatch)
        ExecOp e = xop(K_RS_ADAMW, static_cast<uint16_t>((zero3 ? 1 : 0) | 2 | (staged ? 4 : 0) | (staged && !last ? 8 : 0) |
                                                         (staged && first ? 16 : 0)));
        e.t[3] = staged ? sub(grad_stage[layer & 1], TC_GRAD, DT_FP32, 0, hi - lo) : sub(b.flat_grad, TC_GRAD, DT_FP32, lo, hi - lo);
        if (own_lo < own_hi) {
            const uint64_t o = own_lo - static_cast<uint64_t>(dp_rank) * hdr_n_shard;
            if (!staged || last) {
                e.t[0] = sub(b.flat_master, TC_OPTSTATE, DT_FP32, o, own_hi - own_lo);
                e.t[1] = sub(b.flat_m, TC_OPTSTATE, DT_FP32, o, own_hi - own_lo);
                e.t[2] = sub(b.flat_v, TC_OPTSTATE, DT_FP32, o, own_hi - own_lo);
                if (zero3) e.t[4] = sub(b.flat_param, TC_PARAM, DT_BF16, o, own_hi - own_lo);
            }
            if (staged) e.t[5] = sub(grad_acc, TC_GRAD, DT_FP32, o, own_hi - own_lo);
        }
        // replicated parameters: the owners push the bucket's new values to every member, in the launch that updates
        // (a launch that only reduces into the accumulators touches no parameter)
        if (!zero3 && (!staged || last)) e.t[4] = sub(b.flat_param, TC_PARAM, DT_BF16, lo, hi - lo);
        e.i[0] = static_cast<int32_t>(lo >> 9); e.i[1] = static_cast<int32_t>(hi >> 9); e.i[2] = max_ctas;
        e.i[3] = GROUP_DP; e.i[4] = static_cast<int32_t>(b.next_seq++);
        e.f[0] = 1.0f / d.dp;
        b.push(OP_RS_ADAMW, ST_COMM_DP, 18.0 * (hi - lo) / d.dp, 4.0 * (hi - lo), GROUP_DP, mb, &e);   // cost: rank-independent
    };
    int stage_free_ev[2] = {-1, -1};   // sharded gradients: recorded on comm_dp after the bucket that last read a staging buffer
    std::vector<int> send_done(slots, -1);  // event recorded after a slot's activation send

    // ================================================================ forward of one layer
    auto layer_forward = [&](uint16_t mb, const LayerActs& a, const LayerParams& w, int x_next) {
        // attention block
        b.rmsnorm_fwd(a.x, w.g1.w, tp > 1 ? xn_local : a.xn1, a.rstd1, Tl, mb);
        prepare_layer(static_cast<int>(&w - L.data()), false, mb);   // ZeRO-3: this layer's weights, inside the QKV GEMM
        b.col_parallel(tp > 1 ? xn_local : a.xn1, a.xn1, w.wqkv.w, a.qkv, b.Cqkv, H, false, mb);
        {
            ExecOp e = xop(K_ROPE);
            e.t[0] = a.qkv; e.t[1] = rope_tab;
            e.i[0] = T; e.i[1] = b.seq; e.i[2] = b.nh_l; e.i[3] = b.nkv_l; e.i[4] = b.hd;
            b.push(OP_ELEMENTWISE, ST_COMPUTE_HI, 6.0 * T * (b.nh_l + b.nkv_l) * b.hd, 0, 0, mb, &e);
        }
        {
            ExecOp e = xop(K_ATTN_FWD);
            e.t[0] = a.qkv; e.t[1] = a.ao; e.t[2] = a.lse;
            e.i[0] = b.mbsz; e.i[1] = b.seq; e.i[2] = b.nh_l; e.i[3] = b.nkv_l; e.i[4] = b.hd;
            e.f[0] = 1.0f / std::sqrt(static_cast<float>(b.hd));
            b.push(OP_ATTENTION_FWD, ST_COMPUTE_HI, 2.0 * T * b.Hq_l * b.seq, 0, 0, mb, &e);
        }
        b.row_parallel(a.ao, w.wo.w, a.x, a.hmid, partial, rs_tmp, H, b.Hq_l, false, mb);
        if (moe) {
            // router -> dispatch (permute + peer stores) -> expert FFN over the slabs -> combine (peer loads)
            const uint32_t F = m.ffn_hidden, seg_m = xg * moe_cap;
            b.rmsnorm_fwd(a.hmid, w.g2.w, a.xn2, a.rstd2, Tl, mb);
            b.gemm(ST_COMPUTE_HI, a.xn2, w.wr.w, a.logits, -1, Tl, m.num_experts, H, false, false, 1, mb);
            {
                ExecOp e = xop(K_MOE_ROUTE);
                e.t[0] = a.logits; e.t[1] = a.ridx; e.t[2] = a.rw; e.t[3] = a.rpos; e.t[4] = a.counts;
                e.i[0] = Tl; e.i[1] = m.num_experts; e.i[2] = m.moe_top_k; e.i[3] = moe_cap;
                b.push(OP_ELEMENTWISE, ST_COMPUTE_HI, 10.0 * Tl * m.num_experts, 0, 0, mb, &e);
            }
            moe_dispatch(a.xn2, -1, a, a.xs, mb);
            b.gemm_grouped(a.xs, w.wgu.w, a.gu, seg_m, 2 * F, H, false, false, 0, a.cnt_recv, moe_cap, 1, E_l, mb);
            {
                ExecOp e = xop(K_SWIGLU_FWD);
                e.t[0] = a.gu; e.t[1] = a.act;
                e.i[0] = moe_rows; e.i[1] = F;
                b.push(OP_SWIGLU, ST_COMPUTE_HI, 4.0 * moe_rows * F, 0, 0, mb, &e);
            }
            b.gemm_grouped(a.act, w.wd.w, a.ys, seg_m, H, F, false, false, 0, a.cnt_recv, moe_cap, 1, E_l, mb);
            moe_combine(a.hmid, x_next, a.rw, a, a.ys, -1, -1, true, mb);
            return;
        }
        // MLP block
        b.rmsnorm_fwd(a.hmid, w.g2.w, tp > 1 ? xn_local : a.xn2, a.rstd2, Tl, mb);
        if (fuse_swiglu) {
            // gate/up product with SwiGLU in its epilogue: gu and act leave the same kernel
            b.col_parallel(tp > 1 ? xn_local : a.xn2, a.xn2, w.wgu.w, a.gu, 2 * b.F_l, H, false, mb, 4, a.act);
        } else {
            b.col_parallel(tp > 1 ? xn_local : a.xn2, a.xn2, w.wgu.w, a.gu, 2 * b.F_l, H, false, mb);
            ExecOp e = xop(K_SWIGLU_FWD);
            e.t[0] = a.gu; e.t[1] = a.act;
            e.i[0] = T; e.i[1] = b.F_l;
            b.push(OP_SWIGLU, ST_COMPUTE_HI, 4.0 * T * b.F_l, 0, 0, mb, &e);
        }
        b.row_parallel(a.act, w.wd.w, a.hmid, x_next, partial, rs_tmp, H, b.F_l, false, mb);
    };

    // ================================================================ forward of one microbatch
    auto forward = [&](uint16_t mb) {
        const uint32_t s = mb % slots;
        const int tok_mb = b.view(tokens, mb, 1);
        int x = A[s].empty() ? x_out[s] : A[s][0].x;
        if (b.first_stage) {
            if (tp == 1) {
                ExecOp e = xop(K_EMBED_FWD);
                e.t[0] = tok_mb; e.t[1] = embed.w; e.t[2] = x;
                e.i[0] = T; e.i[1] = H; e.i[2] = 0; e.i[3] = b.V_l;
                b.push(OP_ELEMENTWISE, ST_COMPUTE_HI, 0, 2.0 * T * H, 0, mb, &e);
            } else {
                // vocabulary-parallel gather: every rank fills the rows whose token it owns, the
                // reduce-scatter sums the slices and leaves each rank its rows of the sequence
                ExecOp e = xop(K_EMBED_FWD);
                e.t[0] = tok_mb; e.t[1] = embed.w; e.t[2] = partial;
                e.i[0] = T; e.i[1] = H; e.i[2] = b.tp_id * b.V_l; e.i[3] = (b.tp_id + 1) * b.V_l;
                b.push(OP_ELEMENTWISE, ST_COMPUTE_HI, 0, 2.0 * T * H, 0, mb, &e);
                b.sync(ST_COMPUTE_HI, ST_COMM_TP, mb);
                b.nccl(K_NCCL_REDUCE_SCATTER, OP_REDUCE_SCATTER, ST_COMM_TP, partial, x, static_cast<uint64_t>(Tl) * H,
                       DT_BF16, GROUP_TP, -1, mb);
                b.sync(ST_COMM_TP, ST_COMPUTE_HI, mb);
            }
        } else {
            // the slot's previous microbatch must be done with this buffer before it is refilled
            b.sync(ST_COMPUTE_HI, ST_COMM_PP, mb);
            b.nccl(K_NCCL_RECV, OP_PIPE_RECV, ST_COMM_PP, -1, x, static_cast<uint64_t>(Tl) * H, DT_BF16, GROUP_PP,
                   static_cast<int>(pp_prev), mb);
            b.sync(ST_COMM_PP, ST_COMPUTE_HI, mb);
        }
        if (send_done[s] >= 0) {
            // the activation this slot handed to the next stage must have left before it is rewritten
            b.wait(ST_COMPUTE_HI, static_cast<uint32_t>(send_done[s]), mb);
            send_done[s] = -1;
        }
        for (uint32_t l = 0; l < b.layers; ++l)
            layer_forward(mb, A[s][l], L[l], l + 1 < b.layers ? A[s][l + 1].x : x_out[s]);
        if (!b.last_stage) {
            b.sync(ST_COMPUTE_HI, ST_COMM_PP, mb);
            b.nccl(K_NCCL_SEND, OP_PIPE_SEND, ST_COMM_PP, x_out[s], -1, static_cast<uint64_t>(Tl) * H, DT_BF16, GROUP_PP,
                   static_cast<int>(pp_next), mb);
            send_done[s] = static_cast<int>(b.record(ST_COMM_PP, mb));
        } else {
            // final norm; the loss itself is computed chunk by chunk at the start of backward so
            // that the logits never exist for more than `chunk` rows
            b.rmsnorm_fwd(x_out[s], gf.w, tp > 1 ? hf_s[s] : hff_s[s], rstdf_s[s], Tl, mb);
            if (tp > 1) {
                b.sync(ST_COMPUTE_HI, ST_COMM_TP, mb);
                b.nccl(K_NCCL_ALL_GATHER, OP_ALL_GATHER, ST_COMM_TP, hf_s[s], hff_s[s], static_cast<uint64_t>(Tl) * H,
                       DT_BF16, GROUP_TP, -1, mb);
                b.sync(ST_COMM_TP, ST_COMPUTE_HI, mb);
            }
        }
    };

    // ================================================================ backward of one microbatch
    auto backward = [&](uint16_t mb) {
        const uint32_t s = mb % slots;
        const bool first_mb = mb == 0;                 // first gradient contribution overwrites
        const int wg_epi = (first_mb || shard_grads) ? 1 : 2;   // CAI_EPI_F32 / CAI_EPI_F32_ACCUM (staged gradients hold one microbatch)
        bool lo_pending = false;
        // G[M,N] (+)= A[K,M]^T * B[K,N]: a weight gradient; its operands are complete on compute_hi
        auto wgrad = [&](int A, int B, int G, uint32_t M, uint32_t N, uint32_t K) {
            if (!overlap_wgrad) {
                b.gemm(ST_COMPUTE_HI, A, B, G, -1, M, N, K, true, true, wg_epi, mb);
                return;
            }
            b.sync(ST_COMPUTE_HI, ST_COMPUTE_LO, mb);
            b.gemm(ST_COMPUTE_LO, A, B, G, -1, M, N, K, true, true, wg_epi, mb);
            lo_pending = true;
        };
        // compute_hi may overwrite what the deferred weight gradients read only after they have run
        auto join_lo = [&]() {
            if (lo_pending) b.sync(ST_COMPUTE_LO, ST_COMPUTE_HI, mb);
            lo_pending = false;
        };
        const int tok_mb = b.view(tokens, mb, 1);
        if (b.last_stage) {
            // LM head + cross-entropy, `chunk` rows at a time: logits -> dlogits in place ->
            // d(hidden) rows and the head's weight gradient.
            const int dh_rows = tp > 1 ? dhf_full : dstream;   // gradient wrt the normalised hidden, all T rows
            for (uint32_t r0 = 0; r0 < T; r0 += chunk) {
                const uint32_t rows = std::min(chunk, T - r0);
                const int hf_c = b.view(hff_s[s], r0, rows);
                const int lg = rows == chunk ? logits : b.view(logits, 0, rows);
                b.gemm(ST_COMPUTE_HI, hf_c, head.w, lg, -1, rows, b.V_l, H, false, false, 0, mb);
                ExecOp e = xop(tp > 1 ? K_CROSS_ENTROPY_TP : K_CROSS_ENTROPY);
                const int tg = b.tensor_at(TC_COMM, DT_INT32,
                                           out->tensors[targets].offset + (static_cast<uint64_t>(mb) * T + r0) * 4, 1,
                                           rows, rows);
                e.t[0] = lg; e.t[1] = tg; e.t[2] = loss_acc; e.t[3] = ce_scratch;
                e.i[0] = rows; e.i[1] = b.V_l; e.i[2] = b.tp_id * b.V_l; e.i[3] = GROUP_TP; e.i[4] = b.tp_id == 0;
                e.f[0] = static_cast<float>(grad_scale);
                e.f[1] = static_cast<float>(grad_scale / d.dp);  // reported loss is the mean over the global batch
                b.push(OP_ELEMENTWISE, ST_COMPUTE_HI, 5.0 * rows * b.V_l, 0, 0, mb, &e);
                const int dh_c = b.view(dh_rows, r0, rows);
                b.gemm(ST_COMPUTE_HI, lg, head.w, dh_c, -1, rows, H, b.V_l, false, true, 0, mb);
                b.gemm(ST_COMPUTE_HI, lg, hf_c, head.g, -1, b.V_l, H, rows, true, true,
                       (first_mb && r0 == 0) ? 1 : 2, mb);
            }
            if (tp > 1) {
                // partial sums over vocabulary shards -> rows of this rank
                b.sync(ST_COMPUTE_HI, ST_COMM_TP, mb);
                b.nccl(K_NCCL_REDUCE_SCATTER, OP_REDUCE_SCATTER, ST_COMM_TP, dhf_full, dxn, static_cast<uint64_t>(Tl) * H,
                       DT_BF16, GROUP_TP, -1, mb);
                b.sync(ST_COMM_TP, ST_COMPUTE_HI, mb);
            }
            b.rmsnorm_bwd(x_out[s], gf.w, rstdf_s[s], tp > 1 ? dxn : dstream, dstream, gf.g, norm_scratch, Tl, false,
                          !first_mb, mb);
        } else {
            // Gradients travel up the pipeline on their own stream (and communicator): with a
            // single in-order p2p stream per rank, the warm-up sends of one stage and the first
            // gradient send of the next would wait for each other.
            b.sync(ST_COMPUTE_HI, ST_IO, mb);
            b.nccl(K_NCCL_RECV, OP_PIPE_RECV, ST_IO, -1, dstream, static_cast<uint64_t>(Tl) * H, DT_BF16, GROUP_PP,
                   static_cast<int>(pp_next), mb);
            b.sync(ST_IO, ST_COMPUTE_HI, mb);
        }
        for (int l = static_cast<int>(b.layers) - 1; l >= 0; --l) {
            const LayerActs& a = A[s][l];
            const LayerParams& w = L[l];
            const int g_rows = tp > 1 ? dfull : dstream;  // all T rows of the incoming gradient
            const int g_rows_attn = tp > 1 ? dfull_attn : dstream;
            join_lo();
            if (shard_grads && stage_free_ev[l & 1] >= 0) {
                // this layer's weight gradients overwrite a staging buffer the members may still be reading
                b.wait(ST_COMPUTE_HI, static_cast<uint32_t>(stage_free_ev[l & 1]), mb);
                stage_free_ev[l & 1] = -1;
            }
            if (recompute) layer_forward(mb, a, w, x_scratch);
            if (moe) {
                const uint32_t F = m.ffn_hidden, seg_m = xg * moe_cap;
                moe_combine(-1, -1, -1, a, a.ys, dstream, dw_r, false, mb);           // dw[t,s] = <dx_next[t], y(t,s)>
                moe_dispatch(dstream, a.rw, a, dy_s, mb);                              // dy rows = w[t,s] * dx_next[t]
                b.gemm_grouped(dy_s, w.wd.w, dact_s, seg_m, F, H, false, true, 0, a.cnt_recv, moe_cap, 1, E_l, mb);
                b.gemm_grouped(dy_s, a.act, w.wd.g, H, F, seg_m, true, true, wg_epi, a.cnt_recv, moe_cap, 2, E_l, mb);
                {
                    ExecOp e = xop(K_SWIGLU_BWD);
                    e.t[0] = a.gu; e.t[1] = dact_s; e.t[2] = dgu_s;
                    e.i[0] = moe_rows; e.i[1] = F;
                    b.push(OP_SWIGLU, ST_COMPUTE_HI, 8.0 * moe_rows * F, 0, 0, mb, &e);
                }
                b.gemm_grouped(dgu_s, w.wgu.w, dx_s, seg_m, H, 2 * F, false, true, 0, a.cnt_recv, moe_cap, 1, E_l, mb);
                b.gemm_grouped(dgu_s, a.xs, w.wgu.g, 2 * F, H, seg_m, true, true, wg_epi, a.cnt_recv, moe_cap, 2, E_l, mb);
                moe_combine(-1, dxn, -1, a, dx_s, -1, -1, true, mb);                  // dxn2[t] = sum_s dx(t,s)
                {
                    ExecOp e = xop(K_MOE_ROUTE, 1);
                    e.t[0] = a.logits; e.t[1] = a.ridx; e.t[2] = dw_r; e.t[3] = a.rpos; e.t[4] = dlogits;
                    e.i[0] = Tl; e.i[1] = m.num_experts; e.i[2] = m.moe_top_k;
                    b.push(OP_ELEMENTWISE, ST_COMPUTE_HI, 20.0 * Tl * m.num_experts, 0, 0, mb, &e);
                }
                b.gemm(ST_COMPUTE_HI, dlogits, w.wr.w, dxn, dxn, Tl, H, m.num_experts, false, true, 3, mb);   // dxn2 += dlogits * Wr
                b.gemm(ST_COMPUTE_HI, dlogits, a.xn2, w.wr.g, -1, m.num_experts, H, Tl, true, true, wg_epi, mb);
                b.rmsnorm_bwd(a.hmid, w.g2.w, a.rstd2, dxn, dstream, w.g2.g, norm_scratch, Tl, true, !first_mb, mb);
            } else {
            // ---- MLP block: x_next = hmid + act * Wd^T
            prepare_layer(l, true, mb);                                                           // ZeRO-3 re-gather, top of the range first
            if (fuse_swiglu_bwd) {
                // dact = gather(dx) * Wd never reaches memory: the epilogue turns it into [dgate | dup]
                b.col_parallel(dstream, dfull, w.wd.w, dgu, b.F_l, H, true, mb, 5, a.gu);
                wgrad(g_rows, a.act, w.wd.g, H, b.F_l, T);                                        // dWd = dx^T act
            } else {
                b.col_parallel(dstream, dfull, w.wd.w, dact, b.F_l, H, true, mb);                 // dact = gather(dx) * Wd
                wgrad(g_rows, a.act, w.wd.g, H, b.F_l, T);                                        // dWd = dx^T act
                ExecOp e = xop(K_SWIGLU_BWD);
                e.t[0] = a.gu; e.t[1] = dact; e.t[2] = dgu;
                e.i[0] = T; e.i[1] = b.F_l;
                b.push(OP_SWIGLU, ST_COMPUTE_HI, 8.0 * T * b.F_l, 0, 0, mb, &e);
            }
            wgrad(dgu, a.xn2, w.wgu.g, 2 * b.F_l, H, T);
            b.row_parallel(dgu, w.wgu.w, -1, dxn, partial, rs_tmp, H, 2 * b.F_l, true, mb);        // dxn2 = RS(dgu * Wgu)
            b.rmsnorm_bwd(a.hmid, w.g2.w, a.rstd2, dxn, dstream, w.g2.g, norm_scratch, Tl, true, !first_mb, mb);
            }
            // ---- attention block: hmid = x + ao * Wo^T
            b.col_parallel(dstream, dfull_attn, w.wo.w, dao, b.Hq_l, H, true, mb);                // dao = gather(dh) * Wo
            wgrad(g_rows_attn, a.ao, w.wo.g, H, b.Hq_l, T);
            {
                auto attn_bwd = [&](uint16_t parts, uint16_t stream, double flops) {
                    ExecOp e = xop(K_ATTN_BWD, parts);
                    e.t[0] = a.qkv; e.t[1] = a.ao; e.t[2] = dao; e.t[3] = a.lse; e.t[4] = delta; e.t[5] = dqkv;
                    // a part writes only its own columns of dqkv: t[6] names them for the hazard analysis
                    if (parts == 4) e.t[6] = b.colview(dqkv, 0, b.Hq_l);
                    if (parts == 2) e.t[6] = b.colview(dqkv, b.Hq_l, b.Cqkv - b.Hq_l);
                    e.i[0] = b.mbsz; e.i[1] = b.seq; e.i[2] = b.nh_l; e.i[3] = b.nkv_l; e.i[4] = b.hd;
                    e.f[0] = 1.0f / std::sqrt(static_cast<float>(b.hd));
                    b.push(OP_ATTENTION_BWD, stream, flops, 0, 0, mb, &e);
                };
                const double flops = 4.0 * T * b.Hq_l * b.seq;
                if (!overlap_wgrad) {
                    attn_bwd(0, ST_COMPUTE_HI, flops);
                } else {
                    // few heads per GPU leave most SMs idle: dQ (on comm_dp's stream, idle during backward) runs
                    // next to dK/dV; both need delta and write disjoint columns of dqkv
                    attn_bwd(1, ST_COMPUTE_HI, 0);
                    b.sync(ST_COMPUTE_HI, ST_COMM_DP, mb);
                    attn_bwd(4, ST_COMM_DP, 0.4 * flops);
                    attn_bwd(2, ST_COMPUTE_HI, 0.6 * flops);
                    b.sync(ST_COMM_DP, ST_COMPUTE_HI, mb);
                }
            }
            {
                ExecOp e = xop(K_ROPE, 1);
                e.t[0] = dqkv; e.t[1] = rope_tab;
                e.i[0] = T; e.i[1] = b.seq; e.i[2] = b.nh_l; e.i[3] = b.nkv_l; e.i[4] = b.hd;
                b.push(OP_ELEMENTWISE, ST_COMPUTE_HI, 6.0 * T * (b.nh_l + b.nkv_l) * b.hd, 0, 0, mb, &e);
            }
            wgrad(dqkv, a.xn1, w.wqkv.g, b.Cqkv, H, T);
            b.row_parallel(dqkv, w.wqkv.w, -1, dxn, partial, rs_tmp, H, b.Cqkv, true, mb);
            b.rmsnorm_bwd(a.x, w.g1.w, a.rstd1, dxn, dstream, w.g1.g, norm_scratch, Tl, true, !first_mb, mb);
            if (dp_buckets && (shard_grads || mb + 1u == ga)) {
                // the layer's gradients are complete on this rank: its bucket goes to comm_dp and runs under the
                // backward of the layers below (a slice of the SMs is enough to keep NVLink busy). With sharded
                // gradients every microbatch's contribution is reduced into the owners' accumulators.
                b.sync(ST_COMPUTE_HI, ST_COMM_DP, mb);
                if (lo_pending) b.sync(ST_COMPUTE_LO, ST_COMM_DP, mb);
                emit_bucket(layer_range[l].first, layer_range[l].second, 64, mb, l, mb == 0, mb + 1u == ga);
                if (shard_grads) stage_free_ev[l & 1] = static_cast<int>(b.record(ST_COMM_DP, mb));
            }
        }
        join_lo();
        if (b.first_stage) {
            int drows = dstream;
            if (tp > 1) {
                b.sync(ST_COMPUTE_HI, ST_COMM_TP, mb);
                b.nccl(K_NCCL_ALL_GATHER, OP_ALL_GATHER, ST_COMM_TP, dstream, dfull, static_cast<uint64_t>(Tl) * H, DT_BF16,
                       GROUP_TP, -1, mb);
                b.sync(ST_COMM_TP, ST_COMPUTE_HI, mb);
                drows = dfull;
            }
            if (first_mb && !(b.last_stage && b.tied)) {
                ExecOp z = xop(K_ZERO);
                z.t[0] = embed.g;
                b.push(OP_ELEMENTWISE, ST_COMPUTE_HI, 0, 4.0 * b.V_l * H, 0, mb, &z);
            }
            ExecOp e = xop(K_EMBED_BWD);
            e.t[0] = tok_mb; e.t[1] = drows; e.t[2] = embed.g;
            e.i[0] = T; e.i[1] = H; e.i[2] = b.tp_id * b.V_l; e.i[3] = (b.tp_id + 1) * b.V_l;
            b.push(OP_ELEMENTWISE, ST_COMPUTE_HI, 0, 6.0 * T * H, 0, mb, &e);
        } else {
            b.sync(ST_COMPUTE_HI, ST_IO, mb);
            b.nccl(K_NCCL_SEND, OP_PIPE_SEND, ST_IO, dstream, -1, static_cast<uint64_t>(Tl) * H, DT_BF16, GROUP_PP,
                   static_cast<int>(pp_prev), mb);
            // dstream is overwritten by the next backward: the send must finish first
            b.sync(ST_IO, ST_COMPUTE_HI, mb);
        }
    };
    (void)pipe_in; (void)pipe_gin;

    // ================================================================ the step
    {
        ExecOp z = xop(K_ZERO);
        z.t[0] = loss_acc;
        b.push(OP_ELEMENTWISE, ST_COMPUTE_HI, 0, 32, 0, 0, &z);
    }
    gather_group(-1, false, false, 0);   // ZeRO-3: embedding and gains, once per step
    if (fp8 && !zero3)
        for (uint32_t l = 0; l < b.layers; ++l) quant_layer(l, 0);   // weights changed in the last optimizer step
    for (const Tick& t : schedule_1f1b(b.stage, d.pp, ga)) {
        if (t.kind == 0) forward(t.microbatch);
        else backward(t.microbatch);
    }
    // Gains of the norms are replicated over the TP group but each rank saw only its rows.
    if (tp > 1) {
        b.sync(ST_COMPUTE_HI, ST_COMM_TP, 0);
        for (const NamedTensor& nt : out->named) {
            const size_t nlen = std::strlen(nt.name);
            const bool router = moe && nlen > 3 && !std::strcmp(nt.name + nlen - 3, ".wr");   // replicated over tp like the gains
            if (nt.init_std != 0.f && !router) continue;
            if (nt.init_std < 0.f) continue;
            b.nccl(K_NCCL_ALL_REDUCE, OP_ALL_REDUCE, ST_COMM_TP, nt.grad, nt.grad, static_cast<uint64_t>(nt.rows) * nt.cols,
                   DT_FP32, GROUP_TP, -1, 0);
        }
        // each rank accumulated the loss terms of its vocabulary slice
        if (b.last_stage) b.nccl(K_NCCL_ALL_REDUCE, OP_ALL_REDUCE, ST_COMM_TP, loss_acc, loss_acc, 8, DT_FP32, GROUP_TP, -1, 0);
        b.sync(ST_COMM_TP, ST_COMPUTE_HI, 0);
    }
    // optimizer
    if (d.dp > 1 && b.last_stage) {
        b.sync(ST_COMPUTE_HI, ST_COMM_DP, 0);
        b.nccl(K_NCCL_ALL_REDUCE, OP_ALL_REDUCE, ST_COMM_DP, loss_acc, loss_acc, 8, DT_FP32, GROUP_DP, -1, 0);
        b.sync(ST_COMM_DP, ST_COMPUTE_HI, 0);
    }
    if (d.dp > 1) {
        if (b.fused) {
            b.sync(ST_COMPUTE_HI, ST_COMM_DP, 0);
            if (dp_buckets && b.layers > 0) {
                // the layers went out during the backward pass; what is left are the parameters around them
                // (embedding, final gain, head)
                emit_bucket(0, layer_range.front().first, 0, 0);
                emit_bucket(layer_range.back().second, n_rep, 0, 0);
            } else {
                ExecOp e = xop(K_RS_ADAMW, zero3 ? 1 : 0);   // flag 1: bf16 parameters are sharded too, write my shard only
                e.t[0] = b.flat_master; e.t[1] = b.flat_m; e.t[2] = b.flat_v; e.t[3] = b.flat_grad; e.t[4] = b.flat_param;
                e.i[0] = static_cast<int32_t>(n_rep & 0xFFFFFFFFu); e.i[1] = static_cast<int32_t>(n_rep >> 32);
                e.i[2] = static_cast<int32_t>(n_shard & 0xFFFFFFFFu); e.i[3] = GROUP_DP; e.i[4] = static_cast<int32_t>(b.next_seq++);
                e.f[0] = 1.0f / d.dp;
                b.push(OP_RS_ADAMW, ST_COMM_DP, 18.0 * n_shard, 4.0 * n_rep, GROUP_DP, 0, &e);
            }
            b.sync(ST_COMM_DP, ST_COMPUTE_HI, 0);
            if (n_exp) {
                // the experts this rank owns: plain AdamW on the tail of the flat space
                auto tail = [&](int flat, uint16_t tclass, uint16_t dt, uint64_t elem_off) {
                    const TensorDesc& ft = out->tensors[flat];
                    const int id = b.tensor_at(tclass, dt, ft.offset + elem_off * dtype_size(dt), 1, 0, 0);
                    out->tensors[id].nbytes = n_exp * dtype_size(dt);
                    return id;
                };
                ExecOp x = xop(K_ADAMW);
                x.t[0] = tail(b.flat_master, TC_OPTSTATE, DT_FP32, n_shard);
                x.t[1] = tail(b.flat_m, TC_OPTSTATE, DT_FP32, n_shard);
                x.t[2] = tail(b.flat_v, TC_OPTSTATE, DT_FP32, n_shard);
                x.t[3] = tail(b.flat_grad, TC_GRAD, DT_FP32, n_rep);
                x.t[4] = tail(b.flat_param, TC_PARAM, DT_BF16, n_rep);
                x.i[0] = static_cast<int32_t>(n_exp & 0xFFFFFFFFu); x.i[1] = static_cast<int32_t>(n_exp >> 32);
                x.f[0] = 1.0f / d.dp;  // every expert sees tokens of all replicas, each scaled for its local mean
                b.push(OP_OPTIMIZER, ST_COMPUTE_HI, 18.0 * n_exp, 0, 0, 0, &x);
            }
        } else {
            // baseline: all-reduce the gradients, every rank updates everything
            b.sync(ST_COMPUTE_HI, ST_COMM_DP, 0);
            b.nccl(K_NCCL_ALL_REDUCE, OP_ALL_REDUCE, ST_COMM_DP, b.flat_grad, b.flat_grad, n_flat, DT_FP32, GROUP_DP, -1, 0);
            b.sync(ST_COMM_DP, ST_COMPUTE_LO, 0);
            ExecOp e = xop(K_ADAMW);
            e.t[0] = b.flat_master; e.t[1] = b.flat_m; e.t[2] = b.flat_v; e.t[3] = b.flat_grad; e.t[4] = b.flat_param;
            e.i[0] = static_cast<int32_t>(n_flat & 0xFFFFFFFFu); e.i[1] = static_cast<int32_t>(n_flat >> 32);
            e.f[0] = 1.0f / d.dp;
            b.push(OP_OPTIMIZER, ST_COMPUTE_LO, 18.0 * n_flat, 0, 0, 0, &e);
            b.sync(ST_COMPUTE_LO, ST_COMPUTE_HI, 0);
        }
    } else {
        ExecOp e = xop(K_ADAMW);
        e.t[0] = b.flat_master; e.t[1] = b.flat_m; e.t[2] = b.flat_v; e.t[3] = b.flat_grad; e.t[4] = b.flat_param;
        e.i[0] = static_cast<int32_t>(n_flat & 0xFFFFFFFFu); e.i[1] = static_cast<int32_t>(n_flat >> 32);
        e.f[0] = 1.0f;
        b.push(OP_OPTIMIZER, ST_COMPUTE_HI, 18.0 * n_flat, 0, 0, 0, &e);
    }

    // ---------------- arena
    uint64_t want[TC_COUNT];
    // every class segment ends with guard bytes that no tensor covers: the runtime fills them with a pattern and
    // checks them in debug runs, so a kernel that runs past the last tensor of one class into the next is caught
    for (int c = 0; c < TC_COUNT; ++c) want[c] = align_up(b.cursor[c], kTensorAlign) + (b.cursor[c] ? kSegmentGuardBytes : 0);
    Arena arena;
    arena_layout(&arena, want);
    arena_relocate(arena, out->tensors.data(), static_cast<uint32_t>(out->tensors.size()));
    // named tensors keep the flat offset (units of 512 elements) in `master`
    h.num_tensors = static_cast<uint32_t>(out->tensors.size());
    h.num_groups = static_cast<uint32_t>(out->groups.size());
    h.num_ops = static_cast<uint32_t>(out->ops.size());
    h.num_events = b.next_event;
    h.arena_bytes = arena.total;
    // well-known tensors for the runtime
    out->xhdr.num_exec = static_cast<uint32_t>(out->exec.size());
    out->xhdr.num_named = static_cast<uint32_t>(out->named.size());
    NamedTensor wk{};
    auto well_known = [&](const char* name, int id) {
        NamedTensor nt{};
        std::snprintf(nt.name, sizeof nt.name, "%s", name);
        nt.tensor = id;
        nt.grad = -1;
        nt.master = -1;
        nt.rows = id >= 0 ? b.rows_of(id) : 0;
        nt.cols = id >= 0 ? b.cols_of(id) : 0;
        nt.init_std = -1.f;  // marks a runtime buffer, not a parameter
        out->named.push_back(nt);
    };
    (void)wk;
    well_known("@tokens", tokens);
    well_known("@targets", targets);
    well_known("@loss", loss_acc);
    well_known("@signals", signals);
    well_known("@rope_table", rope_tab);
    well_known("@flat_param", b.flat_param);
    well_known("@flat_grad", b.flat_grad);
    well_known("@flat_master", b.flat_master);
    well_known("@flat_m", b.flat_m);
    well_known("@flat_v", b.flat_v);
    {
        // split of the flat space: [0, n_rep) replicated over dp (optimizer shard n_shard), rest local experts
        NamedTensor nt{};
        std::snprintf(nt.name, sizeof nt.name, "@flat_split");
        nt.tensor = -1; nt.grad = -1;
        nt.master = static_cast<int32_t>(hdr_n_rep >> 9);
        nt.rows = static_cast<uint32_t>(hdr_n_shard >> 9);
        nt.cols = 0;
        nt.init_std = -1.f;
        out->named.push_back(nt);
    }
    out->xhdr.num_named = static_cast<uint32_t>(out->named.size());
    return OK;
}

}  // namespace cai
