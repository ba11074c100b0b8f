// refmodel.cc - fp64 oracle (see refmodel.h). Straightforward loops, no blocking, no threads: the
// point is to be obviously right; the loop orders are chosen so that this costs little time.
#include "refmodel.h"

#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace cai {

namespace {

// The three matrix products. Every output element sums its K (or M) products in increasing index order, exactly as
// the textbook triple loop does, and no fused multiply-add is used, so the results are bit-identical to it. The loops
// are only arranged so that the innermost one walks contiguous memory and carries no dependency from one iteration to
// the next (a running sum in the innermost loop is bound by the latency of one floating-point add per product), four
// rows of the second operand are folded into a pass over the output row, and on x86-64 the compiler also emits an AVX2
// clone of each (picked at load time), which changes the width of the loop and not the arithmetic.
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
#define CAI_REF_KERNEL __attribute__((target_clones("avx2", "default"), optimize("O3", "fp-contract=off")))
#elif defined(__GNUC__) && !defined(__clang__)
#define CAI_REF_KERNEL __attribute__((optimize("O3", "fp-contract=off")))
#else
#define CAI_REF_KERNEL
#endif

// y[0..N) += sum over r of coef[r] * rows[r][0..N), r ascending per element (n_rows <= 4)
static inline __attribute__((always_inline)) void fold_rows(double* __restrict y, const double* __restrict b, size_t ldb, const double* coef, int n_rows, int N) {
    if (n_rows == 4) {
        const double c0 = coef[0], c1 = coef[1], c2 = coef[2], c3 = coef[3];
        const double *b0 = b, *b1 = b + ldb, *b2 = b + 2 * ldb, *b3 = b + 3 * ldb;
        for (int j = 0; j < N; ++j) {
            double t = y[j];
            t += c0 * b0[j];
            t += c1 * b1[j];
            t += c2 * b2[j];
            t += c3 * b3[j];
            y[j] = t;
        }
        return;
    }
    for (int r = 0; r < n_rows; ++r) {
        const double c = coef[r];
        const double* br = b + (size_t)r * ldb;
        for (int j = 0; j < N; ++j) y[j] += c * br[j];
    }
}

// y[M,N] (+)= a[M,K] * b[K,N]
CAI_REF_KERNEL void mm(const double* a, const double* b, double* y, int M, int K, int N, bool acc) {
    for (int i = 0; i < M; ++i) {
        double* yr = y + (size_t)i * N;
        if (!acc)
            for (int j = 0; j < N; ++j) yr[j] = 0.0;
        for (int k = 0; k < K; k += 4)
            fold_rows(yr, b + (size_t)k * N, (size_t)N, a + (size_t)i * K + k, K - k < 4 ? K - k : 4, N);
    }
}
// y[M,N] (+)= a[M,K] * b[N,K]^T: b is transposed once (exact) and the product above does the rest
void mm_nt(const double* a, const double* b, double* y, int M, int K, int N, bool acc) {
    std::vector<double> bt((size_t)K * N);
    for (int j = 0; j < N; ++j)
        for (int k = 0; k < K; ++k) bt[(size_t)k * N + j] = b[(size_t)j * K + k];
    mm(a, bt.data(), y, M, K, N, acc);
}
// y[K,N] (+)= a[M,K]^T * b[M,N]  (per output row k: the rows of b folded in, four at a time, in increasing i)
CAI_REF_KERNEL void mm_tn(const double* a, const double* b, double* y, int M, int K, int N, bool acc) {
    if (!acc)
        for (size_t n = 0; n < (size_t)K * N; ++n) y[n] = 0.0;
    for (int i = 0; i < M; i += 4) {
        const int rows = M - i < 4 ? M - i : 4;
        for (int k = 0; k < K; ++k) {
            double coef[4] = {0, 0, 0, 0};
            for (int r = 0; r < rows; ++r) coef[r] = a[(size_t)(i + r) * K + k];
            fold_rows(y + (size_t)k * N, b + (size_t)i * N, (size_t)N, coef, rows, N);
        }
    }
}

void rms_fwd(const double* x, const double* g, double* y, double* recip, int rows, int H, double eps) {
    for (int r = 0; r < rows; ++r) {
        const double* xr = x + (size_t)r * H;
        double ms = 0;
        for (int j = 0; j < H; ++j) ms += xr[j] * xr[j];
        const double rr = 1.0 / std::sqrt(ms / H + eps);
        recip[r] = rr;
        for (int j = 0; j < H; ++j) y[(size_t)r * H + j] = xr[j] * rr * g[j];
    }
}
// dx (+)= d(rmsnorm)/dx * dy ; dg += sum_rows dy * xhat
void rms_bwd(const double* x, const double* g, const double* recip, const double* dy, double* dx, double* dg, int rows,
             int H, bool dx_acc) {
    for (int r = 0; r < rows; ++r) {
        const double *xr = x + (size_t)r * H, *dyr = dy + (size_t)r * H;
        const double rr = recip[r];
        double S = 0;
        for (int j = 0; j < H; ++j) S += dyr[j] * g[j] * xr[j];
        for (int j = 0; j < H; ++j) {
            const double v = rr * dyr[j] * g[j] - rr * rr * rr * xr[j] * S / H;
            double& o = dx[(size_t)r * H + j];
            o = dx_acc ? o + v : v;
            dg[j] += dyr[j] * xr[j] * rr;
        }
    }
}

struct Rng {
    uint64_t s;
    double uniform() {  // xorshift64 (13, 7, 17) -> (0, 1), the generator the reference uses
        s ^= s << 13;
        s ^= s >> 7;
        s ^= s << 17;
        return ((s >> 11) + 1.0) / 9007199254740994.0;
    }
    double normal() {
        const double u1 = uniform(), u2 = uniform();
        return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2);
    }
};

}  // namespace

RefModel::RefModel(const RefSpec& spec, uint64_t seed) : s_(spec) {
    Hq_ = s_.n_heads * s_.head_dim;
    Hkv_ = s_.n_kv_heads * s_.head_dim;
    const int H = s_.hidden, F = s_.ffn, V = s_.vocab;
    size_t o = 0;
    auto take = [&](size_t n) { size_t at = o; o += n; return at; };
    oE_ = take((size_t)V * H);
    oP_ = take(s_.rope ? 0 : (size_t)s_.seq * H);
    ogf_ = take(H);
    lo_.resize(s_.layers);
    for (LayerOff& l : lo_) {
        l.g1 = take(H);
        l.Wq = take((size_t)H * Hq_);
        l.Wk = take((size_t)H * Hkv_);
        l.Wv = take((size_t)H * Hkv_);
        l.Wo = take((size_t)Hq_ * H);
        l.g2 = take(H);
        const size_t ne = s_.experts > 0 ? s_.experts : 1;
        l.Wg = take(ne * H * F);
        l.Wu = take(ne * H * F);
        l.Wd = take(ne * F * H);
        l.Wr = take(s_.experts > 0 ? (size_t)H * s_.experts : 0);
    }
    ohead_ = s_.tied ? oE_ : take((size_t)V * H);
    p_.assign(o, 0.0);
    g_.assign(o, 0.0);
    mom_.assign(o, 0.0);
    vel_.assign(o, 0.0);

    // Same draw order as the reference (E, P, then per layer q/k/v interleaved, o, gate/up interleaved,
    // down), so a multi-head model with the reference init starts from the reference's weights.
    Rng rng{seed ? seed : 0x2545F4914F6CDD1Dull};
    const double std_all = s_.init_std;
    const double se = std_all > 0 ? std_all : 0.02;
    for (size_t i = 0; i < (size_t)V * H; ++i) p_[oE_ + i] = se * rng.normal();
    if (!s_.rope)
        for (size_t i = 0; i < (size_t)s_.seq * H; ++i) p_[oP_ + i] = se * rng.normal();
    for (int j = 0; j < H; ++j) p_[ogf_ + j] = 1.0;
    for (const LayerOff& l : lo_) {
        for (int j = 0; j < H; ++j) p_[l.g1 + j] = p_[l.g2 + j] = 1.0;
        const double sq = std_all > 0 ? std_all : 1.0 / std::sqrt((double)H);
        const double so = std_all > 0 ? std_all : 1.0 / std::sqrt((double)Hq_);
        const double sd = std_all > 0 ? std_all : 1.0 / std::sqrt((double)F);
        if (Hkv_ == Hq_) {
            for (size_t i = 0; i < (size_t)H * Hq_; ++i) {
                p_[l.Wq + i] = sq * rng.normal();
                p_[l.Wk + i] = sq * rng.normal();
                p_[l.Wv + i] = sq * rng.normal();
            }
        } else {
            for (size_t i = 0; i < (size_t)H * Hq_; ++i) p_[l.Wq + i] = sq * rng.normal();
            for (size_t i = 0; i < (size_t)H * Hkv_; ++i) {
                p_[l.Wk + i] = sq * rng.normal();
                p_[l.Wv + i] = sq * rng.normal();
            }
        }
        for (size_t i = 0; i < (size_t)Hq_ * H; ++i) p_[l.Wo + i] = so * rng.normal();
        const size_t ne = s_.experts > 0 ? s_.experts : 1;
        for (size_t e = 0; e < ne; ++e) {
            for (size_t i = 0; i < (size_t)H * F; ++i) {
                p_[l.Wg + e * H * F + i] = sq * rng.normal();
                p_[l.Wu + e * H * F + i] = sq * rng.normal();
            }
            for (size_t i = 0; i < (size_t)F * H; ++i) p_[l.Wd + e * F * H + i] = sd * rng.normal();
        }
        if (s_.experts > 0)
            for (size_t i = 0; i < (size_t)H * s_.experts; ++i) p_[l.Wr + i] = sq * rng.normal();
    }
    if (!s_.tied)
        for (size_t i = 0; i < (size_t)V * H; ++i) p_[ohead_ + i] = se * rng.normal();
}

size_t RefModel::offset(const char* name, size_t* count) const {
    const int H = s_.hidden, F = s_.ffn, V = s_.vocab;
    size_t n = 0, at = (size_t)-1;
    const std::string nm = name;
    if (nm == "E") { at = oE_; n = (size_t)V * H; }
    else if (nm == "P" && !s_.rope) { at = oP_; n = (size_t)s_.seq * H; }
    else if (nm == "gf") { at = ogf_; n = H; }
    else if (nm == "head") { at = ohead_; n = (size_t)V * H; }
    else if (nm.size() > 2 && nm[0] == 'L') {
        const size_t dot = nm.find('.');
        const int l = std::atoi(nm.substr(1, dot - 1).c_str());
        if (dot != std::string::npos && l >= 0 && l < s_.layers) {
            const std::string f = nm.substr(dot + 1);
            const LayerOff& L = lo_[l];
            if (f == "g1") { at = L.g1; n = H; }
            else if (f == "Wq") { at = L.Wq; n = (size_t)H * Hq_; }
            else if (f == "Wk") { at = L.Wk; n = (size_t)H * Hkv_; }
            else if (f == "Wv") { at = L.Wv; n = (size_t)H * Hkv_; }
            else if (f == "Wo") { at = L.Wo; n = (size_t)Hq_ * H; }
            else if (f == "g2") { at = L.g2; n = H; }
            else if (f == "Wg") { at = L.Wg; n = (size_t)H * F * (s_.experts > 0 ? s_.experts : 1); }
            else if (f == "Wu") { at = L.Wu; n = (size_t)H * F * (s_.experts > 0 ? s_.experts : 1); }
            else if (f == "Wd") { at = L.Wd; n = (size_t)F * H * (s_.experts > 0 ? s_.experts : 1); }
            else if (f == "Wr" && s_.experts > 0) { at = L.Wr; n = (size_t)H * s_.experts; }
        }
    }
    if (count) *count = n;
    return at;
}

// Rotate-half rotary embedding on x[B*T, heads*hd]; position = index inside the sequence.
void RefModel::rope_apply(std::vector<double>& x, int B, int heads, bool inverse) const {
    const int T = s_.seq, hd = s_.head_dim, half = hd / 2, W = heads * hd;
    for (int b = 0; b < B; ++b)
        for (int t = 0; t < T; ++t)
            for (int h = 0; h < heads; ++h) {
                double* v = x.data() + ((size_t)(b * T + t) * W) + h * hd;
                for (int i = 0; i < half; ++i) {
                    const double ang = t * std::pow(s_.rope_theta, -(double)i / half);
                    const double c = std::cos(ang), sn = inverse ? -std::sin(ang) : std::sin(ang);
                    const double a = v[i], bb = v[i + half];
                    v[i] = a * c - bb * sn;
                    v[i + half] = bb * c + a * sn;
                }
            }
}

}  // namespace cai

namespace cai {

double RefModel::forward(int B, const int* tokens, const int* targets) {
    const int T = s_.seq, H = s_.hidden, F = s_.ffn, V = s_.vocab, L = s_.layers, nh = s_.n_heads, hd = s_.head_dim;
    const int BT = B * T, rep = nh / s_.n_kv_heads;
    B_ = B;
    acts_.resize(L);
    std::vector<double> x((size_t)BT * H);
    for (int i = 0; i < BT; ++i) {
        const int tok = tokens[i], t = i % T;
        for (int j = 0; j < H; ++j)
            x[(size_t)i * H + j] = p_[oE_ + (size_t)tok * H + j] + (s_.rope ? 0.0 : p_[oP_ + (size_t)t * H + j]);
    }
    const double scale = 1.0 / std::sqrt((double)hd);
    for (int l = 0; l < L; ++l) {
        LayerAct& a = acts_[l];
        const LayerOff& o = lo_[l];
        a.x = x;
        a.r1.assign(BT, 0); a.x1.assign((size_t)BT * H, 0);
        rms_fwd(a.x.data(), &p_[o.g1], a.x1.data(), a.r1.data(), BT, H, s_.eps);
        a.Q.assign((size_t)BT * Hq_, 0); a.K.assign((size_t)BT * Hkv_, 0); a.V.assign((size_t)BT * Hkv_, 0);
        mm(a.x1.data(), &p_[o.Wq], a.Q.data(), BT, H, Hq_, false);
        mm(a.x1.data(), &p_[o.Wk], a.K.data(), BT, H, Hkv_, false);
        mm(a.x1.data(), &p_[o.Wv], a.V.data(), BT, H, Hkv_, false);
        if (s_.rope) {
            rope_apply(a.Q, B, nh, false);
            rope_apply(a.K, B, s_.n_kv_heads, false);
        }
        a.probs.assign((size_t)B * nh * T * T, 0);
        a.ctx.assign((size_t)BT * Hq_, 0);
        for (int b = 0; b < B; ++b)
            for (int h = 0; h < nh; ++h) {
                const int g = h / rep;
                for (int i = 0; i < T; ++i) {
                    const double* qi = &a.Q[(size_t)(b * T + i) * Hq_ + h * hd];
                    double* pr = &a.probs[(((size_t)(b * nh + h) * T) + i) * T];
                    double mx = -1e30;
                    for (int j = 0; j <= i; ++j) {
                        const double* kj = &a.K[(size_t)(b * T + j) * Hkv_ + g * hd];
                        double sc = 0;
                        for (int d = 0; d < hd; ++d) sc += qi[d] * kj[d];
                        sc *= scale;
                        pr[j] = sc;
                        if (sc > mx) mx = sc;
                    }
                    double sum = 0;
                    for (int j = 0; j <= i; ++j) { pr[j] = std::exp(pr[j] - mx); sum += pr[j]; }
                    for (int j = 0; j <= i; ++j) pr[j] /= sum;
                    double* ci = &a.ctx[(size_t)(b * T + i) * Hq_ + h * hd];
                    for (int j = 0; j <= i; ++j) {
                        const double* vj = &a.V[(size_t)(b * T + j) * Hkv_ + g * hd];
                        for (int d = 0; d < hd; ++d) ci[d] += pr[j] * vj[d];
                    }
                }
            }
        a.hmid.assign((size_t)BT * H, 0);
        mm(a.ctx.data(), &p_[o.Wo], a.hmid.data(), BT, Hq_, H, false);
        for (size_t i = 0; i < a.hmid.size(); ++i) a.hmid[i] += a.x[i];
        a.r2.assign(BT, 0); a.x2.assign((size_t)BT * H, 0);
        rms_fwd(a.hmid.data(), &p_[o.g2], a.x2.data(), a.r2.data(), BT, H, s_.eps);
        if (s_.experts > 0) {
            // mixture of experts: softmax router, top-k (ties to the lower index), weights renormalised over the k
            const int E = s_.experts, k = s_.top_k;
            a.rprob.assign((size_t)BT * E, 0);
            mm(a.x2.data(), &p_[o.Wr], a.rprob.data(), BT, H, E, false);
            a.ridx.assign((size_t)BT * k, 0); a.rw.assign((size_t)BT * k, 0);
            a.gate.assign((size_t)BT * k * F, 0); a.up.assign((size_t)BT * k * F, 0); a.act.assign((size_t)BT * k * F, 0);
            a.yexp.assign((size_t)BT * k * H, 0);
            for (int i = 0; i < BT; ++i) {
                double* pr = &a.rprob[(size_t)i * E];
                double mx = pr[0], sum = 0;
                for (int e = 1; e < E; ++e) mx = std::max(mx, pr[e]);
                for (int e = 0; e < E; ++e) { pr[e] = std::exp(pr[e] - mx); sum += pr[e]; }
                for (int e = 0; e < E; ++e) pr[e] /= sum;
                double S = 0;
                for (int s2 = 0; s2 < k; ++s2) {
                    int best = -1;
                    for (int e = 0; e < E; ++e) {
                        bool taken = false;
                        for (int q = 0; q < s2; ++q) taken = taken || a.ridx[(size_t)i * k + q] == e;
                        if (!taken && (best < 0 || pr[e] > pr[best])) best = e;
                    }
                    a.ridx[(size_t)i * k + s2] = best;
                    S += pr[best];
                }
                for (int s2 = 0; s2 < k; ++s2) {
                    const int e = a.ridx[(size_t)i * k + s2];
                    const size_t r = (size_t)i * k + s2;
                    a.rw[r] = pr[e] / S;
                    mm(&a.x2[(size_t)i * H], &p_[o.Wg + (size_t)e * H * F], &a.gate[r * F], 1, H, F, false);
                    mm(&a.x2[(size_t)i * H], &p_[o.Wu + (size_t)e * H * F], &a.up[r * F], 1, H, F, false);
                    for (int j = 0; j < F; ++j) {
                        const double g = a.gate[r * F + j];
                        a.act[r * F + j] = g / (1.0 + std::exp(-g)) * a.up[r * F + j];
                    }
                    mm(&a.act[r * F], &p_[o.Wd + (size_t)e * F * H], &a.yexp[r * H], 1, F, H, false);
                }
                for (int j = 0; j < H; ++j) {
                    double y = a.hmid[(size_t)i * H + j];
                    for (int s2 = 0; s2 < k; ++s2) y += a.rw[(size_t)i * k + s2] * a.yexp[((size_t)i * k + s2) * H + j];
                    x[(size_t)i * H + j] = y;
                }
            }
            continue;
        }
        a.gate.assign((size_t)BT * F, 0); a.up.assign((size_t)BT * F, 0); a.act.assign((size_t)BT * F, 0);
        mm(a.x2.data(), &p_[o.Wg], a.gate.data(), BT, H, F, false);
        mm(a.x2.data(), &p_[o.Wu], a.up.data(), BT, H, F, false);
        for (size_t i = 0; i < a.act.size(); ++i) a.act[i] = a.gate[i] / (1.0 + std::exp(-a.gate[i])) * a.up[i];
        mm(a.act.data(), &p_[o.Wd], x.data(), BT, F, H, false);
        for (size_t i = 0; i < x.size(); ++i) x[i] += a.hmid[i];
    }
    xlast_ = x;
    rf_.assign(BT, 0); hf_.assign((size_t)BT * H, 0);
    rms_fwd(xlast_.data(), &p_[ogf_], hf_.data(), rf_.data(), BT, H, s_.eps);
    logits_.assign((size_t)BT * V, 0);
    mm_nt(hf_.data(), &p_[ohead_], logits_.data(), BT, H, V, false);
    sm_.assign((size_t)BT * V, 0);
    double loss = 0;
    for (int i = 0; i < BT; ++i) {
        const double* lr = &logits_[(size_t)i * V];
        double mx = lr[0];
        for (int j = 1; j < V; ++j) mx = std::max(mx, lr[j]);
        double sum = 0;
        for (int j = 0; j < V; ++j) { sm_[(size_t)i * V + j] = std::exp(lr[j] - mx); sum += sm_[(size_t)i * V + j]; }
        for (int j = 0; j < V; ++j) sm_[(size_t)i * V + j] /= sum;
        loss += -std::log(sm_[(size_t)i * V + targets[i]] + 1e-30);
    }
    return loss / BT;
}

void RefModel::backward(int B, const int* tokens, const int* targets) {
    const int T = s_.seq, H = s_.hidden, F = s_.ffn, V = s_.vocab, L = s_.layers, nh = s_.n_heads, hd = s_.head_dim;
    const int BT = B * T, rep = nh / s_.n_kv_heads;
    std::fill(g_.begin(), g_.end(), 0.0);
    std::vector<double> dlog((size_t)BT * V);
    for (int i = 0; i < BT; ++i)
        for (int j = 0; j < V; ++j) dlog[(size_t)i * V + j] = (sm_[(size_t)i * V + j] - (j == targets[i] ? 1.0 : 0.0)) / BT;
    std::vector<double> dhf((size_t)BT * H), dstream((size_t)BT * H);
    mm(dlog.data(), &p_[ohead_], dhf.data(), BT, V, H, false);           // dhf = dlog * head
    mm_tn(dlog.data(), hf_.data(), &g_[ohead_], BT, V, H, true);         // dhead += dlog^T hf
    rms_bwd(xlast_.data(), &p_[ogf_], rf_.data(), dhf.data(), dstream.data(), &g_[ogf_], BT, H, false);
    const double scale = 1.0 / std::sqrt((double)hd);
    std::vector<double> dact, dgate, dup, dx2, dctx, dQ, dK, dV, dx1, dp(T);
    for (int l = L - 1; l >= 0; --l) {
        const LayerAct& a = acts_[l];
        const LayerOff& o = lo_[l];
        if (s_.experts > 0) {
            const int E = s_.experts, k = s_.top_k;
            dx2.assign((size_t)BT * H, 0);
            std::vector<double> dy(H), da(F), dg(F), du(F), dwv(k), dprob(E), dlogit(E);
            for (int i = 0; i < BT; ++i) {
                const double* ds = &dstream[(size_t)i * H];
                const double* pr = &a.rprob[(size_t)i * E];
                double S = 0;
                for (int s2 = 0; s2 < k; ++s2) S += pr[a.ridx[(size_t)i * k + s2]];
                for (int s2 = 0; s2 < k; ++s2) {
                    const size_t r = (size_t)i * k + s2;
                    const int e = a.ridx[r];
                    double dot = 0;
                    for (int j = 0; j < H; ++j) { dot += ds[j] * a.yexp[r * H + j]; dy[j] = a.rw[r] * ds[j]; }
                    dwv[s2] = dot;
                    // expert e: y = act Wd, act = silu(gate) up, gate = x2 Wg, up = x2 Wu
                    mm_nt(dy.data(), &p_[o.Wd + (size_t)e * F * H], da.data(), 1, H, F, false);
                    mm_tn(&a.act[r * F], dy.data(), &g_[o.Wd + (size_t)e * F * H], 1, F, H, true);
                    for (int j = 0; j < F; ++j) {
                        const double g = a.gate[r * F + j], sg = 1.0 / (1.0 + std::exp(-g));
                        du[j] = da[j] * g * sg;
                        dg[j] = da[j] * a.up[r * F + j] * sg * (1.0 + g * (1.0 - sg));
                    }
                    mm_nt(dg.data(), &p_[o.Wg + (size_t)e * H * F], &dx2[(size_t)i * H], 1, F, H, true);
                    mm_nt(du.data(), &p_[o.Wu + (size_t)e * H * F], &dx2[(size_t)i * H], 1, F, H, true);
                    mm_tn(&a.x2[(size_t)i * H], dg.data(), &g_[o.Wg + (size_t)e * H * F], 1, H, F, true);
                    mm_tn(&a.x2[(size_t)i * H], du.data(), &g_[o.Wu + (size_t)e * H * F], 1, H, F, true);
                }
                // weights w_s = p_s / S over the chosen experts, then the softmax
                double gw = 0;
                for (int s2 = 0; s2 < k; ++s2) gw += dwv[s2] * a.rw[(size_t)i * k + s2];
                std::fill(dprob.begin(), dprob.end(), 0.0);
                for (int s2 = 0; s2 < k; ++s2) dprob[a.ridx[(size_t)i * k + s2]] = (dwv[s2] - gw) / S;
                double gp = 0;
                for (int e = 0; e < E; ++e) gp += dprob[e] * pr[e];
                for (int e = 0; e < E; ++e) dlogit[e] = pr[e] * (dprob[e] - gp);
                mm_nt(dlogit.data(), &p_[o.Wr], &dx2[(size_t)i * H], 1, E, H, true);
                mm_tn(&a.x2[(size_t)i * H], dlogit.data(), &g_[o.Wr], 1, H, E, true);
            }
            rms_bwd(a.hmid.data(), &p_[o.g2], a.r2.data(), dx2.data(), dstream.data(), &g_[o.g2], BT, H, true);
        } else {
        // MLP: x_next = hmid + act Wd
        dact.assign((size_t)BT * F, 0);
        mm_nt(dstream.data(), &p_[o.Wd], dact.data(), BT, H, F, false);
        mm_tn(a.act.data(), dstream.data(), &g_[o.Wd], BT, F, H, true);
        dgate.assign((size_t)BT * F, 0); dup.assign((size_t)BT * F, 0);
        for (size_t i = 0; i < dact.size(); ++i) {
            const double sg = 1.0 / (1.0 + std::exp(-a.gate[i]));
            dup[i] = dact[i] * a.gate[i] * sg;
            dgate[i] = dact[i] * a.up[i] * sg * (1.0 + a.gate[i] * (1.0 - sg));
        }
        dx2.assign((size_t)BT * H, 0);
        mm_nt(dgate.data(), &p_[o.Wg], dx2.data(), BT, F, H, false);
        mm_nt(dup.data(), &p_[o.Wu], dx2.data(), BT, F, H, true);
        mm_tn(a.x2.data(), dgate.data(), &g_[o.Wg], BT, H, F, true);
        mm_tn(a.x2.data(), dup.data(), &g_[o.Wu], BT, H, F, true);
        rms_bwd(a.hmid.data(), &p_[o.g2], a.r2.data(), dx2.data(), dstream.data(), &g_[o.g2], BT, H, true);
        }
        // attention: hmid = x + ctx Wo
        dctx.assign((size_t)BT * Hq_, 0);
        mm_nt(dstream.data(), &p_[o.Wo], dctx.data(), BT, H, Hq_, false);
        mm_tn(a.ctx.data(), dstream.data(), &g_[o.Wo], BT, Hq_, H, true);
        dQ.assign((size_t)BT * Hq_, 0); dK.assign((size_t)BT * Hkv_, 0); dV.assign((size_t)BT * Hkv_, 0);
        for (int b = 0; b < B; ++b)
            for (int h = 0; h < nh; ++h) {
                const int g = h / rep;
                for (int i = 0; i < T; ++i) {
                    const double* pr = &a.probs[(((size_t)(b * nh + h) * T) + i) * T];
                    const double* dci = &dctx[(size_t)(b * T + i) * Hq_ + h * hd];
                    double sps = 0;
                    for (int j = 0; j <= i; ++j) {
                        const double* vj = &a.V[(size_t)(b * T + j) * Hkv_ + g * hd];
                        double d = 0;
                        for (int dd = 0; dd < hd; ++dd) d += dci[dd] * vj[dd];
                        dp[j] = d;
                        sps += pr[j] * d;
                        double* dvj = &dV[(size_t)(b * T + j) * Hkv_ + g * hd];
                        for (int dd = 0; dd < hd; ++dd) dvj[dd] += pr[j] * dci[dd];
                    }
                    const double* qi = &a.Q[(size_t)(b * T + i) * Hq_ + h * hd];
                    double* dqi = &dQ[(size_t)(b * T + i) * Hq_ + h * hd];
                    for (int j = 0; j <= i; ++j) {
                        const double ds = pr[j] * (dp[j] - sps) * scale;
                        const double* kj = &a.K[(size_t)(b * T + j) * Hkv_ + g * hd];
                        double* dkj = &dK[(size_t)(b * T + j) * Hkv_ + g * hd];
                        for (int dd = 0; dd < hd; ++dd) {
                            dqi[dd] += ds * kj[dd];
                            dkj[dd] += ds * qi[dd];
                        }
                    }
                }
            }
        if (s_.rope) {
            rope_apply(dQ, B, nh, true);
            rope_apply(dK, B, s_.n_kv_heads, true);
        }
        dx1.assign((size_t)BT * H, 0);
        mm_nt(dQ.data(), &p_[o.Wq], dx1.data(), BT, Hq_, H, false);
        mm_nt(dK.data(), &p_[o.Wk], dx1.data(), BT, Hkv_, H, true);
        mm_nt(dV.data(), &p_[o.Wv], dx1.data(), BT, Hkv_, H, true);
        mm_tn(a.x1.data(), dQ.data(), &g_[o.Wq], BT, H, Hq_, true);
        mm_tn(a.x1.data(), dK.data(), &g_[o.Wk], BT, H, Hkv_, true);
        mm_tn(a.x1.data(), dV.data(), &g_[o.Wv], BT, H, Hkv_, true);
        rms_bwd(a.x.data(), &p_[o.g1], a.r1.data(), dx1.data(), dstream.data(), &g_[o.g1], BT, H, true);
    }
    for (int i = 0; i < BT; ++i) {
        const int tok = tokens[i], t = i % T;
        for (int j = 0; j < H; ++j) {
            g_[oE_ + (size_t)tok * H + j] += dstream[(size_t)i * H + j];
            if (!s_.rope) g_[oP_ + (size_t)t * H + j] += dstream[(size_t)i * H + j];
        }
    }
}

// Decoupled weight decay applied as p -= lr * (mhat / (sqrt(vhat) + eps) + wd * p) over the whole
// flat vector, gains and embeddings included (reference: src/refmodel.c:481-492).
void RefModel::adamw(double lr, double b1, double b2, double eps, double wd) {
    ++t_;
    const double c1 = 1.0 - std::pow(b1, (double)t_), c2 = 1.0 - std::pow(b2, (double)t_);
    for (size_t i = 0; i < p_.size(); ++i) {
        mom_[i] = b1 * mom_[i] + (1 - b1) * g_[i];
        vel_[i] = b2 * vel_[i] + (1 - b2) * g_[i] * g_[i];
        p_[i] -= lr * ((mom_[i] / c1) / (std::sqrt(vel_[i] / c2) + eps) + wd * p_[i]);
    }
}

double RefModel::accuracy(int B, const int* targets) const {
    const int BT = B * s_.seq, V = s_.vocab;
    int hit = 0;
    for (int i = 0; i < BT; ++i) {
        int best = 0;
        for (int j = 1; j < V; ++j)
            if (logits_[(size_t)i * V + j] > logits_[(size_t)i * V + best]) best = j;
        hit += best == targets[i];
    }
    return (double)hit / BT;
}

// Central differences against backward(): L2 relative error over all parameters (n_probe <= 0)
// or over n_probe pseudo-randomly chosen ones.
double RefModel::grad_check(int B, const int* tokens, const int* targets, int n_probe, double h) {
    forward(B, tokens, targets);
    backward(B, tokens, targets);
    const std::vector<double> analytic = g_;
    const size_t N = p_.size();
    uint64_t state = 88172645463325252ull;
    const size_t count = n_probe <= 0 ? N : (size_t)n_probe;
    double num = 0, den = 0;
    for (size_t c = 0; c < count; ++c) {
        size_t i = c;
        if (n_probe > 0) {
            state ^= state << 13; state ^= state >> 7; state ^= state << 17;
            i = state % N;
        }
        const double keep = p_[i];
        p_[i] = keep + h;
        const double lp = forward(B, tokens, targets);
        p_[i] = keep - h;
        const double lm = forward(B, tokens, targets);
        p_[i] = keep;
        const double fd = (lp - lm) / (2 * h);
        num += (fd - analytic[i]) * (fd - analytic[i]);
        den += fd * fd;
    }
    forward(B, tokens, targets);
    return std::sqrt(num / (den + 1e-30));
}

}  // namespace cai

using cai::RefModel;
using cai::RefSpec;

extern "C" {
void* cai_ref_create(int vocab, int seq, int hidden, int layers, int n_heads, int n_kv_heads, int head_dim, int ffn,
                     double eps, int rope, double rope_theta, int tied, double init_std, uint64_t seed) {
    RefSpec s;
    s.vocab = vocab; s.seq = seq; s.hidden = hidden; s.layers = layers; s.n_heads = n_heads;
    s.n_kv_heads = n_kv_heads > 0 ? n_kv_heads : n_heads;
    s.head_dim = head_dim; s.ffn = ffn; s.eps = eps; s.rope = rope; s.rope_theta = rope_theta; s.tied = tied;
    s.init_std = init_std;
    if (s.n_heads % s.n_kv_heads || (rope && head_dim % 2)) return nullptr;
    return new RefModel(s, seed);
}
void* cai_ref_create_moe(int vocab, int seq, int hidden, int layers, int n_heads, int n_kv_heads, int head_dim, int ffn,
                         double eps, int rope, double rope_theta, int tied, double init_std, int experts, int top_k,
                         uint64_t seed) {
    RefSpec s;
    s.vocab = vocab; s.seq = seq; s.hidden = hidden; s.layers = layers; s.n_heads = n_heads;
    s.n_kv_heads = n_kv_heads > 0 ? n_kv_heads : n_heads;
    s.head_dim = head_dim; s.ffn = ffn; s.eps = eps; s.rope = rope; s.rope_theta = rope_theta; s.tied = tied;
    s.init_std = init_std; s.experts = experts; s.top_k = top_k;
    if (s.n_heads % s.n_kv_heads || (rope && head_dim % 2) || experts < 1 || top_k < 1 || top_k > experts) return nullptr;
    return new RefModel(s, seed);
}
void cai_ref_free(void* m) { delete static_cast<RefModel*>(m); }
size_t cai_ref_param_count(void* m) { return static_cast<RefModel*>(m)->param_count(); }
double* cai_ref_params(void* m) { return static_cast<RefModel*>(m)->params().data(); }
double* cai_ref_grads(void* m) { return static_cast<RefModel*>(m)->grads().data(); }
long long cai_ref_offset(void* m, const char* name, size_t* count) {
    const size_t at = static_cast<RefModel*>(m)->offset(name, count);
    return at == (size_t)-1 ? -1 : (long long)at;
}
double cai_ref_forward(void* m, int B, const int* tokens, const int* targets) {
    return static_cast<RefModel*>(m)->forward(B, tokens, targets);
}
void cai_ref_backward(void* m, int B, const int* tokens, const int* targets) {
    static_cast<RefModel*>(m)->backward(B, tokens, targets);
}
void cai_ref_adamw(void* m, double lr, double b1, double b2, double eps, double wd) {
    static_cast<RefModel*>(m)->adamw(lr, b1, b2, eps, wd);
}
double cai_ref_accuracy(void* m, int B, const int* targets) { return static_cast<RefModel*>(m)->accuracy(B, targets); }
double cai_ref_grad_check(void* m, int B, const int* tokens, const int* targets, int n_probe, double h) {
    return static_cast<RefModel*>(m)->grad_check(B, tokens, targets, n_probe, h);
}
}
