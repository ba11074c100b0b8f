// refmodel.h - the fp64 correctness oracle: a small decoder-only transformer with forward,
// backward, AdamW, accuracy and a finite-difference gradient check, all in double precision on
// the CPU. Device results are compared against it.
//
// It covers the reference's oracle (src/refmodel.c: multi-head attention, learned absolute
// positions, tied embedding, RMSNorm with gain, SwiGLU, no biases) and the features the GPU configs
// need that the reference's oracle lacks: grouped-query attention, rotary position embedding, an
// untied LM head, a choice of initialisation (1/sqrt(fan_in) like the reference, or N(0, std)), and a
// mixture-of-experts MLP (softmax router, top-k, weights renormalised over the chosen experts, no
// capacity limit).
#pragma once

#include <cstddef>
#include <cstdint>
#include <vector>

namespace cai {

struct RefSpec {
    int vocab = 64, seq = 32, hidden = 64, layers = 2, n_heads = 4, n_kv_heads = 4, head_dim = 16, ffn = 128;
    double eps = 1e-6;
    int rope = 0;             // 0: learned absolute positions P[seq, hidden]; 1: rotary embedding on q, k
    double rope_theta = 10000.0;
    int tied = 1;             // LM head shares the embedding matrix
    double init_std = 0.0;    // 0: reference init (E, P ~ 0.02 N; W ~ N / sqrt(fan_in)); > 0: every matrix ~ std * N
    int experts = 0;          // > 0: every layer's MLP is a mixture of this many SwiGLU experts of width ffn
    int top_k = 2;            // experts per token
};

class RefModel {
public:
    RefModel(const RefSpec& spec, uint64_t seed);
    size_t param_count() const { return p_.size(); }
    // tokens / targets: [B * seq]; returns the mean loss and caches activations for backward
    double forward(int B, const int* tokens, const int* targets);
    void backward(int B, const int* tokens, const int* targets);  // fills grads() (zeroed first)
    void adamw(double lr, double b1, double b2, double eps, double wd);
    double accuracy(int B, const int* targets) const;              // top-1 of the last forward
    double grad_check(int B, const int* tokens, const int* targets, int n_probe, double h);
    std::vector<double>& params() { return p_; }
    std::vector<double>& grads() { return g_; }
    const RefSpec& spec() const { return s_; }
    // offset of a named tensor in the flat vectors: "E", "P", "gf", "head", "L<i>.g1|Wq|Wk|Wv|Wo|g2|Wg|Wu|Wd|Wr"
    // (mixture of experts: Wg / Wu / Wd hold the experts back to back, Wr [hidden, experts] is the router)
    size_t offset(const char* name, size_t* count = nullptr) const;

private:
    struct LayerOff { size_t g1, Wq, Wk, Wv, Wo, g2, Wg, Wu, Wd, Wr; };
    struct LayerAct {
        std::vector<double> x, r1, x1, Q, K, V, probs, ctx, hmid, r2, x2, gate, up, act;
        std::vector<double> rprob, rw, yexp;   // mixture of experts: router softmax [BT,E], weights [BT,k], expert outputs [BT*k,H]
        std::vector<int> ridx;                 // chosen experts [BT,k]; gate / up / act are then [BT*k, F]
    };
    RefSpec s_;
    int Hq_, Hkv_;
    size_t oE_, oP_, ogf_, ohead_;
    std::vector<LayerOff> lo_;
    std::vector<double> p_, g_, mom_, vel_;
    long t_ = 0;
    int B_ = 0;
    std::vector<LayerAct> acts_;
    std::vector<double> xlast_, hf_, rf_, logits_, sm_;
    void rope_apply(std::vector<double>& x, int B, int heads, bool inverse) const;
};

}  // namespace cai

// ---- C ABI (ctypes) ----------------------------------------------------------------------------
extern "C" {
void* cai_ref_create(int vocab, int seq, int hidden, int layers, int n_heads, int n_kv_heads, int head_dim, int ffn,
                     double eps, int rope, double rope_theta, int tied, double init_std, uint64_t seed);
void cai_ref_free(void* m);
size_t cai_ref_param_count(void* m);
double* cai_ref_params(void* m);
double* cai_ref_grads(void* m);
long long cai_ref_offset(void* m, const char* name, size_t* count);
double cai_ref_forward(void* m, int B, const int* tokens, const int* targets);
void cai_ref_backward(void* m, int B, const int* tokens, const int* targets);
void cai_ref_adamw(void* m, double lr, double b1, double b2, double eps, double wd);
double cai_ref_accuracy(void* m, int B, const int* targets);
double cai_ref_grad_check(void* m, int B, const int* tokens, const int* targets, int n_probe, double h);
// call before any forward; rebuilds the model with a mixture-of-experts MLP (same seed)
void* cai_ref_create_moe(int vocab, int seq, int hidden, int layers, int n_heads, int n_kv_heads, int head_dim, int ffn,
                         double eps, int rope, double rope_theta, int tied, double init_std, int experts, int top_k,
                         uint64_t seed);
}
