// reftrain [--steps N] [--lr X] [--batch B] [--seed S] [--config1] [--gqa] [--rope]
//
// Trains the fp64 oracle on the CPU. Default run is the reference's (tools/reftrain.c): vocab 64,
// seq 32, hidden 64, 2 layers, 4 heads x 16, ffn 128, prev-token task, fresh random batch per step,
// held-out evaluation batch, AdamW(0.9, 0.999, 1e-8, wd 0.01); exit code 0 iff the evaluation loss
// at least halved. --config1 runs the oracle configuration device results are compared with:
// ffn 256, vocab 256, batch 4, uniform random tokens from seed 0 with next-token targets,
// N(0, 0.02) init, lr 1e-3 (random targets: the curve is the oracle, not a learning test).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../ref/refmodel.h"

static unsigned long rng_state;
static unsigned long next_rand() {
    rng_state ^= rng_state << 13;
    rng_state ^= rng_state >> 7;
    rng_state ^= rng_state << 17;
    return rng_state;
}

int main(int argc, char** argv) {
    int steps = 400, B = 16;
    double lr = 0.01;
    unsigned long seed = 1;
    bool config1 = false, gqa = false, rope = false, have_lr = false, have_b = false, have_seed = false;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "--steps") && i + 1 < argc) steps = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--lr") && i + 1 < argc) { lr = atof(argv[++i]); have_lr = true; }
        else if (!strcmp(argv[i], "--batch") && i + 1 < argc) { B = atoi(argv[++i]); have_b = true; }
        else if (!strcmp(argv[i], "--seed") && i + 1 < argc) { seed = strtoul(argv[++i], nullptr, 10); have_seed = true; }
        else if (!strcmp(argv[i], "--config1")) config1 = true;
        else if (!strcmp(argv[i], "--gqa")) gqa = true;
        else if (!strcmp(argv[i], "--rope")) rope = true;
        else { fprintf(stderr, "unknown arg: %s\n", argv[i]); return 2; }
    }
    cai::RefSpec s;
    s.vocab = 64; s.seq = 32; s.hidden = 64; s.layers = 2; s.n_heads = 4; s.n_kv_heads = gqa ? 2 : 4; s.head_dim = 16;
    s.ffn = 128; s.eps = 1e-6; s.rope = rope ? 1 : 0;
    if (config1) {
        s.ffn = 256; s.vocab = 256; s.init_std = 0.02;
        if (!have_lr) lr = 1e-3;
        if (!have_b) B = 4;
        if (!have_seed) seed = 0;
    }
    cai::RefModel m(s, seed);
    rng_state = seed ? seed * 2654435761ul + 1 : 99;
    const int BT = B * s.seq;
    std::vector<int> tok(BT), tgt(BT), etok(BT), etgt(BT);
    auto gen = [&](std::vector<int>& t, std::vector<int>& y) {
        for (int b = 0; b < B; ++b) {
            int prev = 0;
            std::vector<int> row(s.seq + 1);
            for (int k = 0; k <= s.seq; ++k) row[k] = (int)(next_rand() % (unsigned long)s.vocab);
            for (int k = 0; k < s.seq; ++k) {
                const int idx = b * s.seq + k;
                if (config1) {
                    t[idx] = row[k];
                    y[idx] = row[k + 1];  // next token of a uniform random stream
                } else {
                    t[idx] = row[k];
                    y[idx] = k == 0 ? 0 : prev;  // previous token: forces attention one step back
                    prev = row[k];
                }
            }
        }
    };
    gen(etok, etgt);
    printf("reference model: %zu params | task=%s | vocab=%d seq=%d\n", m.param_count(),
           config1 ? "next-token(random)" : "prev-token", s.vocab, s.seq);
    printf("chance loss ~ ln(vocab) = %.3f\n\n", config1 ? 5.545177 : 4.158883);
    printf(" step |  train loss | eval loss | eval acc\n");
    printf("------+-------------+-----------+---------\n");
    const double eval0 = m.forward(B, etok.data(), etgt.data());
    const int every = steps / 20 ? steps / 20 : 1;
    for (int step = 0; step < steps; ++step) {
        gen(tok, tgt);
        const double tl = m.forward(B, tok.data(), tgt.data());
        m.backward(B, tok.data(), tgt.data());
        m.adamw(lr, 0.9, 0.999, 1e-8, 0.01);
        if (step % every == 0 || step == steps - 1) {
            const double el = m.forward(B, etok.data(), etgt.data());
            const double ea = m.accuracy(B, etgt.data());
            printf("%5d | %11.4f | %9.4f | %6.1f%%\n", step, tl, el, ea * 100.0);
            fflush(stdout);
        }
    }
    const double eval1 = m.forward(B, etok.data(), etgt.data());
    const double acc1 = m.accuracy(B, etgt.data());
    printf("\nresult: eval loss %.4f -> %.4f  (%.1fx lower), eval acc %.1f%%\n", eval0, eval1, eval0 / (eval1 + 1e-9),
           acc1 * 100.0);
    if (config1) return 0;
    return eval1 < eval0 * 0.5 ? 0 : 1;
}
