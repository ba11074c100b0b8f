"""Mixture of experts on one GPU: the router kernels against PyTorch, the dispatch -> segmented GEMM
-> combine chain against a dense per-expert loop, and a full MoE training step (plan compiled for
ep = 1) against the fp32 PyTorch model."""
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _engine(**kw):
    from cai_b200.runtime.engine import Engine
    return Engine(ROOT / "configs" / "tiny_moe.cfg", rank=0, world=1, local_rank=0, **kw)


@pytest.mark.parametrize("T,E,k", [(256, 32, 2), (1000, 64, 8), (64, 256, 4)])
def test_router_forward_backward(T, E, k):
    from cai_b200 import ops
    torch.manual_seed(0)
    logits = torch.randn(T, E, device="cuda") * 2
    idx, w, pos, counts = ops.moe_route_fwd(logits, k, cap=T * k)
    prob = torch.softmax(logits, -1)
    top_p, top_e = prob.topk(k, -1)
    assert torch.equal(idx.long().sort(-1).values, top_e.sort(-1).values)
    ref_w = torch.gather(prob, 1, idx.long())
    ref_w = ref_w / ref_w.sum(-1, keepdim=True)
    assert torch.allclose(w, ref_w, atol=1e-5, rtol=1e-4)
    assert torch.equal(counts.long(), torch.bincount(idx.view(-1).long(), minlength=E))
    # slots inside an expert are a permutation of 0..count-1
    for e in range(0, E, max(1, E // 8)):
        slots = pos[idx == e].long().sort().values
        assert torch.equal(slots, torch.arange(slots.numel(), device="cuda"))
    # backward: d logits of sum(w * dw)
    dw = torch.randn(T, k, device="cuda")
    lg = logits.clone().requires_grad_(True)
    pr = torch.softmax(lg, -1)
    ww = torch.gather(pr, 1, idx.long())
    ww = ww / ww.sum(-1, keepdim=True)
    (ww * dw).sum().backward()
    dl = ops.moe_route_bwd(logits, idx, dw, pos)
    err = (dl.float() - lg.grad).abs().max().item()
    assert err < 2e-2 * lg.grad.abs().max().item() + 1e-3, err


def test_router_capacity_drops():
    from cai_b200 import ops
    logits = torch.zeros(512, 32, device="cuda")
    logits[:, 3] = 5.0   # everyone picks expert 3 first
    idx, w, pos, counts = ops.moe_route_fwd(logits, 2, cap=128)
    first = pos[idx == 3]
    assert (first >= 0).sum().item() == 128 and (first < 0).sum().item() == 512 - 128
    assert counts[3].item() == 512
    # slots go out in token order: the first 128 tokens keep the expert, token t sits in row t, and a second
    # run gives the same assignment
    tok_slot = pos[:, 0] if bool((idx[:, 0] == 3).all()) else pos[idx == 3]
    assert torch.equal(tok_slot[:128].long(), torch.arange(128, device="cuda")) and bool((tok_slot[128:] < 0).all())
    idx2, w2, pos2, counts2 = ops.moe_route_fwd(logits, 2, cap=128)
    assert torch.equal(pos, pos2) and torch.equal(idx, idx2) and torch.equal(counts, counts2)


def test_first_step_loss_and_grads_match_fp32_reference():
    from cai_b200.models.reference_torch import forward_loss
    from cai_b200.runtime.engine import synthetic_batch
    eng = _engine()
    m = eng.model
    rows = eng.hdr.num_microbatches * m.microbatch
    tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows, step=0, seed=0)
    params = {n: eng.param(n).detach().float().clone().requires_grad_(True) for n in eng.parameter_names()}
    assert any(n.endswith("experts.wgu") for n in params) and any(n.endswith(".wr") for n in params)
    ref = forward_loss(params, tok.view(rows, m.seq_len).long().cuda(), tgt.view(rows, m.seq_len).long().cuda(),
                       layers=m.num_layers, heads=m.num_heads, kv_heads=m.num_kv_heads, head_dim=m.head_dim,
                       seq=m.seq_len, eps=eng.train.norm_eps, theta=eng.train.rope_theta, top_k=m.moe_top_k)
    ref.backward()
    loss = eng.step(tok, tgt, lr=0.0)
    assert abs(loss - ref.item()) < 2e-2 * ref.item(), (loss, ref.item())
    for n in eng.parameter_names():
        g, r = eng.grad(n).float(), params[n].grad
        rel = ((g - r).norm() / (r.norm() + 1e-12)).item()
        # The router's top-k choice is discontinuous: bf16 activations flip the choice of about one token
        # in a hundred against the fp32 model, and a flipped token moves its whole contribution to other
        # experts. That is ~10 % of the norm of an expert / gain gradient here and more for the router's own
        # weight (its exact gradient is checked against autograd in test_router_forward_backward).
        tol = 0.35 if n.endswith(".wr") else 0.15 if ("experts" in n or n.endswith(".g2")) else 6e-2
        assert rel < tol, (n, rel)
    eng.close()


def test_moe_loss_falls_and_graph_replay_matches():
    from cai_b200.runtime.engine import synthetic_batch
    curves = []
    for graph in (False, True):
        eng = _engine()
        m = eng.model
        rows = eng.hdr.num_microbatches * m.microbatch
        tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows, step=0, seed=3)
        if graph:
            eng.use_graph(True)
        curves.append([eng.step(tok, tgt) for _ in range(6)])
        eng.close()
    assert curves[0][-1] < curves[0][0] - 0.2, curves
    for a, b in zip(*curves):
        assert abs(a - b) < 0.03 * max(1.0, a), curves


def test_segmented_gemm_skips_dead_rows():
    from cai_b200 import ops
    torch.manual_seed(1)
    cap, nseg, K, N = 256, 6, 512, 384
    counts = torch.tensor([256, 0, 130, 1, 64, 200], device="cuda", dtype=torch.int32)
    A = torch.randn(nseg * cap, K, device="cuda").to(torch.bfloat16)
    B = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    out = torch.full((nseg * cap, N), 7.0, device="cuda", dtype=torch.bfloat16)
    ops.gemm(A, B, out=out, seg_counts=counts, seg_rows=cap, seg_mode=1)
    ref = (A.float() @ B.float().t())
    for s, c in enumerate(counts.tolist()):
        live = out[s * cap:s * cap + c].float()
        assert torch.allclose(live, ref[s * cap:s * cap + c], atol=0.5, rtol=2e-2)
        done = -(-c // 128) * 128   # whole 128-row tiles are computed
        assert torch.all(out[s * cap + done:(s + 1) * cap] == 7.0)
    # weight-gradient form: K is the segmented dimension; dead rows may hold anything past the
    # next multiple of 64, zeros up to it
    X = torch.randn(nseg * cap, 256, device="cuda").to(torch.bfloat16)
    Y = torch.randn(nseg * cap, 320, device="cuda").to(torch.bfloat16)
    Xz, Yz = X.clone(), Y.clone()
    for s, c in enumerate(counts.tolist()):
        pad = -(-c // 64) * 64
        for t in (X, Y, Xz, Yz):
            t[s * cap + c:s * cap + pad] = 0
        Xz[s * cap + pad:(s + 1) * cap] = 0
        X[s * cap + pad:(s + 1) * cap] = float("nan")
    dW = torch.zeros(256, 320, device="cuda")
    ops.gemm(X, Y, trans_a=True, trans_b=True, out=dW, accumulate=True, seg_counts=counts, seg_rows=cap, seg_mode=2)
    refW = Xz.float().t() @ Yz.float()
    assert torch.allclose(dW, refW, atol=0.5, rtol=2e-2)
    # no live rows at all: the product counts as zero
    dW2 = torch.full((256, 320), 3.0, device="cuda")
    ops.gemm(X, Y, trans_a=True, trans_b=True, out=dW2, out_dtype=torch.float32,
             seg_counts=torch.zeros(nseg, device="cuda", dtype=torch.int32), seg_rows=cap, seg_mode=2)
    assert torch.all(dW2 == 0)


def test_dispatch_expert_gemm_combine_single_member():
    """The exchange kernels with a group of one: permute into slabs, per-expert GEMM, weighted gather."""
    import ctypes
    from cai_b200 import ops
    from cai_b200.ops import _lib
    L = _lib.lib()
    torch.manual_seed(2)
    T, H, E, k, cap, F = 384, 256, 32, 2, 128, 128
    sig = int(L.cai_signal_block_bytes())
    slab_off = sig
    ys_off = slab_off + E * cap * H * 2
    cnt_off = ys_off + E * cap * H * 2
    arena = torch.zeros(cnt_off + E * 4 + 256, device="cuda", dtype=torch.uint8)
    base = arena.data_ptr()
    bases = (ctypes.c_void_p * 1)(base)
    epoch = torch.tensor([10], device="cuda", dtype=torch.int32)
    scratch = torch.zeros(4, device="cuda", dtype=torch.int32)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda")
    idx, w, pos, counts = ops.moe_route_fwd(logits, k, cap)
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.cai_moe_dispatch_c(bases, 0, 1, 0, x.data_ptr(), idx.data_ptr(), pos.data_ptr(), None, counts.data_ptr(),
                                    slab_off, cnt_off, T, H, k, E, cap, epoch.data_ptr(), 1, scratch.data_ptr(), st), "dispatch")
    xs = arena[slab_off:ys_off].view(torch.bfloat16).view(E * cap, H)
    ys = arena[ys_off:cnt_off].view(torch.bfloat16).view(E * cap, H)
    cnt = arena[cnt_off:cnt_off + E * 4].view(torch.int32)
    assert torch.equal(cnt, counts.clamp(max=cap))
    W = (torch.randn(E, H, H, device="cuda") * 0.1).to(torch.bfloat16)   # one square "expert" each
    for e in range(E):
        ops.gemm(xs[e * cap:(e + 1) * cap], W[e], out=ys[e * cap:(e + 1) * cap], seg_counts=cnt[e:e + 1], seg_rows=cap,
                 seg_mode=1)
    res = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(res)
    _lib.check(L.cai_moe_combine_c(bases, 0, 1, 0, res.data_ptr(), out.data_ptr(), idx.data_ptr(), pos.data_ptr(), w.data_ptr(),
                                   ys_off, None, None, T, H, k, E, cap, 1, epoch.data_ptr(), 2, st), "combine")
    ref = res.float().clone()
    for s in range(k):
        y = torch.einsum("th,toh->to", x.float(), W[idx[:, s].long()].float())
        ref += (w[:, s, None] * y.to(torch.bfloat16).float()) * (pos[:, s, None] >= 0)
    assert torch.allclose(out.float(), ref, atol=6e-2, rtol=3e-2)
    # gradient of the combine weights
    d = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    dw = torch.empty(T, k, device="cuda")
    _lib.check(L.cai_moe_combine_c(bases, 0, 1, 0, None, None, idx.data_ptr(), pos.data_ptr(), None, ys_off, d.data_ptr(),
                                   dw.data_ptr(), T, H, k, E, cap, 0, epoch.data_ptr(), 3, st), "combine_dw")
    for s in range(k):
        y = torch.einsum("th,toh->to", x.float(), W[idx[:, s].long()].float()).to(torch.bfloat16).float()
        refd = (y * d.float()).sum(-1) * (pos[:, s] >= 0)
        assert torch.allclose(dw[:, s], refd, atol=0.3, rtol=3e-2)
    assert _lib.device_status(clear=True) == 0


def test_grouped_gemm_matches_per_group_products():
    """All local experts in one launch: forward form (rows segmented), weight-gradient form (K segmented)."""
    from cai_b200 import ops
    torch.manual_seed(3)
    G, cap, nsrc, K, N = 5, 128, 2, 256, 320
    M = cap * nsrc                                   # rows per expert: one sub-slab per source member
    counts = torch.tensor([128, 7, 0, 64, 100, 1, 128, 128, 0, 0], device="cuda", dtype=torch.int32)   # [G * nsrc]
    A = torch.randn(G * M, K, device="cuda").to(torch.bfloat16)
    W = (torch.randn(G * N, K, device="cuda") * 0.1).to(torch.bfloat16)
    out = torch.full((G * M, N), 5.0, device="cuda", dtype=torch.bfloat16)
    ops.gemm_grouped(A, W, out, M, N, K, groups=G, seg_counts=counts, seg_rows=cap, seg_mode=1)
    for g in range(G):
        ref = A[g * M:(g + 1) * M].float() @ W[g * N:(g + 1) * N].float().t()
        for s in range(nsrc):
            c = int(counts[g * nsrc + s])
            r0 = g * M + s * cap
            assert torch.allclose(out[r0:r0 + c].float(), ref[s * cap:s * cap + c], atol=0.3, rtol=2e-2), (g, s)
            if c == 0:
                assert torch.all(out[r0:r0 + cap] == 5.0)   # dead sub-slab: tile skipped
    # weight gradient per expert: dW_g[N, K2] = Y_g^T X_g over the live rows
    K2 = 192
    Y = torch.randn(G * M, N, device="cuda").to(torch.bfloat16)
    X = torch.randn(G * M, K2, device="cuda").to(torch.bfloat16)
    for g in range(G):
        for s in range(nsrc):
            c = int(counts[g * nsrc + s])
            r0 = g * M + s * cap
            Y[r0 + c:r0 + cap] = 0
            X[r0 + c:r0 + cap] = 0
    dW = torch.zeros(G * N, K2, device="cuda")
    ops.gemm_grouped(Y, X, dW, N, K2, M, groups=G, trans_a=True, trans_b=True, accumulate=True, seg_counts=counts, seg_rows=cap,
                     seg_mode=2)
    for g in range(G):
        ref = Y[g * M:(g + 1) * M].float().t() @ X[g * M:(g + 1) * M].float()
        assert torch.allclose(dW[g * N:(g + 1) * N], ref, atol=0.5, rtol=2e-2), g
