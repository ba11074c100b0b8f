"""End to end on one GPU: a compiled plan executed by the native runtime, against a plain PyTorch
fp32 model that starts from the same weights."""
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _engine(**kw):
    from cai_b200.runtime.engine import Engine
    return Engine(ROOT / "configs" / "tiny.cfg", rank=0, world=1, local_rank=0, **kw)


def _torch_params(eng, requires_grad=False):
    return {n: eng.param(n).detach().float().clone().requires_grad_(requires_grad) for n in eng.parameter_names()}


def _loss_ref(eng, params, tokens, targets):
    from cai_b200.models.reference_torch import forward_loss
    m = eng.model
    B = eng.hdr.num_microbatches * m.microbatch
    tok = tokens.view(B, m.seq_len).long().cuda()
    tgt = targets.view(B, m.seq_len).long().cuda()
    return forward_loss(params, tok, tgt, layers=m.num_layers, heads=m.num_heads, kv_heads=m.num_kv_heads,
                        head_dim=m.head_dim, seq=m.seq_len, eps=eng.train.norm_eps, theta=eng.train.rope_theta)


def test_first_step_loss_and_grads_match_fp32_reference():
    from cai_b200.runtime.engine import synthetic_batch
    eng = _engine()
    m = eng.model
    rows = eng.hdr.num_microbatches * m.microbatch
    tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows, step=0, seed=0)
    params = _torch_params(eng, requires_grad=True)
    ref = _loss_ref(eng, params, tok, tgt)
    ref.backward()
    loss = eng.step(tok, tgt, lr=0.0)  # lr 0: gradients stay inspectable, weights unchanged
    assert eng.check_canaries()        # nothing wrote outside the arena
    assert abs(loss - ref.item()) < 2e-2 * ref.item(), (loss, ref.item())
    worst = 0.0
    for n in eng.parameter_names():
        g, r = eng.grad(n).float(), params[n].grad
        rel = ((g - r).norm() / (r.norm() + 1e-12)).item()
        worst = max(worst, rel)
        assert rel < 6e-2, (n, rel)
    assert worst > 0
    eng.close()


def test_loss_curve_tracks_fp32_adamw():
    from cai_b200.runtime.engine import synthetic_batch
    eng = _engine()
    m, t = eng.model, eng.train
    rows = eng.hdr.num_microbatches * m.microbatch
    params = _torch_params(eng, requires_grad=True)
    names = list(params)
    mom = {n: torch.zeros_like(params[n]) for n in names}
    vel = {n: torch.zeros_like(params[n]) for n in names}
    # one fixed batch: the loss must fall, and fall the same way on both sides
    tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows, step=0, seed=1)
    ours, theirs = [], []
    for step in range(1, 9):
        ours.append(eng.step(tok, tgt))
        for p in params.values():
            p.grad = None
        ref = _loss_ref(eng, params, tok, tgt)
        ref.backward()
        theirs.append(ref.item())
        with torch.no_grad():
            for n in names:
                g = params[n].grad
                mom[n].mul_(t.beta1).add_(g, alpha=1 - t.beta1)
                vel[n].mul_(t.beta2).addcmul_(g, g, value=1 - t.beta2)
                mh = mom[n] / (1 - t.beta1 ** step)
                vh = vel[n] / (1 - t.beta2 ** step)
                params[n].sub_(t.lr * (mh / (vh.sqrt() + t.adam_eps) + t.weight_decay * params[n]))
    assert ours[-1] < ours[0] - 0.3, ours
    for a, b in zip(ours, theirs):
        assert abs(a - b) < 0.05 * max(1.0, b), (ours, theirs)
    eng.close()


def test_cuda_graph_replay_matches_stream_replay():
    from cai_b200.runtime.engine import synthetic_batch
    m_rows = None
    losses = []
    for graph in (False, True):
        eng = _engine()
        m = eng.model
        m_rows = eng.hdr.num_microbatches * m.microbatch
        cur = []
        for step in range(4):
            tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, m_rows, step=step, seed=3)
            if graph and step == 1:
                eng.use_graph(True)
            cur.append(eng.step(tok, tgt))
        losses.append(cur)
        eng.close()
    for a, b in zip(*losses):
        assert abs(a - b) < 1e-3, losses


def test_trace_has_measured_times():
    from cai_b200.runtime.engine import synthetic_batch
    eng = _engine()
    m = eng.model
    rows = eng.hdr.num_microbatches * m.microbatch
    tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows, step=0, seed=0)
    eng.step(tok, tgt)
    recs = eng.trace_step(tok, tgt)
    assert len(recs) >= 40
    assert all(r.end_s >= r.start_s for r in recs)
    assert sum(r.end_s - r.start_s for r in recs) > 0
    eng.close()


def test_loss_curve_matches_fp64_oracle():
    """Device (bf16) training against the fp64 CPU oracle started from the same weights."""
    from cai_b200.models.oracle import Oracle, load_engine_weights
    from cai_b200.runtime.engine import synthetic_batch
    eng = _engine()
    m, t = eng.model, eng.train
    rows = eng.hdr.num_microbatches * m.microbatch
    ora = Oracle(vocab=m.vocab_size, seq=m.seq_len, hidden=m.hidden_size, layers=m.num_layers, n_heads=m.num_heads,
                 n_kv_heads=m.num_kv_heads, head_dim=m.head_dim, ffn=m.ffn_hidden, eps=t.norm_eps, rope=True,
                 rope_theta=t.rope_theta, tied=True, init_std=0.02, seed=1)
    load_engine_weights(ora, eng)
    tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows, step=0, seed=5)
    dev, ref = [], []
    for _ in range(5):
        dev.append(eng.step(tok, tgt))
        ref.append(ora.forward(tok.numpy(), tgt.numpy()))
        ora.backward(tok.numpy(), tgt.numpy())
        ora.adamw(t.lr, t.beta1, t.beta2, t.adam_eps, t.weight_decay)
    assert ref[-1] < ref[0] - 0.2
    for a, b in zip(dev, ref):
        assert abs(a - b) < 0.03 * max(1.0, b), (dev, ref)
    eng.close()


def test_checkpoint_resume_reproduces_the_curve(tmp_path):
    from cai_b200 import plan as planlib
    from cai_b200.runtime.engine import synthetic_batch
    eng = _engine()
    m = eng.model
    rows = eng.hdr.num_microbatches * m.microbatch
    batches = [synthetic_batch(m.vocab_size, m.seq_len, rows, step=s % 2, seed=9) for s in range(6)]
    for s in range(3):
        eng.step(*batches[s])
    eng.save_checkpoint(tmp_path / "ck", "periodic")
    tail = [eng.step(*batches[s]) for s in range(3, 6)]
    assert eng.wait_checkpoint() == 0
    eng.close()
    raw = (tmp_path / "ck.latest.rank000000").read_bytes()
    assert int.from_bytes(raw[:4], "little") == 3 and (tmp_path / "ck.periodic.rank000000").exists()

    eng2 = _engine()
    assert eng2.load_checkpoint(tmp_path / "ck") and eng2.step_count == 3
    tail2 = [eng2.step(*batches[s]) for s in range(3, 6)]
    assert all(abs(a - b) < 2e-3 for a, b in zip(tail, tail2)), (tail, tail2)
    assert not eng2.load_checkpoint(tmp_path / "nothing")
    eng2.close()

    # a checkpoint of a different plan is refused
    from cai_b200.runtime.engine import Engine
    other = Engine(config_text=(ROOT / "configs" / "tiny.cfg").read_text() + "\nffn_hidden = 1024\n", rank=0, world=1,
                   local_rank=0)
    with pytest.raises(planlib.PlanError):
        other.load_checkpoint(tmp_path / "ck")
    other.close()


def test_activation_recompute_gives_the_same_training_run():
    """recompute = 1 keeps only each layer's input and re-runs the layer forward inside backward:
    same losses, same gradients, smaller activation arena."""
    from cai_b200.runtime.engine import Engine, synthetic_batch
    text = (ROOT / "configs" / "tiny.cfg").read_text()
    runs = []
    for rc in (0, 1):
        eng = Engine(config_text=text.replace("recompute     = 0", f"recompute     = {rc}"), rank=0, world=1, local_rank=0)
        m = eng.model
        assert m.recompute == rc
        rows = eng.hdr.num_microbatches * m.microbatch
        tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows, step=0, seed=5)
        first = eng.step(tok, tgt, lr=0.0)
        grads = {n: eng.grad(n).float().clone() for n in eng.parameter_names()}
        losses = [first] + [eng.step(tok, tgt) for _ in range(4)]
        runs.append((losses, grads, int(eng.hdr.arena_bytes)))
        eng.close()
    (l0, g0, a0), (l1, g1, a1) = runs
    assert a1 < a0
    for x, y in zip(l0, l1):
        assert abs(x - y) < 1e-3 * max(1.0, abs(x)), (l0, l1)
    for n in g0:
        rel = ((g0[n] - g1[n]).norm() / (g0[n].norm() + 1e-12)).item()
        assert rel < 1e-3, (n, rel)


def test_trainer_prints_measured_stream_stats_and_handles_a_failed_step(tmp_path):
    """The device trainer's summary carries measured per-stream occupancy and the compute stream's idle share,
    its JSONL sink the same fields; a failed step ends the run with exit code 1 and an emergency checkpoint
    that leaves the rolling "latest" file at the last periodic state."""
    import json
    import os
    import subprocess
    import sys
    sink, ck = tmp_path / "log.jsonl", tmp_path / "ck"
    env = dict(os.environ, RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
    cmd = [sys.executable, "-m", "cai_b200.trainer", "--config", str(ROOT / "configs" / "tiny.cfg"), "--jsonl", str(sink),
           "--ckpt", str(ck), "--ckpt-every", "2"]
    r = subprocess.run(cmd + ["--steps", "5"], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-2000:])
    assert "per-stream occupancy (ms), measured on the last step: compute_hi=" in r.stdout
    assert "compute stream idle" in r.stdout and "summary: 4 steps" in r.stdout
    recs = [json.loads(l) for l in sink.read_text().splitlines()]
    assert [x["step"] for x in recs] == [0, 1, 2, 3, 4]
    last = recs[-1]
    assert last["traced"] and set(last["stream_busy_ms"]) == {"compute_hi", "compute_lo", "comm_tp", "comm_pp", "comm_dp", "io"}
    assert last["stream_busy_ms"]["compute_hi"] > 0 and 0.0 <= last["bubble_measured"] < 1.0
    assert all(k in recs[0] for k in ("step_time_s", "mfu", "tokens_per_s", "loss", "bubble_formula"))
    latest = tmp_path / "ck.latest.rank000000"
    assert int.from_bytes(latest.read_bytes()[:4], "little") == 4
    # resume at step 4, fail at step 6: exit 1, emergency file with the last completed step, "latest" untouched
    before = latest.read_bytes()
    r = subprocess.run(cmd + ["--steps", "9", "--ckpt-every", "100", "--fail-at", "6"], capture_output=True, text=True,
                       timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 1 and "step 6 failed" in r.stderr, (r.stdout[-1000:], r.stderr[-2000:])
    em = tmp_path / "ck.emergency.rank000000"
    assert em.exists() and int.from_bytes(em.read_bytes()[:4], "little") == 6
    assert latest.read_bytes() == before


def test_c_trainer_runs_an_executable_plan_on_the_device(tmp_path):
    """`bin/trainer --device`: the C runtime's device backend (kernel library opened at run time) trains the tiny
    model from plan files alone: loss column falls, statistics are measurements, a checkpoint with real state is
    written and resumed."""
    import subprocess
    BIN = ROOT / "bin"
    subprocess.run([BIN / "plan_compiler", ROOT / "configs" / "tiny.cfg", tmp_path, "--quiet", "--rank", "0", "--exec"], check=True,
                   capture_output=True)
    pl, tp, ck = tmp_path / "plan.rank000000.bin", tmp_path / "topology.bin", tmp_path / "ck"
    r = subprocess.run([BIN / "trainer", pl, tp, "--steps", "6", "--device", "--ckpt", ck, "--ckpt-every", "3"], capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-1500:])
    assert "backend=device" in r.stderr and "per-stream occupancy (ms), measured" in r.stdout
    rows = [l.split("|") for l in r.stdout.splitlines() if l[:4].strip().isdigit()]
    losses = [float(x[-1]) for x in rows]
    assert len(losses) == 6 and losses[-1] < losses[0] and all(l == l for l in losses)
    latest = tmp_path / "ck.latest.rank000000"
    assert latest.exists() and latest.stat().st_size > 1_000_000      # parameters + optimizer state, not 12 bytes
    r2 = subprocess.run([BIN / "trainer", pl, tp, "--steps", "8", "--device", "--ckpt", ck, "--ckpt-every", "100"], capture_output=True,
                        text=True, timeout=600)
    assert r2.returncode == 0 and "resumed from checkpoint at step 6" in r2.stderr
    rows2 = [l.split("|") for l in r2.stdout.splitlines() if l[:4].strip().isdigit()]
    assert [int(x[0]) for x in rows2] == [6, 7] and float(rows2[0][-1]) < losses[0]


def test_guard_bytes_between_arena_segments_catch_an_overrun():
    """The compiler leaves guard bytes behind the tensors of every class; after a step they are intact, and a
    write just past the last tensor of a class (what an overrunning kernel would do) is reported."""
    from cai_b200.runtime.engine import synthetic_batch
    eng = _engine()
    m = eng.model
    rows = eng.hdr.num_microbatches * m.microbatch
    tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows, step=0, seed=0)
    eng.step(tok, tgt)
    assert len(eng._inner_guards) >= 4 and all(hi - lo >= 1024 for lo, hi in eng._inner_guards[:-1])
    assert eng.check_canaries()
    lo, hi = eng._inner_guards[1]
    eng.arena[eng._arena_shift + lo] = 0
    with pytest.raises(RuntimeError, match="between arena segments"):
        eng.check_canaries()
    eng.close()


def test_swiglu_fused_into_the_gemms_trains_like_the_standalone_kernels():
    """fuse_swiglu = 0 (stand-alone SwiGLU kernels), 1 (forward in the gate/up GEMM epilogue, the default) and 2 (also
    the backward in the down-gradient GEMM epilogue) are the same arithmetic on the same bf16 intermediates."""
    from cai_b200.runtime.engine import Engine, synthetic_batch
    base = (ROOT / "configs" / "tiny.cfg").read_text()
    curves, grads = [], []
    for mode in (0, 1, 2):
        eng = Engine(config_text=base + f"\nfuse_swiglu = {mode}\n", rank=0, world=1, local_rank=0)
        m = eng.model
        rows = eng.hdr.num_microbatches * m.microbatch
        tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows, step=0, seed=0)
        first = eng.step(tok, tgt, lr=0.0)
        grads.append(eng.grad("L0.wgu").float().clone())
        curves.append([first] + [eng.step(tok, tgt) for _ in range(3)])
        eng.close()
    for c in curves[1:]:
        assert all(abs(a - b) <= 2e-3 * max(1.0, abs(a)) for a, b in zip(curves[0], c)), curves
    for g in grads[1:]:
        assert ((g - grads[0]).norm() / grads[0].norm()).item() < 1e-2


def test_debug_mode_checks_every_operand_extent_before_launch(monkeypatch):
    """CAI_DEBUG_BOUNDS: the executor compares what each kernel will address (rows, columns, pitch of the record)
    with the bytes the plan gives the tensor; the dense, MoE, fp8 and recompute plans all pass these checks."""
    from cai_b200.runtime.engine import Engine, synthetic_batch
    monkeypatch.setenv("CAI_DEBUG_BOUNDS", "1")
    for cfg, extra in (("tiny.cfg", ""), ("tiny_moe.cfg", ""), ("tiny.cfg", "param_dtype = fp8e4m3\n"), ("tiny.cfg", "recompute = 1\nfuse_swiglu = 2\n")):
        eng = Engine(config_text=(ROOT / "configs" / cfg).read_text() + "\n" + extra, rank=0, world=1, local_rank=0)
        m = eng.model
        rows = eng.hdr.num_microbatches * m.microbatch
        tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows, step=0, seed=0)
        a = eng.step(tok, tgt)
        b = eng.step(tok, tgt)
        assert a == a and b == b
        assert eng.check_canaries()
        eng.close()
