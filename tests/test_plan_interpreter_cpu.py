"""Executable plans interpreted on the host, every rank of a job in one process: whatever the layout, the job must
train like the one-device fp32 model (same losses, same parameters after AdamW), because every collective, every
pipeline hand-off and every shard boundary of the op tables is executed for real. No GPU involved."""
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module", autouse=True)
def _built():
    from cai_b200 import _build, plan
    _build.build_host()
    plan.set_log_level("warn")


def _train_both(text, steps=3, seed=1):
    """Losses of the interpreted job and of the reference model over the same batches, and how far their fp32 master
    parameters are apart at the end relative to how far they moved."""
    from cai_b200.models.plan_interpreter import check_against_reference
    return check_against_reference(text, steps, seed)


def _cfg(base, world, keys):
    return ((ROOT / "configs" / base).read_text() +
            f"\ngpus_per_rack = {world}\ngpus_per_tray = {world}\ntrays_per_rack = 1\nnum_racks = 1\n{keys}\n")


LAYOUTS = {
    "one rank": (1, ""),
    "one rank, recompute": (1, "recompute = 1"),
    "one rank, SwiGLU kernels": (1, "fuse_swiglu = 0"),
    "one rank, SwiGLU in both GEMMs": (1, "fuse_swiglu = 2"),
    "tp2 fused": (2, "tp = 2\ncomm = fused"),
    "tp2 fused, one microbatch per launch, serial wgrad": (2, "tp = 2\ncomm = fused\nmb_group = 1\nwgrad_overlap = 0"),
    "tp2 NCCL-only": (2, "tp = 2\ncomm = baseline"),
    "pp2": (2, "pp = 2"),
    "dp2 fused": (2, "comm = fused"),
    "dp2 fused, one bucket": (2, "comm = fused\ndp_buckets = 0"),
    "dp2 NCCL-only": (2, "comm = baseline"),
    "dp2 ZeRO-2": (2, "comm = fused\nzero_stage = 2\nmb_group = 1"),
    "pp2 x dp2 ZeRO-2": (4, "pp = 2\ncomm = fused\nzero_stage = 2"),
    "dp2 ZeRO-3": (2, "comm = fused\nzero_stage = 3"),
    "dp2 ZeRO-3, full gradients": (2, "comm = fused\nzero_stage = 3\ndp_buckets = 0"),
    "tp4 fused": (4, "tp = 4\ncomm = fused"),
    "tp2 x pp2 fused": (4, "tp = 2\npp = 2\ncomm = fused"),
    "tp2 x dp2 fused": (4, "tp = 2\ncomm = fused"),
    "pp2 x dp2 fused": (4, "pp = 2\ncomm = fused"),
    "dp4 ZeRO-3": (4, "comm = fused\nzero_stage = 3"),
    "tp2 x dp2 ZeRO-3": (4, "tp = 2\ncomm = fused\nzero_stage = 3"),
    "pp2 x dp2 ZeRO-3": (4, "pp = 2\ncomm = fused\nzero_stage = 3"),
    "tp2 x pp2 x dp2 fused": (8, "tp = 2\npp = 2\ncomm = fused"),
    "tp2 x pp2 x dp2 ZeRO-3": (8, "tp = 2\npp = 2\ncomm = fused\nzero_stage = 3"),
    "tp4 x dp2 ZeRO-3": (8, "tp = 4\ncomm = fused\nzero_stage = 3"),
    "pp4 x dp2 NCCL-only": (8, "pp = 4\ncomm = baseline"),
}


@pytest.mark.parametrize("name", sorted(LAYOUTS))
def test_every_layout_trains_like_the_one_device_model(name):
    world, keys = LAYOUTS[name]
    losses, drift = _train_both(_cfg("tiny_mp.cfg", world, keys), steps=2)
    for got, want in losses:
        assert got == pytest.approx(want, abs=1.5e-3), (name, losses)
    # parameters after two AdamW steps: apart by a few percent of the distance they moved (bf16 storage of
    # activations and weights turns a few near-zero gradients around; a wrong shard or a lost contribution moves whole tensors)
    assert drift < 0.05, (name, drift)


ODD = {
    "three stages over four layers": (3, "pp = 3"),
    "two stages over five layers": (2, "pp = 2\nnum_layers = 5\ncomm = fused"),
    "three replicas": (3, "comm = fused"),
    "three replicas, ZeRO-3": (3, "comm = fused\nzero_stage = 3"),
    "tp2 x dp3": (6, "tp = 2\ncomm = fused"),
    "one microbatch per step under a pipeline": (2, "pp = 2\ngrad_accum = 1"),
    "three microbatches of one sequence": (2, "comm = fused\nmicrobatch = 1\ngrad_accum = 3"),
    "untied head under tensor parallelism": (2, "tp = 2\ncomm = fused\ntie_embeddings = 0"),
}


@pytest.mark.parametrize("name", sorted(ODD))
def test_shapes_that_do_not_divide_evenly(name):
    world, keys = ODD[name]
    losses, drift = _train_both(_cfg("tiny_mp.cfg", world, keys), steps=2)
    assert all(got == pytest.approx(want, abs=1.5e-3) for got, want in losses) and drift < 0.05, (name, losses, drift)


def test_the_reference_config_with_grouped_query_attention_and_an_untied_head():
    """tiny.cfg has 4 query heads on 2 kv heads; an untied LM head adds a parameter the pipeline's last stage owns."""
    losses, drift = _train_both(_cfg("tiny.cfg", 2, "pp = 2\ntie_embeddings = 0"))
    assert all(got == pytest.approx(want, abs=1.5e-3) for got, want in losses) and drift < 0.05


@pytest.mark.parametrize("world,keys", [(1, ""), (2, "comm = fused\nzero_stage = 3"), (2, "pp = 2"), (2, "tp = 2\ncomm = fused"),
                                        (4, "tp = 2\ncomm = fused\nzero_stage = 3")])
def test_block_scaled_e4m3_linear_layers_stay_close_to_the_fp32_model(world, keys):
    """param_dtype = fp8e4m3: activations quantised per row and 128 columns, weights per 128 x 128 block (again after
    every ZeRO-3 gather), forward and input-gradient products in e4m3. The losses stay within a few 1e-3 of the fp32
    model; the parameters drift further than in bf16 (quantisation noise in every gradient) but nowhere near what a
    misplaced scale table or a stale quantised copy would cause."""
    losses, drift = _train_both(_cfg("tiny_mp.cfg", world, keys + "\nparam_dtype = fp8e4m3"))
    assert all(got == pytest.approx(want, abs=5e-3) for got, want in losses), losses
    assert 0.05 < drift < 0.4, drift




def test_a_run_continues_on_another_layout_from_the_state_of_the_first():
    """Two steps on tp 2 x pp 2, the global state (master, moments, step) moved to dp 2 with ZeRO-3, two more steps: the
    losses of the second half equal those of an uninterrupted one-rank run, so nothing of the optimizer state is lost or
    misplaced when the layout changes (the path a re-sharded checkpoint takes)."""
    from cai_b200 import plan
    from cai_b200.models.plan_interpreter import PlanInterpreter, random_state
    first = PlanInterpreter(_cfg("tiny_mp.cfg", 4, "tp = 2\npp = 2\ncomm = fused\ntie_embeddings = 0"))
    # two replicas with half the accumulation steps: the global batch stays what it was
    second = PlanInterpreter(_cfg("tiny_mp.cfg", 2, "comm = fused\nzero_stage = 3\ntie_embeddings = 0\ngrad_accum = 2"))
    single = PlanInterpreter(_cfg("tiny_mp.cfg", 1, "tie_embeddings = 0"))
    st = random_state(first, seed=4)
    first.load_state(st)
    single.load_state(st)
    m = first.model
    G, S = int(plan.describe(first.config_text)["global_batch"]), int(m.seq_len)
    gen = torch.Generator().manual_seed(9)
    batches = [(torch.randint(0, m.vocab_size, (G, S), generator=gen), torch.randint(0, m.vocab_size, (G, S), generator=gen))
               for _ in range(4)]
    want = [single.step(*b) for b in batches]
    got = [first.step(*b) for b in batches[:2]]
    second.load_state(first.state(), step=first.step_count)
    got += [second.step(*b) for b in batches[2:]]
    assert got == pytest.approx(want, abs=1.5e-3), (got, want)
    with pytest.raises(ValueError, match="sequences"):
        second.step(batches[0][0][:3], batches[0][1][:3])


MOE = {
    "two replicas, experts replicated": ("tiny_moe.cfg", 2, "comm = fused", 2),
    "ep2": ("tiny_moe.cfg", 2, "ep = 2\ncomm = fused", 2),
    "pp2": ("tiny_moe.cfg", 2, "pp = 2\ncomm = fused", 1),
    "pp2 x ep2": ("tiny_moe.cfg", 4, "pp = 2\nep = 2\ncomm = fused", 2),
    "tp2": ("tiny_moe_tp.cfg", 2, "tp = 2\ncomm = fused", 1),
    "tp2 x ep2": ("tiny_moe_tp.cfg", 4, "tp = 2\nep = 2\ncomm = fused", 2),
    "tp2 x pp2 x ep2": ("tiny_moe_tp.cfg", 8, "tp = 2\npp = 2\nep = 2\ncomm = fused", 2),
}


def test_mixture_of_experts_on_one_rank_follows_the_fp32_model():
    """Router (softmax, top-k, renormalised weights), dispatch into the expert slabs, the experts' products over the live
    rows, combine, and all of it backwards. bf16 activations move a few near-tied routing decisions, so the agreement
    with the fp32 model is looser than for the dense decoder."""
    losses, drift = _train_both(_cfg("tiny_moe.cfg", 1, ""))
    # 512 tokens per step and router gradients that pass through bf16 logit gradients: AdamW's normalised steps turn
    # more small gradients around than in the dense tests (the gradients themselves agree with autograd to a cosine
    # of 0.99 and above)
    assert all(got == pytest.approx(want, abs=5e-3) for got, want in losses) and drift < 0.3, (losses, drift)


@pytest.mark.parametrize("name", sorted(MOE))
def test_mixture_of_experts_layouts_train_like_the_one_rank_job(name):
    """Experts spread over an expert-parallel group, beside tensor parallelism (the tp x ep ranks form the group, every
    rank routes its own rows) and inside pipeline stages: same losses as the interpreted one-rank job on the same batches."""
    from cai_b200.models.plan_interpreter import PlanInterpreter, random_state
    base, world, keys, dp = MOE[name]
    job = PlanInterpreter(_cfg(base, world, keys + "\ntie_embeddings = 0"))     # a pipeline unties the head: untie it everywhere
    one = PlanInterpreter(_cfg(base, 1, f"grad_accum = {2 * dp}\ntie_embeddings = 0"))       # the same global batch on one rank
    st = random_state(one, seed=2)
    for k in st:
        if k.endswith(".wr"):
            st[k]["master"] *= 10.0      # a decisive router: fewer near-tied choices for bf16 rounding to turn around
    job.load_state(st)
    one.load_state(st)
    m = one.model
    gen = torch.Generator().manual_seed(6)
    G = one.rows_per_replica
    for step in range(3):
        tok = torch.randint(0, m.vocab_size, (G, int(m.seq_len)), generator=gen)
        tgt = torch.randint(0, m.vocab_size, (G, int(m.seq_len)), generator=gen)
        # the first step sees identical weights. Later the summation orders of the layouts differ in the last bits, a few
        # near-tied routing decisions flip, and the curves part by a few 1e-3
        assert job.step(tok, tgt) == pytest.approx(one.step(tok, tgt), abs=5e-4 if step == 0 else 5e-3), (name, step)
    import numpy as np
    a, b = job.state(), one.state()
    drift = max(float(np.abs(a[k]["master"] - b[k]["master"]).mean() / (np.abs(b[k]["master"] - st[k]["master"]).mean() + 1e-12))
                for k in st)
    assert drift < 0.4, (name, drift)        # a misplaced slab or a lost contribution moves whole tensors (drift near 1 and above)


def test_every_layout_the_advisor_lists_for_four_gpus_computes_the_same_model(tmp_path):
    """The layouts ``cai_b200.plan.advise`` enumerates (tp x pp x dp, ZeRO-1 and ZeRO-3) are not only priced: each one
    compiles, and its interpreted job follows the fp32 model on the same global batch."""
    from cai_b200 import plan
    from cai_b200.plan.advise import candidates
    text = _cfg("tiny_mp.cfg", 1, "grad_accum = 4")          # global batch: 8 sequences
    base = plan.describe(text)
    seen = []
    for cand in candidates(base, 4):
        keys = (f"tp = {cand['tp']}\npp = {cand['pp']}\nzero_stage = {cand['zero_stage']}\ngrad_accum = {cand['grad_accum']}\n"
                "comm = fused")
        losses, drift = _train_both(_cfg("tiny_mp.cfg", 4, keys), steps=2)
        assert all(got == pytest.approx(want, abs=1.5e-3) for got, want in losses) and drift < 0.05, (cand, losses, drift)
        seen.append((cand["tp"], cand["pp"], cand["dp"], cand["zero_stage"]))
    assert {(4, 1, 1, 1), (1, 1, 4, 3), (2, 2, 1, 1), (2, 1, 2, 3), (1, 2, 2, 3), (1, 4, 1, 1)} <= set(seen), seen


RANDOM_ORDER = {
    "tp2 x pp2 fused": ("tiny_mp.cfg", 4, "tp = 2\npp = 2\ncomm = fused"),
    "tp2 x dp2 ZeRO-3": ("tiny_mp.cfg", 4, "tp = 2\ncomm = fused\nzero_stage = 3"),
    "dp2 ZeRO-3, per-layer buckets": ("tiny_mp.cfg", 2, "comm = fused\nzero_stage = 3"),
    "dp2 ZeRO-2": ("tiny_mp.cfg", 2, "comm = fused\nzero_stage = 2\nmb_group = 1"),
    "tp2 NCCL-only": ("tiny_mp.cfg", 2, "tp = 2\ncomm = baseline"),
    "MoE tp2 x ep2": ("tiny_moe_tp.cfg", 4, "tp = 2\nep = 2\ncomm = fused"),
}


def _one_step(job, st, seed=1):
    job.load_state(st)
    m = job.model
    gen = torch.Generator().manual_seed(seed)
    G = job.rows_per_replica * int(job.hdr.dp)
    tok = torch.randint(0, m.vocab_size, (G, int(m.seq_len)), generator=gen)
    tgt = torch.randint(0, m.vocab_size, (G, int(m.seq_len)), generator=gen)
    return job.step(tok, tgt), job.state()


@pytest.mark.parametrize("name", sorted(RANDOM_ORDER))
def test_any_interleaving_the_events_allow_gives_the_same_bits(name):
    """The streams of every rank advance independently, held back only by the plan's record / wait events, and the
    next op is drawn at random: loss and parameters must equal the program-order run bit for bit, or some dependence
    between streams is not ordered by an event (the dynamic counterpart of the static hazard proof)."""
    import numpy as np
    from cai_b200.models.plan_interpreter import PlanInterpreter, random_state
    base, world, keys = RANDOM_ORDER[name]
    text = _cfg(base, world, keys)
    ref = PlanInterpreter(text)
    st = random_state(ref, seed=3)
    want_loss, want = _one_step(ref, st)
    for seed in (1, 2):
        loss, got = _one_step(PlanInterpreter(text, order="random", seed=seed), st)
        assert loss == want_loss, (name, seed)
        assert all(np.array_equal(got[k][key], want[k][key]) for k in want for key in ("master", "m", "v")), (name, seed)


def test_a_missing_wait_shows_up_under_random_interleaving():
    """Control: the weight-gradient GEMMs of a tensor-parallel plan run on the second compute stream behind waits on
    their operands. With those waits disarmed the random interleaving runs some of them early and the step's result
    changes; in program order the same broken plan still looks fine, which is why the check draws."""
    import numpy as np
    from cai_b200 import plan
    from cai_b200.models.plan_interpreter import PlanInterpreter, random_state
    text = _cfg("tiny_mp.cfg", 2, "tp = 2\ncomm = fused")
    ref = PlanInterpreter(text)
    st = random_state(ref, seed=3)
    _, want = _one_step(ref, st)

    def disarm(job):
        n = 0
        for r in job.ranks:
            for op in r.pf.ops:
                if op.kind == plan.OP_EVENT_WAIT and op.stream_id == 1:
                    op.aux0 = 0x7FFFFFFF            # an event nothing records: the wait passes at once
                    n += 1
        return n

    ordered = PlanInterpreter(text)
    assert disarm(ordered) > 0
    _, got = _one_step(ordered, st)
    assert all(np.array_equal(got[k]["master"], want[k]["master"]) for k in want)
    drawn = PlanInterpreter(text, order="random", seed=1)
    disarm(drawn)
    _, got = _one_step(drawn, st)
    assert any(not np.array_equal(got[k]["master"], want[k]["master"]) for k in want)


def test_command_line_check_of_a_configuration(tmp_path, capsys):
    from cai_b200.models import plan_interpreter
    cfg = tmp_path / "job.cfg"
    cfg.write_text(_cfg("tiny_mp.cfg", 2, "pp = 2"))
    assert plan_interpreter.main([str(cfg), "--steps", "2", "--order", "random"]) == 0
    out = capsys.readouterr().out
    assert "step 2: interpreted" in out and out.strip().endswith("PASS")
    assert plan_interpreter.main([str(cfg), "--steps", "1", "--tolerance", "0"]) == 1      # nothing matches to the last bit


SMALL = "\nhidden_size = 256\nffn_hidden = 1024\nnum_layers = 4\nnum_heads = 8\nnum_kv_heads = 8\nvocab_size = 2048\nseq_len = 256\n"
BENCH_LAYOUTS = {
    "tp8": ("tp8", SMALL),                                              # tp 8 fused, microbatches launched together
    "pp2tp4": ("pp2tp4", SMALL + "num_kv_heads = 4\n"),                 # pp 2 x tp 4, full recompute, sixteen microbatches
    "fsdp8b": ("fsdp8b", SMALL),                                        # dp 8, ZeRO-3, e4m3 linear layers
    "moe_ep8": ("moe_ep8", SMALL + "ffn_hidden = 256\n"),               # 64 experts, top-8, ep 8
}


@pytest.mark.parametrize("name", sorted(BENCH_LAYOUTS))
def test_the_benchmark_layouts_scaled_down_on_eight_ranks(name):
    """The layouts ``bench.py`` measures on eight GPUs, with the model shrunk to fit a host: same parallel keys, same
    schedule options, every rank interpreted."""
    import sys
    sys.path.insert(0, str(ROOT))
    import bench
    from cai_b200.models.plan_interpreter import check_against_reference
    config, extra = BENCH_LAYOUTS[name]
    losses, drift = check_against_reference(bench.config_text(8, "fused", config) + extra, steps=2)
    assert all(got == pytest.approx(want, abs=5e-3 if name in ("fsdp8b", "moe_ep8") else 1.5e-3) for got, want in losses), (name, losses)
    # 64 experts share 4096 tokens: most expert rows see a handful of tokens, and AdamW's normalised steps turn their
    # tiny gradients around freely; the dense layouts stay within a few percent, e4m3 within its quantisation noise
    assert drift < {"tp8": 0.05, "pp2tp4": 0.05, "fsdp8b": 0.4, "moe_ep8": 0.9}[name], (name, drift)
