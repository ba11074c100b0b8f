"""GPU-free tests of the offline compiler, verifier, analytic runtime and tools."""
import hashlib
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "bin"


@pytest.fixture(scope="session", autouse=True)
def _built():
    from cai_b200 import _build
    _build.build_host()


def run(*cmd, ok=True):
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True, cwd=ROOT)
    if ok:
        assert r.returncode == 0, r.stdout + r.stderr
    return r


def test_native_selftest():
    r = run(BIN / "cai_selftest")
    assert "0 failures" in r.stdout


GOLDEN = {  # config -> (plan_hash, topology_hash, ops of rank 0, ops of the last-stage sample rank)
    "small": ("61eec02c9563ad48", "a6628b5f000e9efa", 3243, 3303),
    "full220k": ("6435c0f31b2cde67", "03ef8972bac28218", 34563, 30979),
    "full220k_moe": ("5f02c7d3a752a1b4", "03ef8972bac28218", 40707, 36355),
}


@pytest.mark.parametrize("name", list(GOLDEN))
def test_reference_format_golden_values(name, tmp_path):
    """Same configs as the reference ship, same hashes, op counts and file sizes as its compiler."""
    from cai_b200 import plan
    ph, th, ops0, ops_last = GOLDEN[name]
    r = run(BIN / "plan_compiler", ROOT / "configs" / f"{name}.cfg", tmp_path, "--quiet")
    assert f"topology_hash={th}, plan_hash={ph}" in r.stdout
    assert (tmp_path / "topology.bin").stat().st_size == 68
    files = sorted(tmp_path.glob("plan.rank*.bin"))
    p0 = plan.PlanFile(files[0])
    assert p0.hdr.version == 1 and p0.hdr.num_ops == ops0
    assert files[0].stat().st_size == 128 + 24 * p0.hdr.num_tensors + 16 * p0.hdr.num_groups + 32 * ops0
    assert plan.PlanFile(files[1]).hdr.num_ops == ops_last
    assert f"{p0.hdr.plan_hash:016x}" == ph


def test_small_plan_file_is_byte_identical_to_reference_output(tmp_path):
    import hashlib
    run(BIN / "plan_compiler", ROOT / "configs" / "small.cfg", tmp_path, "--quiet", "--rank", "0")
    digest = hashlib.sha256((tmp_path / "plan.rank000000.bin").read_bytes()).hexdigest()
    assert digest == "100247a2a5cbd88bd4d49f4a343269761e23dd48792e5911ef707a7bbc46efc2"
    tdig = hashlib.sha256((tmp_path / "topology.bin").read_bytes()).hexdigest()
    assert tdig == "ca06c2d94267e216a20d448df206c0f30967df9b1f21159f8374d604b7178a9e"


def test_simulated_step_matches_reference_numbers(tmp_path):
    from cai_b200 import plan
    run(BIN / "plan_compiler", ROOT / "configs" / "small.cfg", tmp_path, "--quiet")
    sim = plan.Simulator(tmp_path / "plan.rank000000.bin", tmp_path / "topology.bin", max_steps=3)
    s = sim.step()
    assert abs(s.step_time_s * 1e3 - 98.13) < 0.05 and abs(s.mfu - 0.617) < 0.002
    assert abs(s.bubble_ratio - 2 / 14) < 1e-9
    assert s.stream_busy[5] == 0.0
    sim.close()
    r = run(BIN / "trainer", tmp_path / "plan.rank000000.bin", tmp_path / "topology.bin", "--steps", "2",
            "--trace", tmp_path / "t.csv")
    assert "avg MFU 61.7%" in r.stdout
    lines = (tmp_path / "t.csv").read_text().splitlines()
    assert lines[0] == "op_index,kind,stream,start_us,end_us,dur_us,bytes,flops" and len(lines) > 1000


def test_topology_mismatch_is_refused(tmp_path):
    from cai_b200 import plan
    a, b = tmp_path / "a", tmp_path / "b"
    run(BIN / "plan_compiler", ROOT / "configs" / "small.cfg", a, "--quiet", "--rank", "0")
    run(BIN / "plan_compiler", ROOT / "configs" / "full220k.cfg", b, "--quiet", "--rank", "0")
    with pytest.raises(plan.PlanError, match="topology"):
        plan.Simulator(a / "plan.rank000000.bin", b / "topology.bin")
    r = run(BIN / "trainer", a / "plan.rank000000.bin", b / "topology.bin", ok=False)
    assert r.returncode == 1


def test_linter_verify_recover_tools(tmp_path):
    r = run(BIN / "topology_linter", ROOT / "configs" / "small.cfg")
    assert "RESULT: all checks passed" in r.stdout
    from cai_b200 import plan
    failed, rep = plan.lint(ROOT / "configs" / "small.cfg")             # the same checks through the library
    assert failed == 0 and "TP=4 fits intra-rack" in rep
    bad = tmp_path / "tp_across.cfg"
    bad.write_text((ROOT / "configs" / "b200_tp8.cfg").read_text() + "\ngpus_per_rack = 4\ntrays_per_rack = 1\ngpus_per_tray = 4\nnum_racks = 2\n")
    failed, rep = plan.lint(bad)
    assert failed == 1 and "exceeds gpus_per_rack" in rep
    assert run(BIN / "topology_linter", bad, ok=False).returncode == 1
    r = run(BIN / "plan_verify", ROOT / "configs" / "full220k.cfg")
    assert "tile all 220032 ranks" in r.stdout and "RESULT: all checks passed" in r.stdout
    r = run(BIN / "plan_verify", ROOT / "configs" / "b200_pp2tp4.cfg", "--exec")
    assert "no unordered RAW/WAW/WAR pair" in r.stdout and "pair up in issue order" in r.stdout
    # spare-rank recovery needs spares
    r = run(BIN / "plan_recover", ROOT / "configs" / "small.cfg", 3, tmp_path, ok=False)
    assert r.returncode == 1 and "no spare GPUs" in r.stderr
    cfg = tmp_path / "spare.cfg"
    cfg.write_text((ROOT / "configs" / "small.cfg").read_text().replace("num_racks     = 1", "num_racks = 2")
                   .replace("spare_gpus    = 0", "spare_gpus = 12"))
    r = run(BIN / "plan_recover", cfg, 3, tmp_path)
    assert "different rack" in r.stdout and (tmp_path / "plan.recover.rank000003.bin").exists()
    # the recovery plan is the plan of the failed rank, byte for byte
    run(BIN / "plan_compiler", cfg, tmp_path / "all", "--quiet", "--rank", "3")
    assert (tmp_path / "plan.recover.rank000003.bin").read_bytes() == (tmp_path / "all" / "plan.rank000003.bin").read_bytes()
    # --dir mode checks files on disk
    r = run(BIN / "plan_verify", cfg, "--dir", tmp_path / "all")
    assert "carry the expected hashes" in r.stdout


def test_checkpoint_resume_and_plan_hash_guard(tmp_path):
    from cai_b200 import plan
    run(BIN / "plan_compiler", ROOT / "configs" / "small.cfg", tmp_path, "--quiet", "--rank", "0")
    pl, tp = tmp_path / "plan.rank000000.bin", tmp_path / "topology.bin"
    ck = tmp_path / "ck"
    run(BIN / "trainer", pl, tp, "--steps", "7", "--ckpt", ck)
    assert (tmp_path / "ck.periodic.rank000000").exists() and (tmp_path / "ck.latest.rank000000").exists()
    raw = (tmp_path / "ck.latest.rank000000").read_bytes()
    assert int.from_bytes(raw[:4], "little") == 5 and raw[4:12] == bytes.fromhex("61eec02c9563ad48")[::-1]
    r = run(BIN / "trainer", pl, tp, "--steps", "7", "--ckpt", ck)
    assert "   5 |" in r.stdout and "   0 |" not in r.stdout   # resumed at step 5
    # a checkpoint of another plan is refused
    other = tmp_path / "o"
    run(BIN / "plan_compiler", ROOT / "configs" / "b200_tp8.cfg", other, "--quiet", "--rank", "0")
    sim = plan.Simulator(other / "plan.rank000000.bin", other / "topology.bin", checkpoint_path=ck)
    assert sim.load_checkpoint(ck) != 0
    sim.close()


def test_describe_and_group_members():
    from cai_b200 import plan
    text = (ROOT / "configs" / "b200_pp2tp4.cfg").read_text()
    d = plan.describe(text)
    assert d["tp"] == 4 and d["pp"] == 2 and d["dp"] == 1 and d["world_size"] == 8
    assert abs(d["bubble_ratio"] - 1 / 17) < 1e-6
    assert plan.group_members(text, plan.GROUP_TP, 5) == [4, 5, 6, 7]
    assert plan.group_members(text, plan.GROUP_PP, 5) == [1, 5]
    with pytest.raises(plan.PlanError):
        plan.describe("tp = 5\n")


def test_executable_plan_structure(tmp_path):
    from cai_b200 import plan
    plan.compile_plans(ROOT / "configs" / "tiny.cfg", tmp_path, version=2)
    p = plan.PlanFile(tmp_path / "plan.rank000000.bin")
    assert p.hdr.version == 2 and p.xhdr.num_exec > 50
    names = p.named_dict()
    for n in ("embed", "L0.wqkv", "L1.wd", "gf", "@tokens", "@loss", "@flat_param"):
        assert n in names
    # every parameter sits at the same element offset in the weight and gradient buffers
    for n, nt in names.items():
        if nt.init_std < 0:
            continue
        w, g = p.tensors[nt.tensor], p.tensors[nt.grad]
        base_w, base_g = p.tensors[names["@flat_param"].tensor].offset, p.tensors[names["@flat_grad"].tensor].offset
        assert (w.offset - base_w) // 2 == (g.offset - base_g) // 4 == nt.flat_off512 * 512
    assert all(t.offset + t.nbytes <= p.hdr.arena_bytes for t in p.tensors)


def _variant(tmp_path, name, extra, world=1):
    """tiny_mp.cfg on `world` GPUs with extra keys: compile every rank, run the whole-cluster verifier
    (tiling, event order, arena hazards, pipeline pairing) and return rank 0's plan."""
    from cai_b200 import plan
    text = (ROOT / "configs" / "tiny_mp.cfg").read_text()
    text += f"\ngpus_per_rack = {world}\ngpus_per_tray = {world}\n" + extra
    cfg = tmp_path / f"{name}.cfg"
    cfg.write_text(text)
    plan.compile_plans(cfg, tmp_path / name, version=2)
    problems, report = plan.verify(cfg)
    assert problems == 0, report[-2000:]
    return plan.PlanFile(tmp_path / name / "plan.rank000000.bin")


def test_plan_variants_compile_and_verify(tmp_path):
    from cai_b200 import plan
    kernels = lambda p: {int(x.kernel) for x in p.exec}
    base = _variant(tmp_path, "base", "")
    # activation recompute: more ops (each layer's forward runs twice), smaller arena
    rc = _variant(tmp_path, "recompute", "recompute = 1\n")
    assert len(rc.exec) > len(base.exec) and rc.hdr.arena_bytes < base.hdr.arena_bytes
    # fp8 linear layers: quantisers and the block-scaled GEMM appear, the bf16 GEMM stays for weight gradients
    f8 = _variant(tmp_path, "fp8", "param_dtype = fp8e4m3\n")
    assert {plan.K_QUANT_FP8, plan.K_GEMM_FP8, plan.K_GEMM} <= kernels(f8)
    # ZeRO-3 over two GPUs: the parameter class holds a shard plus staging buffers, gathers precede the GEMMs
    z1 = _variant(tmp_path, "zero1", "comm = fused\n", world=2)
    z3 = _variant(tmp_path, "zero3", "comm = fused\nzero_stage = 3\n", world=2)
    assert plan.K_FSDP_AG_GEMM in kernels(z3) and plan.K_FSDP_AG_GEMM not in kernels(z1)
    n1, n3 = z1.named_dict(), z3.named_dict()
    assert z3.tensors[n3["@flat_param"].tensor].nbytes * 2 <= z1.tensors[n1["@flat_param"].tensor].nbytes + 2048
    fused = [i for i, x in enumerate(z3.exec) if int(x.kernel) == plan.K_FSDP_AG_GEMM and (x.flags & 1)]
    assert fused and all(int(z3.exec[i + 1].kernel) == plan.K_GEMM for i in fused)   # merged into the GEMM that follows
    # tensor parallel: weight gradients leave the critical path (compute_lo), dQ runs beside dK/dV
    tp = _variant(tmp_path, "tp2", "tp = 2\ncomm = fused\nmb_group = 1\n", world=2)
    lo_gemms = [op for op in tp.ops if op.exec and int(tp.exec[op.exec - 1].kernel) == plan.K_GEMM and op.stream_id == 1]
    assert len(lo_gemms) >= 4 * 4 * 4   # 4 layers x 4 microbatches x 4 weight gradients
    # microbatches launched in pairs: half the launches, twice the rows each; left to the compiler, as many as divide
    # grad_accum and keep a launch under 16384 tokens (all four here)
    pair = _variant(tmp_path, "tp2_pairs", "tp = 2\ncomm = fused\nmb_group = 2\n", world=2)
    auto = _variant(tmp_path, "tp2_auto", "tp = 2\ncomm = fused\n", world=2)
    fused_ops = lambda p: [x for x in p.exec if int(x.kernel) in (plan.K_AG_GEMM, plan.K_GEMM_RS)]
    assert len(fused_ops(pair)) * 2 == len(fused_ops(tp)) and fused_ops(pair)[0].i[0] == 2 * fused_ops(tp)[0].i[0]
    assert pair.hdr.num_microbatches == tp.hdr.num_microbatches and pair.hdr.plan_hash == tp.hdr.plan_hash
    assert len(fused_ops(auto)) * 4 == len(fused_ops(tp))
    with pytest.raises(plan.PlanError):
        plan.compile_plans((ROOT / "configs" / "tiny_mp.cfg").read_text() + "\ngpus_per_rack = 2\ngpus_per_tray = 2\npp = 2\nmb_group = 2\n",
                           tmp_path / "bad_group", version=2, text=True)
    off = _variant(tmp_path, "tp2_serial", "tp = 2\ncomm = fused\nwgrad_overlap = 0\n", world=2)
    assert not [op for op in off.ops if op.exec and int(off.exec[op.exec - 1].kernel) == plan.K_GEMM and op.stream_id == 1]
    # refused combinations
    # ZeRO-2: parameters whole as under ZeRO-1, gradients staged per layer and reduced into the owners' accumulators
    z2 = _variant(tmp_path, "zero2", "comm = fused\nzero_stage = 2\nmb_group = 1\n", world=2)
    assert plan.K_FSDP_AG_GEMM not in kernels(z2)
    assert [x for x in z2.exec if int(x.kernel) == plan.K_RS_ADAMW and (x.flags & 4) and not (x.flags & 1)]
    n2 = z2.named_dict()
    assert z2.tensors[n2["@flat_param"].tensor].nbytes == z1.tensors[n1["@flat_param"].tensor].nbytes
    # what it saves grows with the depth: per-layer buffers for two layers and a shard-sized accumulator instead of all gradients
    deep1 = _variant(tmp_path, "zero1_deep", "comm = fused\nnum_layers = 12\n", world=2)
    deep2 = _variant(tmp_path, "zero2_deep", "comm = fused\nzero_stage = 2\nnum_layers = 12\n", world=2)
    assert deep2.class_bytes()["grad"] < 0.8 * deep1.class_bytes()["grad"]
    with pytest.raises(plan.PlanError):      # the staged buckets exist for tp = 1
        plan.compile_plans((ROOT / "configs" / "tiny_mp.cfg").read_text() + "\ngpus_per_rack = 4\ngpus_per_tray = 4\ncomm = fused\nzero_stage = 2\ntp = 2\n",
                           tmp_path / "bad_z2", version=2, text=True)
    # ZeRO-3 beside tensor parallelism: every rank shards its slice of the weights over its data-parallel group; the
    # gathers are kernels of their own (none rides in a GEMM) and the gradients stay whole
    z3tp = _variant(tmp_path, "zero3_tp2", "comm = fused\nzero_stage = 3\ntp = 2\n", world=4)
    gathers = [x for x in z3tp.exec if int(x.kernel) == plan.K_FSDP_AG_GEMM]
    assert gathers and not any(x.flags & 1 for x in gathers) and plan.K_AG_GEMM in kernels(z3tp)
    assert not [x for x in z3tp.exec if int(x.kernel) == plan.K_RS_ADAMW and (x.flags & 4)]
    # e4m3 linear layers under tensor parallelism: the collectives stay calls of their own beside the block-scaled GEMMs
    # (the fused all-gather / reduce-scatter GEMM kernels are bf16 only)
    f8tp = _variant(tmp_path, "fp8_tp2", "param_dtype = fp8e4m3\ntp = 2\ncomm = fused\n", world=2)
    assert plan.K_GEMM_FP8 in kernels(f8tp) and not ({plan.K_AG_GEMM, plan.K_GEMM_RS} & kernels(f8tp))
    with pytest.raises(plan.PlanError):      # experts in e4m3: an error, not a silent bf16 run
        plan.compile_plans((ROOT / "configs" / "tiny_moe.cfg").read_text() + "\nparam_dtype = fp8e4m3\n", tmp_path / "bad_moe", version=2, text=True)
    # ... and beside a pipeline: every stage shards its own parameters
    z3pp = _variant(tmp_path, "zero3_pp2", "comm = fused\nzero_stage = 3\npp = 2\n", world=4)
    assert plan.K_FSDP_AG_GEMM in kernels(z3pp) and z3pp.hdr.num_stages == 2
    for bad in ("zero_stage = 3\ncomm = baseline\n",
                "pp = 2\nvpp = 2\n"):                    # interleaving: an error, not a silent plain 1F1B schedule
        with pytest.raises(plan.PlanError):   # 4 GPUs: dp = 4, or tp = 2 x dp = 2
            plan.compile_plans((ROOT / "configs" / "tiny_mp.cfg").read_text() + "\ngpus_per_rack = 4\ngpus_per_tray = 4\n" + bad,
                               tmp_path / "bad", version=2, text=True)


def test_host_code_is_clean_under_address_and_ub_sanitizers():
    """Plan compiler, verifier (hazard checker), analytic runtime and oracle, built with
    -fsanitize=address,undefined, run the native self-test without a report."""
    from cai_b200 import _build
    exe = _build.build_sanitized_selftest()
    r = subprocess.run([str(exe)], cwd=ROOT, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0"))
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert "0 failures" in out and "runtime error" not in out and "AddressSanitizer" not in out, out[-3000:]


def test_benchmark_configs_compile_for_every_gpu_count(tmp_path):
    """The configs bench.py runs (headline config at tp = 1, 2, 4, 8 and the other named configs on 8 GPUs)
    compile into executable plans; the reference arm reports itself unavailable and exits 0."""
    import json
    import sys
    sys.path.insert(0, str(ROOT))
    import bench
    from cai_b200 import plan
    for n in (1, 2, 4, 8):
        for comm in ("fused", "baseline"):
            plan.compile_plans(bench.config_text(n, comm, "tp8"), tmp_path / f"tp{n}{comm}", ranks=(0, 1), version=2, text=True)
    for name in ("moe_ep8", "fsdp8b", "pp2tp4"):
        plan.compile_plans(bench.config_text(8, "fused", name), tmp_path / name, ranks=(0, 1), version=2, text=True)
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line


def test_backend_selection_at_cai_init(tmp_path):
    """One runtime API for every backend: without a GPU `--device` is refused with a reason, `--backend auto` falls
    back to the analytic backend (the order of the reference's cai_init, src/runtime.c:32-73)."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("checks the fallback on a box without a GPU")
    run(BIN / "plan_compiler", ROOT / "configs" / "tiny.cfg", tmp_path, "--quiet", "--rank", "0", "--exec")
    pl, tp = tmp_path / "plan.rank000000.bin", tmp_path / "topology.bin"
    r = run(BIN / "trainer", pl, tp, "--steps", "2", "--device", ok=False)
    assert r.returncode == 1 and "device backend unavailable" in r.stderr
    r = run(BIN / "trainer", pl, tp, "--steps", "2", "--backend", "auto")
    assert "backend=analytic" in r.stderr and "falling back" in r.stderr and "summary: 2 steps" in r.stdout


def test_arena_by_class_describes_what_a_device_allocates(tmp_path):
    """The executable plan's per-class extents add up to its arena, and under ZeRO-3 the gradient class is the owned
    shard plus two layer-sized stages, not the whole flat space (reference memory model: src/model.c:247-267)."""
    from cai_b200 import plan
    r = run(BIN / "plan_compiler", ROOT / "configs" / "b200_fsdp8b.cfg", tmp_path, "--exec", "--rank", "0")
    assert "arena by class:" in r.stdout
    pf = plan.PlanFile(tmp_path / "plan.rank000000.bin")
    cb = pf.class_bytes()
    total = sum(cb.values())
    assert 0.98 * pf.hdr.arena_bytes <= total <= pf.hdr.arena_bytes
    d = plan.describe((ROOT / "configs" / "b200_fsdp8b.cfg").read_text())
    flat_grad_bytes = 4 * d["total_params"]
    assert cb["grad"] < 0.3 * flat_grad_bytes          # dp = 8: a shard, two layer stages, the resident group
    assert abs(cb["optstate"] - d["mem_opt"]) <= 0.02 * d["mem_opt"]   # master + m + v of the shard, as modelled


@pytest.mark.parametrize("world,keys", [(2, "tp = 2"), (2, "pp = 2"), (4, "tp = 2\nep = 2"), (4, "pp = 2\nep = 2"),
                                        (8, "tp = 2\npp = 2\nep = 2"), (8, "ep = 8")])
def test_moe_layouts_compile_and_verify(tmp_path, world, keys):
    """Mixture-of-experts plans beside tensor and pipeline parallelism (what configs/full220k_moe.cfg mixes; reference
    emission: src/model.c:463-475,584-591): every rank compiles, the cluster verifier finds no unordered access, and
    the experts are spread over the tp x ep ranks of a stage."""
    from cai_b200 import plan
    text = (ROOT / "configs" / "tiny_moe_tp.cfg").read_text()
    text += f"\ngpus_per_rack = {world}\ngpus_per_tray = {world}\ncomm = fused\n{keys}\n"
    cfg = tmp_path / "moe.cfg"
    cfg.write_text(text)
    plan.compile_plans(cfg, tmp_path / "out", version=2)
    problems, report = plan.verify(cfg)
    assert problems == 0, report[-2000:]
    d = plan.describe(text)
    pf = plan.PlanFile(tmp_path / "out" / "plan.rank000000.bin")
    kinds = {int(x.kernel) for x in pf.exec}
    assert {plan.K_MOE_ROUTE, plan.K_MOE_DISPATCH_GEMM, plan.K_MOE_GEMM_COMBINE} <= kinds
    if d["tp"] > 1:
        assert {plan.K_AG_GEMM, plan.K_GEMM_RS} <= kinds     # attention stays tensor parallel around the experts


def test_trace_in_the_trace_event_format(tmp_path):
    """`trainer --trace x.json` writes the op timeline as Trace Event JSON (chrome://tracing, Perfetto): one track per
    logical stream, one complete event per op with the times of the CSV."""
    import csv
    import json
    run(BIN / "plan_compiler", ROOT / "configs" / "small.cfg", tmp_path, "--quiet", "--rank", "0")
    pl, tp = tmp_path / "plan.rank000000.bin", tmp_path / "topology.bin"
    run(BIN / "trainer", pl, tp, "--steps", "1", "--trace", tmp_path / "t.json")
    run(BIN / "trainer", pl, tp, "--steps", "1", "--trace", tmp_path / "t.csv")
    ev = json.loads((tmp_path / "t.json").read_text())["traceEvents"]
    rows = list(csv.DictReader(open(tmp_path / "t.csv")))
    spans = [e for e in ev if e["ph"] == "X"]
    assert len(spans) == len(rows) and {e["args"]["name"] for e in ev if e["ph"] == "M"} >= {"compute_hi", "comm_tp", "io"}
    for e, r in zip(spans[:50], rows[:50]):
        assert e["name"] == r["kind"] and abs(e["ts"] - float(r["start_us"])) < 1e-3 and abs(e["dur"] - float(r["dur_us"])) < 1e-3


# Executable plans of the benchmark configurations, rank 0 and the last rank, as they were when the repository's
# published step times were measured on B200s (sha256, first 16 hex digits). A change of the plan compiler that alters one of them is either
# deliberate (then the step has to be measured again and the digest updated) or a bug.
MEASURED_PLANS = {
    ("tp8", 1, "fused"): ("691edde438fa009a", "691edde438fa009a"),
    ("tp8", 2, "fused"): ("af14005d59482e38", "67362f9f01015e1e"),
    ("tp8", 4, "fused"): ("f074173f27db902b", "91fbd995d635d5cf"),
    ("tp8", 8, "fused"): ("3230a613780c1809", "cab1a76a3f6e89f2"),
    ("tp8", 8, "baseline"): ("37e665126f1978e3", "f43d11d7210b076f"),
    ("moe_ep8", 8, "fused"): ("7ce712fd5b4cd7d5", "fec1ef0e689e7b60"),
    ("fsdp8b", 8, "fused"): ("c6017d080ddc6ceb", "4fba568e1e74895c"),
    ("pp2tp4", 8, "fused"): ("a26a5476ec8825f0", "836a06f629acb32b"),
}


@pytest.mark.parametrize("key", sorted(MEASURED_PLANS))
def test_executable_plans_of_the_measured_configurations_are_unchanged(tmp_path, key):
    import sys
    sys.path.insert(0, str(ROOT))
    import bench
    from cai_b200 import plan
    name, n, comm = key
    plan.compile_plans(bench.config_text(n, comm, name), tmp_path, ranks=(0, n), version=2, text=True)
    got = tuple(hashlib.sha256((tmp_path / f"plan.rank{r:06d}.bin").read_bytes()).hexdigest()[:16] for r in (0, n - 1))
    assert got == MEASURED_PLANS[key]
