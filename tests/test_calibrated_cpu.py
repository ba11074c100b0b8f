"""The calibrated pricing backend: predictions for the headline config against the step times measured on B200s."""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "bin"

# tp = N, fused plans, defaults of the plan compiler: ms per step measured with bench.py on B200s
MEASURED_MS = {1: 433.9, 2: 237.3, 4: 138.7, 8: 108.0}


@pytest.fixture(scope="module", autouse=True)
def _built():
    from cai_b200 import _build
    _build.build_host()


def _plans(tmp_path, n, comm="fused", name="tp8"):
    sys.path.insert(0, str(ROOT))
    import bench
    from cai_b200 import plan
    out = tmp_path / f"{name}_{n}_{comm}"
    plan.compile_plans(bench.config_text(n, comm, name), out, ranks=(0, 1), version=2, text=True)
    return out / "plan.rank000000.bin", out / "topology.bin"


@pytest.mark.parametrize("n", [1, 2, 4, 8])
def test_predicted_step_time_is_within_ten_percent_of_the_measured_one(tmp_path, n):
    from cai_b200 import plan
    pl, tp = _plans(tmp_path, n)
    sim = plan.Simulator(pl, tp, backend="calibrated")
    s = sim.step()
    sim.close()
    predicted = s.step_time_s * 1e3
    assert abs(predicted - MEASURED_MS[n]) <= 0.10 * MEASURED_MS[n], (n, predicted, MEASURED_MS[n])
    # the reference's model (datasheet peaks, every op at 100 % efficiency) is several times too fast for the same plan
    ana = plan.Simulator(pl, tp, backend="analytic")
    a = ana.step()
    ana.close()
    assert a.step_time_s * 1e3 < 0.5 * MEASURED_MS[n]


def test_moe_step_with_grouped_expert_gemms_is_within_ten_percent(tmp_path):
    """Config 4 (64 experts, top-8, ep = 8): 321.8 ms per step measured. The grouped expert GEMMs are priced over the live
    rows of all local experts' slabs, dispatch and combine by the bytes they move."""
    from cai_b200 import plan
    pl, tp = _plans(tmp_path, 8, name="moe_ep8")
    sim = plan.Simulator(pl, tp, backend="calibrated")
    s = sim.step()
    sim.close()
    assert abs(s.step_time_s * 1e3 - 321.8) <= 0.10 * 321.8, s.step_time_s


def test_streams_do_not_overlap_beyond_what_the_sms_allow(tmp_path):
    """At tp = 8 the weight-gradient GEMMs sit on compute_lo beside the fused kernels on compute_hi; the predicted step is
    at least the critical stream and at most the sum of the two."""
    from cai_b200 import plan
    pl, tp = _plans(tmp_path, 8)
    sim = plan.Simulator(pl, tp, backend="calibrated")
    s = sim.step()
    sim.close()
    hi, lo = s.stream_busy[0], s.stream_busy[1]
    assert lo > 0 and hi <= s.step_time_s * 1.0001 and s.step_time_s <= (hi + lo) * 1.0001


def test_calibration_file_overrides_constants_and_unknown_keys_are_refused(tmp_path):
    pl, tp = _plans(tmp_path, 1)
    base = subprocess.run([str(BIN / "trainer"), str(pl), str(tp), "--steps", "1", "--backend", "calibrated"],
                          capture_output=True, text=True)
    assert base.returncode == 0 and "backend=calibrated" in base.stderr
    slow = tmp_path / "slow.cfg"
    slow.write_text("# half the per-SM GEMM rate\ngemm_sm_flops = 3.95e12\ngemm_sm_flops_ta = 3.45e12\n")
    r = subprocess.run([str(BIN / "trainer"), str(pl), str(tp), "--steps", "1", "--calibration", str(slow)],
                       capture_output=True, text=True)
    assert r.returncode == 0 and "backend=calibrated" in r.stderr

    def ms(out):
        line = [l for l in out.splitlines() if l.strip().startswith("0 |")][0]
        return float(line.split("|")[1].split()[0])
    assert ms(r.stdout) > 1.5 * ms(base.stdout)
    bad = tmp_path / "bad.cfg"
    bad.write_text("warp_speed = 9\n")
    r = subprocess.run([str(BIN / "trainer"), str(pl), str(tp), "--steps", "1", "--calibration", str(bad)],
                       capture_output=True, text=True)
    assert r.returncode != 0 and "unknown key" in r.stderr


def test_version_1_plans_fall_back_to_the_analytic_cost(tmp_path):
    """A version-1 plan has no kernel records: the calibrated backend prices it like the analytic one."""
    subprocess.run([str(BIN / "plan_compiler"), str(ROOT / "configs" / "small.cfg"), str(tmp_path), "--quiet"], check=True)
    from cai_b200 import plan
    out = []
    for backend in ("analytic", "calibrated"):
        sim = plan.Simulator(tmp_path / "plan.rank000000.bin", tmp_path / "topology.bin", backend=backend)
        out.append(sim.step().step_time_s)
        sim.close()
    assert out[1] >= out[0] * 0.999   # never below the analytic figure (the SM-work bound can only add)


def test_layout_advisor_ranks_executable_layouts(tmp_path):
    """`python -m cai_b200.plan.advise`: every layout of the headline model on 8 GPUs that keeps the global batch is
    priced; the benchmark's own layout (tp = 8) is among them with the step time the backend predicts for it."""
    from cai_b200.plan import advise
    ok, refused = advise.advise(ROOT / "configs" / "b200_tp8.cfg", gpus=8)
    assert not refused
    layouts = {(r["tp"], r["pp"], r["dp"], r["zero_stage"]) for r in ok}
    assert {(8, 1, 1, 1), (1, 1, 8, 1), (1, 1, 8, 3), (4, 2, 1, 1), (2, 2, 2, 1)} <= layouts
    assert all(r["grad_accum"] * r["dp"] == 8 for r in ok)            # global batch kept
    assert [r["step_ms"] for r in ok] == sorted(r["step_ms"] for r in ok) and all(r["fits"] for r in ok)
    tp8 = next(r for r in ok if (r["tp"], r["pp"]) == (8, 1))
    assert abs(tp8["step_ms"] - MEASURED_MS[8]) <= 0.10 * MEASURED_MS[8]
    r = subprocess.run([sys.executable, "-m", "cai_b200.plan.advise", str(ROOT / "configs" / "b200_moe_ep8.cfg"), "--gpus", "8"],
                       capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0 and "tokens/s" in r.stdout


def test_timelines_of_two_backends_compare_kind_by_kind(tmp_path):
    """`python -m cai_b200.plan.compare`: the predicted timeline (CSV) against the reference model's (Trace Event JSON) for
    the same plan: ops match by index, every kind shows up once per stream, the calibrated sums are the larger ones."""
    from cai_b200.plan import compare
    pl, tp = _plans(tmp_path, 8)
    for backend, out in (("calibrated", "pred.csv"), ("analytic", "ana.json")):
        r = subprocess.run([str(BIN / "trainer"), str(pl), str(tp), "--steps", "1", "--backend", backend, "--trace", str(tmp_path / out)],
                           capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
    table, odd = compare.compare(tmp_path / "pred.csv", tmp_path / "ana.json")
    assert not any(odd.values())
    kinds = {(r["kind"], r["stream"]) for r in table}
    assert {("gemm_rs", "compute_hi"), ("ag_gemm", "compute_hi"), ("gemm", "compute_lo"), ("attn_bwd", "comm_dp")} <= kinds
    assert all(r["a_ms"] >= r["b_ms"] for r in table if r["kind"] in ("gemm", "gemm_rs", "ag_gemm", "attn_fwd", "attn_bwd"))
    r = subprocess.run([sys.executable, "-m", "cai_b200.plan.compare", str(tmp_path / "pred.csv"), str(tmp_path / "ana.json")],
                       capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0 and "sum of op durations" in r.stdout


def test_bundled_calibration_file_spells_out_the_built_in_constants(tmp_path):
    """configs/b200_calibration.cfg documents every constant with its built-in value: loading it changes nothing."""
    pl, tp = _plans(tmp_path, 4)
    outs = []
    for extra in ([], ["--calibration", str(ROOT / "configs" / "b200_calibration.cfg")]):
        r = subprocess.run([str(BIN / "trainer"), str(pl), str(tp), "--steps", "1", "--backend", "calibrated"] + extra,
                           capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        outs.append([l for l in r.stdout.splitlines() if l.strip().startswith("0 |")][0])
    assert outs[0] == outs[1]


def test_fit_recovers_the_constants_a_timeline_was_made_with(tmp_path):
    """`python -m cai_b200.plan.fit`: timelines priced with altered constants (a slower GEMM, another launch cost, other
    attention step times, a slower RoPE) stand in for measured ones; the least-squares fit over three layouts of the
    headline model gives those constants back, and a file written from it reproduces the timelines."""
    from cai_b200.plan import fit
    truth = {"gemm_launch_us": 20.0, "gemm_tile_us": 1.5, "gemm_sm_flops": 5.0e12, "gemm_tile_us_ta": 6.0, "gemm_sm_flops_ta": 4.0e12,
             "attn_fwd_step_us": 2.2, "attn_fwd_fixed_us": 31.0, "attn_dkdv_step_us": 4.4, "attn_dq_step_us": 3.3,
             "attn_bwd_fixed_us": 12.0, "rope_fixed_us": 11.0, "rope_us_per_mb": 0.5, "rmsnorm_bwd_us_per_mb": 0.4}
    cal = tmp_path / "truth.cfg"
    cal.write_text("".join(f"{k} = {v}\n" for k, v in truth.items()))
    pairs = []
    for n in (1, 2, 8):
        pl, tp = _plans(tmp_path, n)
        out = tmp_path / f"measured{n}.csv"
        r = subprocess.run([str(BIN / "trainer"), str(pl), str(tp), "--steps", "1", "--calibration", str(cal), "--trace", str(out)],
                           capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        pairs.append((pl, out))
    consts, report = fit.fit(pairs)
    for k, v in truth.items():
        assert k in consts and abs(consts[k] - v) <= 0.02 * v, (k, consts.get(k), v, report)
    # the command-line form writes a calibration file that the backend accepts and that reproduces the step time
    flat = [str(x) for pair in pairs for x in pair]
    r = subprocess.run([sys.executable, "-m", "cai_b200.plan.fit"] + flat, capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stderr
    fitted = tmp_path / "fitted.cfg"
    fitted.write_text(r.stdout)
    pl, tp = pairs[2][0], pairs[2][0].parent / "topology.bin"

    def ms(calfile):
        rr = subprocess.run([str(BIN / "trainer"), str(pl), str(tp), "--steps", "1", "--calibration", str(calfile)], capture_output=True, text=True)
        assert rr.returncode == 0, rr.stderr
        return float([l for l in rr.stdout.splitlines() if l.strip().startswith("0 |")][0].split("|")[1].split()[0])
    assert abs(ms(fitted) - ms(cal)) <= 0.01 * ms(cal)
