"""Joint replay of all stages of a pipeline: sends meet their receives, no closed bubble formula."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "bin"


@pytest.fixture(scope="module", autouse=True)
def _built():
    from cai_b200 import _build, plan
    _build.build_host()
    plan.set_log_level("warn")


def _stage_plans(tmp_path, text, version):
    from cai_b200 import plan
    d = plan.describe(text)
    plan.compile_plans(text, tmp_path, ranks=(0, d["world_size"]), version=version, text=True)
    stride = d["tp"] * d.get("cp", 1)
    return [tmp_path / f"plan.rank{s * stride:06d}.bin" for s in range(d["pp"])], tmp_path / "topology.bin", d


def test_config_5_is_predicted_within_five_percent_of_the_measured_step(tmp_path):
    """pp 2 x tp 4, 48 layers, full recompute: 2446 ms per step measured on 8 B200s. One stage's busy time stretched by
    the bubble formula gives 2581 ms; the joint replay needs no formula."""
    sys.path.insert(0, str(ROOT))
    import bench
    from cai_b200 import plan
    paths, topo, d = _stage_plans(tmp_path, bench.config_text(8, "fused", "pp2tp4"), 2)
    r = plan.pipeline_replay(paths, topo, backend="calibrated")
    assert abs(r["step_time_s"] * 1e3 - 2446.0) <= 0.05 * 2446.0, r
    # the step is the longer of the longest dependency path and the SM time of the busiest stage; here the stages are
    # SM-bound (weight-gradient GEMMs on the second compute stream fill the gaps of fill and drain)
    assert len(r["stage_finish_s"]) == 2 and max(r["stage_finish_s"]) < r["step_time_s"]
    assert max(r["stage_sm_busy_s"]) == pytest.approx(r["step_time_s"])
    assert all(0.0 <= x < 0.5 for x in r["stage_idle_hi"])
    assert r["bubble_formula"] == pytest.approx(1.0 / 17.0)


def test_one_stage_gives_the_single_plan_replay(tmp_path):
    from cai_b200 import plan
    paths, topo, _ = _stage_plans(tmp_path, (ROOT / "configs" / "tiny.cfg").read_text(), 2)
    for backend in ("analytic", "calibrated"):
        sim = plan.Simulator(paths[0], topo, backend=backend)
        single = sim.step().step_time_s
        sim.close()
        assert plan.pipeline_replay(paths, topo, backend=backend)["step_time_s"] == pytest.approx(single, rel=1e-12)


def test_cost_only_plans_of_the_reference_schedule_replay_without_the_formula(tmp_path):
    """small.cfg (tp 4, pp 3, dp 6; version-1 plans, both directions on one stream, sends that do not wait): the step
    lies between the slowest stage's own critical path and that path stretched by the formula (what the single-plan
    replay reports)."""
    from cai_b200 import plan
    paths, topo, d = _stage_plans(tmp_path, (ROOT / "configs" / "small.cfg").read_text(), 1)
    r = plan.pipeline_replay(paths, topo, backend="analytic")
    stretched = []
    for pth in paths:
        sim = plan.Simulator(pth, topo, backend="analytic")
        stretched.append(sim.step().step_time_s)        # the stage's critical path / (1 - bubble)
        sim.close()
    own_work = max(stretched) * (1.0 - r["bubble_formula"])
    assert own_work < r["step_time_s"] <= max(stretched) * 1.02
    assert r["stage_finish_s"][0] == pytest.approx(r["step_time_s"])       # stage 0 ends the step: it drains last
    # the first stages idle more than the last one, which also runs the LM head and the loss
    assert r["stage_idle_hi"][0] > r["stage_idle_hi"][-1]


def test_a_missing_stage_or_foreign_plan_is_refused(tmp_path):
    from cai_b200 import plan
    a = tmp_path / "a"
    b = tmp_path / "b"
    paths, topo, _ = _stage_plans(a, (ROOT / "configs" / "small.cfg").read_text(), 1)
    with pytest.raises(plan.PlanError, match="stage"):
        plan.pipeline_replay(paths[:2], topo, backend="analytic")
    with pytest.raises(plan.PlanError, match="stage"):
        plan.pipeline_replay([paths[0], paths[2], paths[1]], topo, backend="analytic")
    other, _, _ = _stage_plans(b, (ROOT / "configs" / "small.cfg").read_text() + "\nseq_len = 2048\n", 1)
    with pytest.raises(plan.PlanError, match="different configurations"):
        plan.pipeline_replay([paths[0], other[1], paths[2]], topo, backend="analytic")


def test_trainer_tool_finds_the_sibling_stages_and_writes_one_timeline(tmp_path):
    from cai_b200 import plan
    text = (ROOT / "configs" / "tiny_mp.cfg").read_text() + "\ntp = 2\npp = 2\ngpus_per_rack = 4\ngpus_per_tray = 4\n"
    paths, topo, _ = _stage_plans(tmp_path, text, 2)
    trace = tmp_path / "pipe.json"
    r = subprocess.run([BIN / "trainer", paths[1], topo, "--pipeline", "--backend", "calibrated", "--trace", trace],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    assert "pipeline bubble by formula 20.0%" in r.stdout and "stage |   rank" in r.stdout
    ev = json.loads(trace.read_text())["traceEvents"]
    assert {e["pid"] for e in ev} == {0, 1}
    sends = [e for e in ev if e.get("ph") == "X" and e["name"] == "pipe_send"]
    assert sends and all("microbatch" in e["args"] for e in sends)
    # a stage whose plan file is missing is named
    paths[0].unlink()
    r = subprocess.run([BIN / "trainer", paths[1], topo, "--pipeline"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 1 and "plan.rank000000.bin" in r.stderr


def test_device_trainer_predicts_a_pipelined_job_with_all_stages(tmp_path):
    """The prediction the device trainer prints beside its measurement: joint replay when the job is pipelined and
    the configuration is known, this rank's plan alone otherwise."""
    import types
    from cai_b200 import plan, trainer
    text = (ROOT / "configs" / "tiny_mp.cfg").read_text() + "\ntp = 2\npp = 2\ngpus_per_rack = 4\ngpus_per_tray = 4\n"
    plan.compile_plans(text, tmp_path, ranks=(3, 4), version=2, text=True)      # rank 3: stage 1, tp rank 1
    pf = plan.PlanFile(tmp_path / "plan.rank000003.bin")
    eng = types.SimpleNamespace(hdr=pf.hdr, config_text=text, plan=pf, topology_path=str(tmp_path / "topology.bin"))
    joint = trainer.predicted_step_time(eng, 3)
    eng.config_text = None
    alone = trainer.predicted_step_time(eng, 3)
    assert 0 < joint < alone * 1.2 and joint != alone
