"""Shrinking a run after GPUs were lost: layout choice on the remaining GPUs and the checkpoint rearranged for it."""
from pathlib import Path

import numpy as np
import pytest

from test_reshard_cpu import _cfg, _files, _random_state, _write

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module", autouse=True)
def _built():
    from cai_b200 import _build
    _build.build_host()


def test_four_gpus_minus_one_continue_on_a_layout_that_tiles_and_keep_the_global_batch(tmp_path, capsys):
    from cai_b200 import plan
    from cai_b200.utils import elastic, reshard
    src = _cfg(tmp_path, "src", "tiny_mp.cfg", 4, "tp = 2\npp = 2")
    layout = reshard.layout_of(src)
    state = _random_state([layout], seed=3)
    _write(layout, state, 17, tmp_path / "run")
    out_cfg, out_ck = tmp_path / "shrunk.cfg", tmp_path / "run_shrunk"
    rc = elastic.main(["--config", str(src), "--lost", "1", "--ckpt", str(tmp_path / "run"), "--out-config", str(out_cfg),
                       "--out-ckpt", str(out_ck)])
    assert rc == 0
    text = capsys.readouterr().out
    assert "4 -> 3 GPUs" in text and "global batch kept" in text
    before, after = plan.describe(src.read_text()), plan.describe(out_cfg.read_text())
    assert after["world_size"] <= 3 and after["global_batch"] == before["global_batch"]
    assert after["plan_hash"] != before["plan_hash"] or after["world_size"] != before["world_size"]
    # the new configuration compiles to executable plans that verify, and the checkpoint written for it is the global
    # state of the old run cut for the new layout
    plan.compile_plans(out_cfg.read_text(), tmp_path / "plans", ranks=(0, after["world_size"]), version=2, text=True)
    assert plan.verify(out_cfg, check_exec=True)[0] == 0
    dst = reshard.layout_of(out_cfg)
    _write(dst, state, 17, tmp_path / "direct")
    assert _files(out_ck, len(dst)) == _files(tmp_path / "direct", len(dst))
    got, step = reshard.gather_global(dst, lambda r: reshard.read_rank(out_ck, r))
    assert step == 17 and all(np.array_equal(got[n]["master"], state[n]["master"]) for n in state)


def test_spares_are_left_to_plan_recover_and_bad_counts_are_refused(tmp_path, capsys):
    from cai_b200.utils import elastic
    cfg = tmp_path / "spare.cfg"
    cfg.write_text((ROOT / "configs" / "tiny_mp.cfg").read_text() +
                   "\ngpus_per_rack = 5\ngpus_per_tray = 5\ntrays_per_rack = 1\nnum_racks = 1\nspare_gpus = 1\ntp = 2\npp = 2\n")
    assert elastic.main(["--config", str(cfg), "--lost", "1", "--out-config", str(tmp_path / "o.cfg")]) == 0
    assert "plan_recover" in capsys.readouterr().out and not (tmp_path / "o.cfg").exists()
    assert elastic.main(["--config", str(cfg), "--gpus-left", "9", "--out-config", str(tmp_path / "o.cfg")]) == 2


def test_shrink_prefers_fewer_gpus_only_when_that_is_faster_or_the_only_way(tmp_path):
    from cai_b200.utils import elastic
    text = (ROOT / "configs" / "b200_tp8.cfg").read_text()
    world, best = elastic.shrink(text, 7)
    # 7 GPUs tile neither 8 kv heads, 24 layers nor a global batch of 8: the job continues on fewer
    assert best is not None and world < 7 and 8 % best["dp"] == 0 and best["fits"]
    world6, best6 = elastic.shrink(text, 6)
    assert (world6, best6["tp"], best6["pp"], best6["dp"]) == (world, best["tp"], best["pp"], best["dp"]) or best6["step_ms"] <= best["step_ms"]
