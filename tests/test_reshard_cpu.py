"""Checkpoint resharding between parallel layouts, on the host only."""
import types
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module", autouse=True)
def _built():
    from cai_b200 import _build
    _build.build_host()


def _cfg(tmp_path, name, base, world, keys):
    text = (ROOT / "configs" / base).read_text()
    text += f"\ngpus_per_rack = {world}\ngpus_per_tray = {world}\ntrays_per_rack = 1\nnum_racks = 1\ncomm = fused\ntie_embeddings = 0\n{keys}\n"
    p = tmp_path / f"{name}.cfg"
    p.write_text(text)
    return p


def _random_state(layouts, seed):
    """A global master / m / v tensor per parameter, shapes taken from the layouts' own tables."""
    from cai_b200.utils import reshard
    rng = np.random.default_rng(seed)
    state = {}
    for layout in layouts:
        for rl in layout:
            for name, _, rows, cols in rl.params:
                gshape, _ = rl.slice_of(name, rows, cols)
                if name not in state:
                    state[name] = {k: rng.standard_normal(gshape).astype(np.float32) for k in reshard.STATE}
                assert state[name]["master"].shape == tuple(gshape), name
    return state


def _write(layout, state, step, path):
    from cai_b200.utils import reshard
    for rl in layout:
        reshard.write_rank(path, "periodic", rl, reshard.rank_sections(rl, state, step), step)


def _files(path, world):
    return [Path(f"{path}.latest.rank{r:06d}").read_bytes() for r in range(world)]


LAYOUTS = {
    "dense": ("tiny_mp.cfg", [(4, "tp = 2\npp = 2"), (2, "tp = 1\npp = 1"), (2, "zero_stage = 3"), (4, "tp = 4"),
                              (4, "tp = 2\nzero_stage = 3"), (4, "pp = 2\nzero_stage = 3"), (2, "zero_stage = 2"), (1, "")]),
    "moe": ("tiny_moe_tp.cfg", [(4, "tp = 2\nep = 2"), (2, "ep = 2"), (2, "tp = 2"), (4, "pp = 2\nep = 2"), (1, "")]),
}


@pytest.mark.parametrize("family", sorted(LAYOUTS))
def test_reshard_between_layouts_equals_cutting_the_global_state_directly(tmp_path, family):
    """State written for layout A and resharded to layout B is byte for byte what cutting the same global state for B
    gives, for chains of layouts that change the tensor, pipeline, data and expert split and the ZeRO stage."""
    from cai_b200.utils import reshard
    base, specs = LAYOUTS[family]
    cfgs = [_cfg(tmp_path, f"{family}{i}", base, w, k) for i, (w, k) in enumerate(specs)]
    layouts = [reshard.layout_of(c) for c in cfgs]
    state = _random_state(layouts, seed=7)
    _write(layouts[0], state, 41, tmp_path / "l0")
    # the gather alone gives the global state back exactly
    got, step = reshard.gather_global(layouts[0], lambda r: reshard.read_rank(tmp_path / "l0", r))
    assert step == 41 and set(got) == set(state)
    for name in state:
        for k in reshard.STATE:
            assert np.array_equal(got[name][k], state[name][k]), (name, k)
    prev = tmp_path / "l0"
    for i in range(1, len(layouts)):
        out = tmp_path / f"l{i}"
        s, n, ranks = reshard.reshard(cfgs[i - 1], prev, cfgs[i], out)
        assert s == 41 and ranks == len(layouts[i])
        _write(layouts[i], state, 41, tmp_path / f"direct{i}")
        assert _files(out, ranks) == _files(tmp_path / f"direct{i}", ranks), specs[i]
        prev = out


def test_slicing_rules_are_the_engines(tmp_path):
    """`reshard.global_slice` and `Engine._global_shape_and_slice` (which cuts a rank's shard at initialisation, and is
    what the multi-GPU tests validate against single-GPU training) agree for every parameter of every rank."""
    from cai_b200.runtime.engine import Engine
    from cai_b200.utils import reshard
    for base, specs in LAYOUTS.values():
        for i, (w, k) in enumerate(specs):
            for rl in reshard.layout_of(_cfg(tmp_path, f"s{base}{i}", base, w, k)):
                stub = types.SimpleNamespace(model=rl.model, rank=rl.rank,
                                             hdr=types.SimpleNamespace(tp=rl.tp, ep=rl.ep, num_stages=rl.pp, cp=1))
                for name, _, rows, cols in rl.params:
                    gs_a, (ra, ca) = reshard.global_slice(name, rows, cols, rl.model, rl.tp, rl.tp_id, rl.ep, rl.ep_id)
                    gs_b, (rb, cb) = Engine._global_shape_and_slice(stub, name, rows, cols)
                    assert tuple(gs_a) == tuple(gs_b), name
                    for a, b in ((ra, rb), (ca, cb)):
                        if isinstance(b, torch.Tensor):
                            assert np.array_equal(np.asarray(a), b.numpy()), name
                        else:
                            assert a == b, name


def test_foreign_or_mixed_step_checkpoints_are_refused(tmp_path):
    from cai_b200 import plan
    from cai_b200.utils import reshard
    a = _cfg(tmp_path, "a", "tiny_mp.cfg", 2, "tp = 2")
    b = _cfg(tmp_path, "b", "tiny_mp.cfg", 1, "")
    la = reshard.layout_of(a)
    state = _random_state([la], seed=3)
    _write(la, state, 5, tmp_path / "ck")
    reshard.write_rank(tmp_path / "ck", "periodic", la[1], reshard.rank_sections(la[1], state, 6), 6)   # rank 1 one step ahead
    with pytest.raises(plan.PlanError):
        reshard.reshard(a, tmp_path / "ck", b, tmp_path / "out")
    other = _cfg(tmp_path, "other", "tiny_mp.cfg", 2, "tp = 2\nseq_len = 128")          # another plan hash
    _write(la, state, 5, tmp_path / "ck2")
    with pytest.raises(plan.PlanError):
        reshard.reshard(other, tmp_path / "ck2", b, tmp_path / "out2")


def test_tied_head_is_copied_when_the_destination_unties_it_and_never_dropped_silently(tmp_path):
    """tie_embeddings = 1 holds for unpipelined layouts only. Tied -> pipelined: the head starts as the embedding.
    Pipelined (head trained on its own) -> tied: refused, nothing is thrown away without a word."""
    from cai_b200 import plan
    from cai_b200.utils import reshard
    tied = _cfg(tmp_path, "tied", "tiny_mp.cfg", 1, "tie_embeddings = 1")
    piped = _cfg(tmp_path, "piped", "tiny_mp.cfg", 2, "tie_embeddings = 1\npp = 2")
    lt, lp = reshard.layout_of(tied), reshard.layout_of(piped)
    assert "lm_head" not in {n for n, *_ in lt[0].params} and "lm_head" in {n for n, *_ in lp[1].params}
    state = _random_state([lt], seed=11)
    _write(lt, state, 9, tmp_path / "t")
    reshard.reshard(tied, tmp_path / "t", piped, tmp_path / "p")
    got, _ = reshard.gather_global(lp, lambda r: reshard.read_rank(tmp_path / "p", r))
    assert np.array_equal(got["lm_head"]["master"], state["embed"]["master"])
    reshard.reshard(piped, tmp_path / "p", tied, tmp_path / "t2")          # still equal: allowed
    assert _files(tmp_path / "t2", 1) == _files(tmp_path / "t", 1)
    got["lm_head"]["master"] = got["lm_head"]["master"] + 1.0               # the head has moved away from the embedding
    _write(lp, got, 10, tmp_path / "p2")
    with pytest.raises(plan.PlanError):
        reshard.reshard(piped, tmp_path / "p2", tied, tmp_path / "t3")


def test_checkpoint_inspector_lists_sections_and_notices_damage(tmp_path):
    import subprocess
    import sys
    from cai_b200.utils import ckpt_info, reshard
    cfg = _cfg(tmp_path, "one", "tiny_mp.cfg", 1, "")
    layout = reshard.layout_of(cfg)
    _write(layout, _random_state([layout], seed=5), 17, tmp_path / "ck")
    info = ckpt_info.inspect(tmp_path / "ck", 0)
    assert info["step"] == 17 and info["plan_hash"] == layout[0].plan_hash
    assert [s[0] for s in info["sections"]] == ["param", "master", "m", "v", "meta"] and all(s[2] for s in info["sections"])
    assert dict((s[0], s[1]) for s in info["sections"])["master"] == 4 * layout[0].n_opt
    f = Path(info["file"])
    raw = bytearray(f.read_bytes())
    raw[len(raw) // 2] ^= 0x40                      # one flipped bit in the middle of the file
    f.write_bytes(bytes(raw))
    r = subprocess.run([sys.executable, "-m", "cai_b200.utils.ckpt_info", str(tmp_path / "ck")], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 1 and "CHECKSUM MISMATCH" in r.stdout
