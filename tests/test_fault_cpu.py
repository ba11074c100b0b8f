"""Failure detection and recovery, all on the host: no GPU is faulted, trapped or hung."""
import multiprocessing as mp
import subprocess
import time
from datetime import timedelta
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "bin"


@pytest.fixture(scope="module", autouse=True)
def _built():
    from cai_b200 import _build
    _build.build_host()


def _rank_main(rank, world, port, die_after, q):
    from torch.distributed import TCPStore
    from cai_b200.utils.health import Heartbeat, RankFailure
    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20))
    hb = Heartbeat(store, rank, world)
    try:
        for step in range(1, 6):
            if rank == 1 and step > die_after:
                q.put((rank, "exited", step))
                return                      # leaves between steps, nothing in flight
            hb.beat(step)
            hb.check(step, timeout=1.5)
        q.put((rank, "done", 5))
        time.sleep(0.5)
    except RankFailure as e:
        q.put((rank, "failure", e.missing, e.step))
        time.sleep(0.5)


def test_heartbeat_names_the_rank_that_left():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29871
    procs = [ctx.Process(target=_rank_main, args=(r, 3, port, 2, q)) for r in range(3)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=60)
    got = [q.get(timeout=5) for _ in range(3)]
    by_rank = {g[0]: g for g in got}
    assert by_rank[1][1] == "exited"
    for r in (0, 2):
        assert by_rank[r][1] == "failure" and by_rank[r][2] == [1] and by_rank[r][3] == 3


def _straggler_main(rank, world, port, q):
    from torch.distributed import TCPStore
    from cai_b200.utils.health import Heartbeat
    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20))
    hb = Heartbeat(store, rank, world)
    worst = (0.0, -1)
    for step in range(1, 5):
        if rank == 2 and step == 3:
            time.sleep(0.5)                 # a slow rank: late, but inside the deadline
        hb.beat(step)
        waited, last = hb.check(step, timeout=5.0)
        if step > 1 and waited > worst[0]:  # step 1 absorbs the processes' different start-up times
            worst = (waited, last)
    q.put((rank, worst))
    time.sleep(0.5)


def test_heartbeat_reports_the_rank_everyone_waited_for():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_straggler_main, args=(r, 3, 29873, q)) for r in range(3)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=60)
    got = dict(q.get(timeout=5) for _ in range(3))
    for r in (0, 1):
        waited, last = got[r]
        assert waited > 0.3 and last == 2, got
    assert got[2][0] < 0.3


def _collective_main(rank, world, port, q):
    import torch
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=timedelta(seconds=3))
    x = torch.ones(4)
    dist.all_reduce(x)                      # step 1: everyone takes part
    if rank == 1:
        q.put((rank, "left"))               # leaves between steps, nothing of its own in flight
        time.sleep(6.0)
        return
    t0 = time.monotonic()
    try:
        dist.all_reduce(x)                  # step 2: rank 1 never joins
        q.put((rank, "completed", time.monotonic() - t0))
    except Exception as e:                  # the short process-group timeout ends the wait with an error
        q.put((rank, "error", time.monotonic() - t0, type(e).__name__))


def test_collective_with_a_missing_rank_ends_with_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_collective_main, args=(r, 2, 29875, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict((g[0], g) for g in (q.get(timeout=60) for _ in range(2)))
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    assert got[1][1] == "left"
    assert got[0][1] == "error" and got[0][2] < 20.0, got


def test_watchdog_fires_on_an_overrunning_step_only():
    from cai_b200.utils.health import Watchdog
    hits = []
    wd = Watchdog(0.1, lambda: hits.append(time.monotonic()))
    wd.arm()
    time.sleep(0.03)
    wd.disarm()
    time.sleep(0.2)
    assert not hits
    wd.arm()
    time.sleep(0.3)
    assert len(hits) == 1 and wd.fired
    wd.close()


def test_injected_step_failure_writes_emergency_checkpoint_and_recovers(tmp_path):
    cfg = tmp_path / "spare.cfg"
    cfg.write_text((ROOT / "configs" / "small.cfg").read_text().replace("num_racks     = 1", "num_racks = 2")
                   .replace("spare_gpus    = 0", "spare_gpus = 12"))
    plans = tmp_path / "plans"
    subprocess.run([BIN / "plan_compiler", cfg, plans, "--quiet", "--rank", "7"], check=True, capture_output=True)
    pl, tp, ck = plans / "plan.rank000007.bin", plans / "topology.bin", tmp_path / "ck"
    env = {"RANK": "7", "PATH": "/usr/bin:/bin"}
    r = subprocess.run([BIN / "trainer", pl, tp, "--steps", "10", "--ckpt", ck, "--fail-at", "7"], capture_output=True,
                       text=True, env=env)
    assert r.returncode == 1 and "step 7 failed: backend error" in r.stderr
    em = tmp_path / "ck.emergency.rank000007"
    assert em.exists() and int.from_bytes(em.read_bytes()[:4], "little") == 7
    # the failed rank moves to a spare GPU: identical plan, resume from the rolling checkpoint
    r = subprocess.run([BIN / "plan_recover", cfg, "7", tmp_path / "rec"], capture_output=True, text=True)
    assert r.returncode == 0 and "different rack" in r.stdout
    rec = tmp_path / "rec" / "plan.recover.rank000007.bin"
    assert rec.read_bytes() == pl.read_bytes()
    r = subprocess.run([BIN / "trainer", rec, tp, "--steps", "10", "--ckpt", ck], capture_output=True, text=True, env=env)
    assert r.returncode == 0 and "   7 |" in r.stdout and "   6 |" not in r.stdout and "   9 |" in r.stdout


def test_corrupted_plan_and_missing_files_are_refused(tmp_path):
    from cai_b200 import plan
    subprocess.run([BIN / "plan_compiler", ROOT / "configs" / "small.cfg", tmp_path, "--quiet", "--rank", "0"], check=True,
                   capture_output=True)
    raw = bytearray((tmp_path / "plan.rank000000.bin").read_bytes())
    raw[16] ^= 0xFF                       # flip a byte of topology_hash
    (tmp_path / "bad.bin").write_bytes(raw)
    with pytest.raises(plan.PlanError):
        plan.Simulator(tmp_path / "bad.bin", tmp_path / "topology.bin")
    (tmp_path / "trunc.bin").write_bytes(raw[:1000])
    with pytest.raises(plan.PlanError):
        plan.Simulator(tmp_path / "trunc.bin", tmp_path / "topology.bin")
    with pytest.raises(plan.PlanError):
        plan.Simulator(tmp_path / "plan.rank000000.bin", tmp_path / "no_such_topology.bin")


def test_checkpoint_sections_are_checksummed_and_emergency_files_leave_latest_alone(tmp_path):
    """A flipped byte in a section is caught when the section is read back; a write with roll_latest = 0
    (what the trainer does after a failed step) does not replace the rolling "latest" file."""
    import ctypes
    import numpy as np
    from cai_b200 import plan
    L = plan.lib()
    path = str(tmp_path / "ck").encode()

    def write(tag, step, payload, roll):
        arr = np.frombuffer(payload, dtype=np.uint8).copy()
        names = (ctypes.c_char_p * 1)(b"master")
        data = (ctypes.c_void_p * 1)(ctypes.c_void_p(arr.ctypes.data))
        lens = (ctypes.c_uint64 * 1)(arr.nbytes)
        assert L.cai_ckpt_write2(path, tag, 3, step, 0xABCD, 1, names, data, lens, roll) == 0

    def read(file):
        name = ctypes.create_string_buffer(16)
        n = ctypes.c_uint64(0)
        assert L.cai_ckpt_section(file, 0, name, ctypes.byref(n), None, 0) == 0
        buf = np.empty(n.value, dtype=np.uint8)
        rc = L.cai_ckpt_section(file, 0, name, ctypes.byref(n), ctypes.c_void_p(buf.ctypes.data), buf.nbytes)
        return rc, buf.tobytes()

    good = bytes(range(256)) * 5 + b"tail"            # not a multiple of 8 bytes: the hash covers the tail too
    write(b"periodic", 5, good, 1)
    latest = tmp_path / "ck.latest.rank000003"
    assert read(str(latest).encode()) == (0, good)
    write(b"emergency", 7, b"half-updated state", 0)
    assert (tmp_path / "ck.emergency.rank000003").exists()
    assert read(str(latest).encode()) == (0, good)      # still step 5
    step = ctypes.c_uint32(0)
    assert L.cai_ckpt_probe(path, 3, ctypes.byref(step), None, None, None, 0) == 0 and step.value == 5
    raw = bytearray(latest.read_bytes())
    raw[-7] ^= 0x01
    latest.write_bytes(raw)
    rc, _ = read(str(latest).encode())
    assert rc != 0
