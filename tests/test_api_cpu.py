"""The package's front door: public names resolve lazily, and importing the package needs no GPU and no torch."""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_import_is_light_and_public_names_resolve():
    code = ("import sys, cai_b200\n"
            "assert 'torch' not in sys.modules, 'importing the package must not pull torch in'\n"
            "for n in cai_b200.__all__: assert getattr(cai_b200, n) is not None, n\n"
            "assert cai_b200.plan.PlanFile is cai_b200.PlanFile\n"
            "print(cai_b200.__version__)\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.strip()


def test_unknown_attribute_is_an_attribute_error():
    import cai_b200
    with pytest.raises(AttributeError):
        cai_b200.no_such_thing
    assert not hasattr(cai_b200, "__wrapped__")


def test_log_level_from_the_environment_and_the_api(tmp_path):
    """CAI_LOG_LEVEL sets the native library's starting level; set_log_level overrides it."""
    import os
    code = ("from cai_b200 import plan\n"
            "import sys\n"
            "if len(sys.argv) > 1: plan.set_log_level(sys.argv[1])\n"
            f"plan.compile_plans(open('{ROOT}/configs/tiny.cfg').read(), '{tmp_path}', ranks=(0, 1), version=2, text=True)\n"
            f"s = plan.Simulator('{tmp_path}/plan.rank000000.bin', '{tmp_path}/topology.bin', rank=0)\n"
            "s.step(); s.close()\n")
    def run(env_level=None, arg=None):
        env = {k: v for k, v in os.environ.items() if k != "CAI_LOG_LEVEL"}
        if env_level:
            env["CAI_LOG_LEVEL"] = env_level
        r = subprocess.run([sys.executable, "-c", code] + ([arg] if arg else []), capture_output=True, text=True, cwd=ROOT, env=env, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        return r.stderr
    assert "[cai INFO] plan loaded" in run()
    assert "[cai INFO]" not in run(env_level="warn")
    assert "[cai INFO]" not in run(env_level="0")
    assert "[cai INFO] plan loaded" in run(env_level="warn", arg="info")
    assert "[cai INFO]" not in run(arg="error")
