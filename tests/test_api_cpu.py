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
