"""The parity suites once more on the checked build of the library (-DFFTOPK_CHECKED): every index
the selection logic guarantees to be in range - output slots, reserved candidate slots, staged row
indices, the winner count of every finish - is tested on the device. A failing test raises
FFTOPK_ST_CHECK in the status word, which the suites assert to be zero after every call, and
leaves a record (site, index, limit, block) that the child's session prints when it ends (conftest.py).

Runs in a child process because the library is chosen when the package is first imported
(FFTOPK_LIBRARY)."""
import importlib.util
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parent.parent

def _checked_library() -> Path:
    spec = importlib.util.spec_from_file_location("_fftopk_build", REPO / "flash-float-jit-kernels_b200" / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build_checked_library()


@pytest.mark.timeout(1500)
def test_parity_suites_on_the_checked_build():
    lib = _checked_library()
    env = dict(os.environ, FFTOPK_LIBRARY=str(lib))
    suites = ["tests/test_select_gpu.py", "tests/test_general_k_gpu.py", "tests/test_merge_gpu.py",
              "tests/test_transform_gpu.py", "tests/test_warm_gpu.py"]
    suites = [s for s in suites if (REPO / s).exists()]
    res = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider", *suites],
                         cwd=REPO, env=env, capture_output=True, text=True)
    tail = (res.stdout + res.stderr)[-3000:]
    assert res.returncode == 0, f"checked build: a suite failed\n{tail}"
    assert " passed" in res.stdout
