"""The grouped GEMM picks lone CTAs or CTA pairs (tcgen05 cta_group::2) by shape; the operator
parity tests mostly run shapes that select lone CTAs. Here the same tests run in a child process
with the tile mode forced either way (the library reads FMOE_GEMM_CTAS once per process), so that
every template variant of both modes - gathered rows through the relay warp, SwiGLU, FP8, fused
combine, scattered output rows - is held to the same parity bar."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SELECT = "index_select or silu_jagged or fused_combine or fp8 or layer or swiglu"


@pytest.mark.parametrize("ctas", ["1", "2"])
def test_operator_parity_with_forced_tile_mode(ctas):
    env = dict(os.environ, FMOE_GEMM_CTAS=ctas)
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-k", SELECT, "-p", "no:cacheprovider",
           os.path.join(ROOT, "tests", "test_gpu_parity.py"), os.path.join(ROOT, "tests", "test_gpu_fullsize.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    tail = "\n".join((r.stdout + r.stderr).splitlines()[-25:])
    assert r.returncode == 0, f"FMOE_GEMM_CTAS={ctas}:\n{tail}"
    assert " passed" in r.stdout
