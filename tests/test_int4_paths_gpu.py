"""Every int4 kernel variant against the oracle, each forced with AB_INT4_PATH in a child process
(the launcher reads the variable once).  The default selection is covered by test_int4_gpu.py; this
file keeps the variants that the default does not pick for these shapes under the same parity bar."""
import os
import subprocess
import sys

import pytest

from util import GEMM_TOL

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))

# path -> (shapes M x K x N, words the selection must contain)
PATHS = {
    "row": (["1x4096x4096", "1x1000x384", "1x33x256"], "streaming row kernel"),
    "simt": (["1x4096x1024", "3x512x384"], "row kernel"),
    "mma": (["5x4096x1024", "16x512x384", "20x256x128"], "m16n8k16"),
    "batch": (["1x4096x1024", "16x4096x11008", "16x1024x384", "20x4096x512", "3x48x640"], "cluster"),
    "tc": (["16x512x256", "128x4096x1024", "300x512x256", "5x100x256"], "tcgen05"),
    "tiles": (["16x512x256", "128x4096x1024", "300x512x256", "130x64x128"], "tile kernel"),
}


@pytest.mark.parametrize("path", sorted(PATHS))
def test_forced_variant_matches_the_oracle(path):
    shapes, words = PATHS[path]
    env = dict(os.environ, AB_INT4_PATH=path)
    out = subprocess.run([sys.executable, os.path.join(HERE, "int4_path_check.py"), *shapes], env=env,
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l.split("\t") for l in out.stdout.strip().splitlines()]
    assert len(lines) == len(shapes), out.stdout
    for shape, err, selection in lines:
        assert words in selection, (path, shape, selection)
        assert float(err) <= GEMM_TOL, (path, shape, err)
