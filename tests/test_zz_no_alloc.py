"""The allocation-free int4 entry point against the regular one, on a B200.

Hosts that may not allocate device memory (a plugin living inside another runtime's allocator, a
control loop that must stay out of the driver's allocator, a sandbox with cudaMalloc closed off)
call ab_quant_matmul_int4_noalloc, whose split-K scratch is an array built into the library.  It
must give exactly what ab_launch gives with a caller-supplied workspace, call after call, since
every call reuses the same scratch.  This file sorts last so that a failure here cannot hide the
rest of the suite from a run that stops at the first failure.

Most shapes select kernels that sum their K splits inside a thread-block cluster and need no
scratch at all; the cases below therefore include shapes whose plan DOES spill partial sums to the
scratch (one wave of clusters does not cover N = 32000), assert that it does, and run the older
two-kernel row form (AB_INT4_PATH=simt), which always uses it, in a child process."""
import ctypes as C
import os
import subprocess
import sys

import pytest
import torch

from accel_b200 import _lib, quant, runtime

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SHAPES = [(16, 4096, 4096), (1, 4096, 11008), (5, 1024, 384), (4, 4096, 32000), (2, 4096, 32000)]
SCRATCH_SHAPES = [(4, 4096, 32000)]          # must need scratch under the default selection


def _noalloc(a, codes, scales, zeros, out, M, N, K, stream=None):
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream if stream is None else stream
    _lib.check(L.ab_quant_matmul_int4_noalloc(C.c_void_p(stream), a.data_ptr(), codes.data_ptr(),
                                              scales.data_ptr(), zeros.data_ptr(), out.data_ptr(),
                                              M, N, K))


def _scratch_bytes(M, K, N):
    name = "QuantMatMulInt4" if M > 1 else "QuantMatVecInt4"
    return runtime.workspace_bytes(name, [M * K, K * N // 8, K * N // 128, K * N // 128, M * N],
                                   runtime.gemm_dims(M if M > 1 else 0, N, K))


def _two_calls(M, K, N):
    torch.manual_seed(M * 7 + N)
    mats = [quant.int4_quantize_device(torch.randn(K, N, device=DEV) * 0.02) for _ in range(2)]
    acts = [torch.randn(M, K, device=DEV) for _ in range(2)]
    name = "QuantMatMulInt4" if M > 1 else "QuantMatVecInt4"
    for call in range(2):                      # the second call finds the first one's partial sums
        a, (c, s, z) = acts[call], mats[call]
        want = torch.empty(M, N, device=DEV)
        runtime.launch(name, [a, c, s, z, want], runtime.gemm_dims(M if M > 1 else 0, N, K))
        got = torch.full((M, N), float("nan"), device=DEV)
        _noalloc(a, c, s, z, got, M, N, K)
        torch.cuda.synchronize()
        # same kernels, same split plan, same order of sums: the tolerance of the int4 tests (1e-3
        # relative) is far looser than what is expected here, which is equality
        err = (got - want).abs().max().item() / want.abs().max().item()
        assert err <= 1e-3, (call, err)
        assert torch.equal(got, want), call


@pytest.mark.parametrize("M,K,N", SHAPES)
def test_two_calls_in_a_row_match_the_regular_entry_point(M, K, N):
    _two_calls(M, K, N)


@pytest.mark.parametrize("M,K,N", SCRATCH_SHAPES)
def test_the_scratch_shapes_do_use_the_scratch(M, K, N):
    need = _scratch_bytes(M, K, N)
    assert 0 < need <= 8 << 20, need


def test_the_two_kernel_row_form_in_a_child_process():
    """AB_INT4_PATH is read once per process, so the older row form (partial sums of every K split
    written to the scratch, then a reduce kernel) runs in a child."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, AB_INT4_PATH="simt",
               PYTHONPATH=os.pathsep.join([root, os.path.join(root, "tests"), os.environ.get("PYTHONPATH", "")]))
    r = subprocess.run([sys.executable, os.path.abspath(__file__)], env=env, capture_output=True,
                       text=True, timeout=600, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "scratch bytes" in r.stdout


def test_a_shape_beyond_the_built_in_scratch_is_refused():
    # 64 rows against a 4096 x 32000 matrix wants far more than 8 MiB of partial sums
    M, K, N = 64, 4096, 32000
    need = runtime.workspace_bytes("QuantMatMulInt4", [M * K, K * N // 8, K * N // 128, K * N // 128, M * N],
                                   runtime.gemm_dims(M, N, K))
    assert need > 8 << 20
    t = torch.zeros(64, device=DEV)
    with pytest.raises(_lib.AccelError, match="built-in array holds"):
        _noalloc(t, t, t, t, t, M, N, K)


def test_a_stream_of_another_device_is_refused():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    other = torch.cuda.Stream(device="cuda:1")
    t = torch.zeros(4096, device=DEV)
    with torch.cuda.device(0), pytest.raises(_lib.AccelError, match="belongs to device 1"):
        _noalloc(t, t, t, t, t, 1, 128, 128, stream=other.cuda_stream)


if __name__ == "__main__":
    # the child of test_the_two_kernel_row_form_in_a_child_process
    total = 0
    for shape in [(1, 4096, 11008), (1, 1024, 384), (3, 4096, 4096)]:
        need = _scratch_bytes(*shape)
        total += need
        _two_calls(*shape)
        print(shape, "scratch bytes", need)
    assert total > 0, "no shape used the scratch under AB_INT4_PATH=" + os.environ.get("AB_INT4_PATH", "")
