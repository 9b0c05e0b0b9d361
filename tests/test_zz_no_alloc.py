"""The allocation-free int4 entry point against the regular one, on a B200.

Hosts that may not allocate device memory (a plugin living inside another runtime's allocator, a
control loop that must stay out of the driver's allocator, a sandbox with cudaMalloc closed off)
call ab_quant_matmul_int4_noalloc, whose split-K scratch is an array built into the library.  It
must give exactly what ab_launch gives with a caller-supplied workspace, call after call, since
every call reuses the same scratch.  This file sorts last so that a failure here cannot hide the
rest of the suite from a run that stops at the first failure."""
import ctypes as C

import numpy as np
import pytest
import torch

from accel_b200 import _lib, quant, runtime

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _noalloc(a, codes, scales, zeros, out, M, N, K):
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(L.ab_quant_matmul_int4_noalloc(C.c_void_p(stream), a.data_ptr(), codes.data_ptr(),
                                              scales.data_ptr(), zeros.data_ptr(), out.data_ptr(),
                                              M, N, K))


@pytest.mark.parametrize("M,K,N", [(16, 4096, 4096), (1, 4096, 11008), (5, 1024, 384)])
def test_two_calls_in_a_row_match_the_regular_entry_point(M, K, N):
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


def test_a_shape_beyond_the_built_in_scratch_is_refused():
    # 64 rows against a 4096 x 32000 matrix wants far more than 8 MiB of partial sums
    M, K, N = 64, 4096, 32000
    need = runtime.workspace_bytes("QuantMatMulInt4", [M * K, K * N // 8, K * N // 128, K * N // 128, M * N],
                                   runtime.gemm_dims(M, N, K))
    assert need > 8 << 20
    t = torch.zeros(64, device=DEV)
    with pytest.raises(_lib.AccelError, match="built-in array holds"):
        _noalloc(t, t, t, t, t, M, N, K)
