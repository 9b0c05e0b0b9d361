"""The driver seam (Device / Block / Executable / Fence) on a B200: the lifecycle and the refusals
accel's device layer relies on (internal/driver/driver.go:149-238, plan.go:360-428), and a small
decode-shaped plan run from host buffers to host buffers and checked against the oracle."""
import numpy as np
import pytest

import oracle as orc
from accel_b200 import driver as D
from accel_b200 import runtime as rt
from util import ATTN_TOL, GEMM_TOL, assert_close, attn_scale, normal, paged_fixture

pytestmark = pytest.mark.gpu


def op(block, nbytes=None, offset=0):
    return D.Operand(block=block, offset=offset, size=block.size if nbytes is None else nbytes)


def test_device_info_and_block_round_trip():
    assert D.device_count() >= 1
    info = D.device_info(0)
    assert info["cc"][0] == 10 and info["sm_count"] >= 100 and info["storage_offset_alignment"] == 256
    dev = D.Device(0)
    b = dev.alloc(1 << 20, label="scratch")
    assert b.bytes() is None and b.size == 1 << 20 and b.device_ptr % 256 == 0
    src = np.arange(1000, dtype=np.float32)
    b.write(256, src)
    assert np.array_equal(b.read(256, np.zeros(1000, np.float32)), src)
    with pytest.raises(D.AccelError, match="past"):
        b.write((1 << 20) - 8, src)
    h = dev.alloc(4096, D.MEMORY_HOST_VISIBLE)
    assert h.bytes() is not None
    with pytest.raises(D.AccelError, match="still live"):
        dev.close()                       # a device with live children refuses to close
    b.free(); h.free()
    assert dev.supports_kernel("AttentionDecodeBatched") and not dev.supports_kernel("MatMulTiled")
    dev.close()


def test_a_plan_runs_from_host_buffers_and_matches_the_oracle():
    # RMSNorm -> Int4MatMul -> (copy) -> ElemAdd, then a batched paged attention: the shape of a
    # slice of a decode layer, recorded once and submitted twice with a rewritten host payload
    M, K, N = 4, 256, 256
    x, g = normal(1, (M, K)), normal(2, (K,))
    w = normal(3, (K, N), 0.05)
    p, s, z = orc.int4_quantize(w)
    dev = D.Device(0, use_graphs=True)
    bx, bg = dev.upload(x), dev.upload(g)
    bp, bs, bz = dev.upload(p), dev.upload(s), dev.upload(z)
    bn, by, bc, bo = (dev.alloc(M * max(K, N) * 4) for _ in range(4))
    nodes = [
        D.HostWrite(op(bx, x.nbytes), x.tobytes()),
        D.Dispatch("RMSNorm", [op(bx, x.nbytes), op(bg), op(bn, M * K * 4)], rt.row_dims(M, K, 1e-5)),
        D.Dispatch("QuantMatMulInt4", [op(bn, M * K * 4), op(bp), op(bs), op(bz), op(by, M * N * 4)],
                   rt.gemm_dims(M, N, K)),
        D.Copy(op(by, M * N * 4), op(bc, M * N * 4)),
        D.Dispatch("ElemAdd", [op(by, M * N * 4), op(bc, M * N * 4), op(bo, M * N * 4)]),
    ]
    exe = dev.compile(nodes, collect_timings=True)

    def expect(xin):
        y = orc.quant_matmul_int4(orc.rmsnorm(xin, g, 1e-5), p, s, z, M, N, K)
        return y + y

    f = exe.submit()
    with pytest.raises(D.AccelError, match="in flight"):
        exe.submit()                      # one submission in flight per executable
    f.wait()
    assert f.done() and f.elapsed_ns() > 0
    assert_close(bo.read(0, np.zeros((M, N), np.float32)), expect(x), GEMM_TOL, "plan")
    x2 = normal(9, (M, K))
    exe.set_payload(0, x2.tobytes())      # OpHostWrite's payload is rewritten every submission
    f = exe.submit(); f.wait()
    assert_close(bo.read(0, np.zeros((M, N), np.float32)), expect(x2), GEMM_TOL, "plan, resubmitted")
    exe.close()
    for b in (bx, bg, bp, bs, bz, bn, by, bc, bo):
        b.free()
    dev.close()


def test_slots_rebind_and_uniform_rewrite():
    batch, qH, kvH, Dh, block = 3, 8, 2, 64, 8
    lengths = np.array([40, 9, 300], np.uint32)
    k, v, pages, mp = paged_fixture(4, batch, kvH, Dh, block, lengths)
    q = normal(5, (batch, qH, Dh))
    dev = D.Device(0)
    bq, bk, bv = dev.upload(q), dev.upload(k), dev.upload(v)
    bp, bl = dev.upload(pages), dev.upload(lengths)
    bo = dev.alloc(q.nbytes)
    sc = attn_scale(Dh)
    # K and V arrive through slots 1 and 2, as a State bound at submit time does
    nodes = [D.Dispatch("AttentionDecodeBatched",
                        [op(bq), D.Operand(slot=1, size=k.nbytes), D.Operand(slot=2, size=v.nbytes),
                         op(bp), op(bl), op(bo)],
                        rt.batched_dims(batch, qH, kvH, Dh, block, mp, sc))]
    exe = dev.compile(nodes, n_slots=2)
    with pytest.raises(D.AccelError, match="unbound"):
        exe.submit()
    with pytest.raises(D.AccelError, match="slot 3"):
        exe.rebind([(1, bk, 0), (3, bv, 0)])          # all or nothing: slot 1 stays unbound
    with pytest.raises(D.AccelError, match="unbound"):
        exe.submit()
    exe.rebind([(1, bk, 0), (2, bv, 0)])
    f = exe.submit(); f.wait()
    want = orc.attention_decode_batched(q, k, v, pages, lengths, batch, qH, kvH, Dh, block, mp, sc)
    assert_close(bo.read(0, np.zeros_like(q)).ravel(), want, ATTN_TOL, "slots")
    # the scale lives in the uniform block, which the layer above rewrites before every submit
    exe.set_uniform(0, rt.batched_dims(batch, qH, kvH, Dh, block, mp, sc * 0.5))
    f = exe.submit(); f.wait()
    want = orc.attention_decode_batched(q, k, v, pages, lengths, batch, qH, kvH, Dh, block, mp, sc * 0.5)
    assert_close(bo.read(0, np.zeros_like(q)).ravel(), want, ATTN_TOL, "uniform rewritten")
    exe.close()
    for b in (bq, bk, bv, bp, bl, bo):
        b.free()
    dev.close()


def test_compile_refusals():
    dev = D.Device(0)
    b = dev.alloc(4096)
    with pytest.raises(D.AccelError, match="no CPU fallback"):
        dev.compile([D.Dispatch("MatMulTiled", [op(b), op(b), op(b)], rt.gemm_dims(1, 1, 1))])
    with pytest.raises(D.AccelError, match="takes 3 bindings"):
        dev.compile([D.Dispatch("ElemAdd", [op(b), op(b)])])
    with pytest.raises(D.AccelError, match="uniform block"):
        dev.compile([D.Dispatch("RMSNorm", [op(b), op(b), op(b)])])
    with pytest.raises(D.AccelError, match="multiples of 256"):
        dev.compile([D.Dispatch("ElemAdd", [op(b, 64, 4), op(b, 64), op(b, 64)])])
    with pytest.raises(D.AccelError, match="whole number"):
        dev.compile([D.Dispatch("ElemAdd", [op(b, 6), op(b, 8), op(b, 8)])])
    exe = dev.compile([D.Dispatch("ElemAdd", [op(b, 8192), op(b, 64), op(b, 64)])])
    with pytest.raises(D.AccelError, match="runs past"):
        exe.submit()
    exe.close()
    b.free()
    dev.close()


def test_loss_is_injected_on_the_host_and_is_sticky():
    # CPUOptions.LoseAtSubmission (accel.go:306-314): the second submission reports loss; nothing
    # on the GPU faults, and every later call on the device returns the loss
    dev = D.Device(0, lose_at_submission=2)
    b = dev.alloc(4096)
    b.write(0, np.ones(16, np.float32))
    exe = dev.compile([D.Dispatch("ElemAdd", [op(b, 64), op(b, 64), op(b, 64, 256)])])
    f = exe.submit(); f.wait()
    assert not dev.lost()
    f = exe.submit()
    with pytest.raises(D.DeviceLost):
        f.wait()
    assert dev.lost()
    with pytest.raises(D.DeviceLost):
        exe.submit()
    with pytest.raises(D.DeviceLost):
        dev.alloc(64)
    exe.close(); b.free(); dev.close()


def test_a_block_cannot_be_freed_under_a_live_executable():
    # children before parents: an executable holds device addresses resolved from its blocks
    dev = D.Device(0)
    a, b, spare = dev.alloc(4096), dev.alloc(4096), dev.alloc(4096)
    a.write(0, np.ones(16, np.float32))
    exe = dev.compile([D.Dispatch("ElemAdd", [op(a, 64), op(a, 64), D.Operand(slot=1, size=64)])], n_slots=1)
    exe.rebind([(1, b, 0)])
    for blk in (a, b):
        with pytest.raises(D.AccelError, match="still name this block"):
            blk.free()
    exe.rebind([(1, spare, 0)])           # b is no longer named by the executable
    b.free()
    f = exe.submit(); f.wait()
    assert np.array_equal(spare.read(0, np.zeros(16, np.float32)), np.full(16, 2.0, np.float32))
    exe.close()
    a.free(); spare.free()
    dev.close()


def test_a_fence_that_was_only_polled_or_freed_releases_its_executable():
    dev = D.Device(0)
    b = dev.alloc(4096)
    b.write(0, np.ones(16, np.float32))
    exe = dev.compile([D.Dispatch("ElemAdd", [op(b, 64), op(b, 64), op(b, 64, 256)])])
    f = exe.submit()
    while not f.done():                   # completion learnt by polling, never waited for
        pass
    f2 = exe.submit()                     # not refused as busy
    f2.free()                             # freed unwaited: the executable is released all the same
    f3 = exe.submit(); f3.wait()
    exe.close(); b.free(); dev.close()


def test_every_outstanding_fence_reports_an_injected_loss():
    dev = D.Device(0, lose_at_submission=2)
    b = dev.alloc(4096)
    b.write(0, np.ones(16, np.float32))
    e1 = dev.compile([D.Dispatch("ElemAdd", [op(b, 64), op(b, 64), op(b, 64, 256)])])
    e2 = dev.compile([D.Dispatch("ElemAdd", [op(b, 64), op(b, 64), op(b, 64, 512)])])
    f1 = e1.submit()                      # submission 1: runs
    f2 = e2.submit()                      # submission 2: the loss is injected here, on the host
    with pytest.raises(D.DeviceLost):
        f1.wait()                         # the earlier fence reports the loss too
    with pytest.raises(D.DeviceLost):
        f2.wait()
    e1.close(); e2.close(); b.free(); dev.close()


@pytest.mark.parametrize("graphs", [False, True])
def test_several_submissions_in_flight(graphs):
    """CompileOptions.MaxInFlight (tensor/compile.go:19-27): above one, a submission that finds every
    instance busy lowers a spare, each with its own payload staging, up to the limit; a rebind
    between two submissions applies to the second only."""
    M, K = 4, 256
    g = normal(2, (K,))
    xs = [normal(10 + i, (M, K)) for i in range(3)]
    dev = D.Device(0, use_graphs=graphs)
    bx, bg = dev.alloc(M * K * 4), dev.upload(g)
    outs = [dev.alloc(M * K * 4) for _ in range(3)]
    nodes = [D.HostWrite(op(bx), xs[0].tobytes()),
             D.Dispatch("RMSNorm", [op(bx), op(bg), D.Operand(slot=1, size=M * K * 4)], rt.row_dims(M, K, 1e-5))]
    exe = dev.compile(nodes, n_slots=1, max_in_flight=2)
    fences = []
    for i in range(2):
        exe.rebind([(1, outs[i], 0)])              # allowed with submissions in flight
        exe.set_payload(0, xs[i].tobytes())
        fences.append(exe.submit())
    with pytest.raises(D.AccelError, match="all 2 instances"):
        exe.submit()
    fences[0].wait()
    exe.rebind([(1, outs[2], 0)])
    exe.set_payload(0, xs[2].tobytes())
    fences.append(exe.submit())                   # the first instance again
    for f in fences[1:]:
        f.wait()
    for i in range(3):
        got = outs[i].read(0, np.zeros((M, K), np.float32))
        assert_close(got, orc.rmsnorm(xs[i], g, 1e-5), 1e-6, f"submission {i} ran with its own payload and output")
    with pytest.raises(D.AccelError, match="executable"):
        outs[2].free()                            # still named by the executable's slot
    exe.close()
    for b in (bx, bg, *outs):
        b.free()
    dev.close()


def test_plan_cache_keys_on_what_the_plan_is():
    """tensor.PlanCache (tensor/cache.go:16-164): the same recorded plan compiles once; another
    kernel over the same shapes, or another MaxInFlight, is another plan; the label is not part of
    the key; a closed cache refuses."""
    M, K = 4, 256
    dev = D.Device(0)
    bx, bg, bo = dev.alloc(M * K * 4), dev.alloc(K * 4), dev.alloc(M * K * 4)

    def record(kernel):
        def rec():
            u = rt.row_dims(M, K, 1e-5) if kernel == "RMSNorm" else None
            binds = [op(bx), op(bg), op(bo)] if kernel == "RMSNorm" else [op(bx), op(bx), op(bo)]
            return [D.Dispatch(kernel, binds, u)], 0
        return rec

    cache = D.PlanCache(dev)
    a = cache.compile(record("RMSNorm"), D.CompileOptions(label="first"))
    b = cache.compile(record("RMSNorm"), D.CompileOptions(label="second"))
    assert a is b and len(cache) == 1 and cache.compiles == 1
    c = cache.compile(record("ElemAdd"))
    assert c is not a and len(cache) == 2
    d = cache.compile(record("RMSNorm"), D.CompileOptions(max_in_flight=4))
    assert d is not a and len(cache) == 3
    a.submit().wait()
    cache.close()
    with pytest.raises(D.AccelError, match="closed"):
        cache.compile(record("RMSNorm"))
    for blk in (bx, bg, bo):
        blk.free()
    dev.close()
