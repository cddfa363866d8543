"""The Q8_1 activation ABI on the GPU: producers byte for byte against the reference's analytic fixtures
(nvidia/x/cudaquant/norm_source_test.go:24-66, norm_contract_test.go) and the oracle on seeded rows, consumers
and the matvec over selected experts against the oracle's products on the decoded vector."""
import struct

import numpy as np
import pytest

import lib_b200
from lib_b200 import _capi, synth
from oracle import oracle
from tests import q8_1_cases as cases

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fx", cases.norm_fixtures(), ids=lambda f: f[0])
def test_norm_analytic_fixtures(ctx, fx):
    # the byte-equality check of norm_native_test.go, against the same expected blocks
    name, rows, cols, eps, weighted, x, w, want = fx
    assert ctx.RMSNormQ8_1(x, w, rows, cols, eps, weighted) == want


def test_known_layout_and_saturation(ctx):
    got = ctx.RMSNormQ8_1(np.ones(32, dtype=np.float32), None, 1, 32, 0.0, False)
    assert struct.unpack_from("<HH", got) == (0x2008, 0x5000) and got[4:] == bytes([127] * 32)
    x = np.zeros(32, dtype=np.float32)
    x[0] = 100
    got = ctx.RMSNormQ8_1(x, None, 1, 32, 0.0, False)
    assert got[4] == 127 and got[5:] == bytes(31)


@pytest.mark.parametrize("rows,cols,eps,value,code", [(2 ** 63 - 1, 32, 1.0, 0.0, -4), (1, 32, float("inf"), 0.0, -4),
                                                      (1, 32, 1.0, float("nan"), -12), (1, 32, 0.0, 0.0, -12)],
                         ids=["overflow", "infinite epsilon", "nan input", "zero denominator"])
def test_invalid_inputs(ctx, rows, cols, eps, value, code):
    # norm_contract_test.go:31-52: every one of these is refused
    x = np.zeros(32, dtype=np.float32)
    x[0] = value
    with pytest.raises(lib_b200.QmError) as e:
        ctx.RMSNormQ8_1(x, None, rows, cols, eps, False)
    assert e.value.code == code
    ctx.RMSNormQ8_1(np.ones(32, dtype=np.float32), None, 1, 32, 0.0, False)   # the context stays usable and clean


def test_more_refusals(ctx):
    z, w31 = np.zeros(32, dtype=np.float32), np.zeros(31, dtype=np.float32)
    for args, code in [((z, w31, 1, 32, 1e-5, True), -2), ((np.zeros(33, dtype=np.float32), None, 1, 32, 1e-5, False), -2),
                       ((np.zeros(48, dtype=np.float32), None, 1, 48, 1e-5, False), -4), ((z, None, 1, 32, -1.0, False), -4)]:
        with pytest.raises(lib_b200.QmError) as e:
            ctx.RMSNormQ8_1(*args)
        assert e.value.code == code
    w = np.ones(32, dtype=np.float32)
    w[3] = np.inf
    with pytest.raises(lib_b200.QmError) as e:
        ctx.RMSNormQ8_1(np.ones(32, dtype=np.float32), w, 1, 32, 0.0, True)
    assert e.value.code == -12
    w[3] = 3e38
    with pytest.raises(lib_b200.QmError) as e:
        ctx.RMSNormQ8_1(np.eye(1, 32, 3, dtype=np.float32), w, 1, 32, 0.0, True)
    assert e.value.code == -12


@pytest.mark.parametrize("rows,cols,weighted,scale", [(1, 4096, True, 1.0), (8, 4096, False, 3.0), (3, 14336, True, 0.01),
                                                     (5, 96, True, 100.0), (2, 8192, False, 1e-3)])
def test_norm_matches_oracle_bytes(ctx, rows, cols, weighted, scale):
    x, w = cases.random_rows(rows, cols, seed=rows * 1000 + cols, scale=scale)
    got = ctx.RMSNormQ8_1(x, w, rows, cols, 1e-6, weighted)
    want = oracle.RMSNormQ8_1(x, w, rows, cols, 1e-6, weighted)
    assert got == want


def test_device_entry_point_and_status(ctx, devbuf):
    rows, cols, ldx = 4, 1024, 1100
    x, w = cases.random_rows(rows, ldx, seed=9)
    xd, wd, od = devbuf(x), devbuf(w[:cols].copy()), devbuf(nbytes=rows * cols // 32 * 36)
    ctx.rmsnorm_q8_1(xd.ptr, ldx, wd.ptr, rows, cols, 1e-5, od.ptr)
    got = od.get((rows * cols // 32 * 36,), np.uint8).tobytes()
    assert got == oracle.RMSNormQ8_1(x[:, :cols], w[:cols], rows, cols, 1e-5, True)
    assert ctx.last_status() == (0, 0)
    x[2, 5] = np.inf
    xd2 = devbuf(x)
    ctx.rmsnorm_q8_1(xd2.ptr, ldx, 0, rows, cols, 1e-5, od.ptr)
    assert ctx.last_status() == (-12, 4)      # QM_ERR_DOMAIN; the word is cleared by the read
    assert ctx.last_status() == (0, 0)


def test_swiglu_blocks(ctx, devbuf):
    rng = np.random.default_rng(21)
    for width, slots in [(14336, 2), (80, 3), (2048, 6)]:
        n = width * slots
        gate = (rng.standard_normal(n) * 4).astype(np.float32)
        up = (rng.standard_normal(n) * 4).astype(np.float32)
        gate[1], up[2], up[3] = 60.0, 50.0, -50.0
        wts = rng.uniform(0.1, 1.0, slots).astype(np.float32)
        nblk = (n + 31) // 32
        od = devbuf(np.zeros(nblk * 36, dtype=np.uint8))
        ctx.swiglu_q8_1(devbuf(gate).ptr, devbuf(up).ptr, devbuf(wts).ptr, width, slots, od.ptr)
        got = od.get((nblk, 36), np.uint8)
        want = np.frombuffer(oracle.SwiGLUQ8_1(gate, up, wts, width, slots), dtype=np.uint8).reshape(nblk, 36)
        # expf on the device and in the C library may differ in the last place: d and the sum field within one
        # binary16 step, quants within one, and nearly all of them equal
        gd, wd_ = got[:, :2].copy().view(np.uint16).astype(np.int32), want[:, :2].copy().view(np.uint16).astype(np.int32)
        assert np.abs(gd - wd_).max() <= 1
        gs = got[:, 2:4].copy().view(np.float16).astype(np.float32)
        ws = want[:, 2:4].copy().view(np.float16).astype(np.float32)
        assert np.allclose(gs, ws, rtol=2e-3, atol=2e-3)
        gq, wq = got[:, 4:].view(np.int8).astype(np.int32), want[:, 4:].view(np.int8).astype(np.int32)
        assert np.abs(gq - wq).max() <= 1 and (gq != wq).mean() < 2e-3
        if n % 32:
            assert np.all(got[-1, 4 + n % 32:] == 0)


@pytest.mark.parametrize("fmt,rows,cols", [(8, 96, 1024), (2, 80, 512), (12, 64, 1024), (10, 40, 768), (16, 40, 768)])
@pytest.mark.parametrize("m", [1, 3])
def test_matvec_takes_q8_1(ctx, devbuf, fmt, rows, cols, m):
    raw = synth.weights(fmt, rows, cols, seed=fmt + m)
    w = ctx.store_upload(fmt, rows, cols, raw)
    x, g = cases.random_rows(m, cols, seed=77 + fmt)
    xq = oracle.RMSNormQ8_1(x, g, m, cols, 1e-6, True)
    xqd, yd = devbuf(np.frombuffer(xq, dtype=np.uint8)), devbuf(nbytes=m * rows * 4)
    ctx.matvec_q8_1(w, xqd.ptr, m, cols // 32, yd.ptr, rows)
    got = yd.get((m, rows))
    xf = oracle.DequantizeQ8_1(xq, m * cols).reshape(m, cols)
    want = oracle.MatVec(fmt, raw, rows, cols, xf)
    # normwise, as for float32 activations: 2e-5, or 3e-4 where three and more rows are quantized into two limbs
    tol = 3e-4 if (fmt in (2, 8, 12) and m > 2) else 2e-5
    assert np.linalg.norm(got.astype(np.float64) - want) <= tol * np.linalg.norm(want)
    # and the decoded vector itself, bit for bit
    fd = devbuf(nbytes=m * cols * 4)
    ctx.q8_1_dequantize(xqd.ptr, m, cols // 32, cols, fd.ptr, cols)
    assert np.array_equal(fd.get((m, cols)).view(np.uint32), xf.view(np.uint32))
    w.free()


@pytest.mark.parametrize("fmt", [10, 16])
@pytest.mark.parametrize("q81", [True, False])
def test_matvec_over_selected_experts(ctx, devbuf, fmt, q81):
    experts, rows, cols = 6, 72, 1024
    raw = synth.weights(fmt, experts * rows, cols, seed=5 + fmt)
    w = ctx.store_upload(fmt, experts * rows, cols, raw)
    ids = np.array([4, 0, -1, 5, 9], dtype=np.int32)     # -1 and 9: no such expert
    x, _ = cases.random_rows(1, cols, seed=31)
    xq = oracle.RMSNormQ8_1(x, None, 1, cols, 1e-6, False)
    xf = oracle.DequantizeQ8_1(xq, cols)
    yd = devbuf(nbytes=len(ids) * rows * 4)
    xd = devbuf(np.frombuffer(xq, dtype=np.uint8)) if q81 else devbuf(xf)
    ctx.matvec_selected(w, experts, devbuf(ids).ptr, len(ids), xd.ptr, 0, yd.ptr, _capi.FLAG_X_Q8_1 if q81 else 0)
    got = yd.get((len(ids), rows))
    want = oracle.SelectedMatVecQ8_1(fmt, raw, experts, rows, cols, [4, 0, -1, 5, -1], xq)
    ok = [0, 1, 3]
    assert np.abs(got[ok] - want[ok]).max() <= 2e-5 * np.abs(want[ok]).max()
    assert np.all(got[[2, 4]].view(np.uint32) == 0x7fffffff)
    # one activation vector per slot
    xs, _ = cases.random_rows(len(ids), cols, seed=32)
    xsq = oracle.RMSNormQ8_1(xs, None, len(ids), cols, 1e-6, False)
    xsf = oracle.DequantizeQ8_1(xsq, len(ids) * cols).reshape(len(ids), cols)
    xd = devbuf(np.frombuffer(xsq, dtype=np.uint8)) if q81 else devbuf(xsf)
    ctx.matvec_selected(w, experts, devbuf(ids).ptr, len(ids), xd.ptr, cols // 32 if q81 else cols, yd.ptr,
                        _capi.FLAG_X_Q8_1 if q81 else 0)
    got = yd.get((len(ids), rows))
    rb = len(raw) // (experts * rows)
    for s in ok:
        e = int(ids[s])
        want_s = oracle.MatVec(fmt, raw[e * rows * rb:(e + 1) * rows * rb], rows, cols, xsf[s])
        assert np.abs(got[s] - want_s).max() <= 2e-5 * np.abs(want_s).max()
    w.free()


def test_selected_refusals(ctx, devbuf):
    raw = synth.weights(12, 32, 256, seed=1)
    w = ctx.store_upload(12, 32, 256, raw)
    b = devbuf(nbytes=4096)
    with pytest.raises(lib_b200.QmError) as e:
        ctx.matvec_selected(w, 2, b.ptr, 1, b.ptr, 0, b.ptr)
    assert e.value.code == -3     # Q4_K experts go through the decode-step kernels, not this entry point
    w.free()
    raw = synth.weights(10, 30, 256, seed=1)
    w = ctx.store_upload(10, 30, 256, raw)
    with pytest.raises(lib_b200.QmError) as e:
        ctx.matvec_selected(w, 4, b.ptr, 1, b.ptr, 0, b.ptr)   # 30 rows do not divide into 4 experts
    assert e.value.code == -4
    w.free()
