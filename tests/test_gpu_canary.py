"""Out-of-bounds writes, looked for without a sanitizer: every output of a ragged-shaped call sits
inside a larger allocation filled with a canary pattern, and the bytes in front of and behind the
output must come back untouched.  Plus the two environment knobs read at context creation."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import cases
from oracle import oracle as orc
from torchlette_b200 import backend as tb
from torchlette_b200 import binding as B

pytestmark = pytest.mark.gpu

PAD = 4096  # canary bytes on either side
CANARY = 0x5A


class Guarded:
    """An output tensor of `nbytes` inside a canary-filled torch allocation."""

    def __init__(self, be, shape, dtype):
        self.itemsize = {"f32": 4, "f16": 2, "bf16": 2, "i8": 1}[dtype]
        self.nbytes = int(np.prod(shape)) * self.itemsize
        self.raw = torch.full((PAD + self.nbytes + PAD,), CANARY, dtype=torch.uint8, device=torch.device("cuda", be.device))
        assert self.raw.data_ptr() % 256 == 0
        self.t = tb.CudaTensor(be, list(shape), dtype, self.raw.data_ptr() + PAD, self.nbytes, ownsBuffer=False)

    def check(self):
        torch.cuda.synchronize()
        host = self.raw.cpu().numpy()
        assert (host[:PAD] == CANARY).all(), "bytes in front of the output were written"
        assert (host[PAD + self.nbytes:] == CANARY).all(), "bytes behind the output were written"
        return host[PAD:PAD + self.nbytes]


RAGGED = [(1, 37, 64), (3, 130, 192), (16, 1000, 128), (9, 17, 256), (5, 16, 64)]


@pytest.mark.parametrize("variant", [None] + [(1, 2, 8, 4, 1, 0), (1, 3, 4, 4, 0, 0), (1, 4, 4, 4, 0, 0), (1, 4, 8, 2, 2, 0), (1, 5, 6, 0, 0, 0),
                                              (1, 6, 16, 32, 0, 0), (1, 8, 8, 3, 2, 32), (1, 1, 8, 2, 1, 0), (1, 0, 8, 0, 1, 0)])
@pytest.mark.parametrize("m,n,k", RAGGED)
def test_small_batch_kernels_write_only_their_output(backend, variant, m, n, k):
    be = backend
    cs = cases.per_channel_case(n, k, m, seed=n + k + m, act_dtype="f16", bias=True)
    w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
    x = be.ops.tensorFromArray(cs["x_bits"], [m, k], "f16")
    bias = be.ops.tensorFromArray(cs["bias"], [n], "f32")
    out = Guarded(be, [m, n], "f16")
    plan = tb.detectMatmulEpilogue([("add", bias), ("relu", None), ("cast", "f16")])
    be.forceVariant(variant)
    try:
        try:
            be.ops.matmul(x, be.ops.transpose(w), {"epilogue": plan[0], "epilogueInputs": plan[1], "outBuffer": out.t})
        except tb.TlError as ex:
            if ex.status == B.TL_ERR_UNSUPPORTED:
                pytest.skip(str(ex))
            raise
    finally:
        be.forceVariant(None)
    got = out.check().view(np.float16).reshape(m, n).astype(np.float32)
    ref = orc.linear_reference(cs["x"], orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k), cs["bias"], "relu")
    assert cases.rel_err(got, ref) <= 1e-2
    for t in (x, bias, w.scales, w):
        t.destroy()


@pytest.mark.parametrize("m,n,k", [(40, 130, 128), (200, 129, 256), (129, 1000, 64), (33, 72, 192)])
def test_tensor_core_kernels_write_only_their_output(backend, m, n, k):
    be = backend
    # quantized GEMM (tcgen05, weights from TMEM)
    cs = cases.per_channel_case(n, k, m, seed=n * 3 + m, act_dtype="bf16")
    w = be.createQuantizedWeight(cs["packed"], cs["scales"], n, k, tb.perChannelFormat(k))
    x = be.ops.tensorFromArray(cs["x_bits"], [m, k], "bf16")
    out = Guarded(be, [m, n], "bf16")
    be.ops.matmul(x, be.ops.transpose(w), {"outputDtype": "bf16", "outBuffer": out.t})
    got = orc.bf16_bits_to_f32(out.check().view(np.uint16)).reshape(m, n)
    assert cases.rel_err(got, orc.linear_reference(cs["x"], orc.dequantize_direct_f32(cs["packed"], cs["scales"], k, k))) <= 1e-2
    # dense GEMM (tcgen05, both operands from shared memory): needs n >= 64, k % 8 == 0
    rng = np.random.default_rng(m)
    wd = rng.uniform(-1, 1, (n, k)).astype(np.float16)
    xd = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    wt, xt = be.ops.tensorFromArray(wd, [n, k], "f16"), be.ops.tensorFromArray(xd, [m, k], "f16")
    out2 = Guarded(be, [m, n], "f32")
    assert be.planMatmul(m, n, k, "f16", "f16", transB=True)["variant"].startswith("matmul.tc")
    be.ops.matmul(xt, be.ops.transpose(wt), {"outBuffer": out2.t})
    got2 = out2.check().view(np.float32).reshape(m, n)
    assert cases.rel_err(got2, orc.linear_reference(xd.astype(np.float32), wd.astype(np.float32))) <= 1e-3
    for t in (x, w.scales, w, wt, xt):
        t.destroy()


def test_other_ops_write_only_their_output(backend):
    be = backend
    rng = np.random.default_rng(0)
    # int4 GEMV (both forms), dequant, transposition, rmsnorm, unary with a ragged count
    n, k, g, m = 37, 256, 128, 3
    wv = (rng.uniform(-1, 1, (n, k)) * 0.1).astype(np.float32)
    packed, scales = be.quantizeLinearWeight(wv, g, scheme="int4-grouped")
    w = be.createQuantizedWeight(packed, scales, n, k, tb.StorageFormat("f16", tb.QuantPacking("int4-grouped", g, "f16")))
    xv = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    x = be.ops.tensorFromArray(xv, [m, k], "f16")
    for variant in (None, (1, 1, 8, 1, 1, 0)):
        out = Guarded(be, [m, n], "f32")
        be.forceVariant(variant)
        try:
            be.ops.matmul(x, be.ops.transpose(w), {"outBuffer": out.t})
        finally:
            be.forceVariant(None)
        ref = orc.linear_reference(xv.astype(np.float32), orc.dequantize_int4_to_f32(packed, scales, k, g))
        assert cases.rel_err(out.check().view(np.float32).reshape(m, n), ref) <= 1e-3
    src = be.ops.tensorFromArray(rng.standard_normal((45, 70)).astype(np.float32), [45, 70], "f32")
    tr = Guarded(be, [70, 45], "f32")
    B.check(be._ctx, be._lib.tl_transpose2d(be._ctx, src.buffer, tr.t.buffer, 1, 45, 70, 4))
    assert np.array_equal(tr.check().view(np.float32).reshape(70, 45), be.ops.read(src).T)
    un = Guarded(be, [45 * 70 - 0], "f16")
    B.check(be._ctx, be._lib.tl_unary_op(be._ctx, B.TL_UNARY["silu"], src.buffer, B.TL_F32, un.t.buffer, B.TL_F16, 45 * 70))
    un.check()
    wn = be.ops.tensorFromArray(np.ones(70, np.float32), [70], "f32")
    rn = Guarded(be, [45, 70], "f32")
    B.check(be._ctx, be._lib.tl_rmsnorm(be._ctx, src.buffer, B.TL_F32, wn.buffer, B.TL_F32, rn.t.buffer, B.TL_F32, 45, 70, 1e-6))
    rn.check()
    for t in (x, w.scales, w, src, wn):
        t.destroy()


def test_environment_knobs_variant_and_profile():
    """TORCHLETTE_CUDA_VARIANT forces a kernel from the first call of a fresh context; TORCHLETTE_CUDA_PROFILE=1
    prints one timing line per product call.  Run in a child process: both are read at context creation."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = r'''
import sys, numpy as np
sys.path.insert(0, %r); sys.path.insert(0, %r + "/tests")
import cases
from torchlette_b200 import backend as tb
be = tb.CudaBackend(0)
cs = cases.per_channel_case(256, 512, 4, seed=1, act_dtype="f16")
w = be.createQuantizedWeight(cs["packed"], cs["scales"], 256, 512, tb.perChannelFormat(512))
x = be.ops.tensorFromArray(cs["x_bits"], [4, 512], "f16")
print("PLAN", be.planQuantizedMatmul(4, 256, 512, "f16", "f32", w.format.packing)["variant"])
y = be.linear(x, w)
be.sync()
''' % (root, root)
    env = dict(os.environ, TORCHLETTE_CUDA_VARIANT="1,2,8,4,1,0", TORCHLETTE_CUDA_PROFILE="1")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert "PLAN qgemv.mma" in r.stdout, r.stdout
    assert "[tl profile] matmul_gemv_q8 m=4 n=256 k=512:" in r.stderr, r.stderr
