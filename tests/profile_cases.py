"""Single-kernel driver for profiling: runs one kernel family on one shape a few
times so that a profiler can capture it on a small, bounded case.

    python tests/profile_cases.py gemv --m 1 --n 14336 --k 4096 --variant 1,4,4,4,0,0 --copies 3
    python tests/profile_cases.py gemm --m 2048 --n 14336 --k 4096 --variant 2,0,128,128,4,8 --epilogue gelu
    python tests/profile_cases.py dense --m 2048 --n 14336 --k 4096 --dtype bf16 --epilogue gelu   (tl_matmul, NT)
    python tests/profile_cases.py int4 --m 1 --n 14336 --k 4096 --group 128

Each launch uses its own weight copy (copies x N x K bytes; keep it to a few hundred
MB) so that every launch streams from HBM rather than L2.  Prints "ok" and exits 0.
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from torchlette_b200 import backend as tb  # noqa: E402
from torchlette_b200 import binding as B  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("family", choices=["gemv", "gemm", "dense", "int4"])
    ap.add_argument("--group", type=int, default=128, help="int4: group size")
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=14336)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--variant", default="", help="family,kernel,p0,p1,p2,p3 (empty = the library's own choice)")
    ap.add_argument("--copies", type=int, default=3)
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16"])
    ap.add_argument("--epilogue", default="", help="unary op fused into the store (relu, gelu, silu)")
    a = ap.parse_args()
    be = tb.CudaBackend(0)
    lib, ctx = be._lib, be._ctx
    dev = torch.device("cuda", 0)
    tdt, tid = (torch.float16, B.TL_F16) if a.dtype == "f16" else (torch.bfloat16, B.TL_BF16)
    e = None
    if a.epilogue:
        e = B.Epilogue()
        e.n_ops = 1
        e.ops[0] = B.EpilogueOp(B.TL_EPI_UNARY, B.TL_UNARY[a.epilogue], 0, 0)
    ep = C.byref(e) if e is not None else None
    if a.variant:
        be.forceVariant(tuple(int(v) for v in a.variant.split(",")))
    if a.family == "dense":
        wd = (torch.randn(a.copies, a.n, a.k, device=dev) * 0.05).to(tdt)
        x = torch.randn(a.m, a.k, device=dev).to(tdt)
        y = torch.empty(a.m, a.n, dtype=tdt, device=dev)
        torch.cuda.synchronize(dev)
        for c in range(a.copies):
            B.check(ctx, lib.tl_matmul(ctx, x.data_ptr(), wd[c].data_ptr(), y.data_ptr(), a.m, a.n, a.k, 1, 0, 0, a.m * a.n, 0, 1,
                                       1.0, tid, tid, tid, -1, -1, ep, None))
        be.sync()
        print("ok")
        return
    if a.family == "int4":
        w4 = torch.randint(-2 ** 31, 2 ** 31 - 1, (a.copies, a.n, a.k // 8), dtype=torch.int32, device=dev)
        s4 = torch.empty(a.n, a.k // a.group, device=dev).uniform_(0.01, 0.1).to(torch.float16)
        x = torch.randn(a.m, a.k, device=dev).to(tdt)
        y = torch.empty(a.m, a.n, dtype=tdt, device=dev)
        q4 = B.QuantDesc(B.TL_SCHEME_INT4_GROUPED, a.group, B.TL_F16, B.TL_SCALE_SNORM127)
        torch.cuda.synchronize(dev)
        for c in range(a.copies):
            B.check(ctx, lib.tl_qmatmul_nt(ctx, x.data_ptr(), tid, w4[c].data_ptr(), s4.data_ptr(), y.data_ptr(), tid, a.m, a.n, a.k,
                                           C.byref(q4), 1.0, ep))
        be.sync()
        print("ok")
        return
    w = torch.randint(-127, 128, (a.copies, a.n, a.k), dtype=torch.int8, device=dev)
    s = torch.empty(a.n, dtype=torch.float32, device=dev).uniform_(0.001, 0.01)
    x = torch.randn(a.m, a.k, device=dev).to(tdt)
    y = torch.empty(a.m, a.n, dtype=tdt, device=dev)
    q = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, a.k, B.TL_F32, B.TL_SCALE_DIRECT)
    torch.cuda.synchronize(dev)
    fn = lib.tl_qgemv_nt if a.family == "gemv" else lib.tl_qgemm_nt
    for c in range(a.copies):
        B.check(ctx, fn(ctx, x.data_ptr(), tid, w[c].data_ptr(), s.data_ptr(), y.data_ptr(), tid, a.m, a.n, a.k,
                        C.byref(q), 1.0, C.byref(e) if e is not None else None))
    be.sync()
    print("ok")


if __name__ == "__main__":
    main()
