"""Times one op of libedb200.so in isolation with CUDA events (for tuning and for
small profiler captures).

  python edge-dit.cpp_b200/microbench.py gemm --m 4608 --n 3072 --k 3072 [--wtype q8_0|q4_k] [--epilogue plain|gelu|gate]
  python edge-dit.cpp_b200/microbench.py attention --hn 24 --l 4608 --d 128 [--sage]
  python edge-dit.cpp_b200/microbench.py gemv --n 18432 --k 3072
  python edge-dit.cpp_b200/microbench.py layernorm --rows 4608 --h 3072
  python edge-dit.cpp_b200/microbench.py qkpack --tokens 4608 --heads 24 --d 128
  python edge-dit.cpp_b200/microbench.py sagequant --hn 24 --l 4608 --d 128 [--exact-means]

Prints one JSON line: median time per launch, achieved TFLOP/s or GB/s of the
algorithmic work.  Between timed launches a buffer larger than L2 is rewritten.
"""
from __future__ import annotations

import argparse
import ctypes as C
import importlib.util
import json
import math
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(name):
    key = "edb200_pkg_" + name
    if key in sys.modules:
        return sys.modules[key]
    spec = importlib.util.spec_from_file_location(key, os.path.join(HERE, name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[key] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    import torch

    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "attention", "gemv", "layernorm", "qkpack", "sagequant"])
    ap.add_argument("--m", type=int, default=4608)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=3072)
    ap.add_argument("--wtype", default="q8_0", choices=["q8_0", "q4_k"])
    ap.add_argument("--epilogue", default="plain", choices=["plain", "gelu", "gate"])
    ap.add_argument("--hn", type=int, default=24)
    ap.add_argument("--l", type=int, default=4608)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--sage", action="store_true")
    ap.add_argument("--no-smooth-q", action="store_true", help="Sage attention without the smooth-Q bias")
    ap.add_argument("--exact-means", action="store_true")
    ap.add_argument("--rows", type=int, default=4608)
    ap.add_argument("--h", type=int, default=3072)
    ap.add_argument("--tokens", type=int, default=4608)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args()

    _load("build").build()
    edb = _load("edb200")
    lib = edb.lib()
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    st = edb.current_stream()
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flops = bytes_ = 0.0

    if a.op in ("gemm", "gemv"):
        t = edb.TYPE_Q8_0 if a.wtype == "q8_0" else edb.TYPE_Q4_K
        raw_bytes = a.k // 32 * 34 if a.wtype == "q8_0" else a.k // 256 * 144
        wf = torch.randn(a.n, a.k, device=dev) * 0.02
        raw = torch.empty(a.n, raw_bytes, dtype=torch.uint8, device=dev)
        if a.wtype == "q8_0":
            edb.check(lib.edb200_quantize_rows_q8_0(edb.ptr(wf), edb.ptr(raw), a.n, a.k, st))
        else:
            raw.random_(0, 256)
            v = raw.view(a.n, a.k // 256, 144)
            v[:, :, 0:4] = torch.tensor([0x66, 0x1E, 0x66, 0x1E], dtype=torch.uint8, device=dev)  # d = dmin ~ 6e-3
        w = edb.QWeight(t, raw, a.n, a.k)
        wbytes = lib.edb200_qweight_bytes(w.handle)

    if a.op == "gemm":
        x = torch.randn(a.m, a.k, device=dev).half()
        bias = torch.randn(a.n, device=dev)
        if a.epilogue == "gate":
            res = torch.randn(a.m, a.n, device=dev)
            gate = torch.randn(a.n, device=dev)
            ep = edb.make_epilogue(res, bias=bias, residual=res, gate=gate)
        elif a.epilogue == "gelu":
            y = torch.empty(a.m, a.n, dtype=torch.float16, device=dev)
            ep = edb.make_epilogue(y, bias=bias, act=edb.ACT_GELU_TANH)
        else:
            y = torch.empty(a.m, a.n, dtype=torch.float16, device=dev)
            ep = edb.make_epilogue(y, bias=bias)
        flops = 2.0 * a.m * a.n * a.k
        bytes_ = wbytes + 2.0 * a.m * a.k + 2.0 * a.m * a.n

        def run():
            edb.mul_mat_q(w, x, ep)
    elif a.op == "gemv":
        x = torch.randn(1, a.k, device=dev)
        y = torch.empty(1, a.n, device=dev)
        bytes_ = float(wbytes)

        def run():
            edb.check(lib.edb200_gemv_q(w.handle, edb.ptr(x), 1, a.k, 1, None, edb.ptr(y), a.n, st))
    elif a.op == "attention":
        q, k, v = (torch.randn(a.hn, a.l, a.d, device=dev).half() for _ in range(3))
        out = torch.empty(a.l, a.hn * a.d, dtype=torch.float16, device=dev)
        flops = 4.0 * a.l * a.l * a.d * a.hn
        scale = 1.0 / math.sqrt(a.d)
        if a.sage:
            n = lib.edb200_sage_scratch_bytes(a.hn, a.l, a.d)
            scratch = torch.empty(n, dtype=torch.uint8, device=dev)
            offs, strides = (C.c_int64 * 8)(), (C.c_int * 3)()
            edb.check(lib.edb200_sage_scratch_layout(a.hn, a.l, a.d, offs, strides))
            edb.check(lib.edb200_sage_quantize_qk(edb.ptr(q), edb.ptr(k), a.hn, a.l, a.d, 2 if a.no_smooth_q else 3,
                                                  edb.ptr(scratch), n, st))
            base = scratch.data_ptr()
            bias = 0 if a.no_smooth_q else base + offs[6]

            def run():
                edb.check(lib.edb200_attention_sage_int8(base + offs[0], base + offs[1], edb.ptr(v), base + offs[2],
                                                         strides[0], base + offs[3], strides[1], bias,
                                                         strides[2], a.hn, a.l, a.d, scale, edb.ptr(out),
                                                         edb.TYPE_F16, out.stride(0), st))
        else:
            def run():
                edb.check(lib.edb200_attention_f16(edb.ptr(q), edb.ptr(k), edb.ptr(v), a.hn, a.l, a.l, a.d, scale,
                                                   edb.ptr(out), edb.TYPE_F16, out.stride(0), st))
    elif a.op == "layernorm":
        x = torch.randn(a.rows, a.h, device=dev)
        sh, sc = torch.randn(a.h, device=dev), torch.randn(a.h, device=dev)
        y = torch.empty(a.rows, a.h, dtype=torch.float16, device=dev)
        bytes_ = a.rows * a.h * 6.0

        def run():
            edb.check(lib.edb200_layernorm_modulate(edb.ptr(x), a.h, edb.ptr(sh), edb.ptr(sc), None, None, a.rows,
                                                    a.h, 1e-6, edb.ptr(y), edb.TYPE_F16, a.h, st))
    elif a.op == "qkpack":
        hid = a.heads * a.d
        qkv = torch.randn(a.tokens, 3 * hid, device=dev).half()
        qw, kw = torch.ones(a.d, device=dev), torch.ones(a.d, device=dev)
        pe = torch.randn(a.tokens, a.d // 2, 2, 2, device=dev)
        outs = [torch.empty(a.heads, a.tokens, a.d, dtype=torch.float16, device=dev) for _ in range(3)]
        bytes_ = a.tokens * 3.0 * hid * 4.0

        def run():
            edb.check(lib.edb200_qk_norm_rope_pack(edb.ptr(qkv), edb.TYPE_F16, 3 * hid, 0, hid, 2 * hid, a.tokens,
                                                   a.heads, a.d, edb.ptr(qw), edb.ptr(kw), 1e-6, edb.ptr(pe), 0,
                                                   a.tokens, edb.ptr(outs[0]), edb.ptr(outs[1]), edb.ptr(outs[2]),
                                                   edb.TYPE_F16, st))
    else:  # sagequant
        q, k = (torch.randn(a.hn, a.l, a.d, device=dev).half() for _ in range(2))
        n = lib.edb200_sage_scratch_bytes(a.hn, a.l, a.d)
        scratch = torch.empty(n, dtype=torch.uint8, device=dev)
        flags = 1 if a.exact_means else 3
        bytes_ = a.hn * a.l * a.d * 13.0

        def run():
            edb.check(lib.edb200_sage_quantize_qk(edb.ptr(q), edb.ptr(k), a.hn, a.l, a.d, flags, edb.ptr(scratch), n,
                                                  st))

    for _ in range(a.warmup):
        run()
    torch.cuda.synchronize()
    times = []
    for _ in range(a.iters):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    med = times[len(times) // 2]
    line = {"op": a.op, "args": {k: v for k, v in vars(a).items() if k != "op"}, "ms_median": med, "ms_min": times[0]}
    if flops:
        line["tflops"] = flops / (med * 1e-3) / 1e12
    if bytes_:
        line["gbs"] = bytes_ / (med * 1e-3) / 1e9
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
