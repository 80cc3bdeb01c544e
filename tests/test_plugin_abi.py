"""The reference's operator plugin ABI (ed_cuda_<op>_custom_supported / _compute on ggml_tensor nodes,
src/core/backend/ggml/cuda/ed_cuda_*.h) as exported by this library: the same custom-op nodes are run
by the reference's own CPU callbacks (golden vectors tests/golden/plugin_cases.npz, made from the
reference tree by tests/golden/make_plugin_golden.py; and the compiled callbacks themselves where
oracle/_ref has been built) and by the library's entry points on the GPU.  Bit-exact.

The CPU-side tests also pin more of the numpy oracle to the reference's code: GELU-tanh, the f32
linear with and without the gated residual, the attention layout glue and the where-select."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import plugin_cases as P  # noqa: E402

from oracle import edb_oracle as O  # noqa: E402

GOLD = np.load(os.path.join(HERE, "golden", "plugin_cases.npz"))
REF_LIB = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libedref_cpu.so")


def _bits(a):
    a = np.ascontiguousarray(a)
    return a.view({4: np.uint32, 2: np.uint16, 1: np.uint8}[a.dtype.itemsize])


def _lib_sigs(edb):
    lib = edb.lib()
    lib.edb200_plugin_supported.argtypes = [C.c_int, C.POINTER(P.GgmlTensor)]
    lib.edb200_plugin_supported.restype = C.c_int
    lib.edb200_plugin_compute.argtypes = [C.c_int, C.POINTER(P.GgmlTensor), C.c_void_p, C.c_void_p]
    lib.edb200_plugin_compute.restype = C.c_int
    lib.edb200_plugin_sage_scratch_sizes.argtypes = [C.POINTER(P.GgmlTensor), C.POINTER(C.c_size_t)]
    lib.edb200_plugin_sage_scratch_sizes.restype = C.c_int
    lib.edb200_plugin_tensor_layout.argtypes = [C.POINTER(C.c_size_t)]
    lib.edb200_plugin_tensor_layout.restype = None
    return lib


def test_golden_vectors_cover_every_case():
    assert set(GOLD.files) == set(P.cases())


def test_compiled_reference_callbacks_reproduce_the_golden_vectors():
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libedref_cpu.so not built (needs the reference tree)")
    lib = C.CDLL(REF_LIB)
    for name, node in P.cases().items():
        assert np.array_equal(_bits(P.run_reference(lib, node)), _bits(GOLD[name])), name
    # and on other seeds the callbacks and the numpy restatements below still agree
    for seed in (1, 2):
        for name, node in P.cases(seed).items():
            want = _numpy_restatement(name, node)
            if want is not None:
                assert np.array_equal(_bits(P.run_reference(lib, node)), _bits(want)), (seed, name)


def _numpy_restatement(name, node):
    """The operators that are pure f32 arithmetic without a reduction, or copies: restated in numpy to the bit."""
    f = np.float32
    a = [s[0] for s in node.srcs]
    if node.kind == "modulate":
        return O.modulate(a[0], a[1], a[2])
    if node.kind == "residual_gate":
        return O.residual_gate(a[0], a[1], a[2])
    if node.kind == "where_select":
        return (a[1] + (a[0] * (a[2] - a[1]).astype(f)).astype(f)).astype(f)
    if node.kind == "v_prep":
        v = a[0]                                              # [batch, seq|heads, heads|seq, d]
        seq_major = name.endswith("seq_major")
        x = v if seq_major else v.transpose(0, 2, 1, 3)       # -> [batch, heads, seq, d]
        b, h, s, d = x.shape
        return x.reshape(1, b * h, s, d).astype(np.float16)
    if node.kind == "pair_pack":
        n_head = 4
        rows = np.concatenate([a[0], a[1]], axis=2)           # [1, batch, seq0 + seq1, heads * d]
        _, b, s, hd = rows.shape
        return rows.reshape(b, s, n_head, hd // n_head).transpose(0, 2, 1, 3).astype(np.float16)
    if node.kind == "qkv_pair_pack":
        n_head = 4
        planes = []
        for p in range(3):
            rows = np.concatenate([a[p], a[3 + p]], axis=2)[0, 0]     # [seq, heads * d]
            planes.append(rows.reshape(rows.shape[0], n_head, -1).transpose(1, 0, 2))
        return np.stack(planes).astype(np.float16)
    return None


def test_numpy_restatements_match_the_reference_callbacks():
    for name, node in P.cases().items():
        want = _numpy_restatement(name, node)
        if want is not None:
            assert np.array_equal(_bits(want), _bits(GOLD[name])), name


def test_oracle_gelu_and_linear_against_the_reference_callbacks():
    c = P.cases()
    # GELU-tanh: the reference rounds its f32 result to bf16; the oracle's f32 value must round to the same
    # bf16 or its neighbour (tanhf and numpy's tanh may differ in the last f32 bit)
    g = O.gelu_tanh(c["gelu_bf16"].srcs[0][0])
    got = P._bf16(g)
    want = (GOLD["gelu_bf16"].astype(np.uint32) << 16).view(np.float32)
    have = (got.astype(np.uint32) << 16).view(np.float32)
    # one bf16 step, or an absolute 1e-6 where 1 + tanh cancels (large negative inputs, outputs near zero)
    assert np.all(np.abs(have - want) <= np.abs(want) * 2.0 ** -7 + 1e-6)
    assert (got == GOLD["gelu_bf16"]).mean() > 0.9
    # f32 linear over the concatenation of two inputs (sequential f32 sum in the reference, blocked in numpy)
    x0, x1, w, b = (s[0] for s in c["concat_linear"].srcs)
    x = np.concatenate([x0[0, 0], x1[0, 0]], axis=1)
    y = O.linear(x, w[0, 0], b.reshape(-1))
    assert np.allclose(y, GOLD["concat_linear"][0, 0], rtol=2e-6, atol=2e-6)
    r, _, _, _, _, gate = (s[0] for s in c["concat_linear_residual_gate"].srcs)
    z = O.residual_gate(r[0, 0], y, gate.reshape(1, -1))
    assert np.allclose(z, GOLD["concat_linear_residual_gate"][0, 0], rtol=2e-6, atol=2e-6)
    # rms_norm_mul_f16 and the interleaved rope of the oracle are pinned by tests/test_oracle_ref.py; here the
    # other layouts of the callback are at least consistent with it
    nx, nw = (s[0] for s in c["rms_norm_mul_f16"].srcs)
    assert np.array_equal(_bits(O.rms_norm_mul_f16_callback(nx.reshape(-1, 128), nw.reshape(-1), 1e-6)),
                          _bits(GOLD["rms_norm_mul_f16"].reshape(-1, 128)))


def test_tensor_structure_matches_the_library(edb):
    lib = _lib_sigs(edb)
    words = (C.c_size_t * 8)()
    lib.edb200_plugin_tensor_layout(words)
    assert list(words) == P.layout_words()


def test_supported_decisions(edb):
    """supported() only inspects the node: no device needed.  Every case is accepted by its own entry
    point and by no other; a node that is not a custom op, carries another magic, or has the wrong
    output type is refused."""
    lib = _lib_sigs(edb)
    for name, node in P.cases().items():
        dst, out, keep = node.build(lambda a: a.ctypes.data)
        mine = P.PLUGIN_OF.get(node.kind)
        for which in range(7):
            ok = lib.edb200_plugin_supported(which, C.byref(dst))
            assert ok == (1 if which == mine else 0), (name, which)
        if mine is None:
            continue
        dst.op = 0
        assert lib.edb200_plugin_supported(mine, C.byref(dst)) == 0, name
        dst.op = P.OP_CUSTOM
        saved = dst.type
        dst.type = P.TYPE_F32 if saved != P.TYPE_F32 else P.TYPE_F16
        if node.kind != "rope":                                   # rope has three legal output types
            assert lib.edb200_plugin_supported(mine, C.byref(dst)) == 0, name
        dst.type = saved
        words = (C.c_uint64 * 3)(0, 0, node.ud ^ 0x1)             # a different magic
        C.memmove(dst.op_params, words, 24)
        assert lib.edb200_plugin_supported(mine, C.byref(dst)) == 0, name
    assert lib.edb200_plugin_supported(0, None) == 0


# ----------------------------------------------------------------------------- GPU

torch = pytest.importorskip("torch")


def _device_ptr_factory(cuda, hold):
    """ptr_of for Node.build: uploads the array's whole underlying buffer and returns the device address of
    the array's first element (so strided views stay strided)."""
    def ptr_of(arr):
        base = arr
        while base.base is not None and isinstance(base.base, np.ndarray):
            base = base.base
        flat = np.ascontiguousarray(base).view(np.uint8).reshape(-1)
        t = torch.from_numpy(flat.copy()).to(cuda)
        hold.append(t)
        return t.data_ptr() + (arr.ctypes.data - base.ctypes.data)
    return ptr_of


@pytest.mark.gpu
def test_plugin_compute_matches_the_reference_callbacks(edb, cuda):
    lib = _lib_sigs(edb)
    n0 = lib.edb200_launch_count()
    for name, node in P.cases().items():
        which = P.PLUGIN_OF.get(node.kind)
        if which is None:
            continue
        hold = []
        dst, out, keep = node.build(_device_ptr_factory(cuda, hold))
        assert lib.edb200_plugin_supported(which, C.byref(dst)) == 1, name
        assert lib.edb200_plugin_compute(which, C.byref(dst), None, edb.current_stream()) == 1, name
        torch.cuda.synchronize()
        got = hold[0].cpu().numpy().view(out.dtype).reshape(out.shape)     # the output was uploaded first
        assert np.array_equal(_bits(got), _bits(GOLD[name])), name
    assert lib.edb200_launch_count() > n0


@pytest.mark.gpu
@pytest.mark.parametrize("d,n_head,l,v_packed", [(128, 3, 300, False), (64, 4, 200, False), (128, 2, 128, True)])
def test_sage_plugin_entry_point(edb, cuda, d, n_head, l, v_packed):
    """The INT8-QK attention through the reference's plugin interface (sizes query, caller-allocated scratch
    buffers, f32 output [d, heads, L]) gives the bits of this library's own entry point with the
    reference's summation orders, and stays close to the fp32 attention."""
    import math
    lib = _lib_sigs(edb)
    rng = np.random.default_rng(9)
    q = O.f16_round(rng.standard_normal((n_head, l, d), dtype=np.float32))
    k = O.f16_round(rng.standard_normal((n_head, l, d), dtype=np.float32) + np.float32(0.5))
    v = rng.standard_normal((n_head, l, d), dtype=np.float32)
    hold = []
    ptr_of = _device_ptr_factory(cuda, hold)
    q16, k16 = q.astype(np.float16)[None], k.astype(np.float16)[None]            # ggml [d, L, heads, 1]
    v_arr = np.ascontiguousarray(v)[None] if v_packed else np.ascontiguousarray(v.transpose(1, 0, 2))[None]
    node = P.Node("sage", [(q16, P.TYPE_F16), (k16, P.TYPE_F16), (v_arr, P.TYPE_F32)], P.TYPE_F32, (d, n_head, l, 1),
                  P.userdata("sage", n_head))
    dst, out, keep = node.build(ptr_of)
    assert lib.edb200_plugin_supported(6, C.byref(dst)) == 1
    sizes = (C.c_size_t * 14)()
    assert lib.edb200_plugin_sage_scratch_sizes(C.byref(dst), sizes) == 1
    bufs = [torch.zeros(max(int(s), 16), dtype=torch.uint8, device=cuda) for s in sizes]
    scratch = (C.c_void_p * 14)(*[b.data_ptr() if int(s) > 0 else None for b, s in zip(bufs, sizes)])
    assert lib.edb200_plugin_compute(6, C.byref(dst), scratch, edb.current_stream()) == 1
    torch.cuda.synchronize()
    got = hold[0].cpu().numpy().view(np.float32).reshape(l, n_head * d)
    # the library's own entry point on the same operands (reference orders: no EDB200_SAGE_FAST_MEANS)
    tq, tk = torch.from_numpy(q16[0]).to(cuda), torch.from_numpy(k16[0]).to(cuda)
    tv = torch.from_numpy(v.astype(np.float16)).to(cuda)
    n = lib.edb200_sage_scratch_bytes(n_head, l, d)
    sc = torch.zeros(n, dtype=torch.uint8, device=cuda)
    own = torch.zeros(l, n_head * d, dtype=torch.float32, device=cuda)
    edb.check(lib.edb200_sage_attention(edb.ptr(tq), edb.ptr(tk), edb.ptr(tv), n_head, l, d, 1.0 / math.sqrt(d),
                                        1 if d == 128 else 0, edb.ptr(sc), n, edb.ptr(own), edb.TYPE_F32, n_head * d,
                                        edb.current_stream()))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(got), _bits(own.cpu().numpy()))
    exact = O.attention(q.transpose(1, 0, 2), k.transpose(1, 0, 2), O.f16_round(v).transpose(1, 0, 2))
    assert O.cosine(got, exact) > 0.999 and O.rel_l2(got, exact) < 3e-2
    # f32 q is left to the caller's fallback
    node32 = P.Node("sage", [(q[None], P.TYPE_F32), (k16, P.TYPE_F16), (v_arr, P.TYPE_F32)], P.TYPE_F32, (d, n_head, l, 1),
                    P.userdata("sage", n_head))
    dst32, _, keep32 = node32.build(lambda a: a.ctypes.data)
    assert lib.edb200_plugin_supported(6, C.byref(dst32)) == 0
