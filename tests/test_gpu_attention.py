"""GPU parity tests of the tcgen05 attention kernels and the Sage INT8 quantisers."""
import ctypes as C
import math

import numpy as np
import pytest

from oracle import edb_oracle as O

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(autouse=True, params=["1", "2"], ids=["one_tile_per_cta", "two_tiles_per_cta"])
def _schedule(request, monkeypatch):
    # the launcher picks one or two 128-query tiles per CTA from the grid size; the small
    # shapes here would only reach one of them, so every test runs under both
    monkeypatch.setenv("EDB200_ATTN_QT", request.param)


def _qkv(hn, lq, lk, d, seed, mean_shift=0.0):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((hn, lq, d), dtype=np.float32)
    k = rng.standard_normal((hn, lk, d), dtype=np.float32) + np.float32(mean_shift)
    v = rng.standard_normal((hn, lk, d), dtype=np.float32)
    return O.f16_round(q), O.f16_round(k), O.f16_round(v)


def _ref_attention(q, k, v):
    # oracle takes [L, H, d]
    return O.attention(q.transpose(1, 0, 2), k.transpose(1, 0, 2), v.transpose(1, 0, 2))


@pytest.mark.parametrize("hn,lq,lk,d", [
    (2, 128, 128, 128),     # one tile, one key block
    (3, 300, 300, 128),     # ragged tails on both sides
    (2, 1178, 1178, 64),    # SD3-medium joint length, d = 64
    (2, 640, 77, 128),      # cross attention: fewer keys than one block
    (1, 200, 1500, 128),    # many key blocks: exercises the lazy rescale and both S buffers
])
def test_attention_f16(edb, cuda, hn, lq, lk, d):
    q, k, v = _qkv(hn, lq, lk, d, seed=21)
    tq, tk, tv = (torch.from_numpy(a).to(cuda).half() for a in (q, k, v))
    out = torch.zeros(lq, hn * d + 8, dtype=torch.float32, device=cuda)
    edb.check(edb.lib().edb200_attention_f16(edb.ptr(tq), edb.ptr(tk), edb.ptr(tv), hn, lq, lk, d,
                                             1.0 / math.sqrt(d), edb.ptr(out), edb.TYPE_F32, out.stride(0),
                                             edb.current_stream()))
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    ref = _ref_attention(q, k, v)
    assert np.isfinite(got).all()
    assert not got[:, hn * d:].any()                      # padding columns untouched
    assert O.rel_l2(got[:, : hn * d], ref) < 2e-3, O.rel_l2(got[:, : hn * d], ref)
    assert O.cosine(got[:, : hn * d], ref) > 0.9999


def test_attention_f16_growing_scores(edb, cuda):
    # keys whose scores grow along the sequence force the running maximum to move late
    hn, l, d = 1, 1024, 128
    q, k, v = _qkv(hn, l, l, d, seed=22)
    k = O.f16_round(k * np.linspace(0.2, 3.0, l, dtype=np.float32)[None, :, None])
    tq, tk, tv = (torch.from_numpy(a).to(cuda).half() for a in (q, k, v))
    out = torch.zeros(l, hn * d, dtype=torch.float16, device=cuda)
    edb.check(edb.lib().edb200_attention_f16(edb.ptr(tq), edb.ptr(tk), edb.ptr(tv), hn, l, l, d, 1.0 / math.sqrt(d),
                                             edb.ptr(out), edb.TYPE_F16, out.stride(0), edb.current_stream()))
    assert O.rel_l2(out.float().cpu().numpy(), _ref_attention(q, k, v)) < 3e-3


def _scratch(edb, cuda, hn, l, d):
    n = edb.lib().edb200_sage_scratch_bytes(hn, l, d)
    offs = (C.c_int64 * 8)()
    strides = (C.c_int * 3)()
    edb.check(edb.lib().edb200_sage_scratch_layout(hn, l, d, offs, strides))
    assert offs[7] == n
    return torch.zeros(n, dtype=torch.uint8, device=cuda), list(offs), list(strides)


@pytest.mark.parametrize("fast", [0, 1], ids=["reference_order", "fast_prepass"])
@pytest.mark.parametrize("hn,l,d,smooth_q", [(2, 300, 128, 1), (3, 128, 128, 0), (2, 200, 64, 1), (1, 1178, 64, 0),
                                             (2, 517, 128, 1)])
def test_sage_quantisers_bit_exact(edb, cuda, hn, l, d, smooth_q, fast):
    """fast = 0: the reference kernels' arithmetic and summation orders.  fast = 1
    (EDB200_SAGE_FAST_MEANS, what the step executors run): chunked channel means and the fused
    quantise + bias kernel, against the numpy models of exactly those orders; the quantisation
    arithmetic itself is the reference's in both."""
    q, k, _ = _qkv(hn, l, l, d, seed=23, mean_shift=0.7)
    tq, tk = (torch.from_numpy(a).to(cuda).half() for a in (q, k))
    scratch, offs, strides = _scratch(edb, cuda, hn, l, d)
    edb.check(edb.lib().edb200_sage_quantize_qk(edb.ptr(tq), edb.ptr(tk), hn, l, d, smooth_q | (2 * fast),
                                                edb.ptr(scratch), scratch.numel(), edb.current_stream()))
    torch.cuda.synchronize()
    raw = scratch.cpu().numpy()

    def view(off, count, dt):
        return raw[off: off + count * np.dtype(dt).itemsize].view(dt)

    mean = O.sage_channel_mean_chunked if fast else O.sage_channel_mean
    km = mean(k)
    qm = mean(q) if smooth_q else None
    assert np.array_equal(view(offs[5], hn * d, np.float32).reshape(hn, d).view(np.uint32), km.view(np.uint32))
    q8, qs = O.sage_quant_q(q, qm)
    k8, ks = O.sage_quant_k(k, km)
    assert np.array_equal(view(offs[0], hn * l * d, np.int8).reshape(hn, l, d), q8)
    assert np.array_equal(view(offs[1], hn * l * d, np.int8).reshape(hn, l, d), k8)
    gqs = view(offs[2], hn * strides[0], np.float32).reshape(hn, strides[0])
    gks = view(offs[3], hn * strides[1], np.float32).reshape(hn, strides[1])
    assert np.array_equal(gqs[:, : qs.shape[1]].view(np.uint32), qs.view(np.uint32))
    assert np.array_equal(gks[:, : ks.shape[1]].view(np.uint32), ks.view(np.uint32))
    if smooth_q:
        assert np.array_equal(view(offs[4], hn * d, np.float32).reshape(hn, d).view(np.uint32), qm.view(np.uint32))
        gb = view(offs[6], hn * strides[2], np.float32).reshape(hn, strides[2])
        want = O.sage_smooth_q_bias_fused(k, qm) if fast else O.sage_smooth_q_bias(k, qm)
        assert np.array_equal(gb[:, :l].view(np.uint32), want.view(np.uint32))
        assert not gb[:, l:].any()                       # the padded tail the attention kernel reads is zero


@pytest.mark.parametrize("hn,l,smooth_q,d", [(2, 128, 0, 128), (2, 300, 1, 128), (1, 1100, 1, 128), (2, 128, 0, 64),
                                             (3, 300, 0, 64), (1, 1178, 0, 64), (2, 200, 1, 64)])
def test_sage_attention_matches_int8_model_and_fp32(edb, cuda, hn, l, smooth_q, d):
    q, k, v = _qkv(hn, l, l, d, seed=24, mean_shift=0.5)
    tq, tk, tv = (torch.from_numpy(a).to(cuda).half() for a in (q, k, v))
    scratch, _, _ = _scratch(edb, cuda, hn, l, d)
    out = torch.zeros(l, hn * d, dtype=torch.float32, device=cuda)
    edb.check(edb.lib().edb200_sage_attention(edb.ptr(tq), edb.ptr(tk), edb.ptr(tv), hn, l, d, 1.0 / math.sqrt(d),
                                              smooth_q, edb.ptr(scratch), scratch.numel(), edb.ptr(out), edb.TYPE_F32,
                                              out.stride(0), edb.current_stream()))
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    model = O.sage_attention(q, k, v, smooth_q=bool(smooth_q)).transpose(1, 0, 2).reshape(l, hn * d)
    exact = _ref_attention(q, k, v)
    assert np.isfinite(got).all()
    assert O.rel_l2(got, model) < 3e-3, O.rel_l2(got, model)       # same INT8 arithmetic, f16 P rounding differs
    assert O.cosine(got, exact) > 0.999 and O.rel_l2(got, exact) < 3e-2   # INT8 QK vs the fp32 path


@pytest.mark.parametrize("d", [64, 128])
def test_attention_on_a_padded_layout(edb, cuda, d):
    """Heads `head_rows` rows apart with only the first l rows real (a sequence padded for sequence
    parallelism): the strided entry points give the bits of the dense ones, for f16 and INT8 scores."""
    hn, l, head_rows = 3, 301, 304
    q, k, v = _qkv(hn, l, l, d, seed=26, mean_shift=0.3)
    dense = [torch.from_numpy(a).to(cuda).half() for a in (q, k, v)]
    padded = []
    for t in dense:
        p = torch.full((hn, head_rows, d), float("nan"), dtype=torch.float16, device=cuda)   # padding rows hold NaN
        p[:, :l] = t
        padded.append(p)
    scale = 1.0 / math.sqrt(d)
    a, b = (torch.zeros(l, hn * d, dtype=torch.float32, device=cuda) for _ in range(2))
    edb.check(edb.lib().edb200_attention_f16(*(edb.ptr(t) for t in dense), hn, l, l, d, scale, edb.ptr(a), edb.TYPE_F32,
                                             hn * d, edb.current_stream()))
    edb.check(edb.lib().edb200_attention_f16_strided(*(edb.ptr(t) for t in padded), hn, l, l, head_rows, head_rows, d,
                                                     scale, edb.ptr(b), edb.TYPE_F32, hn * d, None, edb.current_stream()))
    torch.cuda.synchronize()
    assert torch.isfinite(b).all() and torch.equal(a, b)
    scratch, _, _ = _scratch(edb, cuda, hn, l, d)
    for smooth in (0, 1, 3):
        edb.check(edb.lib().edb200_sage_attention(*(edb.ptr(t) for t in dense), hn, l, d, scale, smooth, edb.ptr(scratch),
                                                  scratch.numel(), edb.ptr(a), edb.TYPE_F32, hn * d, edb.current_stream()))
        edb.check(edb.lib().edb200_sage_attention_strided(*(edb.ptr(t) for t in padded), hn, l, head_rows, d, scale,
                                                          smooth, edb.ptr(scratch), scratch.numel(), edb.ptr(b),
                                                          edb.TYPE_F32, hn * d, None, edb.current_stream()))
        torch.cuda.synchronize()
        assert torch.isfinite(b).all() and torch.equal(a, b), smooth


def test_sage_rejects_small_scratch(edb, cuda):
    hn, l, d = 1, 128, 128
    q, k, v = _qkv(hn, l, l, d, seed=25)
    tq, tk, tv = (torch.from_numpy(a).to(cuda).half() for a in (q, k, v))
    scratch = torch.zeros(256, dtype=torch.uint8, device=cuda)
    out = torch.zeros(l, hn * d, dtype=torch.float32, device=cuda)
    st = edb.lib().edb200_sage_attention(edb.ptr(tq), edb.ptr(tk), edb.ptr(tv), hn, l, d, 0.1, 1, edb.ptr(scratch),
                                         256, edb.ptr(out), edb.TYPE_F32, out.stride(0), edb.current_stream())
    assert st == 1 and b"scratch" in edb.lib().edb200_last_error()
