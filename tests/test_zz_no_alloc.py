"""The key-mean entry point that keeps its chunk sums in a fixed device array of the
library (no allocation by the call) against the scratch-buffer entry point.

Collected last on purpose: it must pass on its own and after every other GPU test has
used the library in the same process."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _means_via_scratch(edb, cuda, tk, hn, l, d):
    n = edb.lib().edb200_sage_scratch_bytes(hn, l, d)
    offs = (C.c_int64 * 8)()
    strides = (C.c_int * 3)()
    edb.check(edb.lib().edb200_sage_scratch_layout(hn, l, d, offs, strides))
    scratch = torch.zeros(n, dtype=torch.uint8, device=cuda)
    # bit 1 = chunked means, the summation order the static-scratch entry point uses
    edb.check(edb.lib().edb200_sage_quantize_qk(edb.ptr(tk), edb.ptr(tk), hn, l, d, 2, edb.ptr(scratch),
                                                scratch.numel(), edb.current_stream()))
    torch.cuda.synchronize()
    raw = scratch.cpu().numpy()
    return raw[offs[5]: offs[5] + hn * d * 4].view(np.float32).reshape(hn, d).copy()


@pytest.mark.parametrize("hn,l,d", [(3, 700, 128), (2, 333, 64)])
def test_key_means_static_matches_scratch_entry_point(edb, cuda, hn, l, d):
    rng = np.random.default_rng(5)
    outs = []
    for call in range(2):  # two calls in a row reuse the same fixed array
        k = (rng.standard_normal((hn, l, d)) + 0.5 * call).astype(np.float32)
        tk = torch.from_numpy(k).to(cuda).half().contiguous()
        want = _means_via_scratch(edb, cuda, tk, hn, l, d)
        got = torch.full((hn, d), float("nan"), dtype=torch.float32, device=cuda)
        edb.check(edb.lib().edb200_sage_key_means_static(edb.ptr(tk), hn, l, d, edb.ptr(got), edb.current_stream()))
        torch.cuda.synchronize()
        g = got.cpu().numpy()
        assert np.array_equal(g.view(np.uint32), want.view(np.uint32))
        ref = tk.float().mean(dim=1).cpu().numpy()
        assert np.allclose(g, ref, rtol=0, atol=1e-5)
        outs.append(g)
    assert not np.array_equal(outs[0], outs[1])


def test_key_means_static_rejects_oversize(edb, cuda):
    hn, d = 24, 128
    l = 10880 + 128  # one chunk beyond the 1 MiB of chunk sums
    tk = torch.zeros(1, dtype=torch.float16, device=cuda)  # never read: the size check comes first
    out = torch.zeros((hn, d), dtype=torch.float32, device=cuda)
    st = edb.lib().edb200_sage_key_means_static(edb.ptr(tk), hn, l, d, edb.ptr(out), edb.current_stream())
    assert st != 0
    assert b"exceeds" in edb.lib().edb200_last_error()
