"""CPU: the oracle's block codecs are bit-exact with gguf-py (the only executable
statement of ggml's q8_0 / q4_K formats available without the ggml submodule)."""
import numpy as np
import pytest

from oracle import edb_oracle as O

gguf = pytest.importorskip("gguf")
from gguf import GGMLQuantizationType as T, quants  # noqa: E402


def _data(rows, k, seed, std=0.02):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, k), dtype=np.float32) * np.float32(std)
    x[0, :32] = 0.0                      # an all-zero block (d == 0 branch)
    x[-1, 5] = 3.0                       # an outlier
    return x


@pytest.mark.parametrize("rows,k", [(1, 32), (7, 256), (64, 3072)])
def test_q8_0_quantize_bit_exact(rows, k):
    x = _data(rows, k, 1)
    assert np.array_equal(O.q8_0_quantize(x), quants.quantize(x, T.Q8_0))


@pytest.mark.parametrize("rows,k", [(1, 32), (7, 256), (64, 3072)])
def test_q8_0_dequantize_bit_exact(rows, k):
    q = quants.quantize(_data(rows, k, 2), T.Q8_0)
    a, b = O.q8_0_dequantize(q), quants.dequantize(q, T.Q8_0)
    assert a.dtype == np.float32 and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_q8_0_half_rounding_ties():
    # values exactly half-way between two codes must round away from zero (roundf)
    x = np.zeros((1, 32), dtype=np.float32)
    x[0, 0] = 127.0
    x[0, 1:8] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 63.5]
    q = O.q8_0_quantize(x)
    assert np.array_equal(q, quants.quantize(x, T.Q8_0))
    assert list(q[0, 2:10].view(np.int8)) == [127, 1, 2, 3, -1, -2, -3, 64]


@pytest.mark.parametrize("rows,k", [(1, 256), (5, 512), (16, 3072)])
def test_q4_k_dequantize_bit_exact(rows, k):
    rng = np.random.default_rng(3)
    blocks = rng.integers(0, 256, size=(rows, k // 256 * 144), dtype=np.uint8)
    # keep d / dmin finite: overwrite the two f16 fields of every block
    b = blocks.reshape(-1, 144)
    b[:, 0:2] = rng.uniform(1e-4, 1e-2, size=(b.shape[0], 1)).astype(np.float16).view(np.uint8)
    b[:, 2:4] = rng.uniform(1e-4, 1e-2, size=(b.shape[0], 1)).astype(np.float16).view(np.uint8)
    a, g = O.q4_k_dequantize(blocks), quants.dequantize(blocks, T.Q4_K)
    assert np.array_equal(a.view(np.uint32), g.view(np.uint32))


def test_q4_k_encoder_emits_valid_blocks():
    x = _data(8, 1024, 4)
    q = O.q4_k_quantize(x)
    assert q.shape == (8, 1024 // 256 * 144) and q.dtype == np.uint8
    d = O.q4_k_dequantize(q)
    assert np.array_equal(d.view(np.uint32), quants.dequantize(q, T.Q4_K).view(np.uint32))
    assert O.rel_l2(d[2:], x[2:]) < 0.12   # 4-bit: coarse but sane


def test_q4_k_scale_pack_roundtrip():
    rng = np.random.default_rng(5)
    sc = rng.integers(0, 64, size=(10, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(10, 8), dtype=np.uint8)
    s2, m2 = O._q4k_unpack_scales(O._q4k_pack_scales(sc, mn))
    assert np.array_equal(s2, sc) and np.array_equal(m2, mn)


def test_bf16_round_matches_torch():
    torch = pytest.importorskip("torch")
    x = np.random.default_rng(6).standard_normal(4096).astype(np.float32)
    ref = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(O.bf16_round(x), ref)
