"""Weight providers for the oracles (TEST INFRASTRUCTURE ONLY).

The oracle classes take either a dict {name: (ggml_type, array)} or one of these mappings, which hand
out f32 arrays by name when the oracle asks for them, so that a model of tens of GB never has to sit
in host memory as f32 all at once.
"""
from __future__ import annotations

import re


class DeviceWeights:
    """The parameters a device-resident model actually holds, read back one tensor at a time through
    the library's edb200_*_get_tensor_f32 (quantised weights come back dequantised: exactly the values
    the GPU kernels multiply with).  `model` is one of the binding's model classes.  Small tensors
    (vectors) are cached, matrices are fetched on every use."""

    def __init__(self, model, cache_below: int = 1 << 16):
        self.model = model
        self.names = [n for n, _, _, _, _ in model.tensor_table()]
        self._set = set(self.names)
        self._cache = {}
        self._cache_below = cache_below

    def __contains__(self, name):
        return name in self._set

    def __iter__(self):
        return iter(self.names)

    def keys(self):
        return self.names

    def __getitem__(self, name):
        if name in self._cache:
            return self._cache[name]
        if name not in self._set:
            raise KeyError(name)
        a = self.model.get_tensor(name)
        if a.size < self._cache_below:
            self._cache[name] = a
        return a

    def get(self, name, default=None):
        return self[name] if name in self._set else default


def timing_weights(specs, seed: int = 0, std: float = 0.02) -> dict:
    """{name: f32 array} for CPU *timing* only: uniform values of standard deviation `std` for every
    (name, shape, ...) of `specs`, no quantisation round trip.  Values do not matter for a timing run;
    skipping the normal generator and the block codecs keeps the set-up to seconds."""
    import numpy as np
    rng = np.random.default_rng(seed)
    half = np.float32(std * 3.0 ** 0.5)
    out = {}
    for name, shape, *_ in specs:
        w = rng.random(shape, dtype=np.float32)
        w *= 2 * half
        w -= half
        if name.endswith(".scale") or ("norm" in name and name.endswith(".weight") and len(shape) == 1):
            w += np.float32(1.0)   # norm weights are centred on one
        out[name] = w
    return out


class AliasedBlocks:
    """For CPU *timing* runs: every block index of a stack resolves to block 0 of `weights` (a dict of
    f32 arrays holding one block per stack), so a full-depth pass can be timed with one block's worth of
    memory.  The arithmetic and its cost are those of the full model; the values are not.  `depth` is the
    number of blocks the names pretend to have (for code that counts blocks from the tensor names)."""

    _IDX = re.compile(r"^((?:double_blocks|single_blocks|joint_blocks|transformer_blocks|blocks)\.)(\d+)(\..*)$")

    def __init__(self, weights: dict, depth: int = 1):
        self.w = weights
        self.depth = depth

    def _key(self, name):
        m = self._IDX.match(name)
        return m.group(1) + "0" + m.group(3) if m else name

    def __contains__(self, name):
        return self._key(name) in self.w

    def __iter__(self):
        for name in self.w:
            m = self._IDX.match(name)
            if m and m.group(2) == "0":
                for i in range(self.depth):
                    yield m.group(1) + str(i) + m.group(3)
            elif not m:
                yield name

    def keys(self):
        return list(iter(self))

    def __getitem__(self, name):
        return self.w[self._key(name)]

    def get(self, name, default=None):
        return self.w.get(self._key(name), default)
