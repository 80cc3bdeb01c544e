"""CPU oracle of one Wan 2.1 (t2v) denoising step (TEST INFRASTRUCTURE ONLY).

numpy fp32 restatement of the reference's non-Sage Wan graph
(src/dit_models/models/wan.hpp: Wan::forward :4759-4808, forward_orig :4516-4758,
WanAttentionBlock::forward :4136-4187, WanSelfAttention::forward :3523-3543,
WanT2VCrossAttention::forward_named :3830-3895, Head::forward :4309-4330,
unpatchify :4489-4514; position table gen_wan_pe,
src/dit_models/components/common/rope.hpp:570-622) on dequantised weights.

"parity unpinned": the reference ships no golden tensors for this graph and its own
binary cannot be built without the absent ggml submodule; the ops it is made of are
checked one by one (see edb_oracle.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from . import edb_oracle as O
from .flux_oracle import _name_seed


@dataclass
class WanConfig:
    """Field names follow WanParams (src/dit_models/models/wan.hpp:4382-4405)."""
    dim: int = 5120
    num_heads: int = 40
    ffn_dim: int = 13824
    num_layers: int = 40
    in_dim: int = 16
    out_dim: int = 16
    text_dim: int = 4096
    freq_dim: int = 256
    patch_size: tuple = (1, 2, 2)
    axes_dim: tuple = (44, 42, 42)
    theta: int = 10000
    eps: float = 1e-6
    wtype: int = O.GGML_TYPE_Q8_0

    @property
    def head_dim(self) -> int:
        return self.dim // self.num_heads

    @property
    def patch_features(self) -> int:
        pt, ph, pw = self.patch_size
        return self.in_dim * pt * ph * pw


def wan_tensor_specs(cfg: WanConfig):
    """Ordered (name, shape, quantised?) of every parameter.  Quantised: every 2-D
    weight whose row length is a multiple of the block size except biases, norm
    weights and names containing "embedding" (tensor_should_be_converted,
    src/core/runtime/model_loader.cpp:2141-2172); the Conv3d patch embedding is
    stored as its [dim, in_dim*pt*ph*pw] matrix."""
    D, F = cfg.dim, cfg.ffn_dim
    specs = []

    def lin(name, n_out, n_in, quant):
        specs.append((name + ".weight", (n_out, n_in), quant))
        specs.append((name + ".bias", (n_out,), False))

    lin("patch_embedding", D, cfg.patch_features, False)
    lin("text_embedding.0", D, cfg.text_dim, False)
    lin("text_embedding.2", D, D, False)
    lin("time_embedding.0", D, cfg.freq_dim, False)
    lin("time_embedding.2", D, D, False)
    lin("time_projection.1", 6 * D, D, True)
    for i in range(cfg.num_layers):
        p = f"blocks.{i}."
        specs.append((p + "modulation", (6, D), False))
        for a in ("self_attn", "cross_attn"):
            for l in ("q", "k", "v", "o"):
                lin(p + f"{a}.{l}", D, D, True)
            specs.append((p + f"{a}.norm_q.weight", (D,), False))
            specs.append((p + f"{a}.norm_k.weight", (D,), False))
        specs.append((p + "norm3.weight", (D,), False))
        specs.append((p + "norm3.bias", (D,), False))
        lin(p + "ffn.0", F, D, True)
        lin(p + "ffn.2", D, F, True)
    specs.append(("head.modulation", (2, D), False))
    lin("head.head", cfg.out_dim * cfg.patch_size[0] * cfg.patch_size[1] * cfg.patch_size[2], D, True)
    return specs


def wan_make_weights(cfg: WanConfig, seed: int = 0, std: float = 0.02):
    """Random-init weights N(0, std); norm weights 1 + N(0, std); quantised per
    wan_tensor_specs.  Returns {name: (ggml_type, ndarray)}."""
    out = {}
    for name, shape, quant in wan_tensor_specs(cfg):
        rng = np.random.Generator(np.random.Philox(_name_seed(seed, name)))
        w = (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)
        if ".norm_q." in name or ".norm_k." in name or name.endswith("norm3.weight"):
            w = (w + np.float32(1.0)).astype(np.float32)
        if quant:
            out[name] = (cfg.wtype, O.quantize(w, cfg.wtype))
        else:
            out[name] = (O.GGML_TYPE_F32, w)
    return out


def gelu_erf(x: np.ndarray) -> np.ndarray:
    """0.5*x*(1+erf(x/sqrt(2))): ggml_gelu_erf as selected by ggml_ext_gelu(approximate=false)
    for the text embedder (src/dit_models/models/wan.hpp:4566; src/core/backend/ggml/ggml_extend.hpp:1274-1289)."""
    x = x.astype(np.float32)
    erf = np.vectorize(math.erf, otypes=[np.float64])
    return (0.5 * x.astype(np.float64) * (1.0 + erf(x.astype(np.float64) / math.sqrt(2.0)))).astype(np.float32)


def wan_ids(t_len: int, h_len: int, w_len: int) -> np.ndarray:
    """gen_vid_ids: (t, h, w) index of every token, w fastest (rope.hpp:570-606)."""
    tt, hh, ww = np.meshgrid(np.arange(t_len), np.arange(h_len), np.arange(w_len), indexing="ij")
    return np.stack([tt.reshape(-1), hh.reshape(-1), ww.reshape(-1)], axis=1).astype(np.float32)


def patchify_3d(latent: np.ndarray, patch) -> np.ndarray:
    """[C, T, H, W] -> tokens [t_len*h_len*w_len, C*pt*ph*pw], feature (c, kt, kh, kw):
    the Conv3d patch embedding seen as a linear layer (wan.hpp:4545-4547)."""
    C, T, H, W = latent.shape
    pt, ph, pw = patch
    x = latent.reshape(C, T // pt, pt, H // ph, ph, W // pw, pw)
    x = x.transpose(1, 3, 5, 0, 2, 4, 6)
    return np.ascontiguousarray(x).reshape((T // pt) * (H // ph) * (W // pw), C * pt * ph * pw)


def unpatchify_3d(tokens: np.ndarray, t_len: int, h_len: int, w_len: int, patch, C: int) -> np.ndarray:
    """tokens [L, pt*ph*pw*C] with feature = c + C*(kw + pw*(kh + ph*kt)) -> [C, T, H, W]
    (Wan::unpatchify, wan.hpp:4489-4514)."""
    pt, ph, pw = patch
    x = tokens.reshape(t_len, h_len, w_len, pt, ph, pw, C)
    x = x.transpose(6, 0, 3, 1, 4, 2, 5)
    return np.ascontiguousarray(x).reshape(C, t_len * pt, h_len * ph, w_len * pw)


class WanOracle:
    def __init__(self, cfg: WanConfig, weights: dict):
        self.cfg = cfg
        # a dict {name: (ggml_type, array)} is dequantised up front; anything else is taken as a
        # mapping name -> f32 array that fetches on use (oracle.weights: device read-back, aliased blocks)
        self.w = O.resolve_weights(weights)

    def lin(self, name, x):
        return O.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def prelude(self, tokens, timestep, context):
        """x [L, dim], e [1, dim], e0 [6, dim], context [n_ctx, dim] (wan.hpp:4545-4567)."""
        cfg = self.cfg
        x = self.lin("patch_embedding", tokens)
        e = O.timestep_embedding(np.array([timestep], dtype=np.float32), cfg.freq_dim)
        e = self.lin("time_embedding.2", O.silu(self.lin("time_embedding.0", e)))
        e0 = self.lin("time_projection.1", O.silu(e)).reshape(6, cfg.dim)
        ctx = self.lin("text_embedding.2", gelu_erf(self.lin("text_embedding.0", context)))
        return x, e, e0, ctx

    def heads(self, x):
        return x.reshape(x.shape[0], self.cfg.num_heads, self.cfg.head_dim)

    def self_attention(self, p, y, pe):
        cfg = self.cfg
        q = O.rms_norm(self.lin(p + "q", y), self.w[p + "norm_q.weight"], cfg.eps)   # over the whole row
        k = O.rms_norm(self.lin(p + "k", y), self.w[p + "norm_k.weight"], cfg.eps)
        v = self.lin(p + "v", y)
        q = O.apply_rope(self.heads(q), pe)
        k = O.apply_rope(self.heads(k), pe)
        return self.lin(p + "o", O.attention(q, k, self.heads(v)))

    def cross_attention(self, p, x, ctx):
        cfg = self.cfg
        q = O.rms_norm(self.lin(p + "q", x), self.w[p + "norm_q.weight"], cfg.eps)
        k = O.rms_norm(self.lin(p + "k", ctx), self.w[p + "norm_k.weight"], cfg.eps)
        v = self.lin(p + "v", ctx)
        return self.lin(p + "o", O.attention(self.heads(q), self.heads(k), self.heads(v)))

    def block(self, i, x, e0, ctx, pe):
        cfg = self.cfg
        p = f"blocks.{i}."
        es = (e0 + self.w[p + "modulation"]).astype(np.float32)      # [6, dim]
        y = O.modulate(O.layer_norm(x, cfg.eps), es[0:1], es[1:2])
        x = O.residual_gate(x, self.self_attention(p + "self_attn.", y, pe), es[2:3])
        y = (O.layer_norm(x, cfg.eps) * self.w[p + "norm3.weight"] + self.w[p + "norm3.bias"]).astype(np.float32)
        x = (x + self.cross_attention(p + "cross_attn.", y, ctx)).astype(np.float32)
        y = O.modulate(O.layer_norm(x, cfg.eps), es[3:4], es[4:5])
        y = self.lin(p + "ffn.2", O.gelu_tanh(self.lin(p + "ffn.0", y)))
        return O.residual_gate(x, y, es[5:6])

    def head(self, x, e):
        cfg = self.cfg
        es = (e + self.w["head.modulation"]).astype(np.float32)      # [2, dim]
        return self.lin("head.head", O.modulate(O.layer_norm(x, cfg.eps), es[0:1], es[1:2]))

    def forward(self, latent, timestep, context, taps=None):
        """latent [C, T, H, W] f32, context [n_ctx, text_dim] -> [C, T, H, W]."""
        cfg = self.cfg
        pt, ph, pw = cfg.patch_size
        C, T, H, W = latent.shape
        t_len, h_len, w_len = T // pt, H // ph, W // pw
        x, e, e0, ctx = self.prelude(patchify_3d(latent, cfg.patch_size), timestep, context)
        pe = O.embed_nd(wan_ids(t_len, h_len, w_len), cfg.axes_dim, cfg.theta)
        for i in range(cfg.num_layers):
            x = self.block(i, x, e0, ctx, pe)
            if taps is not None:
                taps[f"block{i}.x"] = x.copy()
        out = self.head(x, e)
        return unpatchify_3d(out, t_len, h_len, w_len, cfg.patch_size, cfg.out_dim)
