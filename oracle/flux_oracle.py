"""CPU oracle of one FLUX.1 denoising step (TEST INFRASTRUCTURE ONLY).

numpy fp32 restatement of the reference's non-Sage FLUX graph
(src/dit_models/models/flux.hpp: Flux::forward_orig :3872-4527,
DoubleStreamBlock::forward :1747-1925, SingleStreamBlock::forward :2974-3034,
LastLayer::forward :3533-3559, Modulation::forward :1617-1634,
MLPEmbedder::forward :1234-1244) on dequantised weights.

"parity unpinned": the reference ships no golden tensors for this graph and its
own binary cannot be built without the absent ggml submodule; this file is
checked only op-by-op (see edb_oracle.py).
"""
from __future__ import annotations

from dataclasses import dataclass, field
import numpy as np

from . import edb_oracle as O


@dataclass
class FluxConfig:
    """Field names follow FluxParams (src/dit_models/models/flux.hpp:3717-3745)."""
    hidden_size: int = 3072
    num_heads: int = 24
    depth: int = 19
    depth_single_blocks: int = 38
    mlp_ratio: float = 4.0
    in_channels: int = 64          # 16 latent channels x 2x2 patch
    context_in_dim: int = 4096
    vec_in_dim: int = 768
    patch_size: int = 2
    axes_dim: tuple = (16, 56, 56)
    theta: int = 10000
    guidance_embed: bool = True
    wtype: int = O.GGML_TYPE_Q8_0

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def mlp_hidden(self) -> int:
        return int(self.hidden_size * self.mlp_ratio)


def flux_tensor_specs(cfg: FluxConfig):
    """Ordered list of (name, shape, quantised?) for every parameter.

    Which tensors are quantised follows tensor_should_be_converted
    (src/core/runtime/model_loader.cpp:2141-2172): every 2-D weight whose row
    length is a multiple of the block size, except biases, norm scales and the
    img_in./txt_in./time_in./vector_in./guidance_in./final_layer. prefixes."""
    H, M = cfg.hidden_size, cfg.mlp_hidden
    specs = []

    def lin(name, n_out, n_in, quant):
        specs.append((name + ".weight", (n_out, n_in), quant))
        specs.append((name + ".bias", (n_out,), False))

    lin("img_in", H, cfg.in_channels, False)
    lin("txt_in", H, cfg.context_in_dim, False)
    lin("time_in.in_layer", H, 256, False)
    lin("time_in.out_layer", H, H, False)
    if cfg.guidance_embed:
        lin("guidance_in.in_layer", H, 256, False)
        lin("guidance_in.out_layer", H, H, False)
    lin("vector_in.in_layer", H, cfg.vec_in_dim, False)
    lin("vector_in.out_layer", H, H, False)
    for i in range(cfg.depth):
        p = f"double_blocks.{i}."
        for s in ("img", "txt"):
            lin(p + f"{s}_mod.lin", 6 * H, H, True)
            lin(p + f"{s}_attn.qkv", 3 * H, H, True)
            specs.append((p + f"{s}_attn.norm.query_norm.scale", (cfg.head_dim,), False))
            specs.append((p + f"{s}_attn.norm.key_norm.scale", (cfg.head_dim,), False))
            lin(p + f"{s}_attn.proj", H, H, True)
            lin(p + f"{s}_mlp.0", M, H, True)
            lin(p + f"{s}_mlp.2", H, M, True)
    for i in range(cfg.depth_single_blocks):
        p = f"single_blocks.{i}."
        lin(p + "modulation.lin", 3 * H, H, True)
        lin(p + "linear1", 3 * H + M, H, True)
        lin(p + "linear2", H, H + M, True)
        specs.append((p + "norm.query_norm.scale", (cfg.head_dim,), False))
        specs.append((p + "norm.key_norm.scale", (cfg.head_dim,), False))
    lin("final_layer.adaLN_modulation.1", 2 * H, H, False)
    lin("final_layer.linear", cfg.patch_size * cfg.patch_size * (cfg.in_channels // (cfg.patch_size ** 2)), H, False)
    return specs


def _name_seed(seed: int, name: str) -> int:
    h = 1469598103934665603
    for ch in name.encode():
        h = ((h ^ ch) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return (h ^ (seed * 0x9E3779B97F4A7C15)) & 0xFFFFFFFFFFFFFFFF


def flux_make_weights(cfg: FluxConfig, seed: int = 0, std: float = 0.02):
    """Random-init weights N(0, std) (norm scales 1 + N(0, std)), quantised per
    flux_tensor_specs.  Returns {name: (ggml_type, ndarray)} where quantised
    tensors are uint8 block bytes."""
    out = {}
    for name, shape, quant in flux_tensor_specs(cfg):
        rng = np.random.Generator(np.random.Philox(_name_seed(seed, name)))
        w = (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)
        if name.endswith(".scale"):
            w = (w + np.float32(1.0)).astype(np.float32)
        if quant:
            out[name] = (cfg.wtype, O.quantize(w, cfg.wtype))
        else:
            out[name] = (O.GGML_TYPE_F32, w)
    return out


def flux_timing_weights(cfg: FluxConfig, seed: int = 0, std: float = 0.02, prefixes=("double_blocks.0.", "single_blocks.0.")):
    """f32 weights for CPU *timing* only: uniform values of standard deviation
    `std`, no quantisation round trip, only the tensors whose names start with
    one of `prefixes`.  Values do not matter for a timing run; skipping the
    normal generator and the block codec keeps the set-up to a few seconds."""
    rng = np.random.default_rng(seed)
    half = np.float32(std * 3.0 ** 0.5)
    out = {}
    for name, shape, _ in flux_tensor_specs(cfg):
        if not name.startswith(tuple(prefixes)):
            continue
        w = rng.random(shape, dtype=np.float32)
        w *= 2 * half
        w -= half
        if name.endswith(".scale"):
            w += np.float32(1.0)
        out[name] = (O.GGML_TYPE_F32, w)
    return out


class FluxOracle:
    def __init__(self, cfg: FluxConfig, weights: dict):
        self.cfg = cfg
        # a dict {name: (ggml_type, array)} is dequantised up front; anything else is taken as a
        # mapping name -> f32 array that fetches on use (oracle.weights: device read-back, aliased blocks)
        self.w = O.resolve_weights(weights)

    def lin(self, name, x):
        return O.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def mlp_embedder(self, name, x):
        return self.lin(name + ".out_layer", O.silu(self.lin(name + ".in_layer", x)))

    def modulation(self, name, vec, n):
        out = self.lin(name, O.silu(vec))          # [1, n*H]
        return [c.reshape(1, -1) for c in np.split(out.reshape(-1), n)]

    def qkv_heads(self, qkv, prefix):
        cfg = self.cfg
        T = qkv.shape[0]
        q, k, v = (qkv[:, i * cfg.hidden_size:(i + 1) * cfg.hidden_size].reshape(T, cfg.num_heads, cfg.head_dim)
                   for i in range(3))
        q = O.rms_norm(q, self.w[prefix + "norm.query_norm.scale"])
        k = O.rms_norm(k, self.w[prefix + "norm.key_norm.scale"])
        return q, k, v

    def attention(self, q, k, v, pe):
        q = O.apply_rope(q, pe)
        k = O.apply_rope(k, pe)
        return O.attention(q, k, v)

    def double_block(self, i, img, txt, vec, pe, taps=None):
        p = f"double_blocks.{i}."
        im = self.modulation(p + "img_mod.lin", vec, 6)
        tm = self.modulation(p + "txt_mod.lin", vec, 6)
        img_mod = O.modulate(O.layer_norm(img), im[0], im[1])
        iq, ik, iv = self.qkv_heads(self.lin(p + "img_attn.qkv", img_mod), p + "img_attn.")
        txt_mod = O.modulate(O.layer_norm(txt), tm[0], tm[1])
        tq, tk, tv = self.qkv_heads(self.lin(p + "txt_attn.qkv", txt_mod), p + "txt_attn.")
        q = np.concatenate([tq, iq], axis=0)
        k = np.concatenate([tk, ik], axis=0)
        v = np.concatenate([tv, iv], axis=0)
        attn = self.attention(q, k, v, pe)
        nt = txt.shape[0]
        txt_attn, img_attn = attn[:nt], attn[nt:]
        img = O.residual_gate(img, self.lin(p + "img_attn.proj", img_attn), im[2])
        h = O.modulate(O.layer_norm(img), im[3], im[4])
        h = self.lin(p + "img_mlp.2", O.gelu_tanh(self.lin(p + "img_mlp.0", h)))
        img = O.residual_gate(img, h, im[5])
        txt = O.residual_gate(txt, self.lin(p + "txt_attn.proj", txt_attn), tm[2])
        h = O.modulate(O.layer_norm(txt), tm[3], tm[4])
        h = self.lin(p + "txt_mlp.2", O.gelu_tanh(self.lin(p + "txt_mlp.0", h)))
        txt = O.residual_gate(txt, h, tm[5])
        if taps is not None:
            taps[f"double{i}.img_modulated"] = img_mod
            taps[f"double{i}.attn.joint_out"] = attn
        return img, txt

    def single_block(self, i, x, vec, pe, taps=None):
        cfg = self.cfg
        p = f"single_blocks.{i}."
        m = self.modulation(p + "modulation.lin", vec, 3)
        x_mod = O.modulate(O.layer_norm(x), m[0], m[1])
        qkv_mlp = self.lin(p + "linear1", x_mod)
        q, k, v = self.qkv_heads(qkv_mlp[:, : 3 * cfg.hidden_size], p)
        attn = self.attention(q, k, v, pe)
        mlp = O.gelu_tanh(qkv_mlp[:, 3 * cfg.hidden_size:])
        out = self.lin(p + "linear2", np.concatenate([attn, mlp], axis=1))
        return O.residual_gate(x, out, m[2])

    def prelude(self, x_tokens, timestep, context, y, guidance):
        cfg = self.cfg
        img = self.lin("img_in", x_tokens)
        vec = self.mlp_embedder("time_in", O.timestep_embedding(np.array([timestep]), 256, 10000, 1000.0))
        if cfg.guidance_embed:
            vec = vec + self.mlp_embedder("guidance_in", O.timestep_embedding(np.array([guidance]), 256, 10000, 1000.0))
        vec = (vec + self.mlp_embedder("vector_in", y.reshape(1, -1))).astype(np.float32)
        txt = self.lin("txt_in", context)
        return img, txt, vec

    def final_layer(self, img, vec):
        m = self.lin("final_layer.adaLN_modulation.1", O.silu(vec)).reshape(-1)
        H = self.cfg.hidden_size
        shift, scale = m[:H].reshape(1, -1), m[H:].reshape(1, -1)
        return self.lin("final_layer.linear", O.modulate(O.layer_norm(img), shift, scale))

    def forward_tokens(self, x_tokens, timestep, context, y, guidance, h_tok, w_tok, taps=None):
        """x_tokens [T_img, in_channels] -> [T_img, out_channels]."""
        cfg = self.cfg
        pe = O.embed_nd(O.flux_ids(h_tok, w_tok, context.shape[0]), cfg.axes_dim, cfg.theta)
        img, txt, vec = self.prelude(x_tokens, timestep, context, y, guidance)
        if taps is not None:
            taps["prelude.img_in"] = img
            taps["prelude.txt_in"] = txt
            taps["prelude.temb"] = vec
        for i in range(cfg.depth):
            img, txt = self.double_block(i, img, txt, vec, pe, taps)
            if taps is not None:
                taps[f"double{i}.img"] = img
                taps[f"double{i}.txt"] = txt
        x = np.concatenate([txt, img], axis=0)
        for i in range(cfg.depth_single_blocks):
            x = self.single_block(i, x, vec, pe, taps)
            if taps is not None:
                taps[f"single{i}.x"] = x
        img = x[txt.shape[0]:]
        return self.final_layer(img, vec)

    def forward(self, latent, timestep, context, y, guidance, taps=None):
        """latent [C, H, W] f32 -> model output [C, H, W] (patchify -> blocks ->
        unpatchify; Flux::forward_flux_chroma, src/dit_models/models/flux.hpp:4633-4691)."""
        C, Hh, Ww = latent.shape
        p = self.cfg.patch_size
        tok = O.patchify(latent, p)
        out = self.forward_tokens(tok, timestep, context, y, guidance, Hh // p, Ww // p, taps)
        return O.unpatchify(out, Hh // p, Ww // p, p)
