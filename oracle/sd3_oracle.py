"""CPU oracle of one SD3-medium (MMDiT) denoising pass (TEST INFRASTRUCTURE ONLY).

numpy fp32 restatement of the reference's MMDiT graph
(src/dit_models/models/mmdit.hpp: MMDiT::forward :3403-3487, cropped_pos_embed
:3263-3301, block_mixing :2685-2775, DismantledBlock::pre_attention :2454-2491 and
post_attention :2606-2626, FinalLayer::forward :3143-3160, TimestepEmbedder :1697-1709,
VectorEmbedder :1721-1730, Mlp :1614-1622) on dequantised weights, for the SD3-medium
variant (no q/k norm, no second self-attention).  One pass is batch 1; the pipeline's
CFG runs two passes and combines them (src/pipelines/sd3_pipeline.cpp:631-669).

"parity unpinned": the reference ships no golden tensors for this graph and its own
binary cannot be built without the absent ggml submodule.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import edb_oracle as O
from .flux_oracle import _name_seed


@dataclass
class SD3Config:
    """Field names follow MMDiT's members (src/dit_models/models/mmdit.hpp:3165-3182)."""
    depth: int = 24                  # hidden_size = 64 * depth, num_heads = depth
    patch_size: int = 2
    in_channels: int = 16
    out_channels: int = 16
    adm_in_channels: int = 2048
    context_size: int = 4096
    pos_embed_max_size: int = 192
    mlp_ratio: float = 4.0
    head_dim: int = 64
    wtype: int = O.GGML_TYPE_Q8_0
    num_heads_override: int = 0      # tests may decouple width from depth

    @property
    def num_heads(self) -> int:
        return self.num_heads_override or self.depth

    @property
    def hidden_size(self) -> int:
        return self.head_dim * self.num_heads

    @property
    def mlp_hidden(self) -> int:
        return int(self.hidden_size * self.mlp_ratio)


def sd3_tensor_specs(cfg: SD3Config, n_blocks: int | None = None):
    """Ordered (name, shape, quantised?).  Not quantised: biases, pos_embed and the
    x_embedder / t_embedder / y_embedder / context_embedder prefixes
    (tensor_should_be_converted, src/core/runtime/model_loader.cpp:2141-2172)."""
    H, M = cfg.hidden_size, cfg.mlp_hidden
    nb = cfg.depth if n_blocks is None else n_blocks
    specs = []

    def lin(name, n_out, n_in, quant):
        specs.append((name + ".weight", (n_out, n_in), quant))
        specs.append((name + ".bias", (n_out,), False))

    lin("x_embedder.proj", H, cfg.in_channels * cfg.patch_size ** 2, False)   # Conv2d as its matrix
    specs.append(("pos_embed", (cfg.pos_embed_max_size ** 2, H), False))
    lin("t_embedder.mlp.0", H, 256, False)
    lin("t_embedder.mlp.2", H, H, False)
    lin("y_embedder.mlp.0", H, cfg.adm_in_channels, False)
    lin("y_embedder.mlp.2", H, H, False)
    lin("context_embedder", H, cfg.context_size, False)
    for i in range(nb):
        for side in ("context_block", "x_block"):
            p = f"joint_blocks.{i}.{side}."
            pre_only = side == "context_block" and i == nb - 1
            lin(p + "adaLN_modulation.1", (2 if pre_only else 6) * H, H, True)
            lin(p + "attn.qkv", 3 * H, H, True)
            if not pre_only:
                lin(p + "attn.proj", H, H, True)
                lin(p + "mlp.fc1", M, H, True)
                lin(p + "mlp.fc2", H, M, True)
    lin("final_layer.adaLN_modulation.1", 2 * H, H, True)
    lin("final_layer.linear", cfg.patch_size ** 2 * cfg.out_channels, H, True)
    return specs


def sd3_make_weights(cfg: SD3Config, seed: int = 0, std: float = 0.02):
    out = {}
    for name, shape, quant in sd3_tensor_specs(cfg):
        rng = np.random.Generator(np.random.Philox(_name_seed(seed, name)))
        w = (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)
        out[name] = (cfg.wtype, O.quantize(w, cfg.wtype)) if quant else (O.GGML_TYPE_F32, w)
    return out


def unpatchify_channel_fastest(t: np.ndarray, h: int, w: int, p: int) -> np.ndarray:
    """tokens [h*w, p*p*C] with feature = c + C*(px + p*py) -> [C, h*p, w*p]
    (DiT::unpatchify, patch_last=false, src/dit_models/components/common/common_dit.hpp:38-64)."""
    C = t.shape[1] // (p * p)
    x = t.reshape(h, w, p, p, C).transpose(4, 0, 2, 1, 3)
    return np.ascontiguousarray(x).reshape(C, h * p, w * p)


class SD3Oracle:
    def __init__(self, cfg: SD3Config, weights: dict):
        self.cfg = cfg
        # a dict {name: (ggml_type, array)} is dequantised up front; anything else is taken as a
        # mapping name -> f32 array that fetches on use (oracle.weights: device read-back, aliased blocks)
        self.w = O.resolve_weights(weights)
        self.n_blocks = 1 + max(int(k.split(".")[1]) for k in weights if k.startswith("joint_blocks."))

    def lin(self, name, x):
        return O.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def cropped_pos_embed(self, h_tok, w_tok):
        m = self.cfg.pos_embed_max_size
        top, left = (m - h_tok) // 2, (m - w_tok) // 2
        grid = self.w["pos_embed"].reshape(m, m, -1)
        return grid[top:top + h_tok, left:left + w_tok].reshape(h_tok * w_tok, -1)

    def heads(self, x):
        return x.reshape(x.shape[0], self.cfg.num_heads, self.cfg.head_dim)

    def joint_block(self, i, context, x, c):
        H = self.cfg.hidden_size
        pre_only = i == self.n_blocks - 1
        pc, px = f"joint_blocks.{i}.context_block.", f"joint_blocks.{i}.x_block."
        mc = self.lin(pc + "adaLN_modulation.1", O.silu(c)).reshape(-1, H)
        mx = self.lin(px + "adaLN_modulation.1", O.silu(c)).reshape(-1, H)
        if pre_only:
            c_shift, c_scale = mc[1:2], mc[0:1]          # (scale, shift) order on the pre_only side
        else:
            c_shift, c_scale = mc[0:1], mc[1:2]
        qkv_c = self.lin(pc + "attn.qkv", O.modulate(O.layer_norm(context), c_shift, c_scale))
        qkv_x = self.lin(px + "attn.qkv", O.modulate(O.layer_norm(x), mx[0:1], mx[1:2]))
        qkv = np.concatenate([qkv_c, qkv_x], axis=0)
        q, k, v = (self.heads(qkv[:, j * H:(j + 1) * H]) for j in range(3))
        attn = O.attention(q, k, v)
        n_ctx = context.shape[0]

        def post(p, xx, a, m):
            xx = O.residual_gate(xx, self.lin(p + "attn.proj", a), m[2:3])
            y = O.modulate(O.layer_norm(xx), m[3:4], m[4:5])
            y = self.lin(p + "mlp.fc2", O.gelu_tanh(self.lin(p + "mlp.fc1", y)))
            return O.residual_gate(xx, y, m[5:6])

        new_context = None if pre_only else post(pc, context, attn[:n_ctx], mc)
        return new_context, post(px, x, attn[n_ctx:], mx)

    def forward(self, latent, timestep, context, y, taps=None):
        """latent [C, H, W], context [n_ctx, 4096], y [2048] -> [C, H, W]."""
        cfg = self.cfg
        p = cfg.patch_size
        C, Hh, Ww = latent.shape
        h_tok, w_tok = Hh // p, Ww // p
        x = self.lin("x_embedder.proj", O.patchify(latent, p)) + self.cropped_pos_embed(h_tok, w_tok)
        x = x.astype(np.float32)
        t_freq = O.timestep_embedding(np.array([timestep], dtype=np.float32), 256)
        c = self.lin("t_embedder.mlp.2", O.silu(self.lin("t_embedder.mlp.0", t_freq)))
        c = (c + self.lin("y_embedder.mlp.2", O.silu(self.lin("y_embedder.mlp.0", y.reshape(1, -1))))).astype(np.float32)
        ctx = self.lin("context_embedder", context)
        for i in range(self.n_blocks):
            ctx, x = self.joint_block(i, ctx, x, c)
            if taps is not None:
                taps[f"block{i}.x"] = x.copy()
                if ctx is not None:
                    taps[f"block{i}.context"] = ctx.copy()
        m = self.lin("final_layer.adaLN_modulation.1", O.silu(c)).reshape(2, -1)
        out = self.lin("final_layer.linear", O.modulate(O.layer_norm(x), m[1:2], m[0:1]))   # (scale, shift) order
        return unpatchify_channel_fastest(out, h_tok, w_tok, p)
