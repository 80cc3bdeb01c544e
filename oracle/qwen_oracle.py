"""CPU oracle of one Qwen-Image denoising pass (TEST INFRASTRUCTURE ONLY).

numpy fp32 restatement of the reference's Qwen-Image graph
(src/dit_models/models/qwen_image.hpp: forward_orig :3116-3301,
QwenImageTransformerBlock::forward :2825-2967, QwenImageAttention::forward :2276-2470,
QwenTimestepProjEmbeddings :2200-2220, AdaLayerNormContinuous :3040-3070; FeedForward
src/dit_models/components/common/common_block.hpp:205-270; position ids
gen_qwen_image_ids, src/dit_models/components/common/rope.hpp:405-438 with the centred
image grid of gen_flux_img_ids :142-182) on dequantised weights.  The reference's
1/128 K/V pre-scale and 1/32, 1/128 linear pre-scales are range tricks for f16
accumulators that cancel exactly in real arithmetic and are not restated.

"parity unpinned": the reference ships no golden tensors for this graph and its own
binary cannot be built without the absent ggml submodule.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import edb_oracle as O
from .flux_oracle import _name_seed


@dataclass
class QwenConfig:
    """Field names follow QwenImageParams (src/dit_models/models/qwen_image.hpp:3074-3114)."""
    num_layers: int = 60
    num_attention_heads: int = 24
    attention_head_dim: int = 128
    in_channels: int = 64            # 16 latent channels x 2x2 patch
    out_channels: int = 16
    joint_attention_dim: int = 3584
    patch_size: int = 2
    axes_dim: tuple = (16, 56, 56)
    theta: int = 10000
    mlp_ratio: float = 4.0
    wtype: int = O.GGML_TYPE_Q4_K

    @property
    def hidden_size(self) -> int:
        return self.num_attention_heads * self.attention_head_dim

    @property
    def mlp_hidden(self) -> int:
        return int(self.hidden_size * self.mlp_ratio)


def qwen_tensor_specs(cfg: QwenConfig):
    """Ordered (name, shape, ggml type).  Every 2-D weight whose row length is a multiple of the
    block size is stored in cfg.wtype, except what tensor_should_be_converted excludes by name
    (src/core/runtime/model_loader.cpp:2141-2172): `img_in.` and `txt_in.` (and biases, norm
    weights) stay f32.  The modulation projections img_mod.1 / txt_mod.1 are floored at q8_0: a
    block type with fewer bits per weight (q4_K) is lifted to q8_0 (set_wtype_override,
    model_loader.cpp:1746-1761)."""
    H, M = cfg.hidden_size, cfg.mlp_hidden
    specs = []
    F32 = O.GGML_TYPE_F32

    def lin(name, n_out, n_in):
        t = cfg.wtype if n_in % 256 == 0 else F32
        if name.startswith("img_in") or name.startswith("txt_in"):
            t = F32
        if (name.endswith("img_mod.1") or name.endswith("txt_mod.1")) and t == O.GGML_TYPE_Q4_K:
            t = O.GGML_TYPE_Q8_0
        specs.append((name + ".weight", (n_out, n_in), t))
        specs.append((name + ".bias", (n_out,), F32))

    lin("time_text_embed.timestep_embedder.linear_1", H, 256)
    lin("time_text_embed.timestep_embedder.linear_2", H, H)
    specs.append(("txt_norm.weight", (cfg.joint_attention_dim,), F32))
    lin("img_in", H, cfg.in_channels)
    lin("txt_in", H, cfg.joint_attention_dim)
    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}."
        lin(p + "img_mod.1", 6 * H, H)
        lin(p + "txt_mod.1", 6 * H, H)
        for l in ("to_q", "to_k", "to_v", "add_q_proj", "add_k_proj", "add_v_proj", "to_out.0", "to_add_out"):
            lin(p + "attn." + l, H, H)
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            specs.append((p + f"attn.{n}.weight", (cfg.attention_head_dim,), F32))
        for s in ("img_mlp", "txt_mlp"):
            lin(p + s + ".net.0.proj", M, H)
            lin(p + s + ".net.2", H, M)
    lin("norm_out.linear", 2 * H, H)
    lin("proj_out", cfg.patch_size ** 2 * cfg.out_channels, H)
    return specs


def qwen_make_weights(cfg: QwenConfig, seed: int = 0, std: float = 0.02):
    out = {}
    for name, shape, t in qwen_tensor_specs(cfg):
        rng = np.random.Generator(np.random.Philox(_name_seed(seed, name)))
        w = (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)
        if name.endswith("txt_norm.weight") or ".attn.norm_" in name:
            w = (w + np.float32(1.0)).astype(np.float32)
        out[name] = (t, O.quantize(w, t)) if t != O.GGML_TYPE_F32 else (O.GGML_TYPE_F32, w)
    return out


def qwen_ids(h_tok: int, w_tok: int, context_len: int) -> np.ndarray:
    """Text ids (s, s, s) with s = max(h_tok/2, w_tok/2) + j first, then image ids
    (0, row - h_tok/2, col - w_tok/2) (rope.hpp:405-438, :142-182 with scale_rope)."""
    start = max(h_tok // 2, w_tok // 2)
    txt = np.repeat((start + np.arange(context_len, dtype=np.float32))[:, None], 3, axis=1)
    img = np.zeros((h_tok * w_tok, 3), dtype=np.float32)
    rr, cc = np.meshgrid(np.arange(h_tok) - h_tok // 2, np.arange(w_tok) - w_tok // 2, indexing="ij")
    img[:, 1] = rr.reshape(-1)
    img[:, 2] = cc.reshape(-1)
    return np.concatenate([txt, img], axis=0).astype(np.float32)


class QwenOracle:
    def __init__(self, cfg: QwenConfig, weights: dict):
        self.cfg = cfg
        # a dict {name: (ggml_type, array)} is dequantised up front; anything else is taken as a
        # mapping name -> f32 array that fetches on use (oracle.weights: device read-back, aliased blocks)
        self.w = O.resolve_weights(weights)

    def lin(self, name, x):
        return O.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def heads(self, x):
        return x.reshape(x.shape[0], self.cfg.num_attention_heads, self.cfg.attention_head_dim)

    def block(self, i, img, txt, t_emb, pe):
        H = self.cfg.hidden_size
        p = f"transformer_blocks.{i}."
        mi = self.lin(p + "img_mod.1", O.silu(t_emb)).reshape(6, H)   # shift1 scale1 gate1 shift2 scale2 gate2
        mt = self.lin(p + "txt_mod.1", O.silu(t_emb)).reshape(6, H)
        xi = O.modulate(O.layer_norm(img), mi[0:1], mi[1:2])
        xt = O.modulate(O.layer_norm(txt), mt[0:1], mt[1:2])
        a = p + "attn."
        iq = O.rms_norm(self.heads(self.lin(a + "to_q", xi)), self.w[a + "norm_q.weight"])
        ik = O.rms_norm(self.heads(self.lin(a + "to_k", xi)), self.w[a + "norm_k.weight"])
        iv = self.heads(self.lin(a + "to_v", xi))
        tq = O.rms_norm(self.heads(self.lin(a + "add_q_proj", xt)), self.w[a + "norm_added_q.weight"])
        tk = O.rms_norm(self.heads(self.lin(a + "add_k_proj", xt)), self.w[a + "norm_added_k.weight"])
        tv = self.heads(self.lin(a + "add_v_proj", xt))
        q = O.apply_rope(np.concatenate([tq, iq], axis=0), pe)
        k = O.apply_rope(np.concatenate([tk, ik], axis=0), pe)
        attn = O.attention(q, k, np.concatenate([tv, iv], axis=0))
        n_txt = txt.shape[0]
        img = O.residual_gate(img, self.lin(a + "to_out.0", attn[n_txt:]), mi[2:3])
        txt = O.residual_gate(txt, self.lin(a + "to_add_out", attn[:n_txt]), mt[2:3])
        yi = self.lin(p + "img_mlp.net.2", O.gelu_tanh(self.lin(p + "img_mlp.net.0.proj",
                                                                  O.modulate(O.layer_norm(img), mi[3:4], mi[4:5]))))
        yt = self.lin(p + "txt_mlp.net.2", O.gelu_tanh(self.lin(p + "txt_mlp.net.0.proj",
                                                                  O.modulate(O.layer_norm(txt), mt[3:4], mt[4:5]))))
        return O.residual_gate(img, yi, mi[5:6]), O.residual_gate(txt, yt, mt[5:6])

    def forward(self, latent, timestep, context, taps=None):
        """latent [C, H, W], context [n_txt, joint_attention_dim] -> [C, H, W]."""
        cfg = self.cfg
        p = cfg.patch_size
        C, Hh, Ww = latent.shape
        h_tok, w_tok = Hh // p, Ww // p
        t_proj = O.timestep_embedding(np.array([timestep], dtype=np.float32), 256)
        t_emb = self.lin("time_text_embed.timestep_embedder.linear_2",
                         O.silu(self.lin("time_text_embed.timestep_embedder.linear_1", t_proj)))
        img = self.lin("img_in", O.patchify(latent, p))
        txt = self.lin("txt_in", O.rms_norm(context, self.w["txt_norm.weight"]))
        pe = O.embed_nd(qwen_ids(h_tok, w_tok, context.shape[0]), cfg.axes_dim, cfg.theta)
        for i in range(cfg.num_layers):
            img, txt = self.block(i, img, txt, t_emb, pe)
            if taps is not None:
                taps[f"block{i}.img"] = img.copy()
                taps[f"block{i}.txt"] = txt.copy()
        m = self.lin("norm_out.linear", O.silu(t_emb)).reshape(2, -1)          # (scale, shift)
        out = self.lin("proj_out", O.modulate(O.layer_norm(img), m[1:2], m[0:1]))
        return O.unpatchify(out, h_tok, w_tok, p)


def true_cfg(cond: np.ndarray, uncond: np.ndarray, cfg_scale: float, patch_size: int) -> np.ndarray:
    """ed_qwen_apply_true_cfg (src/dit_models/pipelines/qwen_image_pipeline.cpp:29-85) on [C, H, W]:
    guided = uncond + s*(cond - uncond) in f32; per patch (all channels) the sums of squares of cond
    and guided are accumulated in double in the order (dy, dx, channel); out = guided * f32(sqrt/sqrt)."""
    f = np.float32
    C, H, W = cond.shape
    p = patch_size
    guided = (uncond + (f(cfg_scale) * (cond - uncond).astype(f)).astype(f)).astype(f)
    out = np.empty_like(guided)
    for py in range(0, H, p):
        for px in range(0, W, p):
            cs = gs = 0.0
            for dy in range(p):
                for dx in range(p):
                    for c in range(C):
                        cv = float(cond[c, py + dy, px + dx])
                        gv = float(guided[c, py + dy, px + dx])
                        cs += cv * cv
                        gs += gv * gv
            r = f(np.sqrt(cs) / np.sqrt(gs)) if gs > 0.0 else f(0.0)
            out[:, py:py + p, px:px + p] = (guided[:, py:py + p, px:px + p] * r).astype(f)
    return out
