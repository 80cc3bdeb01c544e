"""Writes tests/golden/tensor_names.json: tensor names of the diffusers checkpoint layout and what the
reference's own convert_diffusion_model_name (src/utils/name_conversion.cpp) makes of them, per model family.

The conversion is compiled from the reference tree into oracle/_ref/libedref_names.so by oracle/build_ref.sh;
this script only runs where that file exists.  Usage: python tests/golden/make_names_golden.py
"""
import ctypes
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
FAMILIES = {"flux": 0, "sd3": 1, "qwen": 2, "wan": 3}

_MMDIT_BLOCK = [
    "norm1.linear", "norm1_context.linear", "attn.to_q", "attn.to_k", "attn.to_v", "attn.add_q_proj",
    "attn.add_k_proj", "attn.add_v_proj", "attn.to_out.0", "attn.to_add_out", "ff.net.0.proj", "ff.net.2",
    "ff_context.net.0.proj", "ff_context.net.2",
]
_MMDIT_NORMS = ["attn.norm_q.weight", "attn.norm_k.weight", "attn.norm_added_q.weight", "attn.norm_added_k.weight"]


def _wb(stems):
    return [s + e for s in stems for e in (".weight", ".bias")]


def diffusers_names(family):
    names = []
    if family == "flux":
        top = ["time_text_embed.timestep_embedder.linear_1", "time_text_embed.timestep_embedder.linear_2",
               "time_text_embed.text_embedder.linear_1", "time_text_embed.text_embedder.linear_2",
               "time_text_embed.guidance_embedder.linear_1", "time_text_embed.guidance_embedder.linear_2",
               "context_embedder", "x_embedder", "proj_out", "norm_out.linear"]
        names += _wb(top)
        for i in (0, 1, 7, 10, 18):
            names += [f"transformer_blocks.{i}.{n}" for n in _wb(_MMDIT_BLOCK) + _MMDIT_NORMS]
        single = ["norm.linear", "attn.to_q", "attn.to_k", "attn.to_v", "proj_mlp", "proj_out"]
        for i in (0, 3, 11, 30, 37):
            names += [f"single_transformer_blocks.{i}.{n}" for n in _wb(single) + ["attn.norm_q.weight", "attn.norm_k.weight"]]
        # the executors' own layout passes through
        names += ["double_blocks.0.img_attn.qkv.weight", "single_blocks.5.linear1.bias", "img_in.weight",
                  "final_layer.adaLN_modulation.1.weight"]
    elif family == "sd3":
        top = ["time_text_embed.timestep_embedder.linear_1", "time_text_embed.timestep_embedder.linear_2",
               "time_text_embed.text_embedder.linear_1", "time_text_embed.text_embedder.linear_2",
               "pos_embed.proj", "proj_out", "norm_out.linear", "context_embedder"]
        names += _wb(top) + ["pos_embed.pos_embed"]
        extra = ["attn2.to_q", "attn2.to_k", "attn2.to_v", "attn2.to_out.0"]
        for i in (0, 1, 12, 23, 37):
            names += [f"transformer_blocks.{i}.{n}" for n in _wb(_MMDIT_BLOCK + extra) + _MMDIT_NORMS +
                      ["attn2.norm_q.weight", "attn2.norm_k.weight"]]
        names += ["joint_blocks.0.x_block.attn.qkv.weight", "x_embedder.proj.weight", "pos_embed"]
    elif family == "wan":
        top = ["condition_embedder.text_embedder.linear_1", "condition_embedder.text_embedder.linear_2",
               "condition_embedder.time_embedder.linear_1", "condition_embedder.time_embedder.linear_2",
               "condition_embedder.time_proj", "proj_out", "patch_embedding"]
        names += _wb(top) + ["scale_shift_table"]
        block = ["attn1.to_q", "attn1.to_k", "attn1.to_v", "attn1.to_out.0", "attn2.to_q", "attn2.to_k", "attn2.to_v",
                 "attn2.to_out.0", "ffn.net.0.proj", "ffn.net.2", "norm2"]
        for i in (0, 1, 20, 39):
            names += [f"blocks.{i}.{n}" for n in _wb(block) + ["attn1.norm_q.weight", "attn1.norm_k.weight",
                                                              "attn2.norm_q.weight", "attn2.norm_k.weight",
                                                              "scale_shift_table"]]
        names += ["blocks.0.self_attn.q.weight", "blocks.3.norm3.bias", "head.head.weight", "head.modulation",
                  "blocks.2.modulation"]
    elif family == "qwen":   # Qwen-Image keeps the diffusers names
        block = ["attn.to_q", "attn.to_k", "attn.to_v", "attn.add_q_proj", "attn.to_out.0", "attn.to_add_out",
                 "img_mod.1", "txt_mod.1", "img_mlp.net.0.proj", "txt_mlp.net.2"]
        for i in (0, 59):
            names += [f"transformer_blocks.{i}.{n}" for n in _wb(block)]
        names += ["img_in.weight", "txt_in.bias", "time_text_embed.timestep_embedder.linear_1.weight",
                  "norm_out.linear.weight", "proj_out.weight", "txt_norm.weight"]
    return names


def main():
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libedref_names.so"))
    out = {}
    buf = ctypes.create_string_buffer(1024)
    for family, code in FAMILIES.items():
        rows = []
        for name in diffusers_names(family):
            if lib.ref_convert_diffusion_name(code, name.encode(), buf, 1024) != 0:
                raise RuntimeError(name)
            rows.append([name, buf.value.decode()])
        out[family] = rows
    path = os.path.join(HERE, "tensor_names.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=0)
    print(path, {k: len(v) for k, v in out.items()})


if __name__ == "__main__":
    main()
