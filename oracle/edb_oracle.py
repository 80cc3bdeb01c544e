"""CPU oracle for the DiT denoise-step hot path (TEST INFRASTRUCTURE ONLY).

This module is the checker, never the product: only tests, the smoke entry and
the CPU-baseline leg of the benchmark may import it.  It restates, in numpy
fp32, the arithmetic of the reference's non-Sage CPU path for one denoising
step, plus a numpy model of the Sage INT8 quantisers.

Parity status: "parity unpinned" for every op whose arithmetic lives in the
un-vendored ggml submodule (mul_mat, norm, rms_norm, gelu, softmax attention):
the reference ships no golden vectors for them.  What *is* pinned:
  * q8_0 / q4_K block codecs: bit-exact against gguf-py 0.19 `gguf.quants`
    (tests/test_oracle_codecs.py);
  * modulate / residual-gate / RoPE / rms-norm-mul(f16): bit-exact against the
    reference's own CPU custom-op callbacks compiled from the reference tree
    (oracle/build_ref.sh -> oracle/_ref/libedref_cpu.so, fixtures in tests/golden/).

Each function cites the reference file:line it follows (paths are relative to
the reference project root).

Conventions: numpy row-major.  Activations are [tokens, features]; a linear
weight is [out_features, in_features] (ggml ne = [in, out]); quantised weights
are uint8 arrays [out_features, bytes_per_row].
"""
from __future__ import annotations

import math
import numpy as np

QK8_0 = 32
Q8_0_BLOCK_BYTES = 34
QK_K = 256
Q4_K_BLOCK_BYTES = 144

GGML_TYPE_F32 = 0
GGML_TYPE_F16 = 1
GGML_TYPE_Q8_0 = 8
GGML_TYPE_Q4_K = 12
GGML_TYPE_BF16 = 30

# ----------------------------------------------------------------------------
# Block codecs (ggml formats; sizes per gguf-py constants.py GGML_QUANT_SIZES)
# ----------------------------------------------------------------------------


def _roundf(x: np.ndarray) -> np.ndarray:
    """C roundf(): half away from zero (ggml quantize_row_q8_0_ref uses roundf)."""
    a = np.abs(x)
    f = np.floor(a)
    r = f + (a - f >= np.float32(0.5)).astype(np.float32)
    return np.copysign(r, x)


def q8_0_quantize(x: np.ndarray) -> np.ndarray:
    """f32 [rows, K] -> uint8 [rows, K/32*34].

    Follows ggml quantize_row_q8_0_ref as restated by gguf-py
    quants.py Q8_0.quantize_blocks (:378-394): d = amax/127, id = 1/d (0 if d==0),
    q = roundf(x*id), d stored as f16.  This is the quantiser the reference's
    loader calls through ggml_quantize_chunk (src/core/runtime/model_loader.cpp:663-704).
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, K = x.shape
    assert K % QK8_0 == 0
    b = x.reshape(rows * (K // QK8_0), QK8_0)
    d = np.abs(b).max(axis=1, keepdims=True) / np.float32(127)
    with np.errstate(divide="ignore"):
        inv = np.where(d == 0, np.float32(0), np.float32(1) / d).astype(np.float32)
    q = _roundf(b * inv).astype(np.int8)
    out = np.empty((b.shape[0], Q8_0_BLOCK_BYTES), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(rows, (K // QK8_0) * Q8_0_BLOCK_BYTES)


def q8_0_dequantize(q: np.ndarray) -> np.ndarray:
    """uint8 [rows, K/32*34] -> f32 [rows, K]; w = f32(d) * f32(q)
    (gguf-py quants.py Q8_0.dequantize_blocks :396-401)."""
    rows = q.shape[0]
    b = np.ascontiguousarray(q).reshape(-1, Q8_0_BLOCK_BYTES)
    d = b[:, :2].copy().view(np.float16).astype(np.float32)
    v = b[:, 2:].view(np.int8).astype(np.float32)
    return (v * d).reshape(rows, -1)


def _q4k_unpack_scales(s: np.ndarray):
    """12 packed bytes -> 8 six-bit scales, 8 six-bit mins
    (gguf-py quants.py Q4_K.get_scale_min :478-501)."""
    s = s.reshape(-1, 3, 4)
    d, m, md = s[:, 0], s[:, 1], s[:, 2]
    sc = np.concatenate([d & 0x3F, (md & 0x0F) | ((d >> 2) & 0x30)], axis=-1)
    mn = np.concatenate([m & 0x3F, (md >> 4) | ((m >> 2) & 0x30)], axis=-1)
    return sc, mn


def _q4k_pack_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Inverse of _q4k_unpack_scales: [n,8] u8 (<64) x2 -> [n,12] u8."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    out = np.zeros((sc.shape[0], 12), dtype=np.uint8)
    out[:, 0:4] = (sc[:, 0:4] & 0x3F) | ((sc[:, 4:8] & 0x30) << 2)
    out[:, 4:8] = (mn[:, 0:4] & 0x3F) | ((mn[:, 4:8] & 0x30) << 2)
    out[:, 8:12] = (sc[:, 4:8] & 0x0F) | ((mn[:, 4:8] & 0x0F) << 4)
    return out


def q4_k_dequantize(q: np.ndarray) -> np.ndarray:
    """uint8 [rows, K/256*144] -> f32 [rows, K]; w = (d*sc)*q - (dmin*m)
    (gguf-py quants.py Q4_K.dequantize_blocks :504-522)."""
    rows = q.shape[0]
    b = np.ascontiguousarray(q).reshape(-1, Q4_K_BLOCK_BYTES)
    n = b.shape[0]
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)
    sc, mn = _q4k_unpack_scales(b[:, 4:16])
    dd = (d * sc.astype(np.float32)).reshape(n, 8, 1)
    dm = (dmin * mn.astype(np.float32)).reshape(n, 8, 1)
    qs = b[:, 16:].reshape(n, 4, 1, 32) >> np.array([0, 4], dtype=np.uint8).reshape(1, 1, 2, 1)
    qs = (qs & np.uint8(0x0F)).reshape(n, 8, 32).astype(np.float32)
    return (dd * qs - dm).reshape(rows, -1)


def q4_k_quantize(x: np.ndarray) -> np.ndarray:
    """f32 [rows, K] -> valid q4_K blocks, uint8 [rows, K/256*144].

    The reference quantises through ggml's quantize_row_q4_K_impl with an
    all-ones importance vector (tools/imatrix/ggml_quant.py:52-57,
    src/core/runtime/model_loader.cpp:650-661); that routine is in the absent
    ggml submodule and gguf-py has no q4_K encoder, so this is an independent
    min/max encoder that emits valid blocks.  Parity for q4_K is defined on
    identical quantised bytes given to oracle and kernel.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, K = x.shape
    assert K % QK_K == 0
    b = x.reshape(-1, 8, 32)
    n = b.shape[0]
    mins = np.minimum(b.min(axis=2), 0.0)              # [n,8] (<= 0)
    maxs = b.max(axis=2)
    scale = (maxs - mins) / np.float32(15)             # per sub-block step
    d = scale.max(axis=1) / np.float32(63)             # super-block scale of scales
    dmin = (-mins).max(axis=1) / np.float32(63)
    d16 = d.astype(np.float16)
    dmin16 = dmin.astype(np.float16)
    df = d16.astype(np.float32)[:, None]
    dmf = dmin16.astype(np.float32)[:, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(df > 0, np.rint(scale / df), 0.0)
        mn = np.where(dmf > 0, np.rint(-mins / dmf), 0.0)
    sc = np.clip(sc, 0, 63).astype(np.uint8)
    mn = np.clip(mn, 0, 63).astype(np.uint8)
    eff_scale = (df * sc.astype(np.float32))[:, :, None]
    eff_min = (dmf * mn.astype(np.float32))[:, :, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        qv = np.where(eff_scale > 0, np.rint((b + eff_min) / eff_scale), 0.0)
    qv = np.clip(qv, 0, 15).astype(np.uint8)           # [n,8,32]
    qv = qv.reshape(n, 4, 2, 32)
    packed = (qv[:, :, 0, :] | (qv[:, :, 1, :] << 4)).reshape(n, 128)
    out = np.empty((n, Q4_K_BLOCK_BYTES), dtype=np.uint8)
    out[:, 0:2] = d16.reshape(n, 1).view(np.uint8)
    out[:, 2:4] = dmin16.reshape(n, 1).view(np.uint8)
    out[:, 4:16] = _q4k_pack_scales(sc, mn)
    out[:, 16:] = packed
    return out.reshape(rows, (K // QK_K) * Q4_K_BLOCK_BYTES)


def resolve_weights(weights):
    """{name: (ggml_type, array)} -> {name: f32 array} (dequantised); any other mapping is returned as is
    (it must give f32 arrays by name, support .get(name) and iteration over names)."""
    if isinstance(weights, dict):
        return {k: dequantize(v, t) if t != GGML_TYPE_F32 else v for k, (t, v) in weights.items()}
    return weights


def quantize(x: np.ndarray, ggml_type: int) -> np.ndarray:
    if ggml_type == GGML_TYPE_Q8_0:
        return q8_0_quantize(x)
    if ggml_type == GGML_TYPE_Q4_K:
        return q4_k_quantize(x)
    raise ValueError(ggml_type)


def dequantize(q: np.ndarray, ggml_type: int) -> np.ndarray:
    if ggml_type == GGML_TYPE_Q8_0:
        return q8_0_dequantize(q)
    if ggml_type == GGML_TYPE_Q4_K:
        return q4_k_dequantize(q)
    if ggml_type == GGML_TYPE_F32:
        return np.asarray(q, dtype=np.float32)
    raise ValueError(ggml_type)


# ----------------------------------------------------------------------------
# dtype helpers
# ----------------------------------------------------------------------------


def bf16_round(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 -> f32, round-to-nearest-even (what ggml_fp32_to_bf16 does
    for finite values)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(np.float32)


def f16_round(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


# ----------------------------------------------------------------------------
# Elementwise / normalisation ops
# ----------------------------------------------------------------------------


def layer_norm(x: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    """ggml_norm, no affine (call site src/core/backend/ggml/ggml_extend.hpp:1986-1999;
    DiT blocks use eps 1e-6 without affine, src/dit_models/models/flux.hpp:1664-1668).
    ggml's CPU kernel accumulates mean and variance in double."""
    x64 = x.astype(np.float64)
    mean = x64.mean(axis=-1, keepdims=True)
    xc = (x64 - mean).astype(np.float32)
    var = (xc.astype(np.float64) ** 2).mean(axis=-1, keepdims=True)
    scale = (1.0 / np.sqrt(var + eps)).astype(np.float32)
    return xc * scale


def rms_norm(x: np.ndarray, w: np.ndarray | None, eps: float = 1e-6) -> np.ndarray:
    """x * rsqrt(mean(x^2)+eps) * w  (src/dit_models/components/common/normalization.cpp:42-61;
    fused form src/core/backend/ggml/ed_ggml_norm_ext.hpp:223-263)."""
    ss = (x.astype(np.float64) ** 2).mean(axis=-1, keepdims=True)
    scale = (1.0 / np.sqrt(ss + eps)).astype(np.float32)
    y = x * scale
    if w is not None:
        y = y * w
    return y.astype(np.float32)


def rms_norm_mul_f16_callback(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """Exact restatement of rms_norm_mul_f16_cpu_custom_op
    (src/core/backend/ggml/ed_ggml_norm_ext.hpp:223-263): sequential f32 sum of
    squares, scale = 1/sqrt(sum/n + eps), y = f16((v*scale)*w)."""
    x = np.asarray(x, dtype=np.float32)
    n = x.shape[-1]
    flat = x.reshape(-1, n)
    ss = np.zeros(flat.shape[0], dtype=np.float32)
    for i in range(n):                      # sequential f32 accumulation order
        ss = ss + flat[:, i] * flat[:, i]
    scale = np.float32(1.0) / np.sqrt(ss / np.float32(n) + np.float32(eps), dtype=np.float32)
    y = (flat * scale[:, None]) * w.astype(np.float32)[None, :]
    return y.astype(np.float16).reshape(x.shape)


def modulate(x: np.ndarray, shift: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """y = (x + x*scale) + shift, each op rounded to f32, no FMA
    (src/core/backend/ggml/ed_ggml_modulation_ext.hpp:168-199)."""
    prod = (x * scale).astype(np.float32)
    return ((x + prod).astype(np.float32) + shift).astype(np.float32)


def residual_gate(residual: np.ndarray, x: np.ndarray, gate: np.ndarray) -> np.ndarray:
    """y = residual + x*gate (src/core/backend/ggml/ed_ggml_modulation_ext.hpp:201-226)."""
    return (residual + (x * gate).astype(np.float32)).astype(np.float32)


def euler_update(x: np.ndarray, model_out: np.ndarray, sigma: float, sigma_next: float) -> np.ndarray:
    """The sampler's per-step latent update (src/dit_models/pipelines/flux_pipeline.cpp:1111-1112,
    :1290-1297): denoised = model_out*(-sigma) + x; x + ((x - denoised)/sigma)*(sigma_next - sigma),
    or denoised itself when sigma == 0.  float32 operation by operation."""
    f = np.float32
    x = x.astype(f)
    denoised = ((model_out.astype(f) * f(-sigma)).astype(f) + x).astype(f)
    if f(sigma) == f(0.0):
        return denoised
    d = ((x - denoised).astype(f) / f(sigma)).astype(f)
    return (x + (d * (f(sigma_next) - f(sigma))).astype(f)).astype(f)


def flow_update(x: np.ndarray, model_out: np.ndarray, sigma: float, sigma_next: float) -> np.ndarray:
    """SD3's per-step update x += model_out * (sigma_next - sigma)
    (src/dit_models/pipelines/sd3_pipeline.cpp:697), float32 operation by operation."""
    f = np.float32
    dt = f(f(sigma_next) - f(sigma))
    return (x.astype(f) + (model_out.astype(f) * dt).astype(f)).astype(f)


def cfg_combine(uncond: np.ndarray, cond: np.ndarray, cfg_scale: float) -> np.ndarray:
    """uncond + cfg_scale * (cond - uncond) (src/dit_models/pipelines/flux_pipeline.cpp:1258),
    float32 operation by operation."""
    f = np.float32
    u = uncond.astype(f)
    return (u + (f(cfg_scale) * (cond.astype(f) - u).astype(f)).astype(f)).astype(f)


def gelu_tanh(x: np.ndarray) -> np.ndarray:
    """0.5*x*(1+tanh(sqrt(2/pi)*x*(1+0.044715*x*x)))
    (src/core/backend/ggml/ed_ggml_sp_flux_ext.hpp:675-679; ggml_gelu call site
    src/core/backend/ggml/ggml_extend.hpp:1274-1289)."""
    x = x.astype(np.float32)
    c = np.float32(0.7978845608028654)
    k = np.float32(0.044715)
    return (np.float32(0.5) * x * (np.float32(1.0) + np.tanh(c * x * (np.float32(1.0) + k * x * x)))).astype(np.float32)


def silu(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.float32)
    return (x / (np.float32(1.0) + np.exp(-x))).astype(np.float32)


def linear(x: np.ndarray, w_f32: np.ndarray, b: np.ndarray | None = None) -> np.ndarray:
    """y = x @ W^T + b on dequantised fp32 weights (ggml_ext_linear,
    src/core/backend/ggml/ggml_extend.hpp:1308-1347)."""
    y = x.astype(np.float32) @ w_f32.T
    if b is not None:
        y = y + b
    return y.astype(np.float32)


def timestep_embedding(t: np.ndarray, dim: int, max_period: int = 10000, scale: float = 1.0) -> np.ndarray:
    """[N] -> [N, dim] = [cos | sin] (src/core/backend/ggml/ggml_extend.hpp:2078-2105,
    flip_sin_to_cos=true)."""
    t = np.asarray(t, dtype=np.float32).reshape(-1)
    half = dim // 2
    freqs = np.array([np.float32(math.exp(-math.log(max_period) * i / half)) for i in range(half)], dtype=np.float32)
    arg = (t[:, None] * freqs[None, :]).astype(np.float32) * np.float32(scale)
    return np.concatenate([np.cos(arg), np.sin(arg)], axis=1).astype(np.float32)


# ----------------------------------------------------------------------------
# RoPE
# ----------------------------------------------------------------------------


def rope_axis(pos: np.ndarray, dim: int, theta: float) -> np.ndarray:
    """[L] positions -> [L, dim/2, 4] = [cos, -sin, sin, cos]
    (src/dit_models/components/common/rope.hpp:77-127)."""
    half = dim // 2
    if half == 1:
        scale = np.array([0.0], dtype=np.float32)
    else:
        end = np.float32((dim - 2.0) / dim)
        step = end / np.float32(half - 1)
        scale = (np.arange(half, dtype=np.float32) * step).astype(np.float32)
    omega = (np.float32(1.0) / np.power(np.float32(theta), scale, dtype=np.float32)).astype(np.float32)
    ang = (pos.astype(np.float32)[:, None] * omega[None, :]).astype(np.float32)
    c, s = np.cos(ang), np.sin(ang)
    return np.stack([c, -s, s, c], axis=-1).astype(np.float32)


def embed_nd(ids: np.ndarray, axes_dim, theta: float) -> np.ndarray:
    """ids [L, n_axes] -> pe [L, d_head/2, 2, 2]
    (src/dit_models/components/common/rope.hpp:201-260)."""
    parts = [rope_axis(ids[:, a], axes_dim[a], theta) for a in range(len(axes_dim))]
    pe = np.concatenate(parts, axis=1)
    return pe.reshape(pe.shape[0], pe.shape[1], 2, 2)


def flux_ids(h_tok: int, w_tok: int, context_len: int) -> np.ndarray:
    """FLUX.1 position ids: text tokens all-zero, image token (0,row,col); text first
    (src/dit_models/components/common/rope.hpp:130-199,312-337)."""
    txt = np.zeros((context_len, 3), dtype=np.float32)
    img = np.zeros((h_tok * w_tok, 3), dtype=np.float32)
    rr, cc = np.meshgrid(np.arange(h_tok), np.arange(w_tok), indexing="ij")
    img[:, 1] = rr.reshape(-1)
    img[:, 2] = cc.reshape(-1)
    return np.concatenate([txt, img], axis=0)


def apply_rope(x: np.ndarray, pe: np.ndarray) -> np.ndarray:
    """x [L, H, d] (interleaved pairs), pe [L, d/2, 2, 2] -> [L, H, d].
    y0 = x0*pe[0,0] + x1*pe[0,1]; y1 = x0*pe[1,0] + x1*pe[1,1] in the stored
    [[cos,-sin],[sin,cos]] matrix, each product and the sum rounded to f32
    (src/core/backend/ggml/ed_ggml_rope_ext.hpp:105-184: the callback reads
    pe(row,col) at ggml index (row,col,pair,seq), i.e. numpy pe[seq,pair,col,row])."""
    L, H, d = x.shape
    xp = x.reshape(L, H, d // 2, 2).astype(np.float32)
    x0, x1 = xp[..., 0], xp[..., 1]
    p = pe[:L].astype(np.float32)
    # ggml element (row=i0, col=i1) of a [2,2,...] tensor is numpy [..., i1, i0]
    pe00 = p[:, None, :, 0, 0]  # row0,col0 -> cos
    pe10 = p[:, None, :, 0, 1]  # row1,col0 -> -sin
    pe01 = p[:, None, :, 1, 0]  # row0,col1 -> sin
    pe11 = p[:, None, :, 1, 1]  # row1,col1 -> cos
    y0 = ((x0 * pe00).astype(np.float32) + (x1 * pe10).astype(np.float32)).astype(np.float32)
    y1 = ((x0 * pe01).astype(np.float32) + (x1 * pe11).astype(np.float32)).astype(np.float32)
    return np.stack([y0, y1], axis=-1).reshape(L, H, d)


# ----------------------------------------------------------------------------
# Attention
# ----------------------------------------------------------------------------


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float | None = None,
              kv_f16: bool = True) -> np.ndarray:
    """softmax(q k^T * scale) v per head; q [Lq,H,d], k,v [Lk,H,d] -> [Lq, H*d].
    Non-causal, no mask; K and V are rounded to f16 as the reference feeds
    ggml_flash_attn_ext (src/core/backend/ggml/ggml_extend.hpp:1749-1984,
    softmax/accumulate in f32, GGML_PREC_F32 :1895-1899)."""
    Lq, H, d = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if kv_f16:
        k = f16_round(k)
        v = f16_round(v)
    out = np.empty((Lq, H, d), dtype=np.float32)
    for h in range(H):
        s = (q[:, h, :].astype(np.float32) @ k[:, h, :].T.astype(np.float32)) * np.float32(scale)
        s = s - s.max(axis=1, keepdims=True)
        p = np.exp(s, dtype=np.float32)
        p /= p.sum(axis=1, keepdims=True)
        out[:, h, :] = p @ v[:, h, :].astype(np.float32)
    return out.reshape(Lq, H * d)


# ----------------------------------------------------------------------------
# Sage INT8 Q/K quantisers (the reference's INT8 quantiser is its CUDA kernels)
# ----------------------------------------------------------------------------


def sage_channel_mean(x: np.ndarray) -> np.ndarray:
    """x [HN, L, d] -> mean over tokens [HN, d]; sequential f32 sum in token
    order then one division (src/core/backend/ggml/cuda/ed_cuda_sage_attn.cu:209-244)."""
    HN, L, d = x.shape
    acc = np.zeros((HN, d), dtype=np.float32)
    for t in range(L):
        acc = acc + x[:, t, :].astype(np.float32)
    return (acc / np.float32(L)).astype(np.float32)


def sage_channel_mean_chunked(x: np.ndarray) -> np.ndarray:
    """Model of this library's fast channel mean (EDB200_SAGE_FAST_MEANS; no counterpart in the reference,
    whose mean is sage_channel_mean above): the token axis is cut into chunks of 128 rows; inside a
    chunk the rows are dealt round-robin to G = 1024 / d row groups (8 for d = 128, 16 for d = 64), each
    group is summed in row order, the G sums are added as a pairwise tree; the chunk sums are then added
    in chunk order and divided by L.  Every operation rounded to f32."""
    f = np.float32
    HN, L, d = x.shape
    G = 128 // (d // 8)
    total = np.zeros((HN, d), dtype=f)
    for c0 in range(0, L, 128):
        blk = x[:, c0:min(L, c0 + 128), :].astype(f)
        n = blk.shape[1]
        s = np.zeros((G, HN, d), dtype=f)
        for t in range(n):
            s[t % G] = (s[t % G] + blk[:, t, :]).astype(f)
        m = 1
        while m < G:
            for i in range(0, G, 2 * m):
                s[i] = (s[i] + s[i + m]).astype(f)
            m *= 2
        total = (total + s[0]).astype(f)
    return (total / f(L)).astype(f)


def sage_smooth_q_bias_fused(k: np.ndarray, qm: np.ndarray) -> np.ndarray:
    """Model of the bias sum of this library's fused pre-pass kernel (same products as
    sage_smooth_q_bias, another fixed order): per run of 8 channels ((p0+p1)+(p2+p3))+((p4+p5)+(p6+p7)),
    then a pairwise tree over the d/8 runs."""
    f = np.float32
    HN, L, d = k.shape
    p = (k.astype(f) * qm[:, None, :]).astype(f).reshape(HN, L, d // 8, 8)
    a = ((p[..., 0] + p[..., 1]).astype(f) + (p[..., 2] + p[..., 3]).astype(f)).astype(f)
    b = ((p[..., 4] + p[..., 5]).astype(f) + (p[..., 6] + p[..., 7]).astype(f)).astype(f)
    v = (a + b).astype(f)                      # [HN, L, d/8]
    while v.shape[-1] > 1:
        v = (v[..., 0::2] + v[..., 1::2]).astype(f)
    return v[..., 0]


def _sage_quant(x: np.ndarray, mean: np.ndarray | None, blk: int):
    HN, L, d = x.shape
    nblk = (L + blk - 1) // blk
    xs = x.astype(np.float32)
    if mean is not None:
        xs = (xs - mean[:, None, :]).astype(np.float32)
    pad = nblk * blk - L
    xa = np.abs(xs)
    if pad:
        xa = np.concatenate([xa, np.zeros((HN, pad, d), np.float32)], axis=1)
    amax = np.maximum(xa.reshape(HN, nblk, blk * d).max(axis=2), np.float32(1e-7))
    scale = (amax / np.float32(127.0)).astype(np.float32)
    inv = (np.float32(1.0) / scale).astype(np.float32)
    inv_t = np.repeat(inv, blk, axis=1)[:, :L]
    val = (xs * inv_t[:, :, None]).astype(np.float32)
    val = np.maximum(np.minimum(val, np.float32(127.0)), np.float32(-127.0))
    q = np.rint(val).astype(np.int8)       # round-half-even == __float2int_rn
    return q, scale


def sage_quant_q(q: np.ndarray, qm: np.ndarray | None):
    """Per 32-token tile INT8 quantisation of (q - qm): amax = max(1e-7,|.|),
    scale = amax/127, q8 = rn_even(clamp(val*(1/scale), +-127)); scales
    [HN, ceil(L/128)*4] (src/core/backend/ggml/cuda/ed_cuda_sage_attn.cu:61-138)."""
    q8, sc = _sage_quant(q, qm, 32)
    L = q.shape[1]
    n_chunks = ((L + 127) // 128) * 4
    out = np.full((q.shape[0], n_chunks), np.float32(1e-7) / np.float32(127.0), dtype=np.float32)
    out[:, : sc.shape[1]] = sc
    return q8, out


def sage_quant_k(k: np.ndarray, km: np.ndarray | None):
    """Per 64-token block INT8 quantisation of (k - km); scales [HN, ceil(L/64)]
    (src/core/backend/ggml/cuda/ed_cuda_sage_attn.cu:144-204)."""
    return _sage_quant(k, km, 64)


def sage_smooth_q_bias(k: np.ndarray, qm: np.ndarray) -> np.ndarray:
    """bias[hn, j] = sum_d qm[hn,d] * K_orig[hn,j,d]; 32-lane xor-butterfly per
    warp then sequential over d/32 warps
    (src/core/backend/ggml/cuda/ed_cuda_sage_attn.cu:253-281)."""
    HN, L, d = k.shape
    part = (k.astype(np.float32) * qm[:, None, :]).astype(np.float32).reshape(HN, L, d // 32, 32)
    m = 16
    while m > 0:
        idx = np.arange(32) ^ m
        part = (part + part[..., idx]).astype(np.float32)
        m >>= 1
    total = np.zeros((HN, L), dtype=np.float32)
    for w in range(d // 32):
        total = (total + part[:, :, w, 0]).astype(np.float32)
    return total


def sage_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, smooth_q: bool = True,
                   scale: float | None = None) -> np.ndarray:
    """Numpy model of the Sage pipeline (src/core/backend/ggml/cuda/ed_cuda_sage_attn.cu:834-1122):
    smooth-K, optional smooth-Q with rank-1 bias, INT8 QK^T, f32 softmax, f16 P and V.
    q,k,v [HN, L, d] -> [HN, L, d] f32."""
    HN, L, d = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    km = sage_channel_mean(k)
    qm = sage_channel_mean(q) if smooth_q else None
    q8, qs = sage_quant_q(q, qm)
    k8, ks = sage_quant_k(k, km)
    bias = sage_smooth_q_bias(k, qm) if smooth_q else None
    qs_t = np.repeat(qs, 32, axis=1)[:, :L]
    ks_t = np.repeat(ks, 64, axis=1)[:, :L]
    vh = f16_round(v)
    out = np.empty((HN, L, d), dtype=np.float32)
    for h in range(HN):
        s_i = q8[h].astype(np.int32) @ k8[h].astype(np.int32).T
        s = s_i.astype(np.float32) * (qs_t[h][:, None] * ks_t[h][None, :])
        if bias is not None:
            s = s + bias[h][None, :]
        s = s * np.float32(scale)
        s = s - s.max(axis=1, keepdims=True)
        p = np.exp(s, dtype=np.float32)
        l = p.sum(axis=1, keepdims=True)
        out[h] = (f16_round(p) @ vh[h]) / l
    return out


# ----------------------------------------------------------------------------
# Layout glue
# ----------------------------------------------------------------------------


def patchify(x: np.ndarray, p: int = 2) -> np.ndarray:
    """latent [C, H, W] -> tokens [h*w, C*p*p], feature = c*p*p + py*p + px
    (DiT::patchify, patch_last=true, src/dit_models/components/common/common_dit.hpp:7-36)."""
    C, H, W = x.shape
    h, w = H // p, W // p
    t = x.reshape(C, h, p, w, p).transpose(1, 3, 0, 2, 4)
    return np.ascontiguousarray(t).reshape(h * w, C * p * p)


def unpatchify(t: np.ndarray, h: int, w: int, p: int = 2) -> np.ndarray:
    """tokens [h*w, C*p*p] -> [C, h*p, w*p]
    (DiT::unpatchify, src/dit_models/components/common/common_dit.hpp:38-64)."""
    C = t.shape[1] // (p * p)
    x = t.reshape(h, w, C, p, p).transpose(2, 0, 3, 1, 4)
    return np.ascontiguousarray(x).reshape(C, h * p, w * p)


# ----------------------------------------------------------------------------
# Error metrics used by the parity tests
# ----------------------------------------------------------------------------


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    return float(a @ b / max(np.linalg.norm(a) * np.linalg.norm(b), 1e-30))
