"""Weight ingest: the library's GGUF and safetensors readers against files written by gguf-py and the
safetensors package (CPU), and models loaded from such files against the same model loaded tensor by
tensor (GPU)."""
import numpy as np
import pytest

from oracle import edb_oracle as O

gguf = pytest.importorskip("gguf")

_QT = {O.GGML_TYPE_Q8_0: "Q8_0", O.GGML_TYPE_Q4_K: "Q4_K"}


def write_gguf(path, weights, prefix="", extra_tensors=()):
    """weights: {name: (ggml_type, ndarray)} as the oracles make them (raw block bytes for
    quantised tensors, f32 otherwise).  Adds a few key/value pairs of every kind a reader must skip."""
    w = gguf.GGUFWriter(str(path), arch="flux")
    w.add_string("general.name", "edb200 test file")
    w.add_uint32("edb200.answer", 42)
    w.add_array("edb200.floats", [0.5, 1.5, 2.5])
    w.add_array("edb200.strings", ["a", "bc", "def"])
    for name, (t, arr) in list(weights.items()) + list(extra_tensors):
        a = np.ascontiguousarray(arr)
        if t in _QT:
            w.add_tensor(prefix + name, a.view(np.uint8), raw_dtype=getattr(gguf.GGMLQuantizationType, _QT[t]))
        else:
            w.add_tensor(prefix + name, a)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def _sample_weights():
    rng = np.random.default_rng(51)
    wq8 = rng.standard_normal((96, 256), dtype=np.float32) * np.float32(0.02)
    wq4 = rng.standard_normal((64, 512), dtype=np.float32) * np.float32(0.02)
    return {
        "blocks.0.linear.weight": (O.GGML_TYPE_Q8_0, O.quantize(wq8, O.GGML_TYPE_Q8_0)),
        "blocks.0.linear.bias": (O.GGML_TYPE_F32, rng.standard_normal(96, dtype=np.float32)),
        "blocks.1.proj.weight": (O.GGML_TYPE_Q4_K, O.quantize(wq4, O.GGML_TYPE_Q4_K)),
        "norm.scale": (O.GGML_TYPE_F32, rng.standard_normal(128, dtype=np.float32)),
    }


def test_reader_matches_gguf_py(edb, tmp_path):
    path = tmp_path / "w.gguf"
    weights = _sample_weights()
    half = np.arange(24, dtype=np.float16).reshape(4, 6)
    write_gguf(path, weights, prefix="model.diffusion_model.", extra_tensors=[("vae.half", (1, half))])
    ref = {t.name: t for t in gguf.GGUFReader(str(path)).tensors}
    f = edb.GGUF(path)
    assert len(f) == len(ref) == 5
    seen = set()
    for i in range(len(f)):
        name, t, dims, data = f.tensor(i)
        r = ref[name]
        seen.add(name)
        assert t == int(r.tensor_type)
        assert dims == tuple(int(d) for d in r.shape)          # ggml order: row length first
        assert data == r.data.tobytes()
    assert seen == set(ref)
    name, t, dims, data = [f.tensor(i) for i in range(len(f)) if f.tensor(i)[0].endswith("linear.weight")][0]
    assert (t, dims) == (O.GGML_TYPE_Q8_0, (256, 96)) and len(data) == 96 * 256 // 32 * 34
    f.close()


def test_reader_rejects_malformed_files(edb, tmp_path):
    good = tmp_path / "g.gguf"
    write_gguf(good, _sample_weights())
    raw = good.read_bytes()
    cases = {
        "magic": b"GGUX" + raw[4:],
        "version": raw[:4] + (9).to_bytes(4, "little") + raw[8:],
        "truncated table": raw[:200],
        "truncated data": raw[:-64],
        "short": raw[:10],
    }
    for what, blob in cases.items():
        p = tmp_path / "bad.gguf"
        p.write_bytes(blob)
        with pytest.raises(edb.EdbError):
            edb.GGUF(p)
    with pytest.raises(edb.EdbError):
        edb.GGUF(tmp_path / "missing.gguf")


@pytest.mark.gpu
def test_flux_loaded_from_gguf_equals_tensor_by_tensor_load(edb, cuda, tmp_path):
    import torch
    from oracle.flux_oracle import FluxConfig, flux_make_weights
    cfg = FluxConfig(hidden_size=512, num_heads=4, depth=1, depth_single_blocks=1, context_in_dim=256, vec_in_dim=64)
    weights = flux_make_weights(cfg, 17)
    # norm scales stored as f16 in the file (widened on load), an unrelated tensor to skip
    stored = dict(weights)
    k = "double_blocks.0.img_attn.norm.query_norm.scale"
    as_half = weights[k][1].astype(np.float16)
    stored[k] = (1, as_half)
    weights[k] = (O.GGML_TYPE_F32, as_half.astype(np.float32))
    path = tmp_path / "flux.gguf"
    write_gguf(path, stored, prefix="model.diffusion_model.",
               extra_tensors=[("first_stage_model.decoder.w", (O.GGML_TYPE_F32, np.ones(8, dtype=np.float32)))])

    def make():
        return edb.FluxModel(hidden_size=cfg.hidden_size, num_heads=cfg.num_heads, depth=cfg.depth,
                             depth_single_blocks=cfg.depth_single_blocks, mlp_hidden=cfg.mlp_hidden,
                             in_channels=cfg.in_channels, context_in_dim=cfg.context_in_dim,
                             vec_in_dim=cfg.vec_in_dim, axes_dim=cfg.axes_dim, wtype=cfg.wtype)
    a, b = make(), make()
    a.load_numpy(weights)
    assert b.load_gguf(path) == len(weights)
    rng = np.random.default_rng(3)
    lat = torch.from_numpy(rng.standard_normal((16, 16, 16), dtype=np.float32)).to(cuda)
    ctx = torch.from_numpy(rng.standard_normal((12, 256), dtype=np.float32)).to(cuda)
    y = torch.from_numpy(rng.standard_normal(64, dtype=np.float32)).to(cuda)
    outs = []
    for m in (a, b):
        m.prepare(16, 16, 12)
        out = torch.empty_like(lat)
        m.step(lat, 0.5, ctx, y, 3.5, out)
        torch.cuda.synchronize()
        outs.append(out.cpu().numpy())
    assert np.isfinite(outs[0]).all()
    assert np.array_equal(outs[0], outs[1])


# ------------------------------------------------------------------ safetensors

def test_safetensors_reader_matches_the_safetensors_package(edb, tmp_path):
    st = pytest.importorskip("safetensors.numpy")
    rng = np.random.default_rng(61)
    tensors = {
        "model.diffusion_model.a.weight": rng.standard_normal((12, 64), dtype=np.float32),
        "model.diffusion_model.a.bias": rng.standard_normal(12, dtype=np.float32).astype(np.float16),
        "other.ids": np.arange(10, dtype=np.int64),
        "scalar": np.array(3.5, dtype=np.float32),
    }
    path = tmp_path / "w.safetensors"
    st.save_file(tensors, str(path), metadata={"format": "pt", "note": "braces } and [ in \"strings\""})
    f = edb.SafeTensors(path)
    assert len(f) == len(tensors)
    names = {"float32": "F32", "float16": "F16", "int64": "I64"}
    seen = set()
    for i in range(len(f)):
        name, dtype, shape, data = f.tensor(i)
        a = tensors[name]
        seen.add(name)
        assert dtype == names[a.dtype.name]
        assert shape == a.shape
        assert data == a.tobytes()
    assert seen == set(tensors)
    f.close()


def test_safetensors_reader_rejects_malformed_files(edb, tmp_path):
    st = pytest.importorskip("safetensors.numpy")
    good = tmp_path / "g.safetensors"
    st.save_file({"w": np.ones((4, 8), dtype=np.float32)}, str(good))
    raw = good.read_bytes()
    hlen = int.from_bytes(raw[:8], "little")
    header = raw[8:8 + hlen]
    cases = {
        "header length": (hlen + 10_000).to_bytes(8, "little") + raw[8:],
        "truncated data": raw[:-16],
        "not json": raw[:8] + b"[" + header[1:] + raw[8 + hlen:],
        "offsets": raw[:8] + header.replace(b"128", b"124") + raw[8 + hlen:],
        "short": raw[:6],
    }
    assert b"128" in header
    for what, blob in cases.items():
        p = tmp_path / "bad.safetensors"
        p.write_bytes(blob)
        with pytest.raises(edb.EdbError):
            edb.SafeTensors(p)


@pytest.mark.gpu
def test_flux_loaded_from_safetensors_quantises_like_ggml(edb, cuda, tmp_path):
    """An unquantised checkpoint: the loader encodes q8_0 on the device by ggml's rule, so the model
    equals one given the oracle's q8_0 blocks of the same f32 weights."""
    import torch
    st = pytest.importorskip("safetensors.numpy")
    from oracle.flux_oracle import FluxConfig, flux_tensor_specs, _name_seed
    cfg = FluxConfig(hidden_size=512, num_heads=4, depth=1, depth_single_blocks=1, context_in_dim=256, vec_in_dim=64)
    f32, blocks = {}, {}
    for name, shape, quant in flux_tensor_specs(cfg):
        rng = np.random.Generator(np.random.Philox(_name_seed(23, name)))
        w = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        if name.endswith(".scale"):
            w = (w + np.float32(1.0)).astype(np.float32)
        f32["model.diffusion_model." + name] = w
        blocks[name] = (cfg.wtype, O.quantize(w, cfg.wtype)) if quant else (O.GGML_TYPE_F32, w)
    path = tmp_path / "flux.safetensors"
    st.save_file(f32, str(path))

    def make():
        return edb.FluxModel(hidden_size=cfg.hidden_size, num_heads=cfg.num_heads, depth=cfg.depth,
                             depth_single_blocks=cfg.depth_single_blocks, mlp_hidden=cfg.mlp_hidden,
                             in_channels=cfg.in_channels, context_in_dim=cfg.context_in_dim,
                             vec_in_dim=cfg.vec_in_dim, axes_dim=cfg.axes_dim, wtype=cfg.wtype)
    a, b = make(), make()
    a.load_numpy(blocks)
    assert b.load_safetensors(path) == len(blocks)
    rng = np.random.default_rng(4)
    lat = torch.from_numpy(rng.standard_normal((16, 16, 16), dtype=np.float32)).to(cuda)
    ctx = torch.from_numpy(rng.standard_normal((12, 256), dtype=np.float32)).to(cuda)
    y = torch.from_numpy(rng.standard_normal(64, dtype=np.float32)).to(cuda)
    outs = []
    for m in (a, b):
        m.prepare(16, 16, 12)
        out = torch.empty_like(lat)
        m.step(lat, 0.5, ctx, y, 3.5, out)
        torch.cuda.synchronize()
        outs.append(out.cpu().numpy())
    assert np.isfinite(outs[0]).all()
    assert np.array_equal(outs[0], outs[1])


def test_safetensors_index_lists_each_shard_once(edb, tmp_path):
    import json
    index = tmp_path / "diffusion_pytorch_model.safetensors.index.json"
    index.write_text(json.dumps({
        "metadata": {"total_size": 123, "note": "a } brace"},
        "weight_map": {
            "a.weight": "diffusion_pytorch_model-00001-of-00002.safetensors",
            "a.bias": "diffusion_pytorch_model-00001-of-00002.safetensors",
            "b.weight": "diffusion_pytorch_model-00002-of-00002.safetensors",
        },
    }, indent=2))
    files = edb.safetensors_index_files(index)
    assert files == [str(tmp_path / "diffusion_pytorch_model-00001-of-00002.safetensors"),
                     str(tmp_path / "diffusion_pytorch_model-00002-of-00002.safetensors")]
    for bad in ({"weight_map": {"a": "../escape.safetensors"}}, {"weight_map": {}}, {"metadata": {}}, [1, 2]):
        index.write_text(json.dumps(bad))
        with pytest.raises(edb.EdbError):
            edb.safetensors_index_files(index)


# ------------------------------------------------------------------ names, fused tensors, other storage types


def _golden_names():
    import json
    import os
    with open(os.path.join(os.path.dirname(__file__), "golden", "tensor_names.json")) as f:
        return json.load(f)


_FAMILY = {"flux": 0, "sd3": 1, "qwen": 2, "wan": 3}


def _joined(edb, family, name):
    base, part = edb.canonical_tensor_name(_FAMILY[family], name)
    return base if part == 0 else f"{base}.{part}"


def test_canonical_names_equal_the_reference_conversion(edb):
    """Golden vectors: the reference's convert_diffusion_model_name on diffusers-layout names of the four
    families (tests/golden/make_names_golden.py).  The part index is the reference's numeric suffix."""
    golden = _golden_names()
    assert set(golden) == set(_FAMILY)
    for family, rows in golden.items():
        assert len(rows) > 40
        for name, want in rows:
            assert _joined(edb, family, name) == want, (family, name)
    assert edb.canonical_tensor_name(0, "single_transformer_blocks.4.proj_mlp.weight") == ("single_blocks.4.linear1.weight", 3)
    assert edb.canonical_tensor_name(1, "transformer_blocks.2.attn.add_k_proj.bias") == (
        "joint_blocks.2.context_block.attn.qkv.bias", 1)
    # an explicit part suffix is split off whatever the family
    assert edb.canonical_tensor_name(2, "some.linear.weight.2") == ("some.linear.weight", 2)
    with pytest.raises(edb.EdbError):
        edb.canonical_tensor_name(9, "x")


def test_canonical_names_equal_the_compiled_reference(edb):
    """The same against the reference's conversion compiled here, where that library was built, on every
    block index (the golden file samples a few)."""
    import ctypes
    import os
    so = os.path.join(os.path.dirname(os.path.dirname(__file__)), "oracle", "_ref", "libedref_names.so")
    if not os.path.exists(so):
        pytest.skip("oracle/_ref/libedref_names.so not built")
    ref = ctypes.CDLL(so)
    buf = ctypes.create_string_buffer(1024)
    golden = _golden_names()
    import re
    checked = 0
    for family, rows in golden.items():
        depth = {"flux": 19, "sd3": 38, "qwen": 60, "wan": 40}[family]
        for name, _ in rows:
            m = re.match(r"^(transformer_blocks|blocks)\.0\.(.*)$", name)
            variants = [name] if not m else [f"{m.group(1)}.{i}.{m.group(2)}" for i in range(depth)]
            for v in variants:
                assert ref.ref_convert_diffusion_name(_FAMILY[family], v.encode(), buf, 1024) == 0
                assert _joined(edb, family, v) == buf.value.decode(), (family, v)
                checked += 1
    assert checked > 2000


def _flux_small():
    from oracle.flux_oracle import FluxConfig
    return FluxConfig(hidden_size=512, num_heads=4, depth=2, depth_single_blocks=2, context_in_dim=256, vec_in_dim=64)


def _flux_model(edb, cfg, wtype=None):
    return edb.FluxModel(hidden_size=cfg.hidden_size, num_heads=cfg.num_heads, depth=cfg.depth,
                         depth_single_blocks=cfg.depth_single_blocks, mlp_hidden=cfg.mlp_hidden,
                         in_channels=cfg.in_channels, context_in_dim=cfg.context_in_dim, vec_in_dim=cfg.vec_in_dim,
                         axes_dim=cfg.axes_dim, wtype=cfg.wtype if wtype is None else wtype)


def _flux_f32_weights(cfg, seed):
    from oracle.flux_oracle import flux_tensor_specs, _name_seed
    out = {}
    for name, shape, quant in flux_tensor_specs(cfg):
        rng = np.random.Generator(np.random.Philox(_name_seed(seed, name)))
        w = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        if name.endswith(".scale"):
            w = (w + np.float32(1.0)).astype(np.float32)
        out[name] = (w, quant)
    return out


def _to_diffusers_flux(f32, hidden):
    """The executors' FLUX tensors under their diffusers names, fused tensors cut into their projections
    (the inverse of the golden name table)."""
    import re
    golden = _golden_names()["flux"]
    inverse = {}   # name with block index 0 -> [(part, diffusers name)]
    for src, dst in golden:
        m = re.match(r"^(.*\.(?:weight|bias))\.(\d+)$", dst)
        base, part = (m.group(1), int(m.group(2))) if m else (dst, 0)
        if src != dst:
            inverse.setdefault(base, []).append((part, src))
    out = {}
    for name, (w, _) in f32.items():
        m = re.match(r"^(double_blocks|single_blocks)\.(\d+)\.(.*)$", name)
        key = f"{m.group(1)}.0.{m.group(3)}" if m else name
        parts = sorted(inverse[key])

        def rename(n):
            if not m:
                return n
            scope = "transformer_blocks" if m.group(1) == "double_blocks" else "single_transformer_blocks"
            return re.sub(r"^(single_)?transformer_blocks\.0\.", f"{scope}.{m.group(2)}.", n)
        if len(parts) == 1:
            out[rename(parts[0][1])] = w
            continue
        at = 0
        for part, src in parts:   # q, k, v take `hidden` rows each, the MLP projection the rest
            n = hidden if part < 3 else w.shape[0] - 3 * hidden
            out[rename(src)] = np.ascontiguousarray(w[at:at + n])
            at += n
        assert at == w.shape[0]
    return out


def _assert_same_tensors(a, b, names):
    for name in names:
        assert np.array_equal(a.get_tensor(name), b.get_tensor(name)), name


@pytest.mark.gpu
def test_flux_diffusers_layout_checkpoint_is_renamed_and_fused(edb, cuda, tmp_path):
    """A sharded safetensors checkpoint in the diffusers layout (q / k / v / mlp projections as separate
    tensors, in shuffled order, the parts of one tensor in different shards) loads into the same model as
    the fused tensors given one by one."""
    import json
    st = pytest.importorskip("safetensors.numpy")
    cfg = _flux_small()
    f32 = _flux_f32_weights(cfg, 31)
    blocks = {n: ((cfg.wtype, O.quantize(w, cfg.wtype)) if q else (O.GGML_TYPE_F32, w)) for n, (w, q) in f32.items()}
    diff = _to_diffusers_flux(f32, cfg.hidden_size)
    assert "transformer_blocks.1.attn.to_k.weight" in diff and "single_transformer_blocks.1.proj_mlp.bias" in diff
    names = sorted(diff)
    np.random.default_rng(5).shuffle(names)
    shards = [names[0::2], names[1::2]]
    weight_map = {}
    for i, shard in enumerate(shards):
        fname = f"diffusion_pytorch_model-{i + 1:05d}-of-00002.safetensors"
        # half of the tensors as bf16-representable f16 would change the values: store f32 throughout
        st.save_file({n: diff[n] for n in shard}, str(tmp_path / fname))
        weight_map.update({n: fname for n in shard})
    index = tmp_path / "diffusion_pytorch_model.safetensors.index.json"
    index.write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    a, b = _flux_model(edb, cfg), _flux_model(edb, cfg)
    a.load_numpy(blocks)
    assert b.load_safetensors(index, strip_prefix="") == len(blocks)
    _assert_same_tensors(a, b, blocks)

    # one projection missing: the fused tensor is reported by name
    broken = {n: diff[n] for n in names if n != "transformer_blocks.0.attn.to_v.weight"}
    st.save_file(broken, str(tmp_path / "broken.safetensors"))
    c = _flux_model(edb, cfg)
    with pytest.raises(edb.EdbError) as ei:
        c.load_safetensors(tmp_path / "broken.safetensors", strip_prefix="")
    assert "double_blocks.0.img_attn.qkv.weight" in str(ei.value) and "incomplete" in str(ei.value)


@pytest.mark.gpu
def test_gguf_in_other_storage_types_is_converted(edb, cuda, tmp_path):
    """convert_tensor_data: f16 and q8_0 files into a q4_K model, a q4_K file into a q8_0 model (dequantise,
    then encode in the model's type), and pre-quantised q8_0 projections of the diffusers layout
    concatenated block-wise into the fused tensor."""
    cfg = _flux_small()
    f32 = _flux_f32_weights(cfg, 37)
    q8 = {n: ((O.GGML_TYPE_Q8_0, O.quantize(w, O.GGML_TYPE_Q8_0)) if q else (O.GGML_TYPE_F32, w)) for n, (w, q) in f32.items()}
    q4 = {n: ((O.GGML_TYPE_Q4_K, O.quantize(w, O.GGML_TYPE_Q4_K)) if q else (O.GGML_TYPE_F32, w)) for n, (w, q) in f32.items()}
    quantised = [n for n, (_, q) in f32.items() if q]

    def reencoded(blocks, src_type, dst_type):
        out = {}
        for n, (t, arr) in blocks.items():
            if t == src_type:
                w = O.dequantize(arr, src_type).reshape(f32[n][0].shape)
                out[n] = (dst_type, O.quantize(w.astype(np.float32), dst_type))
            else:
                out[n] = (t, arr)
        return out

    # q8_0 file -> q4_K model
    write_gguf(tmp_path / "q8.gguf", q8)
    want = _flux_model(edb, cfg, O.GGML_TYPE_Q4_K)
    want.load_numpy(reencoded(q8, O.GGML_TYPE_Q8_0, O.GGML_TYPE_Q4_K))
    got = _flux_model(edb, cfg, O.GGML_TYPE_Q4_K)
    assert got.load_gguf(tmp_path / "q8.gguf", strip_prefix="") == len(q8)
    _assert_same_tensors(want, got, q8)

    # q4_K file -> q8_0 model
    write_gguf(tmp_path / "q4.gguf", q4)
    want = _flux_model(edb, cfg, O.GGML_TYPE_Q8_0)
    want.load_numpy(reencoded(q4, O.GGML_TYPE_Q4_K, O.GGML_TYPE_Q8_0))
    got = _flux_model(edb, cfg, O.GGML_TYPE_Q8_0)
    assert got.load_gguf(tmp_path / "q4.gguf", strip_prefix="") == len(q4)
    _assert_same_tensors(want, got, q4)

    # f16 file -> q8_0 model
    halves = {n: ((1, w.astype(np.float16)) if q else (O.GGML_TYPE_F32, w)) for n, (w, q) in f32.items()}
    write_gguf(tmp_path / "f16.gguf", halves)
    from_half = {n: ((O.GGML_TYPE_Q8_0, O.quantize(w.astype(np.float16).astype(np.float32), O.GGML_TYPE_Q8_0)) if q
                     else (O.GGML_TYPE_F32, w)) for n, (w, q) in f32.items()}
    want = _flux_model(edb, cfg, O.GGML_TYPE_Q8_0)
    want.load_numpy(from_half)
    got = _flux_model(edb, cfg, O.GGML_TYPE_Q8_0)
    assert got.load_gguf(tmp_path / "f16.gguf", strip_prefix="") == len(halves)
    _assert_same_tensors(want, got, halves)

    # diffusers layout, projections already q8_0: the fused tensor is their blocks back to back
    diff = _to_diffusers_flux(f32, cfg.hidden_size)
    stored = {}
    for n, w in diff.items():
        is_q = w.ndim == 2 and w.shape[1] % 32 == 0 and any(
            n.endswith(s) for s in ("to_q.weight", "to_k.weight", "to_v.weight", "proj_mlp.weight", "add_q_proj.weight",
                                    "add_k_proj.weight", "add_v_proj.weight"))
        stored[n] = (O.GGML_TYPE_Q8_0, O.quantize(w, O.GGML_TYPE_Q8_0)) if is_q else (O.GGML_TYPE_F32, w)
    write_gguf(tmp_path / "diff.gguf", stored)
    want = _flux_model(edb, cfg, O.GGML_TYPE_Q8_0)
    want.load_numpy(q8)
    got = _flux_model(edb, cfg, O.GGML_TYPE_Q8_0)
    assert got.load_gguf(tmp_path / "diff.gguf", strip_prefix="") == len(q8)
    _assert_same_tensors(want, got, q8)
    assert len(quantised) > 10
