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

    # a file whose weights are in another block type is refused, by name
    other = FluxConfig(hidden_size=512, num_heads=4, depth=1, depth_single_blocks=1, context_in_dim=256, vec_in_dim=64,
                       wtype=O.GGML_TYPE_Q4_K)
    c = edb.FluxModel(hidden_size=512, num_heads=4, depth=1, depth_single_blocks=1, context_in_dim=256, vec_in_dim=64,
                      wtype=other.wtype)
    with pytest.raises(edb.EdbError) as ei:
        c.load_gguf(path)
    assert "convert the file first" in str(ei.value)


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
