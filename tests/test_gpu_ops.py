"""GPU parity tests of the C-ABI ops against the numpy oracle (same seeded inputs)."""
import ctypes as C

import numpy as np
import pytest

from oracle import edb_oracle as O

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


_KEEP = []


def dev(a, device):
    """Upload to the device and keep the tensor alive until the test ends: the C
    ABI takes raw pointers, so a temporary freed by Python could be reused by the
    caching allocator while a kernel still reads it."""
    t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
    _KEEP.append(t)
    return t


@pytest.fixture(autouse=True)
def _release_device_temporaries():
    yield
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    _KEEP.clear()


def sync_check(edb):
    torch.cuda.synchronize()


# ---------------------------------------------------------------- codecs --

@pytest.mark.parametrize("rows,k", [(1, 32), (3, 256), (130, 3072)])
def test_dequantize_q8_0_bit_exact(edb, cuda, rows, k):
    x = np.random.default_rng(1).standard_normal((rows, k), dtype=np.float32) * np.float32(0.02)
    blocks = O.q8_0_quantize(x)
    out = torch.empty(rows, k, dtype=torch.float32, device=cuda)
    edb.check(edb.lib().edb200_dequantize_rows(edb.TYPE_Q8_0, edb.ptr(dev(blocks, cuda)), edb.ptr(out), rows, k,
                                               edb.current_stream()))
    ref = O.q8_0_dequantize(blocks)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("rows,k", [(1, 256), (33, 3072)])
def test_dequantize_q4_k_bit_exact(edb, cuda, rows, k):
    x = np.random.default_rng(2).standard_normal((rows, k), dtype=np.float32) * np.float32(0.02)
    blocks = O.q4_k_quantize(x)
    out = torch.empty(rows, k, dtype=torch.float32, device=cuda)
    edb.check(edb.lib().edb200_dequantize_rows(edb.TYPE_Q4_K, edb.ptr(dev(blocks, cuda)), edb.ptr(out), rows, k,
                                               edb.current_stream()))
    ref = O.q4_k_dequantize(blocks)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("rows,k", [(1, 32), (65, 3072)])
def test_quantize_q8_0_bit_exact(edb, cuda, rows, k):
    x = np.random.default_rng(3).standard_normal((rows, k), dtype=np.float32) * np.float32(0.02)
    x[0, :32] = 0.0
    x[0, 1] = 0.0
    out = torch.empty(rows, k // 32 * 34, dtype=torch.uint8, device=cuda)
    edb.check(edb.lib().edb200_quantize_rows_q8_0(edb.ptr(dev(x, cuda)), edb.ptr(out), rows, k,
                                                  edb.current_stream()))
    assert np.array_equal(out.cpu().numpy(), O.q8_0_quantize(x))


@pytest.mark.parametrize("wtype", ["q8_0", "q4_k"])
def test_repack_preserves_values(edb, cuda, wtype):
    n_out, k = 520, 1024   # n_out not a multiple of 256: exercises the padded scale plane
    x = np.random.default_rng(4).standard_normal((n_out, k), dtype=np.float32) * np.float32(0.02)
    t = edb.TYPE_Q8_0 if wtype == "q8_0" else edb.TYPE_Q4_K
    blocks = O.quantize(x, t)
    w = edb.QWeight(t, dev(blocks, cuda), n_out, k)
    out = torch.empty(n_out, k, dtype=torch.float32, device=cuda)
    edb.check(edb.lib().edb200_qweight_dequantize(w.handle, edb.ptr(out), edb.current_stream()))
    ref = O.dequantize(blocks, t)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))


def test_fill_normal_statistics(edb, cuda):
    n = 1 << 20
    out = torch.empty(n, dtype=torch.float32, device=cuda)
    edb.check(edb.lib().edb200_fill_normal(edb.ptr(out), n, 1234, 0.0, 0.02, edb.current_stream()))
    v = out.cpu().numpy()
    assert abs(v.mean()) < 2e-4 and abs(v.std() - 0.02) < 2e-4 and np.isfinite(v).all()


# ----------------------------------------------------------- elementwise --

def test_fused_modulate_bit_exact(edb, cuda):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((77, 1536), dtype=np.float32)
    sh = rng.standard_normal(1536, dtype=np.float32)
    sc = rng.standard_normal(1536, dtype=np.float32)
    y = torch.empty(77, 1536, dtype=torch.float32, device=cuda)
    edb.check(edb.lib().edb200_fused_modulate(edb.ptr(dev(x, cuda)), edb.ptr(dev(sh, cuda)), edb.ptr(dev(sc, cuda)),
                                              edb.ptr(y), 77, 1536, edb.current_stream()))
    assert np.array_equal(y.cpu().numpy().view(np.uint32), O.modulate(x, sh[None], sc[None]).view(np.uint32))


def test_fused_residual_gate_bit_exact(edb, cuda):
    rng = np.random.default_rng(6)
    r = rng.standard_normal((77, 1536), dtype=np.float32)
    x = rng.standard_normal((77, 1536), dtype=np.float32)
    g = rng.standard_normal(1536, dtype=np.float32)
    y = torch.empty(77, 1536, dtype=torch.float32, device=cuda)
    edb.check(edb.lib().edb200_fused_residual_gate(edb.ptr(dev(r, cuda)), edb.ptr(dev(x, cuda)),
                                                   edb.ptr(dev(g, cuda)), edb.ptr(y), 77, 1536,
                                                   edb.current_stream()))
    assert np.array_equal(y.cpu().numpy().view(np.uint32), O.residual_gate(r, x, g[None]).view(np.uint32))


@pytest.mark.parametrize("sigma,sigma_next", [(1.0, 0.9), (0.37, 0.0), (0.0, 0.0), (0.0123, 0.0045)])
def test_euler_update_bit_exact(edb, cuda, sigma, sigma_next):
    rng = np.random.default_rng(31)
    x = rng.standard_normal(16 * 33 * 47, dtype=np.float32)
    v = rng.standard_normal(x.size, dtype=np.float32)
    dx = dev(x, cuda)
    edb.euler_update(dx, dev(v, cuda), sigma, sigma_next)
    want = O.euler_update(x, v, sigma, sigma_next)
    assert np.array_equal(dx.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # SD3's form: x += model_out * (sigma_next - sigma)
    dx = dev(x, cuda)
    edb.check(edb.lib().edb200_flow_update(edb.ptr(dx), edb.ptr(dev(v, cuda)), sigma, sigma_next, x.size,
                                           edb.current_stream()))
    dt = np.float32(np.float32(sigma_next) - np.float32(sigma))
    want = (x + (v * dt).astype(np.float32)).astype(np.float32)
    assert np.array_equal(dx.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("h,dt", [(3072, "bf16"), (1536, "f32"), (5120, "f16")])
def test_layernorm_modulate(edb, cuda, h, dt):
    rng = np.random.default_rng(7)
    rows = 37
    x = (rng.standard_normal((rows, h), dtype=np.float32) * 3 + 1).astype(np.float32)
    sh = rng.standard_normal(h, dtype=np.float32) * 0.1
    sc = rng.standard_normal(h, dtype=np.float32) * 0.1
    tdt = {"bf16": torch.bfloat16, "f32": torch.float32, "f16": torch.float16}[dt]
    y = torch.empty(rows, h, dtype=tdt, device=cuda)
    edb.check(edb.lib().edb200_layernorm_modulate(edb.ptr(dev(x, cuda)), h, edb.ptr(dev(sh, cuda)),
                                                  edb.ptr(dev(sc, cuda)), None, None, rows, h, 1e-6, edb.ptr(y),
                                                  edb.torch_dtype_id(y), h, edb.current_stream()))
    ref = O.modulate(O.layer_norm(x, 1e-6), sh[None], sc[None])
    got = y.float().cpu().numpy()
    tol = {"bf16": 6e-3, "f32": 2e-6, "f16": 8e-4}[dt]
    assert O.rel_l2(got, ref) < tol


@pytest.mark.parametrize("d,in_dt", [(128, "bf16"), (64, "f32")])
def test_qk_norm_rope_pack(edb, cuda, d, in_dt):
    rng = np.random.default_rng(8)
    T, Hh, nt = 50, 3, 6           # 50 tokens written at offset 6 of a 64-token joint sequence
    L = 64
    hid = Hh * d
    qkv = rng.standard_normal((T, 3 * hid + 16), dtype=np.float32)
    if in_dt == "bf16":
        qkv = O.bf16_round(qkv)
    qw = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    kw = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    axes = (16, 56, 56) if d == 128 else (16, 24, 24)
    ids = rng.integers(0, 40, size=(L, 3)).astype(np.float32)
    pe = O.embed_nd(ids, axes, 10000.0)
    tq = dev(qkv, cuda)
    if in_dt == "bf16":
        tq = tq.to(torch.bfloat16)
    outs = [torch.zeros(Hh, L, d, dtype=torch.float32, device=cuda) for _ in range(3)]
    edb.check(edb.lib().edb200_qk_norm_rope_pack(edb.ptr(tq), edb.torch_dtype_id(tq), qkv.shape[1], 0, hid, 2 * hid,
                                                 T, Hh, d, edb.ptr(dev(qw, cuda)), edb.ptr(dev(kw, cuda)), 1e-6,
                                                 edb.ptr(dev(pe, cuda)), nt, L, edb.ptr(outs[0]), edb.ptr(outs[1]),
                                                 edb.ptr(outs[2]), edb.TYPE_F32, edb.current_stream()))
    q = qkv[:, :hid].reshape(T, Hh, d)
    k = qkv[:, hid:2 * hid].reshape(T, Hh, d)
    v = qkv[:, 2 * hid:3 * hid].reshape(T, Hh, d)
    rq = O.apply_rope(O.rms_norm(q, qw), pe[nt:nt + T]).transpose(1, 0, 2)
    rk = O.apply_rope(O.rms_norm(k, kw), pe[nt:nt + T]).transpose(1, 0, 2)
    got = [o.cpu().numpy() for o in outs]
    assert O.rel_l2(got[0][:, nt:nt + T], rq) < 2e-6
    assert O.rel_l2(got[1][:, nt:nt + T], rk) < 2e-6
    assert np.array_equal(got[2][:, nt:nt + T], v.transpose(1, 0, 2))
    assert not got[0][:, :nt].any() and not got[0][:, nt + T:].any()   # rows outside the window untouched


# ------------------------------------------------------- gemv / linear ----

@pytest.mark.parametrize("wtype,m", [("q8_0", 1), ("q8_0", 2), ("q4_k", 1)])
def test_gemv_q(edb, cuda, wtype, m):
    n_out, k = 1000 if wtype == "q8_0" else 1024, 3072
    rng = np.random.default_rng(9)
    t = edb.TYPE_Q8_0 if wtype == "q8_0" else edb.TYPE_Q4_K
    blocks = O.quantize(rng.standard_normal((n_out, k), dtype=np.float32) * np.float32(0.02), t)
    w = edb.QWeight(t, dev(blocks, cuda), n_out, k)
    x = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal(n_out, dtype=np.float32)
    y = torch.empty(m, n_out, dtype=torch.float32, device=cuda)
    edb.check(edb.lib().edb200_gemv_q(w.handle, edb.ptr(dev(x, cuda)), m, k, 1, edb.ptr(dev(b, cuda)), edb.ptr(y),
                                      n_out, edb.current_stream()))
    ref = O.linear(O.silu(x), O.dequantize(blocks, t), b)
    assert O.rel_l2(y.cpu().numpy(), ref) < (2e-3 if wtype == "q4_k" else 1e-5)


@pytest.mark.parametrize("m,k,n,act", [(1, 256, 3072, 2), (300, 64, 200, 0), (70, 4096, 128, 1),
                                         (512, 4096, 3072, 0),   # FLUX txt_in: tiled kernel, full tiles
                                         (130, 48, 64, 0),       # ragged m, one partial n tile, k tail
                                         (4096, 64, 3072, 0),    # FLUX img_in: two k steps
                                         (200, 3072, 64, 2),     # final linear: fewer features than a tile
                                         (20, 256, 96, 0),       # a sequence-parallel rank with few rows
                                         (77, 24, 200, 3)])      # k not a multiple of 16: simple kernel
def test_linear_f32(edb, cuda, m, k, n, act):
    rng = np.random.default_rng(10)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)
    b = rng.standard_normal(n, dtype=np.float32)
    x = rng.standard_normal((m, k), dtype=np.float32)
    y = torch.empty(m, n, dtype=torch.float32, device=cuda)
    edb.check(edb.lib().edb200_linear_f32(edb.ptr(dev(w, cuda)), edb.ptr(dev(b, cuda)), edb.ptr(dev(x, cuda)), m, k,
                                          n, k, 0, act, edb.ptr(y), n, edb.current_stream()))
    ref = O.linear(x, w, b)
    from oracle.wan_oracle import gelu_erf
    ref = {0: lambda v: v, 1: O.gelu_tanh, 2: O.silu, 3: gelu_erf}[act](ref)
    # more than 8 rows go through the tensor cores, which read the f32 operands as tf32 (10 mantissa bits)
    tensor_cores = m > 8 and n >= 32 and k >= 32 and k % 4 == 0
    assert O.rel_l2(y.cpu().numpy(), ref) < (1e-3 if tensor_cores else 1e-5)


# ------------------------------------------------------ quantised GEMM ----

def _gemm_case(edb, cuda, wtype, m, n_out, k, x_dt, seed=11):
    rng = np.random.default_rng(seed)
    t = edb.TYPE_Q8_0 if wtype == "q8_0" else edb.TYPE_Q4_K
    wf = rng.standard_normal((n_out, k), dtype=np.float32) * np.float32(0.02)
    blocks = O.quantize(wf, t)
    w = edb.QWeight(t, dev(blocks, cuda), n_out, k)
    x = rng.standard_normal((m, k), dtype=np.float32)
    xt = dev(x, cuda).to(x_dt)
    xr = xt.float().cpu().numpy()
    return w, xt, xr, O.dequantize(blocks, t), rng


@pytest.mark.parametrize("wtype,m,n_out,k,x_dt", [
    ("q8_0", 128, 256, 64, torch.float16),
    ("q8_0", 128, 256, 256, torch.float16),
    ("q8_0", 300, 768, 3072, torch.float16),      # ragged m, several k stages, 3 column tiles
    ("q8_0", 1000, 2048, 1024, torch.float16),    # more tiles than one wave of a small grid
    ("q4_k", 128, 256, 256, torch.float16),
    ("q4_k", 333, 512, 3072, torch.float16),
])
def test_mul_mat_q_plain(edb, cuda, wtype, m, n_out, k, x_dt):
    w, xt, xr, wd, _ = _gemm_case(edb, cuda, wtype, m, n_out, k, x_dt)
    y = torch.zeros(m, n_out, dtype=torch.float32, device=cuda)
    edb.mul_mat_q(w, xt, edb.make_epilogue(y))
    torch.cuda.synchronize()
    ref = xr @ wd.T
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    assert O.rel_l2(got, ref) < 2e-3, f"rel_l2={O.rel_l2(got, ref)}"
    assert O.cosine(got, ref) > 0.9999


def test_mul_mat_q_bias_gelu_bf16_out(edb, cuda):
    m, n_out, k = 200, 512, 512
    w, xt, xr, wd, rng = _gemm_case(edb, cuda, "q8_0", m, n_out, k, torch.float16, seed=12)
    b = rng.standard_normal(n_out, dtype=np.float32)
    y = torch.zeros(m, n_out, dtype=torch.bfloat16, device=cuda)
    edb.mul_mat_q(w, xt, edb.make_epilogue(y, bias=dev(b, cuda), act=edb.ACT_GELU_TANH))
    ref = O.gelu_tanh(xr @ wd.T + b)
    assert O.rel_l2(y.float().cpu().numpy(), ref) < 8e-3


def test_mul_mat_q_gated_residual_in_place(edb, cuda):
    m, n_out, k = 260, 768, 1024
    w, xt, xr, wd, rng = _gemm_case(edb, cuda, "q8_0", m, n_out, k, torch.float16, seed=13)
    b = rng.standard_normal(n_out, dtype=np.float32)
    g = rng.standard_normal(n_out, dtype=np.float32)
    res = rng.standard_normal((m, n_out), dtype=np.float32)
    stream = dev(res, cuda)
    edb.mul_mat_q(w, xt, edb.make_epilogue(stream, bias=dev(b, cuda), residual=stream, gate=dev(g, cuda)))
    ref = res + g[None] * (xr @ wd.T + b)
    assert O.rel_l2(stream.cpu().numpy(), ref) < 2e-3


@pytest.mark.parametrize("wtype,m,n_out,k", [("q8_0", 260, 768, 8192),     # 6 tiles -> 4 reduction parts
                                              ("q4_k", 576, 3072, 15360),   # a FLUX out-projection on 1/8 of the tokens
                                              ("q8_0", 100, 256, 12288)])   # 192 k-steps: 4 parts of 48
def test_mul_mat_q_split_reduction(edb, cuda, wtype, m, n_out, k):
    # few output tiles and a long reduction: on request the launch cuts k into parts that add
    # into the residual stream with atomics; the result must still be the gated residual
    w, xt, xr, wd, rng = _gemm_case(edb, cuda, wtype, m, n_out, k, torch.float16, seed=15)
    b = rng.standard_normal(n_out, dtype=np.float32)
    g = rng.standard_normal(n_out, dtype=np.float32)
    res = rng.standard_normal((m, n_out), dtype=np.float32)
    stream = dev(res, cuda)
    launches = edb.lib().edb200_launch_count()
    edb.mul_mat_q(w, xt, edb.make_epilogue(stream, bias=dev(b, cuda), residual=stream, gate=dev(g, cuda),
                                           split_k=edb.SPLIT_K_UNORDERED))
    assert edb.lib().edb200_launch_count() == launches + 1, "a split reduction is still one kernel"
    ref = res + g[None] * (xr @ wd.T + b)
    got = stream.cpu().numpy()
    assert np.isfinite(got).all()
    assert O.rel_l2(got, ref) < 2e-3, O.rel_l2(got, ref)
    # without the request the same call sums every output in one fixed order: same bits twice
    outs = []
    for _ in range(2):
        stream = dev(res, cuda)
        edb.mul_mat_q(w, xt, edb.make_epilogue(stream, bias=dev(b, cuda), residual=stream, gate=dev(g, cuda)))
        outs.append(stream.cpu().numpy())
    assert np.array_equal(outs[0], outs[1]), "unsplit sums differ between runs"
    assert O.rel_l2(outs[0], got) < 1e-4, ("split vs unsplit", O.rel_l2(outs[0], got))


def test_mul_mat_q_column_split(edb, cuda):
    # FLUX single-block linear1: qkv columns to one buffer, GELU(mlp) columns into
    # the tail of the linear2 input buffer.
    m, n_out, k, split = 150, 1024, 512, 512
    w, xt, xr, wd, rng = _gemm_case(edb, cuda, "q8_0", m, n_out, k, torch.float16, seed=14)
    b = rng.standard_normal(n_out, dtype=np.float32)
    qkv = torch.zeros(m, split, dtype=torch.bfloat16, device=cuda)
    cat = torch.zeros(m, 256 + (n_out - split), dtype=torch.bfloat16, device=cuda)
    ep = edb.make_epilogue(qkv, bias=dev(b, cuda), split_n=split, out2=cat[:, 256:], act2=edb.ACT_GELU_TANH,
                           ldo2=cat.stride(0))
    edb.mul_mat_q(w, xt, ep)
    full = xr @ wd.T + b
    assert O.rel_l2(qkv.float().cpu().numpy(), full[:, :split]) < 8e-3
    assert O.rel_l2(cat[:, 256:].float().cpu().numpy(), O.gelu_tanh(full[:, split:])) < 8e-3
    assert not cat[:, :256].any()


@pytest.mark.parametrize("heads,d,normed", [(3, 128, True), (4, 64, True), (6, 64, False)])
def test_mul_mat_q_fused_qkv_pack(edb, cuda, heads, d, normed):
    """The QKV projection's own epilogue packs q | k | v head-major with RMSNorm and RoPE on the f32
    accumulators; features past the packed ones take the column split with GELU (FLUX linear1).  Against the
    oracle (fp32 GEMM on the dequantised weights, then norm and rotation) and against the separate
    edb200_qk_norm_rope_pack on the projection's f16 output."""
    import ctypes as C
    if not edb.lib().edb200_mul_mat_q_fuses_qk_pack():
        pytest.skip("the CTA-pair GEMM is switched off")
    k, extra = 512, 256
    hid = heads * d
    m, nt, L = 300, 20, 384            # 300 rows written at token offset 20 of a 384-token sequence
    n_out = 3 * hid + extra
    w, xt, xr, wd, rng = _gemm_case(edb, cuda, "q8_0", m, n_out, k, torch.float16, seed=21)
    bias = rng.standard_normal(n_out, dtype=np.float32) * np.float32(0.1)
    qw = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    kw = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    ids = rng.integers(0, 40, size=(L, 3)).astype(np.float32)
    pe = O.embed_nd(ids, (16, 56, 56) if d == 128 else (16, 24, 24), 10000.0)
    t_bias, t_qw, t_kw, t_pe = dev(bias, cuda), dev(qw, cuda), dev(kw, cuda), dev(pe, cuda)
    outs = [torch.zeros(heads, L, d, dtype=torch.float16, device=cuda) for _ in range(3)]
    qkv = torch.zeros(m, 3 * hid, dtype=torch.float16, device=cuda)
    tail = torch.zeros(m, extra, dtype=torch.float16, device=cuda)
    pack = edb.QkPack()
    pack.n_heads, pack.d_head, pack.eps = heads, d, 1e-6
    if normed:
        pack.q_weight, pack.k_weight, pack.pe = edb.ptr(t_qw), edb.ptr(t_kw), edb.ptr(t_pe)
    pack.tok_off, pack.l_total = nt, L
    pack.q_out, pack.k_out, pack.v_out = (edb.ptr(o) for o in outs)
    ep = edb.make_epilogue(qkv, bias=t_bias, split_n=3 * hid, out2=tail, act2=edb.ACT_GELU_TANH)
    ep.pack = C.cast(C.pointer(pack), C.c_void_p)
    edb.mul_mat_q(w, xt, ep)
    torch.cuda.synchronize()
    got = [o.float().cpu().numpy() for o in outs]

    y = xr @ wd.T + bias
    q = y[:, :hid].reshape(m, heads, d)
    kk = y[:, hid:2 * hid].reshape(m, heads, d)
    v = y[:, 2 * hid:3 * hid].reshape(m, heads, d)
    if normed:
        rq = O.apply_rope(O.rms_norm(q, qw), pe[nt:nt + m]).transpose(1, 0, 2)
        rk = O.apply_rope(O.rms_norm(kk, kw), pe[nt:nt + m]).transpose(1, 0, 2)
    else:                                              # SD3-medium: plain head-major layout
        rq, rk = q.transpose(1, 0, 2), kk.transpose(1, 0, 2)
    assert O.rel_l2(got[0][:, nt:nt + m], rq) < 2e-3
    assert O.rel_l2(got[1][:, nt:nt + m], rk) < 2e-3
    assert O.rel_l2(got[2][:, nt:nt + m], v.transpose(1, 0, 2)) < 2e-3
    for g in got:                                      # rows outside the window untouched
        assert not g[:, :nt].any() and not g[:, nt + m:].any()
    assert not qkv.any().item()                        # the packed features do not reach `out`
    assert O.rel_l2(tail.float().cpu().numpy(), O.gelu_tanh(y[:, 3 * hid:])) < 3e-3

    # the separate path on the same projection
    ep2 = edb.make_epilogue(qkv, bias=t_bias, split_n=3 * hid, out2=tail, act2=edb.ACT_GELU_TANH)
    edb.mul_mat_q(w, xt, ep2)
    outs2 = [torch.zeros(heads, L, d, dtype=torch.float16, device=cuda) for _ in range(3)]
    edb.check(edb.lib().edb200_qk_norm_rope_pack(edb.ptr(qkv), edb.TYPE_F16, 3 * hid, 0, hid, 2 * hid, m, heads, d,
                                                 edb.ptr(t_qw) if normed else None, edb.ptr(t_kw) if normed else None, 1e-6,
                                                 edb.ptr(t_pe) if normed else None, nt, L,
                                                 edb.ptr(outs2[0]), edb.ptr(outs2[1]), edb.ptr(outs2[2]), edb.TYPE_F16,
                                                 edb.current_stream()))
    torch.cuda.synchronize()
    for a, b in zip(outs, outs2):
        assert O.rel_l2(a.float().cpu().numpy(), b.float().cpu().numpy()) < 2e-3
    assert torch.equal(outs[2], outs2[2])              # v is a copy of the same f16 values either way

    # refused: another head width, or packed features that do not end at the split
    pack.d_head = 32
    with pytest.raises(edb.EdbError):
        edb.mul_mat_q(w, xt, ep)
    pack.d_head, pack.n_heads = d, heads - 1
    with pytest.raises(edb.EdbError):
        edb.mul_mat_q(w, xt, ep)


def test_mul_mat_q_pair(edb, cuda):
    w0, x0, xr0, wd0, _ = _gemm_case(edb, cuda, "q8_0", 512, 768, 512, torch.float16, seed=15)
    w1, x1, xr1, wd1, _ = _gemm_case(edb, cuda, "q8_0", 90, 256, 1024, torch.float16, seed=16)
    y0 = torch.zeros(512, 768, dtype=torch.float32, device=cuda)
    y1 = torch.zeros(90, 256, dtype=torch.float32, device=cuda)
    e0, e1 = edb.make_epilogue(y0), edb.make_epilogue(y1)
    edb.check(edb.lib().edb200_mul_mat_q_pair(w0.handle, edb.ptr(x0), 512, x0.stride(0), C.byref(e0), w1.handle,
                                              edb.ptr(x1), 90, x1.stride(0), C.byref(e1), edb.TYPE_F16,
                                              edb.current_stream()))
    assert O.rel_l2(y0.cpu().numpy(), xr0 @ wd0.T) < 2e-3
    assert O.rel_l2(y1.cpu().numpy(), xr1 @ wd1.T) < 2e-3


def test_mul_mat_q_linearity(edb, cuda):
    # size-independent property at a FLUX-sized layer: f(x1 + x2) == f(x1) + f(x2) up to rounding
    m, n_out, k = 512, 3072, 3072
    w, x1, _, _, rng = _gemm_case(edb, cuda, "q8_0", m, n_out, k, torch.float16, seed=17)
    x2 = dev(rng.standard_normal((m, k), dtype=np.float32), cuda).half()
    ys = [torch.zeros(m, n_out, dtype=torch.float32, device=cuda) for _ in range(3)]
    for x, y in zip((x1, x2, (x1.float() + x2.float()).half()), ys):
        edb.mul_mat_q(w, x, edb.make_epilogue(y))
    assert O.rel_l2(ys[2].cpu().numpy(), (ys[0] + ys[1]).cpu().numpy()) < 2e-3


def test_mul_mat_q_rejects_bad_arguments(edb, cuda):
    w, xt, _, _, _ = _gemm_case(edb, cuda, "q8_0", 128, 256, 64, torch.float16)
    y = torch.zeros(128, 256, dtype=torch.float32, device=cuda)
    with pytest.raises(edb.EdbError):
        edb.mul_mat_q(w, xt.float(), edb.make_epilogue(y))          # f32 activations are not accepted
    with pytest.raises(edb.EdbError):
        edb.mul_mat_q(w, xt.bfloat16(), edb.make_epilogue(y))       # operands must share the f16 format
    ep = edb.make_epilogue(y, split_n=100, out2=y)
    with pytest.raises(edb.EdbError):
        edb.mul_mat_q(w, xt, ep)                                     # split not a multiple of 256
