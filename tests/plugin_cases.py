"""Shared by the plugin-ABI tests and the golden generator: custom-op nodes as the reference's graph
builders would hand them to a backend (ggml_tensor structures laid out as include/edb200_ggml.h,
op_params = {callback, n_tasks, userdata}), on seeded inputs.  The same node description is run by the
reference's CPU callback on host memory (oracle/_ref, where built) and by this library's plugin entry
points on device memory."""
import ctypes as C

import numpy as np

TYPE_F32, TYPE_F16, TYPE_BF16 = 0, 1, 30
OP_CUSTOM = 1
NP_OF = {TYPE_F32: np.float32, TYPE_F16: np.float16, TYPE_BF16: np.uint16}
SIZE_OF = {TYPE_F32: 4, TYPE_F16: 2, TYPE_BF16: 2}

# userdata magics and packing: the interface of the reference's custom operators
# (src/core/backend/ggml/ed_ggml_{modulation,norm,rope,attention,sp_flux,sage_attn}_ext.hpp)
MAGIC = {"modulate": 0x45464d4f, "residual_gate": 0x45465247, "where_select": 0x45465753, "rms_norm_mul_f16": 0x45524d48,
         "rope": 0x45525250, "v_prep": 0x45565050, "pair_pack": 0x45505150, "qkv_pair_pack": 0x45514b50,
         "gelu_bf16": 0x45464742, "concat_linear": 0x45464c32, "concat_linear_residual_gate": 0x45464c47,
         "sage": 0x53414751}


class GgmlTensor(C.Structure):
    pass


GgmlTensor._fields_ = [("type", C.c_int), ("ne", C.c_int64 * 4), ("nb", C.c_size_t * 4), ("op", C.c_int),
                       ("op_params", C.c_int32 * 16), ("src", C.POINTER(GgmlTensor) * 10), ("data", C.c_void_p),
                       ("name", C.c_char * 64)]


def layout_words():
    """sizeof and field offsets in the order edb200_plugin_tensor_layout reports them."""
    f = GgmlTensor
    return [C.sizeof(f), f.type.offset, f.ne.offset, f.nb.offset, f.op.offset, f.op_params.offset, f.src.offset, f.data.offset]


def userdata(kind, a=0, b=0, c=0, f=0.0):
    u = MAGIC[kind]
    if kind == "rms_norm_mul_f16":
        u |= int(np.float32(f).view(np.uint32)) << 32
    elif kind == "rope":       # layout, interleaved, d_head
        u |= (a & 0xff) << 32 | (b & 0xff) << 40 | (c & 0xffff) << 48
    elif kind == "v_prep":     # v_is_seq_major
        u |= (a & 0xff) << 32
    elif kind in ("pair_pack", "qkv_pair_pack", "sage"):   # n_head
        u |= (a & 0x7fffffff) << 32
    return u


class Node:
    """A custom-op node: numpy inputs (with optional non-dense strides), output type/shape, userdata."""

    def __init__(self, kind, srcs, out_type, out_ne, ud):
        self.kind, self.srcs, self.out_type, self.out_ne, self.ud = kind, srcs, out_type, tuple(out_ne), ud

    def out_array(self):
        return np.zeros(tuple(reversed(self.out_ne)), dtype=NP_OF[self.out_type])

    def build(self, ptr_of):
        """ctypes structures for the node; ptr_of(array) gives the data address to put into a tensor
        (host address for the reference callback, device address for the plugin).  Returns (dst, keepalive)."""
        keep = []

        def tensor(arr, gtype, ne=None, nb=None):
            t = GgmlTensor()
            t.type = gtype
            shape = tuple(reversed(arr.shape)) if ne is None else ne
            shape = shape + (1,) * (4 - len(shape))
            strides = tuple(reversed(arr.strides)) if nb is None else nb
            for i in range(4):
                t.ne[i] = shape[i]
                # extent-1 dimensions get the dense stride, as ggml always sets it (numpy may report 0 there)
                dense = SIZE_OF[gtype] if i == 0 else t.nb[i - 1] * t.ne[i - 1]
                t.nb[i] = strides[i] if i < len(strides) and shape[i] != 1 else dense
            t.data = ptr_of(arr)
            keep.append(t)
            return t

        out = self.out_array()
        dst = tensor(out, self.out_type, ne=self.out_ne,
                     nb=tuple(SIZE_OF[self.out_type] * int(np.prod(self.out_ne[:i])) for i in range(4)))
        dst.op = OP_CUSTOM
        words = (C.c_uint64 * 3)(0, 0, self.ud)            # {callback, n_tasks (+pad), userdata}
        C.memmove(dst.op_params, words, 24)
        for i, (arr, gtype) in enumerate(self.srcs):
            if arr is None:
                continue
            dst.src[i] = C.pointer(tensor(arr, gtype))
        return dst, out, keep


def _bf16(x):
    """f32 -> bf16 bits, round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + (0x7fff + ((u >> 16) & 1))) >> 16).astype(np.uint16)


def cases(seed=77):
    """{name: Node} over every operator of the plugin surface that has a reference CPU callback."""
    rng = np.random.default_rng(seed)
    f = np.float32
    out = {}
    # arrays are written [ne3, ne2, ne1, ne0] (numpy order), i.e. ggml ne = reversed shape
    x = (rng.standard_normal((2, 3, 5, 32)) * np.exp(rng.uniform(-3, 3, (2, 3, 5, 32)))).astype(f)
    shift, scale = rng.standard_normal((1, 1, 1, 32)).astype(f), rng.standard_normal((1, 1, 1, 32)).astype(f)
    out["modulate"] = Node("modulate", [(x, TYPE_F32), (shift, TYPE_F32), (scale, TYPE_F32)], TYPE_F32, (32, 5, 3, 2),
                           userdata("modulate"))
    # per-batch vectors (broadcast over rows only) and a strided x (every second row of a larger buffer)
    big = rng.standard_normal((2, 3, 10, 32)).astype(f)
    xs = big[:, :, ::2, :]
    sh2, sc2 = rng.standard_normal((2, 1, 1, 32)).astype(f), rng.standard_normal((2, 1, 1, 32)).astype(f)
    out["modulate_strided"] = Node("modulate", [(xs, TYPE_F32), (sh2, TYPE_F32), (sc2, TYPE_F32)], TYPE_F32, (32, 5, 3, 2),
                                   userdata("modulate"))
    res = rng.standard_normal((2, 3, 5, 32)).astype(f)
    gate = rng.standard_normal((2, 1, 1, 32)).astype(f)
    out["residual_gate"] = Node("residual_gate", [(res, TYPE_F32), (x, TYPE_F32), (gate, TYPE_F32)], TYPE_F32, (32, 5, 3, 2),
                                userdata("residual_gate"))
    index = (rng.random((1, 1, 7, 1)) > 0.5).astype(f)
    m0, m1 = rng.standard_normal((2, 1, 1, 48)).astype(f), rng.standard_normal((2, 1, 1, 48)).astype(f)
    out["where_select"] = Node("where_select", [(index, TYPE_F32), (m0, TYPE_F32), (m1, TYPE_F32)], TYPE_F32, (48, 7, 1, 2),
                               userdata("where_select"))
    nx = (rng.standard_normal((1, 2, 9, 128)) * 3).astype(f)
    nw = (1 + 0.1 * rng.standard_normal((1, 1, 1, 128))).astype(f)
    out["rms_norm_mul_f16"] = Node("rms_norm_mul_f16", [(nx, TYPE_F32), (nw, TYPE_F32)], TYPE_F16, (128, 9, 2, 1),
                                   userdata("rms_norm_mul_f16", f=1e-6))
    # rope: d 64, 3 heads, 11 positions, 2 batches; table [seq][pair][col][row] = ggml [2, 2, d/2, seq]
    ang = rng.uniform(-3, 3, (11, 32)).astype(f)
    pe = np.stack([np.stack([np.cos(ang), -np.sin(ang)], -1), np.stack([np.sin(ang), np.cos(ang)], -1)], -2).astype(f)
    rx0 = rng.standard_normal((2, 11, 3, 64)).astype(f)                       # ggml [d, heads, seq, batch]
    out["rope_nseqheaddim"] = Node("rope", [(rx0, TYPE_F32), (pe, TYPE_F32)], TYPE_F32, (64, 11, 6, 1),
                                   userdata("rope", 0, 1, 64))
    rx1 = rng.standard_normal((2, 3, 11, 64)).astype(f)                       # ggml [d, seq, heads, batch]
    out["rope_seqheaddim_f16"] = Node("rope", [(rx1, TYPE_F32), (pe, TYPE_F32)], TYPE_F16, (64, 11, 6, 1),
                                      userdata("rope", 1, 1, 64))
    out["rope_split_halves"] = Node("rope", [(rx1, TYPE_F32), (pe, TYPE_F32)], TYPE_F32, (64, 11, 6, 1),
                                    userdata("rope", 1, 0, 64))
    out["rope_bf16_in"] = Node("rope", [(_bf16(rx0), TYPE_BF16), (pe, TYPE_F32)], TYPE_BF16, (64, 11, 6, 1),
                               userdata("rope", 0, 1, 64))
    # attention layout glue: 4 heads x d 16
    v_tok = rng.standard_normal((2, 13, 4, 16)).astype(f)                     # ggml [d, heads, seq, batch]
    out["v_prep_token_major"] = Node("v_prep", [(v_tok, TYPE_F32)], TYPE_F16, (16, 13, 8, 1), userdata("v_prep", 0))
    v_seq = rng.standard_normal((2, 4, 13, 16)).astype(f)                     # ggml [d, seq, heads, batch]
    out["v_prep_seq_major"] = Node("v_prep", [(v_seq, TYPE_F32)], TYPE_F16, (16, 13, 8, 1), userdata("v_prep", 1))
    first, second = rng.standard_normal((1, 2, 5, 64)).astype(f), rng.standard_normal((1, 2, 9, 64)).astype(f)
    out["pair_pack"] = Node("pair_pack", [(first, TYPE_F32), (second, TYPE_F32)], TYPE_F16, (16, 14, 4, 2),
                            userdata("pair_pack", 4))
    six = [rng.standard_normal((1, 1, n, 64)).astype(f) for n in (5, 5, 5, 9, 9, 9)]
    out["qkv_pair_pack"] = Node("qkv_pair_pack", [(a, TYPE_F32) for a in six], TYPE_F16, (16, 14, 4, 3),
                                userdata("qkv_pair_pack", 4))
    # operators the reference keeps on the CPU path only (no plugin entry point): pins for the oracle
    gx = (rng.standard_normal((1, 1, 6, 40)) * 3).astype(f)
    out["gelu_bf16"] = Node("gelu_bf16", [(gx, TYPE_F32)], TYPE_BF16, (40, 6, 1, 1), userdata("gelu_bf16"))
    x0, x1 = rng.standard_normal((1, 1, 7, 24)).astype(f), rng.standard_normal((1, 1, 7, 40)).astype(f)
    w = (rng.standard_normal((1, 1, 12, 64)) * 0.1).astype(f)                 # ggml [in = 24 + 40, out = 12]
    b = rng.standard_normal((1, 1, 1, 12)).astype(f)
    out["concat_linear"] = Node("concat_linear", [(x0, TYPE_F32), (x1, TYPE_F32), (w, TYPE_F32), (b, TYPE_F32)], TYPE_F32,
                                (12, 7, 1, 1), userdata("concat_linear"))
    r = rng.standard_normal((1, 1, 7, 12)).astype(f)
    g = rng.standard_normal((1, 1, 1, 12)).astype(f)
    out["concat_linear_residual_gate"] = Node(
        "concat_linear_residual_gate", [(r, TYPE_F32), (x0, TYPE_F32), (x1, TYPE_F32), (w, TYPE_F32), (b, TYPE_F32), (g, TYPE_F32)],
        TYPE_F32, (12, 7, 1, 1), userdata("concat_linear_residual_gate"))
    return out


PLUGIN_OF = {"modulate": 0, "residual_gate": 0, "where_select": 0, "rms_norm_mul_f16": 1, "rope": 2, "v_prep": 3,
             "pair_pack": 4, "qkv_pair_pack": 5}


def run_reference(lib, node):
    """The reference's CPU callback on host memory (lib = oracle/_ref/libedref_cpu.so)."""
    import os
    os.environ["ED_FLUX_SP_MLP_GELU_BF16"] = "1"     # the reference keeps its GELU-to-bf16 operator behind this switch
    dst, out, keep = node.build(lambda a: a.ctypes.data)
    lib.ref_custom_op.argtypes = [C.POINTER(GgmlTensor)]
    lib.ref_custom_op.restype = C.c_int
    assert lib.ref_custom_op(C.byref(dst)) == 1, node.kind
    return out
