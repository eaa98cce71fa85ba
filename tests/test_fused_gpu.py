"""GPU parity of the fused channel-last entry points (hyena_se_fwd / hyena_mr_fwd / hyena_li_fwd and the
one-launch decode layer) against the CPU oracle, plus size-independent properties at full benchmark size."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from helpers import DT, TOL, check, cuda, make_block, rel_l2, to_np
from oracle import hyena_oracle as O

pytestmark = pytest.mark.gpu


def _oracle(p, D, K, io, layout, heads=1, flip=False, mirror=False):
    return O.hyena_fused(to_np(p["u"]), to_np(p["w3"]), to_np(p["h"]), None if p["Dp"] is None else to_np(p["Dp"]),
                         D, K, io=io, layout=layout, num_heads=heads, flip_x1x2=flip, mirror=mirror)


def _fused(pc, K, layout, heads=1, flip=False, want_state=True):
    from vortex_b200 import hyena_ops
    if K >= 128:
        return hyena_ops.hyena_mr_fwd(pc["u"], pc["w3"], None, pc["h"], pc["Dp"], layout=layout, num_heads=heads,
                                      flip=flip, want_state=want_state)
    return hyena_ops.hyena_se_fwd(pc["u"], pc["w3"], None, pc["h"], layout=layout, num_heads=heads, flip=flip,
                                  want_state=want_state)


SE_CASES = [
    ("f32", 1, 2048, 768, 48, 7, "split", 1, False),         # configuration 1, full size
    ("bf16", 2, 1000, 256, 16, 7, "interleaved", 1, False),
    ("bf16", 1, 333, 200, 25, 7, "interleaved", 1, True),    # D not a multiple of the 64-channel slab, odd groups
    ("f16", 2, 77, 128, 8, 4, "interleaved", 1, False),
    ("f32", 1, 5, 64, 4, 7, "interleaved", 1, False),        # L < K-1
    ("f32", 2, 1, 64, 4, 7, "split", 1, False),              # single token
    ("bf16", 1, 600, 256, 16, 7, "column_split", 2, True),
    ("f32", 1, 129, 128, 128, 16, "split", 1, False),        # longest CUDA-core filter, per-channel taps
]


@pytest.mark.parametrize("io,B,L,D,G,K,layout,heads,flip", SE_CASES)
def test_fused_se_vs_oracle(io, B, L, D, G, K, layout, heads, flip):
    from vortex_b200 import ops
    p = make_block(31, B, L, D, G, K, io)
    ref, fs_ref, st_ref = _oracle(p, D, K, io, layout, heads, flip)
    y, fs, st = _fused(cuda(p), K, layout, heads, flip)
    ops.device_status()
    assert y.shape == (B, L, D) and y.dtype == DT[io]
    check("test_fused_gpu.py:47 y, ref", rel_l2(y, ref), TOL[io])
    assert np.array_equal(to_np(fs), fs_ref.astype(np.float32))     # copy of the last inputs: bit-exact
    assert st.shape == st_ref.shape
    check("test_fused_gpu.py:50 st, st_ref", rel_l2(st, st_ref), (1e-6 if io == "f32" else 2e-3))   # k*v rounded once to the I/O dtype


MR_CASES = [
    ("bf16", 1, 2048, 256, 16, 128, "interleaved", 1, False),   # configuration 2 shape, reduced B and D
    ("bf16", 3, 1000, 64, 4, 128, "interleaved", 1, False),     # ragged L, stream quad partly idle
    ("bf16", 2, 700, 128, 8, 64, "interleaved", 1, True),       # shorter filter on the tensor-core path, flip
    ("bf16", 4, 300, 64, 4, 128, "split", 1, False),
    ("bf16", 2, 520, 128, 8, 128, "column_split", 2, True),
    ("bf16", 1, 100, 32, 2, 128, "interleaved", 1, False),      # L < K
    ("bf16", 2, 1, 32, 2, 128, "interleaved", 1, False),        # single token
    ("bf16", 1, 8192, 64, 4, 128, "interleaved", 1, False),     # several time segments per sequence
    ("bf16", 2, 1000, 256, 16, 128, "interleaved", 1, False),   # two idle streams in the quad, 16 groups
    ("bf16", 2, 1000, 256, 16, 17, "interleaved", 1, False),    # shortest filter on the tensor-core path
]


@pytest.mark.parametrize("io,B,L,D,G,K,layout,heads,flip", MR_CASES)
def test_fused_mr_vs_oracle(io, B, L, D, G, K, layout, heads, flip):
    """tcgen05 blocked-Toeplitz path: bf16 I/O, fp32 accumulation, k*v carried as bf16 head + remainder."""
    from vortex_b200 import ops
    p = make_block(33, B, L, D, G, K, io)
    ref, fs_ref, st_ref = _oracle(p, D, K, io, layout, heads, flip)
    y, fs, st = _fused(cuda(p), K, layout, heads, flip)
    ops.device_status()
    assert y.shape == (B, L, D) and y.dtype == DT[io]
    check("test_fused_gpu.py:76 y, ref", rel_l2(y, ref), TOL[io])
    assert np.array_equal(to_np(fs), fs_ref.astype(np.float32))
    assert st.shape == st_ref.shape
    check("test_fused_gpu.py:79 st, st_ref", rel_l2(st, st_ref), 2e-3)


def test_fused_mr_exact_on_integers():
    """Integer data small enough for bf16 products and fp32 sums to be exact: output equals the oracle bit for bit
    (pins the Toeplitz expansion, chunk/segment seams, stream skew and channel maps of the tensor-core path)."""
    g = torch.Generator().manual_seed(6)
    B, L, D, G, K = 3, 1300, 64, 4, 128
    u = torch.randint(-1, 2, (B, L, 3 * D), generator=g).float()
    w3 = torch.randint(-1, 2, (3 * D, 1, 3), generator=g).float()
    h = torch.zeros(G, 1, K)
    for pos in (0, 1, 64, K - 1):                      # first, second, a middle and the last tap
        h[:, 0, pos] = torch.randint(0, 2, (G,), generator=g).float() * 2 - 1
    Dp = torch.randint(-1, 2, (D,), generator=g).float()
    p = {"u": u.bfloat16(), "w3": w3.bfloat16(), "h": h.bfloat16(), "Dp": Dp.bfloat16()}
    for layout, heads, flip in (("interleaved", 1, False), ("split", 1, True), ("column_split", 2, False)):
        ref, _, st_ref = _oracle(p, D, K, "f32", layout, heads, flip, mirror=True)
        assert np.abs(ref).max() < 256          # exactly representable in bf16
        y, _, st = _fused(cuda(p), K, layout, heads, flip)
        assert np.array_equal(to_np(y), ref.astype(np.float32)), layout
        assert np.array_equal(to_np(st), st_ref.astype(np.float32))


def test_fused_mr_full_size_properties():
    """Configuration 2 at full size (B=4, L=8192, D=4096, bf16): oracle on a slice of channels, channel-shard
    invariance and causality."""
    from vortex_b200 import hyena_ops
    B, L, D, G, K = 4, 8192, 4096, 256, 128
    p = make_block(1, B, L, D, G, K, "bf16")
    pc = cuda(p)
    y, _, _ = hyena_ops.hyena_mr_fwd(pc["u"], pc["w3"], None, pc["h"], pc["Dp"])
    d0, d1 = 2000, 2032
    sub = {"u": p["u"][::3, :, 3 * d0:3 * d1], "w3": p["w3"][3 * d0:3 * d1], "h": p["h"][d0 // 16:d1 // 16],
           "Dp": p["Dp"][d0:d1]}
    ref, _, _ = _oracle(sub, d1 - d0, K, "bf16", "interleaved")
    check("test_fused_gpu.py:114 y[::3, :, d0:d1], ref", rel_l2(y[::3, :, d0:d1], ref), TOL["bf16"])
    c0, c1 = 1024, 1536
    ys, _, _ = hyena_ops.hyena_mr_fwd(pc["u"][:, :, 3 * c0:3 * c1].contiguous(), pc["w3"][3 * c0:3 * c1], None,
                                      pc["h"][c0 // 16:c1 // 16], pc["Dp"][c0:c1])
    assert torch.equal(ys, y[:, :, c0:c1])
    t0 = 4321
    u2 = pc["u"].clone()
    u2[:, t0:] = -u2[:, t0:]
    y2, _, _ = hyena_ops.hyena_mr_fwd(u2, pc["w3"], None, pc["h"], pc["Dp"])
    assert torch.equal(y2[:, :t0], y[:, :t0]) and not torch.equal(y2[:, t0:], y[:, t0:])


def test_fused_se_exact_on_integers():
    """Small-integer data makes every intermediate exact: fused output and caches equal the oracle bit
    for bit, for every q/k/v layout -- pins the channel maps, tap order, halo handling and cache indexing."""
    g = torch.Generator().manual_seed(5)
    B, L, D, G, K = 2, 700, 128, 8, 7
    u = torch.randint(-2, 3, (B, L, 3 * D), generator=g).float()
    w3 = torch.randint(-1, 2, (3 * D, 1, 3), generator=g).float()
    h = torch.randint(-1, 2, (G, 1, K), generator=g).float()
    p = {"u": u, "w3": w3, "h": h, "Dp": None}
    for layout, heads, flip in (("split", 1, False), ("interleaved", 1, False), ("interleaved", 1, True),
                                ("column_split", 2, False)):
        ref, fs_ref, st_ref = _oracle(p, D, K, "f32", layout, heads, flip, mirror=True)
        y, fs, st = _fused(cuda(p), K, layout, heads, flip)
        assert np.array_equal(to_np(y), ref.astype(np.float32)), layout
        assert np.array_equal(to_np(fs), fs_ref.astype(np.float32))
        assert np.array_equal(to_np(st), st_ref.astype(np.float32))


def test_fused_se_full_size_properties():
    """Configuration-2-sized input (B=4, L=8192, D=4096, bf16) through the SE kernel: oracle on a slice of
    channels, causality, and channel-shard invariance (a shard of channels computed alone is bit-identical)."""
    from vortex_b200 import hyena_ops
    B, L, D, G, K = 4, 8192, 4096, 256, 7
    p = make_block(1, B, L, D, G, K, "bf16")
    pc = cuda(p)
    y, _, _ = hyena_ops.hyena_se_fwd(pc["u"], pc["w3"], None, pc["h"])
    # (1) oracle on channels [1024, 1088) of batch 1 and 3
    d0, d1 = 1024, 1088
    sub = {"u": p["u"][1::2, :, 3 * d0:3 * d1], "w3": p["w3"][3 * d0:3 * d1], "h": p["h"][d0 // 16:d1 // 16], "Dp": None}
    ref, _, _ = _oracle(sub, d1 - d0, K, "bf16", "interleaved")
    check("test_fused_gpu.py:156 y[1::2, :, d0:d1], ref", rel_l2(y[1::2, :, d0:d1], ref), TOL["bf16"])
    # (2) shard invariance: the same 512 channels computed as their own problem give identical bits
    c0, c1 = 2048, 2560
    ys, _, _ = hyena_ops.hyena_se_fwd(pc["u"][:, :, 3 * c0:3 * c1].contiguous(), pc["w3"][3 * c0:3 * c1], None,
                                      pc["h"][c0 // 16:c1 // 16])
    assert torch.equal(ys, y[:, :, c0:c1])
    # (3) causality: changing the input from t0 on leaves every earlier output untouched
    t0 = 5000
    u2 = pc["u"].clone()
    u2[:, t0:] = -u2[:, t0:]
    y2, _, _ = hyena_ops.hyena_se_fwd(u2, pc["w3"], None, pc["h"])
    assert torch.equal(y2[:, :t0], y[:, :t0]) and not torch.equal(y2[:, t0:], y[:, t0:])


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("kind", ["se", "mr", "li"])
def test_decode_layer_matches_step_sequence(io, kind):
    """One-launch decode layer == the reference's sequence step_fir -> interleave/split -> step_fir|step_iir -> gate
    (model.py:318-375), run here through the drop-in engine; caches bit-identical, outputs to rounding."""
    from vortex_b200 import HyenaInferenceEngine, ops
    eng = HyenaInferenceEngine()
    B, D, G = 3, 96, 6
    K = {"se": 7, "mr": 128, "li": 0}[kind]
    g = torch.Generator().manual_seed(17)
    dt = DT[io]
    w3 = (torch.randn(3 * D, 1, 3, generator=g) / 3 ** 0.5).to(dt).cuda()
    fs = torch.randn(B, 3 * D, 2, generator=g).to(dt).cuda()
    Dp = torch.randn(D, generator=g).to(dt).cuda()
    if kind == "li":
        lp = torch.log(0.9 + 0.099 * torch.rand(D, 16, 1, generator=g)).cuda()
        R = torch.randn(D, 16, generator=g).cuda()
        st = torch.randn(B, D, 16, generator=g).cuda()
    else:
        h = (torch.randn(G, 1, K, generator=g) / K ** 0.5).to(dt).cuda()
        st = torch.randn(B, D, K - 1, generator=g).to(dt).cuda()
    fs_a, st_a, fs_b, st_b = fs, st, fs, st
    for step in range(3):
        u = torch.randn(B, 3 * D, generator=g).to(dt).cuda()
        # reference sequence on the drop-in engine
        z, fs_a = eng.step_fir(u, fs_a, w3)
        q, k, v = z[:, 0::3], z[:, 1::3], z[:, 2::3]
        if kind == "li":
            ya, st_a = eng.step_iir(q, k, v, Dp, R, lp, st_a)
            ya = ya.to(dt)
            yb, fs_b, st_b = ops.decode_layer(u, w3, None, fs_b, D, log_poles=lp, residues=R, bias=Dp, iir_state=st_b)
        else:
            ya, st_a = eng.step_fir(k * v, st_a, h.repeat_interleave(D // G, 0), bias=Dp if K >= 128 else None,
                                    flip_filter=K >= 128, gated_bias=K >= 128)
            ya = ya * q
            yb, fs_b, st_b = ops.decode_layer(u, w3, None, fs_b, D, h=h, inner_state=st_b,
                                              bias=Dp if K >= 128 else None, flip_filter=K >= 128, gated_bias=K >= 128)
        assert yb.dtype == dt and fs_b.dtype == torch.float32 and st_b.dtype == torch.float32
        assert torch.equal(fs_a, fs_b)
        check("test_fused_gpu.py:209 yb, ya", rel_l2(yb, ya), (1e-6 if io == "f32" else 2e-3))
        check("test_fused_gpu.py:210 st_b, st_a", rel_l2(st_b, st_a), 1e-6)


def test_fused_li_vs_oracle():
    """A modal system per channel (the fp32-pipe recurrence kernel): nothing between the input rows and the output is
    rounded to the I/O dtype, so the oracle keeps the featurizer output and k*v unrounded too."""
    from vortex_b200 import hyena_ops
    B, L, D, S = 2, 900, 64, 16
    for io in ("f32", "bf16"):
        p = make_block(41, B, L, D, D, 0, io, modal=True, S=S)
        pc = cuda(p)
        y, fs, st = hyena_ops.hyena_li_fwd(pc["u"], pc["w3"], None, pc["log_poles"], pc["residues"], pc["Dp"],
                                           want_state=True)
        zf, fs_ref = O.featurizer(to_np(p["u"]), to_np(p["w3"]), io=io, mirror=False)
        h = O.modal_filter(to_np(p["log_poles"]), to_np(p["residues"]), L)
        ref, kv = O.long_conv_gate(zf, h, to_np(p["Dp"]), D, io=io, layout="interleaved", mirror=False, round_input=False)
        assert y.shape == (B, L, D)
        check("test_fused_gpu.py:227 y, ref", rel_l2(y, ref), TOL[io])
        assert np.array_equal(to_np(fs), fs_ref.astype(np.float32))
        check("test_fused_gpu.py:229 st, O.modal_state(kv, to_np(p['log_poles']))", rel_l2(st, O.modal_state(kv, to_np(p["log_poles"]))), 3e-5)


# B, L, D, S, complex poles, layout, heads, flip
LI_TC_CASES = [
    (2, 900, 64, 16, False, "interleaved", 1, False),     # real poles, ragged last step
    (1, 2500, 128, 16, True, "interleaved", 1, False),    # complex poles, several steps of 4 x 96 samples
    (1, 384, 32, 8, True, "split", 1, False),             # exactly one step, fewer poles than the tile holds
    (2, 200, 64, 16, True, "column_split", 2, True),
    (3, 1, 32, 16, True, "interleaved", 1, True),         # single token
    (1, 10000, 32, 16, True, "interleaved", 1, False),    # long walk: the state carries ~100 chunks
    (1, 15360, 32, 16, True, "interleaved", 1, False),    # walk cut into two time slices handed over through global memory
    (2, 30001, 32, 16, False, "interleaved", 1, False),   # four slices, ragged front padding
]


def _li_oracle(p, L, D, cplx, layout, heads, flip):
    zf, _ = O.featurizer(to_np(p["u"]), to_np(p["w3"]), io="bf16", mirror=False)
    if cplx:
        poles = np.exp(to_np(p["log_poles"])[..., 0]) * np.exp(1j * to_np(p["theta"]))
        h = O.modal_filter_complex(poles, to_np(p["residues"]) + 1j * to_np(p["res_im"]), L)
    else:
        h = O.modal_filter(to_np(p["log_poles"]), to_np(p["residues"]), L)
    return O.long_conv_gate(zf, O.expand_groups(h, D), to_np(p["Dp"]), D, io="bf16", layout=layout, num_heads=heads,
                            flip_x1x2=flip, mirror=False, round_input=False)


@pytest.mark.parametrize("B,L,D,S,cplx,layout,heads,flip", LI_TC_CASES)
def test_fused_li_tensor_core_vs_oracle(B, L, D, S, cplx, layout, heads, flip):
    """tcgen05 chunked state-space scan: bf16 I/O, fp32 states, every fp32 operand carried as bf16 head + remainder."""
    from vortex_b200 import hyena_ops, ops
    p = make_block(43, B, L, D, D // 16, 0, "bf16", modal=True, S=S, complex_poles=cplx)
    pc = cuda(p)
    y, fs, st = hyena_ops.hyena_li_fwd(pc["u"], pc["w3"], None, pc["log_poles"], pc["residues"], pc["Dp"],
                                       theta=pc.get("theta"), res_im=pc.get("res_im"), layout=layout, num_heads=heads,
                                       flip=flip, want_state=True)
    ops.device_status()
    assert y.shape == (B, L, D) and y.dtype == torch.bfloat16
    ref, kv = _li_oracle(p, L, D, cplx, layout, heads, flip)
    check("test_fused_gpu.py:268 y, ref", rel_l2(y, ref), TOL["bf16"])
    # caches: copy of the last inputs (bit-exact) and the modal state after the last token (fp32)
    assert np.array_equal(to_np(fs), to_np(p["u"])[:, max(L - 2, 0):, :].transpose(0, 2, 1))
    lp = np.repeat(to_np(p["log_poles"])[..., 0], 16, axis=0)
    if cplx:
        poles = np.exp(lp) * np.exp(1j * np.repeat(to_np(p["theta"]), 16, axis=0))
        st_ref = O.modal_state_complex(kv, poles)
        assert st.shape == (B, D, S, 2)
        st_c = to_np(st)[..., 0] + 1j * to_np(st)[..., 1]
        assert np.linalg.norm(st_c - st_ref) / np.linalg.norm(st_ref) <= 2e-5
    else:
        st_ref = O.modal_state(kv, lp)
        assert st.shape == (B, D, S)
        check("test_fused_gpu.py:281 st, st_ref", rel_l2(st, st_ref), 2e-5)
    # without caches the same output
    y2, fs2, st2 = hyena_ops.hyena_li_fwd(pc["u"], pc["w3"], None, pc["log_poles"], pc["residues"], pc["Dp"],
                                          theta=pc.get("theta"), res_im=pc.get("res_im"), layout=layout, num_heads=heads,
                                          flip=flip, want_state=False)
    assert fs2 is None and st2 is None and torch.equal(y2, y)


# B, L, D, G, S, complex poles, io, layout, heads, flip, featurizer bias
LI_CC_CASES = [
    (2, 900, 64, 64, 16, False, "bf16", "interleaved", 1, False, False),    # a modal system per channel (Evo 2)
    (1, 5000, 96, 96, 16, False, "f32", "split", 1, False, True),           # fp32 I/O, featurizer bias
    (1, 3000, 64, 8, 8, True, "bf16", "column_split", 2, True, False),      # complex poles, groups of 8 channels
    (3, 1, 256, 256, 16, False, "f32", "interleaved", 1, False, False),     # single token
    (1, 70003, 32, 32, 16, False, "f32", "interleaved", 1, False, False),   # ~1100 time segments, ragged end
    (2, 777, 40, 40, 12, True, "f16", "interleaved", 1, False, False),      # fp16, channels not a multiple of 32
    # rows staged by TMA (16-bit I/O, real poles, interleaved q/k/v, channels a multiple of 128)
    (2, 1000, 128, 128, 16, False, "bf16", "interleaved", 1, False, False),
    (1, 4099, 256, 256, 16, False, "bf16", "interleaved", 1, True, True),   # ragged end, q and k swapped, featurizer bias
    (3, 5, 128, 128, 16, False, "bf16", "interleaved", 1, False, False),    # shorter than one stage
    (1, 20011, 384, 48, 12, False, "f16", "interleaved", 1, False, False),  # fp16, systems shared by 8 channels, 12 poles
    (2, 1, 128, 128, 16, False, "bf16", "interleaved", 1, True, False),     # single token
    # two channels per thread (channels a multiple of 256, no featurizer bias)
    (2, 3001, 256, 256, 16, False, "bf16", "interleaved", 1, False, False),
    (1, 9000, 512, 64, 12, False, "f16", "interleaved", 1, True, False),    # fp16, q and k swapped, shared systems, 12 poles
    (3, 2, 256, 256, 16, False, "bf16", "interleaved", 1, False, False),    # two tokens
]


def _li_cc_oracle(p, L, D, G, cplx, io, layout, heads, flip, b3):
    zf, _ = O.featurizer(to_np(p["u"]), to_np(p["w3"]), bias=None if b3 is None else to_np(b3), io=io, mirror=False)
    if cplx:
        poles = np.exp(to_np(p["log_poles"])[..., 0]) * np.exp(1j * to_np(p["theta"]))
        h = O.modal_filter_complex(poles, to_np(p["residues"]) + 1j * to_np(p["res_im"]), L)
    else:
        h = O.modal_filter(to_np(p["log_poles"]), to_np(p["residues"]), L)
    h = np.repeat(h, D // G, axis=0)
    return O.long_conv_gate(zf, h, to_np(p["Dp"]), D, io=io, layout=layout, num_heads=heads, flip_x1x2=flip, mirror=False,
                            round_input=False)


def _li_state_ref(p, kv, D, G, cplx):
    lp = np.repeat(to_np(p["log_poles"])[..., 0], D // G, axis=0)
    if cplx:
        return O.modal_state_complex(kv, np.exp(lp) * np.exp(1j * np.repeat(to_np(p["theta"]), D // G, axis=0)))
    return O.modal_state(kv, lp)


@pytest.mark.parametrize("B,L,D,G,S,cplx,io,layout,heads,flip,with_b3", LI_CC_CASES)
def test_fused_li_recurrence_vs_oracle(B, L, D, G, S, cplx, io, layout, heads, flip, with_b3):
    """Channel-last fused long-filter block on the fp32 pipe (modal systems not shared by groups of 16 channels,
    any I/O dtype): featurizer + gate + recurrence + skip + gate, segment carries, state after the last token."""
    from vortex_b200 import hyena_ops, ops
    p = make_block(47, B, L, D, G, 0, io, modal=True, S=S, complex_poles=cplx)
    b3 = (0.1 * torch.randn(3 * D, generator=torch.Generator().manual_seed(5))).to(p["u"].dtype) if with_b3 else None
    pc = cuda(p)
    y, fs, st = hyena_ops.hyena_li_fwd(pc["u"], pc["w3"], None if b3 is None else b3.cuda(), pc["log_poles"],
                                       pc["residues"], pc["Dp"], theta=pc.get("theta"), res_im=pc.get("res_im"),
                                       layout=layout, num_heads=heads, flip=flip, want_state=True)
    ops.device_status()
    assert y.shape == (B, L, D) and y.dtype == p["u"].dtype
    ref, kv = _li_cc_oracle(p, L, D, G, cplx, io, layout, heads, flip, b3)
    check("test_fused_gpu.py:333 y, ref", rel_l2(y, ref), (1e-4 if io == "f32" else TOL["bf16"] if io == "bf16" else 5e-4))
    assert np.array_equal(to_np(fs), to_np(p["u"])[:, max(L - 2, 0):, :].transpose(0, 2, 1))
    st_ref = _li_state_ref(p, kv, D, G, cplx)
    tol = 3e-5
    if cplx:
        assert st.shape == (B, D, S, 2)
        st_c = to_np(st)[..., 0] + 1j * to_np(st)[..., 1]
        assert np.linalg.norm(st_c - st_ref) / np.linalg.norm(st_ref) <= tol
    else:
        assert st.shape == (B, D, S)
        check("test_fused_gpu.py:343 st, st_ref", rel_l2(st, st_ref), tol)


@pytest.mark.parametrize("io,cplx,cuts", [("f32", False, (0, 300, 301, 1000)), ("bf16", True, (0, 2, 3, 640, 1000)),
                                          ("bf16", False, (0, 512, 1000)), ("bf16", False, (0, 3, 700, 701, 2500)),
                                          ("bf16", False, (0, 2, 900, 2501))])
def test_fused_li_chunked_prefill_carries_state(io, cplx, cuts):
    """Prefill in chunks, every call starting from the caches the previous one returned (featurizer rows and modal
    state), gives the output and the final caches of one call over the whole sequence."""
    from vortex_b200 import hyena_ops, ops
    B, D, G, S = 2, 64, (8 if cplx else 64), 16
    L = cuts[-1]
    if L == 2500:
        D = G = 128       # the kernels that stage rows by TMA
    if L == 2501:
        D = G = 256       # ... with two channels per thread
    p = make_block(53, B, L, D, G, 0, io, modal=True, S=S, complex_poles=cplx)
    pc = cuda(p)
    kw = dict(theta=pc.get("theta"), res_im=pc.get("res_im"), want_state=True)
    y_all, fs_all, st_all = hyena_ops.hyena_li_fwd(pc["u"], pc["w3"], None, pc["log_poles"], pc["residues"], pc["Dp"], **kw)
    ys, fs, st = [], None, None
    for t0, t1 in zip(cuts[:-1], cuts[1:]):
        yc, fs, st = hyena_ops.hyena_li_fwd(pc["u"][:, t0:t1], pc["w3"], None, pc["log_poles"], pc["residues"], pc["Dp"],
                                            state_in=st, fir_state_in=fs, **kw)
        ys.append(yc)
    ops.device_status()
    y = torch.cat(ys, dim=1)
    assert y.shape == y_all.shape
    check("test_fused_gpu.py:366 y, y_all", rel_l2(y, y_all), (1e-5 if io == "f32" else 1e-3))      # fp32 summation order differs with the segment plan
    assert torch.equal(fs, fs_all)
    check("test_fused_gpu.py:368 st, st_all", rel_l2(st, st_all), 1e-5)
    ref, _ = _li_cc_oracle(p, L, D, G, cplx, io, "interleaved", 1, False, None)
    check("test_fused_gpu.py:370 y, ref", rel_l2(y, ref), (1e-4 if io == "f32" else TOL["bf16"]))


@pytest.mark.parametrize("cplx,cuts", [(True, (0, 768, 1152, 1920)), (False, (0, 384, 2304)), (True, (0, 1000, 1384)),
                                       (True, (0, 500, 1500, 1600, 2601)), (False, (0, 385, 1154))])
def test_fused_li_tensor_core_chunked_prefill(cplx, cuts):
    """Grouped bf16 systems (the tensor-core kernel): chunks that are views of the whole projection buffer, each call
    told that earlier rows precede its view and given the modal state the previous call returned.  Chunks of a
    multiple of 384 rows stay on the tensor-core kernel; the result equals one call over the whole prompt."""
    from vortex_b200 import hyena_ops, ops
    B, D, G, S = 2, 64, 4, 16
    L = cuts[-1]
    p = make_block(61, B, L, D, G, 0, "bf16", modal=True, S=S, complex_poles=cplx)
    pc = cuda(p)
    kw = dict(theta=pc.get("theta"), res_im=pc.get("res_im"), want_state=True)
    y_all, fs_all, st_all = hyena_ops.hyena_li_fwd(pc["u"], pc["w3"], None, pc["log_poles"], pc["residues"], pc["Dp"], **kw)
    ys, st = [], None
    for t0, t1 in zip(cuts[:-1], cuts[1:]):
        yc, fs, st = hyena_ops.hyena_li_fwd(pc["u"][:, t0:t1], pc["w3"], None, pc["log_poles"], pc["residues"], pc["Dp"],
                                            state_in=st, hist_rows=min(t0, 5), **kw)
        ys.append(yc)
    ops.device_status()
    y = torch.cat(ys, dim=1)
    check("test_fused_gpu.py:393 y, y_all", rel_l2(y, y_all), 1e-3)
    assert torch.equal(fs, fs_all)
    check("test_fused_gpu.py:395 st, st_all", rel_l2(st, st_all), 1e-4)
    ref, _ = _li_cc_oracle(p, L, D, G, cplx, "bf16", "interleaved", 1, False, None)
    check("test_fused_gpu.py:397 y, ref", rel_l2(y, ref), TOL["bf16"])


# io, D, G, K, layout, chunk boundaries
FIR_CHUNK_CASES = [
    ("bf16", 64, 4, 128, "interleaved", (0, 1000, 1130, 2500)),     # 128 taps on tensor cores, a chunk of K + 2 rows
    ("bf16", 128, 8, 7, "interleaved", (0, 300, 308, 900)),         # 7 taps on tensor cores
    ("f32", 64, 4, 7, "split", (0, 260, 700)),                      # CUDA-core kernel, plane layout
]


@pytest.mark.parametrize("io,D,G,K,layout,cuts", FIR_CHUNK_CASES)
def test_fused_fir_chunked_prefill(io, D, G, K, layout, cuts):
    """A prompt prefilled in chunks: (a) chunks that are views of the whole projection buffer, every call told that
    K + 1 earlier rows precede its view; (b) the same through the PrefillChunks staging buffer (one chunk shorter than
    the history it keeps).  Output and final caches equal those of one call over the whole prompt."""
    from vortex_b200 import hyena_ops, ops
    B, L = 2, cuts[-1]
    p = make_block(59, B, L, D, G, K, io)
    pc = cuda(p)

    def call(u, hist, want_state=True):
        if K >= 128:
            return hyena_ops.hyena_mr_fwd(u, pc["w3"], None, pc["h"], pc["Dp"], layout=layout, want_state=want_state,
                                          hist_rows=hist)
        return hyena_ops.hyena_se_fwd(u, pc["w3"], None, pc["h"], layout=layout, want_state=want_state, hist_rows=hist)

    y_all, fs_all, st_all = call(pc["u"], 0)
    tol = 1e-6 if io == "f32" else 1e-3          # the 128-row tiles of a chunk start elsewhere: other summation order
    # (a) views
    ys = []
    for t0, t1 in zip(cuts[:-1], cuts[1:]):
        yc, fs, st = call(pc["u"][:, t0:t1], K + 1 if t0 else 0)
        ys.append(yc)
    ops.device_status()
    check("test_fused_gpu.py:432 torch.cat(ys, dim=1), y_all", rel_l2(torch.cat(ys, dim=1), y_all), tol)
    assert torch.equal(fs, fs_all) and torch.equal(st, st_all)
    # (b) staging buffer; chunks: the cuts, then the rest one short chunk at a time
    hist = K + 3
    stage = hyena_ops.PrefillChunks(B, max(b - a for a, b in zip(cuts[:-1], cuts[1:])), 3 * D, hist, device="cuda",
                                    dtype=pc["u"].dtype)
    ys = []
    for t0, t1 in zip(cuts[:-1], cuts[1:]):
        stage.rows(t1 - t0).copy_(pc["u"][:, t0:t1])        # stands for the projection GEMM of the chunk
        yc, fs, st = call(stage.rows(t1 - t0), stage.hist_rows)
        ys.append(yc)
        stage.advance(t1 - t0)
    ops.device_status()
    check("test_fused_gpu.py:445 torch.cat(ys, dim=1), y_all", rel_l2(torch.cat(ys, dim=1), y_all), tol)
    assert torch.equal(fs, fs_all) and torch.equal(st, st_all)
    with pytest.raises(ValueError):
        call(pc["u"][:, 200:300], K)                         # fewer history rows than the filter reaches back


def _group_state_ref(kv, lam, theta=None):
    """State after the last token of channels that share one modal system: kv [B, C, L] float64, lam (and theta) [S].
    The [S, L] weight table is built once (a per-channel table would not fit at full size)."""
    L = kv.shape[-1]
    e = L - 1 - np.arange(L, dtype=np.float64)
    w = np.exp(lam[:, None] * e)
    if theta is not None:
        w = w * np.exp(1j * theta[:, None] * e)
    return np.einsum("bcl,sl->bcs", kv, w)


@pytest.mark.parametrize("kind", ["grouped_complex", "per_channel_real"])
def test_fused_li_full_size_properties(kind):
    """Configuration 3 at its stated size (B=1, L=131072, D=4096, bf16) on both long-filter kernels: the tensor-core
    scan (one complex modal system per group of 16 channels: 256 walks, each cut into time slices that hand their
    state on through global memory) and the recurrence kernel (a real modal system per channel, Evo 2's own shape).
    FFT oracle of length 2L on a 32-channel slice including the state after the last token, channel-shard
    invariance, causality, and a clean device status."""
    from vortex_b200 import hyena_ops, ops
    B, L, D, S = 1, 131072, 4096, 16
    grouped = kind == "grouped_complex"
    G = D // 16 if grouped else D
    p = make_block(2, B, L, D, G, 0, "bf16", modal=True, S=S, complex_poles=grouped)
    pc = cuda(p)

    def run(u, c0=0, c1=D, want_state=False):
        g0, g1 = (c0 // 16, c1 // 16) if grouped else (c0, c1)
        kw = dict(theta=pc["theta"][g0:g1], res_im=pc["res_im"][g0:g1]) if grouped else {}
        return hyena_ops.hyena_li_fwd(u, pc["w3"][3 * c0:3 * c1], None, pc["log_poles"][g0:g1], pc["residues"][g0:g1],
                                      pc["Dp"][c0:c1], want_state=want_state, **kw)

    y, fs, st = run(pc["u"], want_state=True)
    ops.device_status()
    assert y.shape == (B, L, D) and y.dtype == torch.bfloat16
    # (1) FFT oracle on channels [d0, d1)
    d0, d1 = 2016, 2048
    g0, g1 = (d0 // 16, d1 // 16) if grouped else (d0, d1)
    sub = {"u": p["u"][:, :, 3 * d0:3 * d1], "w3": p["w3"][3 * d0:3 * d1], "log_poles": p["log_poles"][g0:g1],
           "residues": p["residues"][g0:g1], "Dp": p["Dp"][d0:d1]}
    if grouped:
        sub["theta"], sub["res_im"] = p["theta"][g0:g1], p["res_im"][g0:g1]
    ref, kv = _li_cc_oracle(sub, L, d1 - d0, g1 - g0, grouped, "bf16", "interleaved", 1, False, None)
    check(f"LI full size ({kind}) y vs FFT oracle", rel_l2(y[:, :, d0:d1], ref), TOL["bf16"])
    lam = to_np(sub["log_poles"])[..., 0].astype(np.float64)
    per = (d1 - d0) // (g1 - g0)
    for gi in range(g1 - g0):
        th = to_np(sub["theta"])[gi].astype(np.float64) if grouped else None
        want = _group_state_ref(kv[:, gi * per:(gi + 1) * per], lam[gi], th)
        got = to_np(st)[:, d0 + gi * per:d0 + (gi + 1) * per].astype(np.float64)
        if grouped:
            got = got[..., 0] + 1j * got[..., 1]
        err = np.linalg.norm(got - want) / np.linalg.norm(want)
        check(f"LI full size ({kind}) end state, system {gi}", err, 5e-5)
        if gi == 1:
            break
    assert np.array_equal(to_np(fs), to_np(p["u"])[:, L - 2:, :].transpose(0, 2, 1))
    # (2) a shard of channels computed as its own problem (what a rank of a channel-sharded run does)
    c0, c1 = 1024, 1536
    ys, _, _ = run(pc["u"][:, :, 3 * c0:3 * c1].contiguous(), c0, c1)
    ops.device_status()
    # (another number of walks / rows changes the time slicing, hence the fp32 summation order: last-place flips)
    check(f"LI full size ({kind}) shard vs full", rel_l2(ys, y[:, :, c0:c1]), 5e-4)
    # (3) causality
    t0 = 100003
    u2 = pc["u"].clone()
    u2[:, t0:] = -u2[:, t0:]
    y2, _, _ = run(u2)
    ops.device_status()
    assert torch.equal(y2[:, :t0], y[:, :t0]) and not torch.equal(y2[:, t0:], y[:, t0:])


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("kind", ["se", "mr", "li"])
def test_engine_fused_prefill_then_fused_decode(io, kind):
    """The engine's opt-in entry points on the reference's cache containers: fused_prefill (one pass over the
    projection output) then three fused_decode steps (one launch per token), against the reference's own sequence
    on the drop-in methods -- parallel_fir / parallel_iir, then step_fir -> interleave -> step_fir | step_iir
    (model.py:221-375).  The featurizer cache is a copy of the inputs (identical); the other caches and the outputs
    agree to the rounding the two-call sequence adds by materialising z and k*v in the I/O dtype."""
    from vortex_b200 import HyenaInferenceEngine
    from vortex_b200.cache import HyenaCascadeFIRInferenceParams, HyenaCascadeIIRInferenceParams
    li = kind == "li"
    B, L, D, G, S = 2, 300, 64, (64 if li else 4), 16
    K = {"se": 7, "mr": 128, "li": 0}[kind]
    if io == "f32" and kind == "mr":
        pytest.skip("the fused 128-tap block is the bf16 tensor-core kernel")
    p = cuda(make_block(71, B, L + 3, D, G, K, io, modal=li, S=S))
    dims = (D, 1, D, S, G)
    eng = HyenaInferenceEngine(layer_idx=4)
    new = HyenaCascadeIIRInferenceParams if li else HyenaCascadeFIRInferenceParams
    ca, cb = new(), new()
    u0 = p["u"][:, :L].contiguous()
    # ---- reference sequence on the drop-in methods
    z, ca.fir_state_dict[4] = eng.parallel_fir(F.conv1d, u0, p["w3"], None, L, dims=dims, gate=False, inference_params=ca)
    z = torch.cat([z[:, 0::3], z[:, 1::3], z[:, 2::3]], dim=1)
    if li:
        ya = eng.parallel_iir(z, None, p["Dp"], L, poles=p["log_poles"], residues=p["residues"], t=None, dims=dims,
                              layer_idx=4, inference_params=ca)
    else:
        hx = p["h"].repeat_interleave(D // G, 0)
        ya, ca.fir_inner_state_dict[4] = eng.parallel_fir(F.conv1d, z, hx, p["Dp"], L, dims=dims, gate=True,
                                                          gated_bias=K >= 128, dim_last=False, fir_length=K,
                                                          inference_params=ca, groups=G)
        ya = ya.permute(0, 2, 1)
    # ---- fused
    kw = dict(log_poles=p["log_poles"], residues=p["residues"]) if li else dict(h=p["h"])
    yb = eng.fused_prefill(u0, p["w3"], None, dims, D=p["Dp"], inference_params=cb, **kw)
    # bf16: the two-call sequence rounds z, k*v and the filter output to bf16 (it sits ~4e-3 from the un-rounded
    # evaluation, like the reference's own bf16 pipeline), the fused pass rounds once (1.7e-3): independent errors
    tol = 1e-5 if io == "f32" else 6e-3
    check(f"fused_prefill vs two-call prefill ({kind}, {io})", rel_l2(yb, ya), tol)
    assert torch.equal(ca.fir_state_dict[4], cb.fir_state_dict[4])
    for step in range(3):
        u = p["u"][:, L + step].contiguous()
        zs, ca.fir_state_dict[4] = eng.step_fir(u, ca.fir_state_dict[4], p["w3"])
        q, k, v = zs[:, 0::3], zs[:, 1::3], zs[:, 2::3]
        if li:
            ya, ca.state_dict[4] = eng.step_iir(q, k, v, p["Dp"], p["residues"], p["log_poles"], ca.state_dict[4])
            ya = ya.to(u.dtype)
        else:
            ya, ca.fir_inner_state_dict[4] = eng.step_fir(k * v, ca.fir_inner_state_dict[4], hx,
                                                          bias=p["Dp"] if K >= 128 else None, flip_filter=K >= 128,
                                                          gated_bias=K >= 128)
            ya = ya * q
        yb = eng.fused_decode(u, p["w3"], None, dims, cb, D=p["Dp"], **kw)
        assert yb.shape == (B, D) and yb.dtype == u.dtype
        check(f"fused_decode vs step sequence ({kind}, {io}, step {step})", rel_l2(yb, ya), 1e-5 if io == "f32" else 8e-3)
        assert torch.equal(ca.fir_state_dict[4], cb.fir_state_dict[4])
        sa, sb = (ca.state_dict[4], cb.state_dict[4]) if li else (ca.fir_inner_state_dict[4], cb.fir_inner_state_dict[4])
        assert sa.shape == sb.shape and sa.dtype == sb.dtype == torch.float32
        check(f"caches after decode step {step} ({kind}, {io})", rel_l2(sb, sa), 1e-5 if io == "f32" else 4e-3)


def test_device_status_reports_a_wait_that_ran_out():
    """Every wait in the kernels is bounded: a waiter that gives up records a code in the device status word, carries
    on and lets the launch end; the host then sees VTX_ERR_DEVICE as a RuntimeError.  Made observable on the one
    wait that polls plain global memory -- a time slice of a long-filter walk waiting for the slice before it --
    by cutting its poll limit to a single poll (the earlier slice needs microseconds, so the flag is not there yet).
    Nothing faults or hangs: the later slice just starts from a zero state, and the next launch is clean again."""
    from vortex_b200 import _lib, hyena_ops, ops
    B, L, D, S = 1, 15360, 32, 16           # two walks of two slices each
    p = make_block(43, B, L, D, D // 16, 0, "bf16", modal=True, S=S, complex_poles=True)
    pc = cuda(p)

    def run():
        return hyena_ops.hyena_li_fwd(pc["u"], pc["w3"], None, pc["log_poles"], pc["residues"], pc["Dp"],
                                      theta=pc["theta"], res_im=pc["res_im"])[0]
    good = run()
    ops.device_status()
    assert _lib.lib().vtx_debug_set_flag_poll_limit(1) == 0
    try:
        bad = run()
        with pytest.raises(RuntimeError, match="bounded wait"):
            ops.device_status()
    finally:
        assert _lib.lib().vtx_debug_set_flag_poll_limit(0) == 0
    assert bad.shape == good.shape
    ops.device_status()                      # the word was cleared by the read above
    assert torch.equal(run(), good)
    ops.device_status()


@pytest.mark.gpu
def test_launch_count_follows_the_kernels_a_call_launches():
    """vtx_launch_count: one launch for a short-filter block, three (segment states, carries, outputs) for a long-filter
    block whose sequence is cut into segments, one when a single segment covers it."""
    from vortex_b200 import hyena_ops, ops
    p = cuda(make_block(3, 2, 4096, 128, 8, 7, "bf16"))
    c0 = ops.launch_count()
    hyena_ops.hyena_se_fwd(p["u"], p["w3"], None, p["h"], want_state=False)
    assert ops.launch_count() - c0 == 1
    q = cuda(make_block(4, 1, 8192, 128, 128, 0, "bf16", modal=True, S=16, complex_poles=False))
    c0 = ops.launch_count()
    hyena_ops.hyena_li_fwd(q["u"], q["w3"], None, q["log_poles"], q["residues"], q["Dp"], want_state=False)
    assert ops.launch_count() - c0 == 3
    c0 = ops.launch_count()
    hyena_ops.hyena_li_fwd(q["u"][:, :64], q["w3"], None, q["log_poles"], q["residues"], q["Dp"], want_state=False)
    assert ops.launch_count() - c0 == 1
    ops.device_status()


@pytest.mark.gpu
def test_fused_mr_call_cut_into_launches():
    """A call large enough to be cut into several launches (24 sequences of 8192 tokens, 4096 channels: 6.4 GB moved)
    gives, bit for bit, what single-launch calls on slices of the batch give, caches included; the oracle agrees on a
    slice of channels of one sequence."""
    from vortex_b200 import hyena_ops, ops
    B, L, D, G, K = 24, 8192, 4096, 256, 128
    g = torch.Generator(device="cuda").manual_seed(11)
    u = torch.empty(B, L, 3 * D, device="cuda", dtype=torch.bfloat16)
    for b in range(B):
        u[b] = torch.randn(L, 3 * D, device="cuda", generator=g).bfloat16()
    w3 = (torch.randn(3 * D, 1, 3, device="cuda", generator=g) / 3 ** 0.5).bfloat16()
    h = (torch.randn(G, 1, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    Dp = torch.randn(D, device="cuda", generator=g).bfloat16()
    c0 = ops.launch_count()
    y, fs, st = hyena_ops.hyena_mr_fwd(u, w3, None, h, Dp, want_state=True)
    assert ops.launch_count() - c0 >= 2
    for b0 in range(0, B, 4):
        c0 = ops.launch_count()
        ys, fss, sts = hyena_ops.hyena_mr_fwd(u[b0:b0 + 4], w3, None, h, Dp, want_state=True)
        assert ops.launch_count() - c0 == 1
        assert torch.equal(ys, y[b0:b0 + 4]) and torch.equal(fss, fs[b0:b0 + 4]) and torch.equal(sts, st[b0:b0 + 4])
    ops.device_status()
    d0, d1, b = 3008, 3040, 17
    sub = {"u": u[b:b + 1, :, 3 * d0:3 * d1].cpu(), "w3": w3[3 * d0:3 * d1].cpu(), "h": h[d0 // 16:d1 // 16].cpu(),
           "Dp": Dp[d0:d1].cpu()}
    ref, _, _ = _oracle(sub, d1 - d0, K, "bf16", "interleaved")
    check("call cut into launches: y[b, :, d0:d1], ref", rel_l2(y[b:b + 1, :, d0:d1], ref), TOL["bf16"])


@pytest.mark.gpu
@pytest.mark.parametrize("kind,layout,heads,flip,flip_filter,with_b3,G", [
    ("mr", "split", 1, True, False, True, 12),            # taps not flipped, q and k swapped, featurizer bias, groups of 8
    ("mr", "column_split", 4, False, True, False, 6),
    ("se", "interleaved", 1, True, True, True, 24),       # q and k swapped on the interleaved fast path, groups of 4
    ("se", "split", 1, False, False, False, 6),
    ("li", "column_split", 2, True, False, True, 96),
])
def test_decode_layer_variants_match_step_sequence(kind, layout, heads, flip, flip_filter, with_b3, G):
    """The specialised one-token kernels under the other channel maps, tap orders and with a featurizer bias, against
    the step sequence of the drop-in engine (bf16 I/O, fp32 caches from the second step on)."""
    from vortex_b200 import HyenaInferenceEngine, ops
    eng = HyenaInferenceEngine()
    B, D = 2, 96
    K = {"se": 7, "mr": 128, "li": 0}[kind]
    g = torch.Generator().manual_seed(23)
    dt = torch.bfloat16
    w3 = (torch.randn(3 * D, 1, 3, generator=g) / 3 ** 0.5).to(dt).cuda()
    b3 = (0.1 * torch.randn(3 * D, generator=g)).to(dt).cuda() if with_b3 else None
    fs = torch.randn(B, 3 * D, 2, generator=g).to(dt).cuda()
    Dp = torch.randn(D, generator=g).to(dt).cuda()
    if kind == "li":
        lp = torch.log(0.9 + 0.099 * torch.rand(G, 16, 1, generator=g)).cuda()
        R = torch.randn(G, 16, generator=g).cuda()
        st = torch.randn(B, D, 16, generator=g).cuda()
    else:
        h = (torch.randn(G, 1, K, generator=g) / K ** 0.5).to(dt).cuda()
        st = torch.randn(B, D, K - 1, generator=g).to(dt).cuda()

    def qkv(z):
        if layout == "interleaved":
            q, k, v = z[:, 0::3], z[:, 1::3], z[:, 2::3]
        elif layout == "split":
            q, k, v = z[:, :D], z[:, D:2 * D], z[:, 2 * D:]
        else:
            z4 = z.reshape(B, heads, 3, D // heads)
            q, k, v = (z4[:, :, i].reshape(B, D) for i in range(3))
        return (k, q, v) if flip else (q, k, v)

    fs_a, st_a, fs_b, st_b = fs, st, fs, st
    for step in range(3):
        u = torch.randn(B, 3 * D, generator=g).to(dt).cuda()
        z, fs_a = eng.step_fir(u, fs_a, w3, bias=b3)
        q, k, v = qkv(z)
        if kind == "li":
            ya, st_a = eng.step_iir(q, k, v, Dp, R.repeat_interleave(D // G, 0), lp.repeat_interleave(D // G, 0), st_a)
            ya = ya.to(dt)
            yb, fs_b, st_b = ops.decode_layer(u, w3, b3, fs_b, D, log_poles=lp, residues=R, bias=Dp, iir_state=st_b,
                                              layout=layout, num_heads=heads, flip=flip)
        else:
            ya, st_a = eng.step_fir(k * v, st_a, h.repeat_interleave(D // G, 0), bias=Dp if K >= 128 else None,
                                    flip_filter=flip_filter, gated_bias=K >= 128)
            ya = ya * q
            yb, fs_b, st_b = ops.decode_layer(u, w3, b3, fs_b, D, h=h, inner_state=st_b, bias=Dp if K >= 128 else None,
                                              flip_filter=flip_filter, gated_bias=K >= 128, layout=layout, num_heads=heads,
                                              flip=flip)
        assert torch.equal(fs_a, fs_b)
        check(f"decode variants {kind}/{layout} step {step}: y", rel_l2(yb, ya), 2e-3)
        check(f"decode variants {kind}/{layout} step {step}: state", rel_l2(st_b, st_a), 1e-6)
    ops.device_status()
