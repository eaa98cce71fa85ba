"""GPU parity: the drop-in engine (CUDA kernels through the C ABI) against the reference's golden
vectors and against the CPU oracle on seeded inputs.  Tolerances are the stated ones: relative L2
<= 1e-4 for fp32 I/O, <= 2e-3 for bf16 I/O against the reference's own path (its golden vectors, or the
oracle with the reference's rounding points); pure-copy caches bit-exact.  The drop-in methods round where
the reference does, so against its bf16 vectors they are bit-identical or differ in single last-place flips;
the few wider bounds below compare quantities that are each rounded to bf16 on their own, and say so."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from helpers import DT, TOL, check, cuda, make_block, rel_l2, to_np
from oracle import hyena_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from vortex_b200 import HyenaInferenceEngine
    return HyenaInferenceEngine(layer_idx=3)


class _P:
    def __init__(self):
        self.state_dict, self.fir_state_dict, self.fir_inner_state_dict = {}, {}, {}


def T(a, io):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DT[io]).cuda()


# ------------------------------------------------------------------ golden vectors of the reference
@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("L", [1, 2, 50])
@pytest.mark.parametrize("tag", ["nobias", "bias"])
def test_golden_featurizer(golden, eng, io, L, tag):
    k = f"feat_{io}_L{L}_{tag}"
    z, st = eng.parallel_fir(F.conv1d, T(golden[k + "_u"], io), T(golden[k + "_w"], io),
                             T(golden[k + "_b"], io) if tag == "bias" else None, L, dims=(16, 1, 16, 16, 16),
                             gate=False, dim_last=True, fir_length=3, inference_params=True)
    assert z.shape == golden[k + "_z"].shape and z.dtype == DT[io]
    check("test_engine_gpu.py:40 z, golden[k + '_z']", rel_l2(z, golden[k + "_z"]), (1e-6 if io == "f32" else 2e-3))
    assert np.array_equal(to_np(st), golden[k + "_state"])
    z2, st2 = eng.parallel_fir(F.conv1d, T(golden[k + "_u"], io), T(golden[k + "_w"], io), None, L,
                               dims=(16, 1, 16, 16, 16), gate=False, inference_params=None)
    assert st2 is None


GCG = [(7, 50, "split"), (7, 4, "split"), (4, 33, "interleaved"), (128, 300, "split"),
       (128, 100, "interleaved"), (7, 40, "column_split"), (128, 200, "column_split")]


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("K,L,layout", GCG)
def test_golden_gate_conv_gate(golden, io, K, L, layout):
    from vortex_b200 import HyenaInferenceEngine
    from oracle.torch_port import _qkv  # noqa: F401  (only to mirror the caller's interleave below)

    k = f"gcg_{io}_K{K}_L{L}_{layout}"
    D, G, H = 32, 2, 4
    z = T(golden[k + "_z"], io)
    if layout == "interleaved":   # what HyenaCascade does before the call (model.py:251-252)
        z = torch.cat([z[:, 0::3], z[:, 1::3], z[:, 2::3]], dim=1)
    h = T(golden[k + "_h"], io).repeat_interleave(D // G, 0)
    eng = HyenaInferenceEngine(hyena_flip_x1x2=layout == "column_split")
    y, st = eng.parallel_fir(F.conv1d, z, h, T(golden[k + "_D"], io) if K >= 128 else None, L,
                             dims=(D, H, D // H, 16, G), gate=True, gated_bias=K >= 128, dim_last=False,
                             column_split_hyena=layout == "column_split", fir_length=K, inference_params=True,
                             groups=G)
    assert y.shape == golden[k + "_y"].shape and y.dtype == DT[io]
    check("test_engine_gpu.py:69 y, golden[k + '_y']", rel_l2(y, golden[k + "_y"]), (1e-5 if io == "f32" else 2e-3))
    assert st.shape == golden[k + "_state"].shape
    assert np.array_equal(to_np(st), golden[k + "_state"])


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("L,layout", [(200, "split"), (64, "interleaved")])
def test_golden_long_conv(golden, eng, io, L, layout):
    k = f"iir_{io}_L{L}_{layout}"
    D, S = 16, 16
    z = T(golden[k + "_z"], io)
    if layout == "interleaved":
        z = torch.cat([z[:, 0::3], z[:, 1::3], z[:, 2::3]], dim=1)
    ip = _P()
    lp, R = T(golden[k + "_lp"], "f32"), T(golden[k + "_R"], "f32")
    y = eng.parallel_iir(z, T(golden[k + "_h"], "f32"), T(golden[k + "_D"], io), L, poles=lp, residues=R,
                         t=None, dims=(D, 1, D, S, D), layer_idx=3, inference_params=ip, prefill_style="fft")
    assert y.shape == (2, L, D) and y.dtype == DT[io]
    check("test_engine_gpu.py:87 y, golden[k + '_y']", rel_l2(y, golden[k + "_y"]), (2e-5 if io == "f32" else 2e-3))
    assert ip.state_dict[3].dtype == torch.float32 and ip.state_dict[3].shape == (2, D, S)
    check("test_engine_gpu.py:89 ip.state_dict[3], golden[k + '_state']", rel_l2(ip.state_dict[3], golden[k + "_state"]), 2e-5)
    y2 = eng.parallel_iir(z, None, T(golden[k + "_D"], io), L, poles=lp, residues=R, t=None,
                          dims=(D, 1, D, S, D), layer_idx=3, inference_params=None)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("io", ["f32", "bf16"])
def test_golden_recurrence_prefill(golden, io):
    """parallel_iir(prefill_style="recurrence") -> the reference's prefill_via_direct_recurrence (engine.py:473-504):
    legacy complex poles [D, S, 1, 2], state in the I/O dtype, real part updated before the imaginary part reads it.
    The state lands in state_dict[engine.layer_idx] (not the layer_idx argument), as in the reference."""
    from vortex_b200 import HyenaInferenceEngine
    k = f"iirrec_{io}"
    D, S, L = 12, 16, 48
    eng5 = HyenaInferenceEngine(layer_idx=5)
    ip = _P()
    y = eng5.parallel_iir(T(golden[k + "_z"], io), None, T(golden[k + "_D"], io), L, poles=T(golden[k + "_p"], "f32"),
                          residues=T(golden[k + "_R"], "f32"), t=None, dims=(D, 1, D, S, D), layer_idx=9,
                          inference_params=ip, prefill_style="recurrence")
    assert y.shape == (2, L, D) and y.dtype == DT[io]
    check(f"recurrence y {io}", rel_l2(y, golden[k + "_y"]), 2e-6 if io == "f32" else 2e-3)
    st = ip.state_dict[5]
    assert st.dtype == torch.float32 and st.shape == (2, D, S, 2) and 9 not in ip.state_dict
    if io == "bf16":        # every state value is a bf16 number: bit-exact unless an fp32 sum differs in its last bit
        check("recurrence state bf16", rel_l2(st, golden[k + "_state"]), 1e-3)
    else:
        check("recurrence state f32", rel_l2(st, golden[k + "_state"]), 2e-6)


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("thr", [24, 160])
def test_golden_long_fir_threshold(golden, eng, io, thr):
    """parallel_iir(long_fir_threshold=...) (engine.py:339-349): the filter cut to its first samples, applied the
    way F.conv1d applies it."""
    k = f"iirfir_{io}_thr{thr}"
    D, S, L = 16, 16, 200
    lp, R = T(golden[k + "_lp"], "f32"), T(golden[k + "_R"], "f32")
    y = eng.parallel_iir(T(golden[k + "_z"], io), T(golden[k + "_h"], "f32"), T(golden[k + "_D"], io), L, poles=lp,
                         residues=R, t=None, dims=(D, 1, D, S, D), layer_idx=0, inference_params=None,
                         long_fir_threshold=thr)
    assert y.shape == (1, L, D) and y.dtype == DT[io]
    check(f"long_fir_threshold {thr} {io}", rel_l2(y, golden[k + "_y"]), 2e-6 if io == "f32" else 2e-3)
    with pytest.raises(AssertionError):          # batch size must be 1 (engine.py:340)
        eng.parallel_iir(T(golden[k + "_z"], io), T(golden[k + "_h"], "f32").expand(2, -1, -1), None, L, poles=lp,
                         residues=R, t=None, dims=(D, 1, D, S, D), layer_idx=0, long_fir_threshold=thr)


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("K,c0,flip,gb", [(3, 2, False, False), (3, 1, False, False), (7, 6, False, False),
                                          (7, 3, False, False), (128, 127, True, True), (128, 20, True, True)])
def test_golden_step_fir(golden, eng, io, K, c0, flip, gb):
    k = f"stepfir_{io}_K{K}_c{c0}"
    w = T(golden[k + "_w"], io)
    b = T(golden[k + "_b"], io) if gb else None
    st = T(golden[k + "_state0"], io)       # the prefill hands the cache over in the I/O dtype
    for i in range(3):
        y, st = eng.step_fir(T(golden[f"{k}_u{i}"], io), st, w, bias=b, gated_bias=gb, flip_filter=flip)
        assert y.dtype == DT[io] and st.dtype == torch.float32
        check(f"test_engine_gpu.py:147 y, golden[f'{k}_y{i}']", rel_l2(y, golden[f"{k}_y{i}"]), (2e-6 if io == "f32" else 2e-3))
        assert st.shape == golden[f"{k}_state{i + 1}"].shape
        assert np.array_equal(to_np(st), golden[f"{k}_state{i + 1}"])   # cache layout and values bit-exact


@pytest.mark.parametrize("io", ["f32", "bf16"])
def test_golden_step_iir(golden, eng, io):
    k = f"stepiir_{io}"
    lp, R, Dp = T(golden[k + "_lp"], "f32"), T(golden[k + "_R"], "f32"), T(golden[k + "_D"], io)
    st = T(golden[k + "_state0"], "f32")
    for i in range(3):
        y, st = eng.step_iir(T(golden[f"{k}_x2{i}"], io), T(golden[f"{k}_x1{i}"], io), T(golden[f"{k}_v{i}"], io),
                             Dp, R, lp, st)
        assert y.dtype == torch.float32
        check("test_engine_gpu.py:161 y, golden[f'(k)_y(i)']", rel_l2(y, golden[f"{k}_y{i}"]), 2e-6)
        check("test_engine_gpu.py:162 st, golden[f'(k)_state(i + 1)']", rel_l2(st, golden[f"{k}_state{i + 1}"]), 2e-6)
    with pytest.raises(NotImplementedError):
        eng.step_iir(st[..., 0], st[..., 0], st[..., 0], Dp, R, lp, st, iir_groups=2)


@pytest.mark.parametrize("hl", [4, 32, 128])
def test_golden_hyena_ops_layout(golden, hl):
    from vortex_b200 import hyena_ops

    k = f"ops_hl{hl}"
    y = hyena_ops.gcg_fwd(T(golden[k + "_x"], "f32"), T(golden[k + "_B"], "f32"), T(golden[k + "_C"], "f32"),
                          T(golden[k + "_h"], "f32"))
    assert y.shape == golden[k + "_y"].shape
    check("test_engine_gpu.py:175 y, golden[k + '_y']", rel_l2(y, golden[k + "_y"]), 1e-5)
    check("test_engine_gpu.py:176 y, golden[k + '_y_chunked']", rel_l2(y, golden[k + "_y_chunked"]), 1e-5)


@pytest.mark.parametrize("hl", [4, 32, 128])
def test_golden_hyena_ops_backward(golden, hl):
    """two_pass_bwd_grouped against the reference's own backward (fp32 vectors of ref_bwd.py), and through autograd."""
    from vortex_b200 import hyena_ops

    k = f"opsbwd_hl{hl}"
    t = {n: T(golden[f"{k}_{n}"], "f32") for n in ("dy", "x", "B", "C", "h", "y2")}
    grads = hyena_ops.two_pass_bwd_grouped(t["dy"], t["x"], t["B"], t["C"], t["h"], t["y2"], version="v2", CHUNK_SIZE=128)
    for name, got in zip(("dx", "dB", "dC", "dh"), grads):
        assert got.shape == golden[f"{k}_{name}"].shape
        check(f"hyena_ops backward hl={hl} {name} vs the reference's", rel_l2(got, golden[f"{k}_{name}"]), 1e-5)
    # without the saved filter output, and through the autograd function of the interface
    grads2 = hyena_ops.gcg_bwd(t["dy"], t["x"], t["B"], t["C"], t["h"])
    leaves = [t[n].clone().requires_grad_(True) for n in ("x", "B", "C", "h")]
    y = hyena_ops.two_pass_chunked_gate_conv_gate(*leaves)
    y.backward(t["dy"])
    for name, a, b in zip(("dx", "dB", "dC", "dh"), grads2, leaves):
        check(f"hyena_ops backward hl={hl} {name}, recomputed y2", rel_l2(a, golden[f"{k}_{name}"]), 1e-5)
        check(f"hyena_ops backward hl={hl} {name}, autograd", rel_l2(b.grad, golden[f"{k}_{name}"]), 1e-5)


@pytest.mark.parametrize("io,bs,l,g,dg,hl", [("bf16", 2, 1000, 4, 16, 7), ("bf16", 1, 777, 3, 24, 128), ("f16", 2, 300, 5, 1, 33),
                                             ("f32", 1, 4099, 2, 64, 128), ("bf16", 3, 5, 2, 16, 128)])
def test_hyena_ops_backward_vs_oracle(io, bs, l, g, dg, hl):
    """Seeded shapes the golden vectors do not cover: ragged lengths, groups of 1 / 24 / 64 channels, 16-bit I/O,
    sequences shorter than the filter."""
    from vortex_b200 import hyena_ops

    gen = torch.Generator().manual_seed(77)
    x, Bm, Cm, dy = (torch.randn(bs, l, g, dg, generator=gen).to(DT[io]) for _ in range(4))
    h = (torch.randn(g, 1, hl, generator=gen) / hl ** 0.5).to(DT[io])
    ref = O.gcg_blgdg_bwd(to_np(dy), to_np(x), to_np(Bm), to_np(Cm), to_np(h))
    got = hyena_ops.gcg_bwd(dy.cuda(), x.cuda(), Bm.cuda(), Cm.cuda(), h.cuda())
    tol = 1e-4 if io == "f32" else TOL["bf16"] if io == "bf16" else 5e-4
    for name, a, b in zip(("dx", "dB", "dC", "dh"), got, ref):
        assert a.shape == b.shape and a.dtype == DT[io]
        # dC = dy * y2, where the forward that recomputes y2 rounds B * x and y2 to the I/O dtype as the reference
        # materialises them: three independent roundings (sqrt(3) x one) on as few as 480 values
        check(f"hyena_ops backward {io} {name} vs oracle", rel_l2(a, b), tol * (2.5 if name == "dC" else 1.0))


# ------------------------------------------------------------------ seeded parity against the oracle
def _engine_block(eng, p, D, G, K, layout, ip=None, heads=1):
    """The reference's two-call sequence (model.py:233-291) on the drop-in engine."""
    dims = (D, heads, D // heads, 16, G)
    z, fs = eng.parallel_fir(F.conv1d, p["u"], p["w3"], None, p["u"].shape[1], dims=dims, gate=False,
                             dim_last=True, fir_length=3, inference_params=ip)
    if layout == "interleaved":
        z = torch.cat([z[:, 0::3], z[:, 1::3], z[:, 2::3]], dim=1)
    h = p["h"].repeat_interleave(D // G, 0)
    y, st = eng.parallel_fir(F.conv1d, z, h, p["Dp"], z.shape[-1], dims=dims, gate=True, gated_bias=K >= 128,
                             dim_last=False, column_split_hyena=layout == "column_split", fir_length=K,
                             inference_params=ip, groups=G)
    return y.permute(0, 2, 1), fs, st


@pytest.mark.parametrize("io,B,L,D,G,K,layout", [
    ("f32", 1, 2048, 768, 48, 7, "split"),          # configuration 1 at full size
    ("bf16", 2, 1000, 256, 16, 7, "interleaved"),
    ("bf16", 1, 2048, 256, 16, 128, "interleaved"),  # configuration 2 shape, reduced B / D
    ("f32", 1, 700, 128, 8, 128, "split"),
    ("f16", 1, 513, 64, 4, 7, "interleaved"),
])
def test_engine_block_vs_oracle(eng, io, B, L, D, G, K, layout):
    p = make_block(7, B, L, D, G, K, io)
    args = (to_np(p["u"]), to_np(p["w3"]), to_np(p["h"]), None if p["Dp"] is None else to_np(p["Dp"]), D, K)
    ref, fs_ref, st_ref = O.hyena_fused(*args, io=io, layout=layout, mirror=True)
    y, fs, st = _engine_block(eng, cuda(p), D, G, K, layout, ip=True)
    assert y.shape == (B, L, D)
    # the two-call sequence materialises z and k*v in the I/O dtype exactly where the reference does:
    # against the reference's own path for that dtype only last-bit flips remain
    check("test_engine_gpu.py:209 y, ref", rel_l2(y, ref), TOL[io])
    assert np.array_equal(to_np(fs), fs_ref.astype(np.float32))      # pure copy of the input: bit-exact
    assert st.shape == st_ref.shape
    check("test_engine_gpu.py:212 st, st_ref", rel_l2(st, st_ref), TOL[io])
    # distance to the un-rounded fp32 evaluation: what the reference's own 16-bit pipeline has too
    # (z, k*v, the filter output and y are each rounded, ~1.7e-3 apiece for bf16)
    wide, _, _ = O.hyena_fused(*args, io=io, layout=layout, mirror=False)
    check("test_engine_gpu.py:216 y, wide", rel_l2(y, wide), {"f32": 1e-4, "bf16": 5e-3, "f16": 7e-4}[io])


def test_integer_inputs_are_exact(eng):
    """With small-integer inputs every product and sum is exact in fp32 and bf16, so outputs and caches
    must equal the oracle bit for bit -- this pins tap order, q/k/v maps and cache indexing."""
    g = torch.Generator().manual_seed(11)
    B, L, D, G = 2, 96, 64, 4
    for K, io in ((7, "f32"), (7, "bf16"), (128, "f32")):
        u = torch.randint(-2, 3, (B, L, 3 * D), generator=g).float()
        w3 = torch.randint(-1, 2, (3 * D, 1, 3), generator=g).float()
        h = torch.randint(-1, 2, (G, 1, K), generator=g).float()
        if K == 128:
            h[:, :, 5:] = 0      # keep the sums small enough to stay exact
        Dp = torch.randint(-1, 2, (D,), generator=g).float() if K >= 128 else None
        p = {"u": u.to(DT[io]), "w3": w3.to(DT[io]), "h": h.to(DT[io]), "Dp": None if Dp is None else Dp.to(DT[io])}
        for layout in ("split", "interleaved"):
            ref, fs_ref, st_ref = O.hyena_fused(to_np(u), to_np(w3), to_np(h), None if Dp is None else to_np(Dp),
                                                D, K, io=io, layout=layout, mirror=True)
            y, fs, st = _engine_block(eng, cuda(p), D, G, K, layout, ip=True)
            if io == "f32":
                assert np.array_equal(to_np(y), ref.astype(np.float32))
            else:
                check("test_engine_gpu.py:239 y, ref", rel_l2(y, ref), 2e-3)   # bf16 outputs can exceed the exactly representable range
            assert np.array_equal(to_np(fs), fs_ref.astype(np.float32))
            assert np.array_equal(to_np(st), st_ref.astype(np.float32))


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("K", [7, 128])
def test_prefill_then_decode_matches_longer_prefill(eng, io, K):
    """engine.step_fir on the caches left by a prefill over L tokens reproduces token L of a prefill
    over L+1 tokens (the reference's own consistency property, checked in its golden vectors too)."""
    B, L, D, G = 2, 300, 64, 4
    p = cuda(make_block(5, B, L + 1, D, G, K, io))
    full, _, _ = _engine_block(eng, p, D, G, K, "interleaved")
    pre = dict(p, u=p["u"][:, :L].contiguous())
    _, fs, st = _engine_block(eng, pre, D, G, K, "interleaved", ip=True)
    assert fs.dtype == DT[io] and st.dtype == DT[io]
    z, fs2 = eng.step_fir(p["u"][:, L], fs, p["w3"])
    q, k, v = z[:, 0::3], z[:, 1::3], z[:, 2::3]
    y, st2 = eng.step_fir(k * v, st, p["h"].repeat_interleave(D // G, 0), bias=p["Dp"], flip_filter=K >= 128,
                          gated_bias=K >= 128)
    y = y * q
    assert fs2.dtype == torch.float32 and st2.dtype == torch.float32 and st2.shape == st.shape
    check("test_engine_gpu.py:261 y, full[:, L]", rel_l2(y, full[:, L]), (1e-5 if io == "f32" else 2e-3))
    assert torch.equal(st2[..., :-1], st[..., 1:].float()) and torch.equal(st2[..., -1], (k * v).float())


@pytest.mark.parametrize("io", ["f32", "bf16"])
def test_long_conv_vs_oracle_and_decode(eng, io):
    B, L, D, S = 2, 1500, 48, 16
    p = make_block(9, B, L + 1, D, D, 0, io, modal=True, S=S)
    pc = cuda(p)
    dims = (D, 1, D, S, D)

    def run(u, ip):
        z, fs = eng.parallel_fir(F.conv1d, u, pc["w3"], None, u.shape[1], dims=dims, gate=False, inference_params=ip)
        z = torch.cat([z[:, 0::3], z[:, 1::3], z[:, 2::3]], dim=1)
        y = eng.parallel_iir(z, None, pc["Dp"], u.shape[1], poles=pc["log_poles"], residues=pc["residues"], t=None,
                             dims=dims, layer_idx=3, inference_params=ip)
        return y, z, fs

    y_full, z_full, _ = run(pc["u"], None)
    zf, _ = O.featurizer(to_np(p["u"]), to_np(p["w3"]), io=io, mirror=True)
    zi = np.concatenate([zf[:, 0::3], zf[:, 1::3], zf[:, 2::3]], axis=1)
    h = O.modal_filter(to_np(p["log_poles"]), to_np(p["residues"]), L + 1)
    ref, kv = O.long_conv_gate(zi, h, to_np(p["Dp"]), D, io=io, mirror=True)
    check("test_engine_gpu.py:284 y_full, ref", rel_l2(y_full, ref), TOL[io])          # the reference's own pipeline for this dtype
    wide, _ = O.long_conv_gate(zi, h, to_np(p["Dp"]), D, io=io, mirror=False)
    check("test_engine_gpu.py:286 y_full, wide", rel_l2(y_full, wide), (1e-4 if io == "f32" else 5e-3))
    ip = _P()
    y_pre, _, fs = run(pc["u"][:, :L].contiguous(), ip)
    st_ref = O.modal_state(O.round_io(kv[..., :L], io), to_np(p["log_poles"]))
    check("test_engine_gpu.py:290 ip.state_dict[3], st_ref", rel_l2(ip.state_dict[3], st_ref), (3e-5 if io == "f32" else 2e-3))
    # one decode step continues the prefill
    z, _ = eng.step_fir(pc["u"][:, L], fs, pc["w3"])
    q, k, v = z[:, 0::3], z[:, 1::3], z[:, 2::3]
    y, st = eng.step_iir(q, k, v, pc["Dp"], pc["residues"], pc["log_poles"], ip.state_dict[3])
    check("test_engine_gpu.py:295 y, y_full[:, L]", rel_l2(y, y_full[:, L]), (1e-4 if io == "f32" else 4e-3))   # bf16: step_iir returns fp32, the prefill output was rounded to bf16 after its own differently ordered sum: two roundings apart


def test_long_conv_segmented_and_complex(eng):
    """B*D too small to fill the GPU -> the time axis is cut into segments with a carry scan; also the
    complex-pole variant (h = sum Re(R p^t)) against the oracle's direct evaluation."""
    from vortex_b200 import ops

    B, L, D, G, S = 1, 6000, 32, 2, 16
    p = make_block(13, B, L, D, G, 0, "f32", modal=True, S=S, complex_poles=True)
    pc = cuda(p)
    g = torch.Generator().manual_seed(3)
    z = torch.randn(B, 3 * D, L, generator=g)
    poles = np.exp(to_np(p["log_poles"])[..., 0]) * np.exp(1j * to_np(p["theta"]))
    res = to_np(p["residues"]) + 1j * to_np(p["res_im"])
    h = np.repeat(O.modal_filter_complex(poles, res, L), D // G, axis=0)
    ref, kv = O.long_conv_gate(to_np(z), h, to_np(p["Dp"]), D, io="f32", mirror=False)
    y, st = ops.iir_fwd(z.cuda(), pc["log_poles"], pc["residues"], pc["Dp"], D, theta=pc["theta"], res_im=pc["res_im"])
    check("test_engine_gpu.py:313 y.permute(0, 2, 1), ref", rel_l2(y.permute(0, 2, 1), ref), 1e-4)
    st_ref = O.modal_state_complex(kv, np.repeat(poles, D // G, axis=0))
    got = to_np(st)
    check("test_engine_gpu.py:316 got[..., 0], st_ref.real) <= 1e-4 and rel_l2(got[..., 1], st_ref.imag", rel_l2(got[..., 0], st_ref.real) <= 1e-4 and rel_l2(got[..., 1], st_ref.imag), 1e-4)
    hf = ops.modal_filter(pc["log_poles"], pc["residues"], 4096, theta=pc["theta"], res_im=pc["res_im"])
    check("test_engine_gpu.py:318 hf, O.modal_filter_complex(poles, res, 4096)", rel_l2(hf, O.modal_filter_complex(poles, res, 4096)), 1e-4)
    # real poles, grouped, segmented
    y2, st2 = ops.iir_fwd(z.cuda(), pc["log_poles"], pc["residues"], pc["Dp"], D)
    h2 = np.repeat(O.modal_filter(to_np(p["log_poles"]), to_np(p["residues"]), L), D // G, axis=0)
    ref2, kv2 = O.long_conv_gate(to_np(z), h2, to_np(p["Dp"]), D, io="f32", mirror=False)
    check("test_engine_gpu.py:323 y2.permute(0, 2, 1), ref2", rel_l2(y2.permute(0, 2, 1), ref2), 1e-4)
    check("test_engine_gpu.py:324 st2, O.modal_state(kv2, np.repeat(to_np(p['log_poles'])[..., 0], D // G, axis=0))", rel_l2(st2, O.modal_state(kv2, np.repeat(to_np(p["log_poles"])[..., 0], D // G, axis=0))), 1e-4)


def test_padding_mask_and_errors(eng):
    B, L, D, G, K = 2, 40, 32, 2, 7
    p = cuda(make_block(21, B, L, D, G, K, "f32"))
    mask = (torch.rand(B, L) > 0.3).float().cuda()
    dims = (D, 1, D, 16, G)
    z, _ = eng.parallel_fir(F.conv1d, p["u"], p["w3"], None, L, dims=dims, gate=False, padding_mask=mask)
    z0, _ = eng.parallel_fir(F.conv1d, p["u"], p["w3"], None, L, dims=dims, gate=False)
    assert torch.equal(z, z0 * mask[:, None])
    h = p["h"].repeat_interleave(D // G, 0)
    y, _ = eng.parallel_fir(F.conv1d, z0, h, None, L, dims=dims, gate=True, dim_last=False, fir_length=K,
                            padding_mask=mask)
    y0, _ = eng.parallel_fir(F.conv1d, z0, h, None, L, dims=dims, gate=True, dim_last=False, fir_length=K)
    assert torch.allclose(y, y0 * mask[:, None], atol=1e-6)
    with pytest.raises(AttributeError):   # the reference dereferences the missing skip parameter
        eng.parallel_fir(F.conv1d, z0, torch.zeros(D, 1, 128).cuda(), None, L, dims=dims, gate=True, dim_last=False,
                         fir_length=128)
    with pytest.raises(NotImplementedError):
        eng.parallel_fir(lambda x: x, p["u"], p["w3"], None, L, dims=dims)
    with pytest.raises(NotImplementedError):
        eng.parallel_iir(z0, None, p["u"][0, 0, :D], L, poles=None, residues=None, t=None, dims=dims, layer_idx=0,
                         use_flashfft=True)


@pytest.mark.parametrize("io,B,D,L,Lh", [("bf16", 2, 24, 75, 16), ("bf16", 3, 64, 256, 4), ("f32", 1, 8, 33, 7),
                                         ("bf16", 1, 16, 8, 16), ("f16", 2, 8, 1, 3)])
def test_hyena_x_vs_oracle(io, B, D, L, Lh):
    """Hyena-X (depthwise FIR on q, k, v and three-way gate) against the oracle with the reference's roundings."""
    import torch
    from helpers import DT, rel_l2, to_np
    from oracle import hyena_oracle as O
    from vortex_b200 import hyena_ops
    g = torch.Generator().manual_seed(77)
    qkv = (torch.rand(B, 3 * D, L, generator=g) - 0.5).to(DT[io])
    h = (torch.rand(3 * D, 1, Lh, generator=g) - 0.5).to(DT[io])
    y = hyena_ops.hyena_x_fwd(qkv.cuda(), h.cuda())
    ref = O.hyena_x(to_np(qkv), to_np(h), io=io)
    assert y.shape == (B, D, L) and y.dtype == DT[io]
    check("test_engine_gpu.py:364 y, ref", rel_l2(y, ref), {"f32": 2e-6, "bf16": 2e-3, "f16": 1e-3}[io])
    q, k, v = qkv.cuda().split([D, D, D], dim=1)
    assert torch.equal(hyena_ops.hyena_x_bdl_fwd(q, k, v, h.cuda()), y)


# ------------------------------------------------------------------ short causal convolution of the conv extension
CC_TOL = {"f32": 2e-6, "bf16": 2e-3, "f16": 1e-3}


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("L", [1, 2, 37])
def test_golden_causal_conv1d(golden, io, W, L):
    """The reference's causal_conv1d_ref vectors: plain, and bias + initial states + SiLU; final states bit-exact."""
    from vortex_b200 import hyena_ops
    k = f"cc1d_{io}_W{W}_L{L}"
    x, w, b, ini = (T(golden[k + s], io) for s in ("_x", "_w", "_b", "_ini"))
    y = hyena_ops.causal_conv1d_fn(x, w)
    assert y.shape == x.shape and y.dtype == DT[io]
    check("test_engine_gpu.py:383 y, golden[k + '_y_plain']", rel_l2(y, golden[k + "_y_plain"]), CC_TOL[io])
    xl = x.transpose(1, 2).contiguous().transpose(1, 2)               # channel-last, as initial states require
    il = ini.transpose(1, 2).contiguous().transpose(1, 2)
    fs = torch.empty_like(il)
    y = hyena_ops.causal_conv1d_fn(xl, w, b, None, il, fs, "silu")
    assert y.stride() == xl.stride()
    check("test_engine_gpu.py:389 y, golden[k + '_y_full']", rel_l2(y, golden[k + "_y_full"]), 2.5 * CC_TOL[io])
    # (wider: causal_conv1d_ref rounds to the I/O dtype BEFORE the SiLU and again after it, the extension's kernel --
    # which this operator replaces -- rounds once; the vectors hold 12..444 numbers, so single flips weigh a lot)
    assert np.array_equal(to_np(fs), golden[k + "_fs_full"])


@pytest.mark.parametrize("io,B,D,L,W,cl", [("bf16", 2, 64, 1000, 4, True), ("bf16", 3, 40, 513, 3, False),
                                            ("f32", 1, 8, 9, 2, True), ("f16", 2, 24, 130, 4, False),
                                            ("bf16", 1, 4096, 2048, 4, True), ("bf16", 2, 24, 1024, 4, False),
                                            ("f32", 2, 5, 36, 3, False), ("bf16", 2, 12, 37, 3, True),
                                            ("f16", 2, 16, 19, 2, True), ("f32", 1, 4, 3, 4, True),
                                            ("bf16", 3, 7, 8, 4, False), ("bf16", 1, 3, 8256, 4, False),
                                            ("f32", 2, 2, 1028, 2, False)])
def test_causal_conv1d_vs_oracle(io, B, D, L, W, cl):
    """Both layouts, packed sequences (seq_idx), initial and final states, against the oracle (kernel rounding)."""
    from vortex_b200 import hyena_ops
    g = torch.Generator().manual_seed(900 + L)
    x = torch.randn(B, D, L, generator=g).to(DT[io])
    w = (torch.randn(D, W, generator=g) / W ** 0.5).to(DT[io])
    b = torch.randn(D, generator=g).to(DT[io])
    ini = torch.randn(B, D, W - 1, generator=g).to(DT[io])
    cuts = torch.sort(torch.randint(1, max(L, 2), (B, 3), generator=g), dim=1).values
    sid = (torch.arange(L)[None, :, None] >= cuts[:, None, :]).sum(-1).to(torch.int32)

    def lay(t):
        t = t.cuda()
        return t.transpose(1, 2).contiguous().transpose(1, 2) if cl else t
    xd = lay(x)
    fs = torch.empty_like(lay(ini))
    y = hyena_ops.causal_conv1d_fn(xd, w.cuda(), b.cuda(), None, lay(ini), fs, "silu")
    ref, rfs = O.causal_conv1d(to_np(x), to_np(w), bias=to_np(b), initial_states=to_np(ini), silu=True, io=io)
    assert y.stride() == xd.stride() and rel_l2(y, ref) <= CC_TOL[io]
    assert np.array_equal(to_np(fs), rfs.astype(np.float32))
    y = hyena_ops.causal_conv1d_fn(xd, w.cuda(), None, sid.cuda(), None, None, None)
    ref, _ = O.causal_conv1d(to_np(x), to_np(w), seq_idx=sid.numpy(), io=io)
    check("test_engine_gpu.py:422 y, ref", rel_l2(y, ref), CC_TOL[io])
    with pytest.raises(NotImplementedError):
        hyena_ops.causal_conv1d_fn(xd, w.cuda(), activation="gelu")
    with pytest.raises(NotImplementedError):
        hyena_ops.causal_conv1d_fn(xd, torch.randn(D, 5).to(DT[io]).cuda())


@pytest.mark.parametrize("io,B,D,Lq,W,SL", [("bf16", 4, 64, 1, 4, 3), ("bf16", 2, 40, 3, 3, 6), ("f32", 3, 8, 1, 2, 1),
                                             ("f16", 2, 16, 5, 4, 4), ("bf16", 8, 4096, 1, 4, 3)])
def test_causal_conv1d_update_vs_oracle(io, B, D, Lq, W, SL):
    """Shift-register state, circular state (cache_seqlens) and indirect rows (conv_state_indices)."""
    from vortex_b200 import hyena_ops
    g = torch.Generator().manual_seed(950 + D)
    x = torch.randn(B, D, Lq, generator=g).to(DT[io])
    st = torch.randn(B, D, SL, generator=g).to(DT[io])
    w = (torch.randn(D, W, generator=g) / W ** 0.5).to(DT[io])
    b = torch.randn(D, generator=g).to(DT[io])
    ref, rst = O.causal_conv1d_update(to_np(x), to_np(st), to_np(w), bias=to_np(b), silu=True, io=io)
    s = st.cuda()
    y = hyena_ops.causal_conv1d_update(x.cuda() if Lq > 1 else x[..., 0].cuda(), s, w.cuda(), b.cuda(), "silu")
    assert y.shape == (x.shape if Lq > 1 else x.shape[:2])
    check("test_engine_gpu.py:443 y.reshape(B, D, Lq), ref", rel_l2(y.reshape(B, D, Lq), ref), CC_TOL[io])
    assert np.array_equal(to_np(s), rst.astype(np.float32))
    if Lq <= SL:
        cs = torch.tensor([7 + 5 * i for i in range(B)], dtype=torch.int32)
        ref, rst = O.causal_conv1d_update(to_np(x), to_np(st), to_np(w), cache_seqlens=cs.numpy(), io=io)
        # indirect rows: the states live in a pool of 2B rows, batch element i uses row 2B-1-2i
        pool = torch.zeros(2 * B, D, SL, dtype=DT[io]).cuda()
        rows = torch.tensor([2 * B - 1 - 2 * i for i in range(B)], dtype=torch.int32)
        pool[rows.long().cuda()] = st.cuda()
        y = hyena_ops.causal_conv1d_update(x.cuda(), pool, w.cuda(), None, None, cs.cuda(), rows.cuda())
        check("test_engine_gpu.py:453 y, ref", rel_l2(y, ref), CC_TOL[io])
        assert np.array_equal(to_np(pool[rows.long().cuda()]), rst.astype(np.float32))
        assert float(pool[(rows.long() - 1).cuda()].abs().sum()) == 0.0


@pytest.mark.parametrize("n", [0, 1, 2])
def test_golden_varlen_states(golden, n):
    from vortex_b200 import hyena_ops
    k = f"vls_{n}"
    want = golden[k + "_st"]
    st = hyena_ops.causal_conv1d_varlen_states(T(golden[k + "_x"], "f32"), torch.from_numpy(golden[k + "_cu"]).cuda(),
                                               want.shape[-1])
    assert st.shape == want.shape and st.stride(1) == 1 and np.array_equal(to_np(st), want)


@pytest.mark.parametrize("io,lens,dim,sl", [("bf16", (8192, 1, 0, 300, 2), 4096, 3), ("f16", (3, 3, 3), 40, 127),
                                             ("f32", (1,), 5, 1)])
def test_varlen_states_vs_oracle(io, lens, dim, sl):
    """Evo 2 width (bf16, 4096 channels), sequences shorter than the state, an empty sequence; bit-exact."""
    from vortex_b200 import hyena_ops
    g = torch.Generator().manual_seed(40 + dim)
    cu = torch.tensor((0,) + tuple(np.cumsum(lens)), dtype=torch.int32)
    x = torch.randn(int(cu[-1]), dim, generator=g).to(DT[io])
    st = hyena_ops.causal_conv1d_varlen_states(x.cuda(), cu.cuda(), sl)
    assert np.array_equal(to_np(st), O.causal_conv1d_varlen_states(to_np(x), cu.numpy(), sl))
    with pytest.raises(TypeError):
        hyena_ops.causal_conv1d_varlen_states(x.cuda(), cu.long().cuda(), sl)


@pytest.mark.parametrize("io,B,G,dg,L,K", [("bf16", 2, 4, 16, 300, 7), ("f32", 1, 3, 4, 65, 4), ("f16", 2, 2, 8, 128, 32)])
def test_inner_hyena_se_layouts(io, B, G, dg, L, K):
    """The reference interface's wrappers over the gate-conv-gate kernel: every input / output layout gives the same
    numbers as the oracle's y = q * conv(h, k * x) with blocked filter groups."""
    from vortex_b200 import hyena_ops
    g = torch.Generator().manual_seed(31 + K)
    D = G * dg
    x, k, q = ((torch.rand(B, D, L, generator=g) - 0.5).to(DT[io]) for _ in range(3))
    h = (torch.randn(G, 1, K, generator=g) / K ** 0.5).to(DT[io])
    # inner_hyena_se_ref in the I/O dtype: k*x, the convolution and the gate each round to it
    kx = O.round_io(to_np(k).astype(np.float64) * to_np(x), io)
    conv = O.round_io(O.causal_fir(kx, O.expand_groups(to_np(h), D), "xcorr"), io)
    ref = O.round_io(to_np(q) * conv, io)
    xc, kc, qc = x.cuda(), k.cuda(), q.cuda()
    y = hyena_ops.inner_hyena_se(xc, kc, qc, h.cuda())
    assert y.shape == (B, D, L) and rel_l2(y, ref) <= TOL[io]
    blgdg = lambda t: t.transpose(1, 2).reshape(B, L, G, dg).contiguous()  # noqa: E731
    bgdgl = lambda t: t.reshape(B, G, dg, L)  # noqa: E731
    y2 = hyena_ops.inner_hyena_se(blgdg(xc), blgdg(kc), blgdg(qc), h.cuda(), input_layout="blgdg", output_layout="blgdg")
    assert y2.shape == (B, L, G, dg) and torch.equal(y2, blgdg(y))
    y3 = hyena_ops.inner_hyena_se(bgdgl(xc), bgdgl(kc), bgdgl(qc), h.cuda()[:, 0], input_layout="bgdgl", output_layout="bld")
    assert torch.equal(y3, y.transpose(1, 2))
    y4 = hyena_ops.two_pass_chunked_gate_conv_gate(blgdg(xc), blgdg(kc), blgdg(qc), h.cuda(), schedule="default", autotune=True)
    # (bf16: this call runs the channel-last tensor-core kernel, the one above the channel-first one: other summation
    # order, so last-place flips of the rounded filter output)
    assert torch.equal(y4, y2) if io != "bf16" else rel_l2(y4, y2) <= 2e-4
    assert rel_l2(y4.reshape(B, L, D).transpose(1, 2), ref) <= TOL[io]
    with pytest.raises(NotImplementedError):
        hyena_ops.inner_hyena_se(xc, kc, qc, h.cuda(), output_layout="lbd")


# ------------------------------------------------------------------ drop-in parallel_fir on the tensor-core kernel
# B, L, D, G, K, layout, heads, flip, bias
TC_CASES = [
    (4, 1000, 256, 16, 128, "split", 1, False, True),        # one box per operand covers the four batch elements
    (3, 2048, 64, 4, 128, "split", 1, False, True),          # batch quad with an idle stream
    (5, 520, 128, 8, 7, "split", 1, True, False),            # two batch quads, the second mostly idle; q/k swapped
    (1, 8192, 64, 4, 128, "split", 1, False, True),          # one sequence: streams are time segments
    (2, 1504, 128, 8, 64, "column_split", 4, False, True),   # per-head column split (head size 32)
    (2, 8, 32, 2, 7, "split", 1, False, False),              # shortest length the path takes
    (1, 136, 32, 1, 128, "split", 1, False, True),           # L barely longer than the filter; 32 channels per filter
    (2, 96, 32, 2, 128, "split", 1, False, True),            # L < K
]


@pytest.mark.parametrize("B,L,D,G,K,layout,heads,flip,with_bias", TC_CASES)
def test_parallel_fir_tensor_core_path(B, L, D, G, K, layout, heads, flip, with_bias):
    """engine.parallel_fir(gate=True) with bf16 operands and filters shared by blocks of 16 channels runs on tcgen05
    (the caller's per-channel expansion of the filters is undone from its ``groups`` argument).  It rounds where the
    reference rounds, so it has to agree with the oracle's mirrored evaluation like the general kernel does -- and
    with that kernel itself (taken here by handing the taps over in fp32) up to last-place flips."""
    from vortex_b200 import HyenaInferenceEngine, ops
    p = make_block(81, B, L, D, G, K, "bf16")
    g = torch.Generator().manual_seed(3)
    z_pre = torch.randn(B, 3 * D, L, generator=g).bfloat16()
    Dp = (0.5 * torch.randn(D, generator=g)).bfloat16() if with_bias else None
    eng = HyenaInferenceEngine(hyena_flip_x1x2=flip)
    dims = (D, heads, D // heads, 16, G)
    hx = p["h"].repeat_interleave(D // G, 0).cuda()
    kw = dict(dims=dims, gate=True, gated_bias=K >= 128 or with_bias, dim_last=False,
              column_split_hyena=layout == "column_split", fir_length=K, inference_params=True)
    y, st = eng.parallel_fir(F.conv1d, z_pre.cuda(), hx, None if Dp is None else Dp.cuda(), L, groups=G, **kw)
    ops.device_status()
    ref, st_ref = O.gate_conv_gate(to_np(z_pre), to_np(p["h"]), None if Dp is None else to_np(Dp), D, K, io="bf16",
                                   layout=layout, num_heads=heads, flip_x1x2=flip, gated_bias=K >= 128 or with_bias)
    assert y.shape == (B, D, L) and y.dtype == torch.bfloat16
    check(f"tensor-core parallel_fir vs mirrored oracle (B={B} L={L} K={K} {layout})", rel_l2(y, ref), TOL["bf16"])
    assert st.shape == st_ref.shape and np.array_equal(to_np(st), st_ref.astype(np.float32))
    # the general kernel on the same data (fp32 taps keep it off the tensor-core path)
    y2, st2 = eng.parallel_fir(F.conv1d, z_pre.cuda(), hx.float(), None if Dp is None else Dp.cuda(), L, groups=G, **kw)
    check(f"tensor-core vs general kernel (B={B} L={L} K={K})", rel_l2(y, y2), 2e-4)
    assert torch.equal(st, st2)
    # without the groups hint the expanded filters are taken as they come (one filter per channel: general kernel)
    y3, _ = eng.parallel_fir(F.conv1d, z_pre.cuda(), hx, None if Dp is None else Dp.cuda(), L, **kw)
    assert torch.equal(y3, y2)
    # rows that differ inside a block: the hint is not trusted
    hbad = hx.clone()
    hbad[1] += 1
    y4, _ = eng.parallel_fir(F.conv1d, z_pre.cuda(), hbad, None if Dp is None else Dp.cuda(), L, groups=G, **kw)
    y5, _ = eng.parallel_fir(F.conv1d, z_pre.cuda(), hbad.float(), None if Dp is None else Dp.cuda(), L, **kw)
    assert torch.equal(y4, y5)


def test_parallel_fir_tensor_core_full_size():
    """Configuration 2 through the drop-in call (B=4, L=8192, D=4096, 128 taps): oracle on a slice of channels, and
    exact integer data over the whole tensor (pins Toeplitz expansion, segment seams, box geometry, channel maps)."""
    from vortex_b200 import HyenaInferenceEngine, ops
    B, L, D, G, K = 4, 8192, 4096, 256, 128
    g = torch.Generator().manual_seed(12)
    eng = HyenaInferenceEngine()
    dims = (D, 1, D, 16, G)
    kw = dict(dims=dims, gate=True, gated_bias=True, dim_last=False, fir_length=K, inference_params=True, groups=G)
    z = torch.randint(-2, 3, (B, 3 * D, L), generator=g).bfloat16()
    h = torch.zeros(G, 1, K)
    for pos in (0, 1, 77, K - 1):
        h[:, 0, pos] = torch.randint(0, 2, (G,), generator=g).float() * 2 - 1
    Dp = torch.randint(-1, 2, (D,), generator=g).bfloat16()
    hx = h.bfloat16().repeat_interleave(D // G, 0).cuda()
    y, st = eng.parallel_fir(F.conv1d, z.cuda(), hx, Dp.cuda(), L, **kw)
    ops.device_status()
    for d0 in (0, 2000, 4080):
        sl = slice(d0, d0 + 16)
        zz = torch.cat([z[:, d0:d0 + 16], z[:, D + d0:D + d0 + 16], z[:, 2 * D + d0:2 * D + d0 + 16]], 1)
        ref, st_ref = O.gate_conv_gate(to_np(zz), to_np(h[d0 // 16:d0 // 16 + 1]), to_np(Dp[sl]), 16, K, io="bf16",
                                       gated_bias=True)
        assert np.array_equal(to_np(y[:, sl]), ref.astype(np.float32)), d0
        assert np.array_equal(to_np(st[:, sl]), st_ref.astype(np.float32))
    p = make_block(1, B, 8, D, G, K, "bf16")          # only the filters of the benchmark configuration are taken
    zr = torch.randn(B, 3 * D, L, generator=g).bfloat16()
    hx = p["h"].repeat_interleave(D // G, 0).cuda()
    y, _ = eng.parallel_fir(F.conv1d, zr.cuda(), hx, Dp.cuda(), L, **kw)
    d0 = 1024
    zz = torch.cat([zr[::3, d0:d0 + 32], zr[::3, D + d0:D + d0 + 32], zr[::3, 2 * D + d0:2 * D + d0 + 32]], 1)
    ref, _ = O.gate_conv_gate(to_np(zz), to_np(p["h"][d0 // 16:d0 // 16 + 2]), to_np(Dp[d0:d0 + 32]), 32, K, io="bf16",
                              gated_bias=True)
    check("tensor-core parallel_fir, configuration 2, vs mirrored oracle", rel_l2(y[::3, d0:d0 + 32], ref), TOL["bf16"])


@pytest.mark.parametrize("io,B,L,C,K,with_bias,with_mask", [
    ("bf16", 2, 264, 200, 3, True, True),      # channels not a multiple of the tile, ragged last time tile
    ("bf16", 1, 8, 48, 3, False, False),       # one short tile
    ("f16", 3, 1024, 192, 4, True, False),
    ("bf16", 2, 4096, 96, 3, False, False),
])
def test_featurizer_tma_kernel(eng, io, B, L, C, K, with_bias, with_mask):
    """The featurizer's 16-bit path (TMA box in, swizzled [channel][time] tile, TMA boxes out) against the mirrored
    oracle, and against the general kernel on the same data (reached through a view whose rows are not 16-byte
    aligned): same arithmetic, identical bits."""
    g = torch.Generator().manual_seed(77)
    u = torch.randn(B, L, C, generator=g).to(DT[io])
    w = (torch.randn(C, 1, K, generator=g) / K ** 0.5).to(DT[io])
    bias = torch.randn(C, generator=g).to(DT[io]) if with_bias else None
    mask = (torch.rand(B, L, generator=g) > 0.2).to(DT[io]) if with_mask else None
    cu = lambda t: None if t is None else t.cuda()  # noqa: E731
    dims = (C // 3, 1, C // 3, 16, C // 3)
    z, st = eng.parallel_fir(F.conv1d, cu(u), cu(w), cu(bias), L, dims=dims, gate=False, fir_length=K,
                             inference_params=True, padding_mask=cu(mask))
    ref, st_ref = O.featurizer(to_np(u), to_np(w), None if bias is None else to_np(bias), io=io,
                               padding_mask=None if mask is None else to_np(mask))
    assert z.shape == (B, C, L) and z.dtype == DT[io]
    check(f"featurizer TMA kernel vs mirrored oracle ({io} L={L} C={C})", rel_l2(z, ref), 1e-4)
    assert np.array_equal(to_np(st), st_ref.astype(np.float32))
    wide = torch.zeros(B, L, C + 1, dtype=DT[io]).cuda()
    wide[..., 1:] = cu(u)
    z2, st2 = eng.parallel_fir(F.conv1d, wide[..., 1:], cu(w), cu(bias), L, dims=dims, gate=False, fir_length=K,
                               inference_params=True, padding_mask=cu(mask))
    assert torch.equal(z, z2) and torch.equal(st, st2)


@pytest.mark.parametrize("bs,l,g,dg,hl,gated", [(2, 1024, 1, 256, 128, False), (2, 8192, 4, 16, 32, False),
                                                 (3, 1000, 2, 32, 4, True), (1, 77, 8, 16, 128, True)])
def test_hyena_ops_channel_last_tensor_core(bs, l, g, dg, hl, gated):
    """hyena_ops.gcg_fwd / two_pass_chunked_gate_conv_gate on bf16 (bs, l, g, dg) operands: the tensor-core kernel in its
    operator-only form reads the layout as it is (no permuted copies) and rounds where the reference does."""
    from vortex_b200 import hyena_ops, ops
    gen = torch.Generator().manual_seed(21)
    x, Bm, Cm = (torch.randn(bs, l, g, dg, generator=gen).bfloat16() for _ in range(3))
    h = (torch.randn(g, 1, hl, generator=gen) / hl ** 0.5).bfloat16()
    bias = (0.5 * torch.randn(g * dg, generator=gen)).bfloat16() if gated else None
    y = hyena_ops.gcg_fwd(x.cuda(), Bm.cuda(), Cm.cuda(), h.cuda(), None if bias is None else bias.cuda(), gated_bias=gated)
    ops.device_status()
    assert y.shape == (bs, l, g, dg) and y.dtype == torch.bfloat16
    # mirrored oracle on the (b, d, l) view: q = C, k = B, v = x
    z = torch.cat([t.reshape(bs, l, g * dg).permute(0, 2, 1) for t in (Cm, Bm, x)], 1)
    # (cross-correlation taps whatever the length: the hyena_ops convention, ref_fwd.py:80-127)
    zz = O.round_io(to_np(z), "bf16")
    q, k, v = O.select_qkv(zz, g * dg)
    kv = O.round_io(k * v, "bf16")
    conv = O.round_io(O.causal_fir(kv, O.expand_groups(to_np(h), g * dg), "xcorr"), "bf16")
    if gated:
        conv = O.round_io(conv + O.round_io(kv * to_np(bias).astype(np.float64)[None, :, None], "bf16"), "bf16")
    ref = O.round_io(q * conv, "bf16")
    check(f"channel-last tensor-core gcg vs mirrored oracle (l={l} dg={dg} hl={hl})",
          rel_l2(y.reshape(bs, l, g * dg).permute(0, 2, 1), ref), TOL["bf16"])
    # and the (b, d, l) route on the same data
    y2 = hyena_ops.hyena_se_bdl(x.cuda().reshape(bs, l, -1).permute(0, 2, 1).contiguous(),
                                Bm.cuda().reshape(bs, l, -1).permute(0, 2, 1).contiguous(),
                                Cm.cuda().reshape(bs, l, -1).permute(0, 2, 1).contiguous(), h.cuda(),
                                None if bias is None else bias.cuda(), gated)
    check("channel-last vs channel-first route", rel_l2(y.reshape(bs, l, -1).permute(0, 2, 1), y2), 2e-4)
    with_state, st = ops.gcg_cl_fwd(Cm.cuda().view(bs, l, -1), Bm.cuda().view(bs, l, -1), x.cuda().view(bs, l, -1), h.cuda(),
                                    None if bias is None else bias.cuda(),
                                    bias_mode=2 if gated else 0, want_state=True)
    assert torch.equal(with_state.view(bs, l, g, dg), y)
    kv = (Bm.float() * x.float()).bfloat16().reshape(bs, l, -1).permute(0, 2, 1)
    assert torch.equal(st.cpu(), kv[..., max(l - (hl - 1), 0):].contiguous())
