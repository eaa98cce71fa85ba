"""Pins the CPU oracle (numpy restatement and torch port) against vectors
produced by the reference's own HyenaInferenceEngine / hyena_ops references."""
import numpy as np
import pytest
import torch

from oracle import hyena_oracle as O
from oracle import torch_port as TP

TOL = {"f32": 2e-6, "bf16": 2e-3}   # bf16: single-ulp flips where fp32 sums differ in the last bit
DT = {"f32": torch.float32, "bf16": torch.bfloat16}


def close(a, b, io, scale=1.0):
    assert a.shape == b.shape, (a.shape, b.shape)
    err = O.rel_l2(a, b)
    assert err <= TOL[io] * scale, err


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("L", [1, 2, 50])
@pytest.mark.parametrize("tag", ["nobias", "bias"])
def test_featurizer(golden, io, L, tag):
    k = f"feat_{io}_L{L}_{tag}"
    u, w, b = golden[k + "_u"], golden[k + "_w"], golden[k + "_b"]
    z, st = O.featurizer(u, w, b if tag == "bias" else None, io=io)
    close(z, golden[k + "_z"], io)
    assert np.array_equal(st.astype(np.float32), golden[k + "_state"])
    zt, stt = TP.featurizer(torch.from_numpy(u).to(DT[io]), torch.from_numpy(w).to(DT[io]),
                            torch.from_numpy(b).to(DT[io]) if tag == "bias" else None)
    assert np.array_equal(zt.float().numpy(), golden[k + "_z"])
    assert np.array_equal(stt.float().numpy(), golden[k + "_state"])


GCG = [(7, 50, "split"), (7, 4, "split"), (4, 33, "interleaved"), (128, 300, "split"),
       (128, 100, "interleaved"), (7, 40, "column_split"), (128, 200, "column_split")]


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("K,L,layout", GCG)
def test_gate_conv_gate(golden, io, K, L, layout):
    k = f"gcg_{io}_K{K}_L{L}_{layout}"
    z, h, Dp = golden[k + "_z"], golden[k + "_h"], golden[k + "_D"]
    flip = layout == "column_split"
    y, st = O.gate_conv_gate(z, h, Dp if K >= 128 else None, 32, K, io=io, layout=layout, num_heads=4,
                             flip_x1x2=flip, gated_bias=K >= 128)
    close(y, golden[k + "_y"], io, scale=5.0 if K >= 128 else 1.0)  # reference MR goes through an fp32 FFT
    assert np.array_equal(st.astype(np.float32), golden[k + "_state"])
    yt, stt = TP.gate_conv_gate(torch.from_numpy(z).to(DT[io]), torch.from_numpy(h).to(DT[io]),
                                torch.from_numpy(Dp).to(DT[io]) if K >= 128 else None, 32, K, layout=layout,
                                num_heads=4, flip=flip, gated_bias=K >= 128)
    close(yt.float().numpy(), golden[k + "_y"], io, scale=0.5)
    assert np.array_equal(stt.float().numpy(), golden[k + "_state"])
    # the "fp32 reference" (no intermediate rounding) stays within the bf16 budget of the mirrored path
    y32, _ = O.gate_conv_gate(z, h, Dp if K >= 128 else None, 32, K, io=io, layout=layout, num_heads=4,
                              flip_x1x2=flip, gated_bias=K >= 128, mirror=False)
    assert O.rel_l2(y32, golden[k + "_y"]) <= (4e-3 if io == "bf16" else 1e-5)


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("L,layout", [(200, "split"), (64, "interleaved")])
def test_long_conv(golden, io, L, layout):
    k = f"iir_{io}_L{L}_{layout}"
    z, lp, R, Dp = golden[k + "_z"], golden[k + "_lp"], golden[k + "_R"], golden[k + "_D"]
    h = O.modal_filter(lp, R, L)
    assert O.rel_l2(h, golden[k + "_h"][0]) < 1e-6
    y, kv = O.long_conv_gate(z, h, Dp, 16, io=io, layout=layout)
    close(y, golden[k + "_y"], io, scale=5.0)
    st = O.modal_state(kv, lp)
    assert O.rel_l2(st, golden[k + "_state"]) < 2e-5   # reference state comes out of a complex64 FFT pair
    yt, stt = TP.long_conv_gate(torch.from_numpy(z).to(DT[io]), torch.from_numpy(golden[k + "_h"][0]),
                                torch.from_numpy(Dp).to(DT[io]), 16, layout=layout,
                                log_poles_d=torch.from_numpy(lp))
    close(yt.float().numpy(), golden[k + "_y"], io, scale=0.5)
    assert O.rel_l2(stt.numpy(), golden[k + "_state"]) < 1e-6


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("K,c0,flip,gb", [(3, 2, False, False), (3, 1, False, False), (7, 6, False, False),
                                          (7, 3, False, False), (128, 127, True, True), (128, 20, True, True)])
def test_step_fir(golden, io, K, c0, flip, gb):
    k = f"stepfir_{io}_K{K}_c{c0}"
    w = golden[k + "_w"]
    b = golden[k + "_b"] if gb else None
    st = golden[k + "_state0"]
    stt = torch.from_numpy(st).to(DT[io])
    for i in range(3):
        u = golden[f"{k}_u{i}"]
        y, st = O.step_fir(u, st, w, bias=b, gated_bias=gb, flip_filter=flip, io=io)
        close(y, golden[f"{k}_y{i}"], io)
        assert st.shape == golden[f"{k}_state{i + 1}"].shape
        assert np.array_equal(st, golden[f"{k}_state{i + 1}"])
        yt, stt = TP.step_fir(torch.from_numpy(u).to(DT[io]), stt, torch.from_numpy(w).to(DT[io]),
                              bias=None if b is None else torch.from_numpy(b).to(DT[io]), gated_bias=gb,
                              flip_filter=flip)
        assert np.array_equal(stt.numpy(), golden[f"{k}_state{i + 1}"])
        close(yt.float().numpy(), golden[f"{k}_y{i}"], io)


@pytest.mark.parametrize("io", ["f32", "bf16"])
def test_step_iir(golden, io):
    k = f"stepiir_{io}"
    lp, R, Dp, st = golden[k + "_lp"], golden[k + "_R"], golden[k + "_D"], golden[k + "_state0"]
    for i in range(3):
        y, st = O.step_iir(golden[f"{k}_x2{i}"], golden[f"{k}_x1{i}"], golden[f"{k}_v{i}"], Dp, R, lp, st)
        # the reference multiplies x1*v in the I/O dtype first; allow that one rounding
        assert O.rel_l2(y, golden[f"{k}_y{i}"]) <= (3e-3 if io == "bf16" else 2e-6)
        assert O.rel_l2(st, golden[f"{k}_state{i + 1}"]) <= (3e-3 if io == "bf16" else 2e-6)


@pytest.mark.parametrize("K", [7, 128])
def test_prefill_decode_continuity(golden, K):
    """The state left by prefill, fed to one decode step, reproduces position L of a
    prefill over L+1 tokens -- in the reference's vectors and in the oracle."""
    k = f"cont_K{K}"
    z, h, Dp = golden[k + "_z"], golden[k + "_h"], golden[k + "_D"]
    assert O.rel_l2(golden[k + "_ystep"], golden[k + "_yfull_last"]) < 1e-5
    D, L = 32, z.shape[-1] - 1
    _, st = O.gate_conv_gate(z[..., :L], h, Dp if K >= 128 else None, D, K, gated_bias=K >= 128)
    assert np.array_equal(st.astype(np.float32), golden[k + "_state"])
    q, kk, v = O.select_qkv(z[..., L].astype(np.float64), D)
    y, st2 = O.step_fir(kk * v, st, O.expand_groups(h, D), bias=Dp if K >= 128 else None,
                        gated_bias=K >= 128, flip_filter=K >= 128)
    assert O.rel_l2(y * q, golden[k + "_yfull_last"]) < 1e-5
    assert np.array_equal(st2, golden[k + "_state2"])


@pytest.mark.parametrize("hl", [4, 32, 128])
def test_hyena_ops_layout(golden, hl):
    k = f"ops_hl{hl}"
    y = O.gcg_blgdg(golden[k + "_x"], golden[k + "_B"], golden[k + "_C"], golden[k + "_h"])
    assert O.rel_l2(y, golden[k + "_y"]) < 2e-6
    assert O.rel_l2(y, golden[k + "_y_chunked"]) < 2e-6
    h = golden[k + "_h"]
    for g in range(h.shape[0]):
        T, Th = O.toeplitz_pair(h[g, 0, ::-1], 128)
        assert np.array_equal(T.astype(np.float32), golden[k + "_T"][g])
        assert np.array_equal(Th.astype(np.float32), golden[k + "_That"][g])


@pytest.mark.parametrize("hl", [4, 32, 128])
def test_hyena_ops_backward(golden, hl):
    """The oracle's backward against the reference's own (ref_bwd.py: gcg_two_pass_chunked_bwd, fp32 on CPU)."""
    k = f"opsbwd_hl{hl}"
    y2 = O.gcg_blgdg(golden[k + "_x"], golden[k + "_B"], np.ones_like(golden[k + "_C"]), golden[k + "_h"])
    assert O.rel_l2(y2, golden[k + "_y2"]) < 2e-6
    grads = O.gcg_blgdg_bwd(golden[k + "_dy"], golden[k + "_x"], golden[k + "_B"], golden[k + "_C"], golden[k + "_h"])
    for name, got in zip(("dx", "dB", "dC", "dh"), grads):
        assert got.shape == golden[f"{k}_{name}"].shape
        assert O.rel_l2(got, golden[f"{k}_{name}"]) < 2e-6, name


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("Lh", [4, 16])
def test_hyena_x(golden, io, Lh):
    k = f"hx_{io}_Lh{Lh}"
    y = O.hyena_x(golden[k + "_qkv"], golden[k + "_h"], io=io)
    close(y, golden[k + "_y"], io, scale=2.0)


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("L", [1, 2, 37])
def test_causal_conv1d(golden, io, W, L):
    """The reference's causal_conv1d_ref: plain, and with bias + initial states + SiLU; final states bit-exact."""
    k = f"cc1d_{io}_W{W}_L{L}"
    x, w, b, ini = (golden[k + s] for s in ("_x", "_w", "_b", "_ini"))
    y, fs = O.causal_conv1d(x, w, io=io)
    close(y, golden[k + "_y_plain"], io)
    assert np.array_equal(fs.astype(np.float32), golden[k + "_fs_plain"])
    ym, fs = O.causal_conv1d(x, w, bias=b, initial_states=ini, silu=True, io=io, mirror=True)
    close(ym, golden[k + "_y_full"], io)
    assert np.array_equal(fs.astype(np.float32), golden[k + "_fs_full"])
    y, _ = O.causal_conv1d(x, w, bias=b, initial_states=ini, silu=True, io=io)      # the kernel's rounding
    # update form == the convolution's last samples, shift-register and circular state
    st0 = np.concatenate([np.zeros_like(ini[..., :1]), ini], axis=-1)          # state_len = W: one spare slot
    yu, st1 = O.causal_conv1d_update(x, st0, w, bias=b, silu=True, io=io)
    assert np.array_equal(yu, y)
    assert np.array_equal(st1[..., -(W - 1):], fs)
    B = x.shape[0]
    cs = np.array([5 + 3 * i for i in range(B)])
    SL = W + 2
    circ = np.zeros(ini.shape[:2] + (SL,))
    for i in range(B):
        for j in range(W - 1):
            circ[i, :, (cs[i] - (W - 1) + j) % SL] = ini[i, :, j]
    if L <= SL:
        yc, circ1 = O.causal_conv1d_update(x, circ, w, bias=b, silu=True, cache_seqlens=cs, io=io)
        assert np.array_equal(yc, y)
        for i in range(B):
            for t in range(L):
                assert np.array_equal(circ1[i, :, (cs[i] + t) % SL], O.round_io(x, io)[i, :, t])


@pytest.mark.parametrize("n", [0, 1, 2])
def test_varlen_states(golden, n):
    """causal_conv1d_varlen_states_ref: the last rows of each packed sequence, bit-exact."""
    k = f"vls_{n}"
    want = golden[k + "_st"]
    st = O.causal_conv1d_varlen_states(golden[k + "_x"], golden[k + "_cu"], want.shape[-1])
    assert st.shape == want.shape and np.array_equal(st, want)


@pytest.mark.parametrize("io", ["f32", "bf16"])
def test_recurrence_prefill(golden, io):
    """prefill_style="recurrence" (engine.py:473-504): the oracle repeats the reference's loop, its update order and
    its rounding of the state to the I/O dtype, so the cached state is reproduced bit for bit."""
    k = f"iirrec_{io}"
    y, st = O.recurrence_prefill(golden[k + "_z"], golden[k + "_p"][:, :, 0], golden[k + "_R"][:, :, 0],
                                 golden[k + "_D"], 12, io=io)
    close(y, golden[k + "_y"], io)
    assert st.dtype == np.float32 and np.array_equal(st, golden[k + "_state"])
    # the reference's update is not a complex product: the true recurrence sigma <- p sigma + x ends elsewhere
    z = O.round_io(golden[k + "_z"], io)
    _, kk, v = O.select_qkv(z, 12, "split")
    p = golden[k + "_p"][:, :, 0, 0] + 1j * golden[k + "_p"][:, :, 0, 1]
    true = O.modal_state_complex(O.round_io(kk * v, io), p)
    got = st[..., 0] + 1j * st[..., 1]
    assert np.linalg.norm(got - true) / np.linalg.norm(true) > 1e-2


@pytest.mark.parametrize("io", ["f32", "bf16"])
@pytest.mark.parametrize("thr", [24, 160])
def test_long_fir_threshold(golden, io, thr):
    """long_fir_threshold (engine.py:339-349): the truncated filter goes through F.conv1d, i.e. as a
    cross-correlation, whatever its length."""
    k = f"iirfir_{io}_thr{thr}"
    y = O.long_fir_gate(golden[k + "_z"], golden[k + "_h"], golden[k + "_D"], 16, thr, io=io)
    close(y, golden[k + "_y"], io)


def test_hyena_ops_backward_matches_autograd():
    """The oracle's backward against torch autograd through a plain float64 forward (F.conv1d on the gated product),
    on a shape the golden vectors do not hold: ragged length, three groups of four channels, seven taps."""
    import torch
    import torch.nn.functional as F

    g = torch.Generator().manual_seed(0)
    bs, l, G, dg, hl = 2, 53, 3, 4, 7
    x, B, C = (torch.randn(bs, l, G, dg, generator=g, dtype=torch.float64, requires_grad=True) for _ in range(3))
    h = torch.randn(G, 1, hl, generator=g, dtype=torch.float64, requires_grad=True)
    y2 = F.conv1d((B * x).reshape(bs, l, G * dg).permute(0, 2, 1), h.repeat_interleave(dg, 0), groups=G * dg,
                  padding=hl - 1)[..., :l]
    y = C * y2.permute(0, 2, 1).reshape(bs, l, G, dg)
    dy = torch.randn(bs, l, G, dg, generator=g, dtype=torch.float64)
    y.backward(dy)
    got = O.gcg_blgdg_bwd(dy.numpy(), x.detach().numpy(), B.detach().numpy(), C.detach().numpy(), h.detach().numpy())
    for a, b in zip(got, (x.grad, B.grad, C.grad, h.grad)):
        assert np.abs(a - b.numpy()).max() < 1e-12
