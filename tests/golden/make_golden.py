"""Generate golden vectors by running the reference's own code on CPU.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

It imports ``vortex.model.engine.HyenaInferenceEngine``, ``vortex.model.utils``
and the pure-PyTorch ``hyena_se`` references (aliased as ``hyena_ops``) and
stores inputs and outputs of small seeded cases in ``tests/golden/*.npz``.
Narrow dtypes are stored as float32 (every bf16 value is exactly
representable).  The committed ``.npz`` files are what the tests read; the
reference checkout is not needed to run the tests.
"""
import os
import sys
import tempfile
import types

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def np32(t):
    return t.detach().to(torch.float32).contiguous().numpy()


def main(ref_root):
    os.chdir(tempfile.mkdtemp())  # the reference's logging module writes a log file into cwd
    sys.path.insert(0, ref_root)
    from vortex.model.engine import HyenaInferenceEngine
    from vortex.model.utils import column_split, interleave  # noqa: F401

    pkg = types.ModuleType("hyena_ops")
    pkg.__path__ = [os.path.join(ref_root, "vortex", "ops", "hyena_se")]
    sys.modules["hyena_ops"] = pkg
    from hyena_ops.ref_fwd import gcg_fwd_ref_corrected, gcg_two_pass_chunked_fwd_corrected
    from hyena_ops.utils import correction_toeplitz, toeplitz

    out = {}
    DT = {"f32": torch.float32, "bf16": torch.bfloat16}

    # ---- featurizer --------------------------------------------------------
    for io, dt in DT.items():
        for L in (1, 2, 50):
            g = torch.Generator().manual_seed(100 + L)
            B, D = 2, 16
            u = torch.randn(B, L, 3 * D, generator=g).to(dt)
            w = (torch.randn(3 * D, 1, 3, generator=g) / 3 ** 0.5).to(dt)
            bias = torch.randn(3 * D, generator=g).to(dt)
            eng = HyenaInferenceEngine()
            dims = (D, 1, D, 16, D)
            for tag, b in (("nobias", None), ("bias", bias)):
                z, st = eng.parallel_fir(F.conv1d, u, w, b, L, dims=dims, gate=False, dim_last=True,
                                         fir_length=3, inference_params=True)
                k = f"feat_{io}_L{L}_{tag}"
                out[k + "_u"], out[k + "_w"], out[k + "_b"] = np32(u), np32(w), np32(bias)
                out[k + "_z"], out[k + "_state"] = np32(z), np32(st)

    # ---- gate-conv-gate, SE (K=7, also 4) and MR (K=128) --------------------
    for io, dt in DT.items():
        for K, L, layout in ((7, 50, "split"), (7, 4, "split"), (4, 33, "interleaved"),
                             (128, 300, "split"), (128, 100, "interleaved"),
                             (7, 40, "column_split"), (128, 200, "column_split")):
            g = torch.Generator().manual_seed(1000 + K + L)
            B, D, G, H = 2, 32, 2, 4
            z_pre = torch.randn(B, 3 * D, L, generator=g).to(dt)
            h = (torch.randn(G, 1, K, generator=g) / K ** 0.5).to(dt)
            Dp = torch.randn(D, generator=g).to(dt)
            flip = layout == "column_split"
            eng = HyenaInferenceEngine(hyena_flip_x1x2=flip)
            dims = (D, H, D // H, 16, G)
            zin = interleave(z_pre) if layout == "interleaved" else z_pre
            hx = h.repeat_interleave(D // G, 0)
            y, st = eng.parallel_fir(F.conv1d, zin, hx, Dp if K >= 128 else None, L, dims=dims, gate=True,
                                     gated_bias=K >= 128, dim_last=False,
                                     column_split_hyena=layout == "column_split", fir_length=K,
                                     inference_params=True, groups=G)
            k = f"gcg_{io}_K{K}_L{L}_{layout}"
            out[k + "_z"], out[k + "_h"], out[k + "_D"] = np32(z_pre), np32(h), np32(Dp)
            out[k + "_y"], out[k + "_state"] = np32(y), np32(st)

    # ---- long convolution (parallel_iir) + modal-fft state -------------------
    class _P:  # stand-in for the inference-params object: only state_dict is touched
        def __init__(self):
            self.state_dict = {}

    for io, dt in DT.items():
        for L, layout in ((200, "split"), (64, "interleaved")):
            g = torch.Generator().manual_seed(2000 + L)
            B, D, S = 2, 16, 16
            z_pre = torch.randn(B, 3 * D, L, generator=g).to(dt)
            mag = 0.9 + 0.099 * torch.rand(D, S, 1, generator=g)
            log_poles = torch.log(mag)
            residues = torch.randn(D, S, generator=g)
            Dp = torch.randn(D, generator=g).to(dt)
            t = torch.arange(L)[None, None]
            h = (residues[..., None] * (log_poles * t).exp()).sum(1)[None]
            eng = HyenaInferenceEngine()
            ip = _P()
            dims = (D, 1, D, S, D)
            zin = interleave(z_pre) if layout == "interleaved" else z_pre
            y = eng.parallel_iir(zin, h, Dp, L, poles=log_poles, residues=residues, t=t, dims=dims,
                                 layer_idx=3, inference_params=ip, prefill_style="fft")
            k = f"iir_{io}_L{L}_{layout}"
            out[k + "_z"], out[k + "_lp"], out[k + "_R"], out[k + "_D"] = (np32(z_pre), np32(log_poles),
                                                                            np32(residues), np32(Dp))
            out[k + "_h"], out[k + "_y"], out[k + "_state"] = np32(h), np32(y), np32(ip.state_dict[3])

    # ---- long convolution, the two other branches of parallel_iir --------------
    # prefill_style="recurrence" (engine.py:314-321,473-504): complex poles / residues as (re, im) pairs
    for io, dt in DT.items():
        g = torch.Generator().manual_seed(2500)
        B, D, S, L = 2, 12, 16, 48
        z_pre = torch.randn(B, 3 * D, L, generator=g).to(dt)
        mag = 0.5 + 0.49 * torch.rand(D, S, generator=g)
        ang = torch.pi * torch.rand(D, S, generator=g)
        poles = torch.stack([mag * torch.cos(ang), mag * torch.sin(ang)], -1)[:, :, None]     # [D, S, 1, 2]
        residues = torch.randn(D, S, 1, 2, generator=g)
        Dp = torch.randn(D, generator=g).to(dt)
        eng = HyenaInferenceEngine(layer_idx=5)
        ip = _P()
        y = eng.parallel_iir(z_pre, None, Dp, L, poles=poles, residues=residues, t=None, dims=(D, 1, D, S, D),
                             layer_idx=5, inference_params=ip, prefill_style="recurrence")
        k = f"iirrec_{io}"
        out[k + "_z"], out[k + "_p"], out[k + "_R"], out[k + "_D"] = np32(z_pre), np32(poles), np32(residues), np32(Dp)
        out[k + "_y"], out[k + "_state"] = np32(y), np32(ip.state_dict[5])
    # long_fir_threshold (engine.py:339-349): the filter cut to its first samples and handed to F.conv1d; the
    # reference can only run it without inference_params (its state prefill reads a spectrum this branch never makes)
    for io, dt in DT.items():
        for thr in (24, 160):
            g = torch.Generator().manual_seed(2600 + thr)
            B, D, S, L = 1, 16, 16, 200
            z_pre = torch.randn(B, 3 * D, L, generator=g).to(dt)
            log_poles = torch.log(0.9 + 0.099 * torch.rand(D, S, 1, generator=g))
            residues = torch.randn(D, S, generator=g)
            Dp = torch.randn(D, generator=g).to(dt)
            t = torch.arange(L)[None, None]
            h = (residues[..., None] * (log_poles * t).exp()).sum(1)[None]
            eng = HyenaInferenceEngine()
            y = eng.parallel_iir(z_pre, h, Dp, L, poles=log_poles, residues=residues, t=t, dims=(D, 1, D, S, D),
                                 layer_idx=0, inference_params=None, long_fir_threshold=thr)
            k = f"iirfir_{io}_thr{thr}"
            out[k + "_z"], out[k + "_lp"], out[k + "_R"], out[k + "_D"] = (np32(z_pre), np32(log_poles),
                                                                            np32(residues), np32(Dp))
            out[k + "_h"], out[k + "_y"] = np32(h), np32(y)

    # ---- decode: step_fir ----------------------------------------------------
    for io, dt in DT.items():
        for K, c0, flip, gb in ((3, 2, False, False), (3, 1, False, False), (7, 6, False, False),
                                (7, 3, False, False), (128, 127, True, True), (128, 20, True, True)):
            g = torch.Generator().manual_seed(3000 + K + c0)
            B, C = 3, 24
            w = (torch.randn(C, 1, K, generator=g) / K ** 0.5).to(dt)
            bias = torch.randn(C, generator=g).to(dt) if gb else None
            state = torch.randn(B, C, c0, generator=g).to(dt)
            eng = HyenaInferenceEngine()
            k = f"stepfir_{io}_K{K}_c{c0}"
            out[k + "_w"], out[k + "_state0"] = np32(w), np32(state)
            if bias is not None:
                out[k + "_b"] = np32(bias)
            for i in range(3):
                u = torch.randn(B, C, generator=g).to(dt)
                y, state = eng.step_fir(u, state, w, bias=bias, gated_bias=gb, flip_filter=flip)
                assert state.dtype == torch.float32 and y.dtype == dt
                out[f"{k}_u{i}"], out[f"{k}_y{i}"], out[f"{k}_state{i + 1}"] = np32(u), np32(y), np32(state)

    # ---- decode: step_iir ----------------------------------------------------
    for io, dt in DT.items():
        g = torch.Generator().manual_seed(4000)
        B, D, S = 3, 24, 16
        log_poles = torch.log(0.9 + 0.099 * torch.rand(D, S, 1, generator=g))
        residues = torch.randn(D, S, generator=g)
        Dp = torch.randn(D, generator=g).to(dt)
        state = torch.randn(B, D, S, generator=g)
        eng = HyenaInferenceEngine()
        k = f"stepiir_{io}"
        out[k + "_lp"], out[k + "_R"], out[k + "_D"], out[k + "_state0"] = (np32(log_poles), np32(residues),
                                                                             np32(Dp), np32(state))
        for i in range(3):
            x2, x1, v = (torch.randn(B, D, generator=g).to(dt) for _ in range(3))
            y, state = eng.step_iir(x2, x1, v, Dp, residues, log_poles, state)
            out[f"{k}_x2{i}"], out[f"{k}_x1{i}"], out[f"{k}_v{i}"] = np32(x2), np32(x1), np32(v)
            out[f"{k}_y{i}"], out[f"{k}_state{i + 1}"] = np32(y), np32(state)

    # ---- prefill -> decode continuity (state handed from prefill to step) -----
    for K in (7, 128):
        g = torch.Generator().manual_seed(5000 + K)
        B, D, G, L = 2, 32, 2, 160
        z_pre = torch.randn(B, 3 * D, L + 1, generator=g)
        h = torch.randn(G, 1, K, generator=g) / K ** 0.5
        Dp = torch.randn(D, generator=g)
        hx = h.repeat_interleave(D // G, 0)
        eng = HyenaInferenceEngine()
        dims = (D, 1, D, 16, G)
        kw = dict(dims=dims, gate=True, gated_bias=K >= 128, dim_last=False, fir_length=K,
                  inference_params=True, groups=G)
        y_full, _ = eng.parallel_fir(F.conv1d, z_pre, hx, Dp if K >= 128 else None, L + 1, **kw)
        _, st = eng.parallel_fir(F.conv1d, z_pre[..., :L], hx, Dp if K >= 128 else None, L, **kw)
        q, kk, v = z_pre[..., L].split([D, D, D], dim=1)
        y_step, st2 = eng.step_fir(kk * v, st, hx, bias=Dp if K >= 128 else None, flip_filter=K >= 128,
                                   gated_bias=K >= 128)
        k = f"cont_K{K}"
        out[k + "_z"], out[k + "_h"], out[k + "_D"] = np32(z_pre), np32(h), np32(Dp)
        out[k + "_yfull_last"], out[k + "_ystep"] = np32(y_full[..., L]), np32(y_step * q)
        out[k + "_state"], out[k + "_state2"] = np32(st), np32(st2)

    # ---- hyena_ops (bs, l, g, dg) references ---------------------------------
    for hl in (4, 32, 128):
        g = torch.Generator().manual_seed(6000 + hl)
        bs, l, gg, dg = 2, 256, 2, 16
        x, Bm, Cm = (torch.randn(bs, l, gg, dg, generator=g) for _ in range(3))
        h = torch.randn(gg, 1, hl, generator=g)
        y = gcg_fwd_ref_corrected(x, Bm, Cm, h)
        y2 = gcg_two_pass_chunked_fwd_corrected(x, Bm, Cm, h, gl=128)
        k = f"ops_hl{hl}"
        out[k + "_x"], out[k + "_B"], out[k + "_C"], out[k + "_h"] = np32(x), np32(Bm), np32(Cm), np32(h)
        out[k + "_y"], out[k + "_y_chunked"] = np32(y), np32(y2)
        hf = h.flip(-1)[:, 0]
        out[k + "_T"], out[k + "_That"] = np32(toeplitz(hf, 128)), np32(correction_toeplitz(hf, 128))

    # ---- hyena_ops backward (ref_bwd.py: gcg_two_pass_chunked_bwd), fp32 on CPU ------------------
    from hyena_ops.ref_bwd import gcg_two_pass_chunked_bwd
    for hl, gg, dg, l in ((4, 2, 16, 256), (32, 3, 8, 384), (128, 2, 16, 512)):
        g = torch.Generator().manual_seed(6500 + hl)
        bs = 2
        x, Bm, Cm, dy = (torch.randn(bs, l, gg, dg, generator=g) for _ in range(4))
        h = torch.randn(gg, 1, hl, generator=g) / hl ** 0.5
        y2 = gcg_fwd_ref_corrected(x, Bm, torch.ones_like(Cm), h)
        dx, dB, dC, dh = gcg_two_pass_chunked_bwd(dy, x, y2, Bm, Cm, h, gl=128)
        k = f"opsbwd_hl{hl}"
        out[k + "_x"], out[k + "_B"], out[k + "_C"], out[k + "_h"] = np32(x), np32(Bm), np32(Cm), np32(h)
        out[k + "_dy"], out[k + "_y2"] = np32(dy), np32(y2)
        out[k + "_dx"], out[k + "_dB"], out[k + "_dC"], out[k + "_dh"] = np32(dx), np32(dB), np32(dC), np32(dh)

    # ---- Hyena-X reference (depthwise FIR on q, k, v, three-way gate) -----------------
    from vortex.ops.hyena_x.triton_indirect_fwd import hyena_x_fwd_ref
    for io, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        for Lh in (4, 16):
            g = torch.Generator().manual_seed(7000 + Lh)
            B, D, L = 2, 24, 75
            qkv = (torch.rand(B, 3 * D, L, generator=g) - 0.5).to(dt)
            h = (torch.rand(3 * D, 1, Lh, generator=g) - 0.5).to(dt)
            k = f"hx_{io}_Lh{Lh}"
            out[k + "_qkv"], out[k + "_h"], out[k + "_y"] = np32(qkv), np32(h), np32(hyena_x_fwd_ref(qkv, h))

    # ---- causal_conv1d reference (width 2..4 depthwise conv, bias, initial / final states, SiLU) --------------
    # the interface module imports its CUDA extension at import time; the reference function itself is pure PyTorch
    sys.modules.setdefault("local_causal_conv1d_cuda", types.ModuleType("local_causal_conv1d_cuda"))
    sys.path.insert(0, os.path.join(ref_root, "vortex", "ops", "conv", "local_causal_conv1d"))
    from causal_conv1d_interface import causal_conv1d_ref
    for io, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        for W in (2, 3, 4):
            for L in (1, 2, 37):
                g = torch.Generator().manual_seed(8000 + 10 * W + L)
                B, D = 2, 12
                x = torch.randn(B, D, L, generator=g).to(dt)
                w = torch.randn(D, W, generator=g).to(dt)
                b = torch.randn(D, generator=g).to(dt)
                ini = torch.randn(B, D, W - 1, generator=g).to(dt)
                k = f"cc1d_{io}_W{W}_L{L}"
                out[k + "_x"], out[k + "_w"], out[k + "_b"], out[k + "_ini"] = np32(x), np32(w), np32(b), np32(ini)
                y0, f0 = causal_conv1d_ref(x, w, None, None, True, None, None)
                y1, f1 = causal_conv1d_ref(x, w, b, ini, True, None, "silu")
                out[k + "_y_plain"], out[k + "_fs_plain"] = np32(y0), np32(f0)
                out[k + "_y_full"], out[k + "_fs_full"] = np32(y1), np32(f1)

    # ---- states of packed sequences (pure copy; the module's Triton import needs no GPU) ----------------------
    from causal_conv1d_varlen import causal_conv1d_varlen_states_ref
    for n, (lens, dim, sl) in enumerate([((5, 1, 9, 3), 12, 3), ((2, 40), 7, 6), ((17,), 33, 16)]):
        g = torch.Generator().manual_seed(8500 + n)
        cu = torch.tensor((0,) + tuple(np.cumsum(lens)), dtype=torch.int32)
        x = torch.randn(int(cu[-1]), dim, generator=g)
        k = f"vls_{n}"
        out[k + "_x"], out[k + "_cu"] = np32(x), cu.numpy()
        out[k + "_st"] = np32(causal_conv1d_varlen_states_ref(x, cu, sl))

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1e6:.2f} MB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python make_golden.py <path to a checkout of the reference>")
    main(sys.argv[1])
