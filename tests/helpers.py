"""Seeded inputs shaped like the benchmark configurations, and comparison helpers."""
import numpy as np
import torch

from oracle import hyena_oracle as O

DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
TOL = {"f32": 1e-4, "bf16": 2e-3, "f16": 1e-3}   # relative L2 against the fp32 oracle (north-star tolerances)


def to_np(t):
    return t.detach().float().cpu().numpy()


def rel_l2(a, b):
    return O.rel_l2(to_np(a) if torch.is_tensor(a) else a, to_np(b) if torch.is_tensor(b) else b)


def check(label, err, tol):
    """Assert err <= tol and leave the measured figure in the captured output (``pytest -s`` or ``-rP`` shows it)."""
    print(f"PARITY {label}: {err:.3e} (tolerance {tol:.1e})")
    assert err <= tol, f"{label}: {err:.3e} > {tol:.1e}"


def make_block(seed, B, L, D, G, K, io, modal=False, S=16, complex_poles=False):
    """Random projection output u [B, L, 3D] and the parameters of one Hyena block (CPU tensors)."""
    g = torch.Generator().manual_seed(seed)
    dt = DT[io]
    p = {"u": torch.randn(B, L, 3 * D, generator=g).to(dt),
         "w3": (torch.randn(3 * D, 1, 3, generator=g) / 3 ** 0.5).to(dt)}
    if not modal:
        w = torch.randn(G, 1, K, generator=g) / K ** 0.5
        if K >= 128:   # decaying medium filter: h[t] = w[t] exp(-alpha t), alpha ~ U(0.01, 0.1)
            alpha = 0.01 + 0.09 * torch.rand(G, 1, 1, generator=g)
            w = w * torch.exp(-alpha * torch.arange(K)[None, None])
        p["h"] = w.to(dt)
        p["Dp"] = (0.5 * torch.randn(D, generator=g)).to(dt) if K >= 128 else None
    else:
        mag = 0.9 + 0.099 * torch.rand(G, S, generator=g)
        p["log_poles"] = torch.log(mag)[..., None]
        p["residues"] = torch.randn(G, S, generator=g)
        if complex_poles:
            p["theta"] = torch.pi * torch.rand(G, S, generator=g)
            p["res_im"] = torch.randn(G, S, generator=g)
        p["Dp"] = torch.randn(D, generator=g).to(dt)
    return p


def cuda(p):
    return {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in p.items()}
