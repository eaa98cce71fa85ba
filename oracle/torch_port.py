"""torch-CPU restatement of the reference Hyena path (TEST INFRASTRUCTURE).

Same operator sequence and dtype flow as the reference engine, expressed with
the CPU library calls the reference itself lands on (``F.conv1d`` for short
filters, ``torch.fft`` for filters of 128 taps and more).  This is the timed
CPU baseline of ``bench.py`` (``cpu_baseline.kind == "port"``) and a second
checker next to the numpy oracle.  Functions cite ``vortex/model/engine.py``
unless stated otherwise.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _qkv(z, D, layout, num_heads, flip):
    """engine.py:150-158 with the caller's interleave (utils.py:26-38)."""
    if layout == "interleaved":
        q, k, v = z[:, 0::3], z[:, 1::3], z[:, 2::3]
    elif layout == "split":
        q, k, v = z[:, :D], z[:, D:2 * D], z[:, 2 * D:]
    elif layout == "column_split":  # utils.py:41-85
        hd = D // num_heads
        zz = z.reshape(z.shape[0], num_heads, 3 * hd, *z.shape[2:])
        q, k, v = (zz[:, :, i * hd:(i + 1) * hd].reshape(z.shape[0], D, *z.shape[2:]) for i in range(3))
    else:
        raise ValueError(layout)
    return (k, q, v) if flip else (q, k, v)


def _depthwise(x, w):
    """engine.py:197-204: fp32 depthwise conv, left padding K-1, cut to L."""
    K = w.shape[-1]
    L = x.shape[-1]
    return F.conv1d(x.float(), w.float().reshape(-1, 1, K), padding=K - 1, groups=x.shape[1])[..., :L]


def _fft_conv(x, h):
    """engine.py:50-73 / 331-337: rfft(2L) product, fp32."""
    L = x.shape[-1]
    n = 2 * L
    Hf = torch.fft.rfft(h.float(), n=n) / n
    Xf = torch.fft.rfft(x.float(), n=n)
    return torch.fft.irfft(Xf * Hf, n=n, norm="forward")[..., :L]


def featurizer(u_blc, w, bias=None):
    """engine.py:188-223,255-260 with gate=False, dim_last=True."""
    x = u_blc.permute(0, 2, 1)
    z = _depthwise(x, w).to(x.dtype)
    if bias is not None:
        z = z + bias[None, :, None]
    K = w.shape[-1]
    return z, x[..., -(K - 1):]


def gate_conv_gate(z_pre, h, bias, D, fir_length, layout="split", num_heads=1,
                   flip=False, gated_bias=False):
    """engine.py:150-159,174-232,255-258 with gate=True, dim_last=False."""
    q, k, v = _qkv(z_pre, D, layout, num_heads, flip)
    kv = k * v
    G = h.shape[0]
    hd = h.reshape(G, -1).repeat_interleave(D // G, 0)  # model.py:261-262
    L = z_pre.shape[-1]
    if fir_length >= 128:
        z = _fft_conv(kv, hd[:, :L]) + kv.float() * bias.float()[None, :, None]
        z = z.to(kv.dtype)
    else:
        z = _depthwise(kv, hd).to(kv.dtype)
        if bias is not None:
            z = z + (bias[None, :, None] * kv if gated_bias else bias[None, :, None])
    return q * z, kv[..., -(fir_length - 1):]


def modal_filter(log_poles, residues, L):
    """model.py:390-398."""
    t = torch.arange(L)[None, None]
    return (residues.float()[..., None] * (log_poles.float() * t).exp()).sum(1)


def long_conv_gate(z_pre, h_dl, bias, D, layout="split", num_heads=1, flip=False,
                   log_poles_d=None):
    """engine.py:282-353,404 (+ 525-559 for the state when log_poles_d
    [D, S, 1] is given).  Returns y [B, L, D] and state [B, D, S] or None."""
    q, k, v = _qkv(z_pre, D, layout, num_heads, flip)
    kv = k * v
    L = kv.shape[-1]
    n = 2 * L
    Hf = torch.fft.rfft(h_dl.float(), n=n) / n
    Xs = torch.fft.fft(kv.float(), n=n)
    y = torch.fft.irfft(Xs[..., : Hf.shape[-1]] * Hf, n=n, norm="forward")[..., :L].to(kv.dtype)
    y = (y + kv * bias[None, :, None]) * q
    state = None
    if log_poles_d is not None:
        t = torch.arange(L)[None, None]
        Ss = torch.fft.fft((log_poles_d.float() * t).exp(), n=n)  # D, S, 2L
        st = torch.fft.ifft(Xs[:, :, None, :] * Ss[None], n=n)
        state = st[..., L - 1].real.float()
    return y.permute(0, 2, 1), state


def step_fir(u, fir_state, weight, bias=None, gated_bias=False, flip_filter=False):
    """engine.py:406-449."""
    w = weight.reshape(weight.shape[0], -1)
    K = w.shape[-1]
    c = fir_state.shape[-1]
    w = (w.flip(-1)[:, -c - 1:] if flip_filter else w[:, : c + 1]).float()[None]
    uf, sf = u.float(), fir_state.float()
    y = w[..., -1] * uf + (sf * w[..., :-1]).sum(-1)
    if bias is not None:
        y = y + (bias.float() * uf if gated_bias else bias.float())
    if c < K - 1:
        sf = torch.cat([sf, uf[..., None]], -1)
    else:
        sf = torch.cat([sf[..., 1:], uf[..., None]], -1)
    return y.to(u.dtype), sf


def step_iir(x2, x1, v, D, residues, log_poles, state):
    """engine.py:451-467."""
    kv = x1 * v
    state = torch.exp(log_poles)[..., 0][None] * state + kv[..., None]
    return x2 * ((residues[None] * state).sum(-1) + D * kv), state
