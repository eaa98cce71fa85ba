"""Tensor-level wrappers over the C ABI.

torch is used for device memory and streams only: every function here allocates its outputs
with torch, hands raw pointers to ``libvortex_b200.so`` on the current stream of the input's
device, and returns.  CPU tensors are rejected -- there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import (BF16, BIAS_ADD, BIAS_GATED, BIAS_NONE, F16, F32, QKV_COLUMN_SPLIT, QKV_INTERLEAVED,
                   QKV_SPLIT, TAPS_CONV, TAPS_XCORR)

_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
LAYOUTS = {"split": QKV_SPLIT, "interleaved": QKV_INTERLEAVED, "column_split": QKV_COLUMN_SPLIT}


def _code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"vortex_b200: unsupported dtype {t.dtype}") from None


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("vortex_b200 kernels need CUDA tensors (there is no CPU path)")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _param(t: Optional[torch.Tensor], like: torch.Tensor) -> Optional[torch.Tensor]:
    """Parameters are read with their own dtype; make them dense and co-located."""
    if t is None:
        return None
    t = t.detach()
    if t.device != like.device:
        raise RuntimeError("vortex_b200: parameter on a different device than the activations")
    if t.dtype not in _DT:
        t = t.float()
    return t.contiguous()


def _stream(t: torch.Tensor):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


class _on:
    """Make the tensor's device current for the duration of a call."""

    def __init__(self, t):
        self.g = torch.cuda.device(t.device)

    def __enter__(self):
        self.g.__enter__()

    def __exit__(self, *a):
        self.g.__exit__(*a)


def device_status() -> None:
    """Raise if a kernel recorded that one of its bounded waits ran out (synchronises)."""
    torch.cuda.synchronize()
    _lib.check(_lib.lib().vtx_device_status())


def launch_count() -> int:
    """Kernels this library has launched since it was loaded (read it before and after a region to count its launches)."""
    return int(_lib.lib().vtx_launch_count())


# ----------------------------------------------------------------------------------------------
def featurizer_fwd(u_blc: torch.Tensor, w: torch.Tensor, bias=None, mask=None, want_state=True):
    """u_blc: logical [B, L, C] (any strides).  Returns z [B, C, L] and state [B, C, min(L,K-1)] or None."""
    _need_cuda(u_blc, w, bias, mask)
    B, L, Cc = u_blc.shape
    w = _param(w, u_blc).reshape(Cc, -1)
    K = w.shape[1]
    bias, mask = _param(bias, u_blc), _param(mask, u_blc)
    z = torch.empty(B, Cc, L, device=u_blc.device, dtype=u_blc.dtype)
    ns = min(L, K - 1)
    state = torch.empty(B, Cc, ns, device=u_blc.device, dtype=u_blc.dtype) if want_state else None
    p = _lib.FeaturizerParams(
        u=_ptr(u_blc), u_stride_b=u_blc.stride(0), u_stride_l=u_blc.stride(1), u_stride_c=u_blc.stride(2),
        w=_ptr(w), w_dtype=_code(w), bias=_ptr(bias), bias_dtype=_code(bias) if bias is not None else 0,
        mask=_ptr(mask), mask_dtype=_code(mask) if mask is not None else 0, z=_ptr(z),
        state=_ptr(state) if (state is not None and ns > 0) else None, B=B, L=L, C=Cc, K=K, io_dtype=_code(u_blc))
    with _on(u_blc):
        _lib.check(_lib.lib().vtx_featurizer_fwd(C.byref(p), _stream(u_blc)))
    return z, state


def _qkv_views(z: torch.Tensor, D: int, layout: str, num_heads: int, flip: bool):
    """z [B, 3D, L] (time stride 1) -> ((q,k,v) tensors sharing storage, head_dim, per-stream (stride_h, stride_d))."""
    sc = z.stride(1)
    if layout == "split":
        views = (z[:, :D], z[:, D:2 * D], z[:, 2 * D:])
        hd, strides = D, (0, sc)
    elif layout == "interleaved":
        views = (z[:, 0::3], z[:, 1::3], z[:, 2::3])
        hd, strides = D, (0, 3 * sc)
    elif layout == "column_split":
        hd = D // num_heads
        views = (z[:, 0:], z[:, hd:], z[:, 2 * hd:])   # base pointers; channel d -> head d//hd, lane d%hd
        strides = (3 * hd * sc, sc)
    else:
        raise ValueError(f"unknown q/k/v layout {layout!r}")
    q, k, v = views
    if flip:
        q, k = k, q
    return (q, k, v), hd, strides


def gcg_fwd(z_pre: torch.Tensor, h: torch.Tensor, bias, D: int, *, taps: int, bias_mode: int, layout="split",
            num_heads=1, flip=False, mask=None, want_state=True, round_kv=True, channel_last_out=False):
    """Gate -> grouped FIR -> gate on the packed channel-first tensor z_pre [B, 3D, L].

    Returns y [B, D, L] (or [B, L, D] when channel_last_out) and state [B, D, min(L, K-1)] or None."""
    _need_cuda(z_pre, h, bias, mask)
    if z_pre.stride(2) != 1:
        z_pre = z_pre.contiguous()
    B, C3, L = z_pre.shape
    if C3 != 3 * D:
        raise ValueError(f"expected {3 * D} packed channels, got {C3}")
    (q, k, v), hd, (sh, sd) = _qkv_views(z_pre, D, layout, num_heads, flip)
    return _gcg_raw(q, k, v, z_pre.stride(0), sh, sd, hd, h, bias, B, L, D, taps=taps, bias_mode=bias_mode, mask=mask,
                    want_state=want_state, round_kv=round_kv, channel_last_out=channel_last_out)


def _gcg_raw(q, k, v, sb, sh, sd, hd, h, bias, B, L, D, *, taps, bias_mode, mask, want_state, round_kv,
             channel_last_out):
    dev, dt = q.device, q.dtype
    h = _param(h, q)
    G = h.shape[0]
    h = h.reshape(G, -1)
    K = h.shape[1]
    bias, mask = _param(bias, q), _param(mask, q)
    if channel_last_out:
        y = torch.empty(B, L, D, device=dev, dtype=dt)
        ysb, ysd, ysl = L * D, 1, D
    else:
        y = torch.empty(B, D, L, device=dev, dtype=dt)
        ysb, ysd, ysl = D * L, L, 1
    ns = min(L, K - 1)
    state = torch.empty(B, D, ns, device=dev, dtype=dt) if want_state else None
    sbs = sb if isinstance(sb, tuple) else (sb, sb, sb)
    shs = sh if isinstance(sh, tuple) else (sh, sh, sh)
    sds = sd if isinstance(sd, tuple) else (sd, sd, sd)
    p = _lib.GcgParams(
        q=_ptr(q), q_stride_b=sbs[0], q_stride_h=shs[0], q_stride_d=sds[0],
        k=_ptr(k), k_stride_b=sbs[1], k_stride_h=shs[1], k_stride_d=sds[1],
        v=_ptr(v), v_stride_b=sbs[2], v_stride_h=shs[2], v_stride_d=sds[2], head_dim=hd,
        h=_ptr(h), h_dtype=_code(h), bias=_ptr(bias), bias_dtype=_code(bias) if bias is not None else 0,
        mask=_ptr(mask), mask_dtype=_code(mask) if mask is not None else 0,
        y=_ptr(y), y_stride_b=ysb, y_stride_d=ysd, y_stride_l=ysl,
        state=_ptr(state) if (state is not None and ns > 0) else None,
        B=B, L=L, D=D, G=G, K=K, taps=taps, bias_mode=bias_mode if bias is not None else BIAS_NONE,
        round_kv=int(round_kv), io_dtype=_DT[dt])
    with _on(q):
        _lib.check(_lib.lib().vtx_gcg_fwd(C.byref(p), _stream(q)))
    return y, state


def gcg_fwd_bdl(q, k, v, h, bias=None, *, taps=TAPS_XCORR, bias_mode=BIAS_NONE, round_kv=True, want_state=False):
    """Three separate contiguous [B, D, L] operands (hyena_ops 'bdl' layout)."""
    _need_cuda(q, k, v, h, bias)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, D, L = q.shape
    return _gcg_raw(q, k, v, D * L, 0, L, D, h, bias, B, L, D, taps=taps, bias_mode=bias_mode, mask=None,
                    want_state=want_state, round_kv=round_kv, channel_last_out=False)


def gcg_cl_ok(q, k, v, h, bias_mode=BIAS_NONE) -> bool:
    """Shapes ``vtx_gcg_cl_fwd`` takes: bf16 channel-last operands [B, L, D] with unit channel stride and 16-byte
    aligned rows, bf16 filters of up to 128 taps shared by a multiple of 16 channels."""
    if not (q.dtype == k.dtype == v.dtype == h.dtype == torch.bfloat16) or q.dim() != 3 or bias_mode == BIAS_ADD:
        return False
    D, G, K = q.shape[-1], h.shape[0], h.shape[-1]
    if K > 128 or D % G or (D // G) % 16:
        return False
    for t in (q, k, v):
        if t.shape != q.shape or t.stride(2) != 1 or t.data_ptr() % 16 or (t.stride(1) * 2) % 16 or (t.stride(0) * 2) % 16:
            return False
    return True


def gcg_cl_fwd(q, k, v, h, bias=None, *, taps=TAPS_XCORR, bias_mode=BIAS_NONE, want_state=False):
    """Gate -> grouped FIR -> gate on channel-last operands q, k, v [B, L, D] (the hyena_ops layout with the group
    axes merged): one launch of the tensor-core kernel.  Returns y [B, L, D] and the inner cache [B, D, min(L, K-1)]
    or None."""
    _need_cuda(q, k, v, h, bias)
    B, L, D = q.shape
    h = _param(h, q)
    G = h.shape[0]
    h = h.reshape(G, -1)
    K = h.shape[1]
    bias = _param(bias, q)
    y = torch.empty(B, L, D, device=q.device, dtype=q.dtype)
    ns = min(L, K - 1)
    state = torch.empty(B, D, ns, device=q.device, dtype=q.dtype) if want_state else None
    p = _lib.GcgClParams(
        q=_ptr(q), q_stride_b=q.stride(0), q_stride_l=q.stride(1), k=_ptr(k), k_stride_b=k.stride(0), k_stride_l=k.stride(1),
        v=_ptr(v), v_stride_b=v.stride(0), v_stride_l=v.stride(1), h=_ptr(h), h_dtype=_code(h),
        bias=_ptr(bias), bias_dtype=_code(bias) if bias is not None else 0, y=_ptr(y), y_stride_b=L * D, y_stride_l=D,
        state=_ptr(state) if (state is not None and ns > 0) else None, B=B, L=L, D=D, G=G, K=K, taps=taps,
        bias_mode=bias_mode if bias is not None else BIAS_NONE, io_dtype=_code(q))
    with _on(q):
        _lib.check(_lib.lib().vtx_gcg_cl_fwd(C.byref(p), _stream(q)))
    return y, state


def gcg_bwd(dy, x, Bg, Cg, y2, h):
    """Backward of y = Cg * xcorr(h_g, Bg * x) on channel-last tensors [B, L, D] (unit channel stride), y2 the filter
    output the forward saved.  Returns dx, dB, dC [B, L, D] in the I/O dtype and dh [G, K] in fp32."""
    _need_cuda(dy, x, Bg, Cg, y2, h)
    B, L, D = x.shape
    ts = []
    for t in (dy, x, Bg, Cg, y2):
        if tuple(t.shape) != (B, L, D) or t.dtype != x.dtype:
            raise ValueError("dy, x, B, C and y2 must have the same shape and dtype")
        ts.append(t if t.stride(2) == 1 else t.contiguous())
    dy, x, Bg, Cg, y2 = ts
    h = _param(h, x)
    G = h.shape[0]
    h = h.reshape(G, -1)
    K = h.shape[1]
    dx, dB, dC = (torch.empty(B, L, D, device=x.device, dtype=x.dtype) for _ in range(3))
    dh = torch.zeros(G, K, device=x.device, dtype=torch.float32)
    p = _lib.GcgBwdParams(
        dy=_ptr(dy), dy_stride_b=dy.stride(0), dy_stride_l=dy.stride(1), x=_ptr(x), x_stride_b=x.stride(0), x_stride_l=x.stride(1),
        Bg=_ptr(Bg), b_stride_b=Bg.stride(0), b_stride_l=Bg.stride(1), C=_ptr(Cg), c_stride_b=Cg.stride(0), c_stride_l=Cg.stride(1),
        y2=_ptr(y2), y2_stride_b=y2.stride(0), y2_stride_l=y2.stride(1), h=_ptr(h), h_dtype=_code(h),
        dx=_ptr(dx), dB=_ptr(dB), dC=_ptr(dC), dh32=_ptr(dh), B=B, L=L, D=D, G=G, K=K, io_dtype=_code(x))
    with _on(x):
        _lib.check(_lib.lib().vtx_gcg_bwd(C.byref(p), _stream(x)))
    return dx, dB, dC, dh


def fused_fir_fwd(u: torch.Tensor, w3, b3, h, bias, D: int, *, taps: int, bias_mode: int, layout="interleaved",
                  num_heads=1, flip=False, want_state=True, hist_rows=0):
    """Channel-last fused block: u [B, L, 3D] -> y [B, L, D], fir_state [B, 3D, min(L,2)], inner [B, D, min(L,K-1)].

    ``hist_rows`` = H > 0 (chunked prefill): ``u`` is a view whose H preceding rows in memory (same row pitch) hold
    the sequence's earlier projection rows, H >= K + 1; the caches returned are then always full."""
    _need_cuda(u, w3, b3, h, bias)
    if u.stride(2) != 1:
        if hist_rows:
            raise ValueError("hist_rows needs u with unit channel stride (a view into the buffer that holds the history)")
        u = u.contiguous()
    B, L, C3 = u.shape
    if C3 != 3 * D:
        raise ValueError(f"expected {3 * D} packed channels, got {C3}")
    w3 = _param(w3, u).reshape(C3, -1)
    h = _param(h, u)
    G = h.shape[0]
    h = h.reshape(G, -1)
    K, K3 = h.shape[1], w3.shape[1]
    b3, bias = _param(b3, u), _param(bias, u)
    y = torch.empty(B, L, D, device=u.device, dtype=u.dtype)
    if hist_rows and u.storage_offset() < hist_rows * u.stride(1):
        raise ValueError(f"hist_rows={hist_rows}: u starts {u.storage_offset() // max(u.stride(1), 1)} rows into its storage")
    n3, ns = (K3 - 1, K - 1) if hist_rows else (min(L, K3 - 1), min(L, K - 1))
    fs = torch.empty(B, C3, n3, device=u.device, dtype=u.dtype) if want_state else None
    ist = torch.empty(B, D, ns, device=u.device, dtype=u.dtype) if want_state else None
    p = _lib.FusedFirParams(
        u=_ptr(u), u_stride_b=u.stride(0), u_stride_l=u.stride(1), w3=_ptr(w3), w3_dtype=_code(w3),
        b3=_ptr(b3), b3_dtype=_code(b3) if b3 is not None else 0, h=_ptr(h), h_dtype=_code(h),
        bias=_ptr(bias), bias_dtype=_code(bias) if bias is not None else 0,
        y=_ptr(y), y_stride_b=L * D, y_stride_l=D,
        fir_state=_ptr(fs) if (fs is not None and fs.numel()) else None,
        inner_state=_ptr(ist) if (ist is not None and ist.numel()) else None,
        B=B, L=L, D=D, G=G, K3=K3, K=K, layout=LAYOUTS[layout], num_heads=num_heads, flip_x1x2=int(flip),
        taps=taps, bias_mode=bias_mode if bias is not None else BIAS_NONE, io_dtype=_code(u), u_hist_rows=hist_rows)
    with _on(u):
        _lib.check(_lib.lib().vtx_fused_fir_fwd(C.byref(p), _stream(u)))
    return y, fs, ist


# ----------------------------------------------------------------------------------------------
def _modal(log_poles, residues, like, theta=None, res_im=None):
    """fp32 [G, S] parameter block; returns (struct, keep-alive tensors)."""
    R = residues.detach().to(device=like.device, dtype=torch.float32).contiguous()
    G, S = R.shape
    lp = log_poles.detach().to(device=like.device, dtype=torch.float32).reshape(G, S).contiguous()
    th = None if theta is None else theta.detach().to(device=like.device, dtype=torch.float32).reshape(G, S).contiguous()
    ri = None if res_im is None else res_im.detach().to(device=like.device, dtype=torch.float32).reshape(G, S).contiguous()
    m = _lib.ModalParams(log_poles=_ptr(lp), theta=_ptr(th), res_re=_ptr(R), res_im=_ptr(ri), G=G, S=S)
    return m, (lp, R, th, ri)


def modal_filter(log_poles, residues, L: int, theta=None, res_im=None) -> torch.Tensor:
    """h [G, L] fp32 = sum_s R exp(lambda t)   (or sum_s Re(R p^t) with theta / res_im)."""
    _need_cuda(residues)
    m, keep = _modal(log_poles, residues, residues, theta, res_im)
    h = torch.empty(m.G, L, device=residues.device, dtype=torch.float32)
    with _on(residues):
        _lib.check(_lib.lib().vtx_modal_filter(C.byref(m), _ptr(h), L, _stream(residues)))
    return h


def fused_iir_fwd(u: torch.Tensor, w3, log_poles, residues, bias, D: int, *, layout="interleaved", num_heads=1,
                  flip=False, theta=None, res_im=None, want_state=False, b3=None, state_in=None, fir_state_in=None,
                  hist_rows=0, out=None):
    """Channel-last fused long-filter block: u [B, L, 3D] -> y [B, L, D] and, on request, the modal state after the
    last token (fp32 [B, D, S], complex poles [B, D, S, 2]).  The library picks the kernel: tensor cores for bf16
    with one modal system per group of 16 channels, the fp32-pipe recurrence otherwise.  ``state_in`` /
    ``fir_state_in`` ([B, 3D, 2]) continue an earlier call (chunked prefill).  ``hist_rows`` = H >= 2 instead of
    ``fir_state_in``: ``u`` is a view whose H preceding rows in memory (same row pitch) hold the sequence's earlier
    projection rows; with it, and L a multiple of 384, a continued call stays on the tensor-core kernel."""
    _need_cuda(u, w3, residues, bias, b3, state_in, fir_state_in)
    if u.stride(2) != 1:
        if hist_rows:
            raise ValueError("hist_rows needs u with unit channel stride (a view into the buffer that holds the history)")
        u = u.contiguous()
    if hist_rows:
        if hist_rows < 2 or fir_state_in is not None:
            raise ValueError("hist_rows must be >= 2 and excludes fir_state_in")
        if u.storage_offset() < hist_rows * u.stride(1):
            raise ValueError(f"hist_rows={hist_rows}: u starts {u.storage_offset() // max(u.stride(1), 1)} rows into its storage")
    B, L, C3 = u.shape
    if C3 != 3 * D:
        raise ValueError(f"expected {3 * D} packed channels, got {C3}")
    w3 = _param(w3, u).reshape(C3, -1)
    bias, b3 = _param(bias, u), _param(b3, u)
    m, keep = _modal(log_poles, residues, u, theta, res_im)
    cplx = theta is not None
    if out is None:
        y = torch.empty(B, L, D, device=u.device, dtype=u.dtype)
    else:       # a [B, L, D] view with unit channel stride (e.g. a range of rows of a larger output)
        if tuple(out.shape) != (B, L, D) or out.dtype != u.dtype or out.stride(2) != 1 or out.device != u.device:
            raise ValueError("out must be a [B, L, D] tensor of u's dtype and device with unit channel stride")
        y = out
    st = None
    if want_state:
        st = torch.empty((B, D, m.S, 2) if cplx else (B, D, m.S), device=u.device, dtype=torch.float32)
    if state_in is not None:
        if tuple(state_in.shape) != ((B, D, m.S, 2) if cplx else (B, D, m.S)):
            raise ValueError(f"state_in has shape {tuple(state_in.shape)}")
        state_in = state_in.to(torch.float32).contiguous()
    if fir_state_in is not None:
        if tuple(fir_state_in.shape) != (B, C3, 2):
            raise ValueError(f"fir_state_in has shape {tuple(fir_state_in.shape)}, expected {(B, C3, 2)}")
        fir_state_in = fir_state_in.contiguous()
    p = _lib.FusedIirParams(
        u=_ptr(u), u_stride_b=u.stride(0), u_stride_l=u.stride(1), w3=_ptr(w3), w3_dtype=_code(w3),
        b3=_ptr(b3), b3_dtype=_code(b3) if b3 is not None else 0,
        modal=m, bias=_ptr(bias), bias_dtype=_code(bias) if bias is not None else 0,
        y=_ptr(y), y_stride_b=y.stride(0), y_stride_l=y.stride(1), state=_ptr(st), scratch=None, B=B, L=L, D=D, K3=w3.shape[1],
        layout=LAYOUTS[layout], num_heads=num_heads, flip_x1x2=int(flip), io_dtype=_code(u),
        state_in=_ptr(state_in), fir_state_in=_ptr(fir_state_in),
        fir_state_dtype=_code(fir_state_in) if fir_state_in is not None else 0, u_hist_rows=int(hist_rows))
    nscratch = _lib.lib().vtx_fused_iir_scratch_bytes(C.byref(p))
    scratch = torch.empty(nscratch, device=u.device, dtype=torch.uint8) if nscratch > 0 else None
    p.scratch = _ptr(scratch)
    with _on(u):
        _lib.check(_lib.lib().vtx_fused_iir_fwd(C.byref(p), _stream(u)))
    del keep
    return (y, st) if want_state else y


def hyena_x_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, h) -> torch.Tensor:
    """o = fir(h_q, q) * fir(h_k, k) * fir(h_v, v); q, k, v [B, D, L], h [3D, 1, Lh] or [3D, Lh] -> [B, D, L]."""
    _need_cuda(q, k, v, h)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if not (q.shape == k.shape == v.shape and q.dtype == k.dtype == v.dtype):
        raise ValueError("q, k, v must share shape and dtype")
    B, D, L = q.shape
    h = _param(h, q).reshape(3 * D, -1)
    y = torch.empty_like(q)
    p = _lib.HyenaXParams(q=_ptr(q), k=_ptr(k), v=_ptr(v), h=_ptr(h), h_dtype=_code(h), y=_ptr(y), B=B, D=D, L=L,
                          Lh=h.shape[1], io_dtype=_code(q))
    with _on(q):
        _lib.check(_lib.lib().vtx_hyena_x_fwd(C.byref(p), _stream(q)))
    return y


def _act_flag(activation) -> int:
    if activation not in (None, "silu", "swish"):
        raise NotImplementedError("activation must be None, silu, or swish")
    return int(activation is not None)


def causal_conv1d_fwd(x: torch.Tensor, weight: torch.Tensor, bias=None, seq_idx=None, initial_states=None,
                      final_states_out=None, activation=None) -> torch.Tensor:
    """Depthwise causal convolution of 2..4 taps (the reference extension's ``causal_conv1d_fwd``,
    ``vortex/ops/conv/csrc/causal_conv1d.cpp:130-236``): x [B, D, L] with time or channels contiguous, weight [D, W],
    bias [D], seq_idx int32 [B, L], initial_states / final_states_out [B, D, W-1] -> out shaped and strided like x."""
    _need_cuda(x, weight, bias, seq_idx, initial_states, final_states_out)
    if x.dim() != 3 or weight.dim() != 2 or weight.shape[0] != x.shape[1]:
        raise ValueError(f"x {tuple(x.shape)} / weight {tuple(weight.shape)}: expected [B, D, L] and [D, W]")
    B, D, L = x.shape
    W = weight.shape[1]
    silu = _act_flag(activation)
    if x.stride(2) != 1 and x.stride(1) != 1:
        x = x.contiguous()
    weight, bias = _param(weight, x), _param(bias, x)
    if bias is not None and tuple(bias.shape) != (D,):
        raise ValueError(f"bias has shape {tuple(bias.shape)}, expected {(D,)}")
    if seq_idx is not None:
        if seq_idx.dtype != torch.int32 or tuple(seq_idx.shape) != (B, L):
            raise ValueError("seq_idx must be int32 of shape [B, L]")
        seq_idx = seq_idx.contiguous()
    for name, t in (("initial_states", initial_states), ("final_states_out", final_states_out)):
        if t is not None and (tuple(t.shape) != (B, D, W - 1) or t.dtype != x.dtype):
            raise ValueError(f"{name} must be [B, D, W-1] of x's dtype")
    out = torch.empty_like(x)              # keeps x's layout (dense time-last or channel-last)
    if out.stride() != x.stride():
        out = torch.empty_strided(x.shape, x.stride(), device=x.device, dtype=x.dtype) if x.is_non_overlapping_and_dense() \
            else torch.empty(x.shape, device=x.device, dtype=x.dtype)
    ini, fs = initial_states, final_states_out
    p = _lib.CausalConv1dParams(
        x=_ptr(x), x_stride_b=x.stride(0), x_stride_d=x.stride(1), x_stride_l=x.stride(2),
        weight=_ptr(weight), weight_dtype=_code(weight), bias=_ptr(bias), bias_dtype=_code(bias) if bias is not None else 0,
        seq_idx=_ptr(seq_idx), initial_states=_ptr(ini),
        is_stride_b=ini.stride(0) if ini is not None else 0, is_stride_d=ini.stride(1) if ini is not None else 0,
        is_stride_l=ini.stride(2) if ini is not None else 0, final_states=_ptr(fs),
        fs_stride_b=fs.stride(0) if fs is not None else 0, fs_stride_d=fs.stride(1) if fs is not None else 0,
        fs_stride_l=fs.stride(2) if fs is not None else 0,
        out=_ptr(out), out_stride_b=out.stride(0), out_stride_d=out.stride(1), out_stride_l=out.stride(2),
        B=B, D=D, L=L, W=W, silu=silu, io_dtype=_code(x))
    with _on(x):
        _lib.check(_lib.lib().vtx_causal_conv1d_fwd(C.byref(p), _stream(x)))
    return out


def causal_conv1d_update(x: torch.Tensor, conv_state: torch.Tensor, weight: torch.Tensor, bias=None, activation=None,
                         cache_seqlens=None, conv_state_indices=None) -> torch.Tensor:
    """Decode-time update of the same convolution (``causal_conv1d.cpp:382-470``): x [B, D] or [B, D, Lq],
    conv_state [rows, D, state_len] updated in place (shift register, or circular with cache_seqlens int32 [B];
    conv_state_indices int32 [B] picks the state row per batch element) -> out shaped like x."""
    _need_cuda(x, conv_state, weight, bias, cache_seqlens, conv_state_indices)
    silu = _act_flag(activation)
    squeeze = x.dim() == 2
    if squeeze:
        x = x.unsqueeze(-1)
    B, D, L = x.shape
    W = weight.shape[1]
    if conv_state.dtype != x.dtype:
        raise TypeError("conv_state must have x's dtype")
    rows = conv_state.shape[0]
    if conv_state.dim() != 3 or conv_state.shape[1] != D or (conv_state_indices is None and rows != B):
        raise ValueError(f"conv_state has shape {tuple(conv_state.shape)}")
    if tuple(weight.shape) != (D, W):
        raise ValueError(f"weight has shape {tuple(weight.shape)}, expected {(D, W)}")
    weight, bias = _param(weight, x), _param(bias, x)
    for name, t in (("cache_seqlens", cache_seqlens), ("conv_state_indices", conv_state_indices)):
        if t is not None and (t.dtype != torch.int32 or tuple(t.shape) != (B,) or t.stride(0) != 1):
            raise ValueError(f"{name} must be a dense int32 vector of length B")
    out = torch.empty_like(x)
    p = _lib.CausalConv1dUpdateParams(
        x=_ptr(x), x_stride_b=x.stride(0), x_stride_d=x.stride(1), x_stride_l=x.stride(2),
        conv_state=_ptr(conv_state), cs_stride_b=conv_state.stride(0), cs_stride_d=conv_state.stride(1),
        cs_stride_l=conv_state.stride(2), state_len=conv_state.shape[2],
        weight=_ptr(weight), weight_dtype=_code(weight), bias=_ptr(bias), bias_dtype=_code(bias) if bias is not None else 0,
        cache_seqlens=_ptr(cache_seqlens), conv_state_indices=_ptr(conv_state_indices),
        out=_ptr(out), out_stride_b=out.stride(0), out_stride_d=out.stride(1), out_stride_l=out.stride(2),
        B=B, D=D, L=L, W=W, silu=silu, io_dtype=_code(x))
    with _on(x):
        _lib.check(_lib.lib().vtx_causal_conv1d_update(C.byref(p), _stream(x)))
    return out.squeeze(-1) if squeeze else out


def causal_conv1d_varlen_states(x: torch.Tensor, cu_seqlens: torch.Tensor, state_len: int) -> torch.Tensor:
    """x [total_tokens, dim] (sequences back to back), cu_seqlens int32 [batch + 1] -> states [batch, dim, state_len]
    (memory [batch, state_len, dim] like the reference's, ``causal_conv1d_varlen.py:42-75``): the last rows of each
    sequence, zeros where a sequence is shorter than state_len."""
    _need_cuda(x, cu_seqlens)
    if x.dim() != 2 or cu_seqlens.dim() != 1 or cu_seqlens.numel() < 2:
        raise ValueError("x must be [total_tokens, dim] and cu_seqlens [batch + 1]")
    if cu_seqlens.dtype != torch.int32:
        raise TypeError("cu_seqlens must be int32")
    if int(state_len) < 1:
        raise ValueError("state_len must be positive")
    cu_seqlens = cu_seqlens.contiguous()
    total, dim = x.shape
    batch = cu_seqlens.numel() - 1
    states = torch.empty(batch, state_len, dim, dtype=x.dtype, device=x.device).transpose(1, 2)
    p = _lib.VarlenStatesParams(
        x=_ptr(x), x_stride_t=x.stride(0), x_stride_c=x.stride(1), cu_seqlens=_ptr(cu_seqlens), states=_ptr(states),
        st_stride_b=states.stride(0), st_stride_c=states.stride(1), st_stride_l=states.stride(2),
        total=total, batch=batch, dim=dim, state_len=int(state_len), io_dtype=_code(x))
    with _on(x):
        _lib.check(_lib.lib().vtx_causal_conv1d_varlen_states(C.byref(p), _stream(x)))
    return states


def iir_fwd(z_pre: torch.Tensor, log_poles, residues, bias, D: int, *, layout="split", num_heads=1, flip=False,
            theta=None, res_im=None, want_state=True, round_kv=True):
    """Gate -> modal long convolution -> gate.  z_pre [B, 3D, L] -> y [B, D, L] (contiguous), state fp32
    [B, D, S] (or [B, D, S, 2] for complex poles) or None."""
    _need_cuda(z_pre, residues, bias)
    if z_pre.stride(2) != 1:
        z_pre = z_pre.contiguous()
    B, C3, L = z_pre.shape
    if C3 != 3 * D:
        raise ValueError(f"expected {3 * D} packed channels, got {C3}")
    (q, k, v), hd, (sh, sd) = _qkv_views(z_pre, D, layout, num_heads, flip)
    m, keep = _modal(log_poles, residues, z_pre, theta, res_im)
    cplx = theta is not None
    bias = _param(bias, z_pre)
    y = torch.empty(B, D, L, device=z_pre.device, dtype=z_pre.dtype)
    state = None
    if want_state:
        state = torch.empty((B, D, m.S, 2) if cplx else (B, D, m.S), device=z_pre.device, dtype=torch.float32)
    nbytes = _lib.lib().vtx_iir_scratch_bytes(B, L, D, m.S, int(cplx))
    scratch = torch.empty(nbytes, device=z_pre.device, dtype=torch.uint8) if nbytes else None
    p = _lib.IirParams(
        q=_ptr(q), q_stride_b=z_pre.stride(0), q_stride_h=sh, q_stride_d=sd,
        k=_ptr(k), k_stride_b=z_pre.stride(0), k_stride_h=sh, k_stride_d=sd,
        v=_ptr(v), v_stride_b=z_pre.stride(0), v_stride_h=sh, v_stride_d=sd, head_dim=hd, modal=m,
        bias=_ptr(bias), bias_dtype=_code(bias) if bias is not None else 0,
        y=_ptr(y), y_stride_b=D * L, y_stride_d=L, y_stride_l=1, state=_ptr(state), scratch=_ptr(scratch),
        B=B, L=L, D=D, round_kv=int(round_kv), io_dtype=_code(z_pre))
    with _on(z_pre):
        _lib.check(_lib.lib().vtx_iir_fwd(C.byref(p), _stream(z_pre)))
    return y, state


def iir_recurrence_fwd(z_pre: torch.Tensor, poles_ri, residues_ri, bias, D: int, *, layout="split", num_heads=1,
                       flip=False):
    """The reference's legacy recurrent prefill (engine.py:473-504): poles_ri / residues_ri [D, S, 2] as (re, im).
    z_pre [B, 3D, L] -> y [B, D, L] and the state fp32 [B, D, S, 2] after the last token."""
    _need_cuda(z_pre, poles_ri, residues_ri, bias)
    if z_pre.stride(2) != 1:
        z_pre = z_pre.contiguous()
    B, C3, L = z_pre.shape
    if C3 != 3 * D:
        raise ValueError(f"expected {3 * D} packed channels, got {C3}")
    if poles_ri.dim() != 3 or poles_ri.shape[-1] != 2 or poles_ri.shape != residues_ri.shape:
        raise ValueError("poles and residues must be [D, S, 2] (re, im)")
    G, S, _ = poles_ri.shape
    f = lambda t: t.detach().to(device=z_pre.device, dtype=torch.float32).contiguous()  # noqa: E731
    pre, pim, rre = f(poles_ri[..., 0]), f(poles_ri[..., 1]), f(residues_ri[..., 0])
    (q, k, v), hd, (sh, sd) = _qkv_views(z_pre, D, layout, num_heads, flip)
    bias = _param(bias, z_pre)
    y = torch.empty(B, D, L, device=z_pre.device, dtype=z_pre.dtype)
    state = torch.empty(B, D, S, 2, device=z_pre.device, dtype=torch.float32)
    m = _lib.ModalParams(log_poles=_ptr(pre), theta=_ptr(pim), res_re=_ptr(rre), res_im=None, G=G, S=S)
    p = _lib.IirParams(
        q=_ptr(q), q_stride_b=z_pre.stride(0), q_stride_h=sh, q_stride_d=sd,
        k=_ptr(k), k_stride_b=z_pre.stride(0), k_stride_h=sh, k_stride_d=sd,
        v=_ptr(v), v_stride_b=z_pre.stride(0), v_stride_h=sh, v_stride_d=sd, head_dim=hd, modal=m,
        bias=_ptr(bias), bias_dtype=_code(bias) if bias is not None else 0,
        y=_ptr(y), y_stride_b=D * L, y_stride_d=L, y_stride_l=1, state=_ptr(state), scratch=None,
        B=B, L=L, D=D, round_kv=1, io_dtype=_code(z_pre))
    with _on(z_pre):
        _lib.check(_lib.lib().vtx_iir_recurrence_fwd(C.byref(p), _stream(z_pre)))
    return y, state


# ----------------------------------------------------------------------------------------------
def step_fir(u: torch.Tensor, fir_state: torch.Tensor, weight, bias=None, gated_bias=False, flip_filter=False):
    """One decode step of a depthwise FIR.  u [B, C]; fir_state [B, C, c]; weight [Gw, 1, K] / [Gw, K].
    Returns y [B, C] (dtype of u) and the new fp32 state [B, C, min(c+1, K-1)]."""
    _need_cuda(u, fir_state, weight, bias)
    u = u.contiguous()
    B, Cc = u.shape
    w = _param(weight, u)
    w = w.reshape(w.shape[0], -1)
    Gw, K = w.shape
    st = fir_state.contiguous()
    if st.dtype not in _DT:
        st = st.float()
    c = st.shape[-1]
    bias = _param(bias, u)
    y = torch.empty_like(u)
    c_out = c + 1 if c < K - 1 else c
    out = torch.empty(B, Cc, c_out, device=u.device, dtype=torch.float32)
    p = _lib.StepFirParams(
        u=_ptr(u), state_in=_ptr(st) if c > 0 else None, state_dtype=_code(st), w=_ptr(w), w_dtype=_code(w),
        bias=_ptr(bias), bias_dtype=_code(bias) if bias is not None else 0, y=_ptr(y),
        state_out=_ptr(out) if c_out > 0 else None, B=B, C=Cc, Gw=Gw, K=K, c=c, flip_filter=int(flip_filter),
        bias_mode=(BIAS_GATED if gated_bias else BIAS_ADD) if bias is not None else BIAS_NONE, io_dtype=_code(u))
    with _on(u):
        _lib.check(_lib.lib().vtx_step_fir(C.byref(p), _stream(u)))
    return y, out


def step_iir(q, k, v, bias, residues, log_poles, state, *, theta=None, res_im=None, inplace=False):
    """One decode step of the modal recurrence.  q, k, v [B, D]; state fp32 [B, D, S(,2)].
    Returns y fp32 [B, D] and the new state."""
    _need_cuda(q, k, v, residues, state)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, D = q.shape
    m, keep = _modal(log_poles, residues, q, theta, res_im)
    bias = _param(bias, q)
    st = state.contiguous()
    if st.dtype != torch.float32:
        st = st.float()
    out = st if inplace else torch.empty_like(st)
    y = torch.empty(B, D, device=q.device, dtype=torch.float32)
    p = _lib.StepIirParams(q=_ptr(q), k=_ptr(k), v=_ptr(v), modal=m, bias=_ptr(bias),
                           bias_dtype=_code(bias) if bias is not None else 0, state_in=_ptr(st), state_out=_ptr(out),
                           y=_ptr(y), B=B, D=D, io_dtype=_code(q))
    with _on(q):
        _lib.check(_lib.lib().vtx_step_iir(C.byref(p), _stream(q)))
    return y, out


def decode_layer(u, w3, b3, fir_state, D, *, h=None, inner_state=None, bias=None, flip_filter=False, gated_bias=False,
                 log_poles=None, residues=None, iir_state=None, theta=None, res_im=None, layout="interleaved",
                 num_heads=1, flip=False):
    """Whole Hyena layer for one token: u [B, 3D] -> y [B, D] plus the new caches.

    FIR layers pass h / inner_state; the long (modal) layer passes log_poles / residues / iir_state.
    Returns (y, new_fir_state fp32, new_inner_or_iir_state)."""
    _need_cuda(u, w3, fir_state)
    u = u.contiguous()
    B, C3 = u.shape
    if C3 != 3 * D:
        raise ValueError(f"expected {3 * D} packed channels, got {C3}")
    w3 = _param(w3, u).reshape(C3, -1)
    K3 = w3.shape[1]
    b3, bias = _param(b3, u), _param(bias, u)
    fs = fir_state.contiguous()
    if fs.shape[-1] != K3 - 1:
        raise NotImplementedError("decode_layer needs a full featurizer cache (prompt of at least K3-1 tokens)")
    fs_out = torch.empty(B, C3, K3 - 1, device=u.device, dtype=torch.float32)
    y = torch.empty(B, D, device=u.device, dtype=u.dtype)
    p = _lib.DecodeLayerParams(
        u=_ptr(u), w3=_ptr(w3), w3_dtype=_code(w3), b3=_ptr(b3), b3_dtype=_code(b3) if b3 is not None else 0,
        fir_state_in=_ptr(fs), fir_state_dtype=_code(fs), fir_state_out=_ptr(fs_out), bias=_ptr(bias),
        bias_dtype=_code(bias) if bias is not None else 0, y=_ptr(y), B=B, D=D, K3=K3, layout=LAYOUTS[layout],
        num_heads=num_heads, flip_x1x2=int(flip), flip_filter=int(flip_filter), io_dtype=_code(u))
    keep = None
    if h is not None:
        h = _param(h, u)
        G = h.shape[0]
        h = h.reshape(G, -1)
        K = h.shape[1]
        ins = inner_state.contiguous()
        if ins.shape[-1] != K - 1:
            raise NotImplementedError("decode_layer needs a full inner cache (prompt of at least K-1 tokens)")
        new_state = torch.empty(B, D, K - 1, device=u.device, dtype=torch.float32)
        p.h, p.h_dtype, p.G, p.K = _ptr(h), _code(h), G, K
        p.inner_state_in, p.inner_state_dtype, p.inner_state_out = _ptr(ins), _code(ins), _ptr(new_state)
        p.bias_mode = (BIAS_GATED if gated_bias else BIAS_ADD) if bias is not None else BIAS_NONE
    else:
        m, keep = _modal(log_poles, residues, u, theta, res_im)
        st = iir_state.contiguous()
        if st.dtype != torch.float32:
            st = st.float()
        new_state = torch.empty_like(st)
        p.modal, p.K, p.G = m, 0, m.G
        p.iir_state_in, p.iir_state_out = _ptr(st), _ptr(new_state)
    with _on(u):
        _lib.check(_lib.lib().vtx_decode_layer(C.byref(p), _stream(u)))
    return y, fs_out, new_state


def iir_fwd_noalloc(z_pre: torch.Tensor, log_poles, residues, bias, D: int, y: torch.Tensor, state: Optional[torch.Tensor],
                    *, layout="split", num_heads=1, flip=False, theta=None, res_im=None, round_kv=True) -> None:
    """``vtx_iir_fwd_noalloc``: the modal long convolution for callers that may not allocate on the device.

    Nothing is allocated here or in the library: ``y`` [B, D, L] (dtype of ``z_pre``) and ``state`` (fp32
    [B, D, S] or [B, D, S, 2], or None) are the caller's, the parameters must already be fp32, contiguous and
    on the device, and the segment carries go into the scratch array built into the library.  Sizes beyond
    that array raise NotImplementedError.  Calls share the array: do not overlap them on the GPU."""
    _need_cuda(z_pre, residues, log_poles, bias, y, state)
    B, C3, L = z_pre.shape
    if C3 != 3 * D or z_pre.stride(2) != 1:
        raise ValueError("z_pre must be [B, 3D, L] with unit time stride")
    for t in (log_poles, residues, theta, res_im):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise ValueError("modal parameters must be contiguous fp32 tensors (no conversion is done on this path)")
    if y.shape != (B, D, L) or not y.is_contiguous() or y.dtype != z_pre.dtype:
        raise ValueError("y must be a contiguous [B, D, L] tensor of the input dtype")
    if residues.dim() != 2:
        raise ValueError("residues must be [G, S]")
    G, S = residues.shape
    cplx = theta is not None
    if state is not None:
        want = (B, D, S, 2) if cplx else (B, D, S)
        if (state.dtype != torch.float32 or tuple(state.shape) != want or not state.is_contiguous()
                or state.device != z_pre.device):
            raise ValueError(f"state must be a contiguous fp32 {want} tensor on the device of z_pre (the kernel "
                             "writes that many floats through the pointer)")
    if y.device != z_pre.device:
        raise ValueError("y must be on the device of z_pre")
    if bias is not None and (tuple(bias.shape) != (D,) or not bias.is_contiguous() or bias.dtype not in _DT):
        raise ValueError(f"bias must be a contiguous [{D}] tensor")
    (q, k, v), hd, (sh, sd) = _qkv_views(z_pre, D, layout, num_heads, flip)
    m = _lib.ModalParams(log_poles=_ptr(log_poles), theta=_ptr(theta), res_re=_ptr(residues), res_im=_ptr(res_im), G=G, S=S)
    p = _lib.IirParams(
        q=_ptr(q), q_stride_b=z_pre.stride(0), q_stride_h=sh, q_stride_d=sd,
        k=_ptr(k), k_stride_b=z_pre.stride(0), k_stride_h=sh, k_stride_d=sd,
        v=_ptr(v), v_stride_b=z_pre.stride(0), v_stride_h=sh, v_stride_d=sd, head_dim=hd, modal=m,
        bias=_ptr(bias), bias_dtype=_code(bias) if bias is not None else 0,
        y=_ptr(y), y_stride_b=D * L, y_stride_d=L, y_stride_l=1, state=_ptr(state), scratch=None,
        B=B, L=L, D=D, round_kv=int(round_kv), io_dtype=_code(z_pre))
    with _on(z_pre):
        _lib.check(_lib.lib().vtx_iir_fwd_noalloc(C.byref(p), _stream(z_pre)))
