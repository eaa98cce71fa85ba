"""numpy restatement of the reference Hyena convolution path (TEST INFRASTRUCTURE).

Every function cites the reference lines (paths relative to the reference
project root) whose behaviour it restates.  Arithmetic is float64 with the
reference's rounding points made explicit:

* ``mirror=True``  -- round wherever the reference materialises a tensor in the
  I/O dtype (this is "the reference's own path" for that dtype);
* ``mirror=False`` -- the "fp32 reference": inputs are the I/O-dtype values,
  all intermediate math is kept wide, nothing is rounded on the way out.

Arrays are plain ``numpy.ndarray``; values of a narrow dtype are carried in
float64 containers that hold exactly representable numbers.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this module.
"""
from __future__ import annotations

import numpy as np

IO_DTYPES = ("f32", "bf16", "f16")


# --------------------------------------------------------------------------
# rounding helpers
# --------------------------------------------------------------------------
def bf16_bits(x32: np.ndarray) -> np.ndarray:
    """float32 array -> uint16 bf16 bit patterns, round-to-nearest-even."""
    x32 = np.ascontiguousarray(x32, dtype=np.float32)
    b = x32.view(np.uint32).astype(np.uint64)
    r = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    nan = np.isnan(x32)
    r = np.where(nan, 0x7FC0, r)
    return r.astype(np.uint16)


def bf16_from_bits(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def round_io(x: np.ndarray, io: str) -> np.ndarray:
    """Round to the I/O dtype (through float32 first, as the reference's fp32
    math followed by ``.to(dtype)`` does) and return float64."""
    x32 = np.asarray(x, dtype=np.float64).astype(np.float32)
    if io == "f32":
        return x32.astype(np.float64)
    if io == "bf16":
        return bf16_from_bits(bf16_bits(x32)).astype(np.float64)
    if io == "f16":
        return x32.astype(np.float16).astype(np.float64)
    raise ValueError(f"io dtype {io!r}")


def _maybe(x, io, mirror):
    return round_io(x, io) if mirror else np.asarray(x, dtype=np.float64)


def rel_l2(a, b) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = float(np.sqrt((b * b).sum()))
    num = float(np.sqrt(((a - b) ** 2).sum()))
    return num / den if den > 0 else num


# --------------------------------------------------------------------------
# q / k / v channel maps
# --------------------------------------------------------------------------
def qkv_index(D: int, layout: str, num_heads: int = 1, flip_x1x2: bool = False):
    """Packed-channel indices (into the 3D featurizer channels) of q (=x2),
    k (=x1), v for every hidden channel d.

    'split'        : engine.py:156   (u.split([D, D, D], dim=1))
    'interleaved'  : utils.py:26-38 followed by engine.py:156
    'column_split' : utils.py:41-85  (per head: [q_h | k_h | v_h])
    flip_x1x2      : engine.py:157-158
    """
    d = np.arange(D)
    if layout == "split":
        q, k, v = d, D + d, 2 * D + d
    elif layout == "interleaved":
        q, k, v = 3 * d, 3 * d + 1, 3 * d + 2
    elif layout == "column_split":
        hd = D // num_heads
        n, j = d // hd, d % hd
        q, k, v = n * 3 * hd + j, n * 3 * hd + hd + j, n * 3 * hd + 2 * hd + j
    else:
        raise ValueError(layout)
    if flip_x1x2:
        q, k = k, q
    return q, k, v


def select_qkv(z, D, layout="split", num_heads=1, flip_x1x2=False):
    """z [B, 3D, L] or [B, 3D] -> (q, k, v) each [B, D, ...]."""
    qi, ki, vi = qkv_index(D, layout, num_heads, flip_x1x2)
    return z[:, qi], z[:, ki], z[:, vi]


def expand_groups(h, D):
    """[G, 1, K] / [G, K] -> [D, K], blocked sharing (model.py:261-262,
    hyena_se/ref_fwd.py:112-113: repeat_interleave)."""
    h = np.asarray(h, dtype=np.float64)
    if h.ndim == 3:
        h = h[:, 0, :]
    G = h.shape[0]
    assert D % G == 0
    return np.repeat(h, D // G, axis=0)


# --------------------------------------------------------------------------
# causal FIR, both tap conventions
# --------------------------------------------------------------------------
def causal_fir(x, h, convention):
    """x [B, C, L], h [C, K] (already per channel).

    'xcorr': y[t] = sum_j h[j] x[t-(K-1)+j]  (F.conv1d with padding K-1,
             engine.py:197-204 -- the LAST tap meets the current sample)
    'conv' : y[t] = sum_j h[j] x[t-j]        (FFT product, engine.py:53-73 --
             the FIRST tap meets the current sample; taps beyond L are cut,
             engine.py:178)
    """
    x = np.asarray(x, dtype=np.float64)
    h = np.asarray(h, dtype=np.float64)
    B, C, L = x.shape
    K = h.shape[-1]
    y = np.zeros_like(x)
    for j in range(K):
        lag = (K - 1 - j) if convention == "xcorr" else j
        if lag >= L:
            continue
        y[:, :, lag:] += h[None, :, j, None] * x[:, :, : L - lag]
    return y


# --------------------------------------------------------------------------
# prefill operators
# --------------------------------------------------------------------------
def featurizer(u_blc, w, bias=None, io="f32", padding_mask=None, mirror=True):
    """engine.parallel_fir(gate=False, dim_last=True)  (engine.py:149,188-227,
    255-260; caller model.py:233-249).

    u_blc [B, L, C] -> z [B, C, L], fir_state [B, C, min(L, K-1)] (a copy of
    the pre-convolution input, packed channel order).
    """
    u = round_io(u_blc, io).transpose(0, 2, 1)  # B, C, L
    w = np.asarray(w, dtype=np.float64)
    if w.ndim == 3:
        w = w[:, 0, :]
    K = w.shape[-1]
    z = _maybe(causal_fir(u, w, "xcorr"), io, mirror)
    if bias is not None:
        z = _maybe(z + np.asarray(bias, dtype=np.float64)[None, :, None], io, mirror)
    if padding_mask is not None:
        z = _maybe(z * np.asarray(padding_mask, dtype=np.float64)[:, None, :], io, mirror)
    state = u[..., -(K - 1):] if K > 1 else u[..., :0]
    return z, np.ascontiguousarray(state)


def gate_conv_gate(z_pre, h, bias, D, fir_length, io="f32", layout="split",
                   num_heads=1, flip_x1x2=False, gated_bias=False,
                   padding_mask=None, mirror=True, round_input=True):
    """engine.parallel_fir(gate=True, dim_last=False)  (engine.py:150-159,
    174-232, 255-258; caller model.py:271-291).

    z_pre [B, 3D, L]; h [G,1,K] or [D,1,K]; returns y [B, D, L] and the inner
    state kv[..., -(K-1):] (engine.py:256).  K < 128 is the cross-correlation
    path; K >= 128 the FFT/convolution path, where `bias` is the per-channel
    skip and is always applied as bias * kv (engine.py:78).
    round_input=False keeps z_pre wide (used when the featurizer output is an
    intermediate of a fused evaluation rather than a materialised tensor).
    """
    z = round_io(z_pre, io) if round_input else np.asarray(z_pre, dtype=np.float64)
    q, k, v = select_qkv(z, D, layout, num_heads, flip_x1x2)
    kv = _maybe(k * v, io, mirror)
    hd = expand_groups(h, D)
    K = fir_length
    L = z.shape[-1]
    if K >= 128:
        conv = causal_fir(kv, hd[:, :L], "conv")
        conv = conv + kv * np.asarray(bias, dtype=np.float64)[None, :, None]
        zc = _maybe(conv, io, mirror)
    else:
        zc = _maybe(causal_fir(kv, hd, "xcorr"), io, mirror)
        if bias is not None:
            b = np.asarray(bias, dtype=np.float64)[None, :, None]
            if gated_bias:
                zc = _maybe(zc + _maybe(b * kv, io, mirror), io, mirror)
            else:
                zc = _maybe(zc + b, io, mirror)
    if padding_mask is not None:
        zc = _maybe(zc * np.asarray(padding_mask, dtype=np.float64)[:, None, :], io, mirror)
    y = _maybe(q * zc, io, mirror)
    state = kv[..., -(K - 1):]
    if not mirror:
        state = round_io(state, io)
    return y, np.ascontiguousarray(state)


def hyena_x(qkv, h, io="f32", mirror=True):
    """Hyena-X forward (vortex/ops/hyena_x/triton_indirect_fwd.py:413-424): depthwise causal FIR
    (cross-correlation taps, F.conv1d with padding L_h - 1 cut to L) on each of the 3D packed channels,
    then o = z_q * z_k * z_v.  qkv [B, 3D, L], h [3D, 1, L_h] or [3D, L_h] -> [B, D, L].
    mirror=True rounds where the reference's bf16 tensors round (conv output, first product, result)."""
    x = round_io(qkv, io)
    w = round_io(np.asarray(h, dtype=np.float64), io)
    if w.ndim == 3:
        w = w[:, 0, :]
    z = _maybe(causal_fir(x, w, "xcorr"), io, mirror)
    D = z.shape[1] // 3
    q, k, v = z[:, :D], z[:, D:2 * D], z[:, 2 * D:]
    return _maybe(_maybe(q * k, io, mirror) * v, io, mirror)


def causal_conv1d(x, weight, bias=None, initial_states=None, seq_idx=None, silu=False, io="f32", mirror=False):
    """Short depthwise causal convolution of the reference's conv extension
    (vortex/ops/conv/local_causal_conv1d/causal_conv1d_interface.py:187-222 causal_conv1d_ref; kernel
    csrc/causal_conv1d_fwd.cu:300-330 for seq_idx):
    out[b,d,t] = bias[d] + sum_w weight[d,w] * xx[b,d,t-(W-1)+w], xx = [initial_states | x] (zeros without initial
    states); with seq_idx a tap counts only if its position lies in this call (t' >= 0) and seq_idx[b,t'] ==
    seq_idx[b,t]; optional SiLU; result rounded to the I/O dtype.  Also returns the final states: the last W-1
    samples of xx.  x [B,D,L], weight [D,W] -> ([B,D,L], [B,D,W-1]).
    mirror=True rounds the convolution result to the I/O dtype before the SiLU, as the PyTorch reference function
    does (its conv1d returns the narrow dtype); the CUDA kernel keeps fp32 up to the final cast (mirror=False)."""
    x = round_io(x, io)
    w = np.asarray(weight, dtype=np.float64)
    B, D, L = x.shape
    W = w.shape[1]
    ini = np.zeros((B, D, W - 1)) if initial_states is None else round_io(initial_states, io)
    xx = np.concatenate([ini, x], axis=-1)
    out = np.zeros((B, D, L))
    if bias is not None:
        out += np.asarray(bias, dtype=np.float64)[None, :, None]
    for j in range(W):
        term = w[None, :, j, None] * xx[..., j:j + L]                    # position t - (W-1) + j
        if seq_idx is not None:
            sid = np.asarray(seq_idx)
            pos = np.arange(L) - (W - 1) + j
            same = np.zeros((B, L), dtype=bool)
            ok = pos >= 0
            same[:, ok] = sid[:, pos[ok]] == sid[:, ok]
            term = term * same[:, None, :]
        out += term
    if mirror:
        out = round_io(out, io)
    if silu:
        out = out / (1.0 + np.exp(-out))
    return round_io(out, io), xx[..., xx.shape[-1] - (W - 1):]


def causal_conv1d_update(x, conv_state, weight, bias=None, silu=False, cache_seqlens=None, io="f32"):
    """Decode-time update of the same convolution (causal_conv1d_interface.py:250-282, kernel
    csrc/causal_conv1d_update.cu): x [B,D,Lq] new samples, conv_state [B,D,state_len] (state_len >= W-1).
    Without cache_seqlens the state is a shift register (new state = last state_len samples of [state | x]); with it
    a circular buffer: the W-1 samples before position cache_seqlens[b] are read, x is written at positions
    cache_seqlens[b] + i (mod state_len).  Returns (out [B,D,Lq], new conv_state)."""
    x = round_io(x, io)
    st = np.array(round_io(conv_state, io))
    w = np.asarray(weight, dtype=np.float64)
    B, D, Lq = x.shape
    W, SL = w.shape[1], st.shape[-1]
    if cache_seqlens is None:
        xn = np.concatenate([st, x], axis=-1)
        new = xn[..., -SL:]
    else:
        cs = np.asarray(cache_seqlens).astype(np.int64)
        widx = (np.arange(-(W - 1), 0)[None, :] + cs[:, None]) % SL                       # [B, W-1]
        hist = np.take_along_axis(st, np.broadcast_to(widx[:, None, :], (B, D, W - 1)), axis=2)
        xn = np.concatenate([hist, x], axis=-1)
        new = st.copy()
        cidx = (np.arange(Lq)[None, :] + cs[:, None]) % SL
        np.put_along_axis(new, np.broadcast_to(cidx[:, None, :], (B, D, Lq)), x, axis=2)
    n = xn.shape[-1]
    out = np.zeros((B, D, Lq))
    if bias is not None:
        out += np.asarray(bias, dtype=np.float64)[None, :, None]
    for j in range(W):
        out += w[None, :, j, None] * xn[..., n - Lq - (W - 1) + j:n - (W - 1) + j]
    if silu:
        out = out / (1.0 + np.exp(-out))
    return round_io(out, io), new


def causal_conv1d_varlen_states(x, cu_seqlens, state_len):
    """causal_conv1d_varlen_states_ref (vortex/ops/conv/local_causal_conv1d/causal_conv1d_varlen.py:78-97): x [total, dim]
    holds packed sequences, cu_seqlens [batch+1] their boundaries -> states [batch, dim, state_len] = the last
    min(state_len, length) rows of each sequence, right-aligned, zeros before.  A pure copy."""
    x = np.asarray(x)
    cu = np.asarray(cu_seqlens).astype(np.int64)
    batch, dim = len(cu) - 1, x.shape[1]
    st = np.zeros((batch, dim, state_len), dtype=x.dtype)
    for i in range(batch):
        end = cu[i + 1]
        start = max(cu[i], end - state_len)
        if end > start:
            st[i, :, state_len - (end - start):] = x[start:end].T
    return st


def modal_filter(log_poles, residues, L):
    """HyenaCascade.compute_filter (model.py:390-398): real modal form,
    h[g, t] = sum_s R[g, s] * exp(lambda[g, s] * t), float32 arithmetic.
    log_poles [G, S, 1] (or [G, S]), residues [G, S] -> [G, L] float32."""
    lp = np.asarray(log_poles, dtype=np.float32).reshape(np.shape(residues))
    R = np.asarray(residues, dtype=np.float32)
    t = np.arange(L, dtype=np.float32)
    return (R[..., None] * np.exp(lp[..., None] * t)).sum(1, dtype=np.float32)


def modal_filter_complex(poles, residues, L):
    """Legacy complex modal form (model.py:842-848): h[g,t] = sum_s Re(R p^t).
    poles, residues complex [G, S] -> [G, L] float64."""
    p = np.asarray(poles, dtype=np.complex128)
    R = np.asarray(residues, dtype=np.complex128)
    t = np.arange(L, dtype=np.float64)
    mag = np.abs(p)[..., None] ** t
    ang = np.angle(p)[..., None] * t
    return (R[..., None] * (mag * np.exp(1j * ang))).real.sum(1)


def _fft_causal_conv(x, h):
    """FFT product of length 2L (engine.py:331-337), float64."""
    L = x.shape[-1]
    n = 2 * L
    X = np.fft.rfft(x, n=n, axis=-1)
    H = np.fft.rfft(h, n=n, axis=-1)
    return np.fft.irfft(X * H, n=n, axis=-1)[..., :L]


def long_conv_gate(z_pre, h, bias, D, io="f32", layout="split", num_heads=1,
                   flip_x1x2=False, mirror=True, round_input=True):
    """engine.parallel_iir, default FFT branch (engine.py:282-353,404).

    z_pre [B, 3D, L], h [D, L] per channel -> y [B, L, D] and kv [B, D, L]
    (the pre-gated signal the state is computed from).  round_input=False keeps
    the featurizer output unrounded (a fused kernel never materialises it)."""
    z = round_io(z_pre, io) if round_input else np.asarray(z_pre, dtype=np.float64)
    q, k, v = select_qkv(z, D, layout, num_heads, flip_x1x2)
    kv = _maybe(k * v, io, mirror)
    h = np.asarray(h, dtype=np.float64)
    if h.ndim == 3:
        h = h[0]
    y = _maybe(_fft_causal_conv(kv, h[None]), io, mirror)
    b = np.asarray(bias, dtype=np.float64)[None, :, None]
    y = _maybe(y + _maybe(kv * b, io, mirror), io, mirror)
    y = _maybe(y * q, io, mirror)
    return y.transpose(0, 2, 1), kv


def long_fir_gate(z_pre, h, bias, D, threshold, io="f32", layout="split", num_heads=1, flip_x1x2=False):
    """engine.parallel_iir with ``long_fir_threshold`` (engine.py:339-353): the long filter cut to its first
    ``threshold`` samples, rounded to the I/O dtype and handed to F.conv1d -- so it is applied as a
    cross-correlation (the LAST kept sample of h meets the current input), whatever its length.  Then the skip
    term and the gate as in the FFT branch.  z_pre [B, 3D, L], h [D, L] per channel -> y [B, L, D]."""
    z = round_io(z_pre, io)
    q, k, v = select_qkv(z, D, layout, num_heads, flip_x1x2)
    kv = round_io(k * v, io)
    h = np.asarray(h, dtype=np.float64)
    if h.ndim == 3:
        h = h[0]
    hk = round_io(h[:, :threshold], io)
    y = round_io(causal_fir(kv, hk, "xcorr"), io)
    b = np.asarray(bias, dtype=np.float64)[None, :, None]
    y = round_io(y + round_io(kv * b, io), io)
    y = round_io(y * q, io)
    return y.transpose(0, 2, 1)


def recurrence_prefill(z_pre, poles_ri, residues_ri, bias, D, io="f32", layout="split", num_heads=1,
                       flip_x1x2=False):
    """engine.parallel_iir with prefill_style="recurrence" -> prefill_via_direct_recurrence (engine.py:314-321,
    473-504), then the skip term and the gate (engine.py:351-353).

    poles_ri, residues_ri [D, S, 2] as (re, im).  The loop is the reference's: the state lives in the I/O dtype
    (it is built from x1*v), its real part is updated in place and the imaginary part then reads the NEW real
    part (engine.py:497-498); every product, difference and sum is a float32 operation of its own; the output
    keeps sum_s Re(R_s) * Re(state_s).  Returns y [B, L, D] and the state [B, D, S, 2] float32."""
    f32 = np.float32
    z = round_io(z_pre, io)
    q, k, v = select_qkv(z, D, layout, num_heads, flip_x1x2)
    x = round_io(k * v, io).astype(f32)                                   # x1v [B, D, L]
    pr, pi = (np.asarray(poles_ri, dtype=f32)[None, ..., j] for j in (0, 1))      # [1, D, S]
    rr = np.asarray(residues_ri, dtype=f32)[None, ..., 0]
    B, _, L = x.shape
    re = np.zeros((B, D, pr.shape[-1]), dtype=f32)
    im = np.zeros_like(re)
    rnd = lambda a: round_io(a, io).astype(f32)  # noqa: E731
    out = np.zeros((B, D, L), dtype=f32)
    for i in range(L):
        re = rnd((pr * re - pi * im) + x[:, :, i, None])
        im = rnd(pr * im + pi * re)
        acc = np.zeros((B, D), dtype=f32)
        for s in range(re.shape[-1]):
            acc = acc + rr[..., s] * re[..., s]
        out[:, :, i] = rnd(acc)
    b = np.asarray(bias, dtype=np.float64)[None, :, None]
    y = round_io(out.astype(np.float64) + round_io(x.astype(np.float64) * b, io), io)
    y = round_io(y * q, io)
    return y.transpose(0, 2, 1), np.stack([re, im], axis=-1)


def modal_state(kv, log_poles_d):
    """IIR state after prefill: what prefill_via_modal_fft extracts at index
    L-1 (engine.py:552-559): state[b,d,s] = sum_j exp(lambda[d,s]*(L-1-j)) kv[b,d,j].
    kv [B, D, L]; log_poles_d [D, S] (per channel) -> [B, D, S] float64."""
    kv = np.asarray(kv, dtype=np.float64)
    lp = np.asarray(log_poles_d, dtype=np.float64).reshape(kv.shape[1], -1)
    L = kv.shape[-1]
    w = np.exp(lp[:, :, None] * (L - 1 - np.arange(L, dtype=np.float64)))  # D,S,L
    return np.einsum("bdl,dsl->bds", kv, w)


def modal_state_complex(kv, poles_d):
    """Complex-pole variant: state[b,d,s] = sum_j p^(L-1-j) kv[j] (complex)."""
    kv = np.asarray(kv, dtype=np.float64)
    p = np.asarray(poles_d, dtype=np.complex128)
    L = kv.shape[-1]
    e = (L - 1 - np.arange(L, dtype=np.float64))
    w = (np.abs(p)[..., None] ** e) * np.exp(1j * np.angle(p)[..., None] * e)
    return np.einsum("bdl,dsl->bds", kv.astype(np.complex128), w)


# --------------------------------------------------------------------------
# decode operators
# --------------------------------------------------------------------------
def step_fir(u, fir_state, weight, bias=None, gated_bias=False, flip_filter=False,
             io="f32"):
    """engine.step_fir (engine.py:406-449).

    u [B, C]; fir_state [B, C, c] (oldest first); weight [C,1,K] or [C,K].
    Returns y [B, C] rounded to the I/O dtype and the new state (float32
    values, engine.py:430,444-449).  While c < K-1 the state grows by one and
    the non-flipped path uses taps [:c+1] (engine.py:424-425)."""
    w = np.asarray(weight, dtype=np.float64)
    if w.ndim == 3:
        w = w[:, 0, :]
    K = w.shape[-1]
    st = np.asarray(fir_state, dtype=np.float64)
    c = st.shape[-1]
    if flip_filter:
        wf = w[:, ::-1][:, K - c - 1:] if c + 1 <= K else w[:, ::-1]
    else:
        wf = w[:, : c + 1]
    u = np.asarray(u, dtype=np.float64)
    h0, hh = wf[:, -1], wf[:, :-1]
    y = h0[None] * u + (st * hh[None]).sum(-1)
    if bias is not None:
        b = np.asarray(bias, dtype=np.float64)[None]
        y = y + (b * u if gated_bias else b)
    if c < K - 1:
        new_state = np.concatenate([st, u[..., None]], axis=-1)
    else:
        new_state = np.concatenate([st[..., 1:], u[..., None]], axis=-1)
    return round_io(y, io), new_state.astype(np.float32)


def step_iir(x2, x1, v, D, residues, log_poles, iir_state):
    """engine.step_iir (engine.py:451-467): real modal recurrence, fp32."""
    x1v = np.asarray(x1, dtype=np.float64) * np.asarray(v, dtype=np.float64)
    R = np.asarray(residues, dtype=np.float64)
    p = np.exp(np.asarray(log_poles, dtype=np.float64).reshape(R.shape))
    st = p[None] * np.asarray(iir_state, dtype=np.float64) + x1v[..., None]
    res = (R[None] * st).sum(-1)
    y = np.asarray(x2, dtype=np.float64) * (res + np.asarray(D, dtype=np.float64)[None] * x1v)
    return y, st


def step_iir_complex(x2, x1, v, D, residues, poles, state):
    """Complex-pole decode step matching modal_filter_complex:
    sigma <- p*sigma + kv ; y = q * (sum_s Re(R sigma) + D kv)."""
    x1v = np.asarray(x1, dtype=np.float64) * np.asarray(v, dtype=np.float64)
    p = np.asarray(poles, dtype=np.complex128)
    R = np.asarray(residues, dtype=np.complex128)
    st = p[None] * np.asarray(state, dtype=np.complex128) + x1v[..., None]
    res = (R[None] * st).real.sum(-1)
    y = np.asarray(x2, dtype=np.float64) * (res + np.asarray(D, dtype=np.float64)[None] * x1v)
    return y, st


# --------------------------------------------------------------------------
# hyena_ops (bs, l, g, dg) convention
# --------------------------------------------------------------------------
def gcg_blgdg(x, Bg, Cg, h):
    """hyena_se/ref_fwd.py:80-127 (gcg_fwd_ref_corrected): y = C * xcorr(h_g, B*x)
    with tensors (bs, l, g, dg), h (g, 1, hl), blocked filter sharing."""
    x = np.asarray(x, dtype=np.float64)
    bs, l, g, dg = x.shape
    Bx = (np.asarray(Bg, dtype=np.float64) * x).reshape(bs, l, g * dg).transpose(0, 2, 1)
    y = causal_fir(Bx, expand_groups(h, g * dg), "xcorr")
    return np.asarray(Cg, dtype=np.float64) * y.transpose(0, 2, 1).reshape(bs, l, g, dg)


def gcg_blgdg_bwd(dy, x, Bg, Cg, h):
    """hyena_se/ref_bwd.py:31-115 (gcg_two_pass_chunked_bwd), un-chunked: gradients of y = C * xcorr(h_g, B*x) with
    tensors (bs, l, g, dg), h (g, 1, hl).  Returns dx, dB, dC (bs, l, g, dg) and dh (g, 1, hl).
    With z = B*x and y2[t] = sum_k h[k] z[t-(hl-1)+k]:  dC = dy*y2;  dz[t] = sum_k h[k] (dy*C)[t+(hl-1)-k];
    dx = dz*B;  dB = dz*x;  dh[k] = sum_{b,t,dg} (dy*C)[t] z[t-(hl-1)+k]."""
    dy, x, Bg, Cg = (np.asarray(t, dtype=np.float64) for t in (dy, x, Bg, Cg))
    h = np.asarray(h, dtype=np.float64)
    bs, l, g, dg = x.shape
    hl = h.shape[-1]
    z = Bg * x
    y2 = gcg_blgdg(x, Bg, np.ones_like(Cg), h)
    g2 = dy * Cg
    dz = np.zeros_like(z)
    dh = np.zeros((g, 1, hl))
    for k in range(hl):
        s = hl - 1 - k                      # y2[t] takes h[k] z[t - s]
        if s >= l:
            continue
        hk = h[:, 0, k][None, None, :, None]
        dz[:, :l - s] += hk * g2[:, s:]
        dh[:, 0, k] = np.einsum("blgd,blgd->g", g2[:, s:], z[:, :l - s])
    return dz * Bg, dz * x, dy * y2, dh


def toeplitz_pair(hf, size):
    """hyena_se/utils.py:5-51: T[i,j] = hf[i-j] (0 <= i-j < hl) and the
    correction T_hat[i,j] = hf[i+size-j] (j >= i, i+size-j < hl), hf = h.flip."""
    hf = np.asarray(hf, dtype=np.float64)
    hl = hf.shape[-1]
    i = np.arange(size)[:, None]
    j = np.arange(size)[None, :]
    d = i - j
    T = np.where((d >= 0) & (d < hl), hf[np.clip(d, 0, hl - 1)], 0.0)
    e = i + size - j
    Th = np.where((j >= i) & (e < hl), hf[np.clip(e, 0, hl - 1)], 0.0)
    return T, Th


def hyena_fused(u_blc, w3, h, bias, D, fir_length, io="f32", layout="interleaved",
                num_heads=1, flip_x1x2=False, mirror=True):
    """Featurizer followed by gate-conv-gate on the channel-last projection
    output (model.py:233-291 end to end).  Returns y [B, L, D], featurizer
    state [B, 3D, 2], inner state [B, D, K-1]."""
    z, st0 = featurizer(u_blc, w3, None, io, None, mirror)
    y, st1 = gate_conv_gate(z, h, bias, D, fir_length, io, layout, num_heads,
                            flip_x1x2, gated_bias=fir_length >= 128, mirror=mirror,
                            round_input=mirror)
    return y.transpose(0, 2, 1), st0, st1
