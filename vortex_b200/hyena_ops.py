"""The ``hyena_ops`` surface: fused forward entry points and the (x, B, C, h) convention.

``hyena_se_fwd`` / ``hyena_mr_fwd`` / ``hyena_li_fwd`` are the names the reference's model code
tries to import (``vortex/model/layers.py:18-21``) without ever defining them; here they take the
projection output ``u [B, L, 3D]`` (channel-last, before the featurizer) and run the whole Hyena
block.  ``gcg_fwd`` follows the reference's gate-conv-gate convention
(``vortex/ops/hyena_se/fwd.py:56-64``, math in ``vortex/ops/hyena_se/ref_fwd.py:80-127``):
``y = C * xcorr(h_g, B * x)`` on ``(bs, l, g, dg)`` tensors with blocked filter sharing.
"""
from __future__ import annotations

import torch

from . import ops
from ._lib import BIAS_ADD, BIAS_GATED, BIAS_NONE, TAPS_CONV, TAPS_XCORR


def _general_fir_block(u, w3, b3, h, D_skip, taps, bias_mode, layout, num_heads, flip, want_state):
    """Any filter length / dtype: featurizer kernel (channel-last -> channel-first) followed by the
    general gate-FIR-gate kernel writing channel-last.  Two launches, z materialised once."""
    D = u.shape[-1] // 3
    z, fs = ops.featurizer_fwd(u, w3, b3, None, want_state=want_state)
    y, st = ops.gcg_fwd(z, h, D_skip, D, taps=taps, bias_mode=bias_mode, layout=layout, num_heads=num_heads,
                        flip=flip, want_state=want_state, round_kv=True, channel_last_out=True)
    return y, fs, st


def _fused_ok(u, h, layout, num_heads):
    """Shapes the single-pass CUDA-core kernel takes (see vtx_fused_fir_fwd in include/vortex_b200.h)."""
    D = u.shape[-1] // 3
    es = u.element_size()
    if h.shape[-1] > 16 or D % 2 or (u.stride(1) * es) % 16 or u.stride(2) != 1 or u.data_ptr() % 16:
        return False
    if layout != "interleaved" and (D * es) % 16:
        return False
    if layout == "column_split" and (D // num_heads) % 64:
        return False
    return True


def _tensor_core_ok(u, b3, h, layout, num_heads):
    """Shapes the tcgen05 blocked-Toeplitz kernel takes: bf16 I/O, up to 128 taps, groups of 16 channels."""
    D = u.shape[-1] // 3
    if u.dtype != torch.bfloat16 or b3 is not None or h.shape[-1] > 128 or h.shape[0] * 16 != D:
        return False
    if (u.stride(1) * 2) % 16 or u.stride(2) != 1 or u.data_ptr() % 16 or (u.stride(0) * 2) % 16:
        return False
    if layout == "column_split" and (D // num_heads) % 16:
        return False
    return True


def _fir_block(u, w3, b3, h, D_skip, taps, bias_mode, layout, num_heads, flip, want_state, hist_rows=0):
    """Kernel choice per workload: tcgen05 blocked-Toeplitz kernel for bf16 I/O with groups of 16 channels and up
    to 128 taps, single-pass CUDA-core kernel for other dtypes / group sizes up to 16 taps, two-launch general path
    otherwise (the choice between the first two is made inside vtx_fused_fir_fwd)."""
    D = u.shape[-1] // 3
    if _fused_ok(u, h, layout, num_heads) or _tensor_core_ok(u, b3, h, layout, num_heads):
        return ops.fused_fir_fwd(u, w3, b3, h, D_skip, D, taps=taps, bias_mode=bias_mode, layout=layout,
                                 num_heads=num_heads, flip=flip, want_state=want_state, hist_rows=hist_rows)
    if hist_rows:
        raise NotImplementedError("chunked prefill (hist_rows) needs a shape the single-pass kernels take")
    return _general_fir_block(u, w3, b3, h, D_skip, taps, bias_mode, layout, num_heads, flip, want_state)


def hyena_se_fwd(u, short_filter_weight, short_filter_bias, h, *, layout="interleaved", num_heads=1, flip=False,
                 want_state=False, hist_rows=0):
    """Hyena-SE block (inner filter shorter than 128 taps, cross-correlation taps, no skip term).
    u [B, L, 3D] -> y [B, L, D] (+ featurizer cache [B, 3D, 2], inner cache [B, D, K-1]).
    ``hist_rows``: see PrefillChunks (the rows before ``u`` in memory are the sequence's earlier rows)."""
    return _fir_block(u, short_filter_weight, short_filter_bias, h, None, TAPS_XCORR, BIAS_NONE, layout, num_heads,
                      flip, want_state, hist_rows)


def hyena_mr_fwd(u, short_filter_weight, short_filter_bias, h, D_skip, *, layout="interleaved", num_heads=1,
                 flip=False, want_state=False, hist_rows=0):
    """Hyena-MR block (128-tap grouped filter, convolution taps, per-channel skip term D_skip)."""
    return _fir_block(u, short_filter_weight, short_filter_bias, h, D_skip, TAPS_CONV, BIAS_GATED, layout, num_heads,
                      flip, want_state, hist_rows)


class PrefillChunks:
    """Staging buffer for prefilling a long prompt in chunks through the FIR blocks (what the reference does token
    by token when it forces a prompt, generation.py:94-101).

    The projection GEMM of a chunk writes its [B, Lc, 3D] output into ``rows(Lc)``; the ``hist`` rows in front of
    it hold the end of the previous chunk, so that ``hyena_se_fwd / hyena_mr_fwd(..., hist_rows=chunks.hist_rows)``
    see the samples their first outputs reach back to.  ``advance(Lc)`` then moves the last ``hist`` rows to the
    front for the next chunk (a copy of hist x 3D elements per sequence).  ``hist`` must be at least K + 1 for the
    longest FIR filter that reads the buffer (130 for the 128-tap filter)."""

    def __init__(self, B, max_chunk, D3, hist, *, device, dtype):
        self.hist, self.max_chunk = int(hist), int(max_chunk)
        self.buf = torch.zeros(B, self.hist + self.max_chunk, D3, device=device, dtype=dtype)
        self.seen = 0            # samples of the sequence consumed so far

    @property
    def hist_rows(self):
        """What to pass as ``hist_rows``: 0 for the first chunk (nothing precedes it), ``hist`` afterwards."""
        return self.hist if self.seen > 0 else 0

    def rows(self, Lc):
        if Lc > self.max_chunk:
            raise ValueError(f"chunk of {Lc} rows > max_chunk {self.max_chunk}")
        return self.buf[:, self.hist:self.hist + Lc]

    def advance(self, Lc):
        # the last `hist` rows seen so far (of this chunk and, for a short chunk, of the history before it)
        tail = self.buf[:, Lc:Lc + self.hist].clone()
        self.buf[:, :self.hist] = tail
        self.seen += Lc


LI_STEP = 384      # rows per step of the tensor-core long-filter kernel (4 chunks of 96)


def hyena_li_fwd(u, short_filter_weight, short_filter_bias, log_poles, residues, D_skip, *, theta=None, res_im=None,
                 layout="interleaved", num_heads=1, flip=False, want_state=False, state_in=None, fir_state_in=None,
                 hist_rows=0):
    """Hyena-LI block (modal long filter).  u [B, L, 3D] -> y [B, L, D], featurizer cache, modal state
    fp32 [B, D, S] (complex poles: [B, D, S, 2]).  ``state_in`` / ``fir_state_in``: the caches a call on the
    preceding chunk of the same sequences returned (chunked prefill).  ``hist_rows`` (see PrefillChunks) replaces
    ``fir_state_in`` when the rows before ``u`` in memory are the sequence's earlier rows; chunks of a multiple of
    384 rows then run on the tensor-core kernel."""
    D = u.shape[-1] // 3
    L = u.shape[1]
    if (state_in is not None and hist_rows and L > LI_STEP and L % LI_STEP and
            _li_tensor_core_ok(u, short_filter_weight, short_filter_bias, residues, layout, num_heads)):
        # a continued call on the tensor-core kernel must be a multiple of its 384-row step (its walk is aligned to
        # the end of the rows and a carried-in state must not decay over padding): the first L % 384 rows go through
        # the recurrence kernel, the rest start from the state it leaves; both write into one output
        r = L % LI_STEP
        kw = dict(layout=layout, num_heads=num_heads, flip=flip, theta=theta, res_im=res_im, b3=short_filter_bias)
        y = torch.empty(u.shape[0], L, D, device=u.device, dtype=u.dtype)
        _, st = ops.fused_iir_fwd(u[:, :r], short_filter_weight, log_poles, residues, D_skip, D, want_state=True,
                                  state_in=state_in, hist_rows=hist_rows, out=y[:, :r], **kw)
        res = ops.fused_iir_fwd(u[:, r:], short_filter_weight, log_poles, residues, D_skip, D, want_state=want_state,
                                state_in=st, hist_rows=hist_rows + r, out=y[:, r:], **kw)
        if not want_state:
            return y, None, None
        return y, u[:, L - 2:].transpose(1, 2).contiguous(), res[1]
    if short_filter_weight.shape[-1] == 3 and residues.shape[-1] <= 16:
        # one pass over the rows; the library routes per-group-of-16 bf16 systems to the tensor-core kernel
        out = ops.fused_iir_fwd(u, short_filter_weight, log_poles, residues, D_skip, D, layout=layout, num_heads=num_heads,
                                flip=flip, theta=theta, res_im=res_im, want_state=want_state, b3=short_filter_bias,
                                state_in=state_in, fir_state_in=fir_state_in, hist_rows=hist_rows)
        if not want_state:
            return out, None, None
        if hist_rows:
            ext = u.as_strided((u.shape[0], u.shape[1] + 2, u.shape[2]), u.stride(), u.storage_offset() - 2 * u.stride(1))
            return out[0], ext[:, -2:].transpose(1, 2).contiguous(), out[1]
        # featurizer cache: the last two input rows, channel-first (a strided copy, no arithmetic)
        L = u.shape[1]
        fs = u[:, max(L - 2, 0):, :].transpose(1, 2)
        if L < 2 and fir_state_in is not None:
            fs = torch.cat([fir_state_in[..., L:].to(u.dtype), fs], dim=-1)
        return out[0], fs.contiguous(), out[1]
    if state_in is not None or fir_state_in is not None or hist_rows:
        raise NotImplementedError("chunked prefill needs a 3-tap featurizer and at most 16 poles")
    z, fs = ops.featurizer_fwd(u, short_filter_weight, short_filter_bias, None, want_state=want_state)
    y, st = ops.iir_fwd(z, log_poles, residues, D_skip, D, layout=layout, num_heads=num_heads, flip=flip, theta=theta,
                        res_im=res_im, want_state=want_state, round_kv=True)
    return y.permute(0, 2, 1), fs, st


def _li_tensor_core_ok(u, w3, b3, residues, layout, num_heads):
    """Shapes the tcgen05 chunked-scan kernel takes (the library checks the same): bf16 I/O, 3-tap featurizer without
    bias, one modal system of up to 16 poles per group of 16 channels."""
    D = u.shape[-1] // 3
    if u.dtype != torch.bfloat16 or b3 is not None or w3.shape[-1] != 3:
        return False
    if residues.shape[0] * 16 != D or residues.shape[-1] > 16:
        return False
    if (u.stride(1) * 2) % 16 or u.stride(2) != 1 or u.data_ptr() % 16 or (u.stride(0) * 2) % 16:
        return False
    if layout == "column_split" and (D // num_heads) % 16:
        return False
    return True


def gcg_fwd(x, B, C, h, bias=None, gated_bias=False):
    """y = C * xcorr(h_g, B * x) for (bs, l, g, dg) tensors, h (g, 1, hl); returns (bs, l, g, dg)."""
    bs, l, g, dg = x.shape
    mode = BIAS_NONE if bias is None else (BIAS_GATED if gated_bias else BIAS_ADD)
    if x.is_contiguous() and B.is_contiguous() and C.is_contiguous():
        # (bs, l, g, dg) contiguous IS channel-last [bs, l, d]: bf16 operands go to the tensor-core kernel as they are
        q3, k3, v3 = (t.view(bs, l, g * dg) for t in (C, B, x))
        if ops.gcg_cl_ok(q3, k3, v3, h, mode):
            y, _ = ops.gcg_cl_fwd(q3, k3, v3, h, bias, taps=TAPS_XCORR, bias_mode=mode)
            return y.view(bs, l, g, dg)
    to_bdl = lambda t: t.reshape(bs, l, g * dg).permute(0, 2, 1).contiguous()  # noqa: E731
    y, _ = ops.gcg_fwd_bdl(to_bdl(C), to_bdl(B), to_bdl(x), h, bias, taps=TAPS_XCORR,
                           bias_mode=BIAS_NONE if bias is None else (BIAS_GATED if gated_bias else BIAS_ADD),
                           round_kv=True)
    return y.permute(0, 2, 1).reshape(bs, l, g, dg)


def hyena_se_bdl(x, k, q, h, bias=None, gated_bias=False):
    """The 'bdl' form of the reference's ``inner_hyena_se_ref`` (``vortex/ops/hyena_se/interface.py:342-397``):
    y = q * causal_conv(h, k * x) with (b, d, l) operands and h (g, 1, hl)."""
    y, _ = ops.gcg_fwd_bdl(q, k, x, h, bias, taps=TAPS_XCORR,
                           bias_mode=BIAS_NONE if bias is None else (BIAS_GATED if gated_bias else BIAS_ADD),
                           round_kv=True)
    return y


def _to_bdl(t, layout, G):
    """One operand in 'bdl' (b, d, l), 'blgdg' (b, l, g, dg) or 'bgdgl' (b, g, dg, l) layout -> (b, d, l); channels of
    a group are consecutive in d (vortex/ops/hyena_se/interface.py:272-319 reshape_inputs)."""
    if layout == "bdl":
        return t
    if layout == "blgdg":
        b, l, g, dg = t.shape
        if g != G:
            raise ValueError("number of groups in feature groups and filter must match")
        return t.reshape(b, l, g * dg).transpose(1, 2)
    if layout == "bgdgl":
        b, g, dg, l = t.shape
        if g != G:
            raise ValueError("number of groups in feature groups and filter must match")
        return t.reshape(b, g * dg, l)
    raise NotImplementedError("input_layout must be bdl, blgdg or bgdgl")


def inner_hyena_se(x, k, q, h, bias=None, input_layout="bdl", output_layout="bdl", inner_layout="blgdg",
                   apply_gated_bias=False, **kernel_options):
    """``inner_hyena_se`` of the reference's hyena_ops interface (``vortex/ops/hyena_se/interface.py:400-443``; math
    ``inner_hyena_se_ref``, ``:342-397``): y = q * causal_conv(h, k * x) with h (g, 1, hl) shared by the dg consecutive
    channels of a group.  ``input_layout``: 'bdl', 'blgdg' or 'bgdgl'; ``output_layout``: 'bdl', 'bld', 'blgdg' or
    'bgdgl'.  The reference's scheduling arguments (schedule, autotune, fwd_kernel_cfg, bwd_kernel_cfg,
    use_fast_causal_conv1d, kernel_path) are accepted and ignored: there is one kernel, and ``inner_layout`` does not
    change the result."""
    if h.dim() == 2:
        h = h.unsqueeze(1)
    G = h.shape[0]
    if not (x.shape == k.shape == q.shape):
        raise ValueError("feature groups must have the same shape")
    xb, kb, qb = (_to_bdl(t, input_layout, G) for t in (x, k, q))
    y = hyena_se_bdl(xb, kb, qb, h, bias, apply_gated_bias)             # (b, d, l)
    b, d, l = y.shape
    if output_layout == "bdl":
        return y
    if output_layout == "bld":
        return y.transpose(1, 2)
    if output_layout == "blgdg":
        return y.transpose(1, 2).reshape(b, l, G, d // G)
    if output_layout == "bgdgl":
        return y.reshape(b, G, d // G, l)
    raise NotImplementedError("output_layout must be bdl, bld, blgdg or bgdgl")


def gcg_bwd(dy, x, B, C, h, y2=None):
    """Gradients of ``gcg_fwd``: (dx, dB, dC, dh) for (bs, l, g, dg) tensors and h (g, 1, hl) -- the reference's
    ``two_pass_bwd_grouped`` (``vortex/ops/hyena_se/bwd.py:11``; math ``ref_bwd.py:31-115``).  ``y2`` is the filter
    output xcorr(h_g, B * x) the reference's forward saves; without it, it is recomputed by one more forward pass."""
    bs, l, g, dg = x.shape
    if y2 is None:
        y2 = gcg_fwd(x, B, torch.ones_like(C), h)
    f = lambda t: t.reshape(bs, l, g * dg)  # noqa: E731
    dx, dB, dC, dh = ops.gcg_bwd(f(dy), f(x), f(B), f(C), f(y2), h)
    return dx.view(bs, l, g, dg), dB.view(bs, l, g, dg), dC.view(bs, l, g, dg), dh.view(g, 1, -1).to(h.dtype)


def two_pass_bwd_grouped(dy, x, B, C, h, y2, **kernel_options):
    """The reference's backward entry point by name (``vortex/ops/hyena_se/bwd.py:11-60``): (dx, dB, dC, dh).  The
    saved Toeplitz matrices, the lagged product and the scheduling arguments are accepted and ignored."""
    return gcg_bwd(dy, x, B, C, h, y2)


class TwoPassChunkedGateConvGate(torch.autograd.Function):
    """y = C * xcorr(h_g, B * x) with its backward (``vortex/ops/hyena_se/interface.py:47-167``): the forward keeps
    the filter output y2, the backward is ``gcg_bwd``."""

    @staticmethod
    def forward(ctx, x, B, C, h):
        y2 = gcg_fwd(x, B, torch.ones_like(C), h)
        ctx.save_for_backward(x, B, C, h, y2)
        return C * y2

    @staticmethod
    def backward(ctx, dy):
        x, B, C, h, y2 = ctx.saved_tensors
        return gcg_bwd(dy.contiguous(), x, B, C, h, y2)


def two_pass_chunked_gate_conv_gate(x, B, C, h, return_toeplitz=False, **kernel_options):
    """The reference's ``two_pass_chunked_gate_conv_gate`` (``vortex/ops/hyena_se/interface.py:170-204``; kernel
    ``two_pass_fwd_grouped``, ``fwd.py:17``): y = C * xcorr(h_g, B * x) on (bs, l, g, dg) tensors, differentiable in
    x, B, C and h.  The chunking and autotuning arguments are accepted and ignored; no Toeplitz matrices are returned
    (the backward here does not use them)."""
    if return_toeplitz:
        raise NotImplementedError("Toeplitz matrices are not materialised: the backward does not use them")
    if torch.is_grad_enabled() and any(t.requires_grad for t in (x, B, C, h)):
        return TwoPassChunkedGateConvGate.apply(x, B, C, h)
    return gcg_fwd(x, B, C, h)


def hyena_x_bdl_fwd(q, k, v, h):
    """Hyena-X forward with the reference's name and (b, d, l) operands
    (``vortex/ops/hyena_x/triton_indirect_fwd.py:262``; math ``hyena_x_fwd_ref``, ``:413-424``)."""
    return ops.hyena_x_fwd(q, k, v, h)


def hyena_x_fwd(qkv, h):
    """The packed form of the reference's ``hyena_x_fwd_ref``: qkv [B, 3D, L] -> [B, D, L]."""
    D = qkv.shape[1] // 3
    return ops.hyena_x_fwd(qkv[:, :D], qkv[:, D:2 * D], qkv[:, 2 * D:], h)


def causal_conv1d_fn(x, weight, bias=None, seq_idx=None, initial_states=None, final_states_out=None, activation=None):
    """``causal_conv1d_fn`` of the reference's conv package
    (``vortex/ops/conv/local_causal_conv1d/causal_conv1d_interface.py:84-112``; math ``causal_conv1d_ref``, ``:187-222``):
    x (b, d, l), weight (d, hl), bias (d,), seq_idx (b, l), initial_states / final_states_out (b, d, hl - 1) -> (b, d, l)."""
    return ops.causal_conv1d_fwd(x, weight, bias, seq_idx, initial_states, final_states_out, activation)


def causal_conv1d_update(x, conv_state, weight, bias=None, activation=None, cache_seqlens=None,
                         conv_state_indices=None):
    """``causal_conv1d_update`` of the same package (``causal_conv1d_interface.py:225-252``): one or a few new samples
    against a cached window; conv_state is updated in place."""
    return ops.causal_conv1d_update(x, conv_state, weight, bias, activation, cache_seqlens, conv_state_indices)


def causal_conv1d_varlen_states(x, cu_seqlens, state_len):
    """``causal_conv1d_varlen_states`` (``vortex/ops/conv/local_causal_conv1d/causal_conv1d_varlen.py:42-75``):
    x (total_tokens, dim), cu_seqlens (batch + 1) int32 -> states (batch, dim, state_len)."""
    return ops.causal_conv1d_varlen_states(x, cu_seqlens, state_len)
