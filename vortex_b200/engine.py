"""Drop-in ``HyenaInferenceEngine`` backed by the sm_100a kernels.

Same constructor, method names, argument meaning, return conventions and cache side effects as
the reference class (``vortex/model/engine.py:112-559``), so ``HyenaCascade`` can hold this engine
unchanged (``vortex/model/model.py:155-160``).  Every method launches hand-written CUDA kernels
through the C ABI; tensors that are not on a CUDA device are rejected.

On top of the drop-in surface the engine offers the fused entry points the reference's model
code looks for but never defines (``vortex/model/layers.py:18-21``): see ``fused_prefill`` /
``fused_decode`` here and ``vortex_b200.hyena_ops``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import ops
from ._lib import BIAS_ADD, BIAS_GATED, BIAS_NONE, TAPS_CONV, TAPS_XCORR

# vortex/model/engine.py:15-22
IIR_PREFILL_MODES = [
    "recurrence",
    "modal-fft",
    "hybrid-modal-recurrence",
    "modal-scan",
    "canonical-fft",
    "iir-fir-caching",
]


def _layout(column_split_hyena: bool) -> str:
    # The caller has already applied `interleave` (model.py:251-252), so at this boundary the packed
    # tensor is either [q | k | v] thirds or per-head column-split (engine.py:153-156).
    return "column_split" if column_split_hyena else "split"


class HyenaInferenceEngine:
    def __init__(
        self,
        fir_fn=None,
        iir_prefill_style="modal-fft",
        layer_idx=None,
        ground_truth_activations_path=None,
        print_activations=False,
        hyena_flip_x1x2=False,
    ) -> None:
        self.fir_fn = fir_fn
        assert iir_prefill_style in IIR_PREFILL_MODES, f"iir_prefill_style must be one of {IIR_PREFILL_MODES}"
        self.iir_prefill_style = iir_prefill_style
        self.layer_idx = layer_idx
        self.low_mem_mode = False
        self.ground_truth_activations_path = ground_truth_activations_path
        self.print_activations = print_activations
        self.hyena_flip_x1x2 = hyena_flip_x1x2
        self._grouped = {}       # (storage pointer, version, shape, groups) -> bool: see _group_filters

    def _group_filters(self, weight, hidden_size, groups):
        """The caller expands grouped filters to one row per channel before the call (``repeat_interleave``,
        model.py:261-262) and passes ``groups`` along, which the reference ignores.  The kernels want the filters
        un-expanded -- the tensor-core path shares one Toeplitz operand among the channels of a group -- so when
        ``groups`` says the rows repeat in blocks, and they do (checked once per weight tensor and version: one
        device-to-host read, cached), every block is handed over as one row."""
        if (groups is None or weight.dim() != 3 or weight.shape[0] != hidden_size or not 0 < groups < hidden_size
                or hidden_size % groups):
            return weight
        key = (weight.data_ptr(), weight._version, tuple(weight.shape), int(groups))
        ok = self._grouped.get(key)
        if ok is None:
            blocks = weight.detach().reshape(groups, hidden_size // groups, -1)
            ok = bool((blocks == blocks[:, :1]).all().item())
            if len(self._grouped) > 64:
                self._grouped.clear()
            self._grouped[key] = ok
        return weight[:: hidden_size // groups] if ok else weight

    # ------------------------------------------------------------------ prefill: FIR paths
    def parallel_fir(
        self,
        fir_fn,
        u,
        weight,
        bias,
        L,
        dims,
        groups=None,
        gated_bias=False,
        column_split_hyena=False,
        dim_last=True,
        fir_length=3,
        gate=False,
        inference_params=None,
        prefill_mode=None,
        padding_mask=None,
    ):
        """engine.py:131-260.  ``gate=False``: featurizer, returns z [B, C, L].  ``gate=True``: split
        q/k/v, k*v, grouped FIR (cross-correlation below 128 taps, convolution + skip term from 128
        taps on), q gate; returns y [B, D, L].  Second return value is the FIR cache (the last
        ``fir_length - 1`` filter inputs) or None when ``inference_params`` is None.  As in the
        reference, ``L``, ``groups`` and ``prefill_mode`` are accepted and not used."""
        if fir_fn is not None and fir_fn is not F.conv1d:
            raise NotImplementedError("custom fir_fn callables (the reference's deprecated path) are not supported")
        want_state = inference_params is not None
        if not gate:
            if fir_length >= 128:
                raise NotImplementedError("ungated filters of 128 taps and more are not a path the model takes")
            u_blc = u if dim_last else u.permute(0, 2, 1)
            return ops.featurizer_fwd(u_blc, weight, bias, padding_mask, want_state=want_state)

        hidden_size, num_heads, _head, _, _ = dims
        z_pre = u.permute(0, 2, 1) if dim_last else u
        if fir_length >= 128:
            if bias is None:
                raise AttributeError("filters of 128 taps and more need the skip parameter `bias` (engine.py:78)")
            taps, bias_mode = TAPS_CONV, BIAS_GATED
        else:
            taps = TAPS_XCORR
            bias_mode = BIAS_NONE if bias is None else (BIAS_GATED if gated_bias else BIAS_ADD)
        weight = self._group_filters(weight, hidden_size, groups)
        return ops.gcg_fwd(z_pre, weight, bias, hidden_size, taps=taps, bias_mode=bias_mode,
                           layout=_layout(column_split_hyena), num_heads=num_heads, flip=self.hyena_flip_x1x2,
                           mask=padding_mask, want_state=want_state, round_kv=True)

    # ------------------------------------------------------------------ prefill: long (modal) path
    def parallel_iir(
        self,
        z_pre,
        h,
        D,
        L,
        poles,
        residues,
        t,
        dims,
        layer_idx,
        inference_params=None,
        prefill_style="fft",
        fftconv_fn=None,
        padding_mask=None,
        use_flashfft=False,
        column_split_hyena=False,
        long_fir_threshold=None,
    ):
        """engine.py:262-404.  Returns y viewed as [B, L, D]; with ``inference_params`` the state after
        the last token lands in ``inference_params.state_dict[layer_idx]`` (fp32 [B, D, S]).

        The filter is evaluated from its modal form (``poles`` = log-poles [G, S, 1], ``residues``
        [G, S]) as a recurrence, which is the same linear operator as the reference's length-2L FFT
        product with ``h = sum_s R exp(lambda t)`` -- ``h`` itself is only read on the
        ``long_fir_threshold`` path, where the reference truncates it to an explicit FIR."""
        hidden_size, num_heads, _head, state_size, _groups = dims
        layout = _layout(column_split_hyena)
        want_state = inference_params is not None
        if use_flashfft:
            raise NotImplementedError("use_flashfft needs the external flashfftconv package; not part of this engine")

        if want_state and prefill_style == "recurrence":
            # legacy complex-pole form (engine.py:473-504): poles/residues [D, S, 1, 2] as (re, im);
            # the output keeps sum_s R_re * Re(sigma_s) and the state is [B, D, S, 2]
            # the kernel follows the reference's loop step for step (update order, state in the I/O dtype)
            y, state = ops.iir_recurrence_fwd(z_pre, poles[:, :, 0], residues[:, :, 0], D, hidden_size, layout=layout,
                                              num_heads=num_heads, flip=self.hyena_flip_x1x2)
            inference_params.state_dict[self.layer_idx] = state
            return y.permute(0, 2, 1)

        if long_fir_threshold is not None:
            assert h.shape[0] == 1, "batch size must be 1 for long_fir_threshold"
            # [D, 1, thr] in the I/O dtype, applied as F.conv1d applies it (engine.py:341-349)
            hk = h[0][:, None][..., :long_fir_threshold].to(z_pre.dtype)
            y, _ = ops.gcg_fwd(z_pre, hk, D, hidden_size, taps=TAPS_XCORR, bias_mode=BIAS_GATED, layout=layout,
                               num_heads=num_heads, flip=self.hyena_flip_x1x2, want_state=False, round_kv=True)
            state = None
            if want_state and prefill_style == "fft":
                _, state = ops.iir_fwd(z_pre, poles, residues, None, hidden_size, layout=layout, num_heads=num_heads,
                                       flip=self.hyena_flip_x1x2, want_state=True)
        else:
            if poles is None or residues is None:
                raise NotImplementedError("parallel_iir evaluates the modal form and needs `poles` and `residues`")
            y, state = ops.iir_fwd(z_pre, poles, residues, D, hidden_size, layout=layout, num_heads=num_heads,
                                   flip=self.hyena_flip_x1x2, want_state=want_state and prefill_style == "fft")

        if want_state:
            if prefill_style == "fft":
                inference_params.state_dict[layer_idx] = state
            elif prefill_style != "recurrence":
                raise NotImplementedError
        return y.permute(0, 2, 1)

    # ------------------------------------------------------------------ decode
    def step_fir(self, u, fir_state, weight, bias=None, gated_bias=False, flip_filter=False):
        """engine.py:406-449.  Returns (y in u's dtype, new fp32 cache).  The cache grows by one sample
        while it is shorter than K-1 and is shifted afterwards, exactly as the reference's."""
        return ops.step_fir(u, fir_state, weight, bias=bias, gated_bias=gated_bias, flip_filter=flip_filter)

    def step_iir(self, x2, x1, v, D, residues, poles, iir_state, iir_groups=1):
        """engine.py:451-467.  ``poles`` holds log-poles [D, S, 1]; returns (y fp32, new state)."""
        if iir_groups > 1:
            raise NotImplementedError
        return ops.step_iir(x2, x1, v, D, residues, poles, iir_state)

    # ------------------------------------------------------------------ unimplemented in the reference too
    def prefill_via_fir_caching(self, u, inference_params, L, *args, **kwargs):
        raise NotImplementedError(":)")

    def prefill_via_hybrid_recurrence(self, inference_params, u, log_poles, x1v_f_a, L, *args, **kwargs):
        raise NotImplementedError(":)")

    def prefill_via_scan(self, u, inference_params=None, *args, **kwargs):
        raise NotImplementedError

    def prefill_via_canonical_fft(self, u, inference_params=None, *args, **kwargs):
        raise NotImplementedError(":)")

    # ------------------------------------------------------------------ fused fast paths (opt-in)
    def fused_prefill(self, u, short_filter_weight, short_filter_bias, dims, *, h=None, D=None, log_poles=None,
                      residues=None, layout="interleaved", inference_params=None):
        """Whole ``HyenaCascade.parallel_forward`` (model.py:221-316) on the projection output
        u [B, L, 3D] in one pass: returns y [B, L, D] and fills the caches of ``self.layer_idx``.
        ``layout`` is the layout of the packed channels BEFORE the caller's ``interleave``:
        "interleaved" for ``config.interleave`` models, "split", or "column_split"."""
        from . import hyena_ops

        hidden_size, num_heads = dims[0], dims[1]
        want = inference_params is not None
        if h is not None:
            K = h.shape[-1]
            y, fs, ist = ops.fused_fir_fwd(u, short_filter_weight, short_filter_bias, h, D, hidden_size,
                                           taps=TAPS_CONV if K >= 128 else TAPS_XCORR,
                                           bias_mode=BIAS_GATED if (K >= 128 and D is not None) else BIAS_NONE,
                                           layout=layout, num_heads=num_heads, flip=self.hyena_flip_x1x2,
                                           want_state=want)
            if want:
                inference_params.fir_state_dict[self.layer_idx] = fs
                inference_params.fir_inner_state_dict[self.layer_idx] = ist
            return y
        y, fs, st = hyena_ops.hyena_li_fwd(u, short_filter_weight, short_filter_bias, log_poles, residues, D,
                                           layout=layout, num_heads=num_heads, flip=self.hyena_flip_x1x2,
                                           want_state=want)
        if want:
            inference_params.fir_state_dict[self.layer_idx] = fs
            inference_params.state_dict[self.layer_idx] = st
        return y

    def fused_decode(self, u, short_filter_weight, short_filter_bias, dims, inference_params, *, h=None, D=None,
                     log_poles=None, residues=None, layout="interleaved"):
        """Whole ``HyenaCascade.sequential_forward`` (model.py:318-375) for one token in one launch:
        u [B, 3D] -> y [B, D]; the caches of ``self.layer_idx`` are replaced by the new ones."""
        hidden_size, num_heads = dims[0], dims[1]
        i = self.layer_idx
        if h is not None:
            K = h.shape[-1]
            y, fs, ist = ops.decode_layer(u, short_filter_weight, short_filter_bias, inference_params.fir_state_dict[i],
                                          hidden_size, h=h, inner_state=inference_params.fir_inner_state_dict[i],
                                          bias=D if K >= 128 else None, flip_filter=K >= 128, gated_bias=K >= 128,
                                          layout=layout, num_heads=num_heads, flip=self.hyena_flip_x1x2)
            inference_params.fir_inner_state_dict[i] = ist
        else:
            y, fs, st = ops.decode_layer(u, short_filter_weight, short_filter_bias, inference_params.fir_state_dict[i],
                                         hidden_size, log_poles=log_poles, residues=residues, bias=D,
                                         iir_state=inference_params.state_dict[i], layout=layout, num_heads=num_heads,
                                         flip=self.hyena_flip_x1x2)
            inference_params.state_dict[i] = st
        inference_params.fir_state_dict[i] = fs
        return y
