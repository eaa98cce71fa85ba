"""CPU checks of the C ABI: the library loads, exports every declared symbol, struct mirrors agree,
and argument validation reports errors instead of launching."""
import ctypes as C
import os
import re

import pytest
import torch

from vortex_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "vortex_b200.h")).read()
    declared = set(re.findall(r"\b(vtx_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    handle = C.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(handle, name), f"{name} is declared in include/vortex_b200.h but not exported"
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)


def test_struct_sizes_match():
    lib = _lib.lib()
    for i, st in enumerate(_lib.STRUCTS):
        assert lib.vtx_struct_size(i) == C.sizeof(st), st.__name__
    assert lib.vtx_struct_size(len(_lib.STRUCTS)) == -1
    assert lib.vtx_abi_version() == _lib.header_abi_version() >= 1002


def test_bad_arguments_are_reported_not_launched():
    lib = _lib.lib()
    p = _lib.GcgParams()          # all null / zero
    rc = lib.vtx_gcg_fwd(C.byref(p), None)
    assert rc == -1 and "null" in _lib.last_error()
    with pytest.raises(ValueError):
        _lib.check(rc)
    f = _lib.FeaturizerParams(u=1, w=1, z=1, B=1, L=4, C=4, K=99)
    assert lib.vtx_featurizer_fwd(C.byref(f), None) == -2
    with pytest.raises(NotImplementedError):
        _lib.check(-2)
    s = _lib.StepFirParams(u=1, w=1, y=1, state_in=1, state_out=1, B=1, C=4, Gw=3, K=3, c=2)
    assert lib.vtx_step_fir(C.byref(s), None) == -1 and "multiple" in _lib.last_error()
    assert lib.vtx_iir_scratch_bytes(1, 131072, 4096, 16, 0) > 0
    assert lib.vtx_iir_scratch_bytes(64, 8192, 4096, 16, 0) == 0


def test_cpu_tensors_are_rejected():
    from vortex_b200 import HyenaInferenceEngine

    eng = HyenaInferenceEngine()
    with pytest.raises(RuntimeError, match="CUDA"):
        eng.step_fir(torch.zeros(2, 4), torch.zeros(2, 4, 2), torch.zeros(4, 1, 3))
    with pytest.raises(RuntimeError, match="CUDA"):
        eng.parallel_fir(torch.nn.functional.conv1d, torch.zeros(1, 8, 12), torch.zeros(12, 1, 3), None, 8,
                         dims=(4, 1, 4, 16, 4))
    with pytest.raises(AssertionError):
        HyenaInferenceEngine(iir_prefill_style="nope")


def test_fused_iir_scratch_plan():
    """Host-side planning of the long-filter kernels (no GPU work).  Tensor-core shapes: no scratch for short walks
    or many walks, a few KB per walk once a launch has too few walks to fill the SMs evenly.  Per-channel systems
    (the recurrence kernel): one state per channel and time segment."""
    from vortex_b200 import _lib
    f = _lib.lib().vtx_fused_iir_scratch_bytes

    def q(B, L, D, G, S=16, cplx=False, io=_lib.BF16):
        p = _lib.FusedIirParams(B=B, L=L, D=D, K3=3, io_dtype=io, y_stride_l=D, y_stride_b=L * D,
                                u_stride_l=3 * D, u_stride_b=3 * D * L)
        p.modal.G, p.modal.S = G, S
        if cplx:
            p.modal.theta = 16       # only tested against NULL
        return f(C.byref(p))

    assert q(1, 1000, 4096, 256) == 0                       # 3 steps: nothing to slice
    assert q(0, 1000, 4096, 256) == 0 and q(1, 0, 4096, 256) == 0
    n = q(1, 131072, 4096, 256)                             # 256 walks on 148 SMs: sliced
    assert n > 0 and n % (32 * 16 * 4 + 4) == 0
    assert q(8, 131072, 4096 * 4, 1024) == 0                # 8192 walks: whole rounds anyway
    n = q(1, 131072, 4096, 4096)                            # a modal system per channel: segments
    assert n > 0 and n % (4096 * 16 * 4) == 0
    assert q(1, 131072, 4096, 4096, cplx=True) == 2 * n
    assert q(1, 40, 4096, 4096) == 0                        # too short to cut


def test_conv_extension_argument_checks():
    """The conv extension's entry points report bad arguments by code before any launch, and the host wrappers
    reject CPU tensors, unknown activations and wrong layouts."""
    from vortex_b200 import hyena_ops
    lib = _lib.lib()
    assert lib.vtx_causal_conv1d_fwd(C.byref(_lib.CausalConv1dParams()), None) == -1
    p = _lib.CausalConv1dParams(x=16, weight=16, out=16, B=1, D=8, L=8, W=5)
    assert lib.vtx_causal_conv1d_fwd(C.byref(p), None) == -2 and "between 2 and 4" in _lib.last_error()
    u = _lib.CausalConv1dUpdateParams(x=16, weight=16, out=16, conv_state=16, B=1, D=8, L=1, W=4, state_len=2)
    assert lib.vtx_causal_conv1d_update(C.byref(u), None) == -1 and "shorter" in _lib.last_error()
    assert lib.vtx_causal_conv1d_varlen_states(C.byref(_lib.VarlenStatesParams()), None) == -1
    x, w = torch.zeros(1, 8, 8), torch.zeros(8, 3)
    with pytest.raises(RuntimeError, match="CUDA"):
        hyena_ops.causal_conv1d_fn(x, w)
    with pytest.raises(RuntimeError, match="CUDA"):
        hyena_ops.causal_conv1d_update(x[..., 0], torch.zeros(1, 8, 2), w)
    with pytest.raises(RuntimeError, match="CUDA"):
        hyena_ops.causal_conv1d_varlen_states(torch.zeros(8, 4), torch.tensor([0, 8], dtype=torch.int32), 2)


def test_interface_layouts_on_cpu():
    """Layout plumbing of inner_hyena_se needs no GPU: every input layout maps to the same (b, d, l) view."""
    from vortex_b200.hyena_ops import _to_bdl
    B, G, dg, L = 2, 3, 4, 5
    x = torch.arange(B * G * dg * L, dtype=torch.float32).reshape(B, G * dg, L)
    assert torch.equal(_to_bdl(x, "bdl", G), x)
    assert torch.equal(_to_bdl(x.transpose(1, 2).reshape(B, L, G, dg), "blgdg", G), x)
    assert torch.equal(_to_bdl(x.reshape(B, G, dg, L), "bgdgl", G), x)
    with pytest.raises(ValueError):
        _to_bdl(x.reshape(B, G, dg, L), "bgdgl", G + 1)
    with pytest.raises(NotImplementedError):
        _to_bdl(x, "lbd", G)


def test_status_codes_map_to_the_reference_exception_types():
    """Bad argument -> ValueError, unsupported -> NotImplementedError, alignment -> ValueError, launch and device
    errors -> RuntimeError (what TORCH_CHECK / assert / NotImplementedError sites of the reference raise)."""
    for rc, exc in ((-1, ValueError), (-2, NotImplementedError), (-3, ValueError), (-4, RuntimeError),
                    (-5, RuntimeError), (-99, RuntimeError)):
        with pytest.raises(exc):
            _lib.check(rc)
    _lib.check(0)
    lib = _lib.lib()
    assert lib.vtx_debug_set_flag_poll_limit(-1) == -1
    assert lib.vtx_debug_set_flag_poll_limit(0) == 0
