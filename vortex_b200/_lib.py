"""ctypes binding of ``libvortex_b200.so`` (the C ABI declared in ``include/vortex_b200.h``).

There is no fallback: if the library is missing, or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libvortex_b200.so")

F32, BF16, F16 = 0, 1, 2
QKV_SPLIT, QKV_INTERLEAVED, QKV_COLUMN_SPLIT = 0, 1, 2
TAPS_XCORR, TAPS_CONV = 0, 1
BIAS_NONE, BIAS_ADD, BIAS_GATED = 0, 1, 2

_p, _i = C.c_void_p, C.c_int64


def header_abi_version() -> int:
    """VTX_ABI_VERSION of include/vortex_b200.h (major * 1000 + minor): the one place the number is written."""
    import re
    path = os.path.join(os.path.dirname(PKG), "include", "vortex_b200.h")
    with open(path) as f:
        m = re.search(r"#define\s+VTX_ABI_VERSION\s+(\d+)", f.read())
    if not m:
        raise RuntimeError(f"{path} does not define VTX_ABI_VERSION")
    return int(m.group(1))


def _struct(name, spec):
    """spec: 'ptr:a i:b ...' -> ctypes.Structure subclass with 8-byte fields only."""
    fields = []
    for item in spec.split():
        kind, fname = item.split(":")
        fields.append((fname, _p if kind == "p" else _i))
    return type(name, (C.Structure,), {"_fields_": fields})


FeaturizerParams = _struct("FeaturizerParams", """
    p:u i:u_stride_b i:u_stride_l i:u_stride_c p:w i:w_dtype p:bias i:bias_dtype p:mask i:mask_dtype
    p:z p:state i:B i:L i:C i:K i:io_dtype""")

GcgParams = _struct("GcgParams", """
    p:q i:q_stride_b i:q_stride_h i:q_stride_d p:k i:k_stride_b i:k_stride_h i:k_stride_d
    p:v i:v_stride_b i:v_stride_h i:v_stride_d i:head_dim
    p:h i:h_dtype p:bias i:bias_dtype p:mask i:mask_dtype
    p:y i:y_stride_b i:y_stride_d i:y_stride_l p:state
    i:B i:L i:D i:G i:K i:taps i:bias_mode i:round_kv i:io_dtype""")

FusedFirParams = _struct("FusedFirParams", """
    p:u i:u_stride_b i:u_stride_l p:w3 i:w3_dtype p:b3 i:b3_dtype p:h i:h_dtype p:bias i:bias_dtype
    p:y i:y_stride_b i:y_stride_l p:fir_state p:inner_state
    i:B i:L i:D i:G i:K3 i:K i:layout i:num_heads i:flip_x1x2 i:taps i:bias_mode i:io_dtype i:u_hist_rows""")

GcgClParams = _struct("GcgClParams", """
    p:q i:q_stride_b i:q_stride_l p:k i:k_stride_b i:k_stride_l p:v i:v_stride_b i:v_stride_l
    p:h i:h_dtype p:bias i:bias_dtype p:y i:y_stride_b i:y_stride_l p:state
    i:B i:L i:D i:G i:K i:taps i:bias_mode i:io_dtype""")

GcgBwdParams = _struct("GcgBwdParams", """
    p:dy i:dy_stride_b i:dy_stride_l p:x i:x_stride_b i:x_stride_l p:Bg i:b_stride_b i:b_stride_l
    p:C i:c_stride_b i:c_stride_l p:y2 i:y2_stride_b i:y2_stride_l p:h i:h_dtype p:dx p:dB p:dC p:dh32
    i:B i:L i:D i:G i:K i:io_dtype""")

ModalParams = _struct("ModalParams", "p:log_poles p:theta p:res_re p:res_im i:G i:S")


HyenaXParams = _struct("HyenaXParams", "p:q p:k p:v p:h i:h_dtype p:y i:B i:D i:L i:Lh i:io_dtype")


CausalConv1dParams = _struct("CausalConv1dParams", """
    p:x i:x_stride_b i:x_stride_d i:x_stride_l p:weight i:weight_dtype p:bias i:bias_dtype p:seq_idx
    p:initial_states i:is_stride_b i:is_stride_d i:is_stride_l p:final_states i:fs_stride_b i:fs_stride_d i:fs_stride_l
    p:out i:out_stride_b i:out_stride_d i:out_stride_l i:B i:D i:L i:W i:silu i:io_dtype""")

CausalConv1dUpdateParams = _struct("CausalConv1dUpdateParams", """
    p:x i:x_stride_b i:x_stride_d i:x_stride_l p:conv_state i:cs_stride_b i:cs_stride_d i:cs_stride_l i:state_len
    p:weight i:weight_dtype p:bias i:bias_dtype p:cache_seqlens p:conv_state_indices
    p:out i:out_stride_b i:out_stride_d i:out_stride_l i:B i:D i:L i:W i:silu i:io_dtype""")


VarlenStatesParams = _struct("VarlenStatesParams", """
    p:x i:x_stride_t i:x_stride_c p:cu_seqlens p:states i:st_stride_b i:st_stride_c i:st_stride_l
    i:total i:batch i:dim i:state_len i:io_dtype""")


class FusedIirParams(C.Structure):
    _fields_ = [("u", _p), ("u_stride_b", _i), ("u_stride_l", _i), ("w3", _p), ("w3_dtype", _i),
                ("b3", _p), ("b3_dtype", _i), ("modal", ModalParams), ("bias", _p), ("bias_dtype", _i),
                ("y", _p), ("y_stride_b", _i), ("y_stride_l", _i), ("state", _p), ("scratch", _p),
                ("B", _i), ("L", _i), ("D", _i), ("K3", _i), ("layout", _i), ("num_heads", _i), ("flip_x1x2", _i),
                ("io_dtype", _i), ("state_in", _p), ("fir_state_in", _p), ("fir_state_dtype", _i),
                ("u_hist_rows", _i)]


class IirParams(C.Structure):
    _fields_ = [("q", _p), ("q_stride_b", _i), ("q_stride_h", _i), ("q_stride_d", _i),
                ("k", _p), ("k_stride_b", _i), ("k_stride_h", _i), ("k_stride_d", _i),
                ("v", _p), ("v_stride_b", _i), ("v_stride_h", _i), ("v_stride_d", _i),
                ("head_dim", _i), ("modal", ModalParams), ("bias", _p), ("bias_dtype", _i),
                ("y", _p), ("y_stride_b", _i), ("y_stride_d", _i), ("y_stride_l", _i),
                ("state", _p), ("scratch", _p), ("B", _i), ("L", _i), ("D", _i),
                ("round_kv", _i), ("io_dtype", _i)]


StepFirParams = _struct("StepFirParams", """
    p:u p:state_in i:state_dtype p:w i:w_dtype p:bias i:bias_dtype p:y p:state_out
    i:B i:C i:Gw i:K i:c i:flip_filter i:bias_mode i:io_dtype""")


class StepIirParams(C.Structure):
    _fields_ = [("q", _p), ("k", _p), ("v", _p), ("modal", ModalParams), ("bias", _p), ("bias_dtype", _i),
                ("state_in", _p), ("state_out", _p), ("y", _p), ("B", _i), ("D", _i), ("io_dtype", _i)]


class DecodeLayerParams(C.Structure):
    _fields_ = [("u", _p), ("w3", _p), ("w3_dtype", _i), ("b3", _p), ("b3_dtype", _i),
                ("fir_state_in", _p), ("fir_state_dtype", _i), ("fir_state_out", _p),
                ("h", _p), ("h_dtype", _i), ("inner_state_in", _p), ("inner_state_dtype", _i),
                ("inner_state_out", _p), ("modal", ModalParams), ("iir_state_in", _p), ("iir_state_out", _p),
                ("bias", _p), ("bias_dtype", _i), ("y", _p),
                ("B", _i), ("D", _i), ("G", _i), ("K3", _i), ("K", _i),
                ("layout", _i), ("num_heads", _i), ("flip_x1x2", _i), ("flip_filter", _i), ("bias_mode", _i),
                ("io_dtype", _i)]


STRUCTS = [FeaturizerParams, GcgParams, FusedFirParams, ModalParams, IirParams, StepFirParams, StepIirParams,
           DecodeLayerParams, FusedIirParams, HyenaXParams, CausalConv1dParams, CausalConv1dUpdateParams,
           VarlenStatesParams, GcgClParams, GcgBwdParams]

# name -> (restype, argtypes); every symbol include/vortex_b200.h declares
SYMBOLS = {
    "vtx_last_error": (C.c_size_t, [C.c_char_p, C.c_size_t]),
    "vtx_abi_version": (_i, []),
    "vtx_struct_size": (_i, [_i]),
    "vtx_device_status": (C.c_int, []),
    "vtx_debug_set_flag_poll_limit": (C.c_int, [_i]),
    "vtx_launch_count": (C.c_int64, []),
    "vtx_featurizer_fwd": (C.c_int, [C.POINTER(FeaturizerParams), _p]),
    "vtx_gcg_fwd": (C.c_int, [C.POINTER(GcgParams), _p]),
    "vtx_gcg_cl_fwd": (C.c_int, [C.POINTER(GcgClParams), _p]),
    "vtx_gcg_bwd": (C.c_int, [C.POINTER(GcgBwdParams), _p]),
    "vtx_fused_fir_fwd": (C.c_int, [C.POINTER(FusedFirParams), _p]),
    "vtx_modal_filter": (C.c_int, [C.POINTER(ModalParams), _p, _i, _p]),
    "vtx_iir_scratch_bytes": (_i, [_i, _i, _i, _i, _i]),
    "vtx_iir_fwd": (C.c_int, [C.POINTER(IirParams), _p]),
    "vtx_iir_fwd_noalloc": (C.c_int, [C.POINTER(IirParams), _p]),
    "vtx_iir_recurrence_fwd": (C.c_int, [C.POINTER(IirParams), _p]),
    "vtx_fused_iir_fwd": (C.c_int, [C.POINTER(FusedIirParams), _p]),
    "vtx_fused_iir_scratch_bytes": (_i, [C.POINTER(FusedIirParams)]),
    "vtx_hyena_x_fwd": (C.c_int, [C.POINTER(HyenaXParams), _p]),
    "vtx_causal_conv1d_fwd": (C.c_int, [C.POINTER(CausalConv1dParams), _p]),
    "vtx_causal_conv1d_update": (C.c_int, [C.POINTER(CausalConv1dUpdateParams), _p]),
    "vtx_causal_conv1d_varlen_states": (C.c_int, [C.POINTER(VarlenStatesParams), _p]),
    "vtx_step_fir": (C.c_int, [C.POINTER(StepFirParams), _p]),
    "vtx_step_iir": (C.c_int, [C.POINTER(StepIirParams), _p]),
    "vtx_decode_layer": (C.c_int, [C.POINTER(DecodeLayerParams), _p]),
}

_ERRORS = {-1: ValueError, -2: NotImplementedError, -3: ValueError, -4: RuntimeError, -5: RuntimeError}
_lib = None


def lib() -> C.CDLL:
    """Load the shared library once.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m vortex_b200.build` "
                "(vortex_b200 has no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)  # AttributeError if the library does not export it
            fn.restype, fn.argtypes = res, args
        want, got = header_abi_version(), handle.vtx_abi_version()
        if got // 1000 != want // 1000 or got < want:
            raise RuntimeError(f"libvortex_b200.so has ABI version {got}, include/vortex_b200.h {want}: rebuild it "
                               "with `python -m vortex_b200.build`")
        for i, st in enumerate(STRUCTS):
            if handle.vtx_struct_size(i) != C.sizeof(st):
                raise RuntimeError(f"ABI mismatch for {st.__name__}: C {handle.vtx_struct_size(i)} vs "
                                   f"ctypes {C.sizeof(st)}")
        _lib = handle
    return _lib


def last_error() -> str:
    buf = C.create_string_buffer(512)
    lib().vtx_last_error(buf, 512)
    return buf.value.decode()


def check(rc: int) -> None:
    if rc != 0:
        raise _ERRORS.get(rc, RuntimeError)(f"vortex_b200: {last_error()} (status {rc})")
