"""vortex_b200: B200-native (sm_100a) kernels for the Hyena convolution path of vortex.

``HyenaInferenceEngine`` is a drop-in for ``vortex.model.engine.HyenaInferenceEngine``;
``hyena_ops`` holds the fused block entry points; ``cache`` the inference-cache containers.
The kernels live in ``lib/libvortex_b200.so`` (build: ``python -m vortex_b200.build``) and are
reached through the C ABI declared in ``include/vortex_b200.h``.
"""
from .cache import HyenaCascadeFIRInferenceParams, HyenaCascadeIIRInferenceParams, InferenceParams  # noqa: F401
from .engine import IIR_PREFILL_MODES, HyenaInferenceEngine  # noqa: F401

__all__ = ["HyenaInferenceEngine", "IIR_PREFILL_MODES", "InferenceParams", "HyenaCascadeIIRInferenceParams",
           "HyenaCascadeFIRInferenceParams"]
