"""Quantized lm_head + fused sampler for vLLM on NVIDIA B200 (sm_100a).

Drop-in for the `vllm-quant-kernels` plugin: same package name, same
`vllm.general_plugins` entry point, same environment variables.  The kernels
are hand-written CUDA in libvqk.so, called through a C ABI.
"""

__version__ = "0.1.0"


def register() -> None:
    """Register quantized kernel plugins with vLLM."""
    from ._registration import register_all

    register_all()
