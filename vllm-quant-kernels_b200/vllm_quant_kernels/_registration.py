"""Registration of the quantized lm_head and the fused sampler with vLLM.

Mirrors the reference's src/vllm_quant_kernels/_registration.py: the same six
environment variables, the same truthy set, the same MXFP4 > MXFP8 > FP8 > W8A8
> INT8 priority and the same stderr banners.
"""

import os

_ENV_INT8 = "VLLM_USE_INT8_LMHEAD"
_ENV_W8A8 = "VLLM_USE_W8A8_LMHEAD"
_ENV_FP8 = "VLLM_USE_FP8_LMHEAD"
_ENV_MXFP8 = "VLLM_USE_MXFP8_LMHEAD"
_ENV_MXFP4 = "VLLM_USE_MXFP4_LMHEAD"
_ENV_SAMPLER = "VLLM_USE_FUSED_SAMPLER"

_ALL_ENVS = (_ENV_INT8, _ENV_W8A8, _ENV_FP8, _ENV_MXFP8, _ENV_MXFP4, _ENV_SAMPLER)


def _env_bool(name: str, default: bool = False) -> bool:
    """Truthy values: 1, true, yes, on (case-insensitive).  Reference: _registration.py:15-20."""
    val = os.environ.get(name, "")
    if val == "":
        return default
    return val.lower() in ("1", "true", "yes", "on")


def selected_mode() -> "str | None":
    """lm_head mode chosen by the environment, in priority order
    (reference: _registration.py:57-68), or None."""
    if _env_bool(_ENV_MXFP4):
        return "mxfp4"
    if _env_bool(_ENV_MXFP8):
        return "mxfp8"
    if _env_bool(_ENV_FP8):
        return "fp8"
    if _env_bool(_ENV_W8A8):
        return "w8a8"
    if _env_bool(_ENV_INT8):
        return "int8"
    return None


def _silence_unknown_env_warning() -> None:
    """Whitelist our variables in vllm.envs (reference: _registration.py:23-31)."""
    try:
        import vllm.envs as vllm_envs
        for var in _ALL_ENVS:
            if var not in vllm_envs.environment_variables:
                vllm_envs.environment_variables[var] = (lambda v=var: os.environ.get(v, ""))
    except Exception:
        pass  # non-fatal: this vLLM may not have the dict


def register_all() -> None:
    """Register all OOT replacements if an env var is set (reference: _registration.py:34-81)."""
    import sys
    _silence_unknown_env_warning()

    quant_dtype = selected_mode()
    use_sampler = _env_bool(_ENV_SAMPLER)

    if quant_dtype is None and not use_sampler:
        print(
            f"[vllm-quant-kernels] Plugin loaded but disabled "
            f"(set {_ENV_MXFP4}=1 | {_ENV_MXFP8}=1 | {_ENV_FP8}=1 | {_ENV_W8A8}=1 | "
            f"{_ENV_INT8}=1 to enable quantized LM head, or {_ENV_SAMPLER}=1 to "
            f"enable the fused sampler).",
            file=sys.stderr, flush=True,
        )
        return

    if quant_dtype is not None:
        from ._quant import QuantizedLogitsProcessor  # noqa: F401  (import registers the OOT layer)
        print(
            f"[vllm-quant-kernels] Registered QuantizedLogitsProcessor as OOT "
            f"replacement for LogitsProcessor (dtype={quant_dtype}).",
            file=sys.stderr, flush=True,
        )

    if use_sampler:
        from ._sampler import install_fused_sampler
        install_fused_sampler()
