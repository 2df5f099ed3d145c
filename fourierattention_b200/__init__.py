"""B200-native (sm_100a) implementation of the Fourier-compressed KV cache and its fused decode
attention, behind the Python API of FourierAttention's ``fourier_attn_triton`` package.

    from fourierattention_b200 import install_aliases
    install_aliases()        # makes `import cache_utils_fourier`, `import modeling_llama_fourier`,
                             # `import fourier_triton_valid4_v2` (and their `lxr_` twins) resolve here

Importing the package loads ``lib/libfourier_b200.so``; there is no fallback if it is missing.
"""
import sys

from . import _lib, ops  # noqa: F401  (fails loudly when the library has not been built)
from . import cache_utils_fourier, fourier_triton_valid4_v2, modeling_llama_fourier  # noqa: F401
from .cache_utils_fourier import DynamicCache, compress_period  # noqa: F401

__version__ = "0.1.0"

_ALIASES = {
    "cache_utils_fourier": cache_utils_fourier,
    "lxr_cache_utils_fourier": cache_utils_fourier,
    "fourier_triton_valid4_v2": fourier_triton_valid4_v2,
    "lxr_fourier_triton_valid4_v2": fourier_triton_valid4_v2,
    "modeling_llama_fourier": modeling_llama_fourier,
    "lxr_modeling_llama_fourier": modeling_llama_fourier,
}


def install_aliases(overwrite: bool = False):
    """Register the reference's module names in ``sys.modules`` so that existing imports keep working."""
    for name, mod in _ALIASES.items():
        if overwrite or name not in sys.modules:
            sys.modules[name] = mod
