"""B200-native NVFP4 mixture-of-experts path of Gemma-4 26B-A4B.

Python mirror of the reference's operator interface for this path
(``gevva::Nvfp4ExpertRunner``, include/gevva/gpu.hpp:217-247, and the inline
router launch ``route_128_top8_kernel``) on top of the C ABI in
``include/gevva_moe.h``.  torch is used for device memory and streams only; all
computation happens in ``libgevva_moe.so``.  There is no CPU fallback: loading
fails loudly when the library has not been built.
"""
from .runtime import (  # noqa: F401
    ExpertWeights,
    GevvaMoeError,
    Nvfp4ExpertRunner,
    library,
    pack_experts,
    route_128_top8,
    route_project,
)

__all__ = [
    "ExpertWeights",
    "GevvaMoeError",
    "Nvfp4ExpertRunner",
    "library",
    "pack_experts",
    "route_128_top8",
    "route_project",
]
