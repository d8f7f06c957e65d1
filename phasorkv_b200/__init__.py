"""phasorkv_b200: the PhasorKey decode path (rotated-latent cache write, query absorption, latent
scoring + softmax + V) as hand-written sm_100a CUDA behind the reference's PhasorKey interface."""
from ._lib import PhasorKVError  # noqa: F401
from .latent import PhasorKey, PagedLatentCache, rope_phasors  # noqa: F401
from .patch import PhasorKeyPatch  # noqa: F401

__all__ = ["PhasorKey", "PagedLatentCache", "PhasorKeyPatch", "PhasorKVError", "rope_phasors"]
