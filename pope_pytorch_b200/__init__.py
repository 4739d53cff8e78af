"""B200-native PoPE attention: same public names as the reference package
(PoPE_pytorch/__init__.py:1-11), kernels in libpope_b200.so."""
from .pope import FactoredPolarEmbed, PoPE, PolarEmbedReturn, apply_pope_to_qk
from .pope_nd import AxialPoPE
from .attention import compute_attn_similarity, compute_attn_similarity_non_fused, flash_attn_with_pope
from .kv_cache import PagedKVCache

__all__ = ["PoPE", "AxialPoPE", "PolarEmbedReturn", "FactoredPolarEmbed", "apply_pope_to_qk", "compute_attn_similarity",
           "compute_attn_similarity_non_fused", "flash_attn_with_pope", "PagedKVCache"]
