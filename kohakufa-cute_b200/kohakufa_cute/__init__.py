"""B200-native attention behind the ``kohakufa_cute`` Python API.

Public functions and their argument semantics follow the reference package
(src/kohakufa_cute/__init__.py:3-20 of the reference project).  Importing this package does
not load the CUDA library; the first CUDA call does.
"""

from .api import (
    attention,
    automatic_scaled_dot_product_attention,
    neighborhood_attention,
    neighborhood_attention_3d,
    scaled_dot_product_attention,
)

__version__ = "0.1.0"
__all__ = [
    "attention",
    "scaled_dot_product_attention",
    "automatic_scaled_dot_product_attention",
    "neighborhood_attention",
    "neighborhood_attention_3d",
]
