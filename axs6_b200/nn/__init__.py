"""V1 (uniform grid) functional surface: mirror of ``axs.nn`` for the accelerated path."""
from .functional import fake_quantize

__all__ = ["fake_quantize"]
