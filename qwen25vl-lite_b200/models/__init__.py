"""Model assembly and the architectures this engine knows.  Importing registers them."""

from . import fatilix, labolix, mozutar, qwen2_5_vl, rirulix  # noqa: F401
from .decoder import DecoderModel, StopRuntime  # noqa: F401
