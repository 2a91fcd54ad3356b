"""neuralnet.cpp_b200 — B200-native (sm_100a) GPT training step for neuralnet.cpp's engine interface.

The package directory name contains a dot, so it is loaded by path (see `load_package` in
`__graft_entry__.py`); inside, modules use relative imports.
"""
from . import _lib
from ._lib import NnbError, call, lib
from .trainer import (ACT_GELU, ACT_SWIGLU, BF16, FP32, NORM_LAYER, NORM_RMS, POS_ALIBI, POS_LEARNED,
                      POS_ROPE, POS_SINUSOIDAL, AsyncInputPipeline, GptConfig, GptTrainer)

__all__ = ["lib", "call", "NnbError", "GptConfig", "GptTrainer", "AsyncInputPipeline", "ACT_GELU", "ACT_SWIGLU", "NORM_LAYER",
           "NORM_RMS", "POS_LEARNED", "POS_SINUSOIDAL", "POS_ALIBI", "POS_ROPE", "FP32", "BF16"]
