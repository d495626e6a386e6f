"""Parts a decoder is put together from: mixers, feed-forwards, norms,
position encodings, block arrangements and the model's two ends."""
from . import (attention, block, embedding, feed_forward, latent_attention, norm, parallel, position,  # noqa: F401
               recurrent, short_conv, token_input)  # (register)
from .linear import Linear
from .registry import (CacheView, Prepared, Runtime, StepContext, StepPlan, WeightStore, build_part,
                       register_part, unregister_part)

__all__ = ["Linear", "CacheView", "Prepared", "Runtime", "StepContext", "StepPlan", "WeightStore",
           "build_part", "register_part", "unregister_part"]
