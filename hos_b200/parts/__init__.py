"""The parts a layer is put together from.  Importing this package registers them."""
from . import (attention, block, differential_attention, embedding, feedforward, gated_attention, latent_attention, moe, norm, rope,  # noqa: F401
               state_mixers, wkv)
