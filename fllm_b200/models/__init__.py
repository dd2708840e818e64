from .decoder import Decoder, KVCache, StepBatch
from .weights import DecoderWeights, LayerWeights, init_random_weights, make_shard_spec

__all__ = ["Decoder", "KVCache", "StepBatch", "DecoderWeights", "LayerWeights",
           "init_random_weights", "make_shard_spec"]
