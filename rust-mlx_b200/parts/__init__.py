from .base import (BuildContext, CacheSpec, DecodeShape, FeedForward, LayerCall, Mixer, Norm, ParamSpec, Part,
                   PositionEncoding)

__all__ = ["BuildContext", "CacheSpec", "DecodeShape", "FeedForward", "LayerCall", "Mixer", "Norm", "ParamSpec", "Part",
           "PositionEncoding"]
