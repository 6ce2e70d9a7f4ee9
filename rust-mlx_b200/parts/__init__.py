from .base import (BuildContext, CacheSpec, FeedForward, LayerCall, Mixer, Norm, ParamSpec, Part,
                   PositionEncoding)

__all__ = ["BuildContext", "CacheSpec", "FeedForward", "LayerCall", "Mixer", "Norm", "ParamSpec", "Part",
           "PositionEncoding"]
