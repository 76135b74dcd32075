from .basic import Embedding, FeedForward, LayerNorm, Linear, RMSNorm, causal_depthwise_conv1d
