"""Layer namespace, same names as the reference's `lf.nn` (lua/luatorch/nn/init.lua:18-45).
Every class is callable as `nn.X(...)` and as `nn.X.new(...)`."""
from .activation import GELU, ReLU, Sigmoid, SiLU, Tanh
from .batchnorm import BatchNorm1d
from .conv2d import Conv2d, to_nchw, to_nhwc
from .dropout import Dropout
from .embedding import Embedding
from .layernorm import LayerNorm
from .linear import Linear
from .loss import CrossEntropyLoss, MAELoss, MSELoss
from .module import Module
from .multihead import FlashMultiHeadAttention, MultiHeadAttention
from .positional import LearnedPE, SinusoidalPE
from .sequential import Sequential
from .transformer import TransformerBlock

__all__ = [
    "Module", "Linear", "Conv2d", "Embedding", "Dropout", "LayerNorm", "BatchNorm1d", "Sequential",
    "MultiHeadAttention", "FlashMultiHeadAttention", "TransformerBlock", "ReLU", "Sigmoid", "Tanh",
    "GELU", "SiLU", "SinusoidalPE", "LearnedPE", "MSELoss", "MAELoss", "CrossEntropyLoss",
    "to_nchw", "to_nhwc",
]
