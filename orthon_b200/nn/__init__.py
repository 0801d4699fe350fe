"""Neural-network modules (reference project: python/orthon/nn/__init__.py)."""
from .module import Module, Parameter  # noqa: F401
from .linear import Linear, FusedLinearReLU  # noqa: F401
from .activations import ReLU, Sigmoid, Tanh, LeakyReLU, GELU  # noqa: F401
from .container import Sequential, Flatten  # noqa: F401
from .conv import Conv2d, MaxPool2d  # noqa: F401
from .dropout import Dropout  # noqa: F401
from .norm import LayerNorm, BatchNorm1d, BatchNorm2d  # noqa: F401
from .embedding import Embedding  # noqa: F401
from .loss import NLLLoss, CrossEntropyLoss  # noqa: F401
from .attention import SelfAttention, MultiHeadSelfAttention  # noqa: F401
from .transformer import TransformerEncoderBlock  # noqa: F401
