"""Module library (reference: rumus/src/nn/)."""
from .modules import (Module, Linear, LayerNorm, RMSNorm, Embedding, Dropout, Flatten,
                      MultiheadAttention, TransformerBlock, scaled_dot_product_attention,
                      use_reference_init, relu, gelu, sigmoid, tanh, leaky_relu, silu, softmax,
                      mse_loss, cross_entropy_loss)
from .vision import (Conv2d, ConvTranspose2d, MaxPool2d, AdaptiveAvgPool2d, BatchNorm2d)
from .quant import QLinear, Q8Linear, QuantizedTensor
from torch.nn import Parameter  # the tensor layer's parameter type (reference: rumus/src/nn/parameter.rs:16-55)
