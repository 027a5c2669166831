from .gpt import GPT, GPTConfig
from .llama import Llama, LlamaConfig
from .resnet import ResNet50, Bottleneck
