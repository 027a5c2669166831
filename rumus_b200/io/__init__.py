from .safetensors import save_safetensors, load_safetensors, load_into, serialize
