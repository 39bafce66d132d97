"""Architectures: each module holds a configuration class and the function that turns it into a
``ModelSpec``, and registers both under the architecture's name."""
from . import llama  # registers LlamaForCausalLM and Qwen3ForCausalLM
from . import givopel  # registers Givopel
from . import guzuvik  # registers Guzuvik
from . import zogevik  # registers Zogevik
from . import sofunex  # registers Sofunex

__all__ = ["llama", "givopel", "guzuvik", "zogevik", "sofunex"]
