from . import llama          # registers "LlamaForCausalLM"
from . import deganex        # registers "Deganex"
from .text_model import TextModel
