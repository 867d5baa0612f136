from . import llama          # registers "LlamaForCausalLM"
from .text_model import TextModel
