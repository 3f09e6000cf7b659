from .causal_lm import CausalLM
from . import qwen3, lokinex, tabedra, kupelix, kozasun  # noqa: F401  (registers the architectures)
from .manifest import manifest_for  # noqa: E402,F401
