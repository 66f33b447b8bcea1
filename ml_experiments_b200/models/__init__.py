"""Model families: GPT (modded-nanogpt trainers), S6 / Ripple sequence models, scatter / hierarchical attention."""
from .gpt import GPT, GPTConfig  # noqa: F401
