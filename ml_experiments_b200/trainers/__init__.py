"""Training loops: the modded-nanogpt GPT trainers and the generic model trainers."""
