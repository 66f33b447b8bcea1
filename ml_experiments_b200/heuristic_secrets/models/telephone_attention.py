"""``heuristic_secrets.models.telephone_attention``: telephone attention (reference:
src/heuristic_secrets/models/telephone_attention.py). Re-exports."""
# ruff: noqa: F401
from ...models.ripple_ops import SDPAttention, TelephoneAttentionND, llama_rmsnorm

HAS_TRITON = True   # "a fused kernel path exists": the CUDA kernels of this package stand where the reference has Triton programs
