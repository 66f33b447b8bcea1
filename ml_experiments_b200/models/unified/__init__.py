"""UnifiedModel family: byte embedding -> [attention | bias projection] -> [multi-kernel SSM | SSM block] layers with
learned-pool feature integration, plus the building blocks (deformable / adaptive convolutions, S6 and SSD mixers)."""
from .attention import AttentionBackbone, AttentionBlock, ContextualAttentionBlock
from .composed import (EmbedPooler, FeatureIntegration, GatedMLP, HeadConfig, HeuristicEmbed, LayerConfig, Model,
                       ModelConfig, UnifiedLayer, UnifiedModel)
from .deform import (AdaptiveConvBiases, AdaptiveConvBranch, AdaptiveDeformConv1d, BiasProjection, ConvBackbone, ConvBlock,
                     DeformConv1d, KernelNet1d, SIRENLayer, deform_sample)
from .layers import (BinaryHead, ByteEmbedding, ClassifierHead, LearnedPooler, MaskHead, RMSNorm, RotaryEmbedding, SEBlock,
                     SwiGLU, apply_rotary_emb, apply_rotary_pos_emb_qk, chunked_local_attention)
from .ssm import MultiKernelSSMBlock, SSMBackbone, SSMBackbone3, SSMBlock, SSMBlock3, SSMMixer, SSMMixer3
