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
from .two_d import (AdaptiveConvBiases2d, AdaptiveConvBranch2d, AdaptiveDeformConv2d, AttentionBlock2d, BiasProjection2d,
                    ContextualAttentionBlock2d, DeformConv2d, HeadConfig2d, LayerConfig2d, Model2d, ModelConfig2d,
                    MultiKernelSSMBlock2d, PixelEmbedding2d, PixelEmbedding2dLearned, RotaryEmbedding2d, SSMBlock3_2d,
                    UnifiedLayer2d, UnifiedModel2d)
