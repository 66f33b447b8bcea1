"""``zoology.mixers.mamba_ssm`` under the reference's module names (the vendored package of the reference:
zoology/mixers/mamba_ssm/). The reference's functions take channel-first tensors and call Triton programs and two
external CUDA extensions; here they are thin layout adapters onto this package's kernels (S6 scan, chunked SSD scan,
causal depthwise convolution) and their PyTorch restatements."""
