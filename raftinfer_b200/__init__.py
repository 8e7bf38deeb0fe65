"""B200-native attention and gated-delta kernels behind RAFTInfer's kernel-launcher API."""
