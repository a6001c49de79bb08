"""Sparse-MLA FP8 MoE decoder layers (DeepSeek-V3.2 / GLM-DSA style) as K1 / K2i / K2 launch sequences."""
