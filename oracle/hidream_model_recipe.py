"""Seeded synthetic weights and inputs for a reduced HiDream-I1 transformer.  TEST INFRASTRUCTURE ONLY.

The golden file ``tests/golden/hidream_model_small.npz`` holds what the unmodified reference model
(``comfy/ldm/hidream/model.py:571-829``) returns for exactly these tensors; the tests rebuild them from the seeds
without needing the reference.  Nothing in the product path imports this file.
"""
from __future__ import annotations

from typing import Dict

import torch

# reduced model: 2 double-stream + 2 single-stream blocks, dim 512 = 4 heads x 128 (the rope axes need 128-wide heads)
CONFIG = dict(patch_size=2, in_channels=16, out_channels=16, num_layers=2, num_single_layers=2, attention_head_dim=128,
              num_attention_heads=4, caption_channels=[96, 64], text_emb_dim=48, num_routed_experts=4,
              num_activated_experts=2, axes_dims_rope=[64, 32, 32], max_resolution=[128, 128], llama_layers=[0, 1, 2, 2])
BATCH, HEIGHT, WIDTH, N_T5, N_LLAMA, LLAMA_LAYERS = 2, 32, 32, 16, 16, 3
W_SEED, X_SEED = 0, 1


def make_state(shapes: Dict[str, torch.Size], dtype: torch.dtype, seed: int = W_SEED) -> Dict[str, torch.Tensor]:
    """One tensor per state-dict key, drawn in the order of ``shapes`` (the model's ``state_dict()`` order): RMSNorm
    weights around 1, biases N(0, 0.1^2), everything else N(0, 0.02^2); drawn in fp32, then cast."""
    g = torch.Generator().manual_seed(seed)
    state = {}
    for key, shape in shapes.items():
        draw = torch.randn(tuple(shape), generator=g, dtype=torch.float32)
        if "rms_norm" in key:
            value = 1.0 + 0.1 * draw
        elif key.endswith("bias"):
            value = 0.1 * draw
        else:
            value = 0.02 * draw
        state[key] = value.to(dtype)
    return state


def make_inputs(dtype: torch.dtype, seed: int = X_SEED):
    """(x latent [B, 16, H, W], t [B], y pooled [B, 48], context T5 [B, 16, 96], llama states [B, 3, 16, 64])."""
    g = torch.Generator().manual_seed(seed)
    c = CONFIG
    x = torch.randn((BATCH, c["in_channels"], HEIGHT, WIDTH), generator=g).to(dtype)
    t = torch.tensor([500.0, 250.0][:BATCH])
    y = torch.randn((BATCH, c["text_emb_dim"]), generator=g).to(dtype)
    context = torch.randn((BATCH, N_T5, c["caption_channels"][0]), generator=g).to(dtype)
    llama = torch.randn((BATCH, LLAMA_LAYERS, N_LLAMA, c["caption_channels"][1]), generator=g).to(dtype)
    return x, t, y, context, llama
