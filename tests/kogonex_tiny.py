"""Small Kogonex configurations for the tests, and helpers that make their model folders.

The configurations differ from one another in every size and option: head counts and groups, key,
value, latent and rotated sizes, windows (also 1, and none), a layer that reads an earlier layer's
cache through a wider window, scaled and plain rotary positions, a rotated part of which only the
head is rotated, convolutions of 1 to 4 taps, experts with and without identity experts and groups,
one choice and several, layers without feed-forward, with and without bigram rows, widths that are
and are not multiples of 8.
"""

from __future__ import annotations

from pathlib import Path

import torch

from acorninfer_b200.config.model_config import (ChannelDeltaConfig, KogonexConfig, KogonexLayer, LatentAttentionConfig,
                                                 RotaryScaling, RoutedExpertsConfig)
from acorninfer_b200.weights.random_init import write_random_model
from acorninfer_b200.weights.safetensors_io import SafetensorsFile, write_safetensors

_SCALED = RotaryScaling(factor=8.0, original=16, fast=4.0, slow=0.5)

KOGO_A = dict(page_size=8, seed=11, cfg=KogonexConfig(
    vocab_size=200, hidden_size=64, norm_eps=1e-6, bigram_buckets=97, bigram_mul_prev=31, bigram_mul_cur=7, layers=(
        KogonexLayer(LatentAttentionConfig(heads=2, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.2, rot_dims=8,
                                           rot_base=1e4, scaling=_SCALED, window=9),
                     RoutedExpertsConfig(ff=48, experts=6, identity=2, top=2, groups=4, keep=2)),
        KogonexLayer(ChannelDeltaConfig(heads=4, kv_heads=2, dim=12, vdim=20, conv=4, decay_rank=6, gate_rank=10), None),
        KogonexLayer(LatentAttentionConfig(heads=3, dim=8, rot_dim=8, vdim=16, kv_rank=40, scale=0.3, rot_dims=8,
                                           rot_base=1e4, scaling=_SCALED, window=21, kv_from=0),
                     RoutedExpertsConfig(ff=24, experts=5, identity=0, top=1)),
        KogonexLayer(ChannelDeltaConfig(heads=2, kv_heads=2, dim=32, vdim=40, conv=1, decay_rank=4, gate_rank=4),
                     RoutedExpertsConfig(ff=32, experts=3, identity=3, top=3, groups=3, keep=3)),
    )))

KOGO_B = dict(page_size=4, seed=22, cfg=KogonexConfig(
    vocab_size=131, hidden_size=60, norm_eps=1e-5, layers=(
        KogonexLayer(ChannelDeltaConfig(heads=3, kv_heads=1, dim=20, vdim=36, conv=2, decay_rank=5, gate_rank=7),
                     RoutedExpertsConfig(ff=40, experts=4, identity=1, top=2)),
        KogonexLayer(LatentAttentionConfig(heads=5, dim=12, rot_dim=12, vdim=12, kv_rank=28, scale=0.25, rot_dims=8,
                                           rot_base=5e3, window=None), None),
        KogonexLayer(LatentAttentionConfig(heads=1, dim=24, rot_dim=4, vdim=20, kv_rank=20, scale=0.2, rot_dims=4,
                                           rot_base=1e5, scaling=RotaryScaling(2.0, 32, 8.0, 2.0), window=1),
                     RoutedExpertsConfig(ff=16, experts=2, identity=2, top=2, groups=2, keep=1)),
    )))

# sizes at which the bfloat16 engine takes its tensor-core products (multiples of 8 everywhere)
KOGO_C = dict(page_size=16, seed=33, cfg=KogonexConfig(
    vocab_size=320, hidden_size=128, norm_eps=1e-5, bigram_buckets=211, bigram_mul_prev=5, bigram_mul_cur=3, layers=(
        KogonexLayer(ChannelDeltaConfig(heads=2, kv_heads=1, dim=64, vdim=64, conv=3, decay_rank=8, gate_rank=16),
                     RoutedExpertsConfig(ff=64, experts=8, identity=0, top=2, groups=2, keep=1)),
        KogonexLayer(LatentAttentionConfig(heads=4, dim=48, rot_dim=16, vdim=40, kv_rank=64, scale=0.15, rot_dims=16,
                                           rot_base=1e6, scaling=RotaryScaling(4.0, 64, 16.0, 1.0), window=40),
                     RoutedExpertsConfig(ff=64, experts=6, identity=2, top=3, groups=2, keep=2)),
        KogonexLayer(LatentAttentionConfig(heads=2, dim=64, rot_dim=16, vdim=48, kv_rank=64, scale=0.1, rot_dims=16,
                                           rot_base=1e6, scaling=RotaryScaling(4.0, 64, 16.0, 1.0), window=17, kv_from=1),
                     None),
    )))

# longer requests: windows of 70 and 130 tokens over pages of 16, attention first and a delta layer last
KOGO_LONG = dict(page_size=16, seed=44, cfg=KogonexConfig(
    vocab_size=700, hidden_size=96, norm_eps=1e-5, bigram_buckets=389, bigram_mul_prev=11, bigram_mul_cur=13, layers=(
        KogonexLayer(LatentAttentionConfig(heads=6, dim=16, rot_dim=32, vdim=24, kv_rank=128, scale=0.12, rot_dims=32,
                                           rot_base=2e5, scaling=RotaryScaling(16.0, 48, 6.0, 1.5), window=70),
                     RoutedExpertsConfig(ff=40, experts=10, identity=2, top=3, groups=3, keep=2)),
        KogonexLayer(LatentAttentionConfig(heads=2, dim=40, rot_dim=32, vdim=56, kv_rank=128, scale=0.1, rot_dims=32,
                                           rot_base=2e5, scaling=RotaryScaling(16.0, 48, 6.0, 1.5), window=130, kv_from=0),
                     None),
        KogonexLayer(ChannelDeltaConfig(heads=4, kv_heads=2, dim=24, vdim=32, conv=3, decay_rank=8, gate_rank=8),
                     RoutedExpertsConfig(ff=48, experts=4, identity=0, top=2, groups=2, keep=2)),
    )))

KOGOS = {"kogo_a": KOGO_A, "kogo_b": KOGO_B, "kogo_c": KOGO_C}


def read_weights(model_dir: Path) -> dict[str, torch.Tensor]:
    f = SafetensorsFile(Path(model_dir) / "model.safetensors")
    return {n: f.tensor(n).clone() for n in f.entries}


def make_model_dir(tmp: Path, tiny: dict, sigma: float = 0.12, sigma_norm: float = 0.2, decisive: bool = False) -> Path:
    """A model folder with random weights; the routers are scaled up so that the choice of experts
    depends on the token and not on the correction alone.  ``decisive``: the corrections are distinct
    multiples of 2 instead, so that they alone decide the choice (the weights still follow the token):
    for runs in bfloat16, where a rounding could flip a close call and, through the recurrent state,
    change every later position of the request."""
    d = write_random_model(tmp, tiny["cfg"], tiny["seed"], sigma, sigma_norm)
    w = read_weights(d)
    for name in w:
        if name.endswith(".router") and not decisive:     # (large logits would make the chosen weights tiny and their ratios coarse in bfloat16)
            w[name] = (w[name].float() * 6).to(w[name].dtype)
        if name.endswith(".correction"):
            n = w[name].numel()
            order = torch.randperm(n, generator=torch.Generator().manual_seed(n + len(name))).float()
            w[name] = (order * 2 if decisive else w[name].float() * 0.1).to(w[name].dtype)
    write_safetensors(d / "model.safetensors", w, {"format": "pt"})
    return d
