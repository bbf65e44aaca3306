"""Small Vagulorn configurations for the tests, and helpers that make their model folders.

The configurations differ from one another in every size and option: the order and kinds of the layers,
head counts and groups, key and value sizes (equal and not), rotated parts (none, a part, the whole head),
blocks and windows of several sizes (also 1, and none), kept first keys (none, fewer and more than a
page), decays (also 1 and 0), state sizes and groups, convolutions of 1 to 4 taps, norm parts (1 and
more), layers without feed-forward, an embedding scale of 1 and others, widths that are and are not
multiples of 8.
"""

from __future__ import annotations

from pathlib import Path

import torch

from acorninfer_b200.config.model_config import (DecayLinearAttentionConfig, MaskedAttentionConfig, SideBySideConfig,
                                                 StateSpaceConfig, VagulornConfig, VagulornLayer)
from acorninfer_b200.weights.random_init import write_random_model
from acorninfer_b200.weights.safetensors_io import SafetensorsFile


def att(heads, kv_heads, dim, vdim, scale, rot_dims=0, rot_base=1e4, mask_size=None, keep_first=0):
    return MaskedAttentionConfig(heads, kv_heads, dim, vdim, scale, rot_dims, rot_base, mask_size, keep_first)


def beside(left, heads, dim, vdim, decay, left_scale=1.0, right_scale=1.0):
    return SideBySideConfig(left, DecayLinearAttentionConfig(heads, dim, vdim, tuple(decay)), left_scale, right_scale)


def L(mixer, ff=None):
    kind = {MaskedAttentionConfig: "attention", SideBySideConfig: "parallel", StateSpaceConfig: "mamba2"}[type(mixer)]
    return VagulornLayer(kind, mixer, ff)


VAGU_A = dict(page_size=8, seed=7, cfg=VagulornConfig(
    vocab_size=210, hidden_size=72, norm_eps=1e-6, embedding_scale=3.0, layers=(
        L(att(heads=4, kv_heads=2, dim=12, vdim=20, scale=0.3, rot_dims=8, rot_base=1e4, mask_size=11), ff=96),
        L(StateSpaceConfig(heads=6, vdim=10, state=7, groups=3, conv=4, norm_groups=3), ff=40),
        L(beside(att(heads=3, kv_heads=1, dim=10, vdim=10, scale=0.25, rot_dims=10, rot_base=500.0, mask_size=9,
                     keep_first=3), heads=2, dim=6, vdim=14, decay=(0.5, 0.97), left_scale=0.7, right_scale=1.3), ff=None),
        L(StateSpaceConfig(heads=2, vdim=24, state=20, groups=1, conv=1, norm_groups=1), ff=64),
    )))

VAGU_B = dict(page_size=4, seed=8, cfg=VagulornConfig(
    vocab_size=133, hidden_size=60, norm_eps=1e-5, embedding_scale=1.0, layers=(
        L(beside(att(heads=2, kv_heads=2, dim=16, vdim=16, scale=0.2, rot_dims=4, rot_base=1e5, mask_size=1, keep_first=2),
                 heads=3, dim=9, vdim=5, decay=(1.0, 0.0, 0.8), left_scale=1.0, right_scale=0.5), ff=48),
        L(att(heads=5, kv_heads=1, dim=8, vdim=6, scale=0.35, rot_dims=0, mask_size=None), ff=None),
        L(StateSpaceConfig(heads=3, vdim=12, state=33, groups=3, conv=2, norm_groups=2), ff=None),
        L(att(heads=2, kv_heads=2, dim=24, vdim=24, scale=0.2, rot_dims=24, rot_base=77.0, mask_size=6), ff=30),
        L(beside(att(heads=1, kv_heads=1, dim=20, vdim=20, scale=0.2, rot_dims=0, mask_size=None),
                 heads=1, dim=40, vdim=8, decay=(0.9,)), ff=20),
    )))

# sizes at which the bfloat16 engine takes its tensor-core paths (head sizes that are multiples of 16, widths of 8)
VAGU_C = dict(page_size=16, seed=9, cfg=VagulornConfig(
    vocab_size=320, hidden_size=128, norm_eps=1e-5, embedding_scale=8.0, layers=(
        L(StateSpaceConfig(heads=4, vdim=32, state=64, groups=2, conv=3, norm_groups=2), ff=192),
        L(beside(att(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, rot_dims=32, rot_base=3e5, mask_size=40,
                     keep_first=5), heads=2, dim=32, vdim=48, decay=(0.7, 0.995), left_scale=0.8, right_scale=0.9), ff=192),
        L(att(heads=6, kv_heads=3, dim=32, vdim=32, scale=0.18, rot_dims=16, rot_base=1e4, mask_size=24), ff=128),
        L(att(heads=2, kv_heads=1, dim=48, vdim=80, scale=0.15, rot_dims=48, rot_base=1e4, mask_size=50), ff=None),
    )))

# longer requests: blocks of 70 and a window of 130 with 20 kept keys over pages of 16, state carried far
VAGU_LONG = dict(page_size=16, seed=10, cfg=VagulornConfig(
    vocab_size=600, hidden_size=96, norm_eps=1e-5, embedding_scale=4.0, layers=(
        L(att(heads=4, kv_heads=2, dim=32, vdim=32, scale=0.18, rot_dims=16, rot_base=2e5, mask_size=70), ff=64),
        L(beside(att(heads=2, kv_heads=1, dim=48, vdim=48, scale=0.15, rot_dims=24, rot_base=1e4, mask_size=130,
                     keep_first=20), heads=3, dim=16, vdim=16, decay=(0.9, 0.99, 0.999), left_scale=0.9, right_scale=0.6), ff=None),
        L(StateSpaceConfig(heads=4, vdim=16, state=24, groups=2, conv=3, norm_groups=4), ff=48),
    )))

VAGUS = {"vagu_a": VAGU_A, "vagu_b": VAGU_B, "vagu_c": VAGU_C}


def read_weights(model_dir: Path) -> dict[str, torch.Tensor]:
    f = SafetensorsFile(Path(model_dir) / "model.safetensors")
    return {n: f.tensor(n).clone() for n in f.entries}


def make_model_dir(tmp: Path, tiny: dict, sigma: float = 0.12, sigma_norm: float = 0.2) -> Path:
    return write_random_model(tmp, tiny["cfg"], tiny["seed"], sigma, sigma_norm)


def random_config(seed: int) -> VagulornConfig:
    """A configuration drawn at random: 3 to 5 layers with each kind of mixer at least once, widths, head counts,
    key, value and state sizes, rotated parts, blocks, windows, kept keys, taps and norm parts from lists that hold
    the sizes real models have (heads of 32 to 128, states of 16 to 128) beside odd ones."""
    import random
    rng = random.Random(seed)
    width = rng.choice([128, 192, 320, 384])
    kinds = ["attention", "parallel", "mamba2"]
    n = rng.randint(3, 5)
    order = [rng.choice(kinds) for _ in range(n)]
    for k in kinds:
        if k not in order:
            order[rng.randrange(n)] = k
    layers = []
    for k in order:
        ff = rng.choice([None, 200, 256, 384])
        if k == "attention":
            d, kv = rng.choice([32, 64, 96, 128]), rng.choice([1, 2, 4])
            dv, rd = rng.choice([d, d, 64, 160]), rng.choice([d, d // 2, d // 4])
            if rng.random() < 0.4:
                d = dv = rd = 128                       # whole head rotated: the products' own rotary epilogue where it applies
            layers.append(L(att(kv * rng.choice([1, 2, 3, 4]), kv, d, dv, d ** -0.5, rot_dims=rd, rot_base=rng.choice([1e4, 3e5]),
                                mask_size=rng.choice([32, 64, 100, 256])), ff))
        elif k == "parallel":
            d, kv = rng.choice([32, 64, 96, 128]), rng.choice([1, 2])
            hr = rng.choice([1, 2, 4, 8])
            layers.append(L(beside(att(kv * rng.choice([1, 2, 4]), kv, d, d, d ** -0.5, rot_dims=rng.choice([d, d // 2]),
                                       mask_size=rng.choice([32, 64, 100]), keep_first=rng.choice([0, 1, 4, 20])),
                                   heads=hr, dim=rng.choice([16, 32, 64, 128]), vdim=rng.choice([16, 32, 64, 128]),
                                   decay=[rng.choice([0.5, 0.9, 0.99, 0.999]) for _ in range(hr)],
                                   left_scale=rng.choice([0.5, 1.0]), right_scale=rng.choice([0.7, 1.2])), ff))
        else:
            g = rng.choice([1, 2, 4])
            heads = g * rng.choice([1, 2, 4])
            layers.append(L(StateSpaceConfig(heads=heads, vdim=rng.choice([16, 32, 48, 64]), state=rng.choice([16, 48, 64, 128]),
                                             groups=g, conv=rng.choice([2, 3, 4]), norm_groups=rng.choice([1, 2, heads])), ff))
    return VagulornConfig(vocab_size=rng.choice([300, 512, 1000]), hidden_size=width, norm_eps=rng.choice([1e-5, 1e-6]),
                          embedding_scale=rng.choice([1.0, 8.0, 20.0]), layers=tuple(layers))
