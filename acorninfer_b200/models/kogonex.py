"""Kogonex as data: which parts each layer has, with which sizes, in which order.

A token's row of the token table plus a hashed bigram row (``bigram_rows`` stage); layers in the
``outnorm`` arrangement (``x += norm1(mixer(x)); x += norm2(ff(x))``), each with its own mixer
(``latent_attention`` or ``channel_delta``) and routed experts or no feed-forward at all; the final
norm and the output matrix.  A latent-attention layer with ``kv_from = j`` becomes a schedule entry
that reads the cache of layer j's entry.  Every latent-attention layer names a position encoding of
its own sizes (layers with equal rotary settings share one).

Tensor names: ``embed``, ``bigram``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.model_config import ChannelDeltaConfig, KogonexConfig, LatentAttentionConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture


def _position(m: LatentAttentionConfig, positions: dict) -> str | None:
    """Name of the position encoding for this layer's rotated part (made on first use)."""
    if m.rot_dims == 0:
        return None
    key = ("rot", m.rot_dim, m.rot_dims, m.rot_base, m.scaling)
    name = f"rot{len(positions)}"
    for have, (k, _) in positions.items():
        if k == key:
            return have
    params = {"head_dim": m.rot_dim, "rotary_dim": m.rot_dims, "theta": m.rot_base, "pairing": "interleaved"}
    if m.scaling is None:
        positions[name] = (key, PartSpec("rope", params))
    else:
        sc = m.scaling
        positions[name] = (key, PartSpec("scaled_rope", {**params, "factor": sc.factor, "original": sc.original,
                                                         "fast": sc.fast, "slow": sc.slow}))
    return name


def kogonex_spec(cfg: KogonexConfig) -> ModelSpec:
    W, eps = cfg.hidden_size, cfg.norm_eps
    positions: dict = {}
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if isinstance(m, LatentAttentionConfig):
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "num_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": eps, "position": _position(m, positions),
                "window": m.window, "own_cache": m.kv_from is None}, p + "mix.")
            schedule.append(ScheduleEntry(i, reads_cache_of=m.kv_from))      # one entry per layer: entry j is layer j
        else:
            assert isinstance(m, ChannelDeltaConfig)
            mixer = PartSpec("channel_delta", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
                "taps": m.conv, "norm_eps": eps, "decay_rank": m.decay_rank, "gate_rank": m.gate_rank}, p + "mix.")
            schedule.append(ScheduleEntry(i))
        norms = {"mixer": PartSpec("rmsnorm", {"width": W, "eps": eps, "tensor": ""}, p + "norm1")}
        ff = None
        if layer.mlp is not None:
            f = layer.mlp
            ff = PartSpec("routed_experts", {"hidden_size": W, "expert_size": f.ff, "num_experts": f.experts,
                                             "num_identity": f.identity, "top": f.top, "groups": f.groups,
                                             "keep": f.keep}, p + "mlp.")
            norms["feed_forward"] = PartSpec("rmsnorm", {"width": W, "eps": eps, "tensor": ""}, p + "norm2")
        layers.append(LayerSpec(PartSpec("outnorm", {}, p), mixer, ff, norms))
    stages = ()
    if cfg.bigram_buckets is not None:
        stages = (PartSpec("bigram_rows", {"width": W, "buckets": cfg.bigram_buckets, "mul_prev": cfg.bigram_mul_prev,
                                           "mul_cur": cfg.bigram_mul_cur, "tensor": "bigram"}, ""),)
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=W, embedding="embed", layers=tuple(layers), schedule=tuple(schedule),
        final_norm=PartSpec("rmsnorm", {"width": W, "eps": eps, "tensor": ""}, "final.norm"), head="head",
        positions={name: spec for name, (_, spec) in positions.items()}, after_embedding=stages)


register_architecture(KogonexConfig.architecture, KogonexConfig, kogonex_spec)
