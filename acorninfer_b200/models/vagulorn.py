"""Vagulorn as data: which parts each layer has, with which sizes, in which order.

A token's row of the token table times a scale; layers in the ``parallel`` arrangement
(``h = LayerNorm(x); x += mixer(h) + ff(h)``), each with its own mixer: ``attention`` within blocks of
positions; ``side_by_side`` of attention (a window with kept first keys, values that are the keys as
projected, a gate per head, interleaved rotary pairs) and ``decay_linear_attention``; or ``state_space``;
and a gated feed-forward with the tanh form of gelu, or none.  The final LayerNorm, and the token table itself
(without the scale) as output matrix.  Every attention names a position encoding of its own sizes (equal
settings share one).

Tensor names: ``embed``, ``l<i>.norm1`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``, ``final.norm`` (+ ``.b``).
"""

from __future__ import annotations

from ..config.model_config import (MaskedAttentionConfig, SideBySideConfig, StateSpaceConfig, VagulornConfig)
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "gate": "g"}


def _position(m: MaskedAttentionConfig, pairing: str, positions: dict) -> str | None:
    """Name of the position encoding for these rotary settings (made on first use)."""
    if m.rot_dims == 0:
        return None
    key = (m.dim, m.rot_dims, m.rot_base, pairing)
    for name, (k, _) in positions.items():
        if k == key:
            return name
    name = f"rot{len(positions)}"
    positions[name] = (key, PartSpec("rope", {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                              "pairing": pairing}))
    return name


def _attention(m: MaskedAttentionConfig, W: int, eps: float, prefix: str, positions: dict, beside: bool) -> PartSpec:
    params = {"hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
              "scale": m.scale, "qk_norm_eps": eps, "names": _ATTENTION_NAMES,
              "position": _position(m, "interleaved" if beside else "half", positions)}
    if beside:      # beside a recurrent mixer: a window with kept first keys, values = keys, a gate per head
        params.update(window=m.mask_size, keep_first=m.keep_first if m.mask_size is not None else 0,
                      values_from_keys=True, head_gate=True)
    else:           # a layer of its own: blocks of positions
        params.update(chunk=m.mask_size)
    return PartSpec("attention", params, prefix)


def vagulorn_spec(cfg: VagulornConfig) -> ModelSpec:
    W, eps = cfg.hidden_size, cfg.norm_eps
    positions: dict = {}
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if isinstance(m, MaskedAttentionConfig):
            mixer = _attention(m, W, eps, p + "mix.", positions, beside=False)
        elif isinstance(m, SideBySideConfig):
            r = m.right
            mixer = PartSpec("side_by_side", {
                "left": _attention(m.left, W, eps, "left.", positions, beside=True),
                "right": PartSpec("decay_linear_attention", {"hidden_size": W, "num_heads": r.heads, "dim": r.dim,
                                                             "vdim": r.vdim, "decay": r.decay, "norm_eps": eps}, "right."),
                "left_scale": m.left_scale, "right_scale": m.right_scale}, p + "mix.")
        else:
            assert isinstance(m, StateSpaceConfig)
            mixer = PartSpec("state_space", {"hidden_size": W, "num_heads": m.heads, "vdim": m.vdim, "state": m.state,
                                             "groups": m.groups, "taps": m.conv, "norm_groups": m.norm_groups,
                                             "norm_eps": eps}, p + "mix.")
        ff = None if layer.ff is None else PartSpec("gated", {
            "hidden_size": W, "intermediate_size": layer.ff, "activation": "gelu_tanh",
            "names": {"gate": "gate", "up": "up", "down": "down"}}, p + "mlp.")
        norms = {"input": PartSpec("layernorm", {"width": W, "eps": eps, "tensor": "", "bias_tensor": ".b"}, p + "norm1")}
        layers.append(LayerSpec(PartSpec("parallel", {}, p), mixer, ff, norms))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=W, embedding="embed", layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("layernorm", {"width": W, "eps": eps, "tensor": "", "bias_tensor": ".b"}, "final.norm"),
        head=None, positions={name: spec for name, (_, spec) in positions.items()},
        embedding_scale=cfg.embedding_scale)


register_architecture(VagulornConfig.architecture, VagulornConfig, vagulorn_spec)
