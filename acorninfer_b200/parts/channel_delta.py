"""Gated delta rule with one decay per key channel, as a mixer with per-request state.

Per token, from the mixer's input h:
  q, k (kv_heads x dim) and v (heads x vdim): projections, a short causal convolution over time per
  channel (``taps`` weights, the last one for the current token, zeros before a request's start),
  silu; q and k are then scaled to unit length per head (``x / sqrt(sum x^2 + 1e-6)``), q further by
  ``dim^-1/2``; head a uses q/k head ``a // (heads / kv_heads)``.
  beta = sigmoid(W_b h) per head;  g = exp(-exp(A_log_a) softplus(W_a2 W_a1 h + dt_bias)) per head and
  key channel;  gate = sigmoid(W_g2 W_g1 h) per head and value channel.
  Per head, on a state S [dim, vdim] that starts at zero:
      S = g[:, None] * S;  u = beta (v - S^T k);  S += k u^T;  o = S^T q
  then o / rms(o) * norm * gate per head, and the output projection.
Everything after the convolutions' silu is float32, and so is the state: S of every head and the
convolutions' last ``taps - 1`` inputs live in the request's state slot (one float32 vector).

The projections are three matrix products: [q | k | v | b] at once, [a1 | g1] at once, and their
up-projections as one block-diagonal matrix (the zero blocks add exact zeros).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, BuildContext, CacheNeeds, Mixer, StateNeeds, TensorSpec


@MIXERS.register("channel_delta")
class ChannelDelta(Mixer):
    graph_safe = True

    def __init__(self, ctx: BuildContext, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int,
                 taps: int, norm_eps: float, decay_rank: int | None = None, gate_rank: int | None = None):
        """``decay_rank`` / ``gate_rank``: inner sizes of the two low-rank projections; None: taken
        from the checkpoint's tensors (``expected_tensors`` then cannot list them: give them when
        writing a model)."""
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be a multiple of num_kv_heads ({num_kv_heads})")
        self.ctx = ctx
        self.hidden_size = hidden_size
        self.H, self.KH, self.dim, self.vdim, self.taps = num_heads, num_kv_heads, dim, vdim, taps
        self.eps = float(norm_eps)
        self.decay_rank, self.gate_rank = decay_rank, gate_rank
        self.channels = 2 * num_kv_heads * dim + num_heads * vdim
        self.state_s = num_heads * dim * vdim                         # floats of S; the convolutions' memory follows
        self.w_main = self.w_low = self.w_up = self.w_o = None

    def tensor_specs(self):
        H, KH, d, v, W = self.H, self.KH, self.dim, self.vdim, self.hidden_size
        ra, rg = self.decay_rank, self.gate_rank
        return {
            "q": TensorSpec((KH * d, W)), "q.conv": TensorSpec((KH * d, self.taps), "conv"),
            "k": TensorSpec((KH * d, W)), "k.conv": TensorSpec((KH * d, self.taps), "conv"),
            "v": TensorSpec((H * v, W)), "v.conv": TensorSpec((H * v, self.taps), "conv"),
            "b": TensorSpec((H, W)), "A_log": TensorSpec((H,), "decay_log"), "norm": TensorSpec((v,), "norm"),
            "a1": TensorSpec((ra, W)), "a2": TensorSpec((H * d, ra)), "dt_bias": TensorSpec((H * d,), "bias"),
            "g1": TensorSpec((rg, W)), "g2": TensorSpec((H * v, rg)),
            "o": TensorSpec((W, H * v)),
        }

    def bind(self, tensors):
        t = tensors
        mats = [t[n] for n in ("q", "k", "v", "b", "a1", "g1", "a2", "g2")]
        dtype = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
        self.w_main = torch.cat([t[n].to(dtype) for n in ("q", "k", "v", "b")], dim=0).contiguous()
        self.w_low = torch.cat([t["a1"].to(dtype), t["g1"].to(dtype)], dim=0).contiguous()
        ra, rg = t["a1"].shape[0], t["g1"].shape[0]
        up = torch.zeros((self.H * (self.dim + self.vdim), ra + rg), dtype=dtype, device=t["a2"].device)
        up[:self.H * self.dim, :ra] = t["a2"].to(dtype)
        up[self.H * self.dim:, ra:] = t["g2"].to(dtype)
        self.w_up = up.contiguous()
        self.w_o = t["o"].contiguous()
        f32 = lambda x: x.to(torch.float32).contiguous()
        self.conv32 = f32(torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0))
        self.a_log32, self.dt_bias32, self.norm32 = f32(t["A_log"]), f32(t["dt_bias"]), f32(t["norm"])

    def cache_needs(self):
        return CacheNeeds(state=StateNeeds((self.state_s + (self.taps - 1) * self.channels,)))

    def forward(self, x, inputs, cache):
        dt = self.ctx.dtype
        main = ops.linear(x, self.w_main, out_dtype=dt)
        up = ops.linear(ops.linear(x, self.w_low, out_dtype=dt), self.w_up, out_dtype=torch.float32)
        q, k, v, beta, g, gate = ops.delta_prep(main, up, self.conv32, cache.state, self.state_s, self.a_log32,
                                                self.dt_bias32, inputs.token_row, inputs.row_start, inputs.row_slot,
                                                self.H, self.KH, self.dim, self.vdim, self.taps)
        ops.conv_state_update(main, cache.state, self.state_s, inputs.row_start, inputs.row_slot, inputs.num_rows,
                              self.channels, self.taps)
        o = ops.delta_rule(q, k, v, beta, g, cache.state, inputs.row_start, inputs.row_slot, inputs.num_rows)
        y = ops.delta_out(o, gate, self.norm32, self.eps, dt)
        return ops.linear(y, self.w_o, out_dtype=dt)
