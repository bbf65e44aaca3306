"""Two recurrent mixers whose per-request state is a matrix per head, updated by a linear recurrence.

Both run on the same kernels (``csrc/linear_recurrence.cu``): per head a float32 state S [N, V] that
starts at zero and, for every token, ``S <- a S + b (w x)^T``, ``y = S^T c (+ skip x)``.

``state_space`` (a selective state space layer in its state-space-duality form; Dao and Gu,
"Transformers are SSMs: Generalized Models and Efficient Algorithms Through Structured State Space
Duality"): one input projection yields ``[z | x | B | C | dt]`` (``inner = heads * vdim`` gate and
input channels, ``groups * state`` write and read keys, a step size per head).  x, B and C pass a short
causal convolution per channel over time (``taps`` weights, the last for the current token, zeros
before a request's start, a bias) and silu;  ``dt = softplus(dt + dt_bias)``;  per head (head h uses the
keys of group ``h // (heads / groups)``)  ``a = exp(-exp(A_log_h) dt)``, ``w = dt``, ``skip = D_h``;
the heads' outputs times ``silu(z)``, RMS-normed in ``norm_groups`` equal parts with one weight, then the
output projection.  The convolution's last ``taps - 1`` inputs are per-request state beside S.

``decay_linear_attention`` (linear attention with a fixed decay per head): ``q, k = silu(W h)`` per head
(``dim`` entries), ``v = silu(W_v h)`` (``vdim``), ``S <- decay_h S + k v^T``, ``o = S^T q``; the heads'
outputs RMS-normed together with a weight, times ``sigmoid(W_g h)``, then the output projection.

Everything after the activations is float32 (step sizes, decays, the state, the norms); the projections
and the convolution's inputs are in the engine's activation dtype.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, BuildContext, CacheNeeds, Mixer, StateNeeds, TensorSpec


class _RecurrentMixer(Mixer):
    """Common to both: the state is one float32 vector per request, S of all heads first, addressed from
    ``state_base`` (a mixer that shares a request's slot with another gets its part of the vector).
    The one host-side value of the step they read is its longest row (long rows are run in segments); it is 1
    in every step of single tokens, the only steps of a model with state that are captured and replayed."""

    graph_safe = True
    adds_residual = True
    state_base = 0

    def forward(self, x, inputs, cache, residual32=None):
        return ops.linear(self.inner(x, inputs, cache), self.w_o, out_dtype=self.ctx.dtype, residual32=residual32)


@MIXERS.register("state_space")
class StateSpace(_RecurrentMixer):
    def __init__(self, ctx: BuildContext, hidden_size: int, num_heads: int, vdim: int, state: int, groups: int,
                 taps: int, norm_groups: int, norm_eps: float):
        if num_heads % groups:
            raise ValueError(f"num_heads ({num_heads}) must be a multiple of groups ({groups})")
        if (num_heads * vdim) % norm_groups:
            raise ValueError(f"heads * vdim ({num_heads * vdim}) must split into norm_groups ({norm_groups}) equal parts")
        self.ctx = ctx
        self.hidden_size = hidden_size
        self.H, self.V, self.N, self.G, self.taps = num_heads, vdim, state, groups, taps
        self.norm_groups, self.eps = norm_groups, float(norm_eps)
        self.inner_size = num_heads * vdim
        self.channels = self.inner_size + 2 * groups * state            # through the convolution: x, B, C
        self.state_s = num_heads * state * vdim                         # floats of S; the convolution's memory follows
        self.w_in = self.w_o = None

    def tensor_specs(self):
        H, W, C = self.H, self.hidden_size, self.channels
        return {
            "in": TensorSpec((self.inner_size + C + H, W)),
            "conv": TensorSpec((C, self.taps), "conv"), "conv.b": TensorSpec((C,), "bias"),
            "dt_bias": TensorSpec((H,), "bias"), "A_log": TensorSpec((H,), "decay_log"), "D": TensorSpec((H,), "norm"),
            "norm": TensorSpec((self.inner_size,), "norm"), "o": TensorSpec((W, self.inner_size)),
        }

    def bind(self, tensors):
        t = tensors
        f32 = lambda x: x.to(torch.float32).contiguous()
        self.w_in, self.w_o = t["in"].contiguous(), t["o"].contiguous()
        self.conv32, self.conv_b32 = f32(t["conv"]), f32(t["conv.b"])
        self.dt_bias32, self.a_log32, self.d32, self.norm32 = f32(t["dt_bias"]), f32(t["A_log"]), f32(t["D"]), f32(t["norm"])

    def state_size(self) -> int:
        return self.state_s + (self.taps - 1) * self.channels

    def cache_needs(self):
        return CacheNeeds(state=StateNeeds((self.state_size(),)))

    def inner(self, x, inputs, cache, out_scale: float = 1.0, out=None):
        I, GN, C = self.inner_size, self.G * self.N, self.channels
        proj = ops.linear(x, self.w_in, out_dtype=self.ctx.dtype)             # [z | x | B | C | dt]
        conv_off = self.state_base + self.state_s
        act, dt, decay = ops.ssm_prep(proj, I, I + C, self.conv32, self.conv_b32, cache.state, conv_off, self.a_log32,
                                      self.dt_bias32, inputs.token_row, inputs.row_start, inputs.row_slot, self.taps,
                                      update_single=True)
        if inputs.plan.max_q_len > 1:       # rows of one token had their convolution memory shifted by ssm_prep
            ops.conv_state_update(proj[:, I:I + C], cache.state, conv_off, inputs.row_start, inputs.row_slot,
                                  inputs.num_rows, C, self.taps, skip_single=True)
        y = ops.linear_scan(act[:, I:I + GN], act[:, I + GN:], act[:, :I], decay, dt, self.d32, cache.state,
                            self.state_base, inputs.row_start, inputs.row_slot, inputs.num_rows, self.H, self.G,
                            self.N, self.V, longest_row=inputs.plan.max_q_len)
        if out is None:
            out = torch.empty((proj.shape[0], I), dtype=self.ctx.dtype, device=proj.device)
        return ops.gated_norm(y, proj[:, :I], self.norm32, self.eps, self.norm_groups, True, out, out_scale)


@MIXERS.register("decay_linear_attention")
class DecayLinearAttention(_RecurrentMixer):
    def __init__(self, ctx: BuildContext, hidden_size: int, num_heads: int, dim: int, vdim: int, decay, norm_eps: float):
        decay = [float(d) for d in decay]
        if len(decay) != num_heads:
            raise ValueError(f"decay must give one number per head ({num_heads}), got {len(decay)}")
        self.ctx = ctx
        self.hidden_size = hidden_size
        self.H, self.dim, self.V = num_heads, dim, vdim
        self.eps = float(norm_eps)
        self.decay = decay
        self._decay32 = None
        self.w_in = self.w_o = None

    def tensor_specs(self):
        H, d, v, W = self.H, self.dim, self.V, self.hidden_size
        return {"q": TensorSpec((H * d, W)), "k": TensorSpec((H * d, W)), "v": TensorSpec((H * v, W)),
                "g": TensorSpec((H * v, W)), "norm": TensorSpec((H * v,), "norm"), "o": TensorSpec((W, H * v))}

    def bind(self, tensors):
        t = tensors
        mats = [t[n] for n in ("q", "k", "v", "g")]
        dtype = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
        self.w_in = torch.cat([m.to(dtype) for m in mats], dim=0).contiguous()
        self.w_o = t["o"].contiguous()
        self.norm32 = t["norm"].to(torch.float32).contiguous()
        self._decay32 = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(self.w_o.device)

    def state_size(self) -> int:
        return self.H * self.dim * self.V

    def cache_needs(self):
        return CacheNeeds(state=StateNeeds((self.state_size(),)))

    def inner(self, x, inputs, cache, out_scale: float = 1.0, out=None):
        Hd, Hv = self.H * self.dim, self.H * self.V
        proj = ops.linear(x, self.w_in, out_dtype=self.ctx.dtype)             # [q | k | v | g]
        act = ops.silu_rows(proj[:, :2 * Hd + Hv])
        y = ops.linear_scan(act[:, Hd:2 * Hd], act[:, :Hd], act[:, 2 * Hd:], self._decay32, None, None, cache.state,
                            self.state_base, inputs.row_start, inputs.row_slot, inputs.num_rows, self.H, self.H,
                            self.dim, self.V, longest_row=inputs.plan.max_q_len)
        if out is None:
            out = torch.empty((proj.shape[0], Hv), dtype=self.ctx.dtype, device=proj.device)
        return ops.gated_norm(y, proj[:, 2 * Hd + Hv:], self.norm32, self.eps, 1, False, out, out_scale)
