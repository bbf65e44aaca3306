"""Rotary position encoding: the constants, and a stand-alone application.

``inv_freq[j] = 1 / theta^(2j / rotary_dim)`` in float32, angle = position * inv_freq[j];
pairing ``half`` rotates (x[j], x[j + rotary_dim/2]), ``interleaved`` rotates (x[2j], x[2j+1]);
dimensions beyond ``rotary_dim`` pass through.  Reference: ``RotaryEmbedding``, ``_rotate_half``,
``_apply_rope`` in ``acorninfer/models/qwen3.py:63-95`` (half pairing, full head rotated).
The mixers' kernels take these constants; nothing here knows about attention.
"""

from __future__ import annotations

import torch

from .base import POSITION_ENCODINGS, BuildContext, PositionEncoding


@POSITION_ENCODINGS.register("rope")
class Rope(PositionEncoding):
    def __init__(self, ctx: BuildContext, head_dim: int, theta: float, rotary_dim: int | None = None,
                 pairing: str = "half"):
        rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rope pairing must be 'half' or 'interleaved', got {pairing!r}")
        if rotary_dim % 2 or not (0 < rotary_dim <= head_dim):
            raise ValueError(f"rotary_dim must be even and in 2..head_dim, got {rotary_dim}")
        self.ctx = ctx
        self.head_dim = head_dim
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.interleaved = pairing == "interleaved"
        self.magnitude = 1.0                  # factor on cos and sin
        self._inv_freq_cpu = 1.0 / (self.theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
        self._inv_freq_dev: torch.Tensor | None = None

    @property
    def inv_freq(self) -> torch.Tensor:
        if self._inv_freq_dev is None:
            self._inv_freq_dev = self._inv_freq_cpu.to(self.ctx.device).contiguous()
        return self._inv_freq_dev

    def table(self, inputs) -> torch.Tensor:
        """cos and sin of every token's angles, [tokens, rotary_dim] float32 (cos, then sin): computed by
        the first layer of a step that asks and kept with the step's inputs for the others."""
        from ..kernels import ops
        key = ("rope.table", self.theta, self.rotary_dim)
        if key not in inputs.extra:
            inputs.extra[key] = ops.rope_table(inputs.positions, self.inv_freq)
        return inputs.extra[key]


@POSITION_ENCODINGS.register("scaled_rope")
class ScaledRope(Rope):
    """Rotary positions with the frequencies stretched for contexts beyond the trained one (YaRN: Peng,
    Quesnelle, Fan, Shippole, "YaRN: Efficient Context Window Extension of Large Language Models").
    With f_i = theta^(-2i / rotary_dim) and pair(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta), the
    pair index that turns t times over ``original`` positions:
        lo = max(floor(pair(fast)), 0),  hi = min(ceil(pair(slow)), rotary_dim - 1),
        ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
        frequency_i = (f_i / factor) ramp_i + f_i (1 - ramp_i),
    and cos and sin are multiplied by ``0.1 ln(factor) + 1`` (``magnitude``)."""

    def __init__(self, ctx: BuildContext, head_dim: int, theta: float, factor: float, original: int, fast: float,
                 slow: float, rotary_dim: int | None = None, pairing: str = "interleaved"):
        super().__init__(ctx, head_dim, theta, rotary_dim, pairing)
        import math
        n = self.rotary_dim

        def pair(turns):
            return n * math.log(original / (2 * math.pi * turns)) / (2 * math.log(theta))

        lo, hi = max(math.floor(pair(fast)), 0), min(math.ceil(pair(slow)), n - 1)
        freq = []
        for i in range(n // 2):
            f = float(theta) ** (-2.0 * i / n)
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            freq.append(f / factor * ramp + f * (1.0 - ramp))
        self._inv_freq_cpu = torch.tensor(freq, dtype=torch.float64).to(torch.float32)
        self.magnitude = 0.1 * math.log(factor) + 1.0


@POSITION_ENCODINGS.register("none")
class NoPosition(PositionEncoding):
    """No position encoding: a rope of zero rotated dimensions."""

    def __init__(self, ctx: BuildContext, head_dim: int):
        self.ctx = ctx
        self.head_dim = head_dim
        self.rotary_dim = 0
        self.interleaved = False
        self._inv = None

    @property
    def inv_freq(self) -> torch.Tensor:
        if self._inv is None:
            self._inv = torch.zeros(0, dtype=torch.float32, device=self.ctx.device)
        return self._inv
