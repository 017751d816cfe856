"""A state-space mixer whose decay is ONE scalar per head and token ("state-space duality", Mamba-2).

One product of the input gives [z | x | B | C | dt]: a gate z and the values x (``n_heads`` heads of
``value_dim``), B and C (``n_groups`` groups of ``state``; head h reads group h // (n_heads / n_groups)) and one
raw step size a head.  x, B and C pass a short causal convolution per channel (with a bias) and silu.  Then, per head,

    dt_t = softplus(raw_t + dt_bias),   S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T,   y_t = S_t^T C_t + D x_t,

the heads side by side are multiplied by silu(z), RMS-normed in ``norm_groups`` equal stretches (each by its own
root mean square), multiplied by a weight, and the output product follows.  The state S (float32, zero when a slot
opens, kept [heads, value_dim, state]) and the convolution's last taps - 1 inputs are the sequence's state.  Step
sizes, decays, the state and the norm are 32-bit in both compute dtypes.
"""
from __future__ import annotations

import torch

from ..cache import StateNeed
from ..core import ConfigError, DType, torch_dtype
from ..csrc import ops
from .linear import linear
from .registry import register_part
from .state_mixers import _StateMixer, _vector


class ScalarDecayStateSpace(_StateMixer):
    """params: ``width``, ``n_heads``, ``value_dim``, ``state``, ``n_groups``, ``taps``, ``norm_groups``, ``eps``.
    weights: ``in`` [2 * inner + 2 * n_groups * state + n_heads, width] (inner = n_heads * value_dim), ``conv``
    [inner + 2 * n_groups * state, taps], ``conv_bias`` [the same channels], ``dt_bias``, ``A_log``, ``D`` [n_heads],
    ``norm`` [inner], ``o`` [width, inner]."""

    @classmethod
    def _sizes(cls, params):
        inner = int(params["n_heads"]) * int(params["value_dim"])
        return inner, int(params["n_groups"]) * int(params["state"])

    @classmethod
    def weight_shapes(cls, params):
        d, nh, taps = params["width"], params["n_heads"], params["taps"]
        inner, gn = cls._sizes(params)
        return {"in": ((2 * inner + 2 * gn + nh, d), "matrix"), "conv": ((inner + 2 * gn, taps), "vector"),
                "conv_bias": ((inner + 2 * gn,), "vector"), "dt_bias": ((nh,), "vector"), "A_log": ((nh,), "vector"),
                "D": ((nh,), "vector"), "norm": ((inner,), "vector"), "o": ((d, inner), "matrix")}

    def __init__(self, params, weights, dtype: DType, device):
        self.n_heads, self.value_dim, self.state, self.n_groups, self.taps, self.norm_groups = (
            int(params[k]) for k in ("n_heads", "value_dim", "state", "n_groups", "taps", "norm_groups"))
        self.eps = float(params["eps"])
        self.inner, self.gn = self._sizes(params)
        if self.n_heads % self.n_groups:
            raise ConfigError(f"{self.n_heads} heads are not a multiple of {self.n_groups} groups")
        if self.inner % self.norm_groups:
            raise ConfigError(f"{self.inner} inner channels are not a multiple of {self.norm_groups} norm groups")
        if not (1 <= self.taps <= 9):
            raise ConfigError(f"a short convolution of {self.taps} taps is outside 1 to 9")
        self.w_in, self.w_o = weights["in"], weights["o"]
        self.conv, self.conv_bias = _vector(weights["conv"]), _vector(weights["conv_bias"])
        self.dt_bias, self.a_log, self.d_skip = (_vector(weights[r]) for r in ("dt_bias", "A_log", "D"))
        self.norm = _vector(weights["norm"])
        self.channels = self.inner + 2 * self.gn
        self.act_dtype = torch_dtype(dtype)

    def cache_need(self):
        needs = [StateNeed((self.n_heads, self.value_dim, self.state), "float32")]
        if self.taps > 1:
            needs.append(StateNeed((self.taps - 1, self.channels), "float32"))
        return needs

    def heads_out(self, h, ctx, store, owns_cache=True):
        self._owning(owns_cache)
        n, inner, gn = h.shape[0], self.inner, self.gn
        p = linear(h, self.w_in, out_dtype=torch.float32)   # z | x | B | C | dt
        xbc = self._rows(ctx)((n, self.channels), dtype=torch.float32, device=h.device)
        conv_state = store[1].state if self.taps > 1 else None
        ops.short_conv(xbc, p[:, inner:], self.conv, conv_state, ctx.cu_seqlens, ctx.seq_slot, ctx.max_new, "silu",
                       bias=self.conv_bias)
        y = self._rows(ctx)((n, inner), dtype=torch.float32, device=h.device)
        ops.ssd_scan(y, xbc, xbc[:, inner:], xbc[:, inner + gn:], p[:, inner + self.channels:], self.dt_bias, self.a_log,
                     self.d_skip, store[0].state, ctx.cu_seqlens, ctx.seq_slot, self.n_heads, self.n_groups, self.state,
                     self.value_dim, max_new=ctx.max_new)
        out = torch.empty((n, inner), dtype=self.act_dtype, device=h.device)
        ops.gated_group_norm(out, y, p, self.norm, self.norm_groups, self.eps)
        return out


register_part("mixer", "scalar_decay_state_space", ScalarDecayStateSpace)
