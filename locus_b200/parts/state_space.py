"""A selective state-space mixer in the form of Mamba-2 (state-space duality): a scalar decay per head and token.

With h the mixer's input, inner = heads * v_dim, N the state size and G groups, one projection gives
[z: inner | x: inner | B: G * N | C: G * N | dt: heads].  x, B and C together pass a causal convolution per channel
over the last ``taps`` tokens (zeros before a request's start), its bias and silu.  dt = softplus(dt + dt_bias).  Per
head (head a uses B and C of group a // (heads / G)) a state S [N, v_dim] is carried from token to token:

    S_t = exp(-exp(A_log) * dt) S_(t-1) + dt * B_t x_t^T,      y_t = S_t^T C_t + D x_t.

y (heads concatenated) is multiplied by silu(z), each of ``norm_groups`` equal parts of the row is divided by its root
mean square, the row is multiplied by a weight and projected by W_o.  The projection's result stays float32; the
convolution, dt, the decay, the recurrence and the norm are float32.  State per request: S [heads, N, v_dim] and the
convolution's last taps - 1 inputs [channels, taps - 1], in one slot.  The recurrence is ``kernels.gated_recurrence``
with keep = the decay, take = dt, k = B, q = C, v = x.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from .base import Mixer, StateSpec, TensorSource, register_mixer


class StateSpace(Mixer):
    can_overwrite = True

    def __init__(self, prefix: str, *, hidden: int, n_heads: int, v_dim: int, state: int, groups: int, taps: int,
                 norm_groups: int, eps: float, out_scale: float = 1.0, names: Optional[dict] = None) -> None:
        """``out_scale``: a factor on the mixer's output (a mixer that runs beside another one)."""
        super().__init__(prefix)
        if n_heads % groups:
            raise ValueError(f"state_space: {n_heads} heads are not a multiple of {groups} groups")
        if (n_heads * v_dim) % norm_groups:
            raise ValueError(f"state_space: {norm_groups} norm groups do not divide the inner width {n_heads * v_dim}")
        if state > K.RECURRENCE_MAX_DIM:
            raise ValueError(f"state_space: state size {state} exceeds {K.RECURRENCE_MAX_DIM}")
        if not (1 <= taps <= K.SSM_MAX_TAPS):
            raise ValueError(f"state_space: a convolution over {taps} tokens (at most {K.SSM_MAX_TAPS})")
        self.hidden, self.H, self.dv, self.N, self.G = int(hidden), int(n_heads), int(v_dim), int(state), int(groups)
        self.taps, self.parts, self.eps, self.out_scale = int(taps), int(norm_groups), float(eps), float(out_scale)
        self.inner = self.H * self.dv
        self.channels = self.inner + 2 * self.G * self.N
        self.used = 2 * self.inner + 2 * self.G * self.N + self.H
        self.width = -(-self.used // 8) * 8
        self.off_xbc, self.off_dt = self.inner, self.inner + self.channels
        self.conv_offset = self.H * self.N * self.dv
        self.names = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log",
                      "D": "D", "norm": "norm", "o": "o", **(names or {})}

    def param_shapes(self):
        return {"w_in": (self.width, self.hidden), "conv": (self.channels, self.taps), "conv_b": (self.channels,),
                "dt_bias": (self.H,), "a_log": (self.H,), "d_skip": (self.H,), "norm": (self.inner,),
                "w_o": (self.hidden, self.inner)}

    def sources(self):
        p, n = self.prefix, self.names
        return [TensorSource(f"{p}.{n['in']}", (self.used, self.hidden), "w_in", 0),
                TensorSource(f"{p}.{n['conv']}", (self.channels, self.taps), "conv"),
                TensorSource(f"{p}.{n['conv_bias']}", (self.channels,), "conv_b", 0, "bias"),
                TensorSource(f"{p}.{n['dt_bias']}", (self.H,), "dt_bias", 0, "bias"),
                TensorSource(f"{p}.{n['A_log']}", (self.H,), "a_log", 0, "bias"),
                TensorSource(f"{p}.{n['D']}", (self.H,), "d_skip", 0, "norm"),
                TensorSource(f"{p}.{n['norm']}", (self.inner,), "norm", 0, "norm"),
                TensorSource(f"{p}.{n['o']}", (self.hidden, self.inner), "w_o")]

    def kernel_modules(self, dtype):
        return ["gemm_simt", "gemv", "recurrence", "state_space"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def cache_needs(self):
        return None, StateSpec((self.conv_offset + self.channels * (self.taps - 1),), torch.float32)

    def bind(self, rt) -> None:
        self.params["w_in"][self.used:].zero_()
        self._scale = None
        if self.out_scale != 1.0:
            self._scale = rt.shared_object(("row_scale", self.out_scale), lambda: torch.full(
                (rt.max_tokens,), self.out_scale, dtype=torch.float32, device=rt.device))

    def forward(self, h, batch, cache, residual, rt, accumulate=True) -> None:
        self.finish(self.prepare(h, batch, cache, rt), residual, rt, accumulate)

    # The mixer in two steps, for a caller that runs it beside another mixer: everything up to the input of the output
    # projection touches only this mixer's own buffers and state; the projection writes (or adds into) ``residual``.
    def prepare(self, h, batch, cache, rt):
        T, H = batch.T, self.H
        proj = rt.rows("ssm.proj", self.width, torch.float32, T)
        K.linear(h, self.params["w_in"], proj)
        if cache.writes:
            state = cache.state
        else:
            state = rt.buf("ssm.state_copy", tuple(cache.state.shape), torch.float32)
            state.copy_(cache.state)
        qn = batch.host_seg_qn
        longest = max(qn) if qn else 0
        act = rt.rows("ssm.act", self.channels, torch.float32, T)
        keep = rt.rows("ssm.keep", H, torch.float32, T)
        take = rt.rows("ssm.take", H, torch.float32, T)
        K.ssm_conv(proj, self.off_xbc, self.off_dt, self.params["conv"], self.params["conv_b"], self.params["dt_bias"],
                   self.params["a_log"], state, self.conv_offset, batch.state_slots, batch.seg_q0, batch.seg_qn,
                   batch.n_seg, act, keep, take, n_heads=H, longest_new=longest)
        y = rt.rows("ssm.y", self.inner, torch.float32, T)
        short = not qn or min(qn) < K.RECURRENCE_CHUNK_FROM
        long = not qn or max(qn) >= K.RECURRENCE_CHUNK_FROM
        K.gated_recurrence(act, self.inner + self.G * self.N, act, self.inner, act, 0, keep, take, state, 0,
                           batch.state_slots, batch.seg_q0, batch.seg_qn, batch.n_seg, y, n_heads=H,
                           heads_per_group=H // self.G, dim=self.N, v_dim=self.dv, short=short, long=long,
                           longest_new=longest)
        o = rt.rows("ssm.o", self.inner, rt.dtype, T)
        K.ssm_out(y, act, proj, 0, self.params["d_skip"], self.params["norm"], self.eps, o, parts=self.parts, v_dim=self.dv)
        return o

    def finish(self, o, residual, rt, accumulate=True) -> None:
        K.linear(o, self.params["w_o"], residual, accumulate=accumulate, row_scale=self._scale)


register_mixer("state_space", StateSpace)
