"""Retention: linear attention with a fixed decay per head and no softmax or denominator.

Per token, with h the mixer's input: q = W_q h, k = (W_k h) * dim^(-1/2) (heads x dim), v = W_v h
(heads x v_dim), and per head a state S [dim, v_dim] that is carried from token to token:

    S_t = decay_h * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t.

Every head's o_t is divided by its root mean square (no weight), the heads are concatenated, multiplied
by silu(W_g h) and projected by W_o.  The state starts at zero, is float32, and lives in the request's
state slot; the four projections are one product whose result stays float32, so that everything that
enters the recurrence is float32.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import kernels as K
from .base import Mixer, StateSpec, TensorSource, register_mixer


class Retention(Mixer):
    can_overwrite = True

    def __init__(self, prefix: str, *, hidden: int, n_heads: int, dim: int, v_dim: int, decay: Sequence[float],
                 eps: float, names: Optional[dict] = None) -> None:
        super().__init__(prefix)
        if len(decay) != n_heads:
            raise ValueError(f"retention: {len(decay)} decays for {n_heads} heads")
        if dim > K.RETENTION_MAX_DIM:
            raise ValueError(f"retention: dim {dim} exceeds {K.RETENTION_MAX_DIM} (a lane keeps its rows of the "
                             "state in registers)")
        self.hidden, self.H, self.d, self.dv = int(hidden), int(n_heads), int(dim), int(v_dim)
        self.decay, self.eps = tuple(float(x) for x in decay), float(eps)
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", **(names or {})}
        self.width = 2 * self.H * self.d + 2 * self.H * self.dv

    def param_shapes(self):
        return {"w_qkvg": (self.width, self.hidden), "w_o": (self.hidden, self.H * self.dv)}

    def sources(self):
        p, n, qk, vv = self.prefix, self.names, self.H * self.d, self.H * self.dv
        return [TensorSource(f"{p}.{n['q']}", (qk, self.hidden), "w_qkvg", 0),
                TensorSource(f"{p}.{n['k']}", (qk, self.hidden), "w_qkvg", qk),
                TensorSource(f"{p}.{n['v']}", (vv, self.hidden), "w_qkvg", 2 * qk),
                TensorSource(f"{p}.{n['g']}", (vv, self.hidden), "w_qkvg", 2 * qk + vv),
                TensorSource(f"{p}.{n['o']}", (self.hidden, vv), "w_o")]

    def kernel_modules(self, dtype):
        return ["gemm_simt", "gemv", "retention"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def cache_needs(self):
        return None, StateSpec((self.H, self.d, self.dv), torch.float32)

    def bind(self, rt) -> None:
        self._decay = torch.tensor(self.decay, dtype=torch.float32, device=rt.device)

    def forward(self, h, batch, cache, residual, rt, accumulate=True) -> None:
        T = batch.T
        qkvg = rt.rows("retention.qkvg", self.width, torch.float32, T)
        K.linear(h, self.params["w_qkvg"], qkvg)
        o_raw = rt.rows("retention.o_raw", self.H * self.dv, torch.float32, T)
        if cache.writes:
            state = cache.state
        else:
            # a call that reads another call's state must leave it as it found it
            state = rt.buf("retention.state_copy", tuple(cache.state.shape), torch.float32)
            state.copy_(cache.state)
        qn = batch.host_seg_qn
        short = not qn or min(qn) < K.RETENTION_CHUNK_FROM
        long = not qn or max(qn) >= K.RETENTION_CHUNK_FROM
        K.retention_scan(qkvg, state, batch.state_slots, batch.seg_q0, batch.seg_qn, batch.n_seg, self._decay,
                         self.d ** -0.5, o_raw, n_heads=self.H, dim=self.d, v_dim=self.dv, short=short, long=long,
                         longest_new=max(qn) if qn else 0)
        o = rt.rows("retention.o", self.H * self.dv, rt.dtype, T)
        K.retention_gate_norm(o_raw, qkvg, 2 * self.H * self.d + self.H * self.dv, self.eps, o, n_heads=self.H,
                              v_dim=self.dv)
        K.linear(o, self.params["w_o"], residual, accumulate=accumulate)


register_mixer("retention", Retention)
