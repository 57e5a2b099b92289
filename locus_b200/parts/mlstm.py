"""mLSTM: a matrix memory with an exponential input gate and a sigmoid forget gate (the mLSTM cell of xLSTM).

Per token, with h the mixer's input: q = (W_q h) * dim^(-1/2), k = W_k h (heads x dim), v = W_v h (heads x v_dim),
and per head the gate pre-activations z_i = w_i . h + b_i, z_f = w_f . h + b_f, soft-capped:

    i = cap * tanh(z_i / cap),      f = logsigmoid(cap * tanh(z_f / cap)).

Per head a matrix S [dim, v_dim], a vector n [dim] and a running maximum m (all zero at a request's start) are
carried from token to token:

    m_t = max(f + m_(t-1), i);   S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T;   n_t likewise with k alone;
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6).

Every head's o is divided by its root mean square, the heads are concatenated, multiplied by a weight and by
sigmoid(W_g h), and projected by W_o.  The six projections are one product whose result stays float32, so
everything that enters the recurrence is float32.  n is kept as one more column of S (the column whose v is 1),
which makes the cell the gated linear recurrence of ``kernels.gated_recurrence`` between two small kernels: the
gates in front of it, division, norm and gate behind it.  State per request: [heads, dim, v_dim + 1] and m [heads].
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from .base import Mixer, StateSpec, TensorSource, register_mixer


class MLstm(Mixer):
    can_overwrite = True

    def __init__(self, prefix: str, *, hidden: int, n_heads: int, dim: int, v_dim: int, gate_cap: float, eps: float,
                 names: Optional[dict] = None) -> None:
        super().__init__(prefix)
        if dim > K.RECURRENCE_MAX_DIM:
            raise ValueError(f"mlstm: dim {dim} exceeds {K.RECURRENCE_MAX_DIM} (a lane keeps its rows of the state in registers)")
        if not gate_cap > 0:
            raise ValueError(f"mlstm: the gates' cap must be positive, got {gate_cap}")
        self.hidden, self.H, self.d, self.dv = int(hidden), int(n_heads), int(dim), int(v_dim)
        self.cap, self.eps = float(gate_cap), float(eps)
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "i": "i", "f": "f", "i_bias": "i.b", "f_bias": "f.b",
                      "norm": "norm", "o": "o", **(names or {})}
        qk, vv = self.H * self.d, self.H * self.dv
        # columns of the one projection: [q | k | v | g | z_i | z_f]
        self.off_k, self.off_v, self.off_g = qk, 2 * qk, 2 * qk + vv
        self.off_i, self.off_f = 2 * qk + 2 * vv, 2 * qk + 2 * vv + self.H
        self.used = 2 * qk + 2 * vv + 2 * self.H
        self.width = -(-self.used // 8) * 8   # rows of the stacked weight, padded so that every product kernel takes it
        self.m_offset = self.H * self.d * (self.dv + 1)

    def sources(self):
        p, n, qk, vv, D = self.prefix, self.names, self.H * self.d, self.H * self.dv, self.hidden
        return [TensorSource(f"{p}.{n['q']}", (qk, D), "w_all", 0),
                TensorSource(f"{p}.{n['k']}", (qk, D), "w_all", self.off_k),
                TensorSource(f"{p}.{n['v']}", (vv, D), "w_all", self.off_v),
                TensorSource(f"{p}.{n['g']}", (vv, D), "w_all", self.off_g),
                TensorSource(f"{p}.{n['i']}", (self.H, D), "w_all", self.off_i),
                TensorSource(f"{p}.{n['f']}", (self.H, D), "w_all", self.off_f),
                TensorSource(f"{p}.{n['i_bias']}", (self.H,), "b_gates", 0, "bias"),
                TensorSource(f"{p}.{n['f_bias']}", (self.H,), "b_gates", self.H, "bias"),
                TensorSource(f"{p}.{n['norm']}", (vv,), "norm", 0, "norm"),
                TensorSource(f"{p}.{n['o']}", (D, vv), "w_o")]

    def param_shapes(self):
        # the gates' biases are loaded as they are stored and widened to the product's bias in bind
        return {"w_all": (self.width, self.hidden), "b_gates": (2 * self.H,), "norm": (self.H * self.dv,),
                "w_o": (self.hidden, self.H * self.dv)}

    def kernel_modules(self, dtype):
        return ["gemm_simt", "gemv", "recurrence", "mlstm"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def cache_needs(self):
        return None, StateSpec((self.m_offset + self.H,), torch.float32)

    def bind(self, rt) -> None:
        # the product's bias: zero for q, k, v and the output gate, the stored biases for the two gates
        b = torch.zeros(self.width, dtype=torch.float32, device=rt.device)
        b[self.off_i:self.used] = self.params["b_gates"].float()
        self._bias = b
        self.params["w_all"][self.used:].zero_()

    def forward(self, h, batch, cache, residual, rt, accumulate=True) -> None:
        T, H = batch.T, self.H
        proj = rt.rows("mlstm.proj", self.width, torch.float32, T)
        K.linear(h, self.params["w_all"], proj, bias=self._bias)
        if cache.writes:
            state = cache.state
        else:
            # a call that reads another call's state must leave it as it found it
            state = rt.buf("mlstm.state_copy", tuple(cache.state.shape), torch.float32)
            state.copy_(cache.state)
        keep = rt.rows("mlstm.keep", H, torch.float32, T)
        take = rt.rows("mlstm.take", H, torch.float32, T)
        m_t = rt.rows("mlstm.m", H, torch.float32, T)
        K.mlstm_gates(proj, self.off_i, self.off_f, self.cap, state, self.m_offset, batch.state_slots, batch.seg_q0,
                      batch.seg_qn, batch.n_seg, keep, take, m_t, n_heads=H)
        o_raw = rt.rows("mlstm.o_raw", H * (self.dv + 1), torch.float32, T)
        qn = batch.host_seg_qn
        short = not qn or min(qn) < K.RECURRENCE_CHUNK_FROM
        long = not qn or max(qn) >= K.RECURRENCE_CHUNK_FROM
        K.gated_recurrence(proj, 0, proj, self.off_k, proj, self.off_v, keep, take, state, 0, batch.state_slots,
                           batch.seg_q0, batch.seg_qn, batch.n_seg, o_raw, n_heads=H, heads_per_group=1, dim=self.d,
                           v_dim=self.dv, ones=True, q_scale=self.d ** -0.5, short=short, long=long,
                           longest_new=max(qn) if qn else 0)
        o = rt.rows("mlstm.o", H * self.dv, rt.dtype, T)
        K.mlstm_out(o_raw, m_t, proj, self.off_g, self.params["norm"], self.eps, o, n_heads=H, v_dim=self.dv)
        K.linear(o, self.params["w_o"], residual, accumulate=accumulate)


register_mixer("mlstm", MLstm)
