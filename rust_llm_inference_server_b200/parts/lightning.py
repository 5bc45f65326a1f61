"""Linear attention with a per-head decay and a float32 state per request."""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..ops.profile import span
from .base import Mixer, StateSpec, register_mixer


class LightningAttention(Mixer):
    """q | k | v | gate come from one stacked projection; the recurrence S <- decay S + k v^T,
    o = S^T q runs in float32 over the step's tokens from the request's state slot; the heads'
    outputs are normed together, gated by sigmoid(W_g h) and projected."""

    graph_safe = True

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        if len(spec.decay) != spec.n_heads:
            raise ValueError(f"{len(spec.decay)} decay factors for {spec.n_heads} heads")
        self.eps = float(np.float32(spec.eps))
        self.decay = torch.tensor([float(g) for g in spec.decay], dtype=torch.float64).to(torch.float32).to(device)

    def tensors(self) -> dict:
        s = self.spec
        return {s.q_proj: (s.n_heads * s.dim, s.hidden), s.k_proj: (s.n_heads * s.dim, s.hidden),
                s.v_proj: (s.n_heads * s.v_dim, s.hidden), s.gate_proj: (s.n_heads * s.v_dim, s.hidden),
                s.out_norm: (s.n_heads * s.v_dim,), s.o_proj: (s.hidden, s.n_heads * s.v_dim)}

    def load(self, src) -> None:
        s = self.spec
        self.w_in = torch.cat([src.get(s.q_proj), src.get(s.k_proj), src.get(s.v_proj), src.get(s.gate_proj)],
                              dim=0).contiguous()
        self.out_norm = src.get(s.out_norm, "vector")
        self.w_o = src.get(s.o_proj).contiguous()

    def state_spec(self):
        s = self.spec
        return StateSpec((s.n_heads, s.v_dim, s.dim), torch.float32)     # S transposed: a column's entries are contiguous

    def forward(self, x, step, cache, state, writes_cache=True):
        s = self.spec
        T, H = x.shape[0], s.n_heads
        qk, hv = H * s.dim, H * s.v_dim
        with span("q|k|v|gate proj"):
            proj = ops.linear(x, self.w_in)
        o = step.buffer("lightning_o", (T, hv), torch.float32)
        with span("decayed recurrence"):
            ops.lightning_scan(proj, 0, qk, 2 * qk, o, state, self.decay, step, H, s.dim, s.v_dim)
        y = step.buffer("lightning_y", (T, hv), self.dtype)
        with span("norm * gate"):
            ops.act_norm(o, self.out_norm, self.eps, y, gate=proj[:, 2 * qk + hv:])
        with span("o proj"):
            return ops.linear(y, self.w_o)


register_mixer("lightning_attention", LightningAttention)
