"""Gated linear attention as a mixer with per-request state: a matrix memory per head whose rows decay, each key
channel at its own data-dependent rate.

Per head, with q = W_q h / sqrt(d), k = W_k h, v = W_v h and the decay's low-rank projection z = A2 (A1 h) + b
(laid out heads x d):

    alpha_t = sigmoid(z_t)^(1 / tau) = exp(logsigmoid(z_t) / tau)        decay per key channel
    S_t = diag(alpha_t) S_{t-1} + k_t v_t^T                              S_0 = 0
    o_t = S_t^T q_t

then each head's o is RMS-normed over its value size with a weight shared by the heads, the heads are
concatenated, multiplied by silu(W_g h) and projected by W_o.  Decays, state and the norm are 32-bit in every
engine dtype; z is a product with a 32-bit result.

The state (S of every head, `gla_state_floats` floats) is one row per request slot in the cache manager's state
rows; it is zeroed when a slot is handed out and carried from step to step.  One kernel runs the recurrence over
any mix of prompt portions and single tokens (csrc/gla.cu).
"""

from __future__ import annotations

import torch

from ..csrc import kernels
from .base import Mixer, ParamDecl, StateNeed
from .linear import linear
from .registry import register_mixer


def gla_state_floats(heads: int, dim: int, vdim: int) -> int:
    """S^T [heads, vdim, dim] (the layout of csrc/gla.cu)."""
    return heads * vdim * dim


@register_mixer("gla")
class GatedLinearAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, decay_rank: int, tau: float,
                 eps: float, names: dict | None = None):
        """`decay_rank`: the inner size of the decay's projection; `tau`: its temperature; `eps`: of the head norm.
        `names`: the checkpoint's names of q, k, v, gate, o, norm, a1, a2, a2_bias behind the mixer's prefix."""
        super().__init__()
        if min(hidden_size, num_heads, head_dim, value_dim, decay_rank) <= 0 or not tau > 0:
            raise ValueError("sizes and tau must be positive")
        if head_dim > 512:
            raise ValueError(f"head_dim={head_dim}: the recurrence kernel takes up to 512")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = hidden_size, num_heads, head_dim, value_dim
        self.decay_rank, self.tau, self.eps = decay_rank, float(tau), float(eps)
        n = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", gate="g_proj.weight", o="o_proj.weight",
                 norm="norm.weight", a1="a_proj.0.weight", a2="a_proj.1.weight", a2_bias="a_proj.1.bias")
        n.update(names or {})
        self.names = n
        self.qk_size = num_heads * head_dim
        self.v_size = num_heads * value_dim

    def param_decls(self):
        H, n, r = self.hidden_size, self.names, self.decay_rank
        return {
            n["q"]: ParamDecl((self.qk_size, H)), n["k"]: ParamDecl((self.qk_size, H)),
            n["v"]: ParamDecl((self.v_size, H)), n["gate"]: ParamDecl((self.v_size, H)),
            n["a1"]: ParamDecl((r, H)), n["a2"]: ParamDecl((self.qk_size, r)),
            n["a2_bias"]: ParamDecl((self.qk_size,), "bias32"),
            n["o"]: ParamDecl((H, self.v_size)), n["norm"]: ParamDecl((self.value_dim,), "norm"),
        }

    def materialize(self, make):
        H, n, qk, vs, r = self.hidden_size, self.names, self.qk_size, self.v_size, self.decay_rank
        # one product for q | k | v | output gate | the decay's inner projection
        self.w_in = make("in_proj.weight", ParamDecl((2 * qk + 2 * vs + r, H)))
        self.tensors[n["q"]] = self.w_in[:qk]
        self.tensors[n["k"]] = self.w_in[qk:2 * qk]
        self.tensors[n["v"]] = self.w_in[2 * qk:2 * qk + vs]
        self.tensors[n["gate"]] = self.w_in[2 * qk + vs:2 * qk + 2 * vs]
        self.tensors[n["a1"]] = self.w_in[2 * qk + 2 * vs:]
        for key, decl in ((n["a2"], ParamDecl((qk, r))), (n["a2_bias"], ParamDecl((qk,), "bias32")),
                          (n["o"], ParamDecl((H, vs))), (n["norm"], ParamDecl((self.value_dim,), "norm"))):
            self.tensors[key] = make(key, decl)

    def state_need(self):
        return StateNeed((gla_state_floats(self.num_heads, self.head_dim, self.value_dim),), torch.float32)

    def activation_elems(self):
        # the input product, z and o in 32-bit (two elements' worth each in a 16-bit engine), the gated o, the output
        return (2 * self.qk_size + 2 * self.v_size + self.decay_rank + 2 * self.qk_size + 3 * self.v_size
                + self.hidden_size)

    def forward(self, x, ctx, cache):
        K = kernels()
        T = x.shape[0]
        n, N, d, dv, qk, vs, r = self.names, self.num_heads, self.head_dim, self.value_dim, self.qk_size, self.v_size, self.decay_rank
        if cache.state is None:
            raise RuntimeError("the gated linear attention mixer was given no state rows")
        ws = ctx.workspace
        y = ws.tokens("gla.in", T, 2 * qk + 2 * vs + r, x.dtype)
        linear(x, self.w_in, y)
        z = ws.tokens("gla.z", T, qk, torch.float32)
        K.linear_f32_out(y[:, 2 * qk + 2 * vs:], self.tensors[n["a2"]], z)
        o = ws.tokens("gla.o", T, vs, torch.float32)
        K.gla_recurrence(y, 0, qk, 2 * qk, z, self.tensors[n["a2_bias"]], 1.0 / self.tau, d ** -0.5, cache.state,
                         ctx.cu_q, ctx.req_slots, ctx.token_req, o, ctx.num_requests, N, d, dv)
        gated = ws.tokens("gla.gated", T, vs, x.dtype)
        K.head_norm_gate(o, y[:, 2 * qk + vs:2 * qk + 2 * vs], self.tensors[n["norm"]], self.eps, gated, N, dv, silu=True)
        out = ws.tokens("mixer.out", T, self.hidden_size, x.dtype)
        linear(gated, self.tensors[n["o"]], out)
        return out
