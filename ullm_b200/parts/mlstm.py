"""Matrix memory with exponential gates (the mLSTM of xLSTM) as a mixer with per-request state.

Per head, with q = W_q h / sqrt(d), k = W_k h, v = W_v h and the gate projections a = W_i h + b_i, c = W_f h + b_f:

    i = cap tanh(a / cap)                 log input gate         (cap = `gate_cap`)
    f = logsigmoid(cap tanh(c / cap))     log forget gate
    m_t = max(f + m_{t-1}, i)             running maximum, m_0 = 0
    S_t = exp(f + m_{t-1} - m_t) S_{t-1} + exp(i - m_t) k v^T        (n_t alike with k alone; S_0 = 0, n_0 = 0)
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)

then each head's o is divided by its root mean square, the heads are concatenated, multiplied by a weight over all
heads and by sigmoid(W_g h), and projected by W_o.  Gates, state and the unit norm are 32-bit in every engine
dtype; the gate projections are a product of their own with a 32-bit result.

The state (S, n, m of every head, `Kernels.mlstm_state_floats` floats) is one row per request slot in the cache
manager's state rows; it is zeroed when a slot is handed out and carried from step to step.  One kernel runs the
recurrence over any mix of prompt portions and single tokens (csrc/mlstm.cu).
"""

from __future__ import annotations

import torch

from ..csrc import kernels
from .base import Mixer, ParamDecl, StateNeed
from .linear import linear
from .registry import register_mixer


def mlstm_state_floats(heads: int, dim: int, vdim: int) -> int:
    """S^T [heads, vdim, dim], n [heads, dim], m [heads] (the layout of csrc/mlstm.cu)."""
    return heads * vdim * dim + heads * dim + heads


@register_mixer("mlstm")
class MLSTM(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, gate_cap: float, eps: float,
                 names: dict | None = None):
        """`names`: the checkpoint's names of q, k, v, gate (the output gate's projection), o, norm, i, i_bias, f,
        f_bias behind the mixer's prefix."""
        super().__init__()
        if min(hidden_size, num_heads, head_dim, value_dim) <= 0 or gate_cap <= 0:
            raise ValueError("sizes and gate_cap must be positive")
        if head_dim > 512:
            raise ValueError(f"head_dim={head_dim}: the recurrence kernel takes up to 512")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = hidden_size, num_heads, head_dim, value_dim
        self.gate_cap, self.eps = float(gate_cap), float(eps)
        n = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", gate="gate_proj.weight", o="o_proj.weight",
                 norm="norm.weight", i="igate.weight", i_bias="igate.bias", f="fgate.weight", f_bias="fgate.bias")
        n.update(names or {})
        self.names = n
        self.qk_size = num_heads * head_dim
        self.v_size = num_heads * value_dim

    def param_decls(self):
        H, n, Hn = self.hidden_size, self.names, self.num_heads
        return {
            n["q"]: ParamDecl((self.qk_size, H)), n["k"]: ParamDecl((self.qk_size, H)),
            n["v"]: ParamDecl((self.v_size, H)), n["gate"]: ParamDecl((self.v_size, H)),
            n["o"]: ParamDecl((H, self.v_size)), n["norm"]: ParamDecl((self.v_size,), "norm"),
            n["i"]: ParamDecl((Hn, H)), n["i_bias"]: ParamDecl((Hn,), "bias32"),
            n["f"]: ParamDecl((Hn, H)), n["f_bias"]: ParamDecl((Hn,), "bias32"),
        }

    def materialize(self, make):
        H, n, Hn, qk, vs = self.hidden_size, self.names, self.num_heads, self.qk_size, self.v_size
        # one product for q | k | v | output gate, one (32-bit result) for the two gates of the recurrence
        self.w_qkvg = make("qkvg_proj.weight", ParamDecl((2 * qk + 2 * vs, H)))
        self.tensors[n["q"]] = self.w_qkvg[:qk]
        self.tensors[n["k"]] = self.w_qkvg[qk:2 * qk]
        self.tensors[n["v"]] = self.w_qkvg[2 * qk:2 * qk + vs]
        self.tensors[n["gate"]] = self.w_qkvg[2 * qk + vs:]
        self.w_if = make("if_gates.weight", ParamDecl((2 * Hn, H)))
        self.tensors[n["i"]] = self.w_if[:Hn]
        self.tensors[n["f"]] = self.w_if[Hn:]
        self.tensors[n["o"]] = make(n["o"], ParamDecl((H, vs)))
        self.tensors[n["norm"]] = make(n["norm"], ParamDecl((vs,), "norm"))
        self.tensors[n["i_bias"]] = make(n["i_bias"], ParamDecl((Hn,), "bias32"))
        self.tensors[n["f_bias"]] = make(n["f_bias"], ParamDecl((Hn,), "bias32"))

    def state_need(self):
        return StateNeed((mlstm_state_floats(self.num_heads, self.head_dim, self.value_dim),), torch.float32)

    def activation_elems(self):
        # q | k | v | g, the gates, o in 32-bit (two elements' worth in a 16-bit engine), the gated o, the output
        return 2 * self.qk_size + 2 * self.v_size + 2 * self.num_heads + 3 * self.v_size + self.hidden_size

    def output_projection(self):
        return None

    def forward(self, x, ctx, cache):
        K = kernels()
        T = x.shape[0]
        n, Hn, d, dv, qk, vs = self.names, self.num_heads, self.head_dim, self.value_dim, self.qk_size, self.v_size
        if cache.state is None:
            raise RuntimeError("the mLSTM mixer was given no state rows")
        ws = ctx.workspace
        qkvg = ws.tokens("mlstm.qkvg", T, 2 * qk + 2 * vs, x.dtype)
        linear(x, self.w_qkvg, qkvg)
        gates = ws.tokens("mlstm.gates", T, 2 * Hn, torch.float32)
        K.linear_f32_out(x, self.w_if, gates)
        o = ws.tokens("mlstm.o", T, vs, torch.float32)
        K.mlstm_recurrence(qkvg, 0, qk, 2 * qk, gates, self.tensors[n["i_bias"]], self.tensors[n["f_bias"]],
                           cache.state, ctx.cu_q, ctx.req_slots, ctx.token_req, o, ctx.num_requests, Hn, d, dv,
                           d ** -0.5, self.gate_cap)
        gated = ws.tokens("mlstm.gated", T, vs, x.dtype)
        K.mlstm_out_gate(o, qkvg[:, 2 * qk + vs:], self.tensors[n["norm"]], self.eps, gated, Hn, dv)
        out = ws.tokens("mixer.out", T, self.hidden_size, x.dtype)
        linear(gated, self.tensors[n["o"]], out)
        return out
