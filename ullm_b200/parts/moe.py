"""Routed feed-forward: a router picks `top` of `num_experts` small gated feed-forwards per token.

    z = W_router h (32-bit);  s = sigmoid(z) (or softmax over the experts);  the `top` largest s are chosen;
    weight c = s of the chosen (optionally renormalized to sum 1);
    y = sum over the chosen of  expert(c h)   (`weight_on` = "input")   or   c expert(h)   ("output"),
    expert(x) = W_down (act(W_gate x) * (W_up x)),  no biases.

The experts' matrices live stacked ([experts, 2 I, hidden] with gate rows on up rows, and [experts, hidden, I]);
the checkpoint's per-expert tensors are views of the stacks.  Nothing of the routing comes back to the host: the
(token, choice) pairs are grouped by expert on the device and a grouped product runs over the groups, so a decode
step with this feed-forward can be recorded into a CUDA graph.
"""

from __future__ import annotations

import torch

from ..csrc import kernels
from .base import FeedForward, ParamDecl
from .registry import register_feed_forward

_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int, activation: str = "silu",
                 scores: str = "sigmoid", renormalize: bool = False, weight_on: str = "output",
                 names: dict | None = None):
        """`names`: router, and per expert (format strings taking the expert's number) gate, up, down."""
        super().__init__()
        if activation not in _ACTIVATIONS:
            raise ValueError(f"activation {activation!r} unknown (have {sorted(_ACTIVATIONS)})")
        if scores not in ("sigmoid", "softmax") or weight_on not in ("input", "output"):
            raise ValueError("scores: 'sigmoid' or 'softmax'; weight_on: 'input' or 'output'")
        if not 0 < top <= num_experts or top > 16 or num_experts > 1024:
            raise ValueError(f"top={top} of {num_experts} experts: the kernels take top <= 16 and up to 1024 experts")
        self.H, self.I, self.E, self.top = hidden_size, intermediate_size, num_experts, top
        self.activation, self.scores, self.renormalize, self.weight_on = activation, scores, bool(renormalize), weight_on
        n = dict(router="router.weight", gate="experts.{}.gate_proj.weight", up="experts.{}.up_proj.weight",
                 down="experts.{}.down_proj.weight")
        n.update(names or {})
        self.names = n

    def param_decls(self):
        n = self.names
        d = {n["router"]: ParamDecl((self.E, self.H))}
        for e in range(self.E):
            d[n["gate"].format(e)] = ParamDecl((self.I, self.H))
            d[n["up"].format(e)] = ParamDecl((self.I, self.H))
            d[n["down"].format(e)] = ParamDecl((self.H, self.I))
        return d

    def materialize(self, make):
        n, E, I, H = self.names, self.E, self.I, self.H
        self.w_router = self.tensors[n["router"]] = make(n["router"], ParamDecl((E, H)))
        self.w_gate_up = make("experts.gate_up.weight", ParamDecl((E, 2 * I, H)))
        self.w_down = make("experts.down.weight", ParamDecl((E, H, I)))
        for e in range(E):
            self.tensors[n["gate"].format(e)] = self.w_gate_up[e, :I]
            self.tensors[n["up"].format(e)] = self.w_gate_up[e, I:]
            self.tensors[n["down"].format(e)] = self.w_down[e]

    def activation_elems(self):
        return self.top * (self.I + self.H) + self.H + self.E

    def forward(self, x, ctx):
        K = kernels()
        T, top, E = x.shape[0], self.top, self.E
        ws = ctx.workspace
        logits = ws.tokens("moe.logits", T, E, torch.float32)
        K.linear_f32_out(x, self.w_router, logits)
        choice = ws.tokens("moe.choice", T, top, torch.int32)
        weight = ws.tokens("moe.weight", T, top, torch.float32)
        K.moe_route(logits, choice, weight, top, self.scores == "softmax", self.renormalize)
        offsets = ws.get("moe.offsets", 1, E + 1, torch.int32)
        order = ws.tokens("moe.sorted", T, top, torch.int32)
        place = ws.tokens("moe.place", T, top, torch.int32)
        K.moe_arrange(choice, T * top, E, offsets, order, place)
        act = ws.tokens("moe.act", T * top, self.I, x.dtype) if top == 1 else ws.get("moe.act", T * top, self.I, x.dtype, reserve=ws.max_tokens * top)
        rows = ws.tokens("moe.rows", T * top, self.H, x.dtype) if top == 1 else ws.get("moe.rows", T * top, self.H, x.dtype, reserve=ws.max_tokens * top)
        on_input = self.weight_on == "input"
        K.moe_grouped_linear(x, self.w_gate_up, offsets, order, weight if on_input else None, act, top, True, True,
                             _ACTIVATIONS[self.activation])
        K.moe_grouped_linear(act, self.w_down, offsets, order, None, rows, top, False, False)
        out = ws.tokens("ffn.out", T, self.H, x.dtype)
        K.moe_combine(rows, place, None if on_input else weight, out, top)
        return out
