"""Plain, slow implementation of the Ludalix decoder: whole sequences, no
cache, one function for each mechanism.  It shares no code with the engine: it
takes a dict of tensors under the checkpoint's names and the config.json dict.

All arithmetic runs in the dtype of the tensors given (float64 in most tests).

The design, in this file's notation (x the residual stream [T, width], m the
residual multiplier, rms(a) = a / sqrt(mean(a^2) + eps)):

    x0       = table[ids] * scale + P,   P[p, 2i] = sin(p f_i), P[p, 2i+1] = cos(p f_i), f_i = 10000^(-2i/width)
    x       <- x + m * w1 * rms(mixer(x))
    x       <- x + m * w2 * rms(ff(x))           (layers that have a feed-forward)
    logits   = head (wf * rms(x))
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------
# small parts
# --------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * weight


def sinusoid(positions: torch.Tensor, width: int, dtype) -> torch.Tensor:
    """[len(positions), width]: even entries sines, odd entries cosines of position * 10000^(-2i/width)."""
    out = torch.zeros(len(positions), width, dtype=dtype)
    p = positions.to(dtype)
    for c in range(width):
        i = c // 2
        ang = p * (10000.0 ** (-2.0 * i / width))
        out[:, c] = torch.sin(ang) if c % 2 == 0 else torch.cos(ang)
    return out


def embed(ids, table: torch.Tensor, scale: float, first_position: int = 0) -> torch.Tensor:
    ids = torch.as_tensor(ids, dtype=torch.long)
    pos = torch.arange(first_position, first_position + len(ids))
    return table[ids] * scale + sinusoid(pos, table.shape[1], table.dtype)


# --------------------------------------------------------------------------
# mixer: matrix memory with exponential gates (mLSTM)
# --------------------------------------------------------------------------
def mlstm_gates(h, w, pre, cap: float):
    """(log input gate, log forget gate), each [T, heads]."""
    i_pre = h @ w[pre + "i"].T + w[pre + "i.b"]
    f_pre = h @ w[pre + "f"].T + w[pre + "f.b"]
    i = cap * torch.tanh(i_pre / cap)
    f = F.logsigmoid(cap * torch.tanh(f_pre / cap))
    return i, f


def mlstm_recurrence(q, k, v, i, f):
    """q, k [T, heads, d]; v [T, heads, dv]; i, f [T, heads] -> o [T, heads, dv], token by token from the zero
    state with the running maximum starting at 0."""
    T, Hn, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(Hn, d, dv, dtype=q.dtype)
    n = torch.zeros(Hn, d, dtype=q.dtype)
    m = torch.zeros(Hn, dtype=q.dtype)
    out = torch.zeros(T, Hn, dv, dtype=q.dtype)
    for t in range(T):
        m_new = torch.maximum(f[t] + m, i[t])
        keep = torch.exp(f[t] + m - m_new)
        take = torch.exp(i[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * (k[t][:, :, None] * v[t][:, None, :])
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    return out


def mlstm_mixer(h, w, pre, mix: dict, eps: float):
    T = h.shape[0]
    Hn, d, dv = mix["heads"], mix["dim"], mix["vdim"]
    q = (h @ w[pre + "q"].T).view(T, Hn, d) * d ** -0.5
    k = (h @ w[pre + "k"].T).view(T, Hn, d)
    v = (h @ w[pre + "v"].T).view(T, Hn, dv)
    i, f = mlstm_gates(h, w, pre, float(mix["gate_cap"]))
    o = mlstm_recurrence(q, k, v, i, f)
    o = unit_rms(o, eps).reshape(T, Hn * dv) * w[pre + "norm"]
    o = o * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


# --------------------------------------------------------------------------
# mixer: attention with a window that keeps the first tokens
# --------------------------------------------------------------------------
def visible(T: int, size: int, keep_first: int) -> torch.Tensor:
    """[T, T] bool: query row sees key column."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def attention_keys_values(h, w, pre, mix: dict, eps: float):
    T = h.shape[0]
    G, d, dv = mix["kv_heads"], mix["dim"], mix["vdim"]
    k = rms_norm((h @ w[pre + "k"].T).view(T, G, d), w[pre + "k.norm"], eps)
    v = (h @ w[pre + "v"].T).view(T, G, dv)
    return k, v


def attention_mixer(h, w, pre, mix: dict, eps: float, kv):
    """kv: (keys after their norm, values) of this layer or of the layer it borrows them from."""
    T = h.shape[0]
    Hn, G, d, dv = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]
    q = rms_norm((h @ w[pre + "q"].T).view(T, Hn, d), w[pre + "q.norm"], eps)
    k, v = kv
    see = visible(T, mix["mask"]["size"], mix["mask"]["keep_first"])
    out = torch.zeros(T, Hn, dv, dtype=h.dtype)
    for hd in range(Hn):
        g = hd // (Hn // G)
        s = (q[:, hd] @ k[:, g].T) * mix["scale"]
        s = s.masked_fill(~see, float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, Hn * dv) @ w[pre + "o"].T


# --------------------------------------------------------------------------
# feed-forwards
# --------------------------------------------------------------------------
def dense_ff(h, w, pre, limit: float):
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[pre + "down"].T


def router_choice(h, w, pre, top: int):
    """(scores of the chosen experts [T, top], their indices [T, top])."""
    s = torch.sigmoid(h @ w[pre + "router"].T)
    return torch.topk(s, top, dim=-1)


def expert_ff(x, w, pre):
    return (F.silu(x @ w[pre + "gate"].T) * (x @ w[pre + "up"].T)) @ w[pre + "down"].T


def moe_ff(h, w, pre, experts: int, top: int):
    score, index = router_choice(h, w, pre, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for s, e in zip(score[t], index[t]):
            out[t] += expert_ff(s * h[t], w, f"{pre}e{int(e)}.")
    return out


def feed_forward(h, w, pre, mlp: dict):
    if mlp["kind"] == "dense":
        return dense_ff(h, w, pre, float(mlp["limit"]))
    if mlp["kind"] == "moe":
        return moe_ff(h, w, pre, mlp["router"]["experts"], mlp["router"]["top"])
    raise ValueError(mlp["kind"])


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------
def forward_stream(ids, w, cfg):
    """The residual stream after every layer, [layers, T, width], for one whole sequence."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = embed(ids, w["embed"], cfg["embedding"]["scale"])
    kv = {}
    streams = []
    for l, layer in enumerate(cfg["layers"]):
        pre, mix = f"l{l}.mix.", layer["mixer"]
        if layer["type"] == "mlstm":
            a = mlstm_mixer(x, w, pre, mix, eps)
        elif layer["type"] == "attention":
            src = mix.get("kv_from")
            if src is None:
                kv[l] = attention_keys_values(x, w, pre, mix, eps)
                src = l
            a = attention_mixer(x, w, pre, mix, eps, kv[src])
        else:
            raise ValueError(layer["type"])
        x = x + mult * rms_norm(a, w[f"l{l}.norm1"], eps)
        if layer.get("mlp") is not None:
            y = feed_forward(x, w, f"l{l}.mlp.", layer["mlp"])
            x = x + mult * rms_norm(y, w[f"l{l}.norm2"], eps)
        streams.append(x)
    return torch.stack(streams)


def forward_logits(ids, w, cfg):
    x = forward_stream(ids, w, cfg)[-1]
    return rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T


def greedy_generate(prompt, w, cfg, n_new: int) -> list[int]:
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(torch.argmax(forward_logits(ids, w, cfg)[-1])))
    return ids[len(prompt):]


# --------------------------------------------------------------------------
# random models for the tests
# --------------------------------------------------------------------------
def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    W = cfg["width"]
    s: dict[str, tuple[int, ...]] = {"embed": (cfg["vocab"], W)}
    for l, layer in enumerate(cfg["layers"]):
        p, mix = f"l{l}.", layer["mixer"]
        s[p + "norm1"] = (W,)
        if layer["type"] == "mlstm":
            Hn, d, dv = mix["heads"], mix["dim"], mix["vdim"]
            s.update({p + "mix.q": (Hn * d, W), p + "mix.k": (Hn * d, W), p + "mix.v": (Hn * dv, W),
                      p + "mix.g": (Hn * dv, W), p + "mix.o": (W, Hn * dv), p + "mix.norm": (Hn * dv,),
                      p + "mix.i": (Hn, W), p + "mix.i.b": (Hn,), p + "mix.f": (Hn, W), p + "mix.f.b": (Hn,)})
        else:
            Hn, G, d, dv = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]
            s.update({p + "mix.q": (Hn * d, W), p + "mix.q.norm": (d,), p + "mix.o": (W, Hn * dv)})
            if mix.get("kv_from") is None:
                s.update({p + "mix.k": (G * d, W), p + "mix.v": (G * dv, W), p + "mix.k.norm": (d,)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        s[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            s.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                s.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
            s[p + "mlp.router"] = (mlp["router"]["experts"], W)
    s["final.norm"] = (W,)
    s["head"] = (cfg["vocab"], W)
    return s


def random_weights(cfg: dict, seed: int, dtype=torch.float32, std_scale: float = 1.0) -> dict[str, torch.Tensor]:
    """Matrices N(0, 1/fan_in) (times std_scale), norm weights around 1, gate biases spread so that both
    branches of the running maximum occur."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm1") or name.endswith("norm2") or name.endswith(".norm") or name == "final.norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(".b"):
            t = 2.0 * torch.randn(shape, generator=g) + (2.0 if name.endswith("f.b") else 0.0)
        elif name == "embed":
            t = torch.randn(shape, generator=g) / cfg["embedding"]["scale"]
        else:
            t = torch.randn(shape, generator=g) * std_scale / math.sqrt(shape[-1])
        w[name] = t.to(dtype)
    return w
