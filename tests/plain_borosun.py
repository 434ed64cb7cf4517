"""A plain, slow implementation of the Borosun decoder, written from the design's equations: one function per
mechanism, whole sequences at once, no cache, no batching, nothing shared with the engine.  It runs on the CPU
in whatever floating type the weights are given in (tests use 64-bit).

`weights` maps tensor names to tensors; `config` is the dict of config.json.

Notation.  x [T, W]: the residual stream of one sequence; h: the normed stream a layer's sublayers read;
p = 0 .. T-1: positions.  Linear maps are stored [out, in] and applied as u W^T.
"""

from __future__ import annotations

import math

import torch


# -- small pieces -----------------------------------------------------------------------------------------
def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def short_conv(u, w):
    """Causal convolution over time on each channel: u [T, C], w [C, taps];
    y_t = sum_j w[:, j] u_(t - taps + 1 + j), where u is zero at negative times."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([u.new_zeros(taps - 1, C), u], 0)
    y = u.new_zeros(T, C)
    for j in range(taps):
        y = y + w[:, j] * padded[j:j + T]
    return y


def rotary_frequencies(dims, base, scaling=None, dtype=torch.float64):
    """f_i = base^(-2i / dims), i < dims / 2, optionally rescaled by wavelength: short waves stay, long waves are
    divided by `factor`, those between are blended."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / dims)
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f.tolist():
            wave = 2.0 * math.pi / fi
            if wave < orig / high:
                out.append(fi)
            elif wave > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wave - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=torch.float64)
    return f.to(dtype)


def rotate(u, positions, freqs):
    """u [T, heads, dim]; the first 2 * len(freqs) dimensions of each head are rotated, dimension i with
    dimension i + len(freqs); the rest pass."""
    half = freqs.numel()
    ang = positions.to(freqs.dtype)[:, None] * freqs[None, :]
    cos, sin = ang.cos()[:, None, :].to(u.dtype), ang.sin()[:, None, :].to(u.dtype)
    a, b, rest = u[..., :half], u[..., half:2 * half], u[..., 2 * half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], -1)


def visible(T, window=None):
    """mask[i, j]: may position i read position j?  Causal, and with a window only the last `window` positions."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if window is not None:
        m = m & (i - j < window)
    return m


def softmax_weights(q, k, scale, mask, softcap=None):
    """q [T, H, d], k [T, G, d] -> weights [H, T, T] (each query head reads key head h // (H / G))."""
    H, G = q.shape[1], k.shape[1]
    kk = k.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if softcap is not None:
        s = softcap * torch.tanh(s / softcap)
    s = s.masked_fill(~mask[None], float("-inf"))
    return torch.softmax(s, -1)


def apply_weights(p, v):
    """p [H, T, T], v [T, G, dv] -> [T, H * dv]; head h reads value head h // (H / G)."""
    H, G = p.shape[0], v.shape[1]
    vv = v.repeat_interleave(H // G, dim=1)
    return torch.einsum("hij,jhd->ihd", p, vv).reshape(p.shape[1], -1)


def mix_values(v, v_first, lam):
    return (1.0 - lam) * v + lam * v_first


# -- the three mixers -------------------------------------------------------------------------------------
def attention_conv_talk(h, m, w, pre, shared):
    """Causal attention with a short convolution behind each projection, scaled rotary frequencies, ordinary
    softmax, weights mixed across heads, optional value mixing."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[pre + "q"].T, h @ w[pre + "k"].T, h @ w[pre + "v"].T
    if m.get("conv"):
        q, k, v = (short_conv(u, w[pre + n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    pos = torch.arange(T)
    rot = m.get("rot")
    q, k = q.view(T, H, d), k.view(T, G, d)
    if rot:
        f = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"), h.dtype)
        q, k = rotate(q, pos, f), rotate(k, pos, f)
    v = _value_mix(v, m, w, pre, shared)
    p = softmax_weights(q, k, m["scale"], visible(T))
    p = torch.einsum("hg,gij->hij", w[pre + "talk"], p)
    return apply_weights(p, v.view(T, G, dv)) @ w[pre + "o"].T


def attention_window_capped(h, m, w, pre, shared, eps):
    """Sliding-window attention: rotation, then unit-RMS queries and keys, capped scores, ordinary softmax."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (h @ w[pre + "q"].T).view(T, H, d), (h @ w[pre + "k"].T).view(T, G, d), h @ w[pre + "v"].T
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        f = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"), h.dtype)
        q, k = rotate(q, pos, f), rotate(k, pos, f)
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    v = _value_mix(v, m, w, pre, shared)
    p = softmax_weights(q, k, m["scale"], visible(T, m["mask"]["size"]), m.get("softcap"))
    return apply_weights(p, v.view(T, G, dv)) @ w[pre + "o"].T


def _value_mix(v, m, w, pre, shared):
    if m.get("v_mix"):
        if "v_first" in shared:
            v = mix_values(v, shared["v_first"], w[pre + "vmix"])
        else:
            shared["v_first"] = v
    return v


def gla_decay(h, m, w, pre):
    """alpha [T, heads * dim] = sigmoid(z)^(1 / tau), z = (h A1^T) A2^T + b."""
    z = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    return torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"])


def gla_recurrence(q, k, v, alpha):
    """Per head: S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k, alpha [T, N, d]; v [T, N, dv]."""
    T, N, d = q.shape
    dv = v.shape[2]
    S = q.new_zeros(N, d, dv)
    out = q.new_zeros(T, N, dv)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("ndv,nd->nv", S, q[t])
    return out


def gla(h, m, w, pre, eps):
    T = h.shape[0]
    N, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(T, N, d) * d ** -0.5
    k = (h @ w[pre + "k"].T).view(T, N, d)
    v = (h @ w[pre + "v"].T).view(T, N, dv)
    alpha = gla_decay(h, m, w, pre).view(T, N, d)
    o = gla_recurrence(q, k, v, alpha)
    o = rms_norm(o, w[pre + "norm"], eps).reshape(T, N * dv)
    gate = h @ w[pre + "g"].T
    return (o * torch.nn.functional.silu(gate)) @ w[pre + "o"].T


# -- feed-forward, layer, model ---------------------------------------------------------------------------
def dense_ff(h, w, pre):
    return (gelu_tanh(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def residual_gate(h, w, name):
    return torch.sigmoid(h @ w[name].T + w[name + ".b"])


def token_side_input(x, tokens, i, side_dim, w, pre, eps):
    """x + unit_rms(P (gelu(G x) * e)) * n, e = the layer's share of the token's side embedding."""
    e = w["side.embed"][tokens][:, i * side_dim:(i + 1) * side_dim]
    g = gelu_tanh(x @ w[pre + "side.gate"].T) * e
    y = g @ w[pre + "side.proj"].T
    return x + rms_norm(y, w[pre + "side.norm"], eps)


def layer(x, tokens, i, L, config, w, shared):
    eps = config["norm"]["eps"]
    pre = f"l{i}."
    h = rms_norm(x, w[pre + "norm1"], eps)
    kind, m = L["type"], L["mixer"]
    if kind == "attention":
        a = attention_conv_talk(h, m, w, pre + "mix.", shared)
    elif kind == "attention_2":
        a = attention_window_capped(h, m, w, pre + "mix.", shared, eps)
    elif kind == "gla":
        a = gla(h, m, w, pre + "mix.", eps)
    else:
        raise ValueError(kind)
    y = residual_gate(h, w, pre + "rg1") * a
    if L.get("mlp") is not None:
        y = y + residual_gate(h, w, pre + "rg2") * dense_ff(h, w, pre + "mlp.")
    x = x + y
    side = config.get("token_side")
    if side:
        x = token_side_input(x, tokens, i, side["dim"], w, pre, eps)
    return x


def forward(config, w, tokens, return_layers=False):
    """tokens: a list of ids of ONE sequence.  Returns logits [T, vocab] (and the stream after every layer)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tokens]
    shared: dict = {}
    after = []
    for i, L in enumerate(config["layers"]):
        x = layer(x, tokens, i, L, config, w, shared)
        after.append(x)
    x = rms_norm(x, w["final.norm"], config["norm"]["eps"])
    logits = x @ w["embed"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(after)) if return_layers else logits


# -- tensor names, shapes and random weights of a configuration ---------------------------------------------
def tensor_shapes(config, decay_rank=5):
    """{name: shape} of every tensor a model of this configuration has."""
    W, V = config["width"], config["vocab"]
    out = {"embed": (V, W), "final.norm": (W,)}
    side = config.get("token_side")
    if side:
        out["side.embed"] = (V, len(config["layers"]) * side["dim"])
    for i, L in enumerate(config["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = (W,)
        out[p + "rg1"], out[p + "rg1.b"] = (W, W), (W,)
        if L["type"] == "gla":
            N, d, dv = m["heads"], m["dim"], m["vdim"]
            r = m.get("decay_rank", decay_rank)
            out.update({p + "mix.q": (N * d, W), p + "mix.k": (N * d, W), p + "mix.v": (N * dv, W),
                        p + "mix.g": (N * dv, W), p + "mix.o": (W, N * dv), p + "mix.norm": (dv,),
                        p + "mix.a1": (r, W), p + "mix.a2": (N * d, r), p + "mix.a2.b": (N * d,)})
        else:
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * dv, W),
                        p + "mix.o": (W, H * dv)})
            if m.get("conv"):
                out.update({p + "mix.q.conv": (H * d, m["conv"]), p + "mix.k.conv": (G * d, m["conv"]),
                            p + "mix.v.conv": (G * dv, m["conv"])})
            if L["type"] == "attention":
                out[p + "mix.talk"] = (H, H)
            if m.get("v_mix"):
                out[p + "mix.vmix"] = ()
        if L.get("mlp") is not None:
            F = L["mlp"]["ff"]
            out.update({p + "mlp.gate": (F, W), p + "mlp.up": (F, W), p + "mlp.down": (W, F),
                        p + "rg2": (W, W), p + "rg2.b": (W,)})
        if side:
            out.update({p + "side.gate": (side["dim"], W), p + "side.proj": (W, side["dim"]), p + "side.norm": (W,)})
    return out


def random_weights(config, seed=0, decay_rank=5):
    """32-bit tensors sized so that every mechanism matters: linear maps keep unit variance, norm weights scatter
    around one, the head mixer around the identity, decays near (but not at) one."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(config, decay_rank).items():
        t = torch.randn(shape, generator=g)
        if name.endswith(("norm1", ".norm", "final.norm")):
            t = 1.0 + 0.2 * t
        elif name.endswith("talk"):
            t = torch.eye(shape[0]) + 0.3 * t
        elif name.endswith("vmix"):
            t = 0.3 + 0.1 * t
        elif name.endswith("a2.b"):
            t = 2.0 + t
        elif name.endswith(".b"):
            t = 0.5 * t
        elif name.endswith(".conv"):
            t = 0.6 * t
        elif name == "embed":
            t = 3.0 * t / math.sqrt(shape[1])  # (logits of a few units: a cap of that order bends but does not flatten them)
        elif name == "side.embed":
            t = t
        elif len(shape) == 2:
            t = t / math.sqrt(shape[1])
        w[name] = t
    return w
