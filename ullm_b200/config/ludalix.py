"""Typed configuration of the Ludalix decoder, read from the keys of its config.json, and its translation into a
ModelSpec.

The design: a scaled token embedding plus an added sinusoid of the position; a list of layers, each with one mixer
(`mlstm`: matrix memory with exponential gates and per-request state; `attention`: grouped-query attention without
rotation, with per-head query / key norms, a window that keeps the first tokens, and optionally the keys and values
of an earlier layer) and an optional feed-forward (`dense`: clamped gated; `moe`: routed experts whose weight
multiplies the expert's input); the norm sits on each sub-layer's output, which is added to a 32-bit residual
stream with a multiplier; a final norm and an output head.

config.json keys: architecture, vocab, width, residual_mult, embedding.scale, norm.eps, layers[] with type,
mixer{...}, mlp{...} | null.  Tensor names: embed, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*, final.norm, head.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .specs import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry

ARCHITECTURE = "Ludalix"
# constants the design fixes
SINUSOID_BASE = 10000.0
CLAMPED_ACT_ALPHA = 1.702


class LudalixConfigError(ValueError):
    pass


def _need(d: dict, key: str, where: str, kind=(int, float)):
    if not isinstance(d, dict) or key not in d:
        raise LudalixConfigError(f"config.json: {where} lacks {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise LudalixConfigError(f"config.json: {where}.{key} = {v!r} is not a number")
    return v


def _positive_int(d: dict, key: str, where: str) -> int:
    v = _need(d, key, where, (int,))
    if v <= 0:
        raise LudalixConfigError(f"config.json: {where}.{key} must be positive, got {v}")
    return v


@dataclass(frozen=True)
class LudalixLayer:
    type: str  # "mlstm" or "attention"
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None


@dataclass(frozen=True)
class LudalixConfig:
    vocab: int
    width: int
    residual_mult: float
    embedding_scale: float
    norm_eps: float
    layers: tuple[LudalixLayer, ...]
    dtype: str = "bfloat16"
    max_positions: int = 1 << 30  # positions are computed, not tabulated: the context is the engine's choice
    raw: dict[str, Any] = field(default_factory=dict, hash=False, compare=False)

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "LudalixConfig":
        vocab, width = _positive_int(d, "vocab", "the config"), _positive_int(d, "width", "the config")
        mult = float(_need(d, "residual_mult", "the config"))
        scale = float(_need(d.get("embedding"), "scale", "embedding"))
        eps = float(_need(d.get("norm"), "eps", "norm"))
        if eps <= 0:
            raise LudalixConfigError("config.json: norm.eps must be positive")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise LudalixConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            if not isinstance(L, dict) or L.get("type") not in ("mlstm", "attention"):
                raise LudalixConfigError(f"config.json: {where}.type must be 'mlstm' or 'attention'")
            mix = L.get("mixer")
            if not isinstance(mix, dict):
                raise LudalixConfigError(f"config.json: {where} lacks 'mixer'")
            for k in ("heads", "dim", "vdim"):
                _positive_int(mix, k, where + ".mixer")
            if L["type"] == "mlstm":
                if float(_need(mix, "gate_cap", where + ".mixer")) <= 0:
                    raise LudalixConfigError(f"config.json: {where}.mixer.gate_cap must be positive")
            else:
                G = _positive_int(mix, "kv_heads", where + ".mixer")
                if mix["heads"] % G:
                    raise LudalixConfigError(f"config.json: {where}.mixer.heads is no multiple of kv_heads")
                _need(mix, "scale", where + ".mixer")
                mask = mix.get("mask")
                _positive_int(mask, "size", where + ".mixer.mask")
                if _need(mask, "keep_first", where + ".mixer.mask", (int,)) < 0:
                    raise LudalixConfigError(f"config.json: {where}.mixer.mask.keep_first must not be negative")
                src = mix.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                        raise LudalixConfigError(f"config.json: {where}.mixer.kv_from must name an earlier layer")
                    other = raw_layers[src]
                    om = other.get("mixer", {}) if isinstance(other, dict) else {}
                    if other.get("type") != "attention" or om.get("kv_from") is not None:
                        raise LudalixConfigError(f"config.json: {where}.mixer.kv_from = {src}: that layer has no keys "
                                                 f"and values of its own")
                    if (om.get("kv_heads"), om.get("dim"), om.get("vdim")) != (G, mix["dim"], mix["vdim"]):
                        raise LudalixConfigError(f"config.json: {where}.mixer.kv_from = {src}: head counts or sizes differ")
            mlp = L.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    raise LudalixConfigError(f"config.json: {where}.mlp.kind must be 'dense' or 'moe'")
                if mlp["kind"] == "dense":
                    _positive_int(mlp, "ff", where + ".mlp")
                    if float(_need(mlp, "limit", where + ".mlp")) <= 0:
                        raise LudalixConfigError(f"config.json: {where}.mlp.limit must be positive")
                else:
                    _positive_int(mlp.get("expert"), "ff", where + ".mlp.expert")
                    E = _positive_int(mlp.get("router"), "experts", where + ".mlp.router")
                    top = _positive_int(mlp.get("router"), "top", where + ".mlp.router")
                    if top > E:
                        raise LudalixConfigError(f"config.json: {where}.mlp.router.top exceeds the experts")
            layers.append(LudalixLayer(L["type"], dict(mix), dict(mlp) if mlp is not None else None))
        dt = d.get("dtype", d.get("torch_dtype", "bfloat16"))
        dt = str(dt).replace("torch.", "")
        if dt not in ("bfloat16", "float32", "float16"):
            raise LudalixConfigError(f"Unsupported dtype {dt!r}")
        return LudalixConfig(vocab, width, mult, scale, eps, tuple(layers), dt, raw=dict(d))

    def to_dict(self) -> dict[str, Any]:
        return dict(self.raw)


def ludalix_model_spec(cfg: LudalixConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    bare = dict(param="")  # a norm's weight is named by its prefix alone
    layers, schedule = [], []
    for i, L in enumerate(cfg.layers):
        mix = L.mixer
        cache_of = None
        if L.type == "mlstm":
            mixer = MixerSpec("mlstm", dict(
                hidden_size=W, num_heads=mix["heads"], head_dim=mix["dim"], value_dim=mix["vdim"],
                gate_cap=float(mix["gate_cap"]), eps=eps,
                names=dict(q="q", k="k", v="v", gate="g", o="o", norm="norm", i="i", i_bias="i.b", f="f", f_bias="f.b")))
        else:
            cache_of = mix.get("kv_from")
            mixer = MixerSpec("paged_attention", dict(
                hidden_size=W, num_heads=mix["heads"], num_kv_heads=mix["kv_heads"], head_dim=mix["dim"],
                value_dim=mix["vdim"], qk_norm=NormSpec("rmsnorm", mix["dim"], eps, bare), position=None,
                window=int(mix["mask"]["size"]), keep_first=int(mix["mask"]["keep_first"]), scale=float(mix["scale"]),
                own_kv=cache_of is None,
                names=dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm")))
        ff = ff_norm = None
        if L.mlp is not None:
            ff_norm = NormSpec("rmsnorm", W, eps, bare)
            if L.mlp["kind"] == "dense":
                ff = FeedForwardSpec("gated_mlp", dict(
                    hidden_size=W, intermediate_size=L.mlp["ff"], activation="swiglu_clamped",
                    limit=float(L.mlp["limit"]), alpha=CLAMPED_ACT_ALPHA, names=dict(gate="gate", up="up", down="down")))
            else:
                ff = FeedForwardSpec("routed_experts", dict(
                    hidden_size=W, intermediate_size=L.mlp["expert"]["ff"], num_experts=L.mlp["router"]["experts"],
                    top=L.mlp["router"]["top"], activation="silu", scores="sigmoid", renormalize=False,
                    weight_on="input", names=dict(router="router", gate="e{}.gate", up="e{}.up", down="e{}.down")))
        layers.append(LayerSpec(
            block="outnorm_residual", mixer=mixer, feed_forward=ff, mixer_norm=NormSpec("rmsnorm", W, eps, bare),
            feed_forward_norm=ff_norm,
            names=dict(mixer="mix.", feed_forward="mlp.", mixer_norm="norm1", feed_forward_norm="norm2"),
            block_args=dict(residual_mult=cfg.residual_mult)))
        schedule.append(ScheduleEntry(i, cache_of))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab, layers=layers, schedule=schedule,
        final_norm=NormSpec("rmsnorm", W, eps, bare), tie_embeddings=False, max_positions=cfg.max_positions,
        dtype=cfg.dtype, embedding_name="embed", layer_name="l{}.", final_norm_name="final.norm", head_name="head",
        embedding_param="", head_param="", embedding_scale=cfg.embedding_scale,
        embedding_position=PositionSpec("sinusoid_added", rotary_dim=W, theta=SINUSOID_BASE), stream_dtype="float32")
