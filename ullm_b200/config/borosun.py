"""Typed configuration of the Borosun decoder, read from the keys of its config.json, and its translation into a
ModelSpec.

The design: a token embedding (also the output head); a list of layers, each with one mixer and an optional dense
feed-forward that read the SAME normed stream and are added to it together, each through a sigmoid gate of its
own, followed by a per-layer token input (a share of a second embedding table, gated by a projection of the
stream, projected back, unit-normed and added); a final norm and capped logits.  The residual stream is 32-bit.

Mixers: `attention` (causal grouped-query attention with a short convolution behind each projection, rotation
with frequencies rescaled by wavelength, softmax weights mixed across heads), `attention_2` (sliding window,
rotation, unit-RMS queries and keys, capped scores), `gla` (gated linear attention with a decay per key channel
and per-request state).  Attention layers that say `v_mix` blend their values with those of the first such layer.

config.json keys: architecture, vocab, width, logit_softcap, norm.eps, token_side.dim, layers[] with type,
mixer{...}, mlp{kind, ff} | null.  Tensor names: embed, side.embed, l<i>.norm1, l<i>.mix.*, l<i>.mlp.*,
l<i>.rg1(.b), l<i>.rg2(.b), l<i>.side.*, final.norm.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .specs import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry, TokenSideSpec

ARCHITECTURE = "Borosun"
MIXER_TYPES = ("attention", "attention_2", "gla")
DEFAULT_DECAY_RANK = 16


class BorosunConfigError(ValueError):
    pass


def _need(d, key: str, where: str, kind=(int, float)):
    if not isinstance(d, dict) or key not in d:
        raise BorosunConfigError(f"config.json: {where} lacks {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise BorosunConfigError(f"config.json: {where}.{key} = {v!r} is not a number")
    return v


def _positive_int(d, key: str, where: str) -> int:
    v = _need(d, key, where, (int,))
    if v <= 0:
        raise BorosunConfigError(f"config.json: {where}.{key} must be positive, got {v}")
    return v


def _positive(d, key: str, where: str) -> float:
    v = float(_need(d, key, where))
    if not v > 0:
        raise BorosunConfigError(f"config.json: {where}.{key} must be positive, got {v}")
    return v


def _check_rotation(mix: dict, where: str) -> None:
    rot = mix.get("rot")
    if rot is None:
        return
    dims = _positive_int(rot, "dims", where + ".rot")
    if dims % 2 or dims > mix["dim"]:
        raise BorosunConfigError(f"config.json: {where}.rot.dims must be even and at most dim")
    _positive(rot, "base", where + ".rot")
    sc = rot.get("scaling")
    if sc is not None:
        for k in ("factor", "low", "high", "original"):
            _positive(sc, k, where + ".rot.scaling")
        if not sc["high"] > sc["low"]:
            raise BorosunConfigError(f"config.json: {where}.rot.scaling.high must exceed low")


@dataclass(frozen=True)
class BorosunLayer:
    type: str
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None


@dataclass(frozen=True)
class BorosunConfig:
    vocab: int
    width: int
    norm_eps: float
    side_dim: int  # 0: no per-layer token input
    logit_softcap: float | None
    layers: tuple[BorosunLayer, ...]
    dtype: str = "bfloat16"
    max_positions: int = 1 << 30  # angles are computed, not tabulated: the context is the engine's choice
    raw: dict[str, Any] = field(default_factory=dict, hash=False, compare=False)

    @staticmethod
    def from_dict(d: dict[str, Any], shapes: dict[str, tuple] | None = None) -> "BorosunConfig":
        """`shapes`: {tensor name: shape} of the model's files, when there are any.  One size of the design is no
        config.json key: the inner size of a `gla` layer's decay projection, which is the first extent of
        `l<i>.mix.a1`.  Without files (random weights) it is the mixer's optional key `decay_rank`, else
        DEFAULT_DECAY_RANK."""
        vocab, width = _positive_int(d, "vocab", "the config"), _positive_int(d, "width", "the config")
        eps = _positive(d.get("norm"), "eps", "norm")
        side = d.get("token_side")
        side_dim = _positive_int(side, "dim", "token_side") if side is not None else 0
        cap = d.get("logit_softcap")
        if cap is not None:
            cap = _positive(d, "logit_softcap", "the config")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise BorosunConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        mixed_width = None
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            if not isinstance(L, dict) or L.get("type") not in MIXER_TYPES:
                raise BorosunConfigError(f"config.json: {where}.type must be one of {MIXER_TYPES}")
            mix = L.get("mixer")
            if not isinstance(mix, dict):
                raise BorosunConfigError(f"config.json: {where} lacks 'mixer'")
            for k in ("heads", "dim", "vdim"):
                _positive_int(mix, k, where + ".mixer")
            mix = dict(mix)
            if L["type"] == "gla":
                _positive(mix, "tau", where + ".mixer")
                name = f"l{i}.mix.a1"
                if shapes is not None and name in shapes:
                    if len(shapes[name]) != 2:
                        raise BorosunConfigError(f"{name} has shape {shapes[name]}, expected [rank, width]")
                    mix["decay_rank"] = int(shapes[name][0])
                elif "decay_rank" in mix:
                    _positive_int(mix, "decay_rank", where + ".mixer")
                else:
                    mix["decay_rank"] = DEFAULT_DECAY_RANK
            else:
                G = _positive_int(mix, "kv_heads", where + ".mixer")
                if mix["heads"] % G:
                    raise BorosunConfigError(f"config.json: {where}.mixer.heads is no multiple of kv_heads")
                _need(mix, "scale", where + ".mixer")
                _check_rotation(mix, where + ".mixer")
                if mix.get("conv") is not None and not 1 <= _positive_int(mix, "conv", where + ".mixer") <= 32:
                    raise BorosunConfigError(f"config.json: {where}.mixer.conv must be 1 to 32 taps")
                if mix.get("softcap") is not None:
                    _positive(mix, "softcap", where + ".mixer")
                if L["type"] == "attention_2":
                    _positive_int(mix.get("mask"), "size", where + ".mixer.mask")
                if mix.get("v_mix"):
                    w = G * mix["vdim"]
                    if mixed_width is not None and w != mixed_width:
                        raise BorosunConfigError(f"config.json: {where}.mixer: value mixing needs kv_heads x vdim = "
                                                 f"{mixed_width} as in the first layer that mixes, got {w}")
                    mixed_width = w
            mlp = L.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise BorosunConfigError(f"config.json: {where}.mlp.kind must be 'dense'")
                _positive_int(mlp, "ff", where + ".mlp")
            layers.append(BorosunLayer(L["type"], dict(mix), dict(mlp) if mlp is not None else None))
        dt = str(d.get("dtype", d.get("torch_dtype", "bfloat16"))).replace("torch.", "")
        if dt not in ("bfloat16", "float32", "float16"):
            raise BorosunConfigError(f"Unsupported dtype {dt!r}")
        return BorosunConfig(vocab, width, eps, side_dim, cap, tuple(layers), dt, raw=dict(d))

    def to_dict(self) -> dict[str, Any]:
        return dict(self.raw)


def _position(mix: dict) -> PositionSpec | None:
    rot = mix.get("rot")
    if rot is None:
        return None
    args = {"scaling": dict(rot["scaling"])} if rot.get("scaling") else {}
    return PositionSpec("rope_computed", rotary_dim=int(rot["dims"]), theta=float(rot["base"]), args=args)


def borosun_model_spec(cfg: BorosunConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    bare = dict(param="")  # a norm's weight is named by its prefix alone
    layers, schedule = [], []
    first_mixed = None  # the first layer whose values the later `v_mix` layers blend in
    for i, L in enumerate(cfg.layers):
        mix = L.mixer
        if L.type == "gla":
            mixer = MixerSpec("gla", dict(
                hidden_size=W, num_heads=mix["heads"], head_dim=mix["dim"], value_dim=mix["vdim"],
                decay_rank=int(mix["decay_rank"]), tau=float(mix["tau"]), eps=eps,
                names=dict(q="q", k="k", v="v", gate="g", o="o", norm="norm", a1="a1", a2="a2", a2_bias="a2.b")))
        else:
            value_mix = None
            if mix.get("v_mix"):
                value_mix = "first" if first_mixed is None else "mix"
                first_mixed = i if first_mixed is None else first_mixed
            common = dict(
                hidden_size=W, num_heads=mix["heads"], num_kv_heads=mix["kv_heads"], head_dim=mix["dim"],
                value_dim=mix["vdim"], position=_position(mix), scale=float(mix["scale"]), value_mix=value_mix,
                score_cap=float(mix["softcap"]) if mix.get("softcap") is not None else None,
                conv_taps=int(mix.get("conv") or 0), norm_eps=eps,
                names=dict(q="q", k="k", v="v", o="o", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", talk="talk",
                           vmix="vmix"))
            if L.type == "attention":
                mixer = MixerSpec("paged_attention", dict(common, talking_heads=True))
            else:
                mixer = MixerSpec("paged_attention", dict(common, window=int(mix["mask"]["size"]),
                                                          unit_norm_after_rotation=True))
        ff = None
        if L.mlp is not None:
            ff = FeedForwardSpec("gated_mlp", dict(hidden_size=W, intermediate_size=L.mlp["ff"], activation="gelu_tanh",
                                                   names=dict(gate="gate", up="up", down="down")))
        layers.append(LayerSpec(
            block="parallel_gated", mixer=mixer, feed_forward=ff, mixer_norm=NormSpec("rmsnorm", W, eps, bare),
            feed_forward_norm=None,
            names=dict(mixer="mix.", feed_forward="mlp.", mixer_norm="norm1", gate1="rg1", gate1_bias="rg1.b",
                       gate2="rg2", gate2_bias="rg2.b", side_gate="side.gate", side_proj="side.proj",
                       side_norm="side.norm"),
            block_args=dict(gated=True, side_dim=cfg.side_dim, side_index=i, eps=eps)))
        schedule.append(ScheduleEntry(i))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab, layers=layers, schedule=schedule,
        final_norm=NormSpec("rmsnorm", W, eps, bare), tie_embeddings=True, max_positions=cfg.max_positions,
        dtype=cfg.dtype, embedding_name="embed", layer_name="l{}.", final_norm_name="final.norm", head_name="head",
        embedding_param="", head_param="", stream_dtype="float32", logit_softcap=cfg.logit_softcap,
        token_side=TokenSideSpec("side.embed", cfg.side_dim, len(cfg.layers)) if cfg.side_dim else None)
