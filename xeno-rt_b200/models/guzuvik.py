"""Guzuvik: a decoder whose input is a token embedding plus a hashed embedding of the (previous, current) token pair,
and whose layers norm each sublayer before AND after it: x <- x + LN(mixer(LN(x))), then, where the layer has a
feed-forward, x <- x + LN(ff(LN(x))), with layer norms that carry a weight and a bias.  A layer's mixer is a
state-space recurrence with a scalar decay per head ("mamba2") or softmax attention without rotation ("attention":
biases on q, k, v; unit-RMS q and k; a tanh cap on the scores; a penalty that grows with the distance, head h losing
2^(-8 (h + 1) / heads) a position; a window that also keeps a sequence's first tokens; values blended with those of
the first blending layer; one sigmoid gate a head).  A feed-forward is dense with a squared relu, or a mixture of
small gated experts.  The logits are the final norm times the embedding table.

config.json keys: ``architecture`` "Guzuvik", ``vocab``, ``width``, ``norm.eps``, ``embedding.bigram`` (``buckets``,
``mul_prev``, ``mul_cur``), ``layers`` (a list of ``{"type", "mixer", "mlp"}``; ``mlp`` null, ``{"kind": "dense", "ff"}``
or ``{"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}}``), ``max_positions`` (optional).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from ..config import ModelConfig, register_architecture
from ..core import ConfigError
from ..parts import LayerSpec, ModelSpec, PartSpec, SchedulePlace
from .givopel import DEFAULT_MAX_POSITIONS, _positive, _positive_int

DISTANCE_RATE = 8.0    # head h's distance slope is 2^(-DISTANCE_RATE (h + 1) / heads)
EXPERT_ALPHA = 1.702   # an expert's gate is g * sigmoid(EXPERT_ALPHA g)


def _check_state_space(problems, where, m):
    heads = _positive_int(problems, where, m, "heads")
    groups = _positive_int(problems, where, m, "groups")
    vdim = _positive_int(problems, where, m, "vdim")
    norm_groups = _positive_int(problems, where, m, "norm_groups")
    for key in ("state", "conv"):
        _positive_int(problems, where, m, key)
    if heads % groups:
        problems.append(f"{where}: {heads} heads are not a multiple of {groups} groups")
    if (heads * vdim) % norm_groups:
        problems.append(f"{where}: {heads * vdim} inner channels are not a multiple of {norm_groups} norm_groups")


def _check_attention(problems, where, m):
    heads, kv = _positive_int(problems, where, m, "heads"), _positive_int(problems, where, m, "kv_heads")
    for key in ("dim", "vdim"):
        _positive_int(problems, where, m, key)
    for key in ("scale", "softcap"):
        _positive(problems, where, m, key)
    if heads % kv:
        problems.append(f"{where}: {heads} heads are not a multiple of {kv} kv_heads")
    mask = m.get("mask")
    if not isinstance(mask, dict):
        problems.append(f"{where}.mask must be an object with size and keep_first")
    else:
        _positive_int(problems, where + ".mask", mask, "size")
        keep = mask.get("keep_first")
        if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
            problems.append(f"{where}.mask.keep_first must be an integer >= 0, got {keep!r}")
    if not isinstance(m.get("v_mix", False), bool):
        problems.append(f"{where}.v_mix must be true or false")


def _check_mlp(problems, where, mlp):
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        problems.append(f"{where}.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} is not dense or moe")
    elif mlp["kind"] == "dense":
        _positive_int(problems, where, mlp, "ff")
    else:
        _positive_int(problems, where + ".expert", mlp.get("expert"), "ff")
        _positive(problems, where + ".expert", mlp.get("expert"), "limit")
        experts = _positive_int(problems, where + ".router", mlp.get("router"), "experts")
        top = _positive_int(problems, where + ".router", mlp.get("router"), "top")
        if top > experts:
            problems.append(f"{where}.router: top {top} exceeds the {experts} experts")


@dataclass(frozen=True)
class GuzuvikConfig(ModelConfig):
    architecture: str
    vocab: int
    width: int
    layers: tuple          # of dicts as config.json writes them (checked)
    norm_eps: float
    buckets: int
    mul_prev: int
    mul_cur: int
    max_positions: int
    eos_token_ids: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "GuzuvikConfig":
        problems: list[str] = []
        vocab = _positive_int(problems, "config", raw, "vocab")
        width = _positive_int(problems, "config", raw, "width")
        eps = _positive(problems, "norm", raw.get("norm"), "eps")
        pair = raw.get("embedding", {}).get("bigram") if isinstance(raw.get("embedding"), dict) else None
        buckets = _positive_int(problems, "embedding.bigram", pair, "buckets")
        muls = []
        for key in ("mul_prev", "mul_cur"):
            v = pair.get(key) if isinstance(pair, dict) else None
            if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                problems.append(f"embedding.bigram.{key} must be an integer >= 0, got {v!r}")
                v = 0
            muls.append(v)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            problems.append("'layers' must be a non-empty list")
            layers = []
        blended = None
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                problems.append(f"{where} must be an object with a 'mixer'")
                continue
            kind, m = layer.get("type"), layer["mixer"]
            if kind == "mamba2":
                _check_state_space(problems, where + ".mixer", m)
            elif kind == "attention":
                _check_attention(problems, where + ".mixer", m)
                if m.get("v_mix") is True:
                    sizes = (m.get("kv_heads"), m.get("vdim"))
                    if blended is not None and sizes != blended:
                        problems.append(f"{where}.mixer: layers that blend values must have the same kv_heads and vdim")
                    blended = blended or sizes
            else:
                problems.append(f"{where}.type {kind!r} is not one of mamba2, attention")
            if layer.get("mlp") is not None:
                _check_mlp(problems, where + ".mlp", layer["mlp"])
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
            problems.append(f"max_positions must be a positive integer, got {max_positions!r}")
        if problems:
            raise ConfigError("config.json: " + "; ".join(problems))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(architecture="Guzuvik", vocab=vocab, width=width, layers=tuple(copy.deepcopy(layers)), norm_eps=eps,
                   buckets=buckets, mul_prev=muls[0], mul_cur=muls[1], max_positions=max_positions, eos_token_ids=eos)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}},
               "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps}}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def _norm(width, eps, name):
    return PartSpec("layernorm", {"width": width, "eps": eps, "bias": True}, {"weight": name, "bias": name + ".b"})


def _state_space_spec(width, eps, m, prefix):
    params = {"width": width, "n_heads": m["heads"], "value_dim": m["vdim"], "state": m["state"], "n_groups": m["groups"],
              "taps": m["conv"], "norm_groups": m["norm_groups"], "eps": eps}
    names = {r: prefix + r for r in ("in", "conv", "dt_bias", "A_log", "D", "norm", "o")}
    names["conv_bias"] = prefix + "conv.b"
    return PartSpec("scalar_decay_state_space", params, names)


def _attention_spec(width, eps, m, prefix):
    params = {"width": width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
              "v_head_dim": m["vdim"], "qk_norm": "unit", "eps": eps, "window": m["mask"]["size"],
              "keep_first": m["mask"]["keep_first"], "scale": m["scale"], "softcap": m["softcap"],
              "distance_rate": DISTANCE_RATE, "bias": True, "gate": "sigmoid_head",
              "value_blend": "v_mix" if m.get("v_mix") else None, "position": {"kind": "none", "params": {}}}
    names = {r: prefix + r for r in ("q", "k", "v", "g", "o")}
    names.update({"q_bias": prefix + "q.b", "k_bias": prefix + "k.b", "v_bias": prefix + "v.b"})
    if m.get("v_mix"):
        names["blend"] = prefix + "vmix"
    return PartSpec("attention", params, names)


def _feed_forward_spec(width, mlp, prefix):
    if mlp["kind"] == "dense":
        return PartSpec("relu_squared", {"width": width, "inner": mlp["ff"]}, {"up": prefix + "up", "down": prefix + "down"})
    n = mlp["router"]["experts"]
    names = {"router": prefix + "router", "router_bias": prefix + "router.b"}
    for i in range(n):
        names.update({f"gate{i}": f"{prefix}e{i}.gate", f"up{i}": f"{prefix}e{i}.up", f"down{i}": f"{prefix}e{i}.down"})
    return PartSpec("routed_experts", {"width": width, "inner": mlp["expert"]["ff"], "experts": n,
                                       "top": mlp["router"]["top"], "limit": mlp["expert"]["limit"],
                                       "alpha": EXPERT_ALPHA}, names)


def build_spec(cfg: GuzuvikConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    layers, ignorable = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        mixer = (_state_space_spec if layer["type"] == "mamba2" else _attention_spec)(d, eps, m, p + "mix.")
        if layer["type"] == "attention" and not m.get("v_mix"):
            ignorable.append(p + "mix.vmix")
        parts = {"mixer_norm": ("norm", _norm(d, eps, p + "norm1")), "mixer": ("mixer", mixer),
                 "mixer_post": ("norm", _norm(d, eps, p + "norm1b"))}
        if layer.get("mlp"):
            parts.update({"ffn_norm": ("norm", _norm(d, eps, p + "norm2")),
                          "ffn": ("feed_forward", _feed_forward_spec(d, layer["mlp"], p + "mlp.")),
                          "ffn_post": ("norm", _norm(d, eps, p + "norm2b"))})
        else:
            ignorable += [p + n + s for n in ("norm2", "norm2b") for s in ("", ".b")]
        layers.append(LayerSpec(parts, "sandwich_residual"))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=d, max_positions=cfg.max_positions,
        embedding=PartSpec("token_pair", {"vocab_size": cfg.vocab, "width": d, "buckets": cfg.buckets,
                                          "mul_prev": cfg.mul_prev, "mul_cur": cfg.mul_cur},
                           {"weight": "embed", "pairs": "bigram"}),
        layers=layers, schedule=[SchedulePlace(i) for i in range(len(layers))],
        final_norm=_norm(d, eps, "final.norm"),
        lm_head=PartSpec("linear", {"vocab_size": cfg.vocab, "width": d}, {"weight": "embed"}),
        stop_ids=tuple(cfg.eos_token_ids), ignorable_tensors=tuple(ignorable))


register_architecture("Guzuvik", GuzuvikConfig, build_spec)
