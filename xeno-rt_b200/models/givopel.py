"""Givopel: a decoder whose layers each add a mixer and a feed-forward that read ONE layer norm of the stream,
x <- x + mixer(h) + feed_forward(h).  A layer's mixer is a gated linear attention ("gla"), or two mixers side
by side ("parallel": softmax attention with blended rotary positions and an output gate, and a gated delta
rule with short convolutions), whose results are RMS-normed over the width and averaged.  A stretch of
layers (``loop``) runs several times in a row with the same weights and a cache of its own each time; every
pass begins by mixing the stream with the embedding output through one matrix.  The output is a layer norm,
the head matrix, a scale and a soft cap.

config.json keys: ``architecture`` "Givopel", ``vocab``, ``width``, ``norm.eps``, ``layers`` (a list of
``{"type", "mixer", "mlp"}``), ``loop`` (``start``, ``stop``, ``times``; optional), ``logit_scale``,
``logit_softcap`` (optional), ``max_positions`` (optional).  The ranks of the low-rank products are sizes of
tensors only: they are read from the model file's shapes at load, or from the optional keys ``decay_rank`` /
``gate_rank`` of a mixer where there is no file (random weights).
"""
from __future__ import annotations

import copy
import dataclasses
from dataclasses import dataclass

from ..config import ModelConfig, register_architecture
from ..core import ConfigError
from ..parts import LayerSpec, ModelSpec, PartSpec, SchedulePlace

DEFAULT_MAX_POSITIONS = 1 << 20  # the design has no table that grows with the positions; the cache's size is the limit


def _positive_int(problems, where, d, key):
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        problems.append(f"{where}.{key} must be a positive integer, got {v!r}")
        return 1
    return v


def _positive(problems, where, d, key):
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not v > 0:
        problems.append(f"{where}.{key} must be a positive number, got {v!r}")
        return 1.0
    return float(v)


def _check_attention(problems, where, m):
    heads, kv = _positive_int(problems, where, m, "heads"), _positive_int(problems, where, m, "kv_heads")
    dim = _positive_int(problems, where, m, "dim")
    _positive_int(problems, where, m, "vdim")
    _positive(problems, where, m, "scale")
    if heads % kv:
        problems.append(f"{where}: {heads} heads are not a multiple of {kv} kv_heads")
    rot = m.get("rot")
    if rot is not None:
        dims = _positive_int(problems, where + ".rot", rot, "dims")
        _positive(problems, where + ".rot", rot, "base")
        if dims % 2 or dims > dim:
            problems.append(f"{where}.rot.dims {dims} must be even and at most dim {dim}")
        scaling = rot.get("scaling")
        if scaling is not None:
            for key in ("factor", "original", "fast", "slow"):
                _positive(problems, where + ".rot.scaling", scaling, key)


def _check_delta(problems, where, m):
    heads, kv = _positive_int(problems, where, m, "heads"), _positive_int(problems, where, m, "kv_heads")
    for key in ("dim", "vdim", "conv"):
        _positive_int(problems, where, m, key)
    if heads % kv:
        problems.append(f"{where}: {heads} heads are not a multiple of {kv} kv_heads")


def _check_gla(problems, where, m):
    for key in ("heads", "dim", "vdim"):
        _positive_int(problems, where, m, key)
    _positive(problems, where, m, "tau")


@dataclass(frozen=True)
class GivopelConfig(ModelConfig):
    architecture: str
    vocab: int
    width: int
    layers: tuple          # of dicts as config.json writes them (checked)
    loop: tuple | None     # (start, stop, times)
    norm_eps: float
    logit_scale: float
    logit_softcap: float | None
    max_positions: int
    eos_token_ids: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "GivopelConfig":
        problems: list[str] = []
        vocab = _positive_int(problems, "config", raw, "vocab")
        width = _positive_int(problems, "config", raw, "width")
        eps = _positive(problems, "norm", raw.get("norm"), "eps")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            problems.append("'layers' must be a non-empty list")
            layers = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                problems.append(f"{where} must be an object with a 'mixer'")
                continue
            kind, m = layer.get("type"), layer["mixer"]
            if kind == "gla":
                _check_gla(problems, where + ".mixer", m)
            elif kind == "parallel":
                for side, check in (("left", _check_attention), ("right", _check_delta)):
                    if not isinstance(m.get(side), dict):
                        problems.append(f"{where}.mixer.{side} is missing")
                    else:
                        check(problems, f"{where}.mixer.{side}", m[side])
            else:
                problems.append(f"{where}.type {kind!r} is not one of gla, parallel")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    problems.append(f"{where}.mlp.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} is not dense")
                else:
                    _positive_int(problems, where + ".mlp", mlp, "ff")
        loop = raw.get("loop")
        if loop is not None:
            start, stop, times = loop.get("start"), loop.get("stop"), loop.get("times")
            ok = all(isinstance(v, int) and not isinstance(v, bool) for v in (start, stop, times))
            if not ok or not (0 <= start < stop <= len(layers)) or times < 1:
                problems.append(f"loop {loop!r} must give 0 <= start < stop <= {len(layers)} layers and times >= 1")
                loop = None
            else:
                loop = (start, stop, times)
        scale = raw.get("logit_scale", 1.0)
        if isinstance(scale, bool) or not isinstance(scale, (int, float)) or scale == 0:
            problems.append(f"logit_scale must be a number other than 0, got {scale!r}")
        cap = raw.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or not cap > 0):
            problems.append(f"logit_softcap must be a positive number, got {cap!r}")
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
            problems.append(f"max_positions must be a positive integer, got {max_positions!r}")
        if problems:
            raise ConfigError("config.json: " + "; ".join(problems))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(architecture="Givopel", vocab=vocab, width=width, layers=tuple(copy.deepcopy(layers)), loop=loop,
                   norm_eps=eps, logit_scale=float(scale), logit_softcap=None if cap is None else float(cap),
                   max_positions=max_positions, eos_token_ids=eos)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
               "logit_scale": self.logit_scale}
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    def with_tensor_shapes(self, shapes: dict) -> "GivopelConfig":
        """The same configuration with the sizes that only tensors give (the ranks of the low-rank products)
        taken from ``shapes`` ({tensor name: shape}) wherever the configuration does not name them."""
        layers = copy.deepcopy(list(self.layers))
        for i, layer in enumerate(layers):
            m = layer["mixer"]
            targets = [(m["right"], f"l{i}.mix.right.")] if layer["type"] == "parallel" else [(m, f"l{i}.mix.")]
            for target, prefix in targets:
                for key, tensor in (("decay_rank", "a1"), ("gate_rank", "g1")):
                    shape = shapes.get(prefix + tensor)
                    if key not in target and shape is not None and len(shape) == 2:
                        target[key] = int(shape[0])
        return dataclasses.replace(self, layers=tuple(layers))

    def order(self) -> list:
        """[(layer, whether a pass of the loop begins with it)] in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        order = [(i, False) for i in range(start)]
        for _ in range(times):
            order += [(i, i == start) for i in range(start, stop)]
        return order + [(i, False) for i in range(stop, n)]


def _rank(m: dict, key: str, where: str) -> int:
    if key not in m:
        raise ConfigError(f"{where}: {key} is not known: it is neither in the configuration nor in a model file's shapes")
    return int(m[key])


def _attention_spec(width: int, eps: float, m: dict, prefix: str):
    position = {"kind": "none", "params": {}}
    if m.get("rot"):
        rot = m["rot"]
        position = {"kind": "blended_rotary", "params": {"rope_dim": rot["dims"], "base": rot["base"],
                                                         "pairing": "interleaved", "scaling": rot.get("scaling")}}
    params = {"width": width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
              "v_head_dim": m["vdim"], "qk_norm": False, "eps": eps, "window": None, "scale": m["scale"],
              "gate": "sigmoid", "position": position}
    return "attention", params, {r: prefix + r for r in ("q", "k", "v", "g", "o")}


def _delta_spec(width: int, eps: float, m: dict, prefix: str):
    params = {"width": width, "n_heads": m["heads"], "n_qk_heads": m["kv_heads"], "key_dim": m["dim"],
              "value_dim": m["vdim"], "taps": m["conv"], "decay_rank": _rank(m, "decay_rank", prefix + "a1"),
              "gate_rank": _rank(m, "gate_rank", prefix + "g1"), "eps": eps}
    names = {r: prefix + r for r in ("q", "k", "v", "b", "A_log", "a1", "a2", "dt_bias", "g1", "g2", "norm", "o")}
    names.update({"q_conv": prefix + "q.conv", "k_conv": prefix + "k.conv", "v_conv": prefix + "v.conv"})
    return "gated_delta_rule", params, names


def build_spec(cfg: GivopelConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "gla":
            mixer = PartSpec("gated_linear_attention",
                             {"width": d, "n_heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
                              "decay_rank": _rank(m, "decay_rank", p + "mix.a1"), "tau": m["tau"], "eps": eps},
                             {**{r: p + "mix." + r for r in ("q", "k", "v", "g", "o", "norm", "a1", "a2")},
                              "a2_bias": p + "mix.a2.b"})
        else:
            branches, names = [], {}
            for side, make in (("left", _attention_spec), ("right", _delta_spec)):
                kind, params, own = make(d, eps, m[side], f"{p}mix.{side}.")
                branches.append({"name": side, "kind": kind, "params": params})
                names.update({f"{side}.{role}": tensor for role, tensor in own.items()})
                names[f"{side}.out"] = f"{p}mix.{side}.out"
            mixer = PartSpec("side_by_side", {"width": d, "eps": eps, "branches": branches}, names)
        parts = {"norm": ("norm", PartSpec("layernorm", {"width": d, "eps": eps}, {"weight": p + "norm1"})),
                 "mixer": ("mixer", mixer)}
        if layer.get("mlp"):
            parts["ffn"] = ("feed_forward", PartSpec("swiglu", {"width": d, "inner": layer["mlp"]["ff"]},
                                                    {r: p + "mlp." + r for r in ("gate", "up", "down")}))
        layers.append(LayerSpec(parts, "parallel_residual"))
    stream_parts = {}
    if cfg.loop is not None:
        stream_parts["loop_in"] = PartSpec("mix_with_embedding", {"width": d}, {"weight": "loop.in"})
    schedule = [SchedulePlace(i, before="loop_in" if first else None) for i, first in cfg.order()]
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=d, max_positions=cfg.max_positions,
        embedding=PartSpec("token", {"vocab_size": cfg.vocab, "width": d}, {"weight": "embed"}),
        layers=layers, schedule=schedule,
        final_norm=PartSpec("layernorm", {"width": d, "eps": eps}, {"weight": "final.norm"}),
        lm_head=PartSpec("linear", {"vocab_size": cfg.vocab, "width": d, "scale": cfg.logit_scale,
                                    "softcap": cfg.logit_softcap}, {"weight": "head"}),
        stop_ids=tuple(cfg.eos_token_ids), stream_parts=stream_parts)


register_architecture("Givopel", GivopelConfig, build_spec)
