"""Small Guzuvik configurations and weights for the tests.  Tensor names and shapes are written down here from the
design, not taken from the package, so that a wrong name or shape in the package shows.

The cases differ from one another in every size and option: the order of the layers; layers with a dense
feed-forward, with experts and with none; key and value sizes that differ, that are no multiple of 16, that reach
128; as many kv heads as heads, and one; windows shorter and longer than a cache block, with no kept first tokens,
a few, and more than a block of them; a cap that bends most scores and one that bends few; layers that blend values
and layers that do not, the first blending layer not the first attention layer; state sizes that are no power of
two; one group and as many groups as heads; one norm group and several; convolutions of 1 to 4 taps; more than 32
experts, one expert a token, all experts a token; widths that are no multiple of 8.  Weights are scaled so that
attention is sharp (a missing or extra key changes the result) and the states' decays are close to 1 (what the first
tokens wrote still matters hundreds of tokens on).
"""
from __future__ import annotations

import json
import os

import numpy as np


def _attn(heads, kv, dim, vdim, size, keep, scale, cap, v_mix):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": size, "keep_first": keep},
            "scale": scale, "softcap": cap, "v_mix": v_mix}


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


CASE_MIXED = {
    "architecture": "Guzuvik", "vocab": 101, "width": 64, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 211, "mul_prev": 13, "mul_cur": 5}},
    "layers": [
        {"type": "attention", "mixer": _attn(4, 2, 16, 16, 40, 3, 0.6, 20.0, True), "mlp": _moe(6, 2, 24, 1.5)},
        {"type": "mamba2", "mixer": _ssm(3, 8, 16, 1, 3, 3), "mlp": {"kind": "dense", "ff": 72}},
        {"type": "attention", "mixer": _attn(6, 2, 32, 16, 90, 70, 0.3, 4.0, True), "mlp": None},
        {"type": "mamba2", "mixer": _ssm(4, 16, 8, 2, 4, 1), "mlp": _moe(6, 2, 24, 1.5)},
    ],
}

CASE_ODD = {
    "architecture": "Guzuvik", "vocab": 50, "width": 36, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 17, "mul_prev": 1, "mul_cur": 50}},
    "layers": [
        {"type": "mamba2", "mixer": _ssm(2, 20, 12, 2, 2, 2), "mlp": None},
        {"type": "attention", "mixer": _attn(3, 3, 24, 40, 70, 0, 0.25, 2.0, False), "mlp": _moe(40, 1, 12, 0.7)},
        {"type": "attention", "mixer": _attn(2, 1, 8, 24, 5, 2, 1.0, 30.0, True), "mlp": {"kind": "dense", "ff": 44}},
        {"type": "mamba2", "mixer": _ssm(1, 40, 5, 1, 1, 1), "mlp": {"kind": "dense", "ff": 20}},
        {"type": "attention", "mixer": _attn(4, 1, 16, 24, 64, 64, 0.5, 8.0, True), "mlp": _moe(3, 3, 16, 3.0)},
    ],
}

# heads of 128 and a width of 256: with prompts of more than 128 tokens the tiled tensor-core products run too
CASE_WIDE = {
    "architecture": "Guzuvik", "vocab": 300, "width": 256, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 509, "mul_prev": 7, "mul_cur": 3}},
    "layers": [
        {"type": "mamba2", "mixer": _ssm(4, 64, 128, 2, 4, 4), "mlp": _moe(8, 3, 64, 2.0)},
        {"type": "attention", "mixer": _attn(4, 2, 128, 128, 200, 5, 0.08, 50.0, True), "mlp": {"kind": "dense", "ff": 384}},
        {"type": "attention", "mixer": _attn(4, 2, 64, 128, 130, 66, 0.15, 50.0, True), "mlp": _moe(8, 3, 64, 2.0)},
    ],
}

CASES = {"mixed": (CASE_MIXED, 21), "odd": (CASE_ODD, 22), "wide": (CASE_WIDE, 23)}


def tensor_shapes(config: dict) -> dict:
    """{name: shape} of every tensor of a model of this configuration."""
    d = config["width"]
    shapes = {"embed": (config["vocab"], d), "bigram": (config["embedding"]["bigram"]["buckets"] + 1, d),
              "final.norm": (d,), "final.norm.b": (d,)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        norms = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer.get("mlp") else [])
        for n in norms:
            shapes[p + n] = (d,)
            shapes[p + n + ".b"] = (d,)
        q = p + "mix."
        if layer["type"] == "mamba2":
            H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = H * P, H * P + 2 * G * N
            shapes.update({q + "in": (inner + ch + H, d), q + "conv": (ch, taps), q + "conv.b": (ch,), q + "dt_bias": (H,),
                           q + "A_log": (H,), q + "D": (H,), q + "norm": (inner,), q + "o": (d, inner)})
        else:
            H, G, kd, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({q + "q": (H * kd, d), q + "q.b": (H * kd,), q + "k": (G * kd, d), q + "k.b": (G * kd,),
                           q + "v": (G * vd, d), q + "v.b": (G * vd,), q + "g": (H, d), q + "o": (d, H * vd)})
            if m.get("v_mix"):
                shapes[q + "vmix"] = ()
        mlp = layer.get("mlp")
        if mlp and mlp["kind"] == "dense":
            shapes.update({p + "mlp.up": (mlp["ff"], d), p + "mlp.down": (d, mlp["ff"])})
        elif mlp:
            n, f = mlp["router"]["experts"], mlp["expert"]["ff"]
            shapes.update({p + "mlp.router": (n, d), p + "mlp.router.b": (n,)})
            for e in range(n):
                shapes.update({f"{p}mlp.e{e}.gate": (f, d), f"{p}mlp.e{e}.up": (f, d), f"{p}mlp.e{e}.down": (d, f)})
    return shapes


def _bf16(x: np.ndarray) -> np.ndarray:
    """Rounded to bfloat16 (to nearest even) and back, so that file and oracle hold the same numbers."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return rounded.view(np.float32).reshape(np.shape(x))


def random_weights(config: dict, seed: int) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if name.endswith(".conv"):
            w = rng.normal(0.0, 0.6, shape)
        elif leaf == "A_log":
            w = rng.uniform(-4.0, -2.0, shape)     # decays of 0.9 to 0.99 a token
        elif leaf == "dt_bias":
            w = rng.normal(0.0, 1.0, shape)
        elif leaf == "D":
            w = rng.normal(1.0, 0.5, shape)
        elif leaf == "vmix":
            w = rng.uniform(0.2, 0.6, shape)
        elif leaf == "b":
            w = rng.normal(0.0, 0.5 if name.endswith("router.b") else 0.2, shape)
        elif len(shape) == 1:
            w = 1.0 + rng.normal(0.0, 0.1, shape)  # norm weights
        elif leaf in ("embed", "bigram"):
            w = rng.normal(0.0, 1.0 if leaf == "embed" else 0.5, shape)
        elif leaf == "router":
            w = rng.normal(0.0, 2.0 / np.sqrt(shape[1]), shape)
        elif leaf == "g":
            w = rng.normal(0.0, 2.0 / np.sqrt(shape[1]), shape)
        else:
            w = rng.normal(0.0, 1.0 / np.sqrt(shape[1]), shape)
        out[name] = _bf16(np.asarray(w, dtype=np.float32))
    return out


def write_folder(path: str, config: dict, weights: dict) -> str:
    """config.json and model.safetensors (bfloat16) in ``path``."""
    import torch
    from xeno_rt_b200.weights import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(config, fh)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      {k: torch.from_numpy(np.array(v, dtype=np.float32)).reshape(np.shape(v)).to(torch.bfloat16)
                       for k, v in weights.items()})
    return path


def make_case(tmp_path, name: str):
    """(folder, config, weights) of a named case."""
    config, seed = CASES[name]
    weights = random_weights(config, seed)
    return write_folder(os.path.join(str(tmp_path), name), config, weights), config, weights


def random_config(rng) -> dict:
    """A configuration drawn at random: any order of layers, any of the sizes and options the cases above use and
    more."""
    pick = lambda *values: values[int(rng.integers(len(values)))]
    width = pick(32, 36, 64, 96, 128, 200)
    blend_sizes = (pick(1, 2), pick(8, 16, 24, 32, 64))
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        if rng.random() < 0.5:
            heads, vdim = pick(1, 2, 3, 4, 6), pick(4, 8, 16, 20, 32)
            groups = pick(*[g for g in (1, 2, 3, heads) if heads % g == 0])
            norm_groups = pick(*[g for g in (1, 2, heads) if (heads * vdim) % g == 0])
            layer = {"type": "mamba2", "mixer": _ssm(heads, vdim, pick(4, 5, 12, 16, 32, 48, 64), groups, pick(1, 2, 3, 4),
                                                      norm_groups)}
        else:
            v_mix = bool(rng.random() < 0.6)
            kv, vdim = blend_sizes if v_mix else (pick(1, 2, 3), pick(8, 16, 24, 40, 64))
            heads = kv * pick(1, 2, 3, 4)
            dim = pick(8, 16, 24, 32, 48, 64, 128)
            layer = {"type": "attention",
                     "mixer": _attn(heads, kv, dim, vdim, pick(1, 5, 33, 64, 70, 130, 400), pick(0, 0, 1, 4, 64, 65, 100),
                                    float(pick(0.5, 1.0, 2.0, 4.0)) / np.sqrt(dim), pick(2.0, 10.0, 50.0), v_mix)}
        kind = pick("dense", "moe", None)
        if kind == "dense":
            layer["mlp"] = {"kind": "dense", "ff": pick(20, 44, 64, 136)}
        elif kind == "moe":
            experts = pick(2, 3, 8, 16, 40)
            layer["mlp"] = _moe(experts, pick(*[t for t in (1, 2, 3, experts) if t <= experts]), pick(8, 12, 32), pick(0.7, 2.0, 7.0))
        else:
            layer["mlp"] = None
        layers.append(layer)
    return {"architecture": "Guzuvik", "vocab": pick(50, 101, 256), "width": width, "norm": {"eps": pick(1e-5, 1e-6)},
            "embedding": {"bigram": {"buckets": pick(17, 211, 1009), "mul_prev": pick(1, 13, 29), "mul_cur": pick(5, 11, 50)}},
            "layers": layers}
