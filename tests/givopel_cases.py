"""Small Givopel configurations and weights for the tests.  Tensor names and shapes are written down here
from the design, not taken from the package, so that a wrong name or shape in the package shows.

The cases differ from one another in every size and option: a loop in the middle, at the start or none;
layers with and without a feed-forward; key and value sizes that differ, that are no multiple of 16, that pass
128; rotation over a part of the head or all of it, with and without blended frequencies; fewer q/k heads than
heads in the delta rule; convolutions of 1 to 4 taps; widths and ranks that are no multiple of 8; with and
without a soft cap.  Weights are scaled so that attention is sharp (a missing or extra key changes the
result) and the states' decays are close to 1 (what the first tokens wrote still matters hundreds of tokens on).
"""
from __future__ import annotations

import json
import os

import numpy as np

CASE_LOOP_MIDDLE = {
    "architecture": "Givopel", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 1.7,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "gla", "mixer": {"heads": 3, "dim": 16, "vdim": 24, "tau": 5.0}, "mlp": {"kind": "dense", "ff": 72}},
        {"type": "parallel", "mixer": {
            "left": {"heads": 4, "kv_heads": 1, "dim": 32, "vdim": 16, "scale": 0.5,
                     "rot": {"base": 10000.0, "dims": 16,
                             "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}}},
            "right": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "conv": 4}},
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "parallel", "mixer": {
            "left": {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 40, "scale": 0.9},
            "right": {"heads": 2, "kv_heads": 1, "dim": 40, "vdim": 32, "conv": 2}},
         "mlp": None},
    ],
}
RANKS_LOOP_MIDDLE = {0: {"a1": 8}, 1: {"a1": 8, "g1": 16}, 2: {"a1": 16, "g1": 8}}

CASE_NO_LOOP = {
    "architecture": "Givopel", "vocab": 50, "width": 36, "norm": {"eps": 1e-6}, "logit_scale": 0.25,
    "logit_softcap": 5.0,
    "layers": [
        {"type": "parallel", "mixer": {
            "left": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 16, "scale": 0.7,
                     "rot": {"base": 100.0, "dims": 16}},
            "right": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 72, "conv": 1}},
         "mlp": {"kind": "dense", "ff": 44}},
        {"type": "gla", "mixer": {"heads": 1, "dim": 136, "vdim": 8, "tau": 1.0}, "mlp": None},
    ],
}
RANKS_NO_LOOP = {0: {"a1": 4, "g1": 4}, 1: {"a1": 12}}

# heads of 128 and a width of 256: with prompts of more than 128 tokens every tensor-core kernel of the
# library runs (tiled products, prompt attention on tcgen05, decode attention fed by TMA)
CASE_WIDE = {
    "architecture": "Givopel", "vocab": 300, "width": 256, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
    "logit_softcap": 20.0, "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [
        {"type": "parallel", "mixer": {
            "left": {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.2,
                     "rot": {"base": 50000.0, "dims": 64,
                             "scaling": {"factor": 8.0, "original": 128, "fast": 16.0, "slow": 1.0}}},
            "right": {"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 128, "conv": 3}},
         "mlp": {"kind": "dense", "ff": 256}},
        {"type": "gla", "mixer": {"heads": 4, "dim": 64, "vdim": 64, "tau": 16.0}, "mlp": {"kind": "dense", "ff": 384}},
    ],
}
RANKS_WIDE = {0: {"a1": 32, "g1": 16}, 1: {"a1": 16}}

CASES = {"loop-middle": (CASE_LOOP_MIDDLE, RANKS_LOOP_MIDDLE, 11), "no-loop": (CASE_NO_LOOP, RANKS_NO_LOOP, 12),
         "wide": (CASE_WIDE, RANKS_WIDE, 13)}


def tensor_shapes(config: dict, ranks: dict) -> dict:
    """{name: shape} of every tensor of a model of this configuration."""
    d = config["width"]
    shapes = {"embed": (config["vocab"], d), "final.norm": (d,), "head": (config["vocab"], d)}
    if config.get("loop"):
        shapes["loop.in"] = (d, 2 * d)
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (d,)
        if layer["type"] == "gla":
            H, kd, vd, r = m["heads"], m["dim"], m["vdim"], ranks[i]["a1"]
            shapes.update({p + "mix.q": (H * kd, d), p + "mix.k": (H * kd, d), p + "mix.v": (H * vd, d),
                           p + "mix.g": (H * vd, d), p + "mix.o": (d, H * vd), p + "mix.norm": (vd,),
                           p + "mix.a1": (r, d), p + "mix.a2": (H * kd, r), p + "mix.a2.b": (H * kd,)})
        else:
            a, b = m["left"], m["right"]
            q = p + "mix.left."
            shapes.update({q + "q": (a["heads"] * a["dim"], d), q + "k": (a["kv_heads"] * a["dim"], d),
                           q + "v": (a["kv_heads"] * a["vdim"], d), q + "g": (a["heads"] * a["vdim"], d),
                           q + "o": (d, a["heads"] * a["vdim"]), q + "out": (d,)})
            q = p + "mix.right."
            H, G, kd, vd, taps = b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"]
            ra, rg = ranks[i]["a1"], ranks[i]["g1"]
            shapes.update({q + "q": (G * kd, d), q + "q.conv": (G * kd, taps), q + "k": (G * kd, d),
                           q + "k.conv": (G * kd, taps), q + "v": (H * vd, d), q + "v.conv": (H * vd, taps),
                           q + "b": (H, d), q + "A_log": (H,), q + "norm": (vd,), q + "a1": (ra, d),
                           q + "a2": (H * kd, ra), q + "dt_bias": (H * kd,), q + "g1": (rg, d), q + "g2": (H * vd, rg),
                           q + "o": (d, H * vd), q + "out": (d,)})
        if layer.get("mlp"):
            f = layer["mlp"]["ff"]
            shapes.update({p + "mlp.gate": (f, d), p + "mlp.up": (f, d), p + "mlp.down": (d, f)})
    return shapes


def _bf16(x: np.ndarray) -> np.ndarray:
    """Rounded to bfloat16 (to nearest even) and back, so that file and oracle hold the same numbers."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return rounded.view(np.float32)


def random_weights(config: dict, ranks: dict, seed: int) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(config, ranks).items():
        leaf = name.split(".")[-1]
        if name.endswith(".conv"):
            w = rng.normal(0.0, 0.6, shape)
        elif name.endswith("a2.b"):
            w = rng.normal(2.0, 1.0, shape)        # sigmoid(.)^(1/tau) near 1: a long memory
        elif leaf == "A_log":
            w = rng.uniform(-4.0, -2.0, shape)     # decays of 0.9 to 0.99 a token
        elif leaf == "dt_bias":
            w = rng.normal(0.0, 1.0, shape)
        elif len(shape) == 1:
            w = 1.0 + rng.normal(0.0, 0.1, shape)  # norm weights
        elif leaf in ("q", "k") and ".left." in name:
            w = rng.normal(0.0, 1.2 / np.sqrt(shape[1]), shape)  # sharp attention
        elif leaf == "embed":
            w = rng.normal(0.0, 1.0, shape)
        elif leaf == "b":
            w = rng.normal(0.0, 3.0 / np.sqrt(shape[1]), shape)
        else:
            w = rng.normal(0.0, 1.0 / np.sqrt(shape[1]), shape)
        out[name] = _bf16(w.astype(np.float32))
    return out


def write_folder(path: str, config: dict, weights: dict) -> str:
    """config.json and model.safetensors (bfloat16) in ``path``."""
    import torch
    from xeno_rt_b200.weights import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(config, fh)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      {k: torch.from_numpy(np.ascontiguousarray(v)).to(torch.bfloat16) for k, v in weights.items()})
    return path


def make_case(tmp_path, name: str):
    """(folder, config, weights) of a named case."""
    config, ranks, seed = CASES[name]
    weights = random_weights(config, ranks, seed)
    return write_folder(os.path.join(str(tmp_path), name), config, weights), config, weights
