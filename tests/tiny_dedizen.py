"""Tiny Dedizen configurations of the tests, and weights for them.

The three differ in every size and option: width, vocabulary, layer order (each mixer first, last
and twice), layers without a feed-forward, query heads per key head (1, 2, 3, 5), head sizes, chunk
sizes that are no multiple of a page and larger than a prompt, rotation of a few or of all numbers
of a head, with and without YaRN scaling, one and several memory heads, value sizes beyond one
block of the memory kernel, block-diagonal gates of 1, 3 and 5 blocks, convolutions of 1 (no
state), 2 and 5 taps.

Weights are drawn wide (matrices of unit-order rows, gains around 1, biases, sinks and decay
parameters of order 1) so that a wrong tap, pairing, gate, sink or decay moves the logits by far
more than any tolerance.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from emberserve_b200.config.dedizen import DedizenConfig
from emberserve_b200.weights.safetensors_io import write_safetensors


def _left(heads, kv_heads, dim, chunk, rot_dims, base, scaling=None, scale=None):
    d = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": chunk},
         "scale": scale if scale is not None else 1.7 / math.sqrt(dim)}
    if rot_dims:
        d["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            d["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return d


def _right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _parallel(left, right, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _mlstm(heads, dim, vdim, cap, ff):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _rglru(width, blocks, conv, ff):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


DED_A = {
    "architecture": "Dedizen", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "max_positions": 512,
    "layers": [
        _rglru(36, 3, 2, 40),
        _parallel(_left(6, 2, 8, 5, 4, 100.0, (4.0, 16, 4.0, 1.0)), _right(3, 6, 10, (0.5, 0.9, 0.99)), None),
        _mlstm(3, 10, 6, 4.0, 56),
    ],
}

DED_B = {
    "architecture": "Dedizen", "vocab": 130, "width": 64, "norm": {"eps": 3e-6}, "max_positions": 512,
    "layers": [
        _mlstm(1, 20, 28, 15.0, None),
        _parallel(_left(4, 4, 16, 16, 16, 10000.0), _right(2, 12, 8, (0.8, 0.97)), 72),
        _rglru(40, 1, 1, 24),
        _parallel(_left(2, 1, 24, 400, 6, 50.0, (8.0, 32, 16.0, 2.0), 0.3), _right(5, 4, 4, (0.3, 0.6, 0.9, 0.95, 1.0)), 32),
    ],
}

DED_C = {
    "architecture": "Dedizen", "vocab": 61, "width": 40, "norm": {"eps": 1e-4}, "max_positions": 512,
    "layers": [
        _parallel(_left(5, 1, 8, 3, 0, 0.0), _right(1, 33, 70, (0.93,)), 24),
        _mlstm(4, 9, 65, 2.5, 16),
        _rglru(130, 5, 5, None),
        _rglru(24, 2, 3, 48),
    ],
}

ALL = {"ded_a": DED_A, "ded_b": DED_B, "ded_c": DED_C}
SEEDS = {"ded_a": 20, "ded_b": 21, "ded_c": 22}
PAGE_SIZES = {"ded_a": 4, "ded_b": 16, "ded_c": 8}


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    """Every tensor of a model of this design, by the names the checkpoint uses."""
    w = cfg["width"]
    shapes: dict[str, tuple[int, ...]] = {"embed": (cfg["vocab"], w), "final.norm": (w,)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        shapes[p + "norm1"] = (w,)
        if L["type"] == "parallel":
            a, r = m["left"], m["right"]
            q = p + "mix.left."
            shapes.update({q + "q": (a["heads"] * a["dim"], w), q + "q.b": (a["heads"] * a["dim"],),
                           q + "k": (a["kv_heads"] * a["dim"], w), q + "k.b": (a["kv_heads"] * a["dim"],),
                           q + "sink": (a["heads"],), q + "g": (a["heads"], w), q + "o": (w, a["heads"] * a["vdim"]),
                           q + "out": (w,)})
            q = p + "mix.right."
            shapes.update({q + "q": (r["heads"] * r["dim"], w), q + "k": (r["heads"] * r["dim"], w),
                           q + "v": (r["heads"] * r["vdim"], w), q + "g": (r["heads"] * r["vdim"], w),
                           q + "o": (w, r["heads"] * r["vdim"]), q + "norm": (r["heads"] * r["vdim"],),
                           q + "out": (w,)})
        elif L["type"] == "mlstm":
            q, h = p + "mix.", m["heads"]
            shapes.update({q + "q": (h * m["dim"], w), q + "k": (h * m["dim"], w), q + "v": (h * m["vdim"], w),
                           q + "g": (h * m["vdim"], w), q + "o": (w, h * m["vdim"]), q + "norm": (h * m["vdim"],),
                           q + "i": (h, w), q + "i.b": (h,), q + "f": (h, w), q + "f.b": (h,)})
        else:
            q, c, b = p + "mix.", m["width"], m["blocks"]
            shapes.update({q + "y": (c, w), q + "y.b": (c,), q + "x": (c, w), q + "x.b": (c,),
                           q + "conv": (c, m["conv"]), q + "conv.b": (c,), q + "ra": (b, c // b, c // b),
                           q + "ra.b": (b, c // b), q + "ri": (b, c // b, c // b), q + "ri.b": (b, c // b),
                           q + "lam": (c,), q + "o": (w, c)})
        if L.get("mlp") is not None:
            shapes.update({p + "norm2": (w,), p + "mlp.up": (L["mlp"]["ff"], w), p + "mlp.down": (w, L["mlp"]["ff"])})
    return shapes


def make_weights(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2", "out"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif last == "conv":
            t = 0.7 * torch.randn(shape, generator=gen)
        elif name.endswith("f.b"):
            t = 2.0 + torch.randn(shape, generator=gen)  # forget gates that keep most of the memory
        elif last == "lam":
            t = -2.0 + torch.randn(shape, generator=gen)
        elif last in ("b", "sink"):
            t = 0.5 * torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) * (1.5 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(cfg: dict, out_dir, seed: int, weights: dict[str, torch.Tensor] | None = None) -> Path:
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(out / "model.safetensors", weights if weights is not None else make_weights(cfg, seed))
    return out


def typed(cfg: dict) -> DedizenConfig:
    return DedizenConfig.from_dict(cfg)
