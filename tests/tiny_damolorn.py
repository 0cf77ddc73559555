"""Tiny Damolorn configurations of the tests, and weights for them.

The three differ in every size and option: width, norm groups (1, 2, 3), convolution taps (1,
which keeps no state, 2 and 4), heads (1 to 10: more than one block of the attention kernel
serves), latent ranks that are no multiples of 32 and above 128, fewer rotated dimensions than the
rotated part has, the two mixer variants in either order, dense / routed / absent feed-forwards,
one chosen expert and all experts chosen, no loop, a loop from the first layer, a loop run once.

Weights are drawn wide (matrices of unit-order rows, gains around 1, convolution taps of order 1,
a router whose logits lie far apart) so that a wrong tap, pairing, gate or expert changes the
logits by far more than any tolerance.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from emberserve_b200.config.damolorn import DamolornConfig
from emberserve_b200.weights.safetensors_io import write_safetensors


def _mixer(heads, dim, rot_dim, rot_dims, vdim, kv_rank, q_rank, base):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "rot": {"base": base, "dims": rot_dims}, "scale": 1.0 / math.sqrt(dim + rot_dim)}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


DAM_A = {
    "architecture": "Damolorn", "vocab": 97, "width": 48, "norm": {"eps": 1e-5, "groups": 3},
    "canon": {"taps": 2}, "max_positions": 512,
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(3, 8, 8, 4, 12, 24, 16, 10000.0),
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "latent_attention_2", "mixer": _mixer(2, 16, 4, 4, 6, 36, 20, 300.0), "mlp": _moe(24, 5, 2)},
        {"type": "latent_attention", "mixer": _mixer(3, 8, 8, 8, 12, 24, 16, 50000.0), "mlp": None},
    ],
    "loop": {"start": 0, "stop": 2, "times": 3},
}

DAM_B = {
    "architecture": "Damolorn", "vocab": 130, "width": 64, "norm": {"eps": 3e-6, "groups": 1},
    "canon": {"taps": 4}, "max_positions": 512,
    "layers": [
        {"type": "latent_attention_2", "mixer": _mixer(1, 12, 6, 6, 20, 40, 8, 1000.0), "mlp": _moe(16, 4, 1)},
        {"type": "latent_attention", "mixer": _mixer(5, 4, 12, 12, 8, 52, 28, 200000.0),
         "mlp": {"kind": "dense", "ff": 72}},
    ],
}

DAM_C = {
    "architecture": "Damolorn", "vocab": 61, "width": 40, "norm": {"eps": 1e-4, "groups": 2},
    "canon": {"taps": 1}, "max_positions": 512,
    "layers": [
        {"type": "latent_attention_2", "mixer": _mixer(10, 6, 2, 2, 4, 160, 12, 77.0), "mlp": _moe(8, 3, 3)},
        {"type": "latent_attention", "mixer": _mixer(2, 10, 10, 6, 14, 30, 30, 10000.0), "mlp": _moe(12, 6, 2)},
        {"type": "latent_attention_2", "mixer": _mixer(4, 8, 8, 8, 8, 16, 16, 5000.0),
         "mlp": {"kind": "dense", "ff": 24}},
    ],
    "loop": {"start": 1, "stop": 2, "times": 1},
}

ALL = {"dam_a": DAM_A, "dam_b": DAM_B, "dam_c": DAM_C}
SEEDS = {"dam_a": 10, "dam_b": 11, "dam_c": 12}
PAGE_SIZES = {"dam_a": 4, "dam_b": 16, "dam_c": 8}


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    """Every tensor of a model of this design, by the names the checkpoint uses."""
    w = cfg["width"]
    shapes: dict[str, tuple[int, ...]] = {"embed": (cfg["vocab"], w), "head": (cfg["vocab"], w), "final.norm": (w,)}
    if cfg.get("loop"):
        shapes["loop.step"] = (cfg["loop"]["times"], w)
    taps = (cfg.get("canon") or {}).get("taps", 0)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h, qh = m["heads"], m["dim"] + m["rot_dim"]
        shapes.update({p + "norm1": (w,), p + "norm1b": (w,),
                       p + "mix.dq": (m["q_rank"], w), p + "mix.dq.norm": (m["q_rank"],),
                       p + "mix.uq": (h * qh, m["q_rank"]), p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], w),
                       p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (h * m["dim"], m["kv_rank"]),
                       p + "mix.uv": (h * m["vdim"], m["kv_rank"]), p + "mix.o": (w, h * m["vdim"])})
        if L["type"] == "latent_attention":
            shapes[p + "mix.g"] = (h * m["vdim"], w)
        if taps:
            shapes[p + "canon1"] = (w, taps)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        shapes.update({p + "norm2": (w,), p + "norm2b": (w,)})
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.gate": (mlp["ff"], w), p + "mlp.up": (mlp["ff"], w), p + "mlp.down": (w, mlp["ff"])})
        else:
            ff = mlp["expert"]["ff"]
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], w)
            for e in range(mlp["router"]["experts"]):
                shapes.update({f"{p}mlp.e{e}.gate": (ff, w), f"{p}mlp.e{e}.up": (ff, w), f"{p}mlp.e{e}.down": (w, ff)})
    return shapes


def make_weights(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        if name.endswith("norm") or ".norm" in name and len(shape) == 1:
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif name.endswith("canon1"):
            t = 0.7 * torch.randn(shape, generator=gen)
        elif name.endswith("router"):
            t = 2.0 * torch.randn(shape, generator=gen)
        elif name in ("embed", "loop.step"):
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


def typed(cfg: dict) -> DamolornConfig:
    return DamolornConfig.from_dict(cfg)
