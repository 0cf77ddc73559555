"""A plain, slow implementation of the Damolorn decoder: one function per mechanism, whole
sequences at once, dense masks, no cache and no batching.  It shares no code with the
package; the tests compare the engine with it.

Notation: a sequence is ``x[t, :]`` with positions t = 0, 1, ...; weights are ``[out, in]``
and act as ``x @ W.T``.  Everything is computed in the dtype the tensors are given in
(the tests use float64).
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# ---- reading a model folder ------------------------------------------------------------

def read_safetensors(path) -> dict[str, torch.Tensor]:
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = np.frombuffer(data[lo:hi], dtype=np.uint8)
        kind = info["dtype"]
        if kind == "BF16":
            u = buf.view(np.uint16).astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy())
        elif kind == "F32":
            t = torch.from_numpy(buf.view(np.float32).copy())
        elif kind == "I32":
            t = torch.from_numpy(buf.view(np.int32).copy())
        else:
            raise ValueError(kind)
        out[name] = t.reshape(info["shape"])
    return out


def read_model_dir(model_dir):
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    return cfg, read_safetensors(model_dir / "model.safetensors")


# ---- mechanisms ------------------------------------------------------------------------

def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def grouped_norm(x, w, groups, eps):
    """The width is cut into `groups` equal consecutive parts; each part is divided by its own
    root mean square; the whole is multiplied by w."""
    t, d = x.shape
    parts = x.reshape(t, groups, d // groups)
    return rms(parts, eps).reshape(t, d) * w


def causal_taps(h, w):
    """h + conv(h): conv(h)[t] = sum_j w[:, j] * h[t - taps + 1 + j], zeros before t = 0."""
    t, d = h.shape
    taps = w.shape[1]
    padded = torch.cat([h.new_zeros(taps - 1, d), h], 0)
    out = h.clone()
    for j in range(taps):
        out = out + w[:, j] * padded[j:j + t]
    return out


def rotate(x, base, dims, pairing, positions):
    """Rotary encoding of the first `dims` entries of the last axis of x[t, ..., :].
    pairing 'half': entry i goes with i + dims/2; 'interleaved': entry 2i with 2i + 1.
    The pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p f_i,
    f_i = base^(-2i/dims)."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(a).reshape(shape), torch.sin(a).reshape(shape)
    out = x.clone()
    if pairing == "half":
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    return out


def latent_attention(h, w, m, eps, pairing, gated):
    """The latent-attention mixer on a whole sequence h[t, width].  `w` maps the local names
    (dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o and g) to tensors, `m` is the mixer's sizes."""
    t = h.shape[0]
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(t)
    cq = rms(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).reshape(t, heads, dim + rot)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    kv = h @ w["dkv"].T
    c = rms(kv[:, :rank], eps) * w["dkv.norm"]
    k_rot = kv[:, rank:]  # one rotated key part, shared by the heads
    k_plain = (c @ w["uk"].T).reshape(t, heads, dim)
    v = (c @ w["uv"].T).reshape(t, heads, vdim)
    q_rot = rotate(q_rot, m["rot"]["base"], m["rot"]["dims"], pairing, pos)
    k_rot = rotate(k_rot, m["rot"]["base"], m["rot"]["dims"], pairing, pos)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain)
              + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    hidden = pos[None, :] > pos[:, None]
    scores = scores.masked_fill(hidden[None], float("-inf"))
    p = torch.softmax(scores, -1)
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(t, heads * vdim)
    if gated:
        o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def dense_glu(h, w, act):
    return (act(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def routed_experts(h, w, experts, top):
    """softmax over all experts of the router's logits; the `top` largest are used, weighted
    with their scores as they are (not renormalised); experts are SiLU-gated feed-forwards."""
    s = torch.softmax(h @ w["router"].T, -1)
    val, idx = torch.topk(s, top, dim=-1)
    out = torch.zeros_like(h)
    for e in range(experts):
        we = {k: w[f"e{e}.{k}"] for k in ("gate", "up", "down")}
        y = dense_glu(h, we, torch.nn.functional.silu)
        weight = (val * (idx == e)).sum(-1, keepdim=True)
        out = out + weight * y
    return out


# ---- the model -------------------------------------------------------------------------

def _sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def layer_order(cfg):
    """Layer indices in the order they run, with the number of the pass that begins there
    (None where no pass begins)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["times"] < 1:
        return [(i, None) for i in range(n)]
    out = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            out.append((i, t if i == loop["start"] else None))
    out += [(i, None) for i in range(loop["stop"], n)]
    return out


def forward(cfg, weights, tokens, dtype=torch.float64, want_layers=False):
    """Logits [len(tokens), vocab] of one sequence (and, with `want_layers`, the stream after
    every layer run)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    emb = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = emb.clone()
    streams = []
    for i, begins in layer_order(cfg):
        if begins is not None:
            if begins > 0:
                x = x + emb
            x = x + w["loop.step"][begins]
        L = cfg["layers"][i]
        lw = _sub(w, f"l{i}.")
        h = grouped_norm(x, lw["norm1"], groups, eps)
        h = causal_taps(h, lw["canon1"])
        kind = L["type"]
        pairing = "half" if kind == "latent_attention" else "interleaved"
        a = latent_attention(h, _sub(lw, "mix."), L["mixer"], eps, pairing, gated=(kind == "latent_attention"))
        x = x + grouped_norm(a, lw["norm1b"], groups, eps)
        mlp = L.get("mlp")
        if mlp is not None:
            h = grouped_norm(x, lw["norm2"], groups, eps)
            mw = _sub(lw, "mlp.")
            if mlp["kind"] == "dense":
                f = dense_glu(h, mw, torch.relu)
            else:
                f = routed_experts(h, mw, mlp["router"]["experts"], mlp["router"]["top"])
            x = x + grouped_norm(f, lw["norm2b"], groups, eps)
        streams.append(x)
    logits = grouped_norm(x, w["final.norm"], groups, eps) @ w["head"].T
    if want_layers:
        return logits, torch.stack(streams)
    return logits
