"""A plain, slow implementation of the Rikolix decoder: one function per mechanism, whole sequences at once, float64.
It shares no code with the package: it reads ``config.json`` and the safetensors file itself and has no cache, no state
and no batches.

The model: x = embed[token] * scale.  A layer is x <- x + N1b(mixer(N1(x))), then x <- x + N2b(ff(N2(x))) where the layer
has a feed-forward; every N is an RMS norm whose stored weight w acts as (1 + w).  Two mixers, in an order the
configuration gives:

* ``attention``: grouped-query heads; the whole query projection (all heads at once) and the whole key projection go
  through an RMS norm with a plain weight of their full width; the first ``rot.dims`` entries of each query and key head
  turn by the position (neighbouring entries 2i, 2i + 1 are a pair); the value of position j turns by j over ALL of its
  entries, and a head's summed output at position i is turned back by i; the weight of a visible key is
  sigmoid(score * scale + b_head), not normalised over the keys.
* ``latent_attention``: queries through a normed latent of ``q_rank`` numbers; keys and values of all heads are linear maps
  of one normed latent of ``kv_rank`` numbers per token, plus one rotated key part of ``rot_dim`` numbers that all heads
  share; causal softmax.  A layer with ``kv_from: j`` makes no latent of its own: it reads the latents and rotated key parts
  that layer j made, through its own key and value maps.

Feed-forwards: dense, down(relu(up h)^2), or routed: softmax over router logits of (experts + identity) outputs, a
correction added to the scores for the choice only, the choice restricted to the best groups of neighbouring experts, the
``top`` best chosen, weighted by their uncorrected scores; the last ``identity`` router outputs stand for experts that return
their input.  Logits: the final norm, then the head matrix.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch

DT = torch.float64


# ---- reading a model folder ---------------------------------------------------------------------------------------
def read_model_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    weights = {}
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        index = json.loads(f.read(n))
        base = 8 + n
        kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
        for name, meta in index.items():
            if name == "__metadata__":
                continue
            a, b = meta["data_offsets"]
            f.seek(base + a)
            t = torch.frombuffer(bytearray(f.read(b - a)), dtype=kinds[meta["dtype"]]).reshape(meta["shape"])
            weights[name] = t.to(DT) if t.is_floating_point() else t
    return config, weights


# ---- small pieces ---------------------------------------------------------------------------------------------------
def rms_norm(x, eps, weight=None):
    y = x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def stream_norm(x, eps, stored):
    """The norms around the sublayers and the model's last norm: the stored weight lies around zero."""
    return rms_norm(x, eps, 1.0 + stored)


def turn_pairs(x, positions, base, dims, sign=1.0):
    """x [T, heads, n]: entries (2i, 2i + 1), i < dims/2, turn by sign * position * base^(-2i/dims); the rest stay."""
    if dims == 0:
        return x
    i = torch.arange(dims // 2, dtype=DT)
    angle = sign * positions.to(DT)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = angle.cos()[:, None, :], angle.sin()[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., dims:]], dim=-1)


def causal(T):
    return torch.ones(T, T, dtype=torch.bool).tril()


# ---- the mixers -----------------------------------------------------------------------------------------------------
def sigmoid_attention(h, w, p, m, eps):
    """h [T, D]; ``p`` the tensors' prefix ('l0.mix.'), ``m`` the mixer's entry of the configuration."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    positions = torch.arange(T)
    q = rms_norm(h @ w[p + "q"].T, eps, w[p + "q.norm"]).view(T, H, d)
    k = rms_norm(h @ w[p + "k"].T, eps, w[p + "k.norm"]).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    q, k = turn_pairs(q, positions, base, dims), turn_pairs(k, positions, base, dims)
    v = turn_pairs(v, positions, base, dv)
    out = torch.zeros(T, H, dv, dtype=DT)
    mask = causal(T)
    for head in range(H):
        g = head // (H // G)
        score = q[:, head] @ k[:, g].T * m["scale"] + w[p + "pb"][head]
        weight = torch.sigmoid(score) * mask
        out[:, head] = weight @ v[:, g]
    out = turn_pairs(out, positions, base, dv, sign=-1.0)
    return out.reshape(T, H * dv) @ w[p + "o"].T


def latent_of(h, w, p, m, eps):
    """(normed latent [T, kv_rank], rotated key part [T, rot_dim]) that a layer with a ``dkv`` matrix makes of its input."""
    T = h.shape[0]
    rank, rot = m["kv_rank"], m["rot_dim"]
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :rank], eps, w[p + "dkv.norm"])
    k_rot = turn_pairs(down[:, None, rank:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])[:, 0]
    return c, k_rot


def latent_attention(h, w, p, m, eps, shared=None):
    """``shared``: (latent, rotated key part) of another layer for a layer that makes none.  Returns (out, (latent, key part))."""
    T = h.shape[0]
    H, d, rot, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, k_rot = latent_of(h, w, p, m, eps) if shared is None else shared
    q = (rms_norm(h @ w[p + "dq"].T, eps, w[p + "dq.norm"]) @ w[p + "uq"].T).view(T, H, d + rot)
    q_plain = q[..., :d]
    q_rot = turn_pairs(q[..., d:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[p + "uk"].T).view(T, H, d)
    values = (c @ w[p + "uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=DT)
    mask = causal(T)
    for head in range(H):
        score = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * m["scale"]
        score = score.masked_fill(~mask, -math.inf)
        out[:, head] = torch.softmax(score, dim=-1) @ values[:, head]
    return out.reshape(T, H * dv) @ w[p + "o"].T, (c, k_rot)


# ---- the feed-forwards ------------------------------------------------------------------------------------------------
def squared_relu(z):
    return torch.relu(z) ** 2


def dense_feed_forward(h, w, p):
    return squared_relu(h @ w[p + "up"].T) @ w[p + "down"].T


def route(h, w, p, router):
    """(chosen [T, top] indices into experts + identity, weights [T, top], margin [T]): margin is how far the last chosen
    choice score lies above the best one left out (of the kept groups), for tests that must skip close calls."""
    experts, identity, top = router["experts"], router.get("identity", 0), router["top"]
    total = experts + identity
    score = torch.softmax(h @ w[p + "router"].T, dim=-1)                       # [T, total]
    choice = score + w[p + "correction"] if (p + "correction") in w else score.clone()
    groups = router.get("groups")
    if groups and groups["count"] > 1:
        count, keep = groups["count"], groups["keep"]
        best = choice.view(-1, count, total // count).max(dim=-1).values          # [T, count]
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        choice = choice.masked_fill(~kept.repeat_interleave(total // count, dim=1), -math.inf)
    ranked = choice.sort(dim=-1, descending=True, stable=True)
    chosen = ranked.indices[:, :top]
    margin = ranked.values[:, top - 1] - ranked.values[:, top] if total > top else torch.full((h.shape[0],), math.inf, dtype=DT)
    return chosen, score.gather(1, chosen), margin


def routed_feed_forward(h, w, p, mlp, margins=None):
    router = mlp["router"]
    experts = router["experts"]
    chosen, weights, margin = route(h, w, p, router)
    if margins is not None:
        margins.append(margin)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            if e >= experts:
                out[t] += a * h[t]                                           # an identity expert
            else:
                out[t] += a * (squared_relu(h[t] @ w[f"{p}e{e}.up"].T) @ w[f"{p}e{e}.down"].T)
    return out


# ---- the model --------------------------------------------------------------------------------------------------------
def forward_logits(config, weights, ids, after_layers=None, margins=None):
    """float64 logits [T, vocab] of the whole sequence ``ids``; ``after_layers`` (a list) receives x after every layer."""
    w = weights
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(ids, dtype=torch.long)] * config["embedding"]["scale"]
    kept = {}
    for i, spec in enumerate(config["layers"]):
        name = f"l{i}"
        h = stream_norm(x, eps, w[name + ".norm1"])
        m = spec["mixer"]
        if spec["type"] == "attention":
            mixed = sigmoid_attention(h, w, name + ".mix.", m, eps)
        elif spec["type"] == "latent_attention":
            source = m.get("kv_from")
            mixed, made = latent_attention(h, w, name + ".mix.", m, eps, shared=None if source is None else kept[source])
            if source is None:
                kept[i] = made
        else:
            raise ValueError(spec["type"])
        x = x + stream_norm(mixed, eps, w[name + ".norm1b"])
        mlp = spec.get("mlp")
        if mlp is not None:
            h = stream_norm(x, eps, w[name + ".norm2"])
            fed = dense_feed_forward(h, w, name + ".mlp.") if mlp["kind"] == "dense" else routed_feed_forward(h, w, name + ".mlp.", mlp, margins)
            x = x + stream_norm(fed, eps, w[name + ".norm2b"])
        if after_layers is not None:
            after_layers.append(x)
    return stream_norm(x, eps, w["final.norm"]) @ w["head"].T
