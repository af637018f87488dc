"""A plain, slow implementation of the Fedutar decoder: one function per mechanism, whole sequences at once, float64.
It shares no code with the package: it reads ``config.json`` and the safetensors file itself and has no cache, no state
and no batches.

The model: x = embed[token] * scale.  A layer is x <- x + N1b(mixer(N1(x))), then x <- x + N2b(ff(N2(x))) where the layer
has a feed-forward (every N an RMS norm with a weight).  The mixer is two mixers side by side that read the same rows:
softmax attention (grouped heads, normed queries and keys, no rotation, a query temperature that grows with the logarithm
of the position, an elementwise sigmoid gate on the concatenated heads) and retention (linear attention with one fixed
decay per head, rotated queries and keys, every head's output divided by its root mean square, a silu gate); the result is
a weighted sum of the two.  The feed-forward is dense (silu-gated, with biases) or routed (the top experts by router
logit, softmax over the chosen logits, experts with clamped gate and up products).  A span of layers may run several times
in a row with the same weights; each pass starts with x <- W_in [x; x0], x0 the embedding's output.  Logits come from the
embedding table, scaled and squashed by tanh.
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


def silu(z):
    return z * torch.sigmoid(z)


def rotate(x, positions, base, dims):
    """x [T, heads, dim]: the first ``dims`` entries of every head turn, entry i paired with i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=DT)
    angle = positions.to(DT)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = angle.cos()[:, None, :], angle.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position p."""
    return 1.0 + coef * torch.log(torch.div(positions + 1, every, rounding_mode="floor").to(DT) + 1.0)


# ---- the two mixers and their sum -------------------------------------------------------------------------------------
def softmax_attention(h, w, p, m, eps):
    """The left mixer.  h [T, D]; ``p`` the tensors' prefix ('l0.mix.left.'), ``m`` its entry of the configuration."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    q = rms_norm((h @ w[p + "q"].T).view(T, H, d), eps, w[p + "q.norm"])
    k = rms_norm((h @ w[p + "k"].T).view(T, G, d), eps, w[p + "k.norm"])
    v = (h @ w[p + "v"].T).view(T, G, dv)
    temp = m.get("q_temp")
    if temp:
        q = q * query_temperature(positions, temp["coef"], temp["every"])[:, None, None]
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    seen = positions[None, :] <= positions[:, None]
    scores = scores.masked_fill(~seen, float("-inf"))
    out = torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v).reshape(T, H * dv)
    return (out * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def retention(h, w, p, m, eps):
    """The right mixer, as the recurrence it is defined by: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    q = rotate((h @ w[p + "q"].T).view(T, H, d), positions, rot["base"], rot["dims"])
    k = rotate((h @ w[p + "k"].T).view(T, H, d), positions, rot["base"], rot["dims"]) * d ** -0.5
    v = (h @ w[p + "v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=DT)
    state = torch.zeros(H, d, dv, dtype=DT)
    rows = []
    for t in range(T):
        state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        rows.append(torch.einsum("hdv,hd->hv", state, q[t]))
    out = rms_norm(torch.stack(rows), eps).reshape(T, H * dv)
    return (out * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    return m["left_scale"] * softmax_attention(h, w, p + "left.", m["left"], eps) \
        + m["right_scale"] * retention(h, w, p + "right.", m["right"], eps)


# ---- feed-forwards ---------------------------------------------------------------------------------------------------
def dense_feed_forward(h, w, p):
    gate = h @ w[p + "gate"].T + w[p + "gate.b"]
    up = h @ w[p + "up"].T + w[p + "up.b"]
    return (silu(gate) * up) @ w[p + "down"].T + w[p + "down.b"]


def expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def routed_feed_forward(h, w, p, mlp, gaps=None):
    """``gaps`` (a list) receives, per token, the gap between the last chosen and the first rejected router logit."""
    experts, top, limit = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["limit"]
    logits = h @ w[p + "router"].T
    order = torch.sort(logits, dim=-1, descending=True, stable=True)
    chosen, best = order.indices[:, :top], order.values[:, :top]
    if gaps is not None and top < experts:
        gaps.append(order.values[:, top - 1] - order.values[:, top])
    share = torch.softmax(best, dim=-1)
    out = torch.zeros_like(h)
    for e in range(experts):
        rows, places = (chosen == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += share[rows, places][:, None] * expert(h[rows], w, f"{p}e{e}.", limit)
    return out


# ---- the model ---------------------------------------------------------------------------------------------------------
def layer_forward(x, w, i, spec, eps, gaps=None):
    name = f"l{i}"
    mixed = parallel_mixer(rms_norm(x, eps, w[name + ".norm1"]), w, name + ".mix.", spec["mixer"], eps)
    x = x + rms_norm(mixed, eps, w[name + ".norm1b"])
    mlp = spec.get("mlp")
    if mlp is not None:
        h = rms_norm(x, eps, w[name + ".norm2"])
        fed = dense_feed_forward(h, w, name + ".mlp.") if mlp["kind"] == "dense" else routed_feed_forward(h, w, name + ".mlp.", mlp, gaps)
        x = x + rms_norm(fed, eps, w[name + ".norm2b"])
    return x


def run_order(config):
    """[(layer, starts a pass)]: the layers in the order they run."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(count)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, count)]


def forward_logits(config, weights, ids, after_layers=None, gaps=None):
    """float64 logits [T, vocab] of the whole sequence ``ids``; ``after_layers`` (a list) receives x after every layer run."""
    w = weights
    eps = config["norm"]["eps"]
    x0 = w["embed"][torch.as_tensor(ids, dtype=torch.long)] * config["embedding"]["scale"]
    x = x0
    for i, first_of_pass in run_order(config):
        if first_of_pass:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        x = layer_forward(x, w, i, config["layers"][i], eps, gaps)
        if after_layers is not None:
            after_layers.append(x)
    logits = rms_norm(x, eps, w["final.norm"]) @ w["embed"].T * config.get("logit_scale", 1.0)
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
