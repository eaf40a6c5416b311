"""A plain statement of the Korurax decoder: whole sequences, no cache, no batches, float64, one
function per mechanism.  It shares no code with the package and is slow on purpose.

The design: pre-norm layers (layer norm with a gain and no bias) whose sublayer outputs enter the
stream times a constant; behind every layer the stream becomes a learnt weighted sum of the embedding
and of all layer results so far; two mixers (grouped-query attention inside chunks of the sequence,
with a logarithmic distance penalty, a sink in the softmax and a sigmoid gate per head; attention over
a low-rank latent with a half-split rotated key part shared by the heads); two feed-forwards (a dense
clamped gated one, and a routed mixture of squared-relu experts whose weights are normalised sigmoid
scores); a final norm, the embedding as output head, and a tanh cap on the logits.
"""

import json
import math
import os

import torch

F = torch.float64


def read_model_folder(path):
    """(config dict, {name: float64 tensor})."""
    from safetensors.torch import load_file

    with open(os.path.join(path, "config.json"), "r", encoding="utf-8") as handle:
        cfg = json.load(handle)
    weights = {k: v.to(F) for k, v in load_file(os.path.join(path, "model.safetensors")).items()}
    return cfg, weights


# ------------------------------------------------------------------------------------------ norms

def layer_norm(x, w, eps):
    """``(x - mean) / sqrt(var + eps) * w`` over the last dimension; ``var`` is the mean squared deviation."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(dim=-1, keepdim=True) + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


# ------------------------------------------------------------------------------------------ rotation

def rotate_half_split(x, positions, base, dims):
    """Turns the first ``dims`` entries of the last dimension of ``x`` ``[T, ..., D]``: entry ``i`` with
    entry ``i + dims / 2`` by the angle ``p * base ** (-2i / dims)``; the rest passes unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=F)
    angle = positions.to(F)[:, None] * (base ** (-2.0 * i / dims))[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = angle.cos().reshape(shape), angle.sin().reshape(shape)
    out = x.clone()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


# ------------------------------------------------------------------------------------------ mixers

def chunk_visible(t, size):
    """``[T, T]`` bool: query ``i`` sees key ``j`` when ``j <= i`` and both lie in the same chunk of ``size``
    positions counted from the start of the sequence."""
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    return (j <= i) & (i // size == j // size)


def sink_softmax(scores, visible, sink):
    """Softmax over the visible keys of each row with one more term ``exp(sink)`` in the denominator."""
    s = scores.masked_fill(~visible, -math.inf)
    top = torch.maximum(s.max(dim=-1, keepdim=True).values, sink.reshape(-1, 1, 1).expand(s.shape[0], s.shape[1], 1))
    e = torch.exp(s - top)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink.reshape(-1, 1, 1) - top))


def attend(q, k, v, scale, r1=None, r2=None, sink=None, gate=None, chunk=None, window=None, start=0):
    """``q`` ``[Tq, H, D]`` are the queries of positions ``start .. start + Tq - 1``; ``k`` ``[T, G, D]`` and ``v``
    ``[T, G, Dv]`` the keys and values of positions ``0 .. T - 1``.  ``score = q . k * scale - r1 ln(1 + r2 (i -
    j))``; key ``j`` counts for query ``i`` when ``j <= i``, both lie in the same chunk and ``j > i - window``;
    the softmax has one more term ``exp(sink)`` without a value; the head's output is multiplied by ``gate``
    ``[Tq, H]``.  Returns ``[Tq, H, Dv]``."""
    tq, heads, _ = q.shape
    t, kv_heads, _ = k.shape
    group = heads // kv_heads
    out = torch.zeros(tq, heads, v.shape[2], dtype=F)
    for a in range(tq):
        i = start + a
        for h in range(heads):
            g = h // group
            js = [j for j in range(min(i + 1, t)) if (chunk is None or j // chunk == i // chunk)
                  and (window is None or j > i - window)]
            s = torch.stack([(q[a, h] * k[j, g]).sum() * scale for j in js])
            if r1 is not None:
                d = torch.tensor([float(i - j) for j in js], dtype=F)
                s = s - r1[h] * torch.log1p(r2[h] * d)
            top = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - top)
            denom = e.sum() + (torch.exp(sink[h] - top) if sink is not None else 0.0)
            o = sum(e[n] * v[j, g] for n, j in enumerate(js)) / denom
            out[a, h] = o * (gate[a, h] if gate is not None else 1.0)
    return out


def chunk_attention(h, w, prefix, m):
    """Grouped-query attention without rotation: ``score = q . k * scale - r1 ln(1 + r2 (i - j))``, keys of
    the query's own chunk, a sink per head, the head's output times ``sigmoid(g . h)``.  (The same as
    ``attend``, in matrix form.)"""
    t = h.shape[0]
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[prefix + "q"].T).reshape(t, heads, dim)
    k = (h @ w[prefix + "k"].T).reshape(t, kv_heads, dim)
    v = (h @ w[prefix + "v"].T).reshape(t, kv_heads, vdim)
    gate = torch.sigmoid(h @ w[prefix + "g"].T)                                 # [T, heads]
    group = heads // kv_heads
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    dist = (torch.arange(t)[:, None] - torch.arange(t)[None, :]).clamp(min=0).to(F)
    r1, r2 = w[prefix + "r1"], w[prefix + "r2"]
    scores = scores - r1[:, None, None] * torch.log1p(r2[:, None, None] * dist[None])
    p = sink_softmax(scores, chunk_visible(t, m["mask"]["size"])[None].expand(heads, t, t), w[prefix + "sink"])
    out = torch.einsum("hij,jhd->ihd", p, v) * gate[:, :, None]
    return out.reshape(t, heads * vdim) @ w[prefix + "o"].T


def latent_attention(h, w, prefix, m, eps):
    """Causal attention whose keys and values come from one normed latent per token plus one rotated key
    part that all heads share; queries pass through a normed latent of their own."""
    t = h.shape[0]
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(t)
    cq = rms_norm(h @ w[prefix + "dq"].T, w[prefix + "dq.norm"], eps)
    q = (cq @ w[prefix + "uq"].T).reshape(t, heads, dim + rot)
    q_plain, q_rot = q[..., :dim], rotate_half_split(q[..., dim:], pos, m["rot"]["base"], m["rot"]["dims"])
    down = h @ w[prefix + "dkv"].T
    c = rms_norm(down[:, :rank], w[prefix + "dkv.norm"], eps)
    k_rot = rotate_half_split(down[:, rank:], pos, m["rot"]["base"], m["rot"]["dims"])    # [T, rot]
    k_plain = (c @ w[prefix + "uk"].T).reshape(t, heads, dim)
    v = (c @ w[prefix + "uv"].T).reshape(t, heads, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    causal = torch.arange(t)[None, :] <= torch.arange(t)[:, None]
    p = torch.softmax(scores.masked_fill(~causal[None], -math.inf), dim=-1)
    out = torch.einsum("hij,jhd->ihd", p, v)
    return out.reshape(t, heads * vdim) @ w[prefix + "o"].T


# ------------------------------------------------------------------------------------------ feed-forwards

def clamped_gated(h, w, prefix, limit):
    g = (h @ w[prefix + "gate"].T).clamp(max=limit)
    u = (h @ w[prefix + "up"].T).clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[prefix + "down"].T


def route(h, router, top, scale):
    """``(ids [T, top], weights [T, top])``: the ``top`` largest sigmoid scores, divided by their sum, times
    ``scale``."""
    s = torch.sigmoid(h @ router.T)
    chosen, ids = torch.topk(s, top, dim=-1)
    return ids, chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20) * scale


def routed_experts(h, w, prefix, mlp, ids=None):
    """Every token's chosen experts ``down(relu(up h)^2)``, weighted.  ``ids`` overrides the choice (the
    weights still come from this function's own scores)."""
    r = mlp["router"]
    s = torch.sigmoid(h @ w[prefix + "router"].T)
    if ids is None:
        ids = torch.topk(s, r["top"], dim=-1).indices
    chosen = torch.gather(s, 1, ids.long())
    weights = chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20) * r["scale"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for slot in range(ids.shape[1]):
            e = int(ids[t, slot])
            a = torch.relu(h[t] @ w[f"{prefix}e{e}.up"].T) ** 2
            out[t] += weights[t, slot] * (a @ w[f"{prefix}e{e}.down"].T)
    return out


# ------------------------------------------------------------------------------------------ the model

def forward(cfg, w, tokens, expert_ids=None, return_layers=False):
    """Logits ``[T, vocab]`` of one whole sequence.  ``expert_ids``: ``{layer: ids [T, top]}`` to hold the
    routing to a given choice.  ``return_layers``: also the stream after every layer ``[L, T, width]``."""
    eps = cfg["norm"]["eps"]
    mult = cfg["residual_mult"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tokens]
    results = [x]                     # the embedding output, then every layer's result
    seen = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            a = chunk_attention(h, w, p + "mix.", layer["mixer"])
        elif layer["type"] == "latent_attention":
            a = latent_attention(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + mult * a
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                f = clamped_gated(h, w, p + "mlp.", mlp["limit"])
            else:
                f = routed_experts(h, w, p + "mlp.", mlp, None if expert_ids is None else expert_ids.get(i))
            x = x + mult * f
        results.append(x)
        weights = w[p + "dwa"]
        x = sum(weights[j] * results[j] for j in range(i + 2))
        seen.append(x)
    h = layer_norm(x, w["final.norm"], eps)
    logits = h @ w["embed"].T
    cap = cfg["logit_softcap"]
    logits = cap * torch.tanh(logits / cap)
    if return_layers:
        return logits, torch.stack(seen)
    return logits


def generate(cfg, w, prompt, new_tokens):
    """Greedy continuation, the whole sequence recomputed for every token."""
    seq = list(prompt)
    for _ in range(new_tokens):
        seq.append(int(forward(cfg, w, seq)[-1].argmax()))
    return seq[len(prompt):]
