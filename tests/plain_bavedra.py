"""A plain statement of the Bavedra decoder: whole sequences, no cache, no batches, float64, one
function per mechanism.  It shares no code with the package and is slow on purpose.

The design: an embedding times a constant; pre-norm layers around a residual stream, ``x + mixer(norm1(x))``
then ``x + ff(norm2(x))``; three mixers (``rglru``: a gated branch times a real-gated linear recurrence per
channel behind a short convolution; ``parallel``: grouped-query attention with a rotated part, a sliding
window, a sink of score zero and the unrotated keys as values, next to a selective state-space recurrence
with a matrix state per head, each output normed over the width and the two averaged; ``delta``: the gated
delta rule on unit keys and queries behind short convolutions); two feed-forwards (squared-relu dense; a
mixture of gated experts chosen by group-limited corrected scores, with identity experts and a gated shared
expert) or none; a layer may run another layer's weights on a state of its own; a final norm and an output head.
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


# ------------------------------------------------------------------------------------------ small things

def rms(x, eps):
    """``x / sqrt(mean(x^2) + eps)`` over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.logaddexp(z, torch.zeros_like(z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def short_convolution(x, taps, bias=None):
    """``x`` ``[T, C]``, ``taps`` ``[C, K]``: ``y[t, c] = sum_j taps[c, K - 1 - j] * x[t - j, c]`` with zeros in
    front of the sequence (the last column multiplies the current token)."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros((K - 1, C), dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(K):
        y = y + padded[K - 1 - j:K - 1 - j + T] * taps[:, K - 1 - j]
    return y if bias is None else y + bias


def rotate_pairs(x, positions, base, dims):
    """Turns the first ``dims`` entries of the last dimension of ``x`` ``[T, heads, D]``: entry ``2i`` with
    entry ``2i + 1`` by the angle ``p * base ** (-2i / dims)``."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F)
    angle = positions.to(F)[:, None] * (base ** (-2.0 * i / dims))[None, :]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


# ------------------------------------------------------------------------------------------ rglru

def gated_linear_recurrence(u, r, i, lam):
    """``[T, C]`` each, ``lam`` ``[C]``: ``a = exp(-8 r softplus(lam))``, ``S <- a S + sqrt(1 - a^2) i u`` from
    zero, every token alike."""
    a = torch.exp(-8.0 * r * softplus(lam))
    gain = torch.sqrt(1.0 - a * a)
    S = torch.zeros_like(u[0])
    out = []
    for t in range(u.shape[0]):
        S = a[t] * S + gain[t] * i[t] * u[t]
        out.append(S)
    return torch.stack(out)


def block_gates(u, matrices, biases):
    """``sigmoid`` of a block-diagonal product: ``u`` ``[T, C]`` in ``B`` equal parts, ``matrices`` ``[B, C/B,
    C/B]`` (out, in), ``biases`` ``[B, C/B]``."""
    B = matrices.shape[0]
    parts = u.reshape(u.shape[0], B, -1)
    return torch.sigmoid(torch.einsum("tbi,boi->tbo", parts, matrices) + biases).reshape(u.shape)


def rglru_mixer(h, w, p, m):
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = short_convolution(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    r = block_gates(u, w[p + "ra"], w[p + "ra.b"])
    i = block_gates(u, w[p + "ri"], w[p + "ri.b"])
    S = gated_linear_recurrence(u, r, i, w[p + "lam"])
    return (S * y) @ w[p + "o"].T


# ------------------------------------------------------------------------------------------ parallel: left

def window_attention(q, k, v, scale, window):
    """``q`` ``[T, H, D]``, ``k`` ``[T, G, D]``, ``v`` ``[T, G, V]``.  Query ``i`` sees keys ``j`` with ``0 <= i - j <
    window``; the weights are ``exp(s_j) / (1 + sum exp(s))``: a sink of score zero without a value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            top = torch.clamp(s.max(), min=0.0)
            e = torch.exp(s - top)
            out[i, h] = (e[:, None] * v[lo:i + 1, g]).sum(dim=0) / (torch.exp(-top) + e.sum())
    return out


def left_mixer(h, w, p, m, positions):
    T = h.shape[0]
    q = (h @ w[p + "q"].T).reshape(T, m["heads"], m["dim"])
    k = (h @ w[p + "k"].T).reshape(T, m["kv_heads"], m["dim"])
    v = k
    if m.get("rot") is not None:
        q = rotate_pairs(q, positions, m["rot"]["base"], m["rot"]["dims"])
        k = rotate_pairs(k, positions, m["rot"]["base"], m["rot"]["dims"])
    a = window_attention(q, k, v, m["scale"], m["mask"]["size"] if m.get("mask") is not None else T)
    return a.reshape(T, -1) @ w[p + "o"].T


# ------------------------------------------------------------------------------------------ parallel: right

def state_space_recurrence(x, B, C, dt, A_log, D):
    """``x`` ``[T, H, V]``, ``B``/``C`` ``[T, G, N]``, ``dt`` ``[T, H]`` (already positive).  Per head a state ``S``
    ``[N, V]`` from zero: ``S <- exp(-exp(A_log) dt) S + dt B x^T``, ``y = S^T C + D x``."""
    T, H, V = x.shape
    G = B.shape[1]
    out = torch.zeros_like(x)
    for h in range(H):
        g = h // (H // G)
        S = torch.zeros((B.shape[2], V), dtype=x.dtype)
        for t in range(T):
            S = torch.exp(-torch.exp(A_log[h]) * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            out[t, h] = S.T @ C[t, g] + D[h] * x[t, h]
    return out


def right_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_convolution(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    y = state_space_recurrence(x, B, C, dt, w[p + "A_log"], w[p + "D"]).reshape(T, inner)
    y = y * silu(z)
    parts = m["norm_groups"]
    y = rms(y.reshape(T, parts, -1), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps, positions):
    left = left_mixer(h, w, p + "left.", m["left"], positions)
    right = right_mixer(h, w, p + "right.", m["right"], eps)
    return 0.5 * (norm(left, w[p + "left.out"], eps) + norm(right, w[p + "right.out"], eps))


# ------------------------------------------------------------------------------------------ delta

def unit(x):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def delta_recurrence(q, k, v, beta, g):
    """``q``/``k`` ``[T, G, D]``, ``v`` ``[T, H, V]``, ``beta``/``g`` ``[T, H]``.  Per head a state ``S`` ``[D, V]`` from
    zero; per token: decay, the correction of what the key reads towards the value, the write, then the read."""
    T, H, V = v.shape
    G = q.shape[1]
    out = torch.zeros_like(v)
    for h in range(H):
        c = h // (H // G)
        S = torch.zeros((q.shape[2], V), dtype=v.dtype)
        for t in range(T):
            S = g[t, h] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, c])
            S = S + torch.outer(k[t, c], u)
            out[t, h] = S.T @ q[t, c]
    return out


def delta_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, D)
    k = silu(short_convolution(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, D)
    v = silu(short_convolution(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, V)
    q = unit(q) * D ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = delta_recurrence(q, k, v, beta, g)
    o = rms(o, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).reshape(T, H, V)
    return o.reshape(T, -1) @ w[p + "o"].T


# ------------------------------------------------------------------------------------------ feed-forwards

def dense_feed_forward(h, w, p):
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def gated_expert(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, router):
    """(indices ``[T, top]``, weights ``[T, top]``, scores ``[T, E + I]``).  Softmax over every router output;
    the choice goes by score + correction among the experts of the ``keep`` groups whose best such score is
    largest (the lower index first among equals); the weights are the chosen plain scores over their sum."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"]
    groups = router.get("groups")
    if groups is not None:
        T, n = choice.shape
        per = n // groups["count"]
        best = choice.reshape(T, groups["count"], per).max(dim=-1).values
        order = torch.argsort(best, dim=-1, descending=True, stable=True)[:, :groups["keep"]]
        allowed = torch.zeros((T, groups["count"]), dtype=torch.bool)
        allowed.scatter_(1, order, True)
        choice = torch.where(allowed.repeat_interleave(per, dim=1), choice, torch.full_like(choice, -math.inf))
    index = torch.argsort(choice, dim=-1, descending=True, stable=True)[:, :router["top"]]
    chosen = s.gather(1, index)
    return index, chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20), s


def routed_feed_forward(h, w, p, mlp, chosen=None):
    """``chosen`` (``[T, top]``): use these experts instead of the router's choice (weights still from the scores);
    for comparisons in which a near-tie may fall either way."""
    router = mlp["router"]
    index, weight, s = route(h, w, p, router)
    if chosen is not None:
        index = torch.as_tensor(chosen).long()
        picked = s.gather(1, index)
        weight = picked / (picked.sum(dim=-1, keepdim=True) + 1e-20)
    real = router["experts"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(index[t].tolist(), weight[t]):
            if e >= real:                        # an identity expert hands its input on
                out[t] += a * h[t]
            else:
                out[t] += a * gated_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * gated_expert(h, w, p + "shared.")
    return out


# ------------------------------------------------------------------------------------------ the model

def mixer_of(layer, h, w, p, eps, positions):
    m = layer["mixer"]
    if layer["type"] == "rglru":
        return rglru_mixer(h, w, p, m)
    if layer["type"] == "parallel":
        return parallel_mixer(h, w, p, m, eps, positions)
    if layer["type"] == "delta":
        return delta_mixer(h, w, p, m, eps)
    raise ValueError(layer["type"])


def owner(layers, i):
    """The layer whose tensors layer ``i`` runs: itself, or what its ``weights_of`` leads to."""
    while layers[i].get("weights_of") is not None:
        i = layers[i]["weights_of"]
    return i


def forward(cfg, w, tokens, layers_out=None, routes=None):
    """Logits ``[T, vocab]`` of one sequence from its first token; ``layers_out`` (a list) receives the
    residual stream after every layer; ``routes`` ({layer: ``[T, top]``}) fixes the experts of routed layers."""
    eps = cfg["norm"]["eps"]
    positions = torch.arange(len(tokens))
    x = w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{owner(cfg['layers'], i)}."
        x = x + mixer_of(layer, norm(x, w[p + "norm1"], eps), w, p + "mix.", eps, positions)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                x = x + dense_feed_forward(h, w, p + "mlp.")
            else:
                x = x + routed_feed_forward(h, w, p + "mlp.", mlp, None if routes is None else routes.get(i))
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm(x, w["final.norm"], eps) @ w["head"].T


def generate(cfg, w, prompt, n):
    """Greedy continuation: ``n`` tokens, each the largest logit (the lowest index among equals)."""
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(torch.argmax(forward(cfg, w, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out
