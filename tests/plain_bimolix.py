"""A plain, slow Bimolix on the CPU, one function per mechanism, written from the design's equations.

It shares no code with the package: tensors come as a dict name -> torch tensor, the configuration as
the parsed config.json.  Everything runs in ``dtype`` (float64 by default), a token at a time where
the design is a recurrence, with full score matrices where it is attention.
"""

from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """x / rms(x) * (1 + w): the weight is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_half_layout(x, positions, dims, base):
    """x [tokens, heads, dim]: dimension i of the first ``dims`` turns together with i + dims / 2."""
    half = dims // 2
    freqs = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * freqs[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def retention(h, w, prefix, mixer, eps, state=None, start=0):
    """The retention mixer on the tokens ``h`` [tokens, width] of one sequence that begin at position
    ``start``; ``state`` [heads, dim, vdim] is what the tokens before left (None: zero).  Returns
    (output, new state)."""
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    tokens = h.shape[0]
    q = (h @ w[prefix + ".q"].T).view(tokens, heads, dim)
    k = (h @ w[prefix + ".k"].T).view(tokens, heads, dim)
    v = (h @ w[prefix + ".v"].T).view(tokens, heads, vdim)
    positions = torch.arange(start, start + tokens)
    rot = mixer.get("rot")
    if rot is not None:
        q = rotate_half_layout(q, positions, rot["dims"], rot["base"])
        k = rotate_half_layout(k, positions, rot["dims"], rot["base"])
    k = k * dim ** -0.5
    decay = torch.tensor(mixer["decay"], dtype=h.dtype)
    s = torch.zeros(heads, dim, vdim, dtype=h.dtype) if state is None else state.clone()
    outs = []
    for t in range(tokens):
        s = decay[:, None, None] * s + k[t][:, :, None] * v[t][:, None, :]
        outs.append(torch.einsum("hdv,hd->hv", s, q[t]))
    o = rms(torch.stack(outs), eps).reshape(tokens, heads * vdim)
    g = h @ w[prefix + ".g"].T
    return (o * (g * torch.sigmoid(g))) @ w[prefix + ".o"].T, s


def distance_bucket(n: int, rows: int, bias_max: int) -> int:
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(bias_max / half) * (rows - half))))


def bias_matrix(rel, tokens, bias_max):
    """[heads, tokens, tokens]: the table's entry for the distance i - j (0 where j > i)."""
    by_distance = torch.tensor([distance_bucket(n, rel.shape[0], bias_max) for n in range(tokens)])
    i = torch.arange(tokens)[:, None]
    j = torch.arange(tokens)[None, :]
    bucket = by_distance[(i - j).clamp(min=0)]
    return rel[bucket].permute(2, 0, 1)


def chunk_mask(tokens, size):
    """[tokens, tokens], true where query i sees key j: j <= i, both in the same chunk of ``size``
    positions counted from 0 (``size`` None: no chunks)."""
    i = torch.arange(tokens)[:, None]
    j = torch.arange(tokens)[None, :]
    seen = j <= i
    return seen if size is None else seen & (i // size == j // size)


def softmax_with_one_more(scores, seen):
    """exp(s_j) / (1 + sum over the seen keys of exp(s_j)): one more term of score 0 that has no value."""
    e = torch.where(seen, torch.exp(scores), torch.zeros_like(scores))
    return e / (1.0 + e.sum(-1, keepdim=True))


def chunked_attention(h, w, prefix, mixer, eps):
    """The attention mixer on a whole sequence ``h`` [tokens, width] that begins at position 0."""
    heads, groups, dim = mixer["heads"], mixer["kv_heads"], mixer["dim"]
    tokens = h.shape[0]
    q = (h @ w[prefix + ".q"].T + w[prefix + ".q.b"]).view(tokens, heads, dim)
    k = (h @ w[prefix + ".k"].T + w[prefix + ".k.b"]).view(tokens, groups, dim)
    v = k                                                   # the values are the keys before their norm
    q = rms(q, eps) * w[prefix + ".q.norm"]
    k = rms(k, eps) * w[prefix + ".k.norm"]
    mask = mixer.get("mask")
    seen = chunk_mask(tokens, None if mask is None else mask["size"])
    bias = bias_matrix(w[prefix + ".rel"], tokens, mixer["bias_max"])
    out = torch.zeros(tokens, heads, mixer["vdim"], dtype=h.dtype)
    for head in range(heads):
        kv = head // (heads // groups)
        scores = (q[:, head] @ k[:, kv].T) * mixer["scale"] + bias[head]
        out[:, head] = softmax_with_one_more(scores, seen) @ v[:, kv]
    gate = torch.sigmoid(h @ w[prefix + ".g"].T)
    return (out.reshape(tokens, -1) * gate) @ w[prefix + ".o"].T


def dense_ff(h, w, prefix):
    g = h @ w[prefix + ".gate"].T
    return ((g * torch.sigmoid(g)) * (h @ w[prefix + ".up"].T)) @ w[prefix + ".down"].T


def clamped_expert(h, w, prefix, limit):
    g = torch.clamp(h @ w[prefix + ".gate"].T, max=limit)
    u = torch.clamp(h @ w[prefix + ".up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[prefix + ".down"].T


def route(z, correction, router):
    """Chosen experts and their weights for router logits ``z`` [experts] of one token."""
    experts, top = router["experts"], router["top"]
    s = torch.sigmoid(z)
    choice = s + correction
    groups = router.get("groups")
    if groups is not None:
        size = experts // groups["count"]
        totals = []
        for g in range(groups["count"]):
            best = sorted(choice[g * size:(g + 1) * size].tolist(), reverse=True)[:2]
            totals.append(sum(best))
        kept = sorted(range(groups["count"]), key=lambda g: (-totals[g], g))[:groups["keep"]]
        allowed = [e for e in range(experts) if e // size in kept]
    else:
        allowed = list(range(experts))
    chosen = sorted(allowed, key=lambda e: (-float(choice[e]), e))[:top]
    total = sum(s[e] for e in chosen) + 1e-20
    return chosen, [s[e] / total * router["scale"] for e in chosen]


def moe_ff(h, w, prefix, mlp):
    router = mlp["router"]
    z = h @ w[prefix + ".router"].T
    out = torch.zeros(h.shape[0], w[prefix + ".e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        chosen, weights = route(z[t], w[prefix + ".correction"], router)
        for e, weight in zip(chosen, weights):
            out[t] += weight * clamped_expert(h[t:t + 1], w, f"{prefix}.e{e}", mlp["expert"]["limit"])[0]
    shared = mlp.get("shared")
    if shared is not None:
        gate = torch.sigmoid(h @ w[prefix + ".shared.sg"].T)          # one number a token
        out = out + gate * clamped_expert(h, w, prefix + ".shared", shared["limit"])
    return out


def feed_forward(h, w, prefix, mlp):
    return dense_ff(h, w, prefix) if mlp["kind"] == "dense" else moe_ff(h, w, prefix, mlp)


def forward(config, weights, tokens, dtype=torch.float64, layer_outputs=None):
    """Logits [tokens, vocab] of one whole sequence; ``layer_outputs`` (a list) receives the residual
    stream after every layer."""
    w = {name: t.to(dtype) for name, t in weights.items()}
    eps = config["norm"]["eps"]
    x = norm_one_plus(w["embed"][torch.as_tensor(tokens)], w["embed.norm"], eps)
    for index, layer in enumerate(config["layers"]):
        owner = index
        while config["layers"][owner].get("weights_of") is not None:
            owner = config["layers"][owner]["weights_of"]
        p = f"l{owner}"
        h = norm_one_plus(x, w[p + ".norm1"], eps)
        if layer["type"] == "retention":
            x = x + retention(h, w, p + ".mix", layer["mixer"], eps)[0]
        else:
            x = x + chunked_attention(h, w, p + ".mix", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + feed_forward(norm_one_plus(x, w[p + ".norm2"], eps), w, p + ".mlp", layer["mlp"])
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return norm_one_plus(x, w["final.norm"], eps) @ w["head"].T


def greedy(config, weights, prompt, new_tokens: int) -> list[int]:
    """``new_tokens`` tokens after ``prompt``, each the largest logit of the whole sequence run again."""
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(forward(config, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]
