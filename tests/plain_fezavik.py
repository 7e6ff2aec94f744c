"""A plain, slow Fezavik on the CPU, one function per mechanism, written from the design's equations.

It shares no code with the package: tensors come as a dict name -> torch tensor, the configuration as
the parsed config.json.  Everything runs in ``dtype`` (float64 by default), a token at a time where
the design is a recurrence, with full score matrices where it is attention.
"""

from __future__ import annotations

import math

import torch


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------ positions
def frequencies(rot, dtype):
    """f_i = base^(-2i / dims), then, with ``scaling``, the long waves slowed down: a wave shorter than
    original / high keeps its frequency, one longer than original / low turns ``factor`` times slower,
    and between the two the frequency is blended."""
    dims, base = rot["dims"], rot["base"]
    out = []
    scaling = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, original = (scaling[key] for key in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < original / high:
                pass
            elif wave > original / low:
                f = f / factor
            else:
                s = (original / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=dtype)


def rotate_neighbours(x, positions, rot):
    """x [tokens, heads, dim]: dimensions 2i and 2i + 1 of the first ``dims`` turn together."""
    dims = rot["dims"]
    angle = positions.to(x.dtype)[:, None] * frequencies(rot, x.dtype)[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * cos - v * sin, v * cos + u * sin], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., dims:]], dim=-1)


def rotate_halves(x, positions, rot):
    """x [tokens, heads, dim]: dimension i of the first ``dims`` turns together with i + dims / 2."""
    dims = rot["dims"]
    half = dims // 2
    angle = positions.to(x.dtype)[:, None] * frequencies(rot, x.dtype)[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------ attention
def window_mask(tokens, size):
    """seen[i, j]: 0 <= i - j < size (no ``size``: every key up to the query's own)."""
    i = torch.arange(tokens)[:, None]
    j = torch.arange(tokens)[None, :]
    seen = j <= i
    if size is not None:
        seen &= i - j < size
    return seen


def softmax_with_sink(scores, seen, sink):
    """scores [heads, tokens, tokens]; the denominator holds exp(sink_h) beside the seen keys' terms."""
    scores = scores.masked_fill(~seen[None], -math.inf)
    top = torch.maximum(scores.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(scores - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - top))


def attention(h, w, prefix, mixer, eps):
    """Grouped-query attention on the tokens ``h`` [tokens, width] of one whole sequence."""
    heads, kv, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    tokens = h.shape[0]
    positions = torch.arange(tokens)
    q = rms_norm(h @ w[prefix + ".q"].T, w[prefix + ".q.norm"], eps).view(tokens, heads, dim)
    k = rms_norm(h @ w[prefix + ".k"].T, w[prefix + ".k.norm"], eps).view(tokens, kv, dim)
    v = (h @ w[prefix + ".v"].T).view(tokens, kv, vdim)
    rot = mixer.get("rot")
    if rot is not None:
        q, k = rotate_neighbours(q, positions, rot), rotate_neighbours(k, positions, rot)
    group = heads // kv
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * mixer["scale"]
    mask = mixer.get("mask")
    p = softmax_with_sink(scores, window_mask(tokens, None if mask is None else mask["size"]),
                          w[prefix + ".sink"])
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(tokens, heads * vdim)
    return o @ w[prefix + ".o"].T


def latent_attention(h, w, prefix, mixer, eps):
    """Attention whose queries, keys and values come through latents, on one whole sequence."""
    heads, dim, rot_dim, vdim, rank = (mixer[key] for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    tokens = h.shape[0]
    positions = torch.arange(tokens)
    c_q = rms_norm(h @ w[prefix + ".dq"].T, w[prefix + ".dq.norm"], eps)
    q = (c_q @ w[prefix + ".uq"].T).view(tokens, heads, dim + rot_dim)
    down = h @ w[prefix + ".dkv"].T
    c = rms_norm(down[:, :rank], w[prefix + ".dkv.norm"], eps)
    k_rot = down[:, None, rank:]                                   # one head, shared
    k_plain = (c @ w[prefix + ".uk"].T).view(tokens, heads, dim)
    v = (c @ w[prefix + ".uv"].T).view(tokens, heads, vdim)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    if rot_dim:
        q_rot = rotate_halves(q_rot, positions, mixer["rot"])
        k_rot = rotate_halves(k_rot, positions, mixer["rot"])
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain)
              + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * mixer["scale"]
    mask = mixer.get("mask")
    p = softmax_with_sink(scores, window_mask(tokens, None if mask is None else mask["size"]),
                          w[prefix + ".sink"])
    o = torch.einsum("hij,jhd->ihd", p, v)
    gate = torch.sigmoid(h @ w[prefix + ".g"].T)                   # [tokens, heads]
    return (o * gate[:, :, None]).reshape(tokens, heads * vdim) @ w[prefix + ".o"].T


# ------------------------------------------------------------------ recurrence
def forget_gates(h, w, prefix):
    """f = l + (1 - l) sigmoid(W_f h + b): never below the stored lower bound l."""
    lower = w[prefix + ".lower"]
    return lower + (1.0 - lower) * torch.sigmoid(h @ w[prefix + ".f"].T + w[prefix + ".f.b"])


def gated_recurrence(h, w, prefix, mixer, eps, state=None):
    """The recurrent mixer on the tokens ``h`` of one sequence; ``state`` [heads, dim, vdim] is what the
    tokens before left (None: zero).  Returns (output, new state)."""
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    tokens = h.shape[0]
    q = silu(h @ w[prefix + ".q"].T).view(tokens, heads, dim)
    f = forget_gates(h, w, prefix).view(tokens, heads, dim)
    v = (h @ w[prefix + ".v"].T).view(tokens, heads, vdim)
    s = torch.zeros(heads, dim, vdim, dtype=h.dtype) if state is None else state.clone()
    outs = []
    for t in range(tokens):
        s = f[t][:, :, None] * s + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        outs.append(torch.einsum("hdv,hd->hv", s, q[t]))
    o = rms_norm(torch.stack(outs), w[prefix + ".norm"], eps).reshape(tokens, heads * vdim)
    return o @ w[prefix + ".o"].T, s


# ------------------------------------------------------------------ experts
def route(z, correction, router):
    """From router logits ``z`` [slots] of one token to a list of (slot, weight): the softmax over all slots
    scores them, the ``top`` slots with the largest score + correction are chosen (the lower index of equals),
    and a chosen slot's weight is its score as it is."""
    s = torch.softmax(z, dim=-1)
    choice = (s + correction).tolist()
    order = sorted(range(len(choice)), key=lambda e: (-choice[e], e))
    return [(e, s[e]) for e in order[:router["top"]]]


def expert(h, w, prefix):
    return (silu(h @ w[prefix + ".gate"].T) * (h @ w[prefix + ".up"].T)) @ w[prefix + ".down"].T


def moe_ff(h, w, prefix, mlp):
    """A mixture of experts whose last ``identity`` slots hand their input on unchanged."""
    router = mlp["router"]
    real = router["experts"]
    z = h @ w[prefix + ".router"].T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in route(z[t], w[prefix + ".correction"], router):
            out[t] += weight * (expert(h[t], w, f"{prefix}.e{e}") if e < real else h[t])
    return out


# ------------------------------------------------------------------ the model
def forward(config, weights, tokens, dtype=torch.float64, layer_outputs=None):
    """Logits [tokens, vocab] of one sequence.  ``layer_outputs``: a list that receives the stream after
    every layer."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}"
        h = rms_norm(x, w[p + ".norm1"], eps)
        if layer["type"] == "attention":
            y = attention(h, w, p + ".mix", layer["mixer"], eps)
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, w, p + ".mix", layer["mixer"], eps)
        elif layer["type"] == "hgrn2":
            y, _ = gated_recurrence(h, w, p + ".mix", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, w[p + ".norm1b"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(moe_ff(rms_norm(x, w[p + ".norm2"], eps), w, p + ".mlp", layer["mlp"]),
                             w[p + ".norm2b"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(config, weights, prompt, new_tokens: int) -> list[int]:
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(forward(config, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]
