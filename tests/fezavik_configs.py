"""Small Fezavik configurations for the tests, their weights and their oracle.

The configurations differ in everything config.json can say: width, vocabulary, number and order of layers
(each mixer comes first somewhere), attention with 1, 2, 3 and 4 query heads a kv head, key and value sizes
that are equal or not, multiples of 16 or odd, rotation over a part of a head, over all of it or none, with
and without slowed-down long waves (the three bands all occur among the pairs of "a" and "e"), windows shorter
than a page (7, 1), of a few pages, longer than every prompt and none; latents of 12 to 128 with rotated parts
of 0 to 32; recurrent heads with key sizes from 5 to 130 and values narrower and wider than a block of the
scan's columns; experts with one, some and all slots a token, with no pass-through slots, a few, and more of
them than experts; a layer without a feed-forward; a model without experts and one of recurrent layers only.  Weights are drawn with a spread of 1 / sqrt(fan-in), larger
for routers and for what makes scores, so that scores spread over several units (a wrong window edge or a lost
sink moves a row by far more than rounding), the chosen slots are chosen clearly and the correction changes
some choices.
"""

import json
import math
import random

import torch

import plain_fezavik as plain
from tinyvllm_b200.models import FezavikConfig
from tinyvllm_b200.models.fezavik import FezavikExperts, FezavikLayer, FezavikRotation


def _rot(dims, base, scaling=None):
    return FezavikRotation(dims=dims, base=base, scaling=scaling)


def _a(heads, kv, dim, vdim, window, rot, mlp, scale=None):
    return FezavikLayer(type="attention", heads=heads, kv_heads=kv, dim=dim, vdim=vdim, window=window, rot=rot,
                        scale=scale or 2.0 / math.sqrt(dim), mlp=mlp)


def _l(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, rot, mlp, scale=None):
    return FezavikLayer(type="latent_attention", heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank,
                        kv_rank=kv_rank, window=window, rot=rot, scale=scale or 2.0 / math.sqrt(dim + rot_dim), mlp=mlp)


def _h(heads, dim, vdim, mlp):
    return FezavikLayer(type="hgrn2", heads=heads, dim=dim, vdim=vdim, mlp=mlp)


def _moe(experts, top, ff, identity=0):
    return FezavikExperts(experts=experts, top=top, ff=ff, identity=identity)


FEZAVIK_CONFIGS = {
    # all three mixers, the attention twice; half of a head's dimensions turn, the long waves slowed down (of the
    # four pairs one keeps its frequency, one is blended, two are slowed); windows of one and a half and of two
    # and a half pages; three of eight experts and two pass-through slots
    "a": FezavikConfig(vocab=150, width=64, norm_eps=1e-5, layers=(
        _a(4, 2, 16, 32, 24, _rot(8, 100.0, (8.0, 1.0, 4.0, 64.0)), _moe(8, 3, 24, 2)),
        _h(4, 16, 32, _moe(8, 3, 24, 2)),
        _l(4, 16, 16, 16, 24, 32, 40, _rot(16, 5000.0), _moe(8, 3, 24, 2)),
        _a(4, 2, 16, 32, 24, _rot(8, 100.0, (8.0, 1.0, 4.0, 64.0)), _moe(8, 3, 24, 2)))),
    # sizes no vector access fits, the recurrence first: three query heads on one kv head, a window shorter than
    # a page, no slowed waves, all of three experts and no pass-through slot, a latent layer without a window, a
    # layer without a feed-forward
    "b": FezavikConfig(vocab=97, width=48, norm_eps=1e-6, layers=(
        _h(3, 10, 7, _moe(3, 3, 10)),
        _a(3, 1, 9, 5, 7, _rot(4, 300.0), None),
        _l(3, 6, 4, 5, 10, 12, None, _rot(4, 50.0), _moe(5, 1, 12, 3)),
        _h(2, 6, 20, None))),
    # the latent layer first and without a rotated part; as many kv heads as query heads, all of a head turns, a
    # window longer than every prompt; a key size of 130 in the recurrence and values wider than one block of the
    # scan's columns; two slots of twenty a token, four of them pass-through
    "c": FezavikConfig(vocab=130, width=128, norm_eps=1e-6, layers=(
        _l(2, 24, 0, 40, 20, 48, 33, None, _moe(16, 2, 16, 4)),
        _a(8, 8, 32, 16, 1000, _rot(32, 1000000.0), _moe(16, 2, 16, 4)),
        _h(2, 130, 48, _moe(16, 2, 16, 4)),
        _a(8, 8, 32, 16, None, None, _moe(4, 2, 32, 1)))),
    # a single head everywhere, a window of one position (a query sees itself and the sink alone), more
    # pass-through slots than experts, every slot used, width and vocabulary that are no multiples of four
    "d": FezavikConfig(vocab=101, width=50, norm_eps=1e-5, layers=(
        _a(1, 1, 7, 7, 1, _rot(2, 3.0), _moe(2, 5, 6, 3)),
        _h(1, 5, 3, _moe(4, 2, 6, 1)),
        _l(1, 12, 2, 9, 7, 12, 3, _rot(2, 10.0, (2.0, 1.0, 2.0, 16.0)), None),
        _h(5, 4, 4, _moe(2, 1, 11, 2)))),
    # sizes of the usual kind (powers of two, heads of 64), four query heads a kv head, windows of several pages
    # that long prompts pass many times, slowed waves in both kinds of attention
    "e": FezavikConfig(vocab=300, width=256, norm_eps=1e-6, layers=(
        _a(8, 2, 64, 64, 128, _rot(32, 10000.0, (4.0, 1.0, 4.0, 256.0)), _moe(8, 2, 64, 2)),
        _l(8, 32, 32, 64, 96, 128, 96, _rot(32, 10000.0, (16.0, 2.0, 8.0, 128.0)), _moe(8, 2, 64, 2)),
        _h(4, 64, 128, _moe(8, 2, 64, 2)),
        _a(8, 2, 64, 64, 128, _rot(32, 10000.0, (4.0, 1.0, 4.0, 256.0)), None))),
    # the mixers alone, without any feed-forward: nothing is routed, so 16-bit arithmetic cannot send a token
    # another way and its rows stay within rounding of the plain ones; sizes in steps of 16, which the
    # tensor-core attention kernels take
    "f": FezavikConfig(vocab=120, width=96, norm_eps=1e-5, layers=(
        _a(4, 2, 32, 16, 40, _rot(16, 1000.0, (4.0, 1.0, 4.0, 64.0)), None),
        _l(4, 16, 16, 32, 40, 48, 24, _rot(16, 200.0), None),
        _h(3, 32, 16, None),
        _a(4, 4, 16, 16, None, _rot(16, 50.0), None))),
    # recurrent layers only: no layer keeps keys or values, a request's whole memory is its state slots
    "g": FezavikConfig(vocab=90, width=64, norm_eps=1e-5, layers=(
        _h(2, 16, 16, _moe(4, 2, 16, 1)),
        _h(4, 8, 24, None))),
}
FEZAVIK_SEEDS = {"a": 41, "b": 42, "c": 43, "d": 44, "e": 45, "f": 46, "g": 47}
FEZAVIK_PAGES = {"a": 16, "b": 8, "c": 16, "d": 4, "e": 32, "f": 16, "g": 16}


def tensors_of(config: FezavikConfig, seed: int) -> dict:
    """Checkpoint tensors (float32) of ``config``, drawn from ``seed``."""
    g = torch.Generator().manual_seed(seed)

    def matrix(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)

    def around_one(n):
        return 1.0 + 0.3 * (torch.rand(n, generator=g) - 0.5)

    d = config.width
    t = {"embed": torch.randn(config.vocab, d, generator=g), "final.norm": around_one(d),
         "head": matrix(config.vocab, d, 2.0)}
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        t[p + "norm1"], t[p + "norm1b"] = around_one(d), around_one(d)
        hv = layer.heads * layer.vdim
        if layer.type == "attention":
            t[p + "mix.q"] = matrix(layer.heads * layer.dim, d)
            t[p + "mix.k"] = matrix(layer.kv_heads * layer.dim, d)
            t[p + "mix.v"] = matrix(layer.kv_heads * layer.vdim, d)
            t[p + "mix.q.norm"] = around_one(layer.heads * layer.dim)
            t[p + "mix.k.norm"] = around_one(layer.kv_heads * layer.dim)
            t[p + "mix.sink"] = torch.randn(layer.heads, generator=g) * 1.5
        elif layer.type == "latent_attention":
            t[p + "mix.dq"] = matrix(layer.q_rank, d)
            t[p + "mix.dq.norm"] = around_one(layer.q_rank)
            t[p + "mix.uq"] = matrix(layer.heads * (layer.dim + layer.rot_dim), layer.q_rank)
            t[p + "mix.dkv"] = matrix(layer.kv_rank + layer.rot_dim, d)
            t[p + "mix.dkv.norm"] = around_one(layer.kv_rank)
            t[p + "mix.uk"] = matrix(layer.heads * layer.dim, layer.kv_rank)
            t[p + "mix.uv"] = matrix(hv, layer.kv_rank)
            t[p + "mix.sink"] = torch.randn(layer.heads, generator=g) * 1.5
            t[p + "mix.g"] = matrix(layer.heads, d, 2.0)
        else:
            t[p + "mix.q"] = matrix(layer.heads * layer.dim, d, 1.5)
            t[p + "mix.f"] = matrix(layer.heads * layer.dim, d, 2.0)
            t[p + "mix.f.b"] = torch.randn(layer.heads * layer.dim, generator=g)
            # bounds from 0 to nearly 1: channels that forget at once beside channels that keep hundreds of tokens
            t[p + "mix.lower"] = 1.0 - torch.rand(layer.heads * layer.dim, generator=g) ** 3
            t[p + "mix.v"] = matrix(hv, d)
            t[p + "mix.norm"] = around_one(layer.vdim)
        t[p + "mix.o"] = matrix(d, hv)
        m = layer.mlp
        if m is None:
            continue
        t[p + "norm2"], t[p + "norm2b"] = around_one(d), around_one(d)
        slots = m.experts + m.identity
        t[p + "mlp.router"] = matrix(slots, d, 4.0)
        t[p + "mlp.correction"] = torch.randn(slots, generator=g) * 0.15
        for e in range(m.experts):
            t[p + f"mlp.e{e}.gate"] = matrix(m.ff, d, 2.0)
            t[p + f"mlp.e{e}.up"] = matrix(m.ff, d, 2.0)
            t[p + f"mlp.e{e}.down"] = matrix(d, m.ff)
    return t


def write_folder(folder, config: FezavikConfig, seed: int, dtype=torch.float32):
    """config.json and model.safetensors of ``config`` in ``folder``.  The values are rounded to
    bfloat16 whatever ``dtype`` stores them as, so that both number formats run the same model."""
    from safetensors.torch import save_file

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config.to_json(), indent=1), encoding="utf-8")
    tensors = {name: value.to(torch.bfloat16).to(dtype).contiguous() for name, value in tensors_of(config, seed).items()}
    save_file(tensors, str(folder / "model.safetensors"))
    return folder


def read_folder(folder):
    from safetensors import safe_open

    config = json.loads((folder / "config.json").read_text(encoding="utf-8"))
    tensors = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            tensors[name] = f.get_tensor(name)
    return config, tensors


_oracle: dict = {}


def oracle_logits(folder, requests: dict) -> dict:
    """{request: float32 logits [T, V]} of the plain implementation, remembered per folder and tokens."""
    config, tensors = read_folder(folder)
    out = {}
    for rid, tokens in requests.items():
        key = (str(folder), tuple(tokens))
        if key not in _oracle:
            _oracle[key] = plain.forward(config, tensors, tokens).to(torch.float32)
        out[rid] = _oracle[key]
    return out


_greedy: dict = {}


def greedy_oracle(folder, prompt, new_tokens: int) -> list[int]:
    key = (str(folder), tuple(prompt), new_tokens)
    if key not in _greedy:
        config, tensors = read_folder(folder)
        _greedy[key] = plain.greedy(config, tensors, prompt, new_tokens)
    return _greedy[key]


def tokens_of(vocab: int, count: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]
