"""Small Bimolix configurations for the tests, their weights and their oracle.

The configurations differ in everything config.json can say: width, vocabulary, number and order of
layers, which layers run another layer's weights, retention heads with key and value sizes that are
equal or not (one value size wider than a block of the scan's columns, one key size of 130), turned
dimensions that are all, some or none of a head's, decays from 0.5 to exactly 1; attention with 1, 2
and 3 query heads a kv head, odd head sizes, chunks shorter than a page (7, 1), about a page and longer
than every prompt, distance tables with an even and an odd number of rows whose last bucket begins
inside or beyond the prompts; dense feed-forwards, none, and experts in groups (two of four kept,
groups of one expert, one group, no groups at all), all and one expert a token, shared experts or none.
Weights are drawn with a spread of 1 / sqrt(fan-in), larger for routers and for what makes scores, so
that scores spread over several units, the distance table and the extra term of the denominator matter,
the experts' limits cut, and the chosen experts are chosen clearly.
"""

import json
import math
import random

import torch

import plain_bimolix as plain
from tinyvllm_b200.models import BimolixConfig
from tinyvllm_b200.models.bimolix import BimolixFeedForward, BimolixLayer


def _r(heads, dim, vdim, decay, rot, mlp, weights_of=None):
    return BimolixLayer(type="retention", heads=heads, dim=dim, vdim=vdim, decay=tuple(decay),
                        rot_dims=rot[0] if rot else 0, rot_base=rot[1] if rot else 0.0, mlp=mlp,
                        weights_of=weights_of)


def _a(heads, kv, dim, chunk, rows, far, mlp, weights_of=None, scale=None):
    return BimolixLayer(type="attention", heads=heads, kv_heads=kv, dim=dim, vdim=dim,
                        scale=scale or 2.0 / math.sqrt(dim), bias_max=far, chunk=chunk, mlp=mlp,
                        weights_of=weights_of, rel_rows=rows)


def _dense(ff):
    return BimolixFeedForward(kind="dense", ff=ff)


def _moe(experts, top, ff, limit, groups=1, keep=1, shared=0, shared_limit=0.0, scale=1.0):
    return BimolixFeedForward(kind="moe", ff=ff, limit=limit, experts=experts, top=top, route_scale=scale,
                              groups=groups, keep=keep, shared_ff=shared, shared_limit=shared_limit)


BIMOLIX_CONFIGS = {
    # both mixers twice, the second time with the first's weights; half of a head's dimensions turn; two of
    # four groups of two experts
    "a": BimolixConfig(vocab=150, width=64, norm_eps=1e-5, layers=(
        _r(4, 16, 32, (0.9, 0.97, 0.995, 1.0), (8, 10000.0), _dense(96)),
        _a(4, 2, 16, 24, 12, 40.0, _moe(8, 3, 24, 1.0, groups=4, keep=2, shared=40, shared_limit=1.5, scale=2.0)),
        _r(4, 16, 32, (0.9, 0.97, 0.995, 1.0), (8, 10000.0), _dense(96), weights_of=0),
        _a(4, 2, 16, 24, 12, 40.0, _moe(8, 3, 24, 1.0, groups=4, keep=2, shared=40, shared_limit=1.5, scale=2.0),
           weights_of=1),
        _a(2, 2, 24, 24, 6, 9.0, _dense(40)))),
    # sizes no vector access fits: three query heads on one kv head, a chunk shorter than a page, an odd
    # number of table rows, a layer without a feed-forward, nothing turned, experts without groups of which
    # all are used, no shared expert
    "b": BimolixConfig(vocab=97, width=48, norm_eps=1e-6, layers=(
        _a(3, 1, 9, 7, 5, 11.0, _moe(3, 3, 10, 0.7)),
        _r(3, 10, 7, (0.5, 0.75, 0.99), (4, 300.0), None),
        _r(2, 6, 20, (0.999, 0.8), None, _moe(5, 2, 12, 2.0, shared=5, shared_limit=0.5, scale=0.5)),
        _a(3, 1, 9, 7, 5, 11.0, _moe(3, 3, 10, 0.7), weights_of=0))),
    # a chunk longer than every prompt and a table whose last bucket begins beyond them; a key size of 130
    # and values wider than one block of the scan's columns; one expert of sixteen in groups of one
    "c": BimolixConfig(vocab=130, width=128, norm_eps=1e-6, layers=(
        _r(2, 130, 48, (0.98, 0.9375), (64, 1000000.0), _moe(16, 1, 16, 1.0, groups=16, keep=3, shared=16,
                                                             shared_limit=1.0, scale=1.5)),
        _a(8, 8, 32, 1000, 32, 600.0, _dense(64)),
        _r(2, 130, 48, (0.98, 0.9375), (64, 1000000.0), _moe(16, 1, 16, 1.0, groups=16, keep=3, shared=16,
                                                             shared_limit=1.0, scale=1.5), weights_of=0),
        _a(8, 8, 32, 1000, 32, 600.0, _dense(64), weights_of=1),
        _r(2, 130, 48, (0.98, 0.9375), (64, 1000000.0), _moe(16, 1, 16, 1.0, groups=16, keep=3, shared=16,
                                                             shared_limit=1.0, scale=1.5), weights_of=2))),
    # a single head everywhere, a chunk of one position (a query sees itself alone), a table of two rows, one
    # group that holds all experts, width and vocabulary that are no multiples of four
    "d": BimolixConfig(vocab=101, width=50, norm_eps=1e-5, layers=(
        _a(1, 1, 7, 1, 2, 3.0, None),
        _r(1, 5, 3, (0.96875,), (2, 50.0), _moe(4, 2, 6, 1.0, groups=1, keep=1)),
        _a(1, 1, 12, 33, 9, 20.0, _moe(4, 2, 6, 1.0, groups=2, keep=1, shared=3, shared_limit=2.0)),
        _r(5, 4, 4, (1.0, 0.5, 0.9, 0.99, 0.999), (4, 7.0), _dense(11)))),
    # sizes of the usual kind (powers of two, heads of 64) with an attention layer first, values wider than
    # keys in the retention layers, experts in a retention layer, a chunk of several pages that long prompts
    # cross three times, and a table whose reach is the chunk
    "e": BimolixConfig(vocab=300, width=256, norm_eps=1e-6, layers=(
        _a(8, 2, 64, 128, 16, 128.0, _dense(512)),
        _r(4, 64, 128, (0.9375, 0.984375, 0.99609375, 0.9990234375), (64, 10000.0),
           _moe(8, 2, 64, 2.0, groups=4, keep=2, shared=64, shared_limit=2.0, scale=1.5)),
        _r(4, 64, 128, (0.9375, 0.984375, 0.99609375, 0.9990234375), (64, 10000.0),
           _moe(8, 2, 64, 2.0, groups=4, keep=2, shared=64, shared_limit=2.0, scale=1.5), weights_of=1),
        _a(8, 2, 64, 128, 16, 128.0, _dense(512), weights_of=0))),
}
BIMOLIX_SEEDS = {"a": 31, "b": 32, "c": 33, "d": 34, "e": 35}
BIMOLIX_PAGES = {"a": 16, "b": 8, "c": 16, "d": 4, "e": 32}


def tensors_of(config: BimolixConfig, seed: int) -> dict:
    """Checkpoint tensors (float32) of ``config``, drawn from ``seed``."""
    g = torch.Generator().manual_seed(seed)

    def matrix(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)

    def around_zero(n):
        return 0.3 * (torch.rand(n, generator=g) - 0.5)

    d = config.width
    t = {"embed": torch.randn(config.vocab, d, generator=g), "embed.norm": around_zero(d),
         "final.norm": around_zero(d), "head": matrix(config.vocab, d, 2.0)}
    for i, layer in enumerate(config.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{i}."
        t[p + "norm1"] = around_zero(d)
        hv = layer.heads * layer.vdim
        if layer.type == "retention":
            t[p + "mix.q"] = matrix(layer.heads * layer.dim, d, 1.5)
            t[p + "mix.k"] = matrix(layer.heads * layer.dim, d, 1.5)
            t[p + "mix.v"] = matrix(hv, d)
        else:
            t[p + "mix.q"] = matrix(layer.heads * layer.dim, d, 2.0)
            t[p + "mix.q.b"] = torch.randn(layer.heads * layer.dim, generator=g) * 0.5
            t[p + "mix.k"] = matrix(layer.kv_heads * layer.dim, d, 2.0)
            t[p + "mix.k.b"] = torch.randn(layer.kv_heads * layer.dim, generator=g) * 0.5
            t[p + "mix.q.norm"] = 1.0 + around_zero(layer.dim)
            t[p + "mix.k.norm"] = 1.0 + around_zero(layer.dim)
            t[p + "mix.rel"] = torch.randn(layer.rel_rows, layer.heads, generator=g) * 1.5
        t[p + "mix.g"] = matrix(hv, d, 2.0)
        t[p + "mix.o"] = matrix(d, hv)
        m = layer.mlp
        if m is None:
            continue
        t[p + "norm2"] = around_zero(d)
        if m.kind == "dense":
            t[p + "mlp.gate"] = matrix(m.ff, d, 1.5)
            t[p + "mlp.up"] = matrix(m.ff, d, 1.5)
            t[p + "mlp.down"] = matrix(d, m.ff)
            continue
        t[p + "mlp.router"] = matrix(m.experts, d, 6.0)
        t[p + "mlp.correction"] = torch.randn(m.experts, generator=g) * 0.4
        stems = [(f"mlp.e{e}", m.ff) for e in range(m.experts)] + ([("mlp.shared", m.shared_ff)] if m.shared_ff else [])
        for stem, ff in stems:
            t[p + stem + ".gate"] = matrix(ff, d, 2.0)
            t[p + stem + ".up"] = matrix(ff, d, 2.0)
            t[p + stem + ".down"] = matrix(d, ff)
        if m.shared_ff:
            t[p + "mlp.shared.sg"] = matrix(1, d, 3.0)
    return t


def write_folder(folder, config: BimolixConfig, seed: int, dtype=torch.float32):
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


def greedy_oracle(folder, prompt, new_tokens: int) -> list[int]:
    config, tensors = read_folder(folder)
    return plain.greedy(config, tensors, prompt, new_tokens)


def tokens_of(vocab: int, count: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]
