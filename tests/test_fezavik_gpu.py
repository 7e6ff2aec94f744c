"""Fezavik on the GPU against the plain implementation: each mechanism alone, then whole models through
the step function, the trace program and the generation entry point."""

import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_fezavik as plain
import replay_helpers as rh
from fezavik_configs import (FEZAVIK_CONFIGS, FEZAVIK_PAGES, FEZAVIK_SEEDS, greedy_oracle, oracle_logits,
                             tokens_of, write_folder)

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]
CUDA = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_folder(tmp_path_factory.mktemp(f"fezavik_{name}"), config, FEZAVIK_SEEDS[name])
            for name, config in FEZAVIK_CONFIGS.items()}


def close(got, want, dtype, scale=None, limit=None):
    scale = scale if scale is not None else max(want.abs().max().item(), 1e-6)
    limit = limit or (4e-6 if dtype == torch.float32 else 1.2e-2)
    worst = (got.double().cpu() - want.double().cpu()).abs().max().item() / scale
    assert worst <= limit, f"largest difference {worst:.3g} of the scale, allowed {limit:.3g}"


def rounded(t, dtype):
    """Values of ``t`` as ``dtype`` stores them, in float64."""
    return t.to(dtype).double()


def ints(values):
    return torch.tensor(values, dtype=torch.int32, device=CUDA)


def picking(first, count, width):
    """The matrix W with W x = x[first : first + count]."""
    w = torch.zeros(count, width, dtype=F64)
    w[torch.arange(count), first + torch.arange(count)] = 1.0
    return w


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("heads,dim,vdim", [(4, 16, 32), (3, 10, 7), (2, 6, 20), (2, 130, 48), (1, 5, 3), (5, 4, 4),
                                            (2, 64, 64), (1, 256, 40)])
def test_gated_recurrence_from_a_carried_state(heads, dim, vdim, dtype):
    """Five entries of one step: a long portion from a fresh state, a portion that continues a request from the
    state its earlier tokens left, two single tokens, and a portion of two.  In head 0 one channel writes token 2
    whole (its gate falls to 0 there) and keeps it ever after (its gate is 1 at every other token, so nothing
    else is written): the query 400 tokens later reads along that channel alone and must find token 2's
    value.  The state each entry leaves is the plain implementation's."""
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(heads * 1000 + dim)
    lengths, slots = [403, 40, 1, 1, 2], [3, 0, 5, 1, 4]
    tokens = sum(lengths)
    per = heads * dim
    cols = 2 * per + heads * vdim + 3
    q_at, f_at, v_at = 1, 2 + per, 3 + 2 * per
    proj = torch.randn(tokens, cols, generator=g)
    lower = 1.0 - torch.rand(per, generator=g) ** 3
    bias = torch.randn(per, generator=g)
    # channel 0 of head 0: bound 0, no bias; its gate is sigmoid of the projection: 0 at token 2, 1 elsewhere
    lower[0], bias[0] = 0.0, 0.0
    proj[:403, f_at] = 30.0
    proj[2, f_at] = -30.0
    proj[402, q_at:q_at + dim] = 0.0
    proj[402, q_at] = 9.0
    proj = rounded(proj, dtype)
    w = {"m.q": picking(q_at, per, cols), "m.f": picking(f_at, per, cols), "m.v": picking(v_at, heads * vdim, cols),
         "m.f.b": bias.double(), "m.lower": lower.double(), "m.norm": (1.0 + 0.2 * torch.randn(vdim, generator=g)).double(),
         "m.o": torch.eye(heads * vdim, dtype=F64)}
    mixer = {"heads": heads, "dim": dim, "vdim": vdim}
    eps = 1e-5
    state = torch.randn(6, heads, dim, vdim, generator=g) * 0.3
    state[3] = 0.0
    want, want_state, first = [], state.double().clone(), 0
    for length, slot in zip(lengths, slots):
        out, left = plain.gated_recurrence(proj[first:first + length], w, "m", mixer, eps, state=state[slot].double())
        want.append(out)
        want_state[slot] = left
        first += length
    want = torch.cat(want)
    row_starts = [0]
    for length in lengths:
        row_starts.append(row_starts[-1] + length)
    ways = [(lanes, 0) for lanes in [0] + [n for n in (4, 8, 16, 32) if n * 8 >= dim]]
    ways += [(0, 5), (32, 64), (0, 403), (0, None)]
    for lanes, segment in ways:
        device_state = state.to(CUDA)
        raw = torch.empty(tokens, heads * vdim, dtype=torch.float32, device=CUDA)
        got = kernels.gated_recurrence(
            proj.to(dtype).to(CUDA), q_at=q_at, g_at=f_at, v_at=v_at, heads=heads, dim=dim, vdim=vdim,
            state=device_state, row_starts=ints(row_starts), state_slots=ints(slots),
            token_row=ints([r for r, n in enumerate(lengths) for _ in range(n)]), bias=bias.to(CUDA),
            lower=lower.to(CUDA), query_act="silu", unit_norm=True, norm_weight=w["m.norm"].float().to(CUDA), eps=eps,
            raw_out=raw, lanes=lanes, segment=segment)
        close(got, want, dtype, limit=2e-5 if dtype == torch.float32 else None)
        close(device_state, want_state, torch.float32, limit=2e-5)
        v2 = proj[2, v_at:v_at + vdim]
        o = raw[402, :vdim].double().cpu()
        assert (o @ v2) / (o.norm() * v2.norm()) > 0.99           # the far token is what head 0 reads
        untouched = [s for s in range(6) if s not in slots]
        assert torch.equal(device_state[untouched].cpu(), state[untouched])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("heads,dim,vdim", [(4, 16, 32), (3, 10, 7), (2, 6, 20), (2, 130, 48), (1, 5, 3), (5, 4, 4),
                                            (2, 64, 64), (1, 256, 40), (2, 32, 260), (1, 48, 1024)])
def test_gated_recurrence_one_token_steps(heads, dim, vdim, dtype):
    """A step of single tokens runs as one launch: six requests from carried states in shuffled slots, one row of
    padding between them (no request: zeros out, no state touched), three steps in a row; outputs and states
    against the plain implementation and against the scan, which a step with one longer entry still takes."""
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(heads * 100 + vdim)
    rows, per = 7, heads * dim
    cols = 2 * per + heads * vdim + 5
    q_at, f_at, v_at = 2, 3 + per, 5 + 2 * per
    lower = 1.0 - torch.rand(per, generator=g) ** 3
    bias = torch.randn(per, generator=g)
    weight = 1.0 + 0.2 * torch.randn(vdim, generator=g)
    w = {"m.q": picking(q_at, per, cols), "m.f": picking(f_at, per, cols), "m.v": picking(v_at, heads * vdim, cols),
         "m.f.b": bias.double(), "m.lower": lower.double(), "m.norm": weight.double(), "m.o": torch.eye(heads * vdim, dtype=F64)}
    mixer = {"heads": heads, "dim": dim, "vdim": vdim}
    slots = [5, 2, 7, 0, 6, 1, 3]
    token_row = [0, 1, 2, -1, 4, 5, 6]                 # row 3 is padding
    state = torch.randn(8, heads, dim, vdim, generator=g) * 0.5
    device_state, scanned_state = state.to(CUDA), state.to(CUDA)
    want_state = state.double().clone()
    common = dict(q_at=q_at, g_at=f_at, v_at=v_at, heads=heads, dim=dim, vdim=vdim, row_starts=ints(list(range(rows + 1))),
                  state_slots=ints(slots), token_row=ints(token_row), bias=bias.to(CUDA), lower=lower.to(CUDA),
                  query_act="silu", unit_norm=True, norm_weight=weight.to(CUDA), eps=1e-5)
    for step in range(3):
        proj = rounded(torch.randn(rows, cols, generator=g), dtype)
        want = torch.zeros(rows, heads * vdim, dtype=F64)
        for r in range(rows):
            if token_row[r] < 0:
                continue
            want[r], want_state[slots[r]] = plain.gated_recurrence(proj[r:r + 1], w, "m", mixer, 1e-5,
                                                                   state=want_state[slots[r]])
        got = kernels.gated_recurrence(proj.to(dtype).to(CUDA), state=device_state, **common)
        raw = torch.empty(rows, heads * vdim, dtype=torch.float32, device=CUDA)
        by_scan = kernels.gated_recurrence(proj.to(dtype).to(CUDA), state=scanned_state, raw_out=raw, **common)
        close(got, want, dtype, limit=2e-5 if dtype == torch.float32 else None)
        close(by_scan, want, dtype, limit=2e-5 if dtype == torch.float32 else None)
        assert (got[3] == 0).all()
        close(device_state, want_state, torch.float32, limit=2e-5)
        assert torch.equal(device_state, scanned_state)          # both forms move the state by the same operations
    assert torch.equal(device_state[[4, 0]].cpu(), state[[4, 0]])  # nobody's slot and the padding row's


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_gated_recurrence_with_keys_of_its_own(dtype):
    """The scan's third form: a gate a channel beside keys that are not tied to it, against plain loops."""
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(5)
    heads, dim, vdim, tokens = 3, 12, 20, 70
    per = heads * dim
    proj = rounded(torch.randn(tokens, 3 * per + heads * vdim, generator=g), dtype)
    q, z, k = (proj[:, i * per:(i + 1) * per].view(tokens, heads, dim) for i in range(3))
    v = proj[:, 3 * per:].view(tokens, heads, vdim)
    gates = torch.sigmoid(z)
    s = torch.zeros(heads, dim, vdim, dtype=F64)
    want = []
    for t in range(tokens):
        s = gates[t][:, :, None] * s + k[t][:, :, None] * v[t][:, None, :]
        want.append(torch.einsum("hdv,hd->hv", s, q[t]).reshape(-1))
    want = torch.stack(want)
    for segment in (0, 16):
        state = torch.zeros(1, heads, dim, vdim, device=CUDA)
        raw = torch.empty(tokens, heads * vdim, dtype=torch.float32, device=CUDA)
        kernels.gated_recurrence(
            proj.to(dtype).to(CUDA), q_at=0, g_at=per, k_at=2 * per, v_at=3 * per, heads=heads, dim=dim, vdim=vdim,
            state=state, row_starts=ints([0, tokens]), state_slots=ints([0]), token_row=ints([0] * tokens),
            query_act=None, unit_norm=False, raw_out=raw, segment=segment)
        close(raw, want, torch.float32, limit=2e-5)
        close(state[0], s, torch.float32, limit=2e-5)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("experts,identity,top,ff,renormalise", [
    (8, 2, 3, 24, False), (3, 0, 3, 10, False), (16, 4, 1, 16, False), (2, 3, 5, 6, False), (5, 3, 2, 7, True),
    (40, 8, 6, 8, False)])
def test_softmax_routing_with_pass_through_slots(experts, identity, top, ff, renormalise, dtype):
    """Weights of every slot, the exact zeros of experts that were not chosen, the activation and the sum of the
    pass-through slots' weights against the plain routing; the correction is large enough to change choices."""
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(experts * 10 + top)
    tokens, slots = 37, experts + identity
    z = (torch.randn(tokens, slots, generator=g) * 2.0).float()
    correction = (torch.randn(slots, generator=g) * 0.3).float()
    proj = rounded(torch.randn(tokens, 2 * experts * ff, generator=g), dtype)
    want = torch.zeros(tokens, experts * ff, dtype=F64)
    want_w = torch.zeros(tokens, slots, dtype=F64)
    moved = 0
    for t in range(tokens):
        chosen = plain.route(z[t].double(), correction.double(), {"top": top})
        total = sum(weight for _, weight in chosen) if renormalise else 1.0
        plainly = set(torch.softmax(z[t].double(), -1).topk(top).indices.tolist())
        moved += plainly != {e for e, _ in chosen}
        for e, weight in chosen:
            want_w[t, e] = weight / total
            if e < experts:
                at = 2 * e * ff
                want[t, e * ff:(e + 1) * ff] = weight / total * plain.silu(proj[t, at:at + ff]) * proj[t, at + ff:at + 2 * ff]
    assert moved > 0 or top == slots
    weights_out = torch.empty(tokens, slots, dtype=torch.float32, device=CUDA)
    got, passed = kernels.route_softmax_gated(
        z.to(CUDA), proj.to(dtype).to(CUDA), experts=experts, identity=identity, top=top, ff=ff,
        correction=correction.to(CUDA), renormalise=renormalise, weights_out=weights_out)
    close(weights_out, want_w, torch.float32, scale=1.0)
    close(got, want, dtype)
    assert ((weights_out > 0).sum(1) == top).all()
    assert (got.view(tokens, experts, ff)[weights_out[:, :experts] == 0] == 0).all()     # exact zeros
    if identity:
        close(passed, want_w[:, experts:].sum(1), torch.float32, scale=1.0)
    else:
        assert passed is None


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("width", [50, 64, 384, 4096])
def test_a_norm_behind_and_a_norm_in_front(width, dtype):
    """stream + norm(y + scale * x) and the norm of the new stream in one pass, with and without the scaled term,
    the first norm, the second norm, and on gathered rows."""
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(width)
    tokens = 9
    stream = torch.randn(tokens, width, generator=g) * 3.0
    y = torch.randn(tokens, width, generator=g) * 7.0
    x = rounded(torch.randn(tokens, width, generator=g), dtype)
    scale = torch.rand(tokens, generator=g)
    post = rounded(1.0 + 0.3 * torch.randn(width, generator=g), dtype)
    pre = rounded(1.0 + 0.3 * torch.randn(width, generator=g), dtype)
    eps = 1e-5
    for carried in (False, True):
        for with_post in (True, False):
            t = y.double() + (scale.double()[:, None] * x if carried else 0.0)
            added = plain.rms_norm(t, post, eps) if with_post else t
            new = stream.double() + added
            want = plain.rms_norm(new, pre, eps)
            device_stream = stream.to(CUDA)
            out, updated = kernels.sandwich_norm(
                device_stream, y.to(CUDA), post_weight=post.to(dtype).to(CUDA) if with_post else None,
                pre_weight=pre.to(dtype).to(CUDA), post_eps=eps, pre_eps=eps,
                row_scale=scale.to(CUDA) if carried else None, x=x.to(dtype).to(CUDA) if carried else None,
                out_dtype=dtype)
            assert updated is device_stream
            close(device_stream, new, torch.float32, limit=2e-6)
            close(out, want, dtype, limit=2e-6 if dtype == torch.float32 else 6e-3)
            rows = ints([7, 0, 3])
            again = stream.to(CUDA)
            some, nothing = kernels.sandwich_norm(
                again, y.to(CUDA), post_weight=post.to(dtype).to(CUDA) if with_post else None,
                pre_weight=pre.to(dtype).to(CUDA), post_eps=eps, pre_eps=eps,
                row_scale=scale.to(CUDA) if carried else None, x=x.to(dtype).to(CUDA) if carried else None,
                rows=rows, out_dtype=dtype)
            assert nothing is None and torch.equal(again.cpu(), stream)          # gathered rows write nothing back
            assert torch.equal(some.cpu(), out.cpu()[[7, 0, 3]])
    only = stream.to(CUDA)
    out, _ = kernels.sandwich_norm(only, y.to(CUDA), post_weight=post.to(dtype).to(CUDA), post_eps=eps, out_dtype=dtype)
    assert out is None
    close(only, stream.double() + plain.rms_norm(y.double(), post, eps), torch.float32, limit=2e-6)
    added = y.to(CUDA).clone()
    kernels.add_scaled_rows(added, x.to(dtype).to(CUDA), scale.to(CUDA))
    close(added, y.double() + scale.double()[:, None] * x, torch.float32, limit=2e-6)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("pairing", ["half_split", "interleaved"])
def test_the_rotated_part_of_latent_rows_and_queries(pairing, dtype):
    """Both pairings in the kernel that writes the cached rows and in the one that turns the query heads."""
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(3)
    tokens, q_rank, rank, rot, heads = 11, 10, 12, 6, 3
    rotation = {"dims": rot, "base": 40.0}
    turn = plain.rotate_halves if pairing == "half_split" else plain.rotate_neighbours
    positions = torch.tensor([0, 1, 2, 3, 50, 51, 7, 300, 301, 302, 9])
    proj = rounded(torch.randn(tokens, q_rank + rank + rot, generator=g), dtype)
    q_w = rounded(1.0 + 0.2 * torch.randn(q_rank, generator=g), dtype)
    kv_w = rounded(1.0 + 0.2 * torch.randn(rank, generator=g), dtype)
    inv_freq = plain.frequencies(rotation, F64).float().to(CUDA)
    cache = torch.zeros(4, 1, 8, rank + rot, dtype=dtype, device=CUDA)
    slots = ints(list(range(tokens)))
    q_latent = kernels.latent_prepare(
        proj.to(dtype).to(CUDA), dq_at=0, q_rank=q_rank, q_weight=q_w.to(dtype).to(CUDA), dkv_at=q_rank, kv_rank=rank,
        kv_weight=kv_w.to(dtype).to(CUDA), rot_dim=rot, inv_freq=inv_freq, magnitude=1.0, positions=ints(positions.tolist()),
        slots=slots, key_cache=cache, eps=1e-5, pairing=pairing)
    close(q_latent, plain.rms_norm(proj[:, :q_rank], q_w, 1e-5), dtype, limit=1e-5 if dtype == torch.float32 else 6e-3)
    rows = cache.view(-1, rank + rot)[:tokens]
    close(rows[:, :rank], plain.rms_norm(proj[:, q_rank:q_rank + rank], kv_w, 1e-5), dtype,
          limit=1e-5 if dtype == torch.float32 else 6e-3)
    want = turn(proj[:, None, q_rank + rank:], positions, rotation)[:, 0]
    close(rows[:, rank:], want, dtype, limit=1e-4 if dtype == torch.float32 else 6e-3)
    src = rounded(torch.randn(tokens, heads, rot, generator=g), dtype)
    dst = torch.zeros(tokens, heads, rot + 2, dtype=dtype, device=CUDA)
    kernels.rotate_heads(src.to(dtype).to(CUDA), dst[:, :, 2:], inv_freq, 1.0, ints(positions.tolist()), pairing)
    close(dst[:, :, 2:], turn(src, positions, rotation), dtype, limit=1e-4 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("pairing", ["interleaved", "half_split"])
@pytest.mark.parametrize("heads,kv,dim,vdim,rot", [(4, 2, 16, 32, 8), (3, 1, 9, 5, 4), (8, 8, 32, 16, 32), (1, 1, 7, 7, 2),
                                                   (8, 2, 64, 64, 32)])
def test_norm_over_the_whole_projection_then_rotation_and_store(heads, kv, dim, vdim, rot, pairing, dtype):
    """One kernel: q and k normed over all heads at once, the first dimensions of every head turned by the
    position, q left in place, k and v in the token's cache rows; against the plain norm and rotation.  One
    token has no slot (a padding row): nothing of it is stored."""
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(heads * 10 + dim)
    tokens, page = 9, 4
    positions = torch.tensor([0, 1, 2, 3, 250, 251, 40, 7, 1000])
    slots = [5, 6, 7, 8, 0, 1, -1, 14, 19]
    q_cols, k_cols, v_cols = heads * dim, kv * dim, kv * vdim
    at = 8 if dim % 8 == 0 else 3
    proj = rounded(torch.randn(tokens, at + q_cols + k_cols + v_cols, generator=g) * 2.0, dtype)
    q_w = rounded(1.0 + 0.3 * torch.randn(q_cols, generator=g), dtype)
    k_w = rounded(1.0 + 0.3 * torch.randn(k_cols, generator=g), dtype)
    rotation = {"dims": rot, "base": 77.0}
    turn = plain.rotate_halves if pairing == "half_split" else plain.rotate_neighbours
    eps = 1e-5
    q = turn(plain.rms_norm(proj[:, at:at + q_cols], q_w, eps).view(tokens, heads, dim), positions, rotation)
    k = turn(plain.rms_norm(proj[:, at + q_cols:at + q_cols + k_cols], k_w, eps).view(tokens, kv, dim), positions, rotation)
    v = proj[:, at + q_cols + k_cols:].view(tokens, kv, vdim)
    device = proj.to(dtype).to(CUDA)
    keys = torch.full((5, kv, page, dim), 9.0, dtype=dtype, device=CUDA)
    values = torch.full((5, kv, page, vdim), 9.0, dtype=dtype, device=CUDA)
    kernels.projection_norm(
        device, [(at, q_cols, q_w.to(dtype).to(CUDA), False), (at + q_cols, k_cols, k_w.to(dtype).to(CUDA), False)],
        ints(positions.tolist()), eps,
        rotation=dict(inv_freq=plain.frequencies(rotation, F64).float().to(CUDA), rot_dims=rot, pairing=pairing, head_dim=dim),
        store=dict(slots=ints(slots), key_cache=keys, value_cache=values, v_at=at + q_cols + k_cols))
    limit = 2e-4 if dtype == torch.float32 else 8e-3             # float32 angles at position 1,000
    close(device[:, at:at + q_cols], q.reshape(tokens, -1), dtype, limit=limit)
    close(device[:, at + q_cols:at + q_cols + k_cols], k.reshape(tokens, -1), dtype, limit=limit)
    written = torch.zeros(5 * page, dtype=torch.bool)
    for t, slot in enumerate(slots):
        if slot < 0:
            continue
        written[slot] = True
        close(keys[slot // page, :, slot % page], k[t], dtype, limit=limit)
        assert torch.equal(values[slot // page, :, slot % page].cpu().double(), v[t])
    untouched = keys.permute(0, 2, 1, 3).reshape(5 * page, -1)[~written]
    assert (untouched == 9.0).all()


# ---------------------------------------------------------------- whole models
def requests_of(name):
    vocab = FEZAVIK_CONFIGS[name].vocab
    return {f"{name}{n}": tokens_of(vocab, n, 500 + n) for n in (1, 2, 37, 150, 420)}


def make_runner(folder, dtype, page, pages, max_len=None, max_requests=4):
    from tinyvllm_b200 import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.engine.step import StepRunner

    model = Model(read_model_config(folder).to_spec(), device=CUDA, dtype=dtype).load(folder)
    return StepRunner(model, page_size=page, num_pages=pages, max_requests=max_requests,
                      max_model_len=max_len or pages * page)


def compare(got: dict, folder, requests, dtype, routed=True):
    """float32: every row within rounding of the plain logits.  bfloat16 without routed experts (``routed``
    False): every row within the rounding of 16-bit activations.  bfloat16 with them: 16-bit activations move a
    choice score by a hundredth of its size, and a token whose last chosen slot led the next one by less than
    that goes another way than in the plain implementation; the norm behind the feed-forward gives its output
    the same size whichever way it went, so such a token moves by the whole size of a sublayer's output, and the
    tokens that attend it move with it.  Those rows are judged as a whole: a quarter of them within rounding,
    the median and nine rows in ten within what a few such tokens do (observed: first quartiles up to 0.010,
    medians up to 0.038, ninth deciles up to 0.15)."""
    expected = oracle_logits(folder, requests)
    assert got, "no logits came back"
    errors = []
    for (rid, position), row in got.items():
        want = expected[rid]
        assert torch.isfinite(row).all()
        errors.append((row.double() - want[position].double()).abs().max().item() / want.abs().max().item())
    errors.sort()
    if dtype == torch.float32:
        assert errors[-1] <= 5e-5, f"largest difference {errors[-1]:.3g} of the largest logit"
        return
    quarter, median, ninth = errors[len(errors) // 4], errors[len(errors) // 2], errors[len(errors) * 9 // 10]
    if not routed:
        assert median <= 1.2e-2 and errors[-1] <= 6e-2, f"median {median:.3g}, largest {errors[-1]:.3g} of the largest logit"
        return
    assert quarter <= 2e-2 and median <= 6e-2 and ninth <= 2.5e-1, \
        f"first quartile {quarter:.3g}, median {median:.3g}, ninth decile {ninth:.3g} of the largest logit"


def is_routed(name):
    return any(layer.mlp is not None for layer in FEZAVIK_CONFIGS[name].layers)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", sorted(FEZAVIK_CONFIGS))
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_every_way_of_cutting_gives_the_plain_logits(cut, name, dtype, folders):
    """Whole prompts; prompts whose last 40 tokens come one by one (the short windows pass over decoded tokens
    only); portions of changing size down to two tokens, cut inside pages and windows; up to four live
    requests with portions beside single tokens, in a pool with room for little more than the live tokens
    and four state slots, so that pages and slots that finished requests gave back are taken again."""
    requests = requests_of(name)
    page = FEZAVIK_PAGES[name]
    steps = {"whole": lambda: rh.whole(requests), "tail": lambda: rh.tail_by_one(requests, 40),
             "portions": lambda: rh.portions(requests, 3, sizes=(2, 3, 5, 8, 13, 31, 64, 100, 200)),
             "mixed": lambda: rh.mixed(requests, 4, live=4, decode_tail=20, sizes=(2, 3, 7, 16, 40, 90))}[cut]()
    pages = -(-rh.live_token_need(steps, page) // page) if cut == "mixed" else max(64, -(-448 // page))
    runner = make_runner(folders[name], dtype, page, pages)
    with torch.inference_mode():
        got = rh.run_steps(runner, steps)
    compare(got, folders[name], requests, dtype, routed=is_routed(name))
    assert not runner.manager.open_requests()
    assert all(runner.manager.free_pages(g) == pages for g in range(len(runner.manager.groups)))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_request_is_not_moved_by_its_neighbours(dtype, folders):
    """The same request alone and beside three others, in other pages and another state slot: equal beyond
    rounding."""
    name = "a"
    requests = requests_of(name)
    page = FEZAVIK_PAGES[name]
    alone = {"x": requests["a150"]}
    with torch.inference_mode():
        first = rh.run_steps(make_runner(folders[name], dtype, page, 64), rh.portions(alone, 9, sizes=(7, 50)))
        crowd = dict(list(requests.items())[2:])
        crowd["x"] = requests["a150"]
        second = rh.run_steps(make_runner(folders[name], dtype, page, 96), rh.mixed(crowd, 1, live=4, decode_tail=5))
    scale = oracle_logits(folders[name], alone)["x"].abs().max().item()
    errors = sorted((first[key].double() - second[key].double()).abs().max().item() / scale for key in first)
    if dtype == torch.float32:
        assert errors[-1] <= 2e-5
    else:
        assert errors[len(errors) * 39 // 40 - 1] <= 2e-2


def test_a_slot_that_is_taken_again_starts_from_zero(folders):
    """One state slot and pages for one request: the second request gets the slot and the pages the first
    one left, and its logits are those of a request that runs alone in a fresh pool."""
    name = "d"
    vocab = FEZAVIK_CONFIGS[name].vocab
    requests = {"one": tokens_of(vocab, 50, 1), "two": tokens_of(vocab, 45, 2)}
    runner = make_runner(folders[name], torch.float32, 4, 13, max_len=52, max_requests=1)
    with torch.inference_mode():
        got = rh.run_steps(runner, rh.portions(requests, 6, sizes=(2, 11, 30)))
    compare(got, folders[name], requests, torch.float32)


@pytest.mark.parametrize("name", ["a", "b"])
def test_long_decoding(name, folders):
    """A prompt of five tokens and 330 tokens decoded one by one, float32: the recurrent state runs along 335
    tokens, every window passes over decoded tokens many times and pages are given back on the way."""
    tokens = tokens_of(FEZAVIK_CONFIGS[name].vocab, 335, 9)
    requests = {"long": tokens}
    page = FEZAVIK_PAGES[name]
    runner = make_runner(folders[name], torch.float32, page, 352 // page, max_len=352)
    with torch.inference_mode():
        got = rh.run_steps(runner, rh.tail_by_one(requests, 330))
    compare(got, folders[name], requests, torch.float32)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_trace_program(dtype_name, folders, tmp_path):
    name = "b"
    requests = requests_of(name)
    steps = rh.mixed(requests, 2, live=3)
    need = rh.live_token_need(steps)
    lines = "\n".join(json.dumps(step) for step in steps) + "\n"
    out = tmp_path / "out"
    root = Path(__file__).resolve().parent.parent
    done = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folders[name]),
                           "--dtype", dtype_name, "--out", str(out), "--max-tokens", str(need)],
                          input=lines, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    got = rh.read_trace_output(steps, out, FEZAVIK_CONFIGS[name].vocab)
    compare(got, folders[name], requests, getattr(torch, dtype_name))


@pytest.mark.parametrize("eager", [True, False], ids=["eager", "graphs"])
@pytest.mark.parametrize("name", sorted(FEZAVIK_CONFIGS))
def test_greedy_generation_through_the_engine(name, eager, folders):
    """LLM.generate (scheduler, chunked prefill, decode graphs and runs of decode steps) against greedy
    decoding with the plain implementation, float32."""
    from tinyvllm_b200 import LLM, EngineConfig, SamplingParams

    config = FEZAVIK_CONFIGS[name]
    prompts = [tokens_of(config.vocab, n, 700 + n) for n in (1, 9, 40, 77, 130)]
    engine_config = EngineConfig(
        model=folders[name], dtype="float32", max_model_len=512, max_num_seqs=4, max_num_batched_tokens=64,
        prefill_chunk_size=24, kv_block_size=FEZAVIK_PAGES[name], kv_cache_memory_bytes=16 * 1024 * 1024,
        prefill_reserve_tokens=0, prefill_reserve_requests=0, enforce_eager=eager)
    with LLM(engine_config) as llm:
        outputs = llm.generate(prompts, SamplingParams(max_new_tokens=24, ignore_eos=True))
        if not eager:
            assert llm.engine.graph_steps > 0
    for prompt, output in zip(prompts, outputs):
        assert list(output.output_token_ids) == greedy_oracle(folders[name], prompt, 24)


def test_bfloat16_generation_through_the_engine(folders):
    from tinyvllm_b200 import LLM, EngineConfig, SamplingParams

    name = "a"
    config = FEZAVIK_CONFIGS[name]
    prompts = [tokens_of(config.vocab, n, 800 + n) for n in (70, 3)]
    engine_config = EngineConfig(
        model=folders[name], dtype="bfloat16", max_model_len=256, max_num_seqs=4, max_num_batched_tokens=64,
        prefill_chunk_size=32, kv_block_size=16, kv_cache_memory_bytes=8 * 1024 * 1024,
        prefill_reserve_tokens=0, prefill_reserve_requests=0)
    with LLM(engine_config) as llm:
        outputs = llm.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
    assert all(len(output.output_token_ids) == 12 for output in outputs)
    for prompt, output in zip(prompts, outputs):
        logits = oracle_logits(folders[name], {"g": prompt})["g"][-1]
        top = logits.topk(2).values
        if (top[0] - top[1]).item() > 0.05 * logits.abs().max().item():
            assert output.output_token_ids[0] == int(logits.argmax())


def test_bfloat16_steps_run_on_the_tensor_core_kernels(folders, monkeypatch):
    """Head sizes in steps of 16: prompt portions of both kinds of attention go to the tile kernel, decoded tokens
    to the kernel for single tokens, none to the row kernel; each call carries the window and the sinks, and the
    latent layer's also the gate of one number a head."""
    from tinyvllm_b200.ops import kernels

    seen = {"attention_tiles": [], "attention_tiles_singles": [], "attention_rows": []}
    for fn in seen:
        original = getattr(kernels, fn)

        def watched(*args, _original=original, _fn=fn, **kwargs):
            seen[_fn].append((kwargs.get("window"), kwargs.get("sinks") is not None, bool(kwargs.get("gate_per_head"))))
            return _original(*args, **kwargs)
        monkeypatch.setattr(kernels, fn, watched)
    name = "e"
    requests = {"t": tokens_of(FEZAVIK_CONFIGS[name].vocab, 90, 31)}
    runner = make_runner(folders[name], torch.bfloat16, 16, 16)
    with torch.inference_mode():
        rh.run_steps(runner, rh.tail_by_one(requests, 3))
    calls = [(layer.window, True, layer.type == "latent_attention") for layer in FEZAVIK_CONFIGS[name].layers
             if layer.type != "hgrn2"]
    assert seen["attention_tiles"] == calls                      # one prompt step
    assert seen["attention_tiles_singles"] == calls * 3          # three decoded tokens
    assert not seen["attention_rows"]


def test_command_line(folders, capsys):
    """python -m tinyvllm_b200 on a Fezavik folder: greedy tokens of the plain implementation, also
    streamed, and with weights drawn from a seed instead of the file."""
    from tinyvllm_b200.__main__ import main

    name = "b"
    prompts = [tokens_of(FEZAVIK_CONFIGS[name].vocab, n, 950 + n) for n in (3, 45)]
    want = [greedy_oracle(folders[name], prompt, 10) for prompt in prompts]
    common = ["--model", str(folders[name]), "--max-new-tokens", "10", "--ignore-eos", "--kv-cache-mib", "16",
              "--max-model-len", "256", "--kv-block-size", "8"]
    ids = [arg for prompt in prompts for arg in ("--prompt-ids", ",".join(map(str, prompt)))]
    main(common + ["--dtype", "float32", "--stream"] + ids)
    lines = [json.loads(line) for line in capsys.readouterr().out.strip().splitlines()]
    streamed = {0: [], 1: []}
    for line in lines[:-1]:
        streamed[line["prompt"]].append(line["token_id"])
    assert [streamed[0], streamed[1]] == want
    assert [record["output_token_ids"] for record in lines[-1]["outputs"]] == want
    main(common + ["--dtype", "bfloat16", "--random-weights", "7"] + ids)
    records = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["outputs"]
    assert [len(record["output_token_ids"]) for record in records] == [10, 10]
