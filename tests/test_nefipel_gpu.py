"""The Nefipel design on the GPU against the plain implementation (tests/plain_nefipel.py).

Mechanisms alone (the norm after the sum over the float32 stream; the projection's post-pass with
bias, head norm and both rotations; attention with an output gate; differential attention with its
two maps over shared values; the scored router with groups, identity experts and a gate row; the
expert and dense feed-forwards), then whole models of three small configurations: whole prompts,
prefill against token-by-token decoding, portions down to two tokens, unequal requests in one
batch against each alone, pages used again, the first tokens of a sequence, long decoding, and
greedy generation through `Engine` (scheduler, CUDA graphs, asynchronous scheduling, preemption).

Where random inputs would hide a fault, the inputs are made so that it shows: single tokens'
inputs are scaled so that their values dominate every later row, at page borders, at the borders
of the key segments that decoding cuts long contexts into, and hundreds of tokens back; a
correction large enough to decide the router's choice; a group whose best expert is not the
best overall.

Exactness is tested in float32 (differences of rounding order only); bfloat16 serving is
compared with the float32 oracle with a bound on the error of rounding.
"""
import math

import pytest
import torch

import plain_nefipel as plain
import tiny_nefipel as tiny
from gpu_util import Harness
from vosti_b200 import Engine, ops
from vosti_b200.config import PartSpec
from vosti_b200.config.nefipel import _attention, _feed_forward
from vosti_b200.engine.batch import StepEntry
from vosti_b200.engine.runner import ModelRunner
from vosti_b200.parts import build_feed_forward, build_mixer

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32 = dict(atol=3e-4, rtol=3e-4)


def rounded(*shape, gen, std=1.0, mean=0.0):
    """Random values that bfloat16 holds exactly, as float32 on the CPU."""
    return (mean + std * torch.randn(tuple(shape), generator=gen)).to(torch.bfloat16).float()


def give(part, W, dtype):
    """Hand a part its tensors (keys of `weight_specs`) on the device in the serving layout."""
    assert set(W) == set(part.weight_specs()), (sorted(W), sorted(part.weight_specs()))
    store = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    part.load({k: v.to(DEV, store).contiguous() for k, v in W.items()}, dtype)
    part.setup(torch.device(DEV), dtype)


def weights_of(part, gen):
    return {key: tiny.draw("l0.mix." + key, tuple(w.shape), gen).to(torch.bfloat16).float() for key, w in part.weight_specs().items()}


class Ctx:
    """What a part that keeps nothing needs of a step's context."""

    def __init__(self, dtype):
        self.dtype, self.extras = dtype, {}
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.num_tokens, self.all_decode = 0, False


def run_mixer(mixer, harness, x, sizes, dtype, rid="r"):
    outs, at = [], 0
    for size in sizes:
        ctx = harness.context([StepEntry(rid, [0] * size)])
        outs.append(ops.materialize(mixer.forward(ctx, x[at:at + size].to(DEV, dtype).contiguous(), harness.cache.layer_caches[0])).float().cpu())
        at += size
    assert int(harness.status.item()) == 0
    return torch.cat(outs)


def close(got, want, dtype, what=None):
    if dtype == torch.float32:
        assert torch.allclose(got, want, **F32), (what, float((got - want).abs().max()))
    else:
        assert float((got - want).abs().mean() / want.abs().mean()) < 0.04, what


CUTS = lambda T: ((T,), (T - 33,) + (1,) * 33, (2, 5, 1, 1, 17, 2, 3, T - 31))


# ---------------------------------------------------------------- the norm after the sum
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [200, 67, 1, 4, 1028, 4099])
def test_norm_after_the_sum_over_the_stream(dtype, width):
    gen = torch.Generator().manual_seed(width)
    rows, eps, alpha = 9, 3e-6, 2.25
    stream = 1.5 * torch.randn(rows, width, generator=gen)
    y = rounded(rows, width, gen=gen, std=3.0, mean=0.5)
    z = rounded(rows, width, gen=gen, std=0.7)
    w = rounded(width, gen=gen, std=0.2, mean=1.0)
    store = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    for terms, total in (((y,), alpha * stream.double() + y.double()), ((y, z), alpha * stream.double() + y.double() + z.double())):
        want = plain.rms_norm(total, w.double(), eps)
        x = terms[0].to(DEV) if len(terms) == 1 else ops.DeferredSum(terms[0].to(DEV), terms[1].to(DEV, store))
        for in_place in (False, True):
            old = stream.to(DEV).clone()
            pair = ops.post_norm_stream(old, x, w.to(DEV, store), alpha, eps, dtype, in_place=in_place)
            assert pair.stream.dtype == torch.float32 and pair.rounded.dtype == dtype
            assert (pair.stream.data_ptr() == old.data_ptr()) == in_place
            assert torch.allclose(pair.stream.cpu(), want.float(), atol=2e-5, rtol=2e-5)
            assert torch.equal(pair.rounded.float(), pair.stream.to(dtype).float())       # the same numbers, rounded once
            if not in_place:
                assert torch.equal(old.cpu(), stream)


# ---------------------------------------------------------------- both kinds of attention
YARN = dict(factor=3.0, original=48, fast=4.0, slow=1.0)


def mixer_block(heads, kv, dim, vdim, dims, scaling, diff=None):
    return tiny._mixer(heads, kv, dim, vdim, 3.0 / math.sqrt(dim), 300.0, dims, scaling, diff)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dk,dv,dims,scaling,page", [
    (4, 2, 24, 16, 8, YARN, 8), (2, 1, 16, 40, 2, None, 8), (3, 3, 8, 8, 8, YARN, 4), (1, 1, 34, 10, 6, None, 4),
    (4, 2, 64, 64, 32, dict(factor=8.0, original=64, fast=8.0, slow=1.0), 16), (2, 2, 128, 128, 128, None, 16),
    (6, 1, 64, 64, 64, YARN, 16), (2, 1, 136, 200, 32, YARN, 8)])
def test_gated_attention_mixer_against_plain(dtype, heads, kv, dk, dv, dims, scaling, page):
    gen = torch.Generator().manual_seed(heads * 100 + dk)
    width, T, eps = 72, 150, 1e-5
    block = mixer_block(heads, kv, dk, dv, dims, scaling)
    mixer = build_mixer(_attention(0, block, eps, False), width, None)
    assert {"q.b", "k.b", "v.b", "q.norm", "k.norm", "g"} <= set(mixer.weight_specs())
    W = weights_of(mixer, gen)
    give(mixer, W, dtype)
    x = rounded(T, width, gen=gen)
    want = plain.gated_attention(x.double(), {k: v.double() for k, v in W.items()}, block, eps).float()
    for sizes in CUTS(T):
        harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=-(-T // page) + 1, page_size=page)
        close(run_mixer(mixer, harness, x, sizes, dtype), want, dtype, sizes)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dk,dv,dims,scaling,diff,page", [
    (3, 1, 10, 14, 6, YARN, 0.2, 8), (2, 2, 20, 8, 20, None, 0.45, 8), (1, 1, 2, 3, 2, YARN, 0.1, 4), (4, 2, 64, 64, 64, YARN, 0.3, 16),
    (2, 1, 32, 96, 16, None, 0.25, 16), (8, 2, 40, 88, 40, dict(factor=4.0, original=64, fast=16.0, slow=2.0), 0.7, 8),
    (2, 1, 128, 256, 64, None, 0.5, 16), (4, 2, 64, 128, 64, YARN, 0.3, 16), (2, 1, 128, 64, 32, None, 0.2, 16), (6, 2, 128, 128, 128, None, 0.4, 32),
    (2, 2, 64, 64, 16, None, 0.3, 8)])
def test_differential_attention_mixer_against_plain(dtype, heads, kv, dk, dv, dims, scaling, diff, page):
    gen = torch.Generator().manual_seed(heads * 100 + dk + 1)
    width, T, eps = 72, 150, 1e-5
    block = mixer_block(heads, kv, dk, dv, dims, scaling, diff)
    mixer = build_mixer(_attention(0, block, eps, True), width, None)
    assert {"lq1", "lk1", "lq2", "lk2", "q.norm", "k.norm"} <= set(mixer.weight_specs()) and "g" not in mixer.weight_specs()
    assert tuple(mixer.weight_specs()["q"].shape) == (heads * 2 * dk, width)
    W = weights_of(mixer, gen)
    give(mixer, W, dtype)
    assert mixer.lam == pytest.approx(plain.differential_lambda({k: v.double() for k, v in W.items()}, diff), rel=1e-5)
    # in bfloat16 the maps run as heads of their own where the tensor-core kernels take the wider of the two widths
    assert mixer.expanded == (max(dk, dv) if dtype == torch.bfloat16 and max(dk, dv) in (64, 128) else 0)
    assert mixer.cache_spec().heads == (2 * kv if mixer.expanded else kv)
    x = rounded(T, width, gen=gen)
    want = plain.differential_attention(x.double(), {k: v.double() for k, v in W.items()}, block, eps).float()
    for sizes in CUTS(T):
        harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=-(-T // page) + 1, page_size=page)
        close(run_mixer(mixer, harness, x, sizes, dtype), want, dtype, sizes)


@pytest.mark.parametrize("differential", [False, True])
@pytest.mark.parametrize("dk,dv,page", [(24, 16, 8), (64, 64, 16), (32, 96, 16)])
def test_tokens_far_back_and_at_borders_whose_values_dominate(differential, dk, dv, page):
    """The inputs of single tokens are made two thousand times larger: their keys keep their size (the head
    norm), their values grow, so that every later row is mostly theirs and a kernel that loses one of
    them (the first token, the ends of pages, the ends of the key segments of 256 that decoding cuts
    a long context into, a token hundreds back) is far off. Prompt, then single tokens."""
    gen = torch.Generator().manual_seed(dk + dv)
    width, T, eps = 64, 700, 1e-5
    block = mixer_block(4, 2, dk, dv, 8, None, 0.3 if differential else None)
    x = rounded(T, width, gen=gen)
    marked = [0, page - 1, page, 255, 256, 300, 511, 512, 640, 641]
    for dtype in (torch.float32, torch.bfloat16):
        mixer = build_mixer(_attention(0, block, eps, differential), width, None)
        W = weights_of(mixer, torch.Generator().manual_seed(7))
        if not differential:
            W["v.b"] = torch.zeros_like(W["v.b"])
        give(mixer, W, dtype)
        fn = plain.differential_attention if differential else plain.gated_attention
        for j in marked:
            big = x.clone()
            big[j] *= 2000.0
            want = fn(big.double(), {k: v.double() for k, v in W.items()}, block, eps).float()
            lost = fn(torch.cat([big[:j], big[j + 1:]]).double(), {k: v.double() for k, v in W.items()}, block, eps).float()
            assert float((lost[-45:] - want[-45:]).abs().mean() / want[-45:].abs().mean()) > 0.3     # it matters
            for sizes in ((T,), (T - 40,) + (1,) * 40):
                harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=-(-T // page) + 1, page_size=page)
                got = run_mixer(mixer, harness, big, sizes, dtype)
                close(got[-45:], want[-45:], dtype, (j, sizes))


def test_projection_post_pass_alone():
    """Bias, head norm and both rotations on a given projection, queries and cached keys and values."""
    gen = torch.Generator().manual_seed(11)
    for maps, interleaved, nq, nkv, dk, dv, dims, extra in ((1, False, 4, 2, 24, 16, 8, 5), (2, True, 3, 1, 10, 14, 6, 0), (2, False, 2, 2, 16, 8, 16, 3),
                                                            (1, True, 2, 1, 64, 64, 64, 128)):
        T, page, eps = 21, 4, 1e-5
        width = (nq + nkv) * maps * dk + nkv * dv
        proj = torch.randn(T, width + extra, generator=gen)
        bias = torch.randn(width, generator=gen)
        qn, kn = 1 + 0.2 * torch.randn(dk, generator=gen), 1 + 0.2 * torch.randn(dk, generator=gen)
        rot = dict(base=200.0, dims=dims, scaling=YARN)
        freqs, magnitude = plain.rotation_frequencies(200.0, dims, YARN)
        pos = torch.arange(T)
        full = (proj[:, :width] + bias).double()
        q = plain.rotate(plain.rms_norm(full[:, :nq * maps * dk].view(T, nq * maps, dk), qn.double(), eps), pos, rot, interleaved)
        k = plain.rotate(plain.rms_norm(full[:, nq * maps * dk:(nq + nkv) * maps * dk].view(T, nkv * maps, dk), kn.double(), eps), pos, rot, interleaved)
        v = full[:, (nq + nkv) * maps * dk:].view(T, nkv, dv)
        pages = -(-T // page)
        k_cache = torch.zeros(pages, nkv, page, maps * dk, device=DEV)
        v_cache = torch.zeros(pages, nkv, page, dv, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        slots = torch.arange(T, dtype=torch.int32, device=DEV)
        got = ops.qkv_heads(proj.to(DEV), k_cache, v_cache, nq=nq, nkv=nkv, maps=maps, dk=dk, dv=dv, page_size=page,
                            positions=pos.to(DEV, torch.int32), slot_mapping=slots, out_dtype=torch.float32, status=status,
                            bias=bias.to(DEV), q_norm=qn.to(DEV), k_norm=kn.to(DEV), eps=eps,
                            freq=torch.tensor(freqs, dtype=torch.float32, device=DEV), interleaved=interleaved, magnitude=magnitude)
        assert int(status.item()) == 0
        assert torch.allclose(got.cpu().view(T, nq * maps, dk), q.float(), atol=2e-5, rtol=2e-5)
        k_got = k_cache.permute(0, 2, 1, 3).reshape(pages * page, nkv * maps, dk)[:T].cpu()       # [token, kv head x map, dk]
        v_got = v_cache.permute(0, 2, 1, 3).reshape(pages * page, nkv, dv)[:T].cpu()
        assert torch.allclose(k_got, k.float(), atol=2e-5, rtol=2e-5)
        assert torch.allclose(v_got, v.float(), atol=2e-5, rtol=2e-5)
        # every map a head of its own, D wide: zeros after a head's own elements, a kv head's values once per map
        D = max(dk, dv) + 8
        k_wide = torch.full((pages, nkv * maps, page, D), 7.0, device=DEV)
        v_wide = torch.full((pages, nkv * maps, page, D), 7.0, device=DEV)
        wide = ops.qkv_heads(proj.to(DEV), k_wide, v_wide, nq=nq, nkv=nkv, maps=maps, dk=dk, dv=dv, page_size=page,
                             positions=pos.to(DEV, torch.int32), slot_mapping=slots, out_dtype=torch.float32, status=status,
                             bias=bias.to(DEV), q_norm=qn.to(DEV), k_norm=kn.to(DEV), eps=eps,
                             freq=torch.tensor(freqs, dtype=torch.float32, device=DEV), interleaved=interleaved, magnitude=magnitude,
                             expanded_width=D).cpu().view(T, nq * maps, D)
        assert torch.equal(wide[..., :dk], got.cpu().view(T, nq * maps, dk)) and not wide[..., dk:].any()
        k_rows = k_wide.permute(0, 2, 1, 3).reshape(pages * page, nkv * maps, D)[:T].cpu()
        v_rows = v_wide.permute(0, 2, 1, 3).reshape(pages * page, nkv, maps, D)[:T].cpu()
        assert torch.equal(k_rows[..., :dk], k_got) and not k_rows[..., dk:].any()
        assert all(torch.equal(v_rows[:, :, m, :dv], v_got) for m in range(maps)) and not v_rows[..., dv:].any()


# ---------------------------------------------------------------- feed-forwards
@pytest.mark.parametrize("routed,identity,groups,keep,top,gate", [
    (9, 3, 3, 2, 3, True), (5, 0, 1, 1, 2, False), (2, 1, 2, 1, 1, False), (16, 4, 4, 2, 4, True), (18, 6, 2, 1, 2, True),
    (64, 0, 8, 3, 6, False), (3, 0, 1, 1, 3, True), (40, 8, 40, 5, 5, False)])
def test_scored_router_against_plain(routed, identity, groups, keep, top, gate):
    gen = torch.Generator().manual_seed(routed * 10 + top)
    tokens, k = 300, 72
    x = rounded(tokens, k, gen=gen)
    router = 2.0 / math.sqrt(k) * torch.randn(routed + int(gate), k, generator=gen)
    correction = 0.1 * torch.randn(routed, generator=gen)
    r = dict(experts=routed - identity, identity=identity, top=top, groups=dict(count=groups, keep=keep) if groups > 1 else None)
    for corr in (correction, 10.0 * correction):        # the second decides the choice alone
        want_chosen, want_weights = plain.route(x.double(), {"router": router[:routed].double(), "correction": corr.double()}, r)
        chosen, weights, dense, ident, logits = ops.moe_router_scored(
            x.to(DEV), router.to(DEV), top, identity=identity, correction=corr.to(DEV), groups=groups, keep=keep, gate_row=gate,
            want_logits=True)
        assert torch.allclose(logits.cpu(), (x @ router.T), atol=1e-5, rtol=1e-5)
        # a choice may differ where two corrected scores are equal to rounding: then the sets differ in members of equal score
        got_sets, want_sets = [set(row) for row in chosen.cpu().tolist()], [set(row) for row in want_chosen.tolist()]
        same = [g == w for g, w in zip(got_sets, want_sets)]
        assert sum(same) >= tokens - 2
        order = want_chosen.sort(-1)
        got_order = chosen.cpu().long().sort(-1)
        for t in range(tokens):
            if same[t]:
                assert torch.allclose(weights.cpu()[t][got_order.indices[t]], want_weights[t][order.indices[t]].float(), atol=1e-5, rtol=1e-4)
        assert torch.allclose(weights.sum(-1).cpu(), torch.ones(tokens), atol=1e-5)
        experts = routed - identity
        assert tuple(dense.shape) == (tokens, experts + int(gate))
        rebuilt = torch.zeros(tokens, routed)
        rebuilt.scatter_(1, chosen.cpu().long(), weights.cpu())
        assert torch.equal(dense.cpu()[:, :experts], rebuilt[:, :experts])
        if identity:
            assert torch.allclose(ident.cpu(), rebuilt[:, experts:].sum(-1), atol=1e-6)
        else:
            assert ident is None
        if gate:
            assert torch.allclose(dense.cpu()[:, experts], torch.sigmoid(x @ router[routed]), atol=1e-5)
        if groups > 1:
            per = routed // groups
            assert all(len({e // per for e in row}) <= keep for row in got_sets)


def test_a_group_is_judged_by_its_best_expert_and_unkept_experts_are_never_chosen():
    """Expert 0 has the best score of all but sits in a group whose rival group holds the two next
    best; with one group kept and two chosen, the router keeps group 0 (its best expert wins) and
    must take its second pick from group 0 too, however poor. Negative corrected scores are legal."""
    k = 8
    x = torch.zeros(1, k)
    x[0, 0] = 1.0
    router = torch.zeros(6, k)
    router[:, 0] = torch.tensor([3.0, -4.0, -5.0, 2.5, 2.4, 2.3])
    correction = torch.full((6,), -1.0)                  # every corrected score is negative
    chosen, weights, dense, ident = ops.moe_router_scored(x.to(DEV), router.to(DEV), 2, correction=correction.to(DEV), groups=2, keep=1)
    assert sorted(chosen.cpu().tolist()[0]) == [0, 1]
    want_chosen, want_weights = plain.route(x.double(), {"router": router.double(), "correction": correction.double()},
                                            dict(experts=6, top=2, groups=dict(count=2, keep=1)))
    assert sorted(want_chosen.tolist()[0]) == [0, 1]
    assert torch.allclose(weights.cpu().sort().values, want_weights.float().sort().values, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mlp", [tiny.moe(6, 3, 20, identity=3, groups=(3, 2), shared=36), tiny.moe(5, 2, 24), tiny.moe(1, 1, 48, identity=1, groups=(2, 1)),
                                 tiny.moe(12, 4, 32, identity=4, groups=(4, 2), shared=64), tiny.moe(3, 1, 16, shared=8), tiny.dense(100), tiny.dense(64)])
def test_feed_forwards_against_plain(dtype, mlp):
    gen = torch.Generator().manual_seed(5)
    width, tokens = 72 if mlp.get("ff", 0) != 64 else 128, 90
    part = build_feed_forward(_feed_forward(0, mlp), width)
    W = {key: tiny.draw("l0.mlp." + key, tuple(w.shape), gen).to(torch.bfloat16).float() for key, w in part.weight_specs().items()}
    if mlp["kind"] == "moe":
        W["router"] = (3.0 * W["router"]).to(torch.bfloat16).float()          # decided choices: bfloat16 inputs must not flip them
    give(part, W, dtype)
    fn = plain.dense_feed_forward if mlp["kind"] == "dense" else (lambda h, w: plain.expert_feed_forward(h, w, mlp))
    # a step of few tokens (all experts side by side in one product) and a long portion (rows sorted by expert,
    # here also for few experts a pick)
    part.GROUPED_MIN_RATIO = 0
    for tokens in (90, 300):
        x = rounded(tokens, width, gen=gen)
        want = fn(x.double(), {k: v.double() for k, v in W.items()}).float()
        got = ops.materialize(part.forward(Ctx(dtype), x.to(DEV, dtype))).float().cpu()
        assert got.dtype == torch.float32
        if dtype == torch.float32:
            assert torch.allclose(got, want, atol=1e-3, rtol=3e-4), (tokens, float((got - want).abs().max()))
        else:
            assert float((got - want).abs().mean() / want.abs().mean()) < 0.02, tokens
    if mlp["kind"] == "moe":
        routed = mlp["router"]["experts"] + (mlp["router"].get("identity") or 0)
        assert bool(part.per_expert) == (mlp["router"]["top"] < routed)


# ---------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (config, seed) in tiny.ALL.items():
        folder = tiny.write_model(tmp_path_factory.mktemp(f"nefipel_{name}"), config, seed)
        _, tensors = tiny.tensors_for(config, seed)
        out[name] = (folder, config, tensors)
    return out


def prompt(config, n, seed):
    return torch.randint(0, config["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def logits_of(config, W, tokens):
    return plain.forward(config, W, tokens).float()


def close_rows(got, want, dtype):
    """float32: every row equal up to rounding order. bfloat16: most rows within the rounding of a
    few 8-bit roundings a layer; a row whose router input rounds to another choice may lie further."""
    err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
    if dtype == "float32":
        return bool(err.max() < 2e-4)
    return bool(err.median() < 0.03 and err.quantile(0.9) < 0.1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_whole_prompt_portions_and_decoding_against_plain(models, name, dtype):
    folder, config, W = models[name]
    tokens = prompt(config, 77, 1)
    want = logits_of(config, W, tokens)
    for sizes in ((77,), (45,) + (1,) * 32, (2, 5, 1, 1, 17, 2, 3, 30, 16), (3, 2, 2, 70)):
        page = tiny.PAGE[name]
        runner = ModelRunner(folder, dtype=dtype, num_pages=96 // page, page_size=page, max_requests=2)
        runner.begin("r")
        rows, at = [], 0
        for size in sizes:
            rows.append(runner.step([StepEntry("r", tokens[at:at + size], list(range(size)))]).cpu())
            at += size
        runner.check_status()
        assert close_rows(torch.cat(rows), want, dtype), sizes


WIDE = dict(architecture="Nefipel", vocab=512, width=1024, norm=dict(eps=1e-5), postln_alpha=2.0, embedding=dict(scale=32.0), layers=[
    tiny.gated(8, 2, 128, 128, 0.27, 10000.0, 64, None, tiny.dense(2048)),
    tiny.differential(8, 2, 64, 128, 0.38, 500000.0, 64, dict(factor=8.0, original=64, fast=32.0, slow=1.0), 0.3,
                      tiny.moe(4, 2, 512, identity=2, groups=(2, 1), shared=512)),
    tiny.differential(4, 4, 128, 128, 0.27, 10000.0, 128, None, 0.2, tiny.moe(6, 2, 256)),
])


def test_wide_layers_whose_products_split_their_inner_range(tmp_path):
    """Layer sizes at which the bfloat16 products of a few tokens split their inner range: the kernels
    after them (head post-pass, norm after the sum) add the unsummed splits themselves; the dense
    feed-forward's relu(gate) * up is the product's own last step; both differential layers run their
    maps as heads of their own. Prompt of a few tokens, then token by token, against the plain form."""
    assert ops.library().vosti_gemm_tc_splits(1, 1024, 2048) > 1 and ops.library().vosti_gemm_tc_splits(4, 3072, 1024) > 1
    folder = tiny.write_model(tmp_path / "wide", WIDE, 77)
    _, W = tiny.tensors_for(WIDE, 77)
    tokens = prompt(WIDE, 40, 8)
    want = logits_of(WIDE, W, tokens)
    for dtype in ("bfloat16", "float32"):
        runner = ModelRunner(folder, dtype=dtype, num_pages=4, page_size=16, max_requests=2)
        if dtype == "bfloat16":
            assert [b.mixer.expanded for b in runner.model.blocks] == [0, 128, 128] and runner.model.blocks[0].feed_forward.fused
        runner.begin("r")
        rows = [runner.step([StepEntry("r", tokens[:4], [0, 1, 2, 3])]).cpu()]
        rows += [runner.step([StepEntry("r", [t], [0])]).cpu() for t in tokens[4:]]
        runner.check_status()
        assert close_rows(torch.cat(rows), want, dtype), dtype


def test_a_checkpoint_without_the_unused_norm_gives_the_same_logits(models, tmp_path):
    folder, config, W = models["a"]
    bare = tiny.write_model(tmp_path / "bare", config, tiny.ALL["a"][1], unused=False)
    tokens = prompt(config, 19, 3)
    rows = []
    for f in (folder, bare):
        runner = ModelRunner(f, dtype="float32", num_pages=8, page_size=8, max_requests=1)
        runner.begin("r")
        rows.append(runner.step([StepEntry("r", tokens, list(range(19)))]).cpu())
    assert torch.equal(rows[0], rows[1])


def test_first_tokens_of_a_sequence(models):
    """Requests of one, two and three tokens, and the first rows of a longer one: a softmax over one
    key (the differential maps then cancel up to lambda), position zero (no rotation)."""
    for name in ("a", "b", "c"):
        folder, config, W = models[name]
        page = tiny.PAGE[name]
        runner = ModelRunner(folder, dtype="float32", num_pages=32 // page, page_size=page, max_requests=2)
        for n in (1, 2, 3, 9):
            tokens = prompt(config, n, 40 + n)
            runner.begin("r")
            got = runner.step([StepEntry("r", tokens, list(range(n)))]).cpu()
            runner.finish("r")
            assert close_rows(got, logits_of(config, W, tokens), "float32"), (name, n)
        runner.check_status()


def test_residual_stream_after_every_layer(models):
    for name in ("a", "c"):
        folder, config, W = models[name]
        tokens = prompt(config, 23, 2)
        want = []
        plain.forward(config, W, tokens, streams=want)
        page = tiny.PAGE[name]
        runner = ModelRunner(folder, dtype="float32", num_pages=32 // page, page_size=page, max_requests=1)
        streams = []
        for block in runner.model.blocks:
            inner = block.forward

            def watched(ctx, hidden, residual, cache, writes_cache=True, inner=inner):
                pair, none = inner(ctx, hidden, residual, cache, writes_cache)
                streams.append(pair.stream.cpu().clone())
                return pair, none
            block.forward = watched
        runner.begin("r")
        runner.step([StepEntry("r", tokens, [0])])
        assert len(streams) == len(want) == len(config["layers"])
        for i, (got, expected) in enumerate(zip(streams, want)):
            assert torch.allclose(got, expected.float(), atol=3e-4, rtol=3e-4), (name, i)


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("c", "float32"), ("c", "bfloat16"), ("a", "bfloat16")])
def test_unequal_requests_in_one_batch_with_pages_used_again(models, name, dtype):
    """Four requests through two request slots and a pool that holds two of them: portions of some
    beside single tokens of others; every request equals itself alone."""
    folder, config, W = models[name]
    lengths = {"a": 37, "b": 9, "c": 1, "d": 26}
    tokens = {r: prompt(config, n, 10 + i) for i, (r, n) in enumerate(lengths.items())}
    want = {r: logits_of(config, W, t) for r, t in tokens.items()}
    page = tiny.PAGE[name]
    pool = 80 // page
    runner = ModelRunner(folder, dtype=dtype, num_pages=pool, page_size=page, max_requests=2)
    schedule = [
        [("a", 5), ("b", 2)], [("a", 1), ("b", 6)], [("b", 1), ("a", 20)], [("a", 1)],      # b ends in step 2
        [("c", 1), ("a", 2)], [("d", 3), ("a", 8)], [("d", 1)], [("d", 22)],                # c, then a end
    ]
    at = {r: 0 for r in lengths}
    got = {r: [] for r in lengths}
    for step in schedule:
        entries = []
        for r, n in step:
            if r not in runner.cache.live:
                runner.begin(r)
            entries.append(StepEntry(r, tokens[r][at[r]:at[r] + n], list(range(n))))
        logits = runner.step(entries).cpu()
        row = 0
        for r, n in step:
            got[r].append(logits[row:row + n])
            row += n
            at[r] += n
            if at[r] == lengths[r]:
                runner.finish(r)
    runner.check_status()
    runner.cache.check()
    for r in lengths:
        assert at[r] == lengths[r]
        assert close_rows(torch.cat(got[r]), want[r], dtype), r
    assert runner.cache.available_pages() == pool


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("c", "float32"), ("c", "bfloat16")])
def test_long_decoding_over_several_key_segments(models, name, dtype):
    """A prompt, then token by token until the context is several of the key segments long that decoding
    cuts it into, with a pool little larger than the context."""
    folder, config, W = models[name]
    tokens = prompt(config, 600, 4)
    want = logits_of(config, W, tokens)
    page = tiny.PAGE[name]
    runner = ModelRunner(folder, dtype=dtype, num_pages=608 // page, page_size=page, max_requests=1)
    runner.begin("r")
    rows = [runner.step([StepEntry("r", tokens[:440], list(range(440)))]).cpu()]
    rows += [runner.step([StepEntry("r", [t], [0])]).cpu() for t in tokens[440:]]
    runner.check_status()
    assert close_rows(torch.cat(rows), want, dtype)


@pytest.mark.parametrize("name,dtype,binary", [("a", "float32", True), ("c", "bfloat16", False), ("b", "float32", False)])
def test_trace_replay_of_a_mixed_schedule(models, name, dtype, binary, tmp_path):
    """The trace runner (the program itself, and the class it wraps) over a schedule of up to four
    live requests, portions beside single tokens, requests that sit a step out and a pool smaller
    than the sum of all requests: every row against the plain implementation of the request alone."""
    import numpy as np
    import replay_util as R
    folder, config, W = models[name]
    requests = {f"q{i}": prompt(config, n, 60 + i) for i, n in enumerate([70, 40, 33, 90, 64, 21])}
    steps = R.number(R.mixed_steps(requests, seed=5))
    max_tokens = R.max_live_tokens(steps)
    assert max_tokens < sum(R.roundup64(len(t)) for t in requests.values())
    if binary:
        R.run_binary(folder, dtype, steps, max_tokens, tmp_path)
    else:
        R.run_in_process(folder, dtype, steps, max_tokens, tiny.PAGE[name], tmp_path)
    rows = R.collect(steps, tmp_path, config["vocab"])
    assert len(rows) == sum(len(t) for t in requests.values())
    for rid, tokens in requests.items():
        got = torch.from_numpy(np.stack([rows[(rid, p)] for p in range(len(tokens))]))
        assert close_rows(got, logits_of(config, W, tokens), dtype), rid


def plain_greedy(config, W, tokens, new_tokens):
    tokens, out = list(tokens), []
    for _ in range(new_tokens):
        out.append(int(plain.forward(config, W, tokens)[-1].argmax()))
        tokens.append(out[-1])
    return out


@pytest.mark.parametrize("cuda_graphs,async_scheduling", [(False, False), (True, False), (True, True)])
def test_greedy_generation_through_the_engine(models, cuda_graphs, async_scheduling):
    """The framework's own entry point: scheduler, portions under a token budget, CUDA graphs for
    decode steps, two slots for five requests, so few pages that a request is preempted and
    computed again from its first token."""
    folder, config, W = models["a"]
    prompts = [prompt(config, n, 20 + n) for n in (5, 17, 2, 11, 8)]
    want = [plain_greedy(config, W, p, 10) for p in prompts]
    engine = Engine(folder, dtype="float32", num_blocks=9, block_size=4, max_num_seqs=2, max_num_batched_tokens=16,
                    prefill_chunk_size=8, cuda_graphs=cuda_graphs, async_scheduling=async_scheduling)
    assert engine.runner.spec.architecture == "Nefipel" and not engine.runner.cache.has_state
    assert (engine.graphs is not None) == cuda_graphs
    got = engine.generate(prompts, max_tokens=10, arrival_steps=[0, 0, 1, 4, 20])
    assert got == want
    assert engine.scheduler.preemptions > 0
    if cuda_graphs:
        assert engine.graphs.replays > 0
    engine.runner.cache.check()
    assert engine.runner.cache.available_pages() == 9


def test_generation_reuses_a_shared_prefix(models):
    """No layer keeps state, so pages of a prompt's beginning are shared by later requests that begin alike."""
    folder, config, W = models["c"]
    shared = prompt(config, 48, 90)
    prompts = [shared + prompt(config, n, 91 + n) for n in (5, 9, 3)]
    want = [plain_greedy(config, W, p, 6) for p in prompts]
    engine = Engine(folder, dtype="float32", num_blocks=24, block_size=16, max_num_seqs=2, max_num_batched_tokens=64)
    got = engine.generate(prompts, max_tokens=6, arrival_steps=[0, 6, 12])
    assert got == want


def test_the_command_line_generates_from_a_nefipel_folder(models, capsys):
    from vosti_b200.engine import cli
    folder, config, W = models["b"]
    tokens = prompt(config, 6, 9)
    want = plain_greedy(config, W, tokens, 4)
    code = cli.main(["--model", folder, "--dtype", "float32", "--prompt-ids", ",".join(map(str, tokens)), "--max-tokens", "4"])
    assert code in (0, None)
    assert ",".join(map(str, want)) in capsys.readouterr().out.replace(" ", "")
