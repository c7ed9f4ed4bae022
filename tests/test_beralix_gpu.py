"""The Beralix design on the GPU against the plain implementation (tests/plain_beralix.py).

Mechanisms alone (the layer norm over the stream with a normed, scaled sublayer output on its
way in; the windowed attention with a partial, rescaled rotation and value mixing; the latent
attention; the selective scan with its convolution tail), then whole models of three small
configurations: whole prompts, prefill against token-by-token decoding, portions down to two
tokens, unequal requests in one batch against each alone, pages and state slots used again,
long decoding past every window, and greedy generation through `Engine` (scheduler, CUDA
graphs, asynchronous scheduling, preemption).

Where random inputs would hide a fault, the inputs are made so that it shows: one query and one
key are scaled so that a single score stands out, at the last key a window keeps and the first
one it drops, at page borders, at the borders of the key segments the latent attention cuts long
contexts into, and hundreds of tokens back.

Exactness is tested in float32 (differences of rounding order only); bfloat16 serving is
compared with the float32 oracle with a bound on the error of rounding.
"""
import math

import pytest
import torch

import plain_beralix as plain
import tiny_beralix as tiny
from gpu_util import Harness
from vosti_b200 import Engine, ops
from vosti_b200.config import PartSpec
from vosti_b200.engine.batch import StepEntry
from vosti_b200.engine.runner import ModelRunner
from vosti_b200.parts import build_mixer, build_norm

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
    """Random weights for a mixer by role, of a size that makes every term matter."""
    W = {}
    for key, w in part.weight_specs().items():
        last = key.split(".")[-1]
        if key == "conv":
            W[key] = rounded(*w.shape, gen=gen, std=0.6)
        elif key == "A_log":
            W[key] = rounded(*w.shape, gen=gen, std=0.7, mean=-0.5)
        elif key == "dt.b":
            W[key] = rounded(*w.shape, gen=gen, std=1.0, mean=-1.0)
        elif key == "vmix":
            W[key] = rounded(gen=gen, std=0.1, mean=0.4)
        elif key in ("g", "dt"):
            W[key] = rounded(*w.shape, gen=gen, std=2.0 / math.sqrt(w.shape[-1]))
        elif len(w.shape) == 2:
            W[key] = rounded(*w.shape, gen=gen, std=1.0 / math.sqrt(w.shape[-1]))
        elif last == "b":
            W[key] = rounded(*w.shape, gen=gen, std=0.3)
        else:                                             # norm weights, D
            W[key] = rounded(*w.shape, gen=gen, std=0.2, mean=1.0)
    return W


def run_mixer(mixer, harness, x, sizes, dtype, rid="r", extras=None):
    """The mixer over one request, cut into portions of `sizes`; `extras(at, size)` gives what other
    layers of the step would have published."""
    outs, at = [], 0
    for size in sizes:
        ctx = harness.context([StepEntry(rid, [0] * size)])
        if extras is not None:
            ctx.extras.update(extras(at, size))
        outs.append(ops.materialize(mixer.forward(ctx, x[at:at + size].to(DEV, dtype), harness.cache.layer_caches[0])).float().cpu())
        at += size
    assert int(harness.status.item()) == 0
    return torch.cat(outs)


def close(got, want, dtype, sizes=None):
    if dtype == torch.float32:
        assert torch.allclose(got, want, **F32), (sizes, float((got - want).abs().max()))
    else:
        assert float((got - want).abs().mean() / want.abs().mean()) < 0.04, sizes


CUTS = lambda T: ((T,), (T - 33,) + (1,) * 33, (2, 5, 1, 1, 17, 2, 3, T - 31))


# ---------------------------------------------------------------- layer norm over the stream
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [200, 67, 1, 4, 1024, 1028, 2600, 6148, 8196])      # rows in registers up to 8192, else shared memory
def test_layer_norm_of_the_stream_with_a_normed_scaled_term(dtype, width):
    gen = torch.Generator().manual_seed(width)
    rows, eps = 9, 3e-6
    norm = build_norm(PartSpec.make("layer_norm_stream", eps=eps, bias=True, bias_name="b"), width)
    after = build_norm(PartSpec.make("layer_norm_stream", eps=eps, bias=True, bias_name="b"), width)
    assert set(norm.weight_specs()) == {"weight", "b"}
    Wn = {"weight": rounded(width, gen=gen, std=0.2, mean=1.0), "b": rounded(width, gen=gen, std=0.3)}
    Wa = {"weight": rounded(width, gen=gen, std=0.2, mean=1.0), "b": rounded(width, gen=gen, std=0.3)}
    give(norm, Wn, dtype)
    give(after, Wa, dtype)
    scale = rounded(width, gen=gen, std=0.3, mean=0.8)
    store = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    stream = 3.0 + 2.0 * torch.randn(rows, width, generator=gen)        # a mean far from zero: the variance is of deviations
    y = rounded(rows, width, gen=gen, std=4.0, mean=1.0)

    class C:
        pass
    ctx = C()
    ctx.dtype, ctx.extras = dtype, {}
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    # the norm alone
    want = plain.layer_norm(stream.double(), Wn["weight"].double(), Wn["b"].double(), eps)
    got = norm.forward(ctx, stream.to(DEV)).float().cpu()
    assert torch.allclose(got, want.float(), **tol)
    # a sublayer's output, normed and scaled, joins the stream; the sum is normed for the next sublayer
    term = plain.layer_norm(y.double(), Wa["weight"].double(), Wa["b"].double(), eps) * scale.double()
    total = stream.double() + term
    want = plain.layer_norm(total, Wn["weight"].double(), Wn["b"].double(), eps)
    residual = stream.to(DEV).clone()
    got, new = norm.forward_add(ctx, after.defer(y.to(DEV, dtype), scale.to(DEV, store)), residual)
    assert new.dtype == torch.float32 and torch.allclose(new.cpu(), total.float(), atol=2e-5, rtol=2e-5)
    assert torch.allclose(got.float().cpu(), want.float(), **tol)
    # the first norm of a model: no stream yet
    got, new = norm.forward_add(ctx, y.to(DEV), None)
    assert torch.equal(new.cpu(), y)
    assert torch.allclose(got.float().cpu(), plain.layer_norm(y.double(), Wn["weight"].double(), Wn["b"].double(), eps).float(), **tol)


# ---------------------------------------------------------------- windowed attention, rotation, value mixing
def window_block(heads, kv, dk, dv, window, rot_dims, base, scaling, scale, v_mix=False):
    block = dict(heads=heads, kv_heads=kv, dim=dk, vdim=dv, scale=scale, rot=dict(base=base, dims=rot_dims, scaling=scaling))
    if window:
        block["mask"] = dict(size=window)
    if v_mix:
        block["v_mix"] = True
    return block


def window_spec(block, value_mix=None):
    s = block["rot"].get("scaling")
    scaling = None if s is None else ("yarn", float(s["factor"]), float(s["original"]), float(s["fast"]), float(s["slow"]))
    return PartSpec.make("sink_attention", num_heads=block["heads"], num_kv_heads=block["kv_heads"], head_dim=block["dim"],
                         v_head_dim=block["vdim"], scale=block["scale"], window=block.get("mask", {}).get("size", 0), chunk=0,
                         sink=False, value_mix=value_mix,
                         position=PartSpec.make("rope", theta=block["rot"]["base"], rotary_dim=block["rot"]["dims"],
                                                scaling=scaling, max_positions=0))


YARN = dict(factor=3.0, original=48, fast=4.0, slow=1.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dk,dv,window,rot,scaling,page", [
    (4, 2, 24, 16, 7, 8, YARN, 8), (2, 1, 16, 40, 20, 2, None, 8), (3, 3, 8, 8, 1, 4, YARN, 4), (2, 1, 6, 10, 5, 6, None, 4),
    (4, 2, 64, 64, 48, 32, dict(factor=8.0, original=64, fast=8.0, slow=1.0), 16), (2, 2, 128, 128, 100, 64, None, 16),
    (6, 1, 64, 64, 33, 64, YARN, 16), (2, 1, 32, 32, 0, 32, YARN, 8)])
def test_windowed_attention_mixer_against_plain(dtype, heads, kv, dk, dv, window, rot, scaling, page):
    """With projections, as a layer that gives its values and as one that mixes another layer's in."""
    gen = torch.Generator().manual_seed(heads * 100 + dk + window)
    width, T = 72, 150
    block = window_block(heads, kv, dk, dv, window, rot, 300.0, scaling, 0.9 / math.sqrt(dk) * 3.0, v_mix=True)
    x = rounded(T, width, gen=gen)
    v_first = rounded(T, kv, dv, gen=gen)
    for role in ("source", "mix", None):
        mixer = build_mixer(window_spec(block, role), width, None)
        assert ("vmix" in mixer.weight_specs()) == (role is not None)
        W = weights_of(mixer, gen)
        give(mixer, W, dtype)
        want, v_used = plain.window_attention(x.double(), {k: v.double() for k, v in W.items()}, block,
                                              v_first.double() if role == "mix" else None, role == "mix")
        extras = None
        if role == "mix":
            extras = lambda at, size: {"value_mix.source": v_first[at:at + size].reshape(size, kv * dv).to(DEV, dtype).contiguous()}
        for sizes in CUTS(T):
            harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=-(-T // page) + 1, page_size=page)
            got = run_mixer(mixer, harness, x, sizes, dtype, extras=extras)
            close(got, want.float(), dtype, (role, sizes))
        if role == "source":                 # what it publishes for later layers is its own values of the step's tokens
            harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=-(-T // page) + 1, page_size=page)
            ctx = harness.context([StepEntry("r", [0] * T)])
            mixer.forward(ctx, x.to(DEV, dtype), harness.cache.layer_caches[0])
            published = ctx.extras["value_mix.source"].float().cpu().view(T, kv, dv)
            assert torch.allclose(published, v_used.float(), atol=2e-5 if dtype == torch.float32 else 3e-2)


def plain_windowed(qkv, block):
    T = qkv.shape[0]
    H, G, D, Dv = block["heads"], block["kv_heads"], block["dim"], block["vdim"]
    q, k, v = qkv.double().split([H * D, G * D, G * Dv], dim=-1)
    pos = torch.arange(T)
    q, k = plain.rotate(q.view(T, H, D), pos, block["rot"]), plain.rotate(k.view(T, G, D), pos, block["rot"])
    rep = H // G
    out = plain.softmax_attention(q, k.repeat_interleave(rep, 1), v.view(T, G, Dv).repeat_interleave(rep, 1), block["scale"],
                                  block.get("mask", {}).get("size", 0))
    return out.reshape(T, H * Dv).float()


def run_windowed(mixer, harness, qkv, sizes, dtype, rid="r", trim=False):
    """The kernels behind the mixer's projections, fed with a hand-made q | k | v row per token.
    `trim`: after every step the pages the window has left go back to the pool, as the runner does."""
    cache = harness.cache.layer_caches[0]
    outs, at = [], 0
    for size in sizes:
        ctx = harness.context([StepEntry(rid, [0] * size)])
        group = ctx.group(cache.group)
        part = qkv[at:at + size].to(DEV, dtype).contiguous()
        q = ops.qkv_store(part, cache.k, cache.v, nq=mixer.nq, nkv=mixer.nkv, dk=mixer.dk, dv=mixer.dv,
                          page_size=group.page_size, positions=ctx.positions, slot_mapping=group.slot_mapping,
                          temp_coef=0.0, temp_every=1, status=ctx.status, freq=mixer.freq, magnitude=mixer.magnitude)
        outs.append(ops.attention_sink(ctx, q, cache.k, cache.v, group, nq=mixer.nq, nkv=mixer.nkv, dk=mixer.dk, dv=mixer.dv,
                                       scale=mixer.scale, window=mixer.window, bias=None, sink=None, chunk=0).float().cpu())
        at += size
        if trim:
            harness.cache.trim(rid)
    assert int(harness.status.item()) == 0
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk,window,page", [(24, 40, 8), (64, 48, 16), (64, 120, 16), (64, 16, 16), (32, 33, 4)])
def test_one_key_stands_out_at_the_edges_of_a_window(dtype, dk, window, page):
    """The query of the last position and one key share a large component in a part of the head
    that does not turn. The last `window` positions (the query's own among them) are seen: the
    oldest of them, keys next to page borders and the key before the query give the output their
    value; the key one step further back, and older ones, must not be seen at all. The same for a
    whole prompt, for a token decoded alone and for a short portion."""
    heads, kv, dv, rot = 2, 1, dk, 8
    gen = torch.Generator().manual_seed(dk + window)
    block = window_block(heads, kv, dk, dv, window, rot, 100.0, YARN, 1.0)
    mixer = build_mixer(window_spec(block), 64, None)
    mixer.setup(torch.device(DEV), dtype)
    T = 2 * window + window // 2 + 3
    oldest = T - window                                   # i - j < window  <=>  j > i - window = T - 1 - window
    base = rounded(T, heads * dk + kv * (dk + dv), gen=gen, std=0.1)
    base[:, heads * dk + kv * dk:] = rounded(T, kv * dv, gen=gen)            # values of order one
    border = (oldest // page + 1) * page
    inside = sorted({oldest, oldest + 1, border, border - 1, T - 2} & set(range(oldest, T - 1)))
    outside = [oldest - 1, oldest - 2, oldest - window, 0]
    for target in inside + outside:
        qkv = base.clone()
        qkv[T - 1, dk - 1] = 8.0                          # head 0's query, last element (not rotated)
        qkv[target, heads * dk + dk - 1] = 8.0            # the key at `target`
        want = plain_windowed(qkv, block)
        value = qkv[target, heads * dk + kv * dk:heads * dk + kv * dk + dv]
        seen = torch.allclose(want[T - 1, :dv], value, atol=1e-3)
        assert seen == (target >= oldest), target                             # the oracle agrees with the design
        for sizes in ((T,), (T - 1, 1), (oldest - 1, 3, T - oldest - 2), (T - 2, 2)):
            harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=-(-T // page) + 1, page_size=page)
            got = run_windowed(mixer, harness, qkv, sizes, dtype)
            tol = 2e-5 if dtype == torch.float32 else 3e-2
            assert torch.allclose(got[T - 1], want[T - 1], atol=tol, rtol=tol), (target, sizes)
            assert torch.allclose(got[T - 1, :dv], value, atol=2e-2) == (target >= oldest), (target, sizes)


def test_a_window_passes_over_decoded_tokens_and_its_pages_come_back():
    """Decoding far past the window with a pool that holds little more than the window: the pages
    the window left are used again, and every decoded row still equals the plain one."""
    gen = torch.Generator().manual_seed(3)
    heads, kv, dk, dv, window, page = 2, 2, 16, 24, 11, 4
    block = window_block(heads, kv, dk, dv, window, 16, 50.0, YARN, 0.7)
    mixer = build_mixer(window_spec(block), 64, None)
    mixer.setup(torch.device(DEV), torch.float32)
    T = 90
    qkv = rounded(T, heads * dk + kv * (dk + dv), gen=gen)
    want = plain_windowed(qkv, block)
    harness = Harness([mixer.cache_spec()], [None], torch.float32, num_pages=window // page + 4, page_size=page)
    got = run_windowed(mixer, harness, qkv, (9, 2) + (1,) * (T - 11), torch.float32, trim=True)
    assert torch.allclose(got, want, atol=2e-5, rtol=2e-5)
    harness.cache.check()
    harness.cache.finish("r")
    assert harness.cache.available_pages() == window // page + 4


# ---------------------------------------------------------------- the per-head product
@pytest.mark.parametrize("tokens", [1, 7, 16, 17, 150])
@pytest.mark.parametrize("x_type,y_type", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16),
                                           (torch.float32, torch.float32), (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("inner,outer,contiguous", [(24, 40, "out"), (40, 24, "in"), (136, 200, "in"), (72, 264, "out"),
                                                    (12, 20, "out"), (10, 6, "in")])
def test_head_project_against_einsum(tokens, x_type, y_type, inner, outer, contiguous):
    """y[t, h] = g[t, h] (x[t, h] M_h) for a bfloat16 M_h stored with either axis contiguous, x and y
    strided views of wider rows; sizes in multiples of 8 take the tensor cores, the others the CUDA
    cores. A float32 x keeps 16 bits of its mantissa."""
    gen = torch.Generator().manual_seed(tokens * 131 + inner)
    heads, pad = 3, 8
    x_wide = torch.randn(tokens, heads, inner + pad, generator=gen)
    if x_type == torch.bfloat16:
        x_wide = x_wide.to(torch.bfloat16).float()
    else:
        x_wide = (x_wide.to(torch.bfloat16).float() * (1.0 + 2.0 ** -9))          # needs more than 8 bits
    m = rounded(heads, inner, outer, gen=gen, std=1.0 / math.sqrt(inner))
    gate = torch.rand(tokens, heads, generator=gen)
    want = torch.einsum("thi,hio->tho", x_wide[..., :inner].double(), m.double()) * gate.double()[..., None]
    xd = x_wide.to(DEV, x_type)[..., :inner]
    if contiguous == "out":
        md = m.to(DEV, torch.bfloat16).contiguous()
    else:
        md = m.transpose(1, 2).to(DEV, torch.bfloat16).contiguous().transpose(1, 2)
    y_wide = torch.zeros(tokens, heads, outer + pad, dtype=y_type, device=DEV)
    ops.head_project(xd, md, y_wide[..., :outer], gate=gate.to(DEV))
    torch.cuda.synchronize()
    got = y_wide[..., :outer].double().cpu()
    bound = 2e-5 if y_type == torch.float32 else 6e-3
    assert (got - want).abs().max() <= bound * max(1.0, want.abs().max().item())
    assert y_wide[..., outer:].abs().max().item() == 0.0
    without = torch.zeros(tokens, heads, outer, dtype=y_type, device=DEV)
    ops.head_project(xd, md, without)
    ungated = torch.einsum("thi,hio->tho", x_wide[..., :inner].double(), m.double())
    assert (without.double().cpu() - ungated).abs().max() <= bound * max(1.0, ungated.abs().max().item())


# ---------------------------------------------------------------- latent attention
def latent_block(heads, dim, rot, dv, rank, scale, base, scaling):
    return dict(heads=heads, dim=dim, rot_dim=rot, vdim=dv, kv_rank=rank, scale=scale, rot=dict(base=base, dims=rot, scaling=scaling))


def latent_spec(block, eps, gate=True):
    s = block["rot"].get("scaling")
    scaling = None if s is None else ("yarn", float(s["factor"]), float(s["original"]), float(s["fast"]), float(s["slow"]))
    return PartSpec.make("latent_attention", num_heads=block["heads"], head_dim=block["dim"], rot_dim=block["rot_dim"],
                         v_head_dim=block["vdim"], kv_rank=block["kv_rank"], scale=block["scale"], eps=eps, gate=gate,
                         position=PartSpec.make("rope", theta=block["rot"]["base"], rotary_dim=block["rot_dim"], scaling=scaling,
                                                max_positions=0))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,rot,dv,rank,scaling,page", [
    (3, 20, 6, 10, 40, YARN, 8), (1, 8, 2, 8, 8, None, 4), (5, 12, 10, 24, 24, None, 8), (4, 32, 16, 48, 64, YARN, 16),
    (2, 7, 4, 5, 33, YARN, 4), (2, 64, 32, 64, 160, None, 16), (1, 16, 8, 16, 300, YARN, 8),
    # sizes the tensor-core kernel takes in bfloat16: a tile of 16 rows is one token, four tokens, or cuts across tokens
    (16, 128, 64, 128, 512, YARN, 16), (4, 32, 32, 48, 128, None, 16), (3, 64, 32, 64, 256, YARN, 8), (40, 16, 64, 16, 128, None, 4)])
def test_latent_attention_mixer_against_plain(dtype, heads, dim, rot, dv, rank, scaling, page):
    gen = torch.Generator().manual_seed(heads * 100 + rank)
    width, T, eps = 72, 150, 2e-6
    block = latent_block(heads, dim, rot, dv, rank, 2.5 / math.sqrt(dim + rot), 200.0, scaling)
    mixer = build_mixer(latent_spec(block, eps), width, None)
    assert set(mixer.weight_specs()) == {"q", "dkv", "dkv.norm", "uk", "uv", "g", "o"}
    spec = mixer.cache_spec()
    assert spec.widths == (rank, rot) and spec.heads == 1          # only the latent and the shared rotated part are kept
    W = weights_of(mixer, gen)
    give(mixer, W, dtype)
    x = rounded(T, width, gen=gen)
    want = plain.latent_attention(x.double(), {k: v.double() for k, v in W.items()}, block, eps).float()
    for sizes in CUTS(T):
        harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=-(-T // page) + 1, page_size=page)
        got = run_mixer(mixer, harness, x, sizes, dtype)
        close(got, want, dtype, sizes)


def test_latent_attention_without_a_gate():
    gen = torch.Generator().manual_seed(8)
    width, T, eps = 40, 30, 1e-5
    block = latent_block(2, 12, 4, 6, 16, 0.4, 100.0, None)
    mixer = build_mixer(latent_spec(block, eps, gate=False), width, None)
    assert "g" not in mixer.weight_specs()
    W = weights_of(mixer, gen)
    give(mixer, W, torch.float32)
    x = rounded(T, width, gen=gen)
    ones = dict({k: v.double() for k, v in W.items()}, g=torch.zeros(2, width, dtype=torch.float64))   # sigmoid(0) = 1/2
    want = 2.0 * plain.latent_attention(x.double(), ones, block, eps).float()
    harness = Harness([mixer.cache_spec()], [None], torch.float32, num_pages=8, page_size=4)
    close(run_mixer(mixer, harness, x, (T,), torch.float32), want, torch.float32)


def test_latent_attention_of_unequal_requests_in_one_step_on_the_tensor_cores():
    """A long request decoding one token, a portion in the middle of another and a whole short
    prompt in one step: every row equals its request alone in the plain form."""
    gen = torch.Generator().manual_seed(12)
    width, eps, page, dtype = 96, 1e-5, 16, torch.bfloat16
    block = latent_block(16, 32, 32, 16, 128, 0.3, 10000.0, YARN)
    mixer = build_mixer(latent_spec(block, eps), width, None)
    W = weights_of(mixer, gen)
    give(mixer, W, dtype)
    xs = {r: rounded(n, width, gen=gen) for r, n in (("a", 420), ("b", 77), ("c", 3))}
    want = {r: plain.latent_attention(x.double(), {k: v.double() for k, v in W.items()}, block, eps).float() for r, x in xs.items()}
    harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=40, page_size=page)
    cache = harness.cache.layer_caches[0]
    run = lambda ctx, rows: ops.materialize(mixer.forward(ctx, torch.cat(rows).to(DEV, dtype), cache)).float().cpu()
    got = {r: [] for r in xs}
    got["a"].append(run(harness.context([StepEntry("a", [0] * 419)]), [xs["a"][:419]]))
    got["b"].append(run(harness.context([StepEntry("b", [0] * 20)]), [xs["b"][:20]]))
    rows = run(harness.context([StepEntry("a", [0]), StepEntry("b", [0] * 37), StepEntry("c", [0] * 3)]),
               [xs["a"][419:], xs["b"][20:57], xs["c"]])
    got["a"].append(rows[:1]); got["b"].append(rows[1:38]); got["c"].append(rows[38:])
    rows = run(harness.context([StepEntry("b", [0] * 20)]), [xs["b"][57:]])
    got["b"].append(rows)
    assert int(harness.status.item()) == 0
    for r in xs:
        close(torch.cat(got[r]), want[r], dtype, r)
        worst = (torch.cat(got[r]) - want[r]).abs().max() / want[r].abs().max()
        assert float(worst) < 0.05, (r, float(worst))


@pytest.mark.parametrize("dtype,rank,rot", [(torch.float32, 16, 4), (torch.bfloat16, 16, 4), (torch.bfloat16, 128, 32)])
def test_one_latent_far_back_decides_the_row(dtype, rank, rot):
    """Causal attention over everything: a key hundreds of tokens back, at the first position, next
    to a page border and next to the borders of the pieces the kernel cuts long contexts into
    must weigh as the plain form says. The projections are rows of the identity, so that the
    mixer's input is the q | down | gate row itself; the first latent element of every token is
    zero but the target's, head 0's unrotated key matrix reads that element alone, and the last
    query looks for it."""
    heads, dim, dv, page, eps = 2, 8, 8, 16, 1e-6
    gen = torch.Generator().manual_seed(17)
    qw = heads * (dim + rot)
    width = qw + rank + rot + heads
    block = latent_block(heads, dim, rot, dv, rank, 1.0, 1000.0, YARN)
    mixer = build_mixer(latent_spec(block, eps), width, None)
    eye = torch.eye(width)
    W = {"q": eye[:qw], "dkv": eye[qw:qw + rank + rot], "g": eye[qw + rank + rot:], "dkv.norm": torch.ones(rank),
         "uk": rounded(heads * dim, rank, gen=gen, std=0.1), "uv": rounded(heads * dv, rank, gen=gen, std=0.5),
         "o": rounded(width, heads * dv, gen=gen, std=0.3)}
    W["uk"][:dim] = 0.0
    W["uk"][0, 0] = 1.0                                   # head 0: k[0] = c[0], every other unrotated key element is 0
    give(mixer, W, dtype)
    T = 700
    base = rounded(T, width, gen=gen, std=0.2)
    base[:, qw] = 0.0                                     # the first latent element
    base[:, qw + rank + rot:] = rounded(T, heads, gen=gen)
    Wd = {k: v.double() for k, v in W.items()}
    ctx_cut, small_cut = ops.LATENT_SEGMENT, ops.LATENT_MMA_SEGMENT       # the pieces of either kernel
    assert T > 2 * ctx_cut
    for target in (0, 1, page - 1, page, 63, 64, small_cut - 1, small_cut, small_cut + 1, ctx_cut - 1, ctx_cut, ctx_cut + 1,
                   2 * ctx_cut - 1, 2 * ctx_cut, T - 2, T - 1):
        x = base.clone()
        x[target, qw] = 2.0 * math.sqrt(rank / 16)        # after the unit-RMS norm about 3.7
        x[T - 1, 0] = 16.0                                # head 0's query, first unrotated element
        want = plain.latent_attention(x.double(), Wd, block, eps).float()
        hidden = x.clone()
        hidden[target, qw] = 0.0
        without = plain.latent_attention(hidden.double(), Wd, block, eps).float()
        assert (want[T - 1] - without[T - 1]).abs().max() > 0.05, target       # the target decides the oracle's last row
        for sizes in ((T,), (T - 1, 1), (T - 2, 2), (ctx_cut - 1, 2, T - ctx_cut - 1)):
            harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=-(-T // page) + 1, page_size=page)
            outs, at = [], 0
            for size in sizes:                            # only the last portion's rows are compared
                ctx = harness.context([StepEntry("r", [0] * size)])
                out = ops.materialize(mixer.forward(ctx, x[at:at + size].to(DEV, dtype), harness.cache.layer_caches[0]))
                at += size
            got = out[-1].float().cpu()
            assert int(harness.status.item()) == 0
            tol = 1e-4 if dtype == torch.float32 else 4e-2
            assert torch.allclose(got, want[T - 1], atol=tol, rtol=tol), (target, sizes, float((got - want[T - 1]).abs().max()))


# ---------------------------------------------------------------- selective scan
def scan_spec(inner, states, taps, dt_rank):
    return PartSpec.make("selective_scan", inner=inner, state=states, conv_taps=taps, dt_rank=dt_rank)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,states,taps,dt_rank", [(50, 5, 4, 3), (40, 1, 1, 1), (96, 40, 3, 8), (64, 16, 2, 16), (33, 24, 5, 2),
                                                     (70, 8, 3, 4), (32, 128, 4, 6), (130, 3, 2, 1)])
def test_selective_scan_mixer_against_plain(dtype, inner, states, taps, dt_rank):
    gen = torch.Generator().manual_seed(inner + states)
    width, T = 72, 150
    mixer = build_mixer(scan_spec(inner, states, taps, dt_rank), width, None)
    assert set(mixer.weight_specs()) == {"in", "conv", "conv.b", "x", "dt", "dt.b", "A_log", "D", "o"}
    size = mixer.state_spec().shape[0]
    assert inner * states + (taps - 1) * inner <= size < inner * states + (taps - 1) * inner + 4
    W = weights_of(mixer, gen)
    give(mixer, W, dtype)
    x = rounded(T, width, gen=gen)
    m = dict(inner=inner, state=states, conv=taps, dt_rank=dt_rank)
    want = plain.selective_scan(x.double(), {k: v.double() for k, v in W.items()}, m).float()
    for sizes in CUTS(T) + ((1, 1, 1, 2, 1, 3, T - 9),):           # portions shorter than the convolution's reach from the start
        harness = Harness([None], [mixer.state_spec()], dtype, max_requests=2)
        got = run_mixer(mixer, harness, x, sizes, dtype)
        close(got, want, dtype, sizes)


def test_slow_decay_keeps_what_the_first_token_wrote():
    """Decays next to one and a read-out that looks at one state: after hundreds of tokens the
    output still carries the first token's input, whole, cut, and decoded token by token."""
    gen = torch.Generator().manual_seed(4)
    width, inner, states, taps, dt_rank, T = 24, 16, 6, 3, 2, 400
    mixer = build_mixer(scan_spec(inner, states, taps, dt_rank), width, None)
    W = weights_of(mixer, gen)
    W["A_log"] = torch.full((inner, states), -9.0)                  # A = -exp(-9): exp(dt A) is within 2e-4 of one
    give(mixer, W, torch.float32)
    x = rounded(T, width, gen=gen)
    m = dict(inner=inner, state=states, conv=taps, dt_rank=dt_rank)
    Wd = {k: v.double() for k, v in W.items()}
    want = plain.selective_scan(x.double(), Wd, m).float()
    other = x.clone()
    other[0] = -x[0]
    assert (plain.selective_scan(other.double(), Wd, m).float()[T - 1] - want[T - 1]).abs().max() > 1e-2
    for sizes in ((T,), (T - 1, 1), (3,) + (1,) * (T - 3), (199, 2, 199)):
        harness = Harness([None], [mixer.state_spec()], torch.float32, max_requests=1)
        got = run_mixer(mixer, harness, x, sizes, torch.float32)
        assert torch.allclose(got, want, **F32), sizes


def test_scan_state_of_a_slot_that_is_used_again_and_unequal_requests_in_one_step():
    gen = torch.Generator().manual_seed(6)
    width = 48
    mixer = build_mixer(scan_spec(40, 7, 4, 3), width, None)
    W = weights_of(mixer, gen)
    give(mixer, W, torch.float32)
    m = dict(inner=40, state=7, conv=4, dt_rank=3)
    xs = {r: rounded(n, width, gen=gen) for r, n in (("a", 12), ("b", 30), ("c", 5))}
    want = {r: plain.selective_scan(x.double(), {k: v.double() for k, v in W.items()}, m).float() for r, x in xs.items()}
    harness = Harness([None], [mixer.state_spec()], torch.float32, max_requests=2)
    cache = harness.cache.layer_caches[0]
    run = lambda ctx, rows: ops.materialize(mixer.forward(ctx, torch.cat(rows).to(DEV), cache)).cpu()
    ctx = harness.context([StepEntry("a", [0] * 4), StepEntry("b", [0] * 13)])
    got = run(ctx, [xs["a"][:4], xs["b"][:13]])
    assert torch.allclose(got, torch.cat([want["a"][:4], want["b"][:13]]), **F32)
    ctx = harness.context([StepEntry("b", [0] * 1), StepEntry("a", [0] * 8)])          # a single token beside a portion
    got = run(ctx, [xs["b"][13:14], xs["a"][4:]])
    assert torch.allclose(got, torch.cat([want["b"][13:14], want["a"][4:]]), **F32)
    harness.cache.finish("a")           # c takes the slot a leaves, which the manager clears
    assert cache.state.abs().sum(-1).min() > 0
    ctx = harness.context([StepEntry("c", [0] * 5), StepEntry("b", [0] * 16)])
    got = run(ctx, [xs["c"], xs["b"][14:]])
    assert torch.allclose(got, torch.cat([want["c"], want["b"][14:]]), **F32)
    assert int(harness.status.item()) == 0


@pytest.mark.parametrize("states", [7, 48])
def test_scan_portions_of_several_chunks_beside_short_ones_in_one_step(states):
    """Portions longer than a block's chunk run as chunks side by side; their lengths here fall on,
    just under and just over multiples of the chunk, beside a single token and a short portion."""
    gen = torch.Generator().manual_seed(8 + states)
    width, inner = 40, 70
    mixer = build_mixer(scan_spec(inner, states, 3, 4), width, None)
    W = weights_of(mixer, gen)
    give(mixer, W, torch.float32)
    m = dict(inner=inner, state=states, conv=3, dt_rank=4)
    chunk = ops.library().vosti_scan_chunk(states)
    lengths = {"a": 3 * chunk + 1, "b": 2 * chunk + 5, "c": 4 * chunk, "d": chunk + 9}
    xs = {r: rounded(n, width, gen=gen) for r, n in lengths.items()}
    want = {r: plain.selective_scan(x.double(), {k: v.double() for k, v in W.items()}, m).float() for r, x in xs.items()}
    harness = Harness([None], [mixer.state_spec()], torch.float32, max_requests=4)
    cache = harness.cache.layer_caches[0]
    done = {r: 0 for r in xs}
    def step(*parts):
        ctx = harness.context([StepEntry(r, [0] * n) for r, n in parts])
        rows = [xs[r][done[r]:done[r] + n] for r, n in parts]
        got = ops.materialize(mixer.forward(ctx, torch.cat(rows).to(DEV), cache)).cpu()
        exp = torch.cat([want[r][done[r]:done[r] + n] for r, n in parts])
        assert torch.allclose(got, exp, **F32), (parts, float((got - exp).abs().max()))
        for r, n in parts:
            done[r] += n
    step(("a", 2 * chunk), ("b", chunk + 4), ("d", 3))
    step(("b", 1), ("a", chunk + 1), ("c", 4 * chunk), ("d", chunk - 1))         # a, c: whole chunks and one more token
    step(("d", 7), ("b", chunk))
    assert all(done[r] == lengths[r] for r in xs)
    assert int(harness.status.item()) == 0


# ---------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (config, seed) in tiny.ALL.items():
        folder = tiny.write_model(tmp_path_factory.mktemp(f"beralix_{name}"), config, seed)
        _, tensors = tiny.tensors_for(config, seed)
        out[name] = (folder, config, tensors)
    return out


def prompt(config, n, seed):
    return torch.randint(0, config["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def logits_of(config, W, tokens):
    return plain.forward(config, W, tokens).float()


def close_rows(got, want, dtype):
    """float32: every row equal up to rounding order. bfloat16: every row within the rounding of a
    few 8-bit roundings a layer."""
    err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
    if dtype == "float32":
        return bool(err.max() < 2e-4)
    return bool(err.median() < 0.03 and err.max() < 0.1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_whole_prompt_portions_and_decoding_against_plain(models, name, dtype):
    folder, config, W = models[name]
    tokens = prompt(config, 77, 1)                              # past every window of every layer
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


def test_first_tokens_of_a_sequence(models):
    """Requests of one, two and three tokens, and the first rows of a longer one: zeros before the
    start of the convolution, an empty state, a window that is not full yet, a softmax over one key."""
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
                out, stream = inner(ctx, hidden, residual, cache, writes_cache)
                total = torch.empty_like(stream)                   # the stream with the last sublayer's term added
                ops.layer_norm_stream(out, None, None, 0.0, None, stream=stream, stream_out=total)
                streams.append(total.cpu())
                return out, stream
            block.forward = watched
        runner.begin("r")
        runner.step([StepEntry("r", tokens, [0])])
        assert len(streams) == len(want) == len(config["layers"])
        for i, (got, expected) in enumerate(zip(streams, want)):
            assert torch.allclose(got, expected.float(), atol=3e-4, rtol=3e-4), (name, i)


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("c", "float32"), ("c", "bfloat16"), ("a", "bfloat16"),
                                        ("d", "float32"), ("d", "bfloat16")])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(models, name, dtype):
    """Four requests through two state slots and a pool that holds two of them: portions of some
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
    if dtype != "float32":                  # in the serving type the batch equals each request alone up to rounding order
        for r in lengths:
            alone = ModelRunner(folder, dtype=dtype, num_pages=pool, page_size=page, max_requests=1)
            alone.begin(r)
            single = alone.step([StepEntry(r, tokens[r], list(range(lengths[r])))]).cpu()
            err = (torch.cat(got[r]) - single).pow(2).mean(-1).sqrt() / single.pow(2).mean().sqrt()
            assert float(err.max()) < 0.03, (r, float(err.max()))
    assert runner.cache.available_pages() == pool and len(runner.cache.free_slots) == 2


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_long_decoding_past_every_window(models, name):
    """Token by token for several windows' lengths with a pool little larger than the context:
    the scan's state and tail, the windows' pages and the mixed values are carried on."""
    folder, config, W = models[name]
    tokens = prompt(config, 150, 4)
    want = logits_of(config, W, tokens)
    page = tiny.PAGE[name]
    runner = ModelRunner(folder, dtype="float32", num_pages=160 // page, page_size=page, max_requests=1)
    runner.begin("r")
    rows = [runner.step([StepEntry("r", tokens[:3], [0, 1, 2])]).cpu()]
    rows += [runner.step([StepEntry("r", [t], [0])]).cpu() for t in tokens[3:]]
    runner.check_status()
    assert close_rows(torch.cat(rows), want, "float32")


@pytest.mark.parametrize("name,dtype,binary", [("a", "float32", True), ("d", "bfloat16", False), ("c", "float32", False)])
def test_trace_replay_of_a_mixed_schedule(models, name, dtype, binary, tmp_path):
    """The trace runner (the program itself, and the class it wraps) over a schedule of up to four
    live requests, portions beside single tokens, requests that sit a step out, a pool smaller
    than the sum of all requests and four state slots for six requests: every row against the
    plain implementation of the request alone."""
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
    assert engine.runner.spec.architecture == "Beralix" and engine.runner.cache.has_state
    assert (engine.graphs is not None) == cuda_graphs
    got = engine.generate(prompts, max_tokens=10, arrival_steps=[0, 0, 1, 4, 20])
    assert got == want
    assert engine.scheduler.preemptions > 0
    if cuda_graphs:
        assert engine.graphs.replays > 0
    engine.runner.cache.check()
    assert engine.runner.cache.available_pages() == 9 and len(engine.runner.cache.free_slots) == 2


def test_the_command_line_generates_from_a_beralix_folder(models, capsys):
    from vosti_b200.engine import cli
    folder, config, W = models["b"]
    tokens = prompt(config, 6, 9)
    want = plain_greedy(config, W, tokens, 4)
    code = cli.main(["--model", folder, "--dtype", "float32", "--prompt-ids", ",".join(map(str, tokens)), "--max-tokens", "4"])
    assert code in (0, None)
    assert ",".join(map(str, want)) in capsys.readouterr().out.replace(" ", "")
