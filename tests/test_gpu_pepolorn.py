"""Pepolorn on the GPU against the plain implementation: every mechanism alone, then whole models through every way
of cutting requests into steps, in 32-bit and in bfloat16, with pools so small that pages and slots are used again."""
import copy
import json
import math
import os

import pytest
import torch

import harness
import pepolorn_tiny as pt
import tiny
from plain import pepolorn_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# bfloat16: five or six layers whose sublayers' outputs are brought to unit size each (a small output is scaled up
# together with its rounding) leave the median position at a quarter of this bound; a fault of a mechanism moves
# every logit by its own size
TOL = {torch.float32: (2e-4, 0.0), torch.bfloat16: (0.0, 1e-1)}


def _weights(folder):
    return {k: v for k, v in tiny.read_weights(folder).items()}


def _cfg(folder):
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


CLOSE_CALL = 0.01      # a router's choice decided by less than this may go the other way on bfloat16 inputs


class _Reference(dict):
    """Logits by request, and the positions at which some router's choice was a close call."""
    close = None


def _reference(folder, reqs):
    cfg, w = _cfg(folder), _weights(folder)
    ref = _Reference()
    ref.close = set()
    for rid, toks in reqs.items():
        margins = []
        ref[rid] = plain.forward(cfg, w, toks, torch.float64, margins_out=margins)
        for m in margins:
            ref.close.update((rid, int(p)) for p in (m < CLOSE_CALL).nonzero().reshape(-1))
    return ref


def _compare(got, ref, dtype, loosen=1.0):
    """Every position within the bound in 32-bit.  In bfloat16 the rounding of a router's input can turn a close call
    between two experts; that changes the position's logits outright and, through the recurrent states that take the
    position in, those of the positions after it for a while.  Positions whose own call was close are left out, and
    of the rest the median must be well within the bound and no more than a quarter off; a fault of a mechanism puts
    every position off, and the 32-bit runs of the same schedules are held to every position."""
    atol, rel = TOL[dtype]
    off, ratios = [], []
    skip = getattr(ref, "close", None) or set()
    for (rid, pos), row in got.items():
        if dtype == torch.bfloat16 and (rid, pos) in skip:
            continue
        want = ref[rid][pos]
        bound = loosen * (atol * max(1.0, float(want.abs().max())) + rel * float(want.abs().max()))
        diff = float((row.double() - want).abs().max())
        ratios.append(diff / bound)
        if diff > bound:
            off.append(f"request {rid} position {pos}: max diff {diff:.3e} > {bound:.3e}")
    allowed = len(got) // 4 if dtype == torch.bfloat16 else 0
    assert len(ratios) >= len(got) // 2, "too many close calls for the test to say anything"
    assert sorted(ratios)[len(ratios) // 2] <= 0.5, f"the median position is at {sorted(ratios)[len(ratios) // 2]:.2f} of the bound"
    assert len(off) <= allowed, f"{len(off)} of {len(got)} positions off: " + "; ".join(off[:5])


def _runner(folder, dtype, page_size, num_pages, max_slots=4, graphs=False):
    from prelude_b200.engine.loading import load_model, make_runner
    model = load_model(folder, dtype, DEV)
    runner = make_runner(model, page_size=page_size, num_pages=num_pages, max_slots=max_slots,
                         max_request_tokens=num_pages * page_size if graphs else None)
    if graphs:
        runner.enable_step_graphs()
    return runner


def _steps_through_mixer(part, x, cuts, page, dtype, slots=2, use_slot=0):
    """x [T, width] through the mixer ``part``, cut into the steps ``cuts``; returns its outputs one below the other."""
    from prelude_b200.cache.manager import CacheManager
    from prelude_b200.engine.batch import StepItem, build_step_batch
    from prelude_b200.ops import kernels as K
    dev = torch.device(DEV)
    T = x.shape[0]
    cache = CacheManager([part.cache_need()], page, -(-T // page) + 1, slots, dev, dtype)
    for i in range(use_slot):                      # the request does not get slot 0
        cache.add_request(f"other{i}")
    cache.add_request("a")
    got, at = [], 0
    for n in cuts:
        cache.grow("a", at + n)
        batch = build_step_batch([StepItem("a", [0] * n, at, [])], cache.block_tables(["a"]), [cache.slot_of("a")], dev, 10, 1 << 20)
        cache.zero_fresh_state()
        y = part.forward(x[at:at + n].to(DEV).contiguous(), batch, cache.layer_cache(0), True)
        y = y.materialize(dtype) if isinstance(y, K.PartialSums) else y
        got.append(y.float().cpu())
        assert int(batch.status.item()) == 0
        cache.trim("a")
        at += n
    assert at == T
    return torch.cat(got).double()


def _cuts(T, head):
    return [head] + [1] * (T - head)


def _close(got, want, tol, what):
    assert float((got - want).abs().max()) < tol * float(want.abs().max()), (what, float((got - want).abs().max()), float(want.abs().max()))


def _load(part, w, dtype):
    from prelude_b200.parts.registry import RunContext
    part.load(lambda name: w[name], RunContext(torch.device(DEV), dtype))
    return part


# -- mechanisms alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("heads,kv,dim,vdim,rot,scaling,chunk,page", [
    (4, 2, 12, 20, 6, (4.0, 64, 8.0, 2.0), 7, 4), (8, 2, 64, 64, 32, (16.0, 128, 16.0, 1.0), 48, 16), (2, 1, 10, 6, 10, None, 13, 8),
    (4, 4, 32, 64, 16, (2.0, 40, 4.0, 1.0), 64, 16), (2, 2, 16, 16, 16, (1.0, 32, 4.0, 1.0), 8, 8), (4, 4, 8, 8, None, None, 1, 8),
    (6, 3, 24, 40, 8, (8.0, 50, 6.0, 0.5), 21, 16), (4, 1, 128, 128, 64, (32.0, 256, 32.0, 1.0), 32, 16), (3, 1, 16, 32, 2, None, None, 8)])
def test_chunked_attention_normed_after_its_rotation_equals_the_plain_one(dtype, heads, kv, dim, vdim, rot, scaling, chunk, page):
    """The attention of the parallel mixer alone.  One token is made to stand out: queries of its chunk find it, the first
    query of the next chunk must not.  Whole, with a decoded tail that crosses chunk and page borders, in portions whose
    cuts fall inside chunks, and token by token."""
    from prelude_b200.parts.registry import make_part
    from prelude_b200.config.pepolorn import _chunked_attention
    from prelude_b200.config.reader import _Reader
    width, T, head_tokens = 48, 100, 55
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    scale = 6.0 if dtype == torch.float32 else 3.0          # unit q and k: a score is scale times a cosine times the head's size
    m = pt.left(heads, kv, dim, vdim, scale / math.sqrt(dim), chunk, rot, 70.0, scaling)
    w = {"mix.q": torch.randn(heads * dim, width, generator=g) * 0.3, "mix.k": torch.randn(kv * dim, width, generator=g) * 0.3,
         "mix.v": torch.randn(kv * vdim, width, generator=g) * 0.3, "mix.o": torch.randn(width, heads * vdim, generator=g) * 0.2}
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g)
    x[58] *= 3.0
    x = x.to(dtype)
    wd = {k[4:]: v.double() for k, v in w.items()}
    want = plain.chunked_attention(x.double(), wd, m, 1e-5)
    if chunk is not None and chunk < 40:
        free = plain.chunked_attention(x.double(), wd, {k: v for k, v in m.items() if k != "mask"}, 1e-5)
        assert float((free - want).abs().max()) > 0.02 * float(want.abs().max())                # the mask matters here
    if scaling is not None and scaling[0] > 1.0 and rot < dim:
        # norming before the rotation instead of after it would show: the turned part grows by the amplitude
        rates, amp = plain.ramped_rates(rot, 70.0, m["rot"]["scaling"])
        q = plain.unit_rms((x.double() @ wd["q"].T).reshape(T, heads, dim), 1e-5)
        assert amp > 1.05 and float((plain.rotate_halves(q, torch.arange(T), rates, amp) ** 2).mean()) > 1.0 + 0.05 * rot / dim
    problems = []
    spec = _chunked_attention(_Reader(m, "left", problems), width, 1e-5, problems)
    assert not problems
    part = _load(make_part("mixer", spec, "mix"), w, dtype)
    tol = 5e-5 if dtype == torch.float32 else 4e-2
    for cuts in (_cuts(T, head_tokens), [T], [2, 30, 3, 26, 2, 37], [1] * T):
        _close(_steps_through_mixer(part, x, cuts, page, dtype), want, tol, cuts[:3])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("heads,dim,vdim,decays", [
    (3, 10, 6, (0.5, 0.9, 0.99)), (2, 128, 64, (0.9, 0.995)), (2, 9, 11, (0.8, 0.97)), (1, 16, 16, (1.0,)), (4, 8, 24, (0.6, 0.7, 0.8, 0.9)),
    (8, 32, 16, (0.3, 0.5, 0.7, 0.8, 0.9, 0.95, 0.98, 0.999)), (2, 64, 48, (0.0, 0.95)), (1, 200, 17, (0.97,)), (5, 20, 40, (0.2, 0.4, 0.6, 0.8, 1.0))])
def test_decayed_linear_attention_equals_the_plain_one(dtype, heads, dim, vdim, decays):
    """Linear attention with a decaying state alone: a whole sequence at once, token by token and in portions of one to
    three tokens; in a state slot other than the first; decays from forgetting at once to never, so that a state that is
    lost, carried in fewer bits or started from another sequence's shows."""
    from prelude_b200.config.spec import DecayedLinearAttentionSpec
    from prelude_b200.parts.registry import make_part
    width, T = 40, 90
    g = torch.Generator().manual_seed(heads * 10 + dim)
    w = {"mix.q": torch.randn(heads * dim, width, generator=g) * 0.3, "mix.k": torch.randn(heads * dim, width, generator=g) * 0.3,
         "mix.v": torch.randn(heads * vdim, width, generator=g) * 0.3, "mix.g": torch.randn(heads * vdim, width, generator=g) * 0.3,
         "mix.norm": 1.0 + 0.3 * torch.randn(heads * vdim, generator=g), "mix.o": torch.randn(width, heads * vdim, generator=g) * 0.2}
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g).to(dtype)
    m = pt.right(heads, dim, vdim, decays)
    want = plain.decayed_linear_attention(x.double(), {k[4:]: v.double() for k, v in w.items()}, m, 1e-5)
    part = _load(make_part("mixer", DecayedLinearAttentionSpec(width, heads, dim, vdim, tuple(decays), 1e-5), "mix"), w, dtype)
    tol = 5e-5 if dtype == torch.float32 else 4e-2
    for cuts, slot in (([T], 0), (_cuts(T, 40), 1), ([2, 1, 1, 2, 3, 1, 30, 2, 48], 2), ([1] * T, 0)):
        _close(_steps_through_mixer(part, x, cuts, 16, dtype, slots=3, use_slot=slot), want, tol, cuts[:3])


def test_a_decaying_state_carries_what_was_written_hundreds_of_tokens_ago():
    """A slow decay keeps an early token's write readable after 400 more tokens, a fast one beside it does not; the
    kernel's state must show both as the plain loop does, in prompt steps and token by token."""
    from prelude_b200.config.spec import DecayedLinearAttentionSpec
    from prelude_b200.parts.registry import make_part
    width, T, heads, dim = 32, 420, 2, 16
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, width, generator=g) * 0.3
    x[5] *= 12.0
    w = {"mix.q": torch.randn(heads * dim, width, generator=g) * 0.3, "mix.k": torch.randn(heads * dim, width, generator=g) * 0.3,
         "mix.v": torch.randn(heads * dim, width, generator=g) * 0.3, "mix.g": torch.randn(heads * dim, width, generator=g) * 0.3,
         "mix.norm": torch.ones(heads * dim), "mix.o": torch.randn(width, heads * dim, generator=g) * 0.2}
    # queries must not tell the heads apart by size: the slow head is what the far write comes through
    m = pt.right(heads, dim, dim, (0.999, 0.5))
    wd = {k[4:]: v.double() for k, v in w.items()}
    want = plain.decayed_linear_attention(x.double(), wd, m, 1e-5)
    x0 = x.clone()
    x0[5] = x[5] / 12.0
    assert float((plain.decayed_linear_attention(x0.double(), wd, m, 1e-5)[-10:] - want[-10:]).abs().max()) > 0.05 * float(want[-10:].abs().max())
    part = _load(make_part("mixer", DecayedLinearAttentionSpec(width, heads, dim, dim, (0.999, 0.5), 1e-5), "mix"), w, torch.float32)
    for cuts in ([T], [3, 200, 2, 150] + [1] * 65):
        _close(_steps_through_mixer(part, x, cuts, 16, torch.float32), want, 1e-4, cuts[:3])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("heads,groups,state,vdim,taps,parts", [(4, 2, 10, 6, 3, 3), (3, 1, 9, 11, 5, 1), (4, 1, 64, 32, 4, 1), (8, 4, 32, 16, 4, 2),
                                                                 (1, 1, 8, 16, 1, 1), (2, 2, 16, 8, 2, 2), (2, 1, 200, 24, 4, 4)])
def test_state_space_mixer_alone_as_a_layers_mixer(dtype, heads, groups, state, vdim, taps, parts):
    """The state-space mixer on its own (not beside an attention): whole, token by token, in portions shorter than the
    convolution is long, in a slot other than the first."""
    from prelude_b200.config.spec import StateSpaceSpec
    from prelude_b200.parts.registry import make_part
    width, T = 40, 90
    g = torch.Generator().manual_seed(heads * 10 + state)
    inner, ch = heads * vdim, heads * vdim + 2 * groups * state
    w = {"mix.in": torch.randn(inner + ch + heads, width, generator=g) * 0.3, "mix.conv": torch.randn(ch, taps, generator=g) * 0.5,
         "mix.conv.b": torch.randn(ch, generator=g) * 0.3, "mix.dt_bias": torch.randn(heads, generator=g), "mix.A_log": torch.linspace(-3.0, 1.0, heads),
         "mix.D": torch.randn(heads, generator=g), "mix.norm": 1.0 + 0.3 * torch.randn(inner, generator=g),
         "mix.o": torch.randn(width, inner, generator=g) * 0.2}
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g).to(dtype)
    m = pt.mamba2(heads, groups, state, vdim, taps, parts, None)["mixer"]
    want = plain.mamba2(x.double(), {k[4:]: v.double() for k, v in w.items()}, m, 1e-5)
    part = _load(make_part("mixer", StateSpaceSpec(width, heads, vdim, state, groups, taps, parts, 1e-5), "mix"), w, dtype)
    tol = 5e-5 if dtype == torch.float32 else 4e-2
    for cuts, slot in (([T], 0), (_cuts(T, 40), 1), ([2, 1, 1, 2, 3, 1, 30, 2, 48], 2)):
        _close(_steps_through_mixer(part, x, cuts, 16, dtype, slots=3, use_slot=slot), want, tol, cuts[:3])


@pytest.mark.parametrize("experts,top,groups", [(6, 2, (3, 2)), (5, 3, None), (16, 2, (2, 1)), (4, 1, (4, 4)), (2, 1, (2, 1)), (12, 4, (4, 2)),
                                                (64, 6, (8, 3)), (40, 5, (5, 5)), (9, 9, (3, 3))])
def test_router_chooses_by_corrected_scores_and_weighs_by_plain_ones(experts, top, groups):
    """Random logits and corrections large enough to make many choice scores negative; the kernel's experts and weights
    against the plain router's.  Whole groups whose choice scores are all negative must lose as negative sums."""
    from prelude_b200.ops import kernels as K
    g = torch.Generator().manual_seed(experts * 7 + top)
    T = 300
    logits = torch.randn(T, experts, generator=g) * 2.0
    corr = torch.randn(experts, generator=g) * 0.8 - 0.5
    r = pt.moe(experts, top, 8, groups)["router"]
    want_ids, want_w = plain.route(logits.double(), torch.eye(experts, dtype=torch.float64), corr.double(), r)
    assert int(((torch.sigmoid(logits) + corr) < 0).sum()) > T          # negative choice scores are common
    for correction in (corr, None):
        if correction is None:
            want_ids, want_w = plain.route(logits.double(), torch.eye(experts, dtype=torch.float64), torch.zeros(experts, dtype=torch.float64), r)
        ids, w = K.moe_route(logits.to(DEV), top, r.get("groups", {}).get("count", 1), r.get("groups", {}).get("keep", 1), 2, False,
                             None if correction is None else correction.to(DEV))
        ids, w = ids.cpu().long(), w.cpu().double()
        order, want_order = ids.sort(dim=1).indices, want_ids.sort(dim=1).indices
        assert torch.equal(torch.gather(ids, 1, order), torch.gather(want_ids, 1, want_order))
        assert float((torch.gather(w, 1, order) - torch.gather(want_w, 1, want_order)).abs().max()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("T,experts,width,pad", [(1, 6, 44, 0), (9, 32, 2048, 0), (300, 5, 128, 8), (17, 64, 200, 0), (8, 12, 100, 4), (40, 3, 7, 0)])
def test_router_logits_are_32_bit_sums_of_exact_products(dtype, T, experts, width, pad):
    """The router's logits against 64-bit sums, at widths the 16-byte loads take and at widths they do not, from a view
    whose rows are further apart than they are long."""
    from prelude_b200.ops import kernels as K
    g = torch.Generator().manual_seed(T + experts)
    x = torch.randn(T, width + pad, generator=g).to(dtype)
    w = torch.randn(experts, width, generator=g).to(dtype)
    got = K.router_logits(x.to(DEV)[:, :width], w.to(DEV)).cpu().double()
    want = x[:, :width].double() @ w.double().T
    assert got.shape == want.shape and float((got - want).abs().max()) < 2e-6 * max(1.0, float(want.abs().max())) * math.sqrt(width)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("experts,top,ff,groups,T", [(6, 2, 10, (3, 2), 37), (5, 3, 14, None, 1), (8, 4, 64, (4, 2), 300), (2, 1, 16, (2, 1), 9),
                                                      (16, 2, 32, (2, 1), 70)])
def test_routed_feed_forward_equals_the_plain_one(dtype, experts, top, ff, groups, T):
    from prelude_b200.config.pepolorn import _feed_forward
    from prelude_b200.config.reader import _Reader
    from prelude_b200.ops import kernels as K
    from prelude_b200.parts.registry import make_part
    width = 48
    g = torch.Generator().manual_seed(experts + T)
    mlp = pt.moe(experts, top, ff, groups)
    w = {"mlp.router": torch.randn(experts, width, generator=g) * 0.4, "mlp.correction": torch.randn(experts, generator=g) * 0.6 - 0.3}
    for e in range(experts):
        w.update({f"mlp.e{e}.gate": torch.randn(ff, width, generator=g) * 0.3, f"mlp.e{e}.up": torch.randn(ff, width, generator=g) * 0.3,
                  f"mlp.e{e}.down": torch.randn(width, ff, generator=g) * 0.3})
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g).to(dtype)
    wd = {k[4:]: v.double() for k, v in w.items()}
    want = plain.routed_ff(x.double(), wd, mlp)
    no_corr = plain.routed_ff(x.double(), dict(wd, correction=torch.zeros(experts, dtype=torch.float64)), mlp)
    if T > 8 and top < experts:
        assert float((want - no_corr).abs().max()) > 0.05 * float(want.abs().max())            # the correction changes choices
    problems = []
    part = _load(make_part("feed_forward", _feed_forward(_Reader(mlp, "mlp", problems), width, problems), "mlp"), w, dtype)
    y = part.forward(x.to(DEV))
    y = y.materialize(dtype) if isinstance(y, K.PartialSums) else y
    got = y.float().cpu().double()
    tol = 5e-5 if dtype == torch.float32 else 4e-2
    if dtype == torch.float32:
        _close(got, want, tol, "routed")
    else:       # a router's close call may go the other way in bfloat16 inputs of 300 tokens: all but a few rows agree
        bad = ((got - want).abs().max(dim=1).values > tol * float(want.abs().max())).sum()
        assert int(bad) <= T // 50, int(bad)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("ff,T", [(24, 37), (192, 5), (96, 1), (40, 300), (1024, 800)])
def test_feed_forward_gated_by_the_tanh_form_of_gelu_equals_the_plain_one(dtype, ff, T):
    from prelude_b200.config.spec import GatedMlpSpec
    from prelude_b200.ops import kernels as K
    from prelude_b200.parts.registry import make_part
    width = 64
    g = torch.Generator().manual_seed(ff + T)
    w = {"mlp.gate": torch.randn(ff, width, generator=g) * 0.4, "mlp.up": torch.randn(ff, width, generator=g) * 0.3,
         "mlp.down": torch.randn(width, ff, generator=g) * 0.3}
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g).to(dtype)
    wd = {k[4:]: v.double() for k, v in w.items()}
    want = plain.dense_ff(x.double(), wd)
    silu_gated = (plain.silu(x.double() @ wd["gate"].T) * (x.double() @ wd["up"].T)) @ wd["down"].T
    assert float((want - silu_gated).abs().max()) > 0.02 * float(want.abs().max())              # another activation would show
    part = _load(make_part("feed_forward", GatedMlpSpec(width, ff, "gelu_tanh", "gate", "up", "down"), "mlp"), w, dtype)
    y = part.forward(x.to(DEV))
    y = y.materialize(dtype) if isinstance(y, K.PartialSums) else y
    _close(y.float().cpu().double(), want, 5e-5 if dtype == torch.float32 else 3e-2, "dense")


# -- whole models ----------------------------------------------------------------------------------------------------
REQUESTS = {"A": {"a1": 1, "a2": 2, "a19": 19, "a70": 70, "a33": 33}, "B": {"b3": 3, "b150": 150, "b64": 64, "b41": 41, "b97": 97},
            "C": {"c1": 1, "c9": 9, "c40": 40, "c17": 17}}


def _requests(which):
    v = pt.PARAMS[which][0]["vocab"]
    return {rid: tiny.random_ids(n, v, sum(map(ord, rid))) for rid, n in REQUESTS[which].items()}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("pepolorn")
    return {(w, d): pt.make_folder(root, w, d) for w in "ABC" for d in (torch.float32, torch.bfloat16)}


@pytest.fixture(scope="module")
def references(folders):
    return {w: _reference(folders[(w, torch.bfloat16)], _requests(w)) for w in "ABC"}, \
           {w: _reference(folders[(w, torch.float32)], _requests(w)) for w in "ABC"}


def test_the_stream_after_every_layer_equals_the_plain_one(folders):
    """Layer by layer in 32-bit: the first layer that differs names the mechanism.  A layer that runs another layer's
    weights counts each time it runs."""
    from prelude_b200.engine.batch import StepItem, build_step_batch
    from prelude_b200.engine.loading import load_model, make_runner
    from prelude_b200.engine.runner import StepEntry
    from prelude_b200.ops import kernels as K
    from prelude_b200.ops.linear import step_status
    for which in "ABC":
        folder = folders[(which, torch.float32)]
        cfg, w = _cfg(folder), _weights(folder)
        toks = tiny.random_ids(45, cfg["vocab"], 4)
        want = []
        plain.forward(cfg, w, toks, torch.float64, layers_out=want)
        model = load_model(folder, torch.float32, DEV)
        assert len(model.order) == len(cfg["layers"]) == len(want)
        runner = make_runner(model, page_size=pt.PARAMS[which][2], num_pages=16, max_slots=1)
        runner.reserve([StepEntry("x", toks, [])])
        batch = build_step_batch([StepItem("x", toks, 0, [])], runner.cache.block_tables(["x"]), [runner.cache.slot_of("x")], runner.device,
                                 model.spec.vocab_size, model.spec.max_positions)
        runner.cache.zero_fresh_state()
        with step_status(batch.status):
            res = model.embedding.forward(batch)
            delta = None
            for i, call in enumerate(model.order):
                delta = model.blocks[call.block].forward(delta, res, batch, runner.caches[call.cache], call.writes_cache)
                assert isinstance(delta, K.Normed)           # the block leaves its last sublayer's output to be normed and added
                x = delta.x.parts.sum(0) if isinstance(delta.x, K.PartialSums) else delta.x.float()
                normed = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + delta.eps) * delta.weight
                got = (res + normed).cpu().double()
                assert float((got - want[i]).abs().max()) < 1e-4 * max(1.0, float(want[i].abs().max())), f"{which}: layer {i}"
        assert int(batch.status.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["A", "B", "C"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed", "mixed_graphs"])
def test_cuts_match_plain(folders, references, which, dtype, cut):
    """Whole prompts, a decoded tail that crosses chunks and page borders, portions down to two tokens, and mixed
    batches in a pool that holds less than all requests (pages and slots used again), launched and captured."""
    reqs = _requests(which)
    ref = references[0 if dtype == torch.bfloat16 else 1][which]
    page = pt.PARAMS[which][2]
    make = {"whole": harness.whole, "tail_decode": lambda r: harness.tail_decode(r, 40), "portions": harness.portions,
            "mixed": lambda r: harness.mixed(r, max_live=3), "mixed_graphs": lambda r: harness.mixed(r, max_live=3, seed=5)}[cut]
    schedule = make(reqs)
    num_pages = harness.peak_tokens(schedule, page) // page
    if cut.startswith("mixed"):
        assert num_pages < sum(-(-len(t) // page) for t in reqs.values())
    runner = _runner(folders[(which, dtype)], dtype, page, num_pages, max_slots=3 if cut.startswith("mixed") else 1,
                     graphs=cut == "mixed_graphs")
    got = harness.run_schedule(runner, schedule)
    assert len(got) == sum(len(t) for t in reqs.values())
    _compare(got, ref, dtype)
    runner.cache.check()
    assert runner.cache.used_pages() == 0
    if cut == "mixed_graphs":
        assert runner.graph_steps_run > 0


@pytest.mark.parametrize("which", ["A", "B"])
def test_batched_requests_equal_each_alone_in_32_bit(folders, which):
    reqs = _requests(which)
    page = pt.PARAMS[which][2]
    folder = folders[(which, torch.float32)]
    alone = harness.run_schedule(_runner(folder, torch.float32, page, 64), harness.whole(reqs))
    together = harness.run_schedule(_runner(folder, torch.float32, page, 64, max_slots=5),
                                    [([(rid, toks, list(range(len(toks)))) for rid, toks in reqs.items()], list(reqs))])
    for key, row in alone.items():
        assert float((row - together[key]).abs().max()) <= 2e-5 * float(row.abs().max()), key


def test_cuts_agree_in_32_bit(folders):
    """However a request is cut, its logits agree to rounding of the last bits."""
    reqs = {"a70": _requests("A")["a70"]}
    folder = folders[("A", torch.float32)]
    a = harness.run_schedule(_runner(folder, torch.float32, 4, 20), harness.whole(reqs))
    b = harness.run_schedule(_runner(folder, torch.float32, 4, 20), harness.portions(reqs))
    c = harness.run_schedule(_runner(folder, torch.float32, 4, 20), harness.tail_decode(reqs, 50))
    for key, row in a.items():
        bound = 2e-5 * float(row.abs().max())
        assert float((row - b[key]).abs().max()) <= bound and float((row - c[key]).abs().max()) <= bound, key


def test_sharp_attention_finds_keys_at_every_edge_of_a_chunk(tmp_path):
    """A scale turned up makes every softmax pick few keys, wherever they lie: at the start of the query's chunk tens of
    positions back, on either side of a page border, and just outside the chunk (where it must not be found).  32-bit,
    prompt in one step, in portions, and with a decoded tail longer than the chunks."""
    cfg = copy.deepcopy(pt.PEPOLORN_A)
    cfg["layers"][0]["mixer"]["left"].update(scale=2.5, mask={"size": 37})
    cfg["layers"][2]["mixer"]["left"].update(scale=2.5, mask={"size": 37})
    cfg["layers"][4]["mixer"]["left"].update(scale=3.0, mask={"size": 50})
    tensors = pt.tensors_of(cfg, seed=21, std=0.25, norm_jitter=0.3)
    folder = pt.make_folder_from_tensors(tmp_path, "sharp", cfg, tensors)
    reqs = {"s": tiny.random_ids(300, cfg["vocab"], 77)}
    ref = _reference(folder, reqs)
    flat = _reference(pt.make_folder_from_tensors(tmp_path, "flat", pt.PEPOLORN_A, tensors), reqs)
    assert float((ref["s"][200:] - flat["s"][200:]).abs().max()) > 0.1 * float(ref["s"].abs().max())        # the masks and scales matter
    for schedule in (harness.whole(reqs), harness.portions(reqs, (37, 2, 64, 3, 29)), harness.tail_decode(reqs, 70)):
        got = harness.run_schedule(_runner(folder, torch.float32, 16, 19), schedule)
        _compare(got, ref, torch.float32, loosen=5.0)        # scores of tens: their 32-bit rounding shows in the weights


def test_long_decoding_through_freed_and_reused_slots(folders):
    """Two requests decoded token by token for 120 steps side by side after short prompts, then a third takes the
    slot (its states, its convolution inputs) and the pages that the first gave back."""
    cfg = pt.PEPOLORN_A
    reqs = {"a": tiny.random_ids(130, cfg["vocab"], 1), "b": tiny.random_ids(127, cfg["vocab"], 2), "c": tiny.random_ids(60, cfg["vocab"], 3)}
    ref = _reference(folders[("A", torch.float32)], reqs)
    steps = [([("a", reqs["a"][:10], list(range(10))), ("b", reqs["b"][:7], list(range(7)))], [])]
    for i in range(120):
        steps.append(([("a", reqs["a"][10 + i:11 + i], [0]), ("b", reqs["b"][7 + i:8 + i], [0])], ["a", "b"] if i == 119 else []))
    steps.append(([("c", reqs["c"], list(range(60)))], ["c"]))
    runner = _runner(folders[("A", torch.float32)], torch.float32, 4, 66, max_slots=2)
    _compare(harness.run_schedule(runner, steps), ref, torch.float32)
    runner.cache.check()


@pytest.mark.parametrize("which,lens,new", [("A", [1, 5, 17], 20), ("B", [9, 64, 2, 31], 12), ("C", [4, 11], 15)])
def test_greedy_generation_through_the_engine_equals_the_plain_one(folders, which, lens, new):
    from prelude_b200 import Engine
    folder = folders[(which, torch.float32)]
    cfg, w = _cfg(folder), _weights(folder)
    prompts = [tiny.random_ids(n, cfg["vocab"], 50 + n) for n in lens]
    want = []
    for p in prompts:
        seq = list(p)
        for _ in range(new):
            seq.append(int(plain.forward(cfg, w, seq, torch.float64)[-1].argmax()))
        want.append(seq[len(p):])
    eng = Engine(folder, dtype="f32", page_size=pt.PARAMS[which][2], num_pages=64, max_running_requests=4)
    assert eng.caps.cuda_graph and eng.caps.state_slots and eng.caps.kv_cache
    got = eng.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)
    assert [r.token_ids for r in got] == want
    # portions of a few tokens beside decoding requests, launched kernel by kernel: the same tokens
    eng2 = Engine(folder, dtype="f32", page_size=pt.PARAMS[which][2], num_pages=64, max_running_requests=4,
                  max_num_batched_tokens=7, long_prefill_token_threshold=3, cuda_graph=False)
    assert [r.token_ids for r in eng2.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)] == want
    assert eng.cache.used_pages() == 0 and eng2.cache.used_pages() == 0


def test_generation_in_bfloat16_runs_captured_steps(folders):
    from prelude_b200 import Engine
    folder = folders[("B", torch.bfloat16)]
    prompts = [tiny.random_ids(n, pt.PEPOLORN_B["vocab"], 50 + n) for n in (40, 7, 90)]
    eng = Engine(folder, dtype="bf16", page_size=16, num_pages=64, max_running_requests=4)
    got = eng.generate(prompts, temperature=0.0, max_new_tokens=16, ignore_eos=True)
    eng2 = Engine(folder, dtype="bf16", page_size=16, num_pages=64, max_running_requests=4, cuda_graph=False)
    got2 = eng2.generate(prompts, temperature=0.0, max_new_tokens=16, ignore_eos=True)
    assert all(len(r.token_ids) == 16 for r in got)
    # captured and launched steps run the same kernels on the same numbers
    assert [r.token_ids for r in got] == [r.token_ids for r in got2]


def test_trace_replay_of_a_pepolorn_folder(folders, tmp_path):
    import subprocess
    import sys
    import numpy as np
    folder = folders[("A", torch.float32)]
    cfg = _cfg(folder)
    toks = tiny.random_ids(30, cfg["vocab"], 9)
    ref = plain.forward(cfg, _weights(folder), toks, torch.float64)
    lines = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:11], "want": [0, 10]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[11:13], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[13:], "want": [16]}], "end": ["x"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="".join(json.dumps(x) + "\n" for x in lines), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [x for x in r.stdout.split("\n") if x.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()
    a = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    b = np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1)
    for row, pos in ((a[0], 0), (a[1], 10), (b[0], 29)):
        assert float(np.abs(row - ref[pos].numpy()).max()) < 2e-4 * float(ref[pos].abs().max())


def test_command_line_generates_from_a_pepolorn_folder(folders):
    import subprocess
    import sys
    folder = folders[("B", torch.float32)]
    cfg, w = _cfg(folder), _weights(folder)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "prelude"), "--model", folder, "--dtype", "f32", "--prompt-ids", "5,17,3,200",
                          "--max-new-tokens", "5", "--temperature", "0", "--num-pages", "16", "--page-size", "16", "--ignore-eos"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    seq = [5, 17, 3, 200]
    for _ in range(5):
        seq.append(int(plain.forward(cfg, w, seq, torch.float64)[-1].argmax()))
    assert json.loads(out.stdout.strip().splitlines()[0])["token_ids"] == seq[4:]
