"""Nedesun on the GPU against the plain implementation: every mechanism alone, then whole models through every way
of cutting requests into steps, in 32-bit and in bfloat16, with pools so small that pages and slots are used again."""
import copy
import json
import math
import os

import pytest
import torch

import harness
import nedesun_tiny as nt
import tiny
from plain import nedesun_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# bfloat16: five to seven layers whose side-by-side members and recurrent heads are brought to unit size each (a small
# output is scaled up together with its rounding) leave the median position at a quarter of this bound; a fault of a
# mechanism moves every logit by its own size
TOL = {torch.float32: (2e-4, 0.0), torch.bfloat16: (0.0, 8e-2)}


def _weights(folder):
    return {k: v for k, v in tiny.read_weights(folder).items()}


def _cfg(folder):
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def _reference(folder, reqs):
    cfg, w = _cfg(folder), _weights(folder)
    return {rid: plain.forward(cfg, w, toks, torch.float64) for rid, toks in reqs.items()}


def _compare(got, ref, dtype, loosen=1.0):
    """Every position within the bound in 32-bit; in bfloat16 the median well within it and no more than a tenth of
    the positions off (a fault of a mechanism puts every position after it off)."""
    atol, rel = TOL[dtype]
    off, ratios = [], []
    for (rid, pos), row in got.items():
        want = ref[rid][pos]
        bound = loosen * (atol * max(1.0, float(want.abs().max())) + rel * float(want.abs().max()))
        diff = float((row.double() - want).abs().max())
        ratios.append(diff / bound)
        if diff > bound:
            off.append(f"request {rid} position {pos}: max diff {diff:.3e} > {bound:.3e}")
    allowed = len(got) // 10 if dtype == torch.bfloat16 else 0
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


def _steps_through_mixers(parts, x, cuts, page, dtype, slots=2, use_slot=0):
    """x [T, width] through the mixers ``parts`` (each reads x; later ones may read what earlier ones left in the step's
    workspace), cut into the steps ``cuts``; returns every mixer's outputs one below the other."""
    from prelude_b200.cache.manager import CacheManager
    from prelude_b200.engine.batch import StepItem, build_step_batch
    dev = torch.device(DEV)
    T = x.shape[0]
    cache = CacheManager([p.cache_need() for p in parts], page, -(-T // page) + 1, slots, dev, dtype)
    for i in range(use_slot):                      # the request does not get slot 0
        cache.add_request(f"other{i}")
    cache.add_request("a")
    got, at = [[] for _ in parts], 0
    for n in cuts:
        cache.grow("a", at + n)
        batch = build_step_batch([StepItem("a", [0] * n, at, [])], cache.block_tables(["a"]), [cache.slot_of("a")], dev, 10, 1 << 20)
        cache.zero_fresh_state()
        xs = x[at:at + n].to(DEV).contiguous()
        for i, part in enumerate(parts):
            got[i].append(part.forward(xs, batch, cache.layer_cache(i), True).float().cpu())
        assert int(batch.status.item()) == 0
        cache.trim("a")
        at += n
    assert at == T
    return [torch.cat(g).double() for g in got]


def _cuts(T, head):
    return [head] + [1] * (T - head)


def _close(got, want, tol, what):
    assert float((got - want).abs().max()) < tol * float(want.abs().max()), what


# -- mechanisms alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("heads,kv,dim,vdim,rot,chunk,cap,page", [
    (3, 1, 10, 14, 6, 9, 5.0, 4), (8, 2, 64, 64, 64, 48, 30.0, 16), (2, 2, 12, 6, 12, 13, 2.5, 8), (4, 2, 32, 64, 16, 64, 15.0, 16),
    (1, 1, 16, 16, 2, 1, 50.0, 8), (6, 3, 24, 40, 8, 21, 4.0, 16), (4, 1, 128, 128, 64, 32, 20.0, 16), (2, 1, 8, 16, None, None, None, 8)])
def test_chunked_attention_with_blended_values_equals_the_plain_one(dtype, heads, kv, dim, vdim, rot, chunk, cap, page):
    """Two attention mixers on one input: the first keeps its values, the second blends its own with them.  One token
    is made to stand out: queries of its chunk find it, the first query of the next chunk must not.  Scores are large
    enough for the cap to bend them.  Whole, with a decoded tail that crosses chunk and page borders, and in portions
    whose cuts fall inside chunks."""
    from prelude_b200.config.spec import MaskedAttentionSpec, NoPositionSpec, RotaryRatesSpec, ValueBlendSpec
    from prelude_b200.parts.registry import RunContext, make_part
    width, T, head_tokens = 48, 100, 55
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    scale = (3.0 if dtype == torch.float32 else 1.2) / math.sqrt(dim)
    m = nt.attention(heads, kv, dim, vdim, scale, chunk, rot, 70.0, cap, True, None)["mixer"]
    if chunk is None:
        del m["mask"]
    if rot is None:
        del m["rot"]
    if cap is None:
        del m["softcap"]
    w = {}
    for p in ("a", "b"):
        w.update({f"{p}.q": torch.randn(heads * dim, width, generator=g) * 0.3, f"{p}.k": torch.randn(kv * dim, width, generator=g) * 0.3,
                  f"{p}.v": torch.randn(kv * vdim, width, generator=g) * 0.3, f"{p}.o": torch.randn(width, heads * vdim, generator=g) * 0.2,
                  f"{p}.q.b": torch.randn(heads * dim, generator=g) * 0.5, f"{p}.k.b": torch.randn(kv * dim, generator=g) * 0.5,
                  f"{p}.v.b": torch.randn(kv * vdim, generator=g) * 0.5, f"{p}.o.b": torch.randn(width, generator=g) * 0.5,
                  f"{p}.g": torch.randn(heads, width, generator=g) * 0.3, f"{p}.vmix": torch.tensor(0.35 if p == "b" else 0.9)})
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g)
    x[58] *= 3.0
    x = x.to(dtype)
    wd = {k: v.double() for k, v in w.items()}
    shared = {}
    want = [plain.chunked_attention(x.double(), wd, p, m, 1e-5, shared) for p in ("a", "b")]
    if cap is not None and cap < 10.0:
        free = plain.chunked_attention(x.double(), wd, "a", dict(m, softcap=None, v_mix=False), 1e-5, {})
        assert float((free - want[0]).abs().max()) > 0.02 * float(want[0].abs().max())          # the cap matters here
    alone = plain.chunked_attention(x.double(), wd, "b", dict(m, v_mix=False), 1e-5, {})
    assert float((alone - want[1]).abs().max()) > 0.02 * float(want[1].abs().max())             # and so does the blend
    position = NoPositionSpec() if rot is None else RotaryRatesSpec(rot, 70.0, False, None)
    parts = []
    for p, source in (("a", True), ("b", False)):
        spec = MaskedAttentionSpec(width, heads, kv, dim, vdim, scale, position, qkv_bias=True, o_bias=True, chunk=chunk, softcap=cap,
                                   head_gate=True, value_blend=ValueBlendSpec("shared", source))
        part = make_part("mixer", spec, p)
        part.load(lambda name: w[name], RunContext(torch.device(DEV), dtype))
        parts.append(part)
    tol = 5e-5 if dtype == torch.float32 else 4e-2
    for cuts in (_cuts(T, head_tokens), [T], [2, 30, 3, 26, 2, 37]):
        got = _steps_through_mixers(parts, x, cuts, page, dtype)
        _close(got[0], want[0], tol, ("source", cuts[:3]))
        _close(got[1], want[1], tol, ("blended", cuts[:3]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("heads,kv,dim,vdim,window,keep,page", [
    (4, 2, 12, 20, 7, 3, 4), (8, 2, 64, 64, 50, 5, 16), (2, 1, 10, 6, 19, 6, 8), (4, 4, 32, 32, 33, 16, 16), (2, 1, 16, 16, 8, 0, 8),
    (4, 4, 8, 8, 1, 1, 8), (6, 3, 16, 48, None, 0, 8), (4, 1, 128, 128, 16, 18, 16), (3, 3, 24, 40, 30, 40, 16)])
def test_window_attention_with_kept_first_tokens_and_a_sink_equals_the_plain_one(dtype, heads, kv, dim, vdim, window, keep, page):
    """The attention of the parallel mixer alone.  An early token stands out: while it is among the kept ones every later
    query finds it, however far; a token past them is lost at the very query that leaves it behind.  Sinks take a good
    share of every softmax.  Pages that hold neither kept tokens nor the window are given back between steps."""
    from prelude_b200.config.spec import MaskedAttentionSpec, NoPositionSpec
    from prelude_b200.parts.registry import RunContext, make_part
    width, T, head_tokens = 40, 110, 61
    g = torch.Generator().manual_seed(heads * 100 + dim + (window or 0))
    scale = (3.0 if dtype == torch.float32 else 1.2) / math.sqrt(dim)
    m = nt.left(heads, kv, dim, vdim, scale, window, keep)
    if window is None:
        del m["mask"]
    w = {"mix.q": torch.randn(heads * dim, width, generator=g) * 0.3, "mix.k": torch.randn(kv * dim, width, generator=g) * 0.3,
         "mix.v": torch.randn(kv * vdim, width, generator=g) * 0.3, "mix.o": torch.randn(width, heads * vdim, generator=g) * 0.2,
         "mix.q.norm": 1.0 + 0.4 * torch.randn(dim, generator=g), "mix.k.norm": 1.0 + 0.4 * torch.randn(dim, generator=g),
         "mix.sink": torch.linspace(0.5, 2.5, heads)}
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g)
    x[1] *= 3.0
    x[58] *= 3.0
    x = x.to(dtype)
    wd = {k: v.double() for k, v in w.items()}
    want = plain.window_sink_attention(x.double(), wd, "mix", m, 1e-5)
    no_sink = plain.window_sink_attention(x.double(), dict(wd, **{"mix.sink": wd["mix.sink"] - 50.0}), "mix", m, 1e-5)
    assert float((want - no_sink).abs().max()) > 0.02 * float(want.abs().max())                 # the sinks matter here
    if keep and window is not None and keep < T - window:
        forgot = plain.window_sink_attention(x.double(), wd, "mix", dict(m, mask={"size": window, "keep_first": 0}), 1e-5)
        assert float((want - forgot).abs().max()) > 0.02 * float(want.abs().max())              # and the kept tokens
    spec = MaskedAttentionSpec(width, heads, kv, dim, vdim, scale, NoPositionSpec(), head_norm_eps=1e-5, window=window,
                               keep_first=keep if window is not None else 0, sink=True)
    part = make_part("mixer", spec, "mix")
    part.load(lambda name: w[name], RunContext(torch.device(DEV), dtype))
    tol = 5e-5 if dtype == torch.float32 else 4e-2
    for cuts in (_cuts(T, head_tokens), [T], [2, 30, 3, 26, 2, 47], [1] * T):
        got = _steps_through_mixers([part], x, cuts, page, dtype)[0]
        _close(got, want, tol, cuts[:3])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("heads,kv,dim,vdim,taps", [(4, 2, 10, 6, 3), (4, 2, 64, 32, 4), (3, 3, 9, 11, 5), (1, 1, 16, 16, 1), (8, 4, 32, 16, 4),
                                                    (4, 4, 8, 24, 2), (2, 1, 128, 128, 4), (6, 2, 20, 40, 3), (2, 2, 200, 17, 4)])
def test_gated_delta_rule_mixer_equals_the_plain_one(dtype, heads, kv, dim, vdim, taps):
    """The gated delta rule alone: a whole sequence at once, token by token, and in portions shorter than the
    convolution is long; in a state slot other than the first; decays between slow and fast, so that a state that is
    lost, carried in fewer bits or started from another sequence's shows."""
    from prelude_b200.config.spec import GatedDeltaSpec
    from prelude_b200.parts.registry import RunContext, make_part
    width, T = 40, 90
    g = torch.Generator().manual_seed(heads * 10 + dim)
    m = nt.right(heads, kv, dim, vdim, taps)
    qk, inner = kv * dim, heads * vdim
    w = {"mix.q": torch.randn(qk, width, generator=g) * 0.3, "mix.k": torch.randn(qk, width, generator=g) * 0.3,
         "mix.v": torch.randn(inner, width, generator=g) * 0.3, "mix.q.conv": torch.randn(qk, taps, generator=g) * 0.5,
         "mix.k.conv": torch.randn(qk, taps, generator=g) * 0.5, "mix.v.conv": torch.randn(inner, taps, generator=g) * 0.5,
         "mix.b": torch.randn(heads, width, generator=g) * 0.3, "mix.a": torch.randn(heads, width, generator=g) * 0.3,
         "mix.A_log": torch.linspace(-3.0, 1.0, heads), "mix.dt_bias": torch.randn(heads, generator=g),
         "mix.g": torch.randn(inner, width, generator=g) * 0.3, "mix.norm": 1.0 + 0.3 * torch.randn(vdim, generator=g),
         "mix.o": torch.randn(width, inner, generator=g) * 0.2}
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g).to(dtype)
    want = plain.gated_delta_rule(x.double(), {k: v.double() for k, v in w.items()}, "mix", m, 1e-5)
    part = make_part("mixer", GatedDeltaSpec(width, heads, kv, dim, vdim, taps, 1e-5), "mix")
    part.load(lambda name: w[name], RunContext(torch.device(DEV), dtype))
    tol = 5e-5 if dtype == torch.float32 else 4e-2
    for cuts, slot in (([T], 0), (_cuts(T, 40), 1), ([2, 1, 1, 2, 3, 1, 30, 2, 48], 2), ([1] * T, 0)):
        got = _steps_through_mixers([part], x, cuts, 16, dtype, slots=3, use_slot=slot)[0]
        _close(got, want, tol, cuts[:3])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("heads,dim,rank", [(3, 12, 5), (4, 32, 16), (1, 32, 8), (2, 64, 32), (2, 22, 3), (5, 8, 1), (1, 128, 64), (2, 200, 24)])
def test_decaying_state_time_mixing_equals_the_plain_one(dtype, heads, dim, rank):
    """Time mixing alone.  The first token is blended with zeros, a step's first token with the input the sequence
    carried; decays between fast and very slow; a bonus that weighs the current token differently per channel."""
    from prelude_b200.config.spec import WkvSpec
    from prelude_b200.parts.registry import RunContext, make_part
    width, T = 40, 90
    g = torch.Generator().manual_seed(heads * 10 + dim)
    inner = heads * dim
    m = {"heads": heads, "dim": dim}
    w = {f"mix.mu.{s}": torch.rand(width, generator=g) for s in "rkvgw"}
    w.update({"mix.r": torch.randn(inner, width, generator=g) * 0.3, "mix.k": torch.randn(inner, width, generator=g) * 0.3,
              "mix.v": torch.randn(inner, width, generator=g) * 0.3, "mix.g": torch.randn(inner, width, generator=g) * 0.3,
              "mix.w1": torch.randn(rank, width, generator=g) * 0.3, "mix.w2": torch.randn(inner, rank, generator=g) * 0.5,
              "mix.w0": torch.linspace(-5.0, 0.7, inner), "mix.u": torch.randn(heads, dim, generator=g),
              "mix.norm": 1.0 + 0.3 * torch.randn(inner, generator=g), "mix.o": torch.randn(width, inner, generator=g) * 0.2})
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g).to(dtype)
    want = plain.wkv(x.double(), {k: v.double() for k, v in w.items()}, "mix", m, 1e-5)
    part = make_part("mixer", WkvSpec(width, heads, dim, None, 1e-5), "mix")
    part.load(lambda name: w[name], RunContext(torch.device(DEV), dtype))
    tol = 5e-5 if dtype == torch.float32 else 4e-2
    for cuts, slot in (([T], 0), (_cuts(T, 40), 1), ([2, 1, 1, 2, 3, 1, 30, 2, 48], 2), ([1] * T, 0)):
        got = _steps_through_mixers([part], x, cuts, 16, dtype, slots=3, use_slot=slot)[0]
        _close(got, want, tol, cuts[:3])


def test_a_recurrent_state_carries_what_was_written_hundreds_of_tokens_ago():
    """A slow decay keeps an early token's write readable after 400 more tokens; the kernels' state must show it as
    the plain loop does, in prompt steps and token by token."""
    from prelude_b200.config.spec import GatedDeltaSpec, WkvSpec
    from prelude_b200.parts.registry import RunContext, make_part
    width, T = 32, 420
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, width, generator=g) * 0.3
    x[5] *= 12.0
    heads, dim = 2, 16
    inner = heads * dim
    wk = {f"mix.mu.{s}": torch.rand(width, generator=g) for s in "rkvgw"}
    wk.update({"mix.r": torch.randn(inner, width, generator=g) * 0.3, "mix.k": torch.randn(inner, width, generator=g) * 0.3,
               "mix.v": torch.randn(inner, width, generator=g) * 0.3, "mix.g": torch.randn(inner, width, generator=g) * 0.3,
               "mix.w1": torch.randn(4, width, generator=g) * 0.1, "mix.w2": torch.randn(inner, 4, generator=g) * 0.1,
               "mix.w0": torch.full((inner,), -7.0), "mix.u": torch.zeros(heads, dim), "mix.norm": torch.ones(inner),
               "mix.o": torch.randn(width, inner, generator=g) * 0.2})
    gd = {"mix.q": torch.randn(inner, width, generator=g) * 0.3, "mix.k": torch.randn(inner, width, generator=g) * 0.3,
          "mix.v": torch.randn(inner, width, generator=g) * 0.3, "mix.q.conv": torch.randn(inner, 2, generator=g) * 0.5,
          "mix.k.conv": torch.randn(inner, 2, generator=g) * 0.5, "mix.v.conv": torch.randn(inner, 2, generator=g) * 0.5,
          "mix.b": torch.randn(heads, width, generator=g) * 0.1 - 3.0, "mix.a": torch.randn(heads, width, generator=g) * 0.1,
          "mix.A_log": torch.full((heads,), -7.0), "mix.dt_bias": torch.zeros(heads), "mix.g": torch.randn(inner, width, generator=g) * 0.3,
          "mix.norm": torch.ones(dim), "mix.o": torch.randn(width, inner, generator=g) * 0.2}
    for w, spec, fn, m in ((wk, WkvSpec(width, heads, dim, None, 1e-5), plain.wkv, {"heads": heads, "dim": dim}),
                           (gd, GatedDeltaSpec(width, heads, heads, dim, dim, 2, 1e-5), plain.gated_delta_rule, nt.right(heads, heads, dim, dim, 2))):
        wd = {k: v.double() for k, v in w.items()}
        want = fn(x.double(), wd, "mix", m, 1e-5)
        x0 = x.clone()
        x0[5] = x[5] / 12.0
        assert float((fn(x0.double(), wd, "mix", m, 1e-5)[-10:] - want[-10:]).abs().max()) > 0.05 * float(want[-10:].abs().max())
        part = make_part("mixer", spec, "mix")
        part.load(lambda name: w[name], RunContext(torch.device(DEV), torch.float32))
        for cuts in ([T], [3, 200, 2, 150] + [1] * 65):
            got = _steps_through_mixers([part], x, cuts, 16, torch.float32)[0]
            _close(got, want, 1e-4, cuts[:3])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_embedding_rows_are_scaled_in_32_bit(dtype):
    from prelude_b200.config.spec import ScaledEmbeddingSpec
    from prelude_b200.parts.registry import RunContext, make_part
    g = torch.Generator().manual_seed(8)
    table = torch.randn(37, 52, generator=g).to(dtype)
    part = make_part("embedding", ScaledEmbeddingSpec(37, 52, 1.7, name="embed"), "")
    part.load(lambda name: table, RunContext(torch.device(DEV), dtype))
    import types
    ids = torch.tensor([5, 0, 36, 5, 17], dtype=torch.int32, device=DEV)
    got = part.forward(types.SimpleNamespace(token_ids=ids))
    assert got.dtype == torch.float32
    assert float((got.cpu().double() - table[ids.cpu().long()].double() * 1.7).abs().max()) < 1e-6


# -- whole models ----------------------------------------------------------------------------------------------------
REQUESTS = {"N": {"n1": 1, "n2": 2, "n19": 19, "n70": 70, "n33": 33}, "P": {"p3": 3, "p150": 150, "p64": 64, "p41": 41, "p97": 97},
            "Q": {"q1": 1, "q9": 9, "q40": 40, "q17": 17}}


def _requests(which):
    v = nt.PARAMS[which][0]["vocab"]
    return {rid: tiny.random_ids(n, v, sum(map(ord, rid))) for rid, n in REQUESTS[which].items()}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("nedesun")
    return {(w, d): nt.make_folder(root, w, d) for w in "NPQ" for d in (torch.float32, torch.bfloat16)}


@pytest.fixture(scope="module")
def references(folders):
    return {w: _reference(folders[(w, torch.bfloat16)], _requests(w)) for w in "NPQ"}, \
           {w: _reference(folders[(w, torch.float32)], _requests(w)) for w in "NPQ"}


def test_the_stream_after_every_layer_equals_the_plain_one(folders):
    """Layer by layer in 32-bit: the first layer that differs names the mechanism."""
    from prelude_b200.engine.batch import StepItem, build_step_batch
    from prelude_b200.engine.loading import load_model, make_runner
    from prelude_b200.engine.runner import StepEntry
    from prelude_b200.ops import kernels as K
    from prelude_b200.ops.linear import step_status
    for which in "NPQ":
        folder = folders[(which, torch.float32)]
        cfg, w = _cfg(folder), _weights(folder)
        toks = tiny.random_ids(45, cfg["vocab"], 4)
        want = []
        plain.forward(cfg, w, toks, torch.float64, layers_out=want)
        model = load_model(folder, torch.float32, DEV)
        runner = make_runner(model, page_size=nt.PARAMS[which][2], num_pages=16, max_slots=1)
        runner.reserve([StepEntry("x", toks, [])])
        batch = build_step_batch([StepItem("x", toks, 0, [])], runner.cache.block_tables(["x"]), [runner.cache.slot_of("x")], runner.device,
                                 model.spec.vocab_size, model.spec.max_positions)
        runner.cache.zero_fresh_state()
        with step_status(batch.status):
            res = model.embedding.forward(batch)
            delta = None
            for i, call in enumerate(model.order):
                delta = model.blocks[call.block].forward(delta, res, batch, runner.caches[call.cache], call.writes_cache)
                x, scale = (delta.x, delta.scale) if isinstance(delta, K.Scaled) else (delta, 1.0)
                if isinstance(x, K.PartialSums):
                    x = x.parts.sum(0)
                got = (res + scale * x.float()).cpu().double()      # the block leaves its last sublayer's output to be added by the next norm
                assert float((got - want[i]).abs().max()) < 1e-4 * max(1.0, float(want[i].abs().max())), f"{which}: layer {i}"
        assert int(batch.status.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["N", "P", "Q"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed", "mixed_graphs"])
def test_cuts_match_plain(folders, references, which, dtype, cut):
    """Whole prompts, a decoded tail that crosses windows, chunks and page borders, portions down to two tokens, and
    mixed batches in a pool that holds less than all requests (pages and slots used again), launched and captured."""
    reqs = _requests(which)
    ref = references[0 if dtype == torch.bfloat16 else 1][which]
    page = nt.PARAMS[which][2]
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


@pytest.mark.parametrize("which", ["N", "P"])
def test_batched_requests_equal_each_alone_in_32_bit(folders, which):
    reqs = _requests(which)
    page = nt.PARAMS[which][2]
    folder = folders[(which, torch.float32)]
    alone = harness.run_schedule(_runner(folder, torch.float32, page, 64), harness.whole(reqs))
    together = harness.run_schedule(_runner(folder, torch.float32, page, 64, max_slots=5),
                                    [([(rid, toks, list(range(len(toks)))) for rid, toks in reqs.items()], list(reqs))])
    for key, row in alone.items():
        assert float((row - together[key]).abs().max()) <= 2e-5 * float(row.abs().max()), key


def test_cuts_agree_in_32_bit(folders):
    """However a request is cut, its logits agree to rounding of the last bits."""
    reqs = {"n70": _requests("N")["n70"]}
    folder = folders[("N", torch.float32)]
    a = harness.run_schedule(_runner(folder, torch.float32, 4, 20), harness.whole(reqs))
    b = harness.run_schedule(_runner(folder, torch.float32, 4, 20), harness.portions(reqs))
    c = harness.run_schedule(_runner(folder, torch.float32, 4, 20), harness.tail_decode(reqs, 50))
    for key, row in a.items():
        bound = 2e-5 * float(row.abs().max())
        assert float((row - b[key]).abs().max()) <= bound and float((row - c[key]).abs().max()) <= bound, key


def test_sharp_attention_finds_keys_far_back_and_at_every_edge(tmp_path):
    """Query and key matrices scaled up make every softmax pick few keys, wherever they lie: among the kept first
    tokens hundreds of positions back, on either side of a page border, just inside a window or chunk and just outside
    (where it must not be found).  32-bit, prompt in one step, in portions, and with a decoded tail longer than the
    windows and chunks."""
    cfg = copy.deepcopy(nt.NEDESUN_N)
    tensors = nt.random_tensors(cfg, seed=21, std=0.25, norm_jitter=0.3)
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] == "attention":
            for n in ("q", "k"):
                tensors[f"l{i}.mix.{n}"] = tensors[f"l{i}.mix.{n}"] * 2.0
        if layer["type"] == "parallel":
            for n in ("q.norm", "k.norm"):
                tensors[f"l{i}.mix.left.{n}"] = tensors[f"l{i}.mix.left.{n}"] * 2.0
            tensors[f"l{i}.mix.left.sink"] = tensors[f"l{i}.mix.left.sink"] + 2.0
    folder = nt.make_folder_from_tensors(tmp_path, "sharp", cfg, tensors)
    reqs = {"s": tiny.random_ids(300, cfg["vocab"], 77)}
    ref = _reference(folder, reqs)
    for schedule in (harness.whole(reqs), harness.portions(reqs, (37, 2, 64, 3, 29)), harness.tail_decode(reqs, 70)):
        got = harness.run_schedule(_runner(folder, torch.float32, 16, 19), schedule)
        _compare(got, ref, torch.float32, loosen=5.0)        # scores of tens: their 32-bit rounding shows in the weights


def test_long_decoding_through_freed_and_reused_slots(folders):
    """Two requests decoded token by token for 120 steps side by side after short prompts, then a third takes the
    slot (its states, its convolution inputs, its previous token) and the pages that the first gave back."""
    cfg = nt.NEDESUN_N
    reqs = {"a": tiny.random_ids(130, cfg["vocab"], 1), "b": tiny.random_ids(127, cfg["vocab"], 2), "c": tiny.random_ids(60, cfg["vocab"], 3)}
    ref = _reference(folders[("N", torch.float32)], reqs)
    steps = [([("a", reqs["a"][:10], list(range(10))), ("b", reqs["b"][:7], list(range(7)))], [])]
    for i in range(120):
        steps.append(([("a", reqs["a"][10 + i:11 + i], [0]), ("b", reqs["b"][7 + i:8 + i], [0])], ["a", "b"] if i == 119 else []))
    steps.append(([("c", reqs["c"], list(range(60)))], ["c"]))
    runner = _runner(folders[("N", torch.float32)], torch.float32, 4, 66, max_slots=2)
    _compare(harness.run_schedule(runner, steps), ref, torch.float32)
    runner.cache.check()


@pytest.mark.parametrize("which,lens,new", [("N", [1, 5, 17], 20), ("P", [9, 64, 2, 31], 12)])
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
    eng = Engine(folder, dtype="f32", page_size=nt.PARAMS[which][2], num_pages=64, max_running_requests=4)
    assert eng.caps.cuda_graph and eng.caps.state_slots
    got = eng.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)
    assert [r.token_ids for r in got] == want
    # portions of a few tokens beside decoding requests, launched kernel by kernel: the same tokens
    eng2 = Engine(folder, dtype="f32", page_size=nt.PARAMS[which][2], num_pages=64, max_running_requests=4,
                  max_num_batched_tokens=7, long_prefill_token_threshold=3, cuda_graph=False)
    assert [r.token_ids for r in eng2.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)] == want
    assert eng.cache.used_pages() == 0 and eng2.cache.used_pages() == 0


def test_generation_in_bfloat16_runs_captured_steps(folders):
    from prelude_b200 import Engine
    folder = folders[("P", torch.bfloat16)]
    prompts = [tiny.random_ids(n, nt.NEDESUN_P["vocab"], 50 + n) for n in (40, 7, 90)]
    eng = Engine(folder, dtype="bf16", page_size=16, num_pages=64, max_running_requests=4)
    got = eng.generate(prompts, temperature=0.0, max_new_tokens=16, ignore_eos=True)
    eng2 = Engine(folder, dtype="bf16", page_size=16, num_pages=64, max_running_requests=4, cuda_graph=False)
    got2 = eng2.generate(prompts, temperature=0.0, max_new_tokens=16, ignore_eos=True)
    assert all(len(r.token_ids) == 16 for r in got)
    # captured and launched steps run the same kernels on the same numbers
    assert [r.token_ids for r in got] == [r.token_ids for r in got2]


def test_trace_replay_of_a_nedesun_folder(folders, tmp_path):
    import subprocess
    import sys
    import numpy as np
    folder = folders[("N", torch.float32)]
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


def test_command_line_generates_from_a_nedesun_folder(folders):
    import subprocess
    import sys
    folder = folders[("P", torch.float32)]
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


# -- the tcgen05 prompt kernel with masks, cap, sink and gate against the general kernel -------------------------------------
@pytest.mark.parametrize("heads,kv,dim,page,window,keep,chunk,cap,sink,gate", [
    (8, 2, 128, 16, 300, 40, None, None, True, False), (8, 2, 128, 16, None, 0, 200, 30.0, False, True), (4, 4, 64, 16, 100, 0, None, None, True, False),
    (16, 2, 64, 32, None, 0, 128, 5.0, False, True), (4, 1, 128, 16, 129, 130, None, None, False, False), (8, 8, 128, 128, 50, 7, None, 8.0, True, True),
    (2, 1, 64, 8, None, 0, 1000, None, False, False), (8, 2, 128, 16, 700, 300, None, None, True, False), (32, 1, 64, 16, None, 0, 77, 20.0, True, True),
    (8, 2, 128, 64, 256, 128, None, None, True, False), (4, 2, 128, 16, None, 0, None, 12.0, True, True)])
def test_prompt_kernel_with_masks_equals_the_general_kernel(heads, kv, dim, page, window, keep, chunk, cap, sink, gate):
    """Random keys and values in scattered pages; requests of unequal length: a long prompt from position 0, a portion far
    into a long context whose pages behind the window (but for the kept first tokens) and behind the chunk were given
    back, a portion that starts inside a key tile, a short one.  Both kernels read the same pages."""
    from prelude_b200.cache.manager import CacheManager
    from prelude_b200.engine.batch import StepItem, build_step_batch
    from prelude_b200.ops import paged_general as G
    from prelude_b200.parts.registry import KvPagesNeed
    dev = torch.device(DEV)
    g = torch.Generator().manual_seed(heads * 31 + dim + (window or 0) + (chunk or 0))
    need = KvPagesNeed(kv, dim, window, v_heads=kv, v_head_dim=dim, keep_first=keep if window else 0, chunk=chunk)
    shape = [(0, 700), (1900, 300), (333, 150), (64, 40), (5, 2)]
    cache = CacheManager([need], page, sum(-(-(a + b) // page) for a, b in shape) + 3, 8, dev, torch.bfloat16)
    items, slots = [], []
    for i, (have, new) in enumerate(shape):
        cache.add_request(i)
        if have:
            cache.grow(i, have)
            cache.trim(i)                                  # as after the step that brought the tokens before
        cache.grow(i, have + new)
        items.append(StepItem(i, [0] * new, have, []))
        slots.append(cache.slot_of(i))
    cache.check()
    lc = cache.layer_cache(0)
    lc.k_pages.copy_(torch.randn(lc.k_pages.shape, generator=g).to(dev, torch.bfloat16))
    lc.v_pages.copy_(torch.randn(lc.v_pages.shape, generator=g).to(dev, torch.bfloat16))
    batch = build_step_batch(items, cache.block_tables(list(range(len(shape)))), slots, dev, 10, 1 << 20)
    if window or chunk:
        assert int((batch.block_tables[0][1][:100] < 0).sum()) > 0          # pages were given back
    q = (torch.randn(batch.n_tokens, heads, dim, generator=g) * 1.5).to(dev, torch.bfloat16)
    sinks = torch.linspace(-1.0, 3.0, heads).to(dev) if sink else None
    gates = torch.randn(batch.n_tokens, heads + 3, generator=g).to(dev, torch.bfloat16)[:, :heads] if gate else None
    scale = 1.0 / math.sqrt(dim)
    assert G._l.library().pb_attention_prefill_tc_plain_pages_supported(heads, kv, dim, page)
    old = G.PROMPT_KERNEL
    try:
        G.PROMPT_KERNEL = "mma"
        want = G.attention_general(q, lc.k_pages, lc.v_pages, dim, batch, 0, scale, window, sinks, keep_first=keep, chunk=chunk, softcap=cap,
                                   gate=gates).float().clone()
        G.PROMPT_KERNEL = "auto"
        got = G.attention_general(q, lc.k_pages, lc.v_pages, dim, batch, 0, scale, window, sinks, keep_first=keep, chunk=chunk, softcap=cap,
                                  gate=gates).float()
    finally:
        G.PROMPT_KERNEL = old
    assert int(batch.status.item()) == 0
    err = (got - want).abs()
    assert float(err.max()) < 4e-2 * float(want.abs().max()) and float(err.mean()) < 4e-3 * float(want.abs().max()), \
        (float(err.max()), float(err.mean()), float(want.abs().max()), int(err.max(dim=-1).values.max(dim=-1).values.argmax()))
