"""Pepolorn without a GPU: configuration, run order with layers that run another layer's weights, tensor list,
refusals, cache needs, pages given back behind chunks, and the oracle's mechanisms on inputs with known answers."""
import copy
import math

import pytest
import torch

import pepolorn_tiny as pt
from plain import pepolorn_plain as plain
from prelude_b200.config import ConfigError, load_model_config
from prelude_b200.config.spec import (DecayedLinearAttentionSpec, GatedMlpSpec, MaskedAttentionSpec, NoPositionSpec, ParallelMixerSpec,
                                      RotaryRampScaling, RotaryRatesSpec, RoutedExpertsSpec, StateSpaceSpec)
from prelude_b200.parts.model import DecoderModel
from prelude_b200.parts.registry import CombinedNeed, KvPagesNeed, StateNeed


def test_every_layer_is_parsed_on_its_own():
    spec = load_model_config(pt.PEPOLORN_A).to_model_spec()
    assert spec.architecture == "Pepolorn" and spec.vocab_size == 101 and spec.hidden_size == 44 and spec.tie_embeddings
    assert spec.final_norm.eps == 1e-5 and spec.final_norm.offset == 1.0 and spec.head.tied and spec.embed_name == "embed"
    assert [type(b.mixer) for b in spec.blocks] == [ParallelMixerSpec, StateSpaceSpec, StateSpaceSpec, ParallelMixerSpec]
    assert all(b.kind == "postnorm_residual" and b.mixer_norm is None and b.mixer_post_norm.offset == 1.0 for b in spec.blocks)
    assert [b.prefix for b in spec.blocks] == ["l0", "l1", "l3", "l4"]
    par = spec.blocks[0].mixer
    att, lin = par.mixers
    assert isinstance(att, MaskedAttentionSpec) and isinstance(lin, DecayedLinearAttentionSpec)
    assert par.scales == (0.7, 1.3) and par.names == ("left", "right") and par.member_norms is None
    assert (att.num_heads, att.num_kv_heads, att.head_dim, att.value_dim, att.chunk, att.softmax_scale) == (4, 2, 12, 20, 7, 0.3)
    assert att.head_norm_eps == 1e-5 and not att.head_norm_scale and att.head_norm_after_rotation
    assert not att.qkv_bias and not att.o_bias and not att.sink and not att.head_gate and att.window is None and att.softcap is None
    assert isinstance(att.position, RotaryRatesSpec) and (att.position.dims, att.position.base, att.position.adjacent) == (6, 50.0, False)
    assert att.position.scaling == RotaryRampScaling(factor=4.0, original=64.0, fast=8.0, slow=2.0, amplitude_slope=0.1)
    assert (lin.num_heads, lin.head_dim, lin.value_dim, lin.decays) == (3, 10, 6, (0.5, 0.9, 0.99))
    ssm = spec.blocks[1].mixer
    assert (ssm.num_heads, ssm.groups, ssm.state, ssm.head_dim, ssm.conv_taps, ssm.norm_groups) == (4, 2, 10, 6, 3, 3)
    routed, gated = spec.blocks[0].feed_forward, spec.blocks[1].feed_forward
    assert isinstance(routed, RoutedExpertsSpec) and isinstance(gated, GatedMlpSpec)
    assert (routed.n_experts, routed.top_k, routed.expert_size, routed.n_groups, routed.keep_groups, routed.group_score_top) == (6, 2, 10, 3, 2, 2)
    assert routed.correction_name == "correction" and not routed.renormalize
    assert (gated.intermediate_size, gated.activation) == (24, "gelu_tanh")
    assert spec.blocks[2].feed_forward is None and spec.blocks[2].ff_post_norm is None
    later = spec.blocks[3]
    assert later.mixer.mixers[0].position.scaling is None and later.feed_forward.n_groups == 1 and later.feed_forward.keep_groups == 1


def test_a_layer_that_runs_another_layers_weights_is_a_second_call_of_its_block():
    for cfg, order in ((pt.PEPOLORN_A, [0, 1, 0, 2, 3, 2]), (pt.PEPOLORN_B, [0, 1, 2, 1, 3]), (pt.PEPOLORN_C, [0, 1, 2, 3, 0])):
        spec = load_model_config(cfg).to_model_spec()
        assert [c.block for c in spec.order] == order
        resolved = spec.resolved_order()
        assert [c.cache for c in resolved] == list(range(len(order))) and all(c.writes_cache for c in resolved)     # a cache of its own
        model = DecoderModel(spec)
        needs = model.cache_needs()
        assert len(needs) == len(order) and all(n is not None for n in needs)
    # the source may come later in the list, and a chain ends at the layer that has the tensors
    cfg = copy.deepcopy(pt.PEPOLORN_C)
    cfg["layers"][0], cfg["layers"][4] = cfg["layers"][4], cfg["layers"][0]
    cfg["layers"][0]["weights_of"] = 4
    cfg["layers"].append(dict(copy.deepcopy(cfg["layers"][0]), weights_of=0))
    spec = load_model_config(cfg).to_model_spec()
    assert [c.block for c in spec.order] == [0, 1, 2, 3, 0, 0] and spec.blocks[0].prefix == "l4"
    req, _ = DecoderModel(spec).tensors()
    assert "l4.mix.left.q" in req and not any(n.startswith("l0.") or n.startswith("l5.") for n in req)


def test_tensor_list_has_the_designs_names_and_shapes():
    req, opt = DecoderModel(load_model_config(pt.PEPOLORN_A).to_model_spec()).tensors()
    want = {"embed": (101, 44), "final.norm": (44,), "l0.norm1": (44,), "l0.norm2": (44,), "l0.mix.left.q": (48, 44), "l0.mix.left.k": (24, 44),
            "l0.mix.left.v": (40, 44), "l0.mix.left.o": (44, 80), "l0.mix.right.q": (30, 44), "l0.mix.right.k": (30, 44),
            "l0.mix.right.v": (18, 44), "l0.mix.right.g": (18, 44), "l0.mix.right.norm": (18,), "l0.mix.right.o": (44, 18),
            "l0.mlp.router": (6, 44), "l0.mlp.correction": (6,), "l0.mlp.e0.gate": (10, 44), "l0.mlp.e5.up": (10, 44), "l0.mlp.e3.down": (44, 10),
            "l1.mix.in": (24 + 24 + 40 + 4, 44), "l1.mix.conv": (64, 3), "l1.mix.conv.b": (64,), "l1.mix.dt_bias": (4,), "l1.mix.A_log": (4,),
            "l1.mix.D": (4,), "l1.mix.norm": (24,), "l1.mix.o": (44, 24), "l1.mlp.gate": (24, 44), "l1.mlp.up": (24, 44), "l1.mlp.down": (44, 24),
            "l3.norm1": (44,), "l3.mix.in": (33 + 33 + 18 + 3, 44), "l3.mix.conv": (51, 5), "l4.mlp.e4.gate": (14, 44), "l4.mlp.correction": (5,)}
    for name, shape in want.items():
        assert tuple(req[name].shape) == shape, name
    assert not any(n.startswith(("l2.", "l5.")) for n in req)                     # they run the weights of layers 0 and 3
    assert "l3.norm2" not in req and not any(n.startswith("l3.mlp") for n in req)
    assert not any(n.endswith((".b", ".sink", "q.norm", "k.norm")) and ".left." in n for n in req)
    assert "head" not in req and "head" in opt                                    # the head is the embedding table
    assert req["l0.norm1"].role == "norm_zero" and req["l0.mix.right.norm"].role == "norm"


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][1].update(type="window"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(heads=5), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=14), "at most the head's 12"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=5), "even"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5, 0.9]), "one non-negative number for each of the 3 heads"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "equal parts"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "cannot come from"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "unknown kind"),
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
    (lambda c: c["layers"][2].update(weights_of=9), "weights_of"),
    (lambda c: c["layers"][3]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "non-empty"),
])
def test_a_configuration_that_cannot_be_run_is_refused_with_the_reason(change, word):
    cfg = copy.deepcopy(pt.PEPOLORN_A)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        load_model_config(cfg)
    assert word in str(e.value)


def test_options_left_out_of_a_mixer_are_off():
    spec = load_model_config(pt.PEPOLORN_C).to_model_spec()
    att = spec.blocks[2].mixer.mixers[0]
    assert isinstance(att.position, NoPositionSpec) and att.chunk == 1
    cfg = copy.deepcopy(pt.PEPOLORN_C)
    cfg["layers"][2]["mixer"]["left"].pop("mask")
    cfg["layers"][1]["mlp"]["router"].pop("groups")
    spec = load_model_config(cfg).to_model_spec()
    assert spec.blocks[2].mixer.mixers[0].chunk is None
    assert (spec.blocks[1].feed_forward.n_groups, spec.blocks[1].feed_forward.keep_groups) == (1, 1)


def test_cache_needs_of_every_mixer():
    model = DecoderModel(load_model_config(pt.PEPOLORN_A).to_model_spec())
    needs = model.cache_needs()
    par = CombinedNeed((KvPagesNeed(2, 12, None, v_heads=2, v_head_dim=20, chunk=7), StateNeed((3, 10, 6), torch.float32)))
    assert needs[0] == par and needs[2] == par
    assert needs[1] == CombinedNeed((StateNeed((4, 10, 6), torch.float32), StateNeed((2, 64), None)))
    assert needs[3] == needs[5] == CombinedNeed((StateNeed((3, 9, 11), torch.float32), StateNeed((4, 51), None)))
    caps = model.runtime_caps()
    assert caps.kv_cache and caps.state_slots and caps.cuda_graph


def test_pages_behind_a_chunk_are_given_back_and_two_calls_of_a_block_hold_pages_of_their_own():
    from prelude_b200.cache.manager import CacheManager
    model = DecoderModel(load_model_config(pt.PEPOLORN_A).to_model_spec())
    cache = CacheManager(model.cache_needs(), 4, 40, 2, torch.device("cpu"), torch.float32)
    assert cache.group_of[(0, 0)] == cache.group_of[(2, 0)] != cache.group_of[(4, 0)]       # equal needs share a pool, not pages
    assert len(cache.groups[cache.group_of[(0, 0)]].members) == 2
    cache.add_request("a")
    cache.grow("a", 30)
    cache.trim("a")
    cache.check()
    tables = cache.block_tables(["a"])
    held = lambda row: [i for i, p in enumerate(row) if int(p) >= 0]
    # the next query is position 30: with chunks of 7 its chunk began at 28, with chunks of 13 at 26
    assert held(tables[cache.group_of[(0, 0)]][0]) == [7] and held(tables[cache.group_of[(4, 0)]][0]) == [6, 7]


# -- the oracle's mechanisms on inputs with known answers ----------------------------------------------------------------
def test_plain_chunk_mask():
    seen = plain.chunk_mask(7, 3)
    assert seen.tolist() == [[j <= i and i // 3 == j // 3 for j in range(7)] for i in range(7)]
    assert plain.chunk_mask(4, None).tolist() == [[j <= i for j in range(4)] for i in range(4)]


def test_plain_rates_follow_the_ramp_and_the_amplitude_grows_with_the_factor():
    rates, amp = plain.ramped_rates(8, 100.0, None)
    assert amp == 1.0 and rates == [100.0 ** (-2 * i / 8) for i in range(4)]
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}
    rates, amp = plain.ramped_rates(6, 50.0, sc)
    assert abs(amp - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    f = [50.0 ** (-2 * i / 6) for i in range(3)]
    # the ramp runs from pair 0 (where 8 turns fit the original length) to pair 2
    assert rates[0] == f[0] and abs(rates[1] - (0.5 * f[1] / 4 + 0.5 * f[1])) < 1e-15 and abs(rates[2] - f[2] / 4) < 1e-15
    from prelude_b200.config.spec import RotaryRatesSpec, RotaryRampScaling
    from prelude_b200.parts.rope import rotary_rates
    got, got_amp = rotary_rates(RotaryRatesSpec(6, 50.0, False, RotaryRampScaling(4.0, 64, 8.0, 2.0)))
    assert got == rates and got_amp == amp


def test_plain_rotation_pairs_halves_and_the_norm_after_it_sees_the_amplitude():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64)
    y = plain.rotate_halves(x, torch.tensor([3]), [0.5, 0.25], 2.0)
    c0, s0, c1, s1 = math.cos(1.5), math.sin(1.5), math.cos(0.75), math.sin(0.75)
    want = [2 * (1 * c0 - 3 * s0), 2 * (2 * c1 - 4 * s1), 2 * (3 * c0 + 1 * s0), 2 * (4 * c1 + 2 * s1), 5.0]
    assert torch.allclose(y.reshape(-1), torch.tensor(want, dtype=torch.float64), atol=1e-14)
    # the turned part is twice as long, the rest is not: norming before and after the rotation differ
    before = plain.rotate_halves(plain.unit_rms(x, 0.0), torch.tensor([3]), [0.5, 0.25], 2.0)
    after = plain.unit_rms(y, 0.0)
    assert float((before - after).abs().max()) > 0.1 and abs(float((after * after).mean()) - 1.0) < 1e-12


def test_plain_decayed_state_in_closed_form():
    T, d, e = 6, 3, 2
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(T, 1, n, generator=g, dtype=torch.float64) for n in (d, d, e))
    o = plain.decayed_state(q, k, v, torch.tensor([0.5], dtype=torch.float64))
    for t in range(T):
        want = sum(0.5 ** (t - j) * float(q[t, 0] @ k[j, 0]) * v[j, 0] for j in range(t + 1))
        assert torch.allclose(o[t, 0], want, atol=1e-12)
    keep = plain.decayed_state(q, k, v, torch.tensor([1.0], dtype=torch.float64))
    assert torch.allclose(keep[-1, 0], sum(float(q[-1, 0] @ k[j, 0]) * v[j, 0] for j in range(T)), atol=1e-12)


def test_plain_router_chooses_by_corrected_scores_inside_the_kept_groups_and_weighs_by_the_plain_ones():
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}
    logits = torch.tensor([[2.0, -1.0, 0.5, 0.4, -3.0, 3.0]], dtype=torch.float64)
    eye = torch.eye(6, dtype=torch.float64)
    zero = torch.zeros(6, dtype=torch.float64)
    s = torch.sigmoid(logits[0])
    # groups (0,1) (2,3) (4,5): sums of the two largest are s0+s1, s2+s3, s4+s5; the last is the smallest
    ids, w = plain.route(logits, eye, zero, r)
    assert sorted(ids[0].tolist()) == [0, 2] and torch.allclose(w[0], s[ids[0]])
    # a correction that lifts the last group and sinks the first below zero: all of group 0's choice scores are negative,
    # the group must lose as a negative sum, not as zero
    corr = torch.tensor([-2.0, -2.0, -1.5, -1.4, 1.0, -0.9], dtype=torch.float64)
    ids, w = plain.route(logits, eye, corr, r)
    assert sorted(ids[0].tolist()) == [4, 5] and torch.allclose(w[0], s[ids[0]])            # weights without the correction
    # with every group kept expert 0 (choice score about -1.1) loses to expert 3 (about -0.8) although its plain score is largest
    ids, _ = plain.route(logits, eye, torch.tensor([-2.0, -9.0, -9.0, -1.4, -9.0, 0.0], dtype=torch.float64), {"experts": 6, "top": 2})
    assert sorted(ids[0].tolist()) == [3, 5]


def test_plain_gelu_and_norm():
    z = torch.tensor([-2.0, 0.0, 0.5, 3.0], dtype=torch.float64)
    want = [0.5 * t * (1 + math.tanh(math.sqrt(2 / math.pi) * (t + 0.044715 * t ** 3))) for t in z.tolist()]
    assert torch.allclose(plain.gelu_tanh(z), torch.tensor(want, dtype=torch.float64), atol=1e-15)
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    got = plain.zero_centred_norm(x, torch.tensor([0.0, -0.5], dtype=torch.float64), 0.0)
    assert torch.allclose(got, torch.tensor([[3.0 / math.sqrt(12.5), 0.5 * 4.0 / math.sqrt(12.5)]], dtype=torch.float64))
