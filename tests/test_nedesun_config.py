"""Nedesun without a GPU: configuration, run order, tensor list, refusals, cache needs, page bookkeeping behind windows
that keep the first tokens and behind chunks, and the oracle's mechanisms on inputs with known answers."""
import copy
import math

import pytest
import torch

import nedesun_tiny as nt
from plain import nedesun_plain as plain
from prelude_b200.config import ConfigError, load_model_config
from prelude_b200.config.spec import (GatedDeltaSpec, MaskedAttentionSpec, NoPositionSpec, ParallelMixerSpec, RotaryRatesSpec, WkvSpec)
from prelude_b200.parts.model import DecoderModel
from prelude_b200.parts.registry import CombinedNeed, KvPagesNeed, StateNeed


def test_every_layer_is_parsed_on_its_own():
    spec = load_model_config(nt.NEDESUN_N).to_model_spec()
    assert spec.architecture == "Nedesun" and spec.vocab_size == 101 and spec.hidden_size == 44 and spec.tie_embeddings
    assert spec.embedding.scale == 1.7 and spec.embedding.name == "embed" and spec.final_norm.eps == 1e-5
    kinds = [type(b.mixer) for b in spec.blocks]
    assert kinds == [ParallelMixerSpec, MaskedAttentionSpec, WkvSpec, MaskedAttentionSpec, MaskedAttentionSpec, ParallelMixerSpec, WkvSpec]
    assert all(b.kind == "prenorm_residual" and b.residual_scale == 0.45 for b in spec.blocks)
    assert [b.feed_forward is None for b in spec.blocks] == [False, False, True, True, False, True, False]
    assert spec.blocks[2].ff_norm is None and spec.blocks[1].feed_forward.intermediate_size == 56
    par = spec.blocks[0].mixer
    left, right = par.mixers
    assert isinstance(left, MaskedAttentionSpec) and isinstance(right, GatedDeltaSpec) and par.scales == (0.5, 0.5)
    assert par.names == ("left", "right") and par.member_norms is not None and par.member_norms[0].suffix == ".out"
    assert (left.num_heads, left.num_kv_heads, left.head_dim, left.value_dim, left.window, left.keep_first) == (4, 2, 12, 20, 7, 3)
    assert left.sink and left.head_norm_eps == 1e-5 and isinstance(left.position, NoPositionSpec) and left.chunk is None
    assert not left.qkv_bias and not left.o_bias and not left.head_gate and left.softcap is None and left.value_blend is None
    assert (right.num_heads, right.num_kv_heads, right.head_dim, right.value_dim, right.conv_taps) == (4, 2, 10, 6, 3)
    att = spec.blocks[1].mixer
    assert (att.num_heads, att.num_kv_heads, att.head_dim, att.value_dim, att.chunk, att.softcap) == (3, 1, 10, 14, 9, 5.0)
    assert att.qkv_bias and att.o_bias and att.head_gate and not att.sink and att.head_norm_eps is None and att.window is None
    assert isinstance(att.position, RotaryRatesSpec) and (att.position.dims, att.position.base, att.position.adjacent) == (6, 50.0, False)
    assert att.value_blend.source and spec.blocks[3].mixer.value_blend is None and not spec.blocks[4].mixer.value_blend.source
    wk = spec.blocks[6].mixer
    assert (wk.num_heads, wk.head_dim, wk.decay_rank) == (2, 22, None)


def test_tensor_list_has_the_designs_names_and_shapes():
    req, _ = DecoderModel(load_model_config(nt.NEDESUN_N).to_model_spec()).tensors()
    want = {"embed": (101, 44), "final.norm": (44,), "l0.norm1": (44,), "l0.norm2": (44,), "l0.mix.left.q": (48, 44), "l0.mix.left.k": (24, 44),
            "l0.mix.left.v": (40, 44), "l0.mix.left.o": (44, 80), "l0.mix.left.q.norm": (12,), "l0.mix.left.k.norm": (12,),
            "l0.mix.left.sink": (4,), "l0.mix.left.out": (44,), "l0.mix.right.out": (44,), "l0.mix.right.q": (20, 44),
            "l0.mix.right.v": (24, 44), "l0.mix.right.q.conv": (20, 3), "l0.mix.right.v.conv": (24, 3), "l0.mix.right.b": (4, 44),
            "l0.mix.right.a": (4, 44), "l0.mix.right.A_log": (4,), "l0.mix.right.dt_bias": (4,), "l0.mix.right.g": (24, 44),
            "l0.mix.right.norm": (6,), "l0.mix.right.o": (44, 24), "l0.mlp.gate": (24, 44), "l0.mlp.up": (24, 44), "l0.mlp.down": (44, 24),
            "l1.mix.q": (30, 44), "l1.mix.q.b": (30,), "l1.mix.k": (10, 44), "l1.mix.v.b": (14,), "l1.mix.o": (44, 42), "l1.mix.o.b": (44,),
            "l1.mix.g": (3, 44), "l1.mix.vmix": (), "l4.mix.vmix": (), "l2.mix.mu.w": (44,), "l2.mix.r": (36, 44), "l2.mix.w0": (36,),
            "l2.mix.u": (3, 12), "l2.mix.norm": (36,), "l2.mix.o": (44, 36)}
    for name, shape in want.items():
        assert tuple(req[name].shape) == shape, name
    assert "l2.norm2" not in req and not any(n.startswith("l2.mlp") for n in req) and "l3.mix.vmix" not in req
    assert "l1.mix.sink" not in req and "l0.mix.left.q.b" not in req and "l1.mix.q.norm" not in req


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][1].update(type="window"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(heads=5), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=12), "at most the head's 10"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=5), "even"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(keep_first=-1), "non-negative"),
    (lambda c: c["layers"][4]["mixer"].update(vdim=6), "blended values"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "unknown kind"),
    (lambda c: c["layers"][2]["mixer"].pop("dim"), "dim"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "non-empty"),
])
def test_a_configuration_that_cannot_be_run_is_refused_with_the_reason(change, word):
    cfg = copy.deepcopy(nt.NEDESUN_N)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        load_model_config(cfg)
    assert word in str(e.value)


def test_options_left_out_of_a_mixer_are_off():
    cfg = copy.deepcopy(nt.NEDESUN_Q)
    att = cfg["layers"][2]["mixer"]
    for key in ("mask", "rot", "softcap", "v_mix"):
        att.pop(key)
    cfg["layers"][4]["mixer"]["v_mix"] = False
    cfg["layers"][1]["mixer"]["left"].pop("mask")
    cfg["layers"][3]["mixer"]["left"]["mask"].pop("keep_first")
    spec = load_model_config(cfg).to_model_spec()
    a = spec.blocks[2].mixer
    assert a.chunk is None and a.softcap is None and a.value_blend is None and isinstance(a.position, NoPositionSpec)
    assert spec.blocks[1].mixer.mixers[0].window is None and spec.blocks[3].mixer.mixers[0].keep_first == 0
    req, _ = DecoderModel(spec).tensors()
    assert not any(n.endswith(".vmix") for n in req)


def test_cache_needs_of_every_mixer():
    model = DecoderModel(load_model_config(nt.NEDESUN_N).to_model_spec())
    needs = [b.cache_need() for b in model.blocks]
    assert needs[0] == CombinedNeed((KvPagesNeed(2, 12, 7, v_heads=2, v_head_dim=20, keep_first=3),
                                     CombinedNeed((StateNeed((4, 10, 6), torch.float32), StateNeed((2, 64), None)))))
    assert needs[1] == KvPagesNeed(1, 10, None, v_heads=1, v_head_dim=14, chunk=9)
    assert needs[2] == CombinedNeed((StateNeed((3, 12, 12), torch.float32), StateNeed((1, 44), None)))
    assert needs[5].parts[1].parts[1] == StateNeed((4, 2 * 27 + 33), None)


def test_pages_behind_a_window_are_given_back_but_for_the_kept_first_tokens():
    from prelude_b200.cache.manager import CacheManager
    page = 4
    cache = CacheManager([KvPagesNeed(1, 8, 6, keep_first=5), KvPagesNeed(1, 8, None, chunk=8)], page, 40, 2, torch.device("cpu"), torch.float32)
    cache.add_request("a")
    cache.grow("a", 30)
    cache.trim("a")
    cache.check()
    tables = cache.block_tables(["a"])
    win, chk = (tables[cache.group_of[i]][0] for i in (0, 1))
    held = lambda row: [i for i, p in enumerate(row) if int(p) >= 0]
    # the next query is position 30: it sees 25..29 and 0..4 behind the window; its chunk started at 24
    assert held(win) == [0, 1, 6, 7] and held(chk) == [6, 7]
    cache.grow("a", 33)
    cache.trim("a")
    assert held(cache.block_tables(["a"])[cache.group_of[1]][0]) == [8]
    cache.release("a")
    cache.check()
    assert cache.used_pages() == 0


# -- the oracle's mechanisms on inputs with known answers ---------------------------------------------------------------
def test_who_sees_whom():
    see = plain.visible(12, window=4, keep_first=2)
    assert see[9].nonzero().flatten().tolist() == [0, 1, 6, 7, 8, 9] and see[3].nonzero().flatten().tolist() == [0, 1, 2, 3]
    see = plain.visible(12, chunk=5)
    assert see[9].nonzero().flatten().tolist() == [5, 6, 7, 8, 9] and see[10].nonzero().flatten().tolist() == [10]
    assert plain.visible(5)[4].all() and not plain.visible(5)[2, 3]


def test_a_sink_only_takes_weight():
    q, k, v = torch.zeros(3, 2, 4, dtype=torch.float64), torch.zeros(3, 1, 4, dtype=torch.float64), torch.ones(3, 1, 2, dtype=torch.float64)
    out = plain.softmax_attention(q, k, v, 1.0, plain.visible(3), sink=torch.tensor([0.0, math.log(3.0)], dtype=torch.float64))
    # scores 0 over t + 1 keys: the weights sum to (t + 1) / (t + 1 + exp(sink))
    assert torch.allclose(out[:, 0, 0], torch.tensor([1 / 2, 2 / 3, 3 / 4], dtype=torch.float64))
    assert torch.allclose(out[:, 1, 0], torch.tensor([1 / 4, 2 / 5, 3 / 6], dtype=torch.float64))


def test_capped_scores_stay_under_the_cap():
    q = torch.full((2, 1, 1), 100.0, dtype=torch.float64)
    k = torch.tensor([[[1.0]], [[-1.0]]], dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[0.0]]], dtype=torch.float64)
    out = plain.softmax_attention(q, k, v, 1.0, plain.visible(2), softcap=2.0)
    assert abs(float(out[1, 0, 0]) - 1.0 / (1.0 + math.exp(-4.0))) < 1e-9


def test_halves_are_paired_and_the_rest_passes():
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0, 0] = 1.0
    x[:, 0, 1] = 1.0
    x[:, 0, 5] = 7.0
    y = plain.rotate_half_pairs(x, 4, 100.0)
    for t in range(3):
        assert abs(float(y[t, 0, 0]) - math.cos(t)) < 1e-12 and abs(float(y[t, 0, 2]) - math.sin(t)) < 1e-12
        assert abs(float(y[t, 0, 1]) - math.cos(t * 0.1)) < 1e-12 and abs(float(y[t, 0, 3]) - math.sin(t * 0.1)) < 1e-12
        assert float(y[t, 0, 4]) == 0.0 and float(y[t, 0, 5]) == 7.0


def test_the_last_tap_is_the_current_token():
    x = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    y = plain.causal_conv(x, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64))
    assert y.flatten().tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]


def _delta_weights(width, beta_logit, a_log):
    eye = torch.eye(width, dtype=torch.float64)
    return {"m.q": eye, "m.k": eye, "m.v": eye, "m.g": eye, "m.q.conv": torch.ones(width, 1, dtype=torch.float64),
            "m.k.conv": torch.ones(width, 1, dtype=torch.float64), "m.v.conv": torch.ones(width, 1, dtype=torch.float64),
            "m.b": torch.zeros(1, width, dtype=torch.float64), "m.a": torch.zeros(1, width, dtype=torch.float64),
            "m.A_log": torch.tensor([a_log], dtype=torch.float64), "m.dt_bias": torch.tensor([0.0], dtype=torch.float64),
            "m.norm": torch.ones(width, dtype=torch.float64), "m.o": eye, "beta": beta_logit}


def test_the_delta_rule_reads_its_own_write_and_forgets_by_its_decay():
    """One head, keys along one axis: with beta = 1/2 the state moves half the way to each value; the read-out sees it."""
    d = 4
    w = _delta_weights(d, 0.0, -50.0)                    # decay exp(-exp(-50) * softplus(0)) = 1
    x = torch.zeros(3, d, dtype=torch.float64)
    x[:, 0] = 5.0                                         # q, k, v all along axis 0 (after SiLU still along axis 0)
    m = nt.right(1, 1, d, d, 1)
    out = plain.gated_delta_rule(x, w, "m", m, 0.0)
    s = float(plain.silu(torch.tensor(5.0, dtype=torch.float64)))
    # unit key e0, value s e0: S00 goes 0 -> s/2 -> 3s/4 -> 7s/8; o = S00 * (1 / sqrt(d)) along axis 0; then unit root mean
    # square over d and the gate silu(x): only the direction and sign survive the norm
    o = out[:, 0] / s
    assert torch.allclose(o, torch.full((3,), math.sqrt(d), dtype=torch.float64), atol=1e-9)
    # a fast decay wipes the state before every write: the read-out is beta * v . q each time, and the norm hides it as well;
    # compare the states' effect through a second value axis instead
    x2 = torch.zeros(2, d, dtype=torch.float64)
    x2[0, 0], x2[0, 1] = 5.0, 5.0
    x2[1, 0] = 5.0
    keep = plain.gated_delta_rule(x2, _delta_weights(d, 0.0, -50.0), "m", m, 0.0)
    wipe = plain.gated_delta_rule(x2, _delta_weights(d, 0.0, 5.0), "m", m, 0.0)
    assert float((keep[1] - wipe[1]).abs().max()) > 1e-3 and torch.allclose(keep[0], wipe[0])


def test_time_mixing_weighs_the_current_token_by_its_bonus_and_decays_the_rest():
    d = 2
    eye = torch.eye(d, dtype=torch.float64)
    w = {f"m.mu.{s}": torch.zeros(d, dtype=torch.float64) for s in "rkvgw"}
    w.update({"m.r": eye, "m.k": eye, "m.v": eye, "m.g": eye, "m.w1": torch.zeros(1, d, dtype=torch.float64),
              "m.w2": torch.zeros(d, 1, dtype=torch.float64), "m.w0": torch.full((d,), math.log(math.log(2.0)), dtype=torch.float64),
              "m.u": torch.tensor([[3.0, 3.0]], dtype=torch.float64), "m.norm": torch.ones(d, dtype=torch.float64), "m.o": eye})
    x = torch.tensor([[1.0, 0.0], [1.0, 0.0], [1.0, 0.0]], dtype=torch.float64)
    # r = k = v = e0: o_t[0] = S00 + 3 with S00 = 0, 1, 1/2 + 1; the norm and gate follow
    seen = []
    orig = plain.rms_norm
    try:
        plain.rms_norm = lambda o, g, eps: (seen.append(o.clone()), orig(o, g, eps))[1]
        plain.wkv(x, w, "m", {"heads": 1, "dim": d}, 0.0)
    finally:
        plain.rms_norm = orig
    assert torch.allclose(seen[0][:, 0, 0], torch.tensor([3.0, 4.0, 4.5], dtype=torch.float64))
    # the blend reads the previous token: with mu = 1 every reader sees only the token before
    w1 = dict(w, **{f"m.mu.{s}": torch.ones(d, dtype=torch.float64) for s in "rkvgw"})
    y = plain.wkv(torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=torch.float64), w1, "m", {"heads": 1, "dim": d}, 1e-6)
    assert float(y[0].abs().max()) == 0.0 and float(y[1, 0]) != 0.0 and float(y[1, 1]) == 0.0
