"""Torinex on the host: configuration, registry, run list, weight plan, and the plain implementation's own checks."""
import copy
import math

import pytest
import torch

import plain_torinex as P
import torinex_kit as K
from llm_infer_rust_b200 import ConfigError, resolve_architecture

ALL = dict(K.CONFIGS, blocks=K.ONLY_BLOCKS, far=K.ONLY_FAR, one=K.ONE_EXPERT)


def test_the_architecture_is_found_by_its_name_and_every_size_comes_from_the_file():
    raw = K.CONFIGS["T1"]
    arch = resolve_architecture(raw)
    assert arch.name == "Torinex"
    c = arch.parse_config(raw)
    assert (c.vocab, c.width, c.eps, c.side_dim, len(c.layers)) == (97, 40, 1e-5, 6, 4)
    a, b, d = c.layers[0], c.layers[1], c.layers[2]
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.chunk, a.rot_base, a.rot_dims, a.kv_from) == \
        (4, 2, 12, 8, 0.3, 24, 10000.0, 8, None)
    f = a.ff
    assert (f.kind, f.expert.ff, f.expert.limit, f.experts, f.top, f.groups, f.keep, f.shared.ff, f.shared.limit) == \
        ("moe", 20, 1.5, 8, 3, 4, 2, 28, 2.5)
    assert b.kv_from == 0 and b.ff.kind == "dense" and b.ff.ff == 56
    assert d.chunk is None and d.rot_dims == 0 and d.ff is None            # what the file does not mention does not exist
    g = c.layers[3].ff
    assert (g.groups, g.keep, g.shared, g.top) == (1, 1, None, 2)
    spec = arch.model_spec(c)
    assert [(e.layer, e.reads) for e in spec.run_list] == [(0, None), (1, 0), (2, None), (3, 2)]
    m0, m1, m2 = (spec.layers[i]["mixer"] for i in range(3))
    assert m0["chunk"] == 24 and m0["sink"] == "zero" and m0["qk_norm_scope"] == "projection" and m0["own_kv"]
    assert not m1["own_kv"] and m2.get("position_encoding") is None and m2["chunk"] is None
    assert "feed_forward" not in spec.layers[2].parts and "token_side" in spec.layers[2].parts
    assert spec.layers[0]["feed_forward"].kind == "routed_experts" and spec.layers[1]["feed_forward"]["activation"] == "relu_squared"
    assert spec.layers[3]["token_side"]["column"] == 18 and spec.layers[3]["token_side"]["table_width"] == 24
    assert spec.lm_head["tied"] and spec.embedding["out_dtype"] == "float32"
    assert "token_side" not in arch.model_spec(arch.parse_config(K.CONFIGS["T2"])).layers[0].parts


@pytest.mark.parametrize("change,message", [
    (lambda r: r.pop("vocab"), "vocab"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][0].update(type="mamba"), "type"),
    (lambda r: r["layers"][1]["mlp"].update(kind="experts"), "mlp.kind"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda r: r["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda r: r["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"].update(kv_from=1), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=0), "kv_from"),
    (lambda r: r["token_side"].pop("dim"), "dim"),
])
def test_a_configuration_that_lacks_or_contradicts_is_refused(change, message):
    raw = copy.deepcopy(K.CONFIGS["T1"])
    change(raw)
    with pytest.raises(ConfigError, match=message):
        resolve_architecture(raw).parse_config(raw)


@pytest.mark.parametrize("name", sorted(ALL))
def test_the_weight_plan_names_every_tensor_of_a_checkpoint_once(name):
    raw = ALL[name]
    arch = resolve_architecture(raw)
    plan = arch.weight_plan(arch.parse_config(raw))
    names = [s.name for b in plan for s in b.sources]
    assert len(names) == len(set(names))
    w = K.random_weights(raw, 1)
    assert {s.name: tuple(s.shape) for b in plan for s in b.sources} == {n: tuple(t.shape) for n, t in w.items()}
    reads = [i for i, l in enumerate(raw["layers"]) if l["mixer"].get("kv_from") is not None]
    for i in reads:                      # a layer on another's keys has no key and value tensors of its own
        assert not any(n.startswith(f"l{i}.mix.k") or n.startswith(f"l{i}.mix.v") for n in names)
    params = [b.param for b in plan]
    assert "lm_head.weight" in params and [b.alias_of for b in plan if b.param == "lm_head.weight"] == ["embedding.weight"]


# ----------------------------------------------------------------------------- the plain implementation's own checks
def test_plain_pieces_against_numbers_worked_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    assert torch.allclose(P.rms_norm(x, w, 0.0), torch.tensor([[2 * 3 / math.sqrt(12.5), 0.5 * 4 / math.sqrt(12.5)]], dtype=torch.float64))
    assert torch.allclose(P.relu_squared(torch.tensor([-2.0, 3.0])), torch.tensor([0.0, 9.0]))
    assert abs(float(P.gelu_tanh(torch.tensor(1.0, dtype=torch.float64))) - 0.8411919906082768) < 1e-12
    # a quarter turn of the pair (1, 0) at position 1 with frequency pi / 2 (base chosen so that f_0 = 1: angle = p)
    v = torch.zeros(3, 1, 4, dtype=torch.float64)
    v[:, 0, 0] = 1.0
    v[:, 0, 3] = 7.0
    r = P.rotate_pairs(v, 10.0, 2)
    assert torch.allclose(r[2, 0], torch.tensor([math.cos(2.0), math.sin(2.0), 0.0, 7.0], dtype=torch.float64))
    assert torch.equal(P.chunk_mask(5, 2), torch.tensor([[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 0, 1, 0, 0], [0, 0, 1, 1, 0],
                                                         [0, 0, 0, 0, 1]], dtype=torch.bool))
    # one key with score 0 and the sink: each takes half
    q = torch.zeros(1, 1, 2, dtype=torch.float64)
    o = P.sink_softmax_attention(q, torch.ones(1, 1, 2, dtype=torch.float64), torch.tensor([[[4.0, 8.0]]], dtype=torch.float64),
                                 1.0, P.causal_mask(1))
    assert torch.allclose(o, torch.tensor([[[2.0, 4.0]]], dtype=torch.float64))


def test_plain_routing_groups_and_weights():
    z = torch.log(torch.tensor([[0.05, 0.30, 0.10, 0.20, 0.25, 0.10]], dtype=torch.float64))
    chosen, weight = P.route(z, 2, 3, 2)          # groups (0,1) (2,3) (4,5): maxima 0.30, 0.20, 0.25: the first and the last
    assert chosen.tolist() == [[1, 4]] and torch.allclose(weight, torch.tensor([[0.30, 0.25]], dtype=torch.float64))
    chosen, weight = P.route(z, 3, 3, 1)[0], None
    assert sorted(chosen.tolist()[0][:2]) == [0, 1]
    chosen, _ = P.route(z, 3, 1, 1)
    assert chosen.tolist() == [[1, 4, 3]]
    w = {"gate": torch.tensor([[2.0]], dtype=torch.float64), "up": torch.tensor([[-3.0]], dtype=torch.float64),
         "down": torch.tensor([[1.0]], dtype=torch.float64)}
    y = P.clamped_expert(torch.tensor([[1.0]], dtype=torch.float64), w, "", 1.5)        # g = 1.5, u = -1.5
    assert abs(float(y) - 1.5 / (1 + math.exp(-1.702 * 1.5)) * (-0.5)) < 1e-12


def test_plain_model_is_causal_and_a_layer_on_anothers_keys_differs_from_one_on_its_own():
    raw = K.CONFIGS["T1"]
    w = K.random_weights(raw, 3)
    ids = K.tokens(raw["vocab"], 40, 2)
    full = K.oracle(raw, w, ids)
    assert abs(full[:25] - K.oracle(raw, w, ids[:25])).max() < 1e-9
    other = copy.deepcopy(raw)
    other["layers"][1]["mixer"].pop("kv_from")
    w2 = dict(K.random_weights(other, 3))
    w2.update({n: t for n, t in w.items() if n in w2 and t.shape == w2[n].shape})
    assert abs(full - K.oracle(other, w2, ids)).max() > 1e-3
