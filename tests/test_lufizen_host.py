"""Lufizen on the host: configuration, registry, weight plan, frequencies, and the plain implementation's own checks."""
import copy
import math

import pytest
import torch

import lufizen_kit as K
import plain_lufizen as P
from llm_infer_rust_b200 import ConfigError, resolve_architecture

ALL = dict(K.CONFIGS, attention=K.ONLY_ATTENTION, latent=K.ONLY_LATENT, one=K.ONE_EXPERT)


def test_the_architecture_is_found_by_its_name_and_every_size_comes_from_the_file():
    raw = K.CONFIGS["L1"]
    arch = resolve_architecture(raw)
    assert arch.name == "Lufizen"
    c = arch.parse_config(raw)
    assert (c.vocab, c.width, c.eps, c.embedding_scale, c.logit_scale, len(c.layers)) == (97, 40, 1e-5, 2.0, 0.5, 4)
    a, b, d = c.layers[0], c.layers[1], c.layers[2]
    assert (a.kind, a.heads, a.kv_heads, a.dim, a.vdim, a.scale) == ("attention", 4, 2, 12, 12, 0.3)
    assert (a.rot.base, a.rot.dims, a.rot.scaling) == (300.0, 8, (8.0, 1.0, 4.0, 64.0))
    f = a.ff
    assert (f.ff, f.experts, f.top, f.scale, f.groups, f.keep, f.shared_ff) == (20, 8, 3, 2.0, 4, 2, 28)
    assert (b.kind, b.heads, b.dim, b.rot_dim, b.vdim, b.kv_rank, b.q_rank, b.rot.dims, b.rot.scaling) == \
        ("latent_attention", 3, 10, 4, 14, 24, 18, 4, None)
    assert (b.ff.groups, b.ff.keep, b.ff.shared_ff) == (1, 1, 0)
    assert d.rot is None and d.ff is None                  # what the file does not mention does not exist
    import copy
    bare = copy.deepcopy(raw)
    bare["layers"][2]["mixer"].pop("vdim")                 # an attention layer's values are as wide as its keys
    assert arch.parse_config(bare).layers[2].vdim == 10
    spec = arch.model_spec(c)
    assert [(e.layer, e.reads) for e in spec.run_list] == [(0, None), (1, None), (2, None), (3, None)]
    m0, m1, m2 = (spec.layers[i]["mixer"] for i in range(3))
    assert m0.kind == "grouped_attention" and m0["values_from_keys"] and not m0["qk_norm_weight"]
    assert m0["qk_norm_order"] == "after_rotation" and m0["sink"] is True and m0["softmax_scale"] == 0.3
    assert spec.position_encodings[m0["position_encoding"]]["pairing"] == "half_split"
    assert spec.position_encodings[m0["position_encoding"]]["wavelength_scaling"]["original"] == 64.0
    assert m1.kind == "latent_attention" and m1["gate"] == "head" and m1["q_rank"] == 18 and not m1.get("sink")
    assert spec.position_encodings[m1["position_encoding"]]["pairing"] == "interleaved"
    assert m2.get("position_encoding") is None
    assert "feed_forward" not in spec.layers[2].parts and "ff_norm" not in spec.layers[2].parts
    ff = spec.layers[0]["feed_forward"]
    assert (ff.kind, ff["scores"], ff["correction"], ff["group_members"], ff["weight_scale"], ff["shared_gated"]) == \
        ("routed_experts", "sigmoid", True, 2, 2.0, True)
    assert not spec.layers[1]["feed_forward"]["shared_gated"]
    assert spec.layers[0].block.kind == "post_norm_stream"
    assert spec.embedding["scale"] == 2.0 and spec.embedding["out_dtype"] == "float32"
    assert spec.lm_head["logit_scale"] == 0.5 and not spec.lm_head["tied"]


@pytest.mark.parametrize("change,message", [
    (lambda r: r.pop("vocab"), "vocab"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r.pop("embedding"), "embedding"),
    (lambda r: r.pop("logit_scale"), "logit_scale"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][0]["mixer"].update(vdim=10), "vdim"),
    (lambda r: r["layers"][0].update(type="mamba"), "type"),
    (lambda r: r["layers"][0]["mlp"].update(kind="dense"), "mlp.kind"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda r: r["layers"][0]["mlp"]["router"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda r: r["layers"][0]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"]["rot"]["scaling"].pop("original"), "original"),
    (lambda r: r["layers"][0]["mixer"]["rot"]["scaling"].update(high=1.0), "high"),
    (lambda r: r["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda r: r["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=2), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"].pop("rot"), "rot"),
])
def test_a_configuration_that_lacks_or_contradicts_is_refused(change, message):
    raw = copy.deepcopy(K.CONFIGS["L1"])
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
    assert not any(".mix.v" in n for n in names if not n.endswith(".mix.uv"))       # the design has no value projection
    assert "lm_head.weight" in [b.param for b in plan]


def test_the_random_writer_makes_a_folder_that_the_plan_reads(tmp_path):
    from llm_infer_rust_b200 import random_tensors, write_random_model
    raw = K.CONFIGS["L2"]
    folder = write_random_model(str(tmp_path), raw, seed=3, std=0.1, dtype="bfloat16")
    drawn = random_tensors(raw, 3, std=0.1, dtype="bfloat16")
    w = K.random_weights(raw, 1)
    assert {n: tuple(t.shape) for n, t in drawn.items()} == {n: tuple(t.shape) for n, t in w.items()}
    assert folder


# ----------------------------------------------------------------------------- stretched frequencies (the product's part)
@pytest.mark.parametrize("rot", [
    {"base": 300.0, "dims": 8, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}},
    {"base": 10000.0, "dims": 64, "scaling": {"factor": 32.0, "low": 1.0, "high": 4.0, "original": 8192}},
    {"base": 77.0, "dims": 2, "scaling": {"factor": 2.0, "low": 1.0, "high": 3.0, "original": 32}},
    {"base": 500000.0, "dims": 30, "scaling": {"factor": 3.0, "low": 2.0, "high": 16.0, "original": 1000}},
    {"base": 5000.0, "dims": 16},
])
def test_frequencies_stretched_by_wavelength(rot):
    from llm_infer_rust_b200.config.spec import PartSpec
    from llm_infer_rust_b200.parts.base import BuildEnv
    from llm_infer_rust_b200.parts.position import RotaryFrequencies
    params = {"rotary_dim": rot["dims"], "theta": rot["base"], "pairing": "half_split"}
    if rot.get("scaling"):
        params["wavelength_scaling"] = rot["scaling"]
    part = RotaryFrequencies(PartSpec("rotary_frequencies", params), BuildEnv(torch.float32, torch.device("cpu"), {}))
    want = P.frequencies(rot)
    assert part.inv_freq.dtype == torch.float32 and part.inv_freq.shape == want.shape
    assert ((part.inv_freq.double() - want).abs() / want).max() < 1e-7


def test_the_three_ranges_of_the_stretch_by_hand():
    rot = {"base": 100.0, "dims": 6, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 40}}
    f = P.frequencies(rot).tolist()
    plain = [100.0 ** (-2 * i / 6) for i in range(3)]         # wavelengths 6.28, 29.2, 135.4; the band is 10 .. 40
    assert abs(f[0] - plain[0]) < 1e-15
    s = (40 / (2 * math.pi / plain[1]) - 1.0) / 3.0
    assert abs(f[1] - ((1 - s) * plain[1] / 4 + s * plain[1])) < 1e-15 and 0 < s < 1
    assert abs(f[2] - plain[2] / 4) < 1e-15


# ----------------------------------------------------------------------------- the plain implementation's own checks
def test_plain_pieces_against_numbers_worked_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    assert torch.allclose(P.rms_norm(x, w, 0.0), torch.tensor([[2 * 3 / math.sqrt(12.5), 0.5 * 4 / math.sqrt(12.5)]], dtype=torch.float64))
    assert torch.allclose(P.rms_norm(x, None, 0.0), torch.tensor([[3 / math.sqrt(12.5), 4 / math.sqrt(12.5)]], dtype=torch.float64))
    assert abs(float(P.silu(torch.tensor(2.0, dtype=torch.float64))) - 2.0 / (1 + math.exp(-2.0))) < 1e-15
    # position 2 with frequency 1: the pair (1, 0) turns to (cos 2, sin 2), in both layouts; a fifth coordinate passes
    f = torch.tensor([1.0, 0.5], dtype=torch.float64)
    v = torch.zeros(3, 1, 5, dtype=torch.float64)
    v[:, 0, 0] = 1.0
    v[:, 0, 4] = 7.0
    half = P.rotate(v, f, "half")[2, 0]
    assert torch.allclose(half, torch.tensor([math.cos(2.0), 0.0, math.sin(2.0), 0.0, 7.0], dtype=torch.float64))
    inter = P.rotate(v, f, "interleaved")[2, 0]
    assert torch.allclose(inter, torch.tensor([math.cos(2.0), math.sin(2.0), 0.0, 0.0, 7.0], dtype=torch.float64))
    # one key with score 0 and a sink of 0: each takes half; a sink of log 3: the key keeps a quarter; no sink: all
    q = torch.zeros(1, 1, 2, dtype=torch.float64)
    k, val = torch.ones(1, 1, 2, dtype=torch.float64), torch.tensor([[[4.0, 8.0]]], dtype=torch.float64)
    for sink, share in ((torch.tensor([0.0]), 0.5), (torch.tensor([math.log(3.0)]), 0.25), (None, 1.0)):
        o = P.softmax_attention(q, k, val, 1.0, P.causal_mask(1), sink)
        assert torch.allclose(o, val * share)


def test_plain_routing_correction_groups_and_weights():
    logit = lambda p: math.log(p / (1 - p))
    s = [0.50, 0.10, 0.30, 0.35, 0.45, 0.05]                      # groups (0,1) (2,3) (4,5)
    z = torch.tensor([[logit(p) for p in s]], dtype=torch.float64)
    none = torch.zeros(6, dtype=torch.float64)
    # sums of two: 0.60, 0.65, 0.50: the middle group wins although the best single expert is in the first
    chosen, weight = P.route(z, none, 2, 3, 1, 2.0)
    assert chosen.tolist() == [[3, 2]] and torch.allclose(weight, torch.tensor([[0.70, 0.60]], dtype=torch.float64))
    # two groups kept: the first two; the best three of their four members
    chosen, weight = P.route(z, none, 3, 3, 2, 1.0)
    assert chosen.tolist() == [[0, 3, 2]]
    # the correction moves the choice, not the weight: expert 5 is lifted over everything
    corr = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 1.0], dtype=torch.float64)
    chosen, weight = P.route(z, corr, 2, 3, 1, 1.0)               # sums 0.60, 0.65, 1.50
    assert chosen.tolist() == [[5, 4]] and torch.allclose(weight, torch.tensor([[0.05, 0.45]], dtype=torch.float64))
    # choice scores below zero: a shut group stays shut although its members' scores (near 0) beat the open ones'
    corr = torch.tensor([-3.0, -3.0, -2.0, -2.0, -5.0, -5.0], dtype=torch.float64)
    chosen, _ = P.route(z, corr, 2, 3, 1, 1.0)
    assert sorted(chosen.tolist()[0]) == [2, 3]
    # without groups every expert is open
    chosen, _ = P.route(z, none, 3, 1, 1, 1.0)
    assert chosen.tolist() == [[0, 4, 3]]
    assert P.route_margin(z, none, 2, 3, 1).item() == pytest.approx(0.05)
    w = {"gate": torch.tensor([[2.0]], dtype=torch.float64), "up": torch.tensor([[-3.0]], dtype=torch.float64),
         "down": torch.tensor([[0.5]], dtype=torch.float64)}
    y = P.expert(torch.tensor([[1.0]], dtype=torch.float64), w, "")
    assert abs(float(y) - 0.5 * (2.0 / (1 + math.exp(-2.0))) * -3.0) < 1e-12


def test_plain_model_is_causal_and_its_mechanisms_show():
    raw = K.CONFIGS["L1"]
    w = K.random_weights(raw, 3)
    ids = K.tokens(raw["vocab"], 40, 2)
    full = K.oracle(raw, w, ids)
    assert abs(full[:25] - K.oracle(raw, w, ids[:25])).max() < 1e-9
    for name, change in (("l0.mix.sink", 3.0), ("l0.mlp.correction", 0.7), ("l0.mlp.shared.sg", 0.5), ("l1.mix.g", 0.5),
                         ("l1.mix.dq.norm", 0.5)):
        w2 = dict(w)
        # the same shift for every expert would leave the choice alone: every second entry is moved
        w2[name] = w[name] + change * (torch.arange(w[name].numel()).reshape(w[name].shape) % 2)
        assert abs(full - K.oracle(raw, w2, ids)).max() > 1e-3, name
    assert abs(full - K.oracle(dict(raw, logit_scale=1.0), w, ids)).max() > 1e-3
    assert abs(full - K.oracle(dict(raw, embedding={"scale": 1.0}), w, ids)).max() > 1e-3
