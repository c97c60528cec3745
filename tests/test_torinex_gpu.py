"""Torinex through the engine against the plain implementation (``plain_torinex.py``), in float32 and bfloat16.

Mechanisms alone (kernels against the plain functions, and one-layer models), whole prompts against token-by-token
decoding, portions down to two tokens, batches of unequal requests against each alone, pages and slots that are freed
and used again, keys that stand out just inside and just outside a block's edge, the sink, far keys, long decoding,
greedy generation through the scheduler, and trace replay through ``bin/trace_run``.
"""
import math

import numpy as np
import pytest
import torch

import plain_torinex as P
import torinex_kit as K

pytestmark = pytest.mark.gpu

PORTIONS = [2, 37, 3, 16, 64, 5, 1, 22]


def cut(total, sizes):
    out, k = [], 0
    while total > 0:
        n = min(total, sizes[k % len(sizes)])
        out.append(n)
        total -= n
        k += 1
    return out


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, weights, folder stored in bfloat16)."""
    out = {}
    named = dict(K.CONFIGS, blocks=K.ONLY_BLOCKS, far=K.ONLY_FAR, one=K.ONE_EXPERT)
    for i, (name, raw) in enumerate(named.items()):
        w = K.random_weights(raw, 500 + i)
        out[name] = (raw, w, K.write_model(str(tmp_path_factory.mktemp("torinex_" + name)), raw, w))
    return out


def _i32(x, dev="cuda"):
    return torch.tensor(x, dtype=torch.int32, device=dev)


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("y_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [44, 264, 13000])
def test_norm_on_the_output_added_into_the_stream(width, y_dtype):
    """x <- x + N(y + bias) in place on a float32 stream, with the rounded copy for the next product; then the plain
    norm of chosen rows (the model's last norm)."""
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(width)
    T, eps = 7, 1e-5
    x = torch.randn(T, width, generator=g) * 3
    y = (torch.randn(T, width, generator=g) * 5).to(y_dtype)
    bias, w = torch.randn(width, generator=g), 1.0 + 0.3 * torch.randn(width, generator=g)
    for b in (None, bias):
        want = x.double() + P.rms_norm(y.double() + (0 if b is None else b.double()), w.double(), eps)
        stream = x.to(dev).clone()
        for cast_to in (torch.bfloat16, torch.float32, None):
            stream.copy_(x)
            got = ops.norm_add(stream, y.to(dev), w.to(dev), eps, bias=None if b is None else b.to(dev), cast_to=cast_to)
            torch.testing.assert_close(stream.cpu().double(), want, rtol=1e-5, atol=1e-5)
            if cast_to is torch.bfloat16:
                assert torch.equal(got, stream.to(torch.bfloat16))
            elif cast_to is torch.float32:
                assert got.data_ptr() == stream.data_ptr()
            else:
                assert got is None
    rows = _i32([5, 0, 5, 2])
    for out_dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        got = ops.norm_rows(x.to(dev), w.to(dev), eps, out_dtype, rows=rows)
        torch.testing.assert_close(got.cpu().double(), P.rms_norm(x.double(), w.double(), eps)[[5, 0, 5, 2]], rtol=tol, atol=tol)
        assert ops.norm_rows(x.to(dev), w.to(dev), eps, out_dtype).shape == (T, width)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,rot,interleaved", [(4, 2, 12, 8, 8, True), (3, 3, 16, 16, 16, True), (6, 1, 10, 14, 0, True),
                                                      (2, 1, 160, 136, 30, True), (5, 1, 8, 8, 4, False)])
def test_norm_over_the_whole_projection_rotation_and_cache_store(H, G, d, dv, rot, interleaved, dtype):
    """Bias, ONE norm over all of q's columns and one over all of k's, the rotation of a part of every head, q out and
    k, v into scrambled cache slots; and the same for a layer that has q alone."""
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(H * 100 + d)
    T, page, eps, base = 21, 4, 1e-5, 1000.0
    nq, nk, nv = H * d, G * d, G * dv
    packed = K.bf16_values(torch.randn(T, nq + nk + nv + 5, generator=g) * 2)          # columns behind v are ignored
    bias = torch.randn(nq + nk + nv, generator=g)
    qw, kw = 1 + 0.3 * torch.randn(nq, generator=g), 1 + 0.3 * torch.randn(nk, generator=g)
    positions = torch.randint(0, 3000, (T,), generator=g)
    inv_freq = torch.pow(torch.tensor(base, dtype=torch.float64), -torch.arange(0, max(rot, 2), 2, dtype=torch.float64) / max(rot, 2)).float()

    def rotated(x, heads):
        x = x.reshape(T, heads, d)
        if not rot:
            return x
        out = x.clone()
        for t in range(T):
            if interleaved:
                out[t:t + 1] = P.rotate_pairs(x[t:t + 1], base, rot, first_position=int(positions[t]), angle_dtype=torch.float32)
            else:                                           # pairs (i, i + rot / 2): the plain function on reordered columns
                order = [c for i in range(rot // 2) for c in (i, i + rot // 2)]
                turned = P.rotate_pairs(x[t:t + 1][..., order], base, rot, first_position=int(positions[t]),
                                            angle_dtype=torch.float32)
                out[t:t + 1, :, order] = turned
        return out

    pd = packed.double()
    want_q = rotated(P.rms_norm(pd[:, :nq] + bias[:nq].double(), qw.double(), eps), H)
    want_k = rotated(P.rms_norm(pd[:, nq:nq + nk] + bias[nq:nq + nk].double(), kw.double(), eps), G)
    want_v = (pd[:, nq + nk:nq + nk + nv] + bias[nq + nk:].double()).reshape(T, G, dv)
    pages = -(-T // page)
    slots = torch.randperm(pages * page, generator=g)[:T] + page                   # page 0 is never written
    k_cache = torch.full((pages + 1, G, page, d), 9.0, device=dev, dtype=dtype)
    v_cache = torch.full((pages + 1, G, page, dv), 9.0, device=dev, dtype=dtype)
    q = torch.empty((T, nq), device=dev, dtype=dtype)
    kw_args = dict(bias=bias.to(dev), q_weight=qw.to(dev), k_weight=kw.to(dev), eps=eps,
                   inv_freq=inv_freq.to(dev) if rot else None, rot_dims=rot, interleaved=interleaved)
    ops.joint_heads_prepare(packed.to(dev, dtype), q, k_cache, v_cache, _i32(positions.tolist()), _i32(slots.tolist()),
                            H, G, d, dv, **kw_args)
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(q.cpu().double().reshape(T, H, d), want_q, rtol=tol, atol=tol)
    for t in range(T):
        pg, off = int(slots[t]) // page, int(slots[t]) % page
        torch.testing.assert_close(k_cache[pg, :, off].cpu().double(), want_k[t], rtol=tol, atol=tol)
        torch.testing.assert_close(v_cache[pg, :, off].cpu().double(), want_v[t], rtol=tol, atol=tol)
    assert float(k_cache[0].min()) == 9.0 and float(v_cache[0].max()) == 9.0
    # q alone: nothing is stored
    before = k_cache.clone()
    q2 = torch.empty_like(q)
    kw_args.update(bias=bias[:nq].to(dev).contiguous(), k_weight=None)
    ops.joint_heads_prepare(packed[:, :nq].to(dev, dtype).contiguous(), q2, None, None, _i32(positions.tolist()), None,
                            H, G, d, dv, has_kv=False, **kw_args)
    torch.testing.assert_close(q2.cpu().double().reshape(T, H, d), want_q, rtol=tol, atol=tol)
    assert torch.equal(before, k_cache)
    ops.check_errors(dev)


@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,width,experts,top,groups,keep", [(1, 40, 8, 3, 4, 2), (19, 44, 15, 4, 5, 2), (70, 64, 5, 2, 1, 1),
                                                                  (9, 33, 6, 6, 1, 1), (130, 72, 64, 8, 8, 4), (40, 36, 6, 1, 6, 1)])
def test_router_softmax_groups_and_top_experts(tokens, width, experts, top, groups, keep, x_dtype):
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(tokens + experts)
    x = K.bf16_values(torch.randn(tokens, width, generator=g))
    w = K.bf16_values(torch.randn(experts, width, generator=g) * 3.0 * width ** -0.5)
    chosen, weight = P.route(x.double() @ w.double().T, top, groups, keep)
    for w_dtype in (torch.float32, torch.bfloat16):
        choice, gains = ops.expert_router(x.to(dev, x_dtype), w.to(dev, w_dtype), top, groups, keep)
        assert torch.equal(choice.cpu().long(), chosen), "the chosen experts, best first"
        torch.testing.assert_close(gains.cpu().double(), weight, rtol=2e-5, atol=1e-7)
    # the other forms of the part: a sigmoid of every logit, the chosen weights divided by their sum
    z = x.double() @ w.double().T
    s = torch.sigmoid(z)
    per = experts // groups
    best = s.reshape(tokens, groups, per).max(-1).values.topk(keep, -1).indices
    allowed = torch.zeros(tokens, groups, dtype=torch.bool).scatter_(1, best, True).repeat_interleave(per, 1)
    picked = s.masked_fill(~allowed, -1.0).topk(top, -1).indices
    choice, gains = ops.expert_router(x.to(dev, x_dtype), w.to(dev), top, groups, keep, scores="sigmoid", renormalize=True)
    assert torch.equal(choice.cpu().long(), picked)
    torch.testing.assert_close(gains.cpu().double(), s.gather(1, picked) / s.gather(1, picked).sum(-1, keepdim=True),
                               rtol=2e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,width,ff,experts,top", [(1, 40, 24, 5, 2), (70, 44, 20, 4, 1), (300, 64, 48, 3, 3),
                                                         (130, 248, 88, 12, 4), (700, 184, 136, 9, 2)])
def test_routed_experts_with_clamped_gates_weights_and_a_shared_share(tokens, width, ff, experts, top, dtype):
    """Few and many pairs (the second take the tcgen05 products in bfloat16), experts with many, few and no tokens,
    gates and ups beyond the limit, a weight for every pair, what every token gets besides added in float."""
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(tokens + top)
    limit = 1.25
    w = {}
    for e in range(experts):
        w[f"e{e}.gate"] = K.bf16_values(torch.randn(ff, width, generator=g) * 1.5 * width ** -0.5)
        w[f"e{e}.up"] = K.bf16_values(torch.randn(ff, width, generator=g) * 1.5 * width ** -0.5)
        w[f"e{e}.down"] = K.bf16_values(torch.randn(width, ff, generator=g) * ff ** -0.5)
    choice = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(tokens)])
    choice[: min(tokens, 40)] = choice[0]                          # many tokens on the same experts, others on few
    gains = torch.rand(tokens, top, generator=g)
    x = K.bf16_values(torch.randn(tokens, width, generator=g))
    add = K.bf16_values(torch.randn(tokens, width, generator=g))
    wd = {n: t.double() for n, t in w.items()}
    want = add.double().clone()
    for t in range(tokens):
        for e, s in zip(choice[t].tolist(), gains[t].double()):
            want[t] += s * P.clamped_expert(x[t:t + 1].double(), wd, f"e{e}.", limit)[0]
    gate_up = torch.cat([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(experts)]).view(experts, 2 * ff, width)
    down = torch.cat([w[f"e{e}.down"] for e in range(experts)]).view(experts, width, ff)
    args = (x.to(dev, dtype), choice.to(dev, torch.int32), gains.to(dev), gate_up.to(dev, dtype).contiguous(),
            down.to(dev, dtype).contiguous(), "clamped_swish", limit, 1.702)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for a in (add.to(dev, dtype), add.to(dev)):                    # the share in the engine's dtype and in float32
        got = ops.routed_experts(*args, add=a)
        assert got.dtype == torch.float32
        torch.testing.assert_close(got.cpu().double(), want, rtol=tol, atol=tol)
    got = ops.routed_experts(*args)
    torch.testing.assert_close(got.cpu().double(), want - add.double(), rtol=tol, atol=tol)
    if dtype == torch.bfloat16 and width % 8 == 0 and ff % 8 == 0 and tokens * top >= 128:
        for tensor_memory in (True, False):                        # both kinds of product on the same step
            again = ops.routed_experts(*args, add=add.to(dev), tensor_memory=tensor_memory)
            torch.testing.assert_close(again.cpu().double(), want, rtol=tol, atol=tol)
    ops.check_errors(dev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [70, 72])
def test_activations_gates_bias_and_the_token_table(dtype, width):
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(width)
    T = 11
    z = K.bf16_values(torch.randn(T, width, generator=g) * 3)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    got = ops.activate(z.to(dev, dtype), "relu_squared")
    torch.testing.assert_close(got.cpu().double(), P.relu_squared(z.double()), rtol=tol, atol=tol)
    gu = K.bf16_values(torch.randn(T, 2 * width, generator=g) * 3)
    gate, up = gu[:, :width].double(), gu[:, width:].double()
    for limit in (0.75, 7.0):
        gc, uc = torch.clamp(gate, max=limit), torch.clamp(up, -limit, limit)
        want = gc * P.sigmoid(1.702 * gc) * (uc + 1.0)
        got = ops.glu_columns(gu.to(dev, dtype), "clamped_swish", limit, 1.702)
        torch.testing.assert_close(got.cpu().double(), want, rtol=tol, atol=tol * 8)
    got = ops.glu_columns(gu.to(dev, dtype), "silu")
    torch.testing.assert_close(got.cpu().double(), gate * P.sigmoid(gate) * up, rtol=tol, atol=tol * 8)
    bias = torch.randn(width, generator=g)
    got = ops.add_row_bias(z.to(dev, dtype).clone(), bias.to(dev))
    torch.testing.assert_close(got.cpu().double(), z.double() + bias.double(), rtol=tol, atol=tol)
    vocab, columns, column = 23, width + 9, 4
    table = K.bf16_values(torch.randn(vocab, columns + width, generator=g))
    ids = torch.randint(0, vocab, (T,), generator=g)
    got = ops.act_table_mul(z.to(dev, dtype), "gelu_tanh", table.to(dev, dtype), _i32(ids.tolist()), column)
    want = P.gelu_tanh(z.double()) * table.double()[ids][:, column:column + width]
    torch.testing.assert_close(got.cpu().double(), want, rtol=tol, atol=tol * 4)
    ops.check_errors(dev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,width,dim,layer", [(1, 40, 6, 2), (7, 264, 16, 0), (16, 72, 1, 3), (3, 1032, 24, 1)])
def test_token_table_read_of_a_few_tokens_in_one_kernel(tokens, width, dim, layer, dtype):
    """The gated read of the layer's columns of the second table, normed and added into the float stream, for a step
    of few tokens (one kernel) against the plain function; the rounded copy is the new stream rounded once."""
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(width + dim)
    vocab, layers, eps = 37, 4, 1e-5
    w = {"side.embed": K.bf16_values(torch.randn(vocab, layers * dim, generator=g)),
         "s.side.gate": K.bf16_values(torch.randn(dim, width, generator=g) * width ** -0.5),
         "s.side.proj": K.bf16_values(torch.randn(width, dim, generator=g)),
         "s.side.norm": 0.7 + 0.3 * torch.randn(width, generator=g)}
    ids = torch.randint(0, vocab, (tokens,), generator=g).tolist()
    stream = torch.randn(tokens, width, generator=g) * 2
    x = K.bf16_values(stream) if dtype == torch.bfloat16 else stream
    want = stream.double() + P.token_side(x.double(), ids, {n: t.double() for n, t in w.items()}, "s.", layer, dim, eps)
    s_dev = stream.to(dev).clone()
    x_dev = s_dev if dtype == torch.float32 else x.to(dev, dtype)
    got = ops.token_side_few(s_dev, x_dev, w["s.side.gate"].to(dev, dtype), w["side.embed"].to(dev, dtype), _i32(ids),
                             layer * dim, w["s.side.proj"].to(dev, dtype), w["s.side.norm"].to(dev), eps, "gelu_tanh",
                             cast_to=dtype)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    torch.testing.assert_close(s_dev.cpu().double(), want, rtol=tol, atol=tol)
    assert torch.equal(got, s_dev.to(dtype))
    ops.check_errors(dev)


def _attend_in_portions(q, k, v, portions, dtype, chunk, scale, page=8):
    """q [T, H, d], k [T, G, d], v [T, G, dv] stored in pages handed out in a scrambled order and read by the attention
    kernels portion by portion, with the sink of score 0; the outputs [T, H, dv]."""
    from llm_infer_rust_b200.kernels import ops
    dev = torch.device("cuda")
    T, H, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    pages = -(-T // page)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(7)) + 1
    k_cache = torch.full((pages + 1, G, page, d), 55.0, device=dev, dtype=dtype)        # stale values everywhere
    v_cache = torch.full((pages + 1, G, page, dv), 55.0, device=dev, dtype=dtype)
    table = order.to(torch.int32).reshape(1, -1).to(dev)
    sinks = torch.zeros(H, device=dev)
    out, at = [], 0
    for n in portions:
        for p_ in range(at, at + n):
            k_cache[int(order[p_ // page]), :, p_ % page] = k[p_].to(dev, dtype)
            v_cache[int(order[p_ // page]), :, p_ % page] = v[p_].to(dev, dtype)
        qo = q[at:at + n].reshape(n, -1).to(dev, dtype).contiguous()
        o = torch.empty((n, H * dv), device=dev, dtype=dtype)
        args = (table, _i32([0, n]), _i32([at + n]))
        if n > 1:
            ops.prefill_attention(qo, k_cache, v_cache, o, *args, _i32([at]), _i32([0]), 1, n, H, G, d, page, None,
                                  scale, v_head_dim=dv, precise_weights=True, chunk=chunk, sinks=sinks)
        else:
            splits = 1 if at <= 40 else (2 if at <= 80 else 3)      # one CTA, a cluster of two, parts merged by a kernel
            need = ops.decode_scratch_floats(1, H, max(d, dv), splits)
            scratch = torch.empty(max(need, 1), device=dev)
            ops.decode_attention(qo, k_cache, v_cache, o, scratch, *args, _i32([0]), 1, H, G, d, page, None, scale,
                                 splits, v_head_dim=dv, precise_weights=True, chunk=chunk, sinks=sinks)
        out.append(o.cpu().float().reshape(n, H, dv))
        at += n
    ops.check_errors(dev)
    return torch.cat(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("size", [24, 5, 8, 1, None])
@pytest.mark.parametrize("d,dv,H,G", [(12, 14, 4, 2), (32, 32, 8, 1), (64, 64, 2, 2)])
def test_keys_at_a_blocks_edges_the_first_key_and_the_sink(size, d, dv, H, G, dtype):
    """For chosen queries, in prompt portions and decoded alone, the key just OUTSIDE the block is made to fit the
    query far better than any other (it would take all the weight if it were seen), and for others the block's first
    key, or the very first key of the sequence; for others every key fits so badly that the sink takes the weight."""
    g = torch.Generator().manual_seed((size or 0) + d)
    T = 100
    q = K.bf16_values(torch.randn(T, H, d, generator=g))
    k = K.bf16_values(torch.randn(T, G, d, generator=g))
    v = K.bf16_values(torch.randn(T, G, dv, generator=g))
    portions = [30, 2, 9, 1, 1, 1, 20, 1, 1, 17] + [1] * 17
    assert sum(portions) == T
    for i in (25, 31, 41, 42, 43, 55, 63, 64, 70, 83, 90, 99):                # in portions and decoded alone
        edge = (i - i % size - 1) if size else 0                              # the last key that is NOT seen
        for j, boost in ((edge, 6.0), (edge + 1, 4.0), (0, 3.0)):
            if 0 <= j <= i:
                k[j, :, :] = K.bf16_values(boost * q[i, 0:1, :] / q[i, 0].norm() * 2.0)
    for i in (28, 44, 77, 95):                                               # nothing fits: the sink decides
        q[i] = K.bf16_values(-4.0 * k[max(0, i - 3):i + 1].mean((0, 1)) - 3.0 * k[i, 0])
    visible = P.chunk_mask(T, size) if size else P.causal_mask(T)
    rep = H // G
    want = P.sink_softmax_attention(q.double(), k.double().repeat_interleave(rep, 1), v.double().repeat_interleave(rep, 1),
                                    0.7, visible)
    got = _attend_in_portions(q, k, v, portions, dtype, size, 0.7)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    torch.testing.assert_close(got.double(), want, rtol=tol, atol=tol)
    # the sink is not a rounding matter: without it the same rows come out far away
    assert (want.abs().sum(-1) < 0.5 * v.double().abs().sum(-1).mean()).any()


# ----------------------------------------------------------------------------- models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["T1", "T2", "T3", "blocks", "far", "one"])
def test_whole_decoded_and_in_portions(name, dtype, models):
    if name == "one" and dtype == "bfloat16":
        pytest.skip("one expert a token: a near tie between two experts shows in full; compared in float32")
    raw, w, folder = models[name]
    T = 150
    ids = K.tokens(raw["vocab"], T, 3)
    want, close = K.oracle_and_close_calls(raw, w, ids)
    eng = K.make_engine(folder, dtype, page_size=8, pool_tokens=256)
    tol = K.tolerance(name, dtype)
    K.check_clear(K.run_alone(eng, 1, ids, [T]), want, close, dtype, "whole", tol)
    K.check_clear(K.run_alone(eng, 2, ids, [T - 40] + [1] * 40), want, close, dtype, "last 40 decoded", tol)
    K.check_clear(K.run_alone(eng, 3, ids, cut(T, PORTIONS)), want, close, dtype, "in portions", tol)
    K.check_clear(K.run_alone(eng, 4, ids[:24], [1] * 24), want[:24], close[:24], dtype, "token by token from the first", tol)
    K.check_clear(K.run_alone(eng, 5, ids[:61], [2] * 30 + [1]), want[:61], close[:61], dtype, "two tokens at a time", tol)
    assert eng.cache.manager.check() == ""


@pytest.mark.parametrize("dim,vdim,heads,kv", [(24, 24, 3, 1), (80, 80, 4, 2), (96, 96, 2, 1), (128, 128, 4, 2),
                                               (256, 256, 2, 1), (128, 64, 2, 2)])
def test_head_sizes_of_every_kernel_family(dim, vdim, heads, kv, tmp_path):
    """Head sizes beyond the fixed configurations': multiples of 16 up to 256 (tensor-core kernels in bfloat16), one
    that is none, and values narrower than keys; two layers, the second on the first one's keys, whole, decoded and in
    portions."""
    raw = K.config(83, 64, 1e-5, [
        K.attention(heads, kv, dim, vdim, dim ** -0.5, 40, (10000.0, dim - 8), mlp=K.dense(48)),
        K.attention(heads, kv, dim, vdim, 0.9 * dim ** -0.5, 23, (10000.0, dim - 8), kv_from=0)], side=4)
    T = 130
    ids = K.tokens(raw["vocab"], T, dim)
    w = K.random_weights(raw, 900 + dim)
    folder = K.write_model(str(tmp_path / "m"), raw, w)
    want, close = K.oracle_and_close_calls(raw, w, ids)
    for dtype in ("float32", "bfloat16"):
        eng = K.make_engine(folder, dtype, page_size=16, pool_tokens=256)
        K.check_clear(K.run_alone(eng, 1, ids, [T]), want, close, dtype, "whole")
        K.check_clear(K.run_alone(eng, 2, ids, [T - 50] + [1] * 50), want, close, dtype, "last 50 decoded")
        K.check_clear(K.run_alone(eng, 3, ids, cut(T, [33, 2, 64, 7])), want, close, dtype, "in portions")
        eng.check_kernel_errors()
        del eng


def test_every_layer_against_the_plain_stream(models):
    """The float32 stream after every layer, whole and cut into portions."""
    from llm_infer_rust_b200.engine import StepEntry
    raw, w, folder = models["T1"]
    ids = K.tokens(raw["vocab"], 60, 5)
    layers = []
    P.forward(raw, w, ids, dtype=torch.float64, layers_out=layers)
    eng = K.make_engine(folder, "float32", page_size=8, pool_tokens=128)
    caught = []
    for block in eng.model.blocks:
        def wrapped(h, residual, ctx, cache, inner=block.forward):
            out = inner(h, residual, ctx, cache)
            caught.append(out[0].detach().cpu().double().clone())
            return out
        block.forward = wrapped
    eng.open_request(1)
    for lo, hi in ((0, 33), (33, 35), (35, 60)):
        eng.step([StepEntry(1, ids[lo:hi], [])])
    n = len(raw["layers"])
    for i in range(n):
        got = torch.cat([caught[s * n + i] for s in range(3)])
        torch.testing.assert_close(got, layers[i], rtol=3e-5, atol=3e-5, msg=lambda m, i=i: f"layer {i}: {m}")


def drawn_config(seed):
    """A configuration whose every size, option and layer order is drawn: any model of the design must run as it is."""
    import random
    rng = random.Random(seed)
    even = lambda lo, hi: 2 * rng.randint(lo // 2, hi // 2)

    def feed_forward():
        kind = rng.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            return None
        if kind == "dense":
            return K.dense(rng.randint(8, 64))
        groups = rng.choice([None, None, 2, 3, 4])
        per = rng.randint(1, 4)
        experts = per * (groups or rng.randint(2, 3))
        keep = rng.randint(1, groups) if groups else None
        if groups and keep * per < 2:
            keep = 2
        allowed = keep * per if groups else experts
        top = rng.randint(2, allowed)            # two or more: the lesser of two nearly equal experts counts little
        shared = (rng.randint(8, 40), rng.uniform(0.5, 4.0)) if rng.random() < 0.6 else None
        return K.moe(rng.randint(8, 40), rng.uniform(0.5, 4.0), experts, top, (groups, keep) if groups else None, shared)

    layers, own = [], []
    for i in range(rng.randint(2, 6)):
        if own and rng.random() < 0.45:
            j = rng.choice(own)
            m = layers[j]["mixer"]
            layers.append(K.attention(m["heads"], m["kv_heads"], m["dim"], m["vdim"], rng.uniform(0.1, 0.5),
                                      rng.choice([None, rng.randint(1, 70)]),
                                      (m["rot"]["base"], m["rot"]["dims"]) if "rot" in m else None, kv_from=j,
                                      mlp=feed_forward()))
            continue
        kv = rng.randint(1, 3)
        dim = rng.choice([16, 32, 48, 64]) if rng.random() < 0.4 else even(4, 40)
        vdim = dim if rng.random() < 0.5 else even(4, 40)
        rot = None if rng.random() < 0.2 else (rng.choice([50.0, 10000.0, 300000.0]), even(2, dim))
        layers.append(K.attention(kv * rng.randint(1, 4), kv, dim, vdim, rng.uniform(0.1, 0.5),
                                  rng.choice([None, rng.randint(1, 70)]), rot, mlp=feed_forward()))
        own.append(i)
    # a token input one column wide is the sign of one number times a fixed vector, and a sign that rounding flips
    # shows in full: the fixed configurations have that width, the drawn ones three columns or more
    return K.config(rng.randint(50, 300), even(24, 96), rng.choice([1e-5, 1e-6, 3e-4]), layers,
                    side=rng.choice([None, 3, 4, 9, 16]))


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(seed, tmp_path):
    raw = drawn_config(seed)
    T = 90
    ids = K.tokens(raw["vocab"], T, seed)
    w = K.clear_weights(raw, 700 + seed, ids)
    folder = K.write_model(str(tmp_path / "m"), raw, w)
    want, close = K.oracle_and_close_calls(raw, w, ids)
    for dtype in ("float32", "bfloat16"):
        eng = K.make_engine(folder, dtype, page_size=(4, 8, 16)[seed % 3], pool_tokens=256)
        K.check_clear(K.run_alone(eng, 1, ids, [T]), want, close, dtype, f"{seed} whole")
        K.check_clear(K.run_alone(eng, 2, ids, [T - 30] + [1] * 30), want, close, dtype, f"{seed} last 30 decoded")
        K.check_clear(K.run_alone(eng, 3, ids, cut(T, [2, 17, 3, 40, 1, 5])), want, close, dtype, f"{seed} in portions")
        assert eng.cache.manager.check() == ""
        del eng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_with_sharp_scores(dtype, models):
    """Prompts of hundreds of tokens over many pages; scores so sharp that the best key inside the block, wherever it
    lies, takes nearly all of a position's weight (or the sink does), also for the layer that reads the other's keys."""
    for name in ("blocks", "far"):
        raw, w, folder = models[name]
        T = 500
        ids = K.tokens(raw["vocab"], T, 11)
        want = K.oracle(raw, w, ids)
        eng = K.make_engine(folder, dtype, page_size=16, pool_tokens=512)
        tol = K.tolerance(name, dtype)
        K.check(K.run_alone(eng, 1, ids, [T]), want, dtype, name + " whole", tol)
        K.check(K.run_alone(eng, 2, ids, [T - 70, 37, 2] + [1] * 31), want, dtype, name + " tail decoded", tol)
        K.check(K.run_alone(eng, 3, ids, cut(T, [127, 2, 16, 129, 15, 1 + 16 * 7])), want, dtype, name + " in portions", tol)
        del eng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["T1", "T2"])
def test_mixed_batches_with_pages_and_slots_used_again(name, dtype, models):
    """Up to three live requests of unequal length in a pool that holds far less than all of them: portions of some
    beside decoded tokens of others, and every position's logits as alone."""
    from llm_infer_rust_b200.engine import StepEntry
    from replay_driver import mixed_schedule
    raw, w, folder = models[name]
    lengths = {"a": 90, "b": 37, "c": 120, "d": 5, "e": 64, "f": 101}
    reqs = {r: (K.tokens(raw["vocab"], n, 20 + i), max(2, n - 12 - i)) for i, (r, n) in enumerate(lengths.items())}
    want = {r: K.oracle_and_close_calls(raw, w, ids) for r, (ids, _) in reqs.items()}
    eng = K.make_engine(folder, dtype, page_size=8, pool_tokens=320, max_requests=3)
    got = {r: [] for r in reqs}
    number = {r: i + 1 for i, r in enumerate(reqs)}
    opened = set()
    for entries, end in mixed_schedule(reqs, 320, seed=4, max_live=3):
        batch = []
        for r, toks, wanted in entries:
            if r not in opened:
                eng.open_request(number[r])
                opened.add(r)
            batch.append(StepEntry(number[r], list(toks), list(wanted)))
        logits = eng.step(batch).cpu().numpy()
        at = 0
        for r, toks, _ in entries:
            got[r].append(logits[at:at + len(toks)].copy())
            at += len(toks)
        for r in end:
            eng.close_request(number[r])
        assert eng.cache.manager.check() == ""
    eng.check_kernel_errors()
    for r in reqs:
        K.check_clear(np.concatenate(got[r]), *want[r], dtype, f"request {r} in mixed batches")


def test_pages_that_are_used_again_hold_nothing_of_their_last_user(models):
    """One request at a time in a pool of a few pages: the second gets the pages that the first one left full."""
    raw, w, folder = models["T1"]
    eng = K.make_engine(folder, "float32", page_size=4, pool_tokens=64, max_requests=1)
    first, second = K.tokens(raw["vocab"], 50, 1), K.tokens(raw["vocab"], 33, 2)
    K.check(K.run_alone(eng, 1, first, [20, 30]), K.oracle(raw, w, first), "float32", "first user of the pages")
    K.check(K.run_alone(eng, 2, second, [1, 1, 31]), K.oracle(raw, w, second), "float32", "second user of the pages")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, models):
    raw, w, folder = models["T1"]
    ids = K.tokens(raw["vocab"], 260, 8)
    eng = K.make_engine(folder, dtype, page_size=16, pool_tokens=320)
    K.check_clear(K.run_alone(eng, 1, ids, [6] + [1] * 254), *K.oracle_and_close_calls(raw, w, ids), dtype,
                  "254 tokens decoded one by one")


@pytest.mark.parametrize("dtype,graphs,portion_graphs", [("float32", 0, 0), ("bfloat16", 0, 0), ("bfloat16", 4, 0),
                                                         ("bfloat16", 4, 64)])
def test_greedy_generation_through_the_scheduler(dtype, graphs, portion_graphs, models):
    """``Engine.generate``: prompts cut by the scheduler's token budget, more prompts than slots, decode graphs in
    bfloat16, and graphs of prompt portions whose shape comes again.  float32: the tokens are the plain
    implementation's; bfloat16: every generated token is one whose plain logit is within a small margin of the best."""
    from llm_infer_rust_b200 import SamplingParams
    raw, w, folder = models["T2"]
    prompts = [K.tokens(raw["vocab"], n, 40 + n) for n in (5, 23, 1, 12, 30, 64, 50)]
    eng = K.make_engine(folder, dtype, page_size=8, pool_tokens=512, max_requests=3, cuda_graph_bs=graphs,
                        chunked_prefill_size=16, max_prefill_tokens_per_batch=16,
                        prefill_cuda_graph_max_tokens=portion_graphs)
    results = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    eng.check_kernel_errors()
    for prompt, res in zip(prompts, results):
        assert len(res.tokens) == 12
        logits = K.oracle(raw, w, prompt + res.tokens)
        for i, tok in enumerate(res.tokens):
            row = logits[len(prompt) - 1 + i]
            margin = 1e-4 if dtype == "float32" else 0.05 * max(1.0, np.abs(row).max())
            assert row[tok] >= row.max() - margin, f"token {i} of a prompt of {len(prompt)}: {tok} is not the best"


def test_trace_replay_as_a_user_runs_it(models, tmp_path):
    from replay_driver import Replay, run_alone
    raw, w, folder = models["T3"]
    ids = K.tokens(raw["vocab"], 70, 9)
    want, close = K.oracle_and_close_calls(raw, w, ids)
    for dtype in ("bfloat16", "float32"):
        rp = Replay(folder, dtype, 128, str(tmp_path / dtype), raw["vocab"], ["--page-size", "8"])
        try:
            # the runner's path is what is tested here; the engine's numbers are held to the tighter bound above
            K.check_clear(run_alone(rp, "x", ids, [33, 2, 3] + [1] * 32), want, close, dtype, "replay",
                          1e-4 if dtype == "float32" else None)
        finally:
            assert rp.close() == 0


def test_command_line_random_weights_mode(tmp_path):
    """The command line writes a random Torinex model from a configuration and serves it; the same folder through
    ``Engine.generate`` gives the same tokens."""
    import json
    import os
    import subprocess
    import sys
    from llm_infer_rust_b200 import SamplingParams
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(K.CONFIGS["T1"]))
    made = tmp_path / "made"
    cmd = [sys.executable, "-m", "llm_infer_rust_b200", "--model-path", str(made), "--random-weights", "--config",
           str(cfg), "--seed", "5", "--dtype", "float32", "--page-size", "4", "--max-total-tokens", "256",
           "--max-running-req", "2", "--max-seq-len", "64", "--cuda-graph-bs", "0", "--prompt-ids", "1,2,3",
           "--prompt-ids", "9,8,7,6,5", "--max-tokens", "6", "--ignore-eos"]
    done = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    lines = [json.loads(x) for x in done.stdout.strip().splitlines()]
    assert sorted(os.listdir(made)) == ["config.json", "model.safetensors"]
    eng = K.make_engine(str(made), "float32", page_size=4, pool_tokens=256, max_requests=2)
    want = eng.generate([[1, 2, 3], [9, 8, 7, 6, 5]], SamplingParams(max_tokens=6, ignore_eos=True))
    assert [x["output_ids"] for x in lines] == [r.tokens for r in want]
    eng.check_kernel_errors()
