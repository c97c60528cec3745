#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with its share of the roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--shape 0.6b|8b|32b] [--layers L]
                    [--batch B] [--context C] [--point-shapes 8b,32b] [--no-points] [--impl ours|reference]

A step is one decode step of a batch of B requests whose context ends at C tokens: the
requests are prefilled with random token ids up to C - W - K tokens, W + K tokens are
decoded greedily, and the last K steps are timed.  One JSON line is printed:

* ``value``: decoded tokens a second, timed on the device (CUDA events around K steps that are
  queued back to back: each step's sampled tokens go to the next step on the device);
* ``e2e``: the same through ``Engine.add_request`` / ``Engine.schedule_step``: prompts go in as
  host token ids, every step's index arrays are copied from pinned host memory, its sampled ids
  are read back to the host and returned to the caller step by step (the scheduler loop launches
  the next decode step before it has read the running one's ids, so a decoded token reaches the
  next step on the device as well as the host);
* ``prefill``: one step of 2,048 prompt tokens; ``frac`` = its FLOPs / time / the bfloat16 peak;
* ``roofline``: bytes that a decode step must read (every weight once and the cache of the live
  requests) / its time, against the measured copy bandwidth;
* ``points``: decoded tokens a second at batch 1 and 64 at the same context and at the headline batch at half the
  context, each with ``_frac``, its share of the roofline (bytes as above / time / measured copy bandwidth); then the
  same figures (``<shape>_decode_b1`` ... ``<shape>_prefill_frac``) for the other shapes of ``--point-shapes``, by
  default the Qwen3-8B and Qwen3-32B layer sizes with all their layers (each engine is built, measured with a quarter
  of the steps and released before the next);
* ``routing``: which products of a decode step ran on this package's few-row kernels and which on the library (a
  rule of sizes, not a measurement: the same line again on the same machine takes the same kernels).

``--design kefetar`` leaves all of the above aside and prints another line: prefill and decode throughput of Kefetar
(gated convolutional attention and decay retention over a float32 stream) at two layer sizes, beside dense Qwen3 at
the same width, heads, head size and parameter count, and every kernel of the new design alone beside the like
kernel of Qwen3's path, each with its share of its roofline (``--design-sizes``, ``--layers``, default 8).

``--design mukenex`` does the same for Mukenex (latent attention over a window with sinks, grouped attention over
blocks of positions, lightning retention, experts chosen by a table, a residual of four streams).

``--design torinex`` does the same for Torinex (attention over blocks of positions with projection-wide norms and one
added to the softmax's denominator, layers that read another layer's keys and values, routed experts with groups and
a shared expert, a per-layer token input, norms on the sublayers' outputs over a float32 stream); its routed experts
also stand beside Mukenex's.

``--design lufizen`` does the same for Lufizen (attention whose values are the projected keys, with a plain norm after
a stretched rotation and learned sinks; latent attention with queries through a latent and a gate a head; a router
with a choice correction and groups ranked by their two best members; a gated shared expert), beside Torinex, the
closest earlier design, and Qwen3.

Peaks come from MEASURED_PEAKS.json beside this file when it is there.  Weights are random
(drawn on the device), token ids are synthetic.  One GPU only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = {
    "0.6b": dict(num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
                 head_dim=128, intermediate_size=3072, vocab_size=151936, tie_word_embeddings=True,
                 max_position_embeddings=40960),
    "8b": dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
               head_dim=128, intermediate_size=12288, vocab_size=151936, tie_word_embeddings=False,
               max_position_embeddings=40960),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8,
                head_dim=128, intermediate_size=25600, vocab_size=151936, tie_word_embeddings=False,
                max_position_embeddings=40960),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
REFERENCE_UNAVAILABLE = ("the reference is a Rust binary over libtorch: pip install --no-deps of it succeeds but installs "
                         "metadata only (no module, no binary); building it needs cargo/rustc and torch==2.13.0, "
                         "neither of which this image has")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            p = json.load(fh)
        return {k: float(p.get(k, FALLBACK_PEAKS[k])) for k in FALLBACK_PEAKS}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        self.thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no sample"]}
        reasons = [n for i, n in enumerate(self.NAMES) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": statistics.median(int(s[0]) for s in self.samples),
                "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons, "samples": len(self.samples)}


def model_numbers(raw):
    """Parameter counts and per-token cache bytes of a dense Qwen3 shape (bfloat16)."""
    L, H, nh, nkv, d = (raw["num_hidden_layers"], raw["hidden_size"], raw["num_attention_heads"],
                        raw["num_key_value_heads"], raw["head_dim"])
    I, V = raw["intermediate_size"], raw["vocab_size"]
    layer_matrix = (nh + 2 * nkv) * d * H + H * nh * d + 3 * I * H
    layer_params = layer_matrix + 2 * H + 2 * d
    head = V * H
    embed = 0 if raw["tie_word_embeddings"] else V * H
    return dict(layer_matrix=layer_matrix, params=L * layer_params + head + embed + H,
                decode_weight_bytes=2 * (L * layer_params + head + H), kv_bytes_per_token=L * 2 * nkv * d * 2)


def prefill_flops(raw, T):
    n = model_numbers(raw)
    L, nh, d = raw["num_hidden_layers"], raw["num_attention_heads"], raw["head_dim"]
    return 2.0 * T * n["layer_matrix"] * L + L * nh * 4.0 * d * T * (T + 1) / 2 + 2.0 * raw["vocab_size"] * raw["hidden_size"]


def random_prompt(vocab, n, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def fill_requests(engine, ids, prompt_len, vocab, chunk=4096):
    """Open the requests and run their prompts through the step function, in portions."""
    from llm_infer_rust_b200.engine import StepEntry
    for r in ids:
        engine.open_request(r)
        prompt = random_prompt(vocab, prompt_len, 1000 + r)
        for at in range(0, prompt_len, chunk):
            engine.step([StepEntry(r, prompt[at:at + chunk], [])])


def decode_device_timed(engine, batch, context, steps, warmup, vocab):
    """Tokens a second of `steps` decode steps that end at `context` tokens, timed on the device."""
    import torch
    from llm_infer_rust_b200 import SamplingParams
    from llm_infer_rust_b200.engine import StepEntry
    from llm_infer_rust_b200.kernels import ops
    ids = list(range(1, batch + 1))
    fill_requests(engine, ids, context - steps - warmup, vocab)
    rows = [(SamplingParams(), 0, 0)] * batch
    entries = [StepEntry(r, [0], [0]) for r in ids]
    tokens = torch.zeros(batch, dtype=torch.int32, device=engine.device)
    for _ in range(warmup):
        tokens = engine.sampler.sample_device(engine.step(entries, device_tokens=tokens), rows)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = ops.launch_count()
    start.record()
    for _ in range(steps):
        tokens = engine.sampler.sample_device(engine.step(entries, device_tokens=tokens), rows)
    end.record()
    torch.cuda.synchronize()
    launches = ops.launch_count() - launches
    ms = start.elapsed_time(end) / steps
    engine.check_kernel_errors()
    mean_context = context - (steps + 1) / 2.0
    for r in ids:
        engine.close_request(r)
    return dict(tokens_per_s=batch * 1000.0 / ms, ms_per_step=ms, launches=launches, mean_context=mean_context)


def decode_end_to_end(engine, batch, context, steps, warmup, vocab):
    """The same through the public scheduler loop: host token ids in, host token ids out, every step."""
    import torch
    from llm_infer_rust_b200 import SamplingParams
    # prompts enter one a step, so the first request decodes up to `batch` tokens before the last is in
    prompt_len = context - steps - warmup - batch
    sp = SamplingParams(max_tokens=steps + warmup + 2 * batch + 8, ignore_eos=True)
    for r in range(batch):
        engine.add_request(random_prompt(vocab, prompt_len, 2000 + r), sp)
    while engine.scheduler.num_pending() or any(
            engine.scheduler.status_of(u) != engine._rt.Status.Decoding for u in list(engine._params)):
        engine.schedule_step()                               # prompts, in portions
    for _ in range(warmup - 1):
        engine.schedule_step()
    h2d = engine.last_upload_bytes
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += len(engine.schedule_step())
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    for u in list(engine._params):
        engine.abort_request(u)
    while not engine.is_idle():
        engine.schedule_step()
    assert produced == batch * steps, (produced, batch, steps)
    return dict(tokens_per_s=produced / elapsed, h2d=h2d, d2h=4 * batch)


def prefill_timed(engine, T, vocab, repeats=3):
    import torch
    from llm_infer_rust_b200.engine import StepEntry
    best = None
    for k in range(repeats + 1):
        prompt = random_prompt(vocab, T, 3000 + k)
        engine.open_request(9000 + k)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([StepEntry(9000 + k, prompt, [T - 1])])
        end.record()
        torch.cuda.synchronize()
        engine.close_request(9000 + k)
        if k > 0:                                             # the first run warms up
            ms = start.elapsed_time(end)
            best = ms if best is None else min(best, ms)
    return best


def step_bytes(numbers, batch, mean_context):
    """Bytes that a decode step has to read: every weight once and the cache of the live requests."""
    return numbers["decode_weight_bytes"] + batch * mean_context * numbers["kv_bytes_per_token"]


def routing_of(engine, rows):
    """Which way the products of a step of `rows` tokens go: this package's few-row kernels (the ring kernel, or the
    streaming kernel for the largest weights) or the library."""
    from llm_infer_rust_b200.kernels import ops
    block = engine.model.blocks[0]
    mixer, ff = block.mixer, block.feed_forward
    products = {"qkv": (mixer.params["qkv_proj"], ops.EPI_QKV, mixer.d), "o": (mixer.params["o_proj"], ops.EPI_PLAIN_BF16, 0),
                "gate_up": (ff.params["gate_up_proj"], ops.EPI_SWIGLU, 0), "down": (ff.params["down_proj"], ops.EPI_PLAIN_BF16, 0),
                "head": (engine.model.lm_head.params["weight"], ops.EPI_PLAIN_F32, 0)}
    library = [name for name, (w, mode, d) in products.items() if not ops.few_row_takes(rows, w, engine.dtype, mode, d)]
    streamed = [name for name, (w, mode, d) in products.items()
                if name not in library and mode != ops.EPI_QKV and ops.stream_takes(rows, w, engine.dtype, mode)]
    return (f"{ops.few_row_route} kernel" + (f", streaming kernel for {'+'.join(streamed)}" if streamed else "")
            + (f", library for {'+'.join(library)}" if library else ""))


def build_engine(shape_name, layers, biggest, context):
    from llm_infer_rust_b200.engine import Engine
    shape = dict(SHAPES[shape_name])
    full_layers = shape["num_hidden_layers"]
    if layers:
        shape["num_hidden_layers"] = min(layers, full_layers)
    raw = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], rope_theta=1e6, rms_norm_eps=1e-6,
               torch_dtype="bfloat16", eos_token_id=None, **shape)
    pool_tokens = biggest * (context + 128) + 4096
    engine = Engine(None, random_weights_config=raw, random_weights_seed=0, dtype="bfloat16",
                    max_running_req=biggest, max_seq_len=context + 64, page_size=16,
                    max_total_tokens=pool_tokens, cuda_graph_bs=biggest, chunked_prefill_size=4096,
                    prefill_cuda_graph_max_tokens=2048, log_level="warn")
    return engine, raw, full_layers


def release():
    """Give the memory of an engine that the caller has just dropped back to the device (the next engine sizes its
    cache pool from what is free)."""
    import gc
    import torch
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()


def measure_point_shape(shape_name, context, steps, warmup, peak):
    """Decode at batch 1 / 8 / 64 and a prefill of 2,048 tokens at another shape, each with its share of the roofline."""
    engine, raw, _ = build_engine(shape_name, None, 64, context)
    numbers, vocab = model_numbers(raw), raw["vocab_size"]
    out = {}
    prefill_ms = prefill_timed(engine, 2048, vocab)
    tag = shape_name.replace(".", "")
    out[f"{tag}_prefill_tok_s"] = round(2048 * 1000.0 / prefill_ms, 1)
    out[f"{tag}_prefill_frac"] = round(prefill_flops(raw, 2048) / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)
    for b in (1, 8, 64):
        run = decode_device_timed(engine, b, context, steps, warmup, vocab)
        out[f"{tag}_decode_b{b}"] = round(run["tokens_per_s"], 1)
        out[f"{tag}_decode_b{b}_frac"] = round(step_bytes(numbers, b, run["mean_context"]) / (run["ms_per_step"] * 1e-3) / 1e9
                                               / peak["hbm_gbs"], 4)
    routing = f"{shape_name}: {routing_of(engine, 8)}"
    del engine
    release()
    return out, routing


# ----------------------------------------------------------------------------- --design kefetar
DESIGN_SIZES = {
    "1k": dict(width=1024, heads=16, kv_heads=8, head_dim=128, inter=3072, vocab=151936),
    "4k": dict(width=4096, heads=32, kv_heads=8, head_dim=128, inter=12288, vocab=151936),
}


def kefetar_config(size, layers):
    """Attention and retention layers in turn, each with a feed-forward; the feed-forward is 1.5 x Qwen3's
    intermediate size, which gives its two matrices the parameters of Qwen3's three."""
    z = DESIGN_SIZES[size]
    attn = {"type": "attention", "mlp": {"kind": "dense", "ff": z["inter"] * 3 // 2},
            "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["head_dim"], "vdim": z["head_dim"],
                      "conv": 3, "scale": z["head_dim"] ** -0.5, "softcap": 50.0, "v_mix": True,
                      "rot": {"base": 1e6, "dims": z["head_dim"], "scaling": {"factor": 4.0}}}}
    ret = {"type": "retention", "mlp": {"kind": "dense", "ff": z["inter"] * 3 // 2},
           "mixer": {"heads": z["heads"], "dim": z["head_dim"], "vdim": z["head_dim"],
                     "decay": [1.0 - 2.0 ** (-5 - 3 * h / max(1, z["heads"] - 1)) for h in range(z["heads"])],
                     "rot": {"base": 1e6, "dims": z["head_dim"] // 2}}}
    return {"architecture": "Kefetar", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5},
            "canon": {"taps": 3}, "layers": [attn if i % 2 == 0 else ret for i in range(layers)]}


def qwen3_config(size, layers):
    z = DESIGN_SIZES[size]
    return dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], rope_theta=1e6, rms_norm_eps=1e-6,
                torch_dtype="bfloat16", eos_token_id=None, num_hidden_layers=layers, hidden_size=z["width"],
                num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"], head_dim=z["head_dim"],
                intermediate_size=z["inter"], vocab_size=z["vocab"], tie_word_embeddings=False,
                max_position_embeddings=40960)


def design_engine(raw, biggest, context, graphs=True):
    from llm_infer_rust_b200.engine import Engine
    return Engine(None, random_weights_config=raw, random_weights_seed=0, dtype="bfloat16", max_running_req=biggest,
                  max_seq_len=context + 64, page_size=16, max_total_tokens=biggest * (context + 128) + 4096,
                  cuda_graph_bs=biggest if graphs else 0, chunked_prefill_size=4096, log_level="warn")


def timed_alone(fn, flush, repeats=7):
    """Median device time in microseconds of one call of ``fn``, the second-level cache flushed before every call."""
    import torch
    for _ in range(3):
        fn()
    times = []
    for _ in range(repeats):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) * 1e3)
    return statistics.median(times)


def kernel_table(size, peak):
    """Every kernel of the new design alone, beside the like kernel of Qwen3's path, at one layer's sizes: a prompt
    portion of 2,048 tokens and a decode step of 8 rows at 2,048 tokens.  ``frac``: bytes that must move / time / the
    measured copy bandwidth, or FLOPs / time / the peak named in ``of``."""
    import types
    import torch
    from llm_infer_rust_b200.kernels import ops
    z = DESIGN_SIZES[size]
    W, nh, nkv, d, F = z["width"], z["heads"], z["kv_heads"], z["head_dim"], z["inter"] * 3 // 2
    dev, bf = torch.device("cuda"), torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    page, ctx_len, rows_dec = 16, 2048, 8
    out = {}

    def put(name, us, nbytes=None, flops=None, of="hbm"):
        rec = {"us": round(us, 2)}
        if nbytes is not None:
            rec["gb_s"] = round(nbytes / us / 1e3, 1)
            rec["frac"] = round(nbytes / us / 1e3 / peak["hbm_gbs"], 3)
        if flops is not None:
            top = {"bf16": peak["bf16_tflops"], "fp32": peak["fp32_tflops"]}[of]
            rec["tflops"] = round(flops / us / 1e6, 2)
            rec["frac"] = round(flops / us / 1e6 / top, 3)
            rec["of"] = of
        out[name] = rec

    def step(rows):
        cu, row_of, pos = [0], [], []
        for r, (prefix, n) in enumerate(rows):
            cu.append(cu[-1] + n)
            row_of += [r] * n
            pos += list(range(prefix, prefix + n))
        R = len(rows)
        width = -(-max(p + n for p, n in rows) // page)
        table = torch.arange(1, R * width + 1, dtype=torch.int32, device=dev).view(R, width).contiguous()
        slots = [int(table[r, (p + i) // page]) * page + (p + i) % page for r, (p, n) in enumerate(rows) for i in range(n)]
        return types.SimpleNamespace(
            num_rows=R, row_of_token=i32(row_of), cu_q=i32(cu), positions=i32(pos), prefix_len=i32([p for p, _ in rows]),
            kv_len=i32([p + n for p, n in rows]), state_slots=i32(list(range(1, R + 1))), slots=i32(slots), table=table,
            rows=i32(list(range(R))), tokens=cu[-1], pages=R * width + 1, max_q_len=max(n for _, n in rows),
            num_prefill=sum(n > 1 for _, n in rows))

    for phase, c in (("prefill", step([(0, ctx_len)])), ("decode", step([(ctx_len - 1, 1)] * rows_dec))):
        T = c.tokens
        x = torch.randn(T, W, device=dev)
        y = torch.randn(T, W, device=dev).to(bf)
        gain = torch.ones(1, device=dev)
        res_b, xb = torch.randn(T, W, device=dev).to(bf), torch.randn(T, W, device=dev).to(bf)
        wn = torch.ones(W, dtype=bf, device=dev)
        # --- norm sites
        scale = ops.residual_scale(x, y, gain, 1e-5)
        put(f"{phase}.kefetar.residual_scale", timed_alone(lambda: ops.residual_scale(x, y, gain, 1e-5), flush), T * W * 10)
        cw = torch.randn(W, 3, device=dev) * 0.1
        cstate = torch.zeros(rows_dec + 1, 2, W, device=dev)
        put(f"{phase}.kefetar.causal_taps", timed_alone(
            lambda: ops.causal_taps(x, cw, cstate, c, bf, scale=scale, identity=True), flush), T * W * 6)
        put(f"{phase}.qwen3.add_rms_norm", timed_alone(lambda: ops.add_rms_norm(xb, res_b, wn, 1e-6), flush), T * W * 8)
        # --- between the projection and attention
        cq = (nh + 2 * nkv) * d
        packed = (torch.randn(T, cq + nh * d, device=dev) * 0.5).to(bf)
        k_cache = torch.zeros(c.pages, nkv, page, d, dtype=bf, device=dev).normal_()
        v_cache = torch.zeros(c.pages, nkv, page, d, dtype=bf, device=dev).normal_()
        q = torch.empty(T, nh * d, dtype=bf, device=dev)
        qw = torch.randn(cq, 3, device=dev) * 0.3
        qstate = torch.zeros(rows_dec + 1, 2, cq, device=dev)
        inv_freq = torch.pow(torch.tensor(1e6), -torch.arange(0, d, 2) / d).to(dev)
        vfirst, lam = torch.randn(T, nkv * d, device=dev), torch.full((1,), 0.5, device=dev)
        put(f"{phase}.kefetar.conv_qkv_post", timed_alone(lambda: ops.conv_qkv_post(
            packed, qw, qstate, c, q, k_cache, v_cache, inv_freq, d, c.slots, nh, nkv, d, d, vmix=lam, v_first=vfirst,
            v_mode=2), flush), T * cq * 4 + T * nkv * d * 4)
        qkv = packed[:, :cq].contiguous()
        cos, sin = torch.ones(4096, d // 2, device=dev), torch.zeros(4096, d // 2, device=dev)
        hn = torch.ones(d, dtype=bf, device=dev)
        put(f"{phase}.qwen3.qkv_post", timed_alone(lambda: ops.qkv_post(
            qkv, q, k_cache, v_cache, hn, hn, 1e-6, cos, sin, d, c.positions, c.slots, nh, nkv, d), flush), T * cq * 4)
        # --- attention
        o = torch.empty(T, nh * d, dtype=bf, device=dev)
        if phase == "prefill":
            fl = 4.0 * nh * d * T * (T + 1) / 2
            put("prefill.kefetar.attention_softcap", timed_alone(lambda: ops.prefill_attention(
                q, k_cache, v_cache, o, c.table, c.cu_q, c.kv_len, c.prefix_len, c.rows, 1, T, nh, nkv, d, page, None,
                d ** -0.5, v_head_dim=d, softcap=50.0, precise_weights=True), flush, repeats=3), flops=fl, of="bf16")
            put("prefill.qwen3.attention", timed_alone(lambda: ops.prefill_attention(
                q, k_cache, v_cache, o, c.table, c.cu_q, c.kv_len, c.prefix_len, c.rows, 1, T, nh, nkv, d, page, None,
                d ** -0.5), flush), flops=fl, of="bf16")
        else:
            from llm_infer_rust_b200.parts.attention import decode_splits
            kvb = rows_dec * ctx_len * nkv * d * 2 * 2
            for name, kw, plain in (("kefetar.attention_softcap", dict(v_head_dim=d, softcap=50.0, precise_weights=True), True),
                                    ("qwen3.attention", {}, True)):
                splits = decode_splits(ops.decode_ctas_per_split(bf, rows_dec, nh, nkv, d, page, plain), ctx_len, 148)
                need = ops.decode_scratch_floats(rows_dec, nh, d, splits)
                scratch = torch.empty(max(need, 1), device=dev)
                put(f"decode.{name}", timed_alone(lambda: ops.decode_attention(
                    q, k_cache, v_cache, o, scratch, c.table, c.cu_q, c.kv_len, c.rows, rows_dec, nh, nkv, d, page, None,
                    d ** -0.5, splits, **kw), flush), kvb)
        # --- gates and activations
        put(f"{phase}.kefetar.sigmoid_gate_mul", timed_alone(lambda: ops.sigmoid_gate_mul(o, packed, cq), flush), T * nh * d * 6)
        zf = (torch.randn(T, F, device=dev)).to(bf)
        coef = torch.ones(4, device=dev)
        put(f"{phase}.kefetar.poly_norm", timed_alone(lambda: ops.poly_norm(zf, coef, 1e-5), flush), T * F * 4)
        gu = torch.randn(T, 2 * z["inter"], device=dev).to(bf)
        put(f"{phase}.qwen3.silu_mul", timed_alone(lambda: ops.silu_mul(gu), flush), T * z["inter"] * 6)
        # --- retention
        rp = (torch.randn(T, nh * 4 * d, device=dev) * 0.3).to(bf)
        rstate = torch.zeros(rows_dec + 1, nh, d, d, device=dev)
        decay = torch.full((nh,), 0.99, device=dev)
        rf = inv_freq[: d // 4].contiguous()
        us = timed_alone(lambda: ops.retention(rp, rstate, decay, rf, d // 2, d ** -0.5, c, nh, d, d), flush,
                         repeats=3 if phase == "prefill" else 7)
        if phase == "prefill":
            put("prefill.kefetar.retention", us, flops=4.0 * T * nh * d * d, of="fp32")
        else:
            put("decode.kefetar.retention", us, rows_dec * nh * d * d * 8)
        ro = torch.randn(T, nh * d, device=dev)
        put(f"{phase}.kefetar.head_unit_norm_gate", timed_alone(
            lambda: ops.head_unit_norm_gate(ro, rp, nh * 3 * d, nh, d, 1e-5), flush), T * nh * d * 8)
    return out


# ----------------------------------------------------------------------------- --design mukenex
def mukenex_config(size, layers):
    """Lightning, latent-attention and block-attention layers in turn over four residual streams.  Routed layers
    take two of eight experts of half Qwen3's intermediate size (the active parameters of Qwen3's three matrices),
    dense ones 1.5 x Qwen3's intermediate size in two matrices."""
    z = DESIGN_SIZES[size]
    H, G, d, W = z["heads"], z["kv_heads"], z["head_dim"], z["width"]
    rank = 256 if W <= 1024 else 384
    moe = {"kind": "moe", "expert": {"ff": z["inter"] // 2}, "router": {"experts": 8, "top": 2}}
    dense = {"kind": "dense", "ff": z["inter"] * 3 // 2}
    lightning = {"type": "lightning", "mlp": dense,
                 "mixer": {"heads": H, "dim": d, "vdim": d,
                           "decay": [1.0 - 2.0 ** (-5 - 3 * h / max(1, H - 1)) for h in range(H)]}}
    latent = {"type": "latent_attention", "mlp": moe,
              "mixer": {"heads": H, "dim": d, "rot_dim": 64, "vdim": d, "kv_rank": rank, "scale": (d + 64) ** -0.5,
                        "rot": {"base": 1e6, "dims": 64}, "mask": {"size": 1024}}}
    blocks = {"type": "attention", "mlp": moe,
              "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "mask": {"size": 1024}}}
    return {"architecture": "Mukenex", "vocab": z["vocab"], "width": W, "norm": {"eps": 1e-5}, "streams": 4,
            "logit_softcap": 30.0, "layers": [(lightning, latent, blocks)[i % 3] for i in range(layers)]}


def mukenex_kernel_table(size, peak):
    """Every kernel of Mukenex alone, beside the like kernel of Qwen3's path, at one layer's sizes: a prompt portion of
    2,048 tokens and a decode step of 8 rows at 2,048 tokens (``frac`` as in ``kernel_table``)."""
    import types
    import torch
    from llm_infer_rust_b200.kernels import ops
    from llm_infer_rust_b200.parts.attention import decode_splits
    z = DESIGN_SIZES[size]
    W, nh, nkv, d, I = z["width"], z["heads"], z["kv_heads"], z["head_dim"], z["inter"]
    rank, r, S, E, top, ffe, window = (256 if W <= 1024 else 384), 64, 4, 8, 2, z["inter"] // 2, 1024
    dev, bf = torch.device("cuda"), torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    page, ctx_len, rows_dec = 16, 2048, 8
    out = {}

    def put(name, us, nbytes=None, flops=None, of="hbm"):
        rec = {"us": round(us, 2)}
        if nbytes is not None:
            rec["gb_s"] = round(nbytes / us / 1e3, 1)
            rec["frac"] = round(nbytes / us / 1e3 / peak["hbm_gbs"], 3)
        if flops is not None:
            top_ = {"bf16": peak["bf16_tflops"], "fp32": peak["fp32_tflops"]}[of]
            rec["tflops"] = round(flops / us / 1e6, 2)
            rec["frac"] = round(flops / us / 1e6 / top_, 3)
            rec["of"] = of
        out[name] = rec

    def step(rows):
        cu, pos = [0], []
        for prefix, n in rows:
            cu.append(cu[-1] + n)
            pos += list(range(prefix, prefix + n))
        R = len(rows)
        width = -(-max(p + n for p, n in rows) // page)
        table = torch.arange(1, R * width + 1, dtype=torch.int32, device=dev).view(R, width).contiguous()
        slots = [int(table[r_, (p + i) // page]) * page + (p + i) % page for r_, (p, n) in enumerate(rows) for i in range(n)]
        return types.SimpleNamespace(
            num_rows=R, cu_q=i32(cu), positions=i32(pos), prefix_len=i32([p for p, _ in rows]),
            kv_len=i32([p + n for p, n in rows]), state_slots=i32(list(range(1, R + 1))), slots=i32(slots), table=table,
            rows=i32(list(range(R))), tokens=cu[-1], pages=R * width + 1, max_q_len=max(n for _, n in rows),
            num_prefill=sum(n > 1 for _, n in rows))

    def seen(T, size_, blocks):         # (query, key) pairs of a prompt of T tokens under a window or blocks of size_
        return sum((p % size_ if blocks else min(p, size_ - 1)) + 1 for p in range(T))

    for phase, c in (("prefill", step([(0, ctx_len)])), ("decode", step([(ctx_len - 1, 1)] * rows_dec))):
        T = c.tokens
        # --- the residual: write-back of one sublayer, read and norm of the next
        streams = torch.randn(T, S, W, device=dev)
        y = torch.randn(T, W, device=dev).to(bf)
        coef = torch.rand(S * (S + 2), device=dev)
        wn = torch.zeros(W, device=dev)
        put(f"{phase}.mukenex.stream_step", timed_alone(lambda: ops.stream_step(
            streams, wn, 1.0, 1e-5, bf, y=y, before=coef, read_in=coef[:S]), flush), T * W * (8 * S + 4))
        res_b, xb = torch.randn(T, W, device=dev).to(bf), torch.randn(T, W, device=dev).to(bf)
        wb = torch.ones(W, dtype=bf, device=dev)
        put(f"{phase}.qwen3.add_rms_norm", timed_alone(lambda: ops.add_rms_norm(xb, res_b, wb, 1e-6), flush), T * W * 8)
        # --- between the projection and attention
        cq = (nh + 2 * nkv) * d
        packed = (torch.randn(T, cq, device=dev) * 0.5).to(bf)
        k_cache = torch.zeros(c.pages, nkv, page, d, dtype=bf, device=dev).normal_()
        v_cache = torch.zeros(c.pages, nkv, page, d, dtype=bf, device=dev).normal_()
        q = torch.empty(T, nh * d, dtype=bf, device=dev)
        bias, hw = torch.zeros(cq, device=dev), torch.ones(d, device=dev)
        put(f"{phase}.mukenex.heads_prepare", timed_alone(lambda: ops.heads_prepare(
            packed, q, k_cache, v_cache, c.positions, c.slots, nh, nkv, d, d, bias=bias, q_weight=hw, k_weight=hw,
            eps=1e-5), flush), T * cq * 4)
        cos, sin = torch.ones(4096, d // 2, device=dev), torch.zeros(4096, d // 2, device=dev)
        hn = torch.ones(d, dtype=bf, device=dev)
        put(f"{phase}.qwen3.qkv_post", timed_alone(lambda: ops.qkv_post(
            packed, q, k_cache, v_cache, hn, hn, 1e-6, cos, sin, d, c.positions, c.slots, nh, nkv, d), flush), T * cq * 4)
        lq = nh * (d + r)
        lpacked = (torch.randn(T, lq + rank + r, device=dev) * 0.5).to(bf)
        lk = torch.zeros(c.pages, 1, page, rank + r, dtype=bf, device=dev).normal_()
        uk_t = (torch.randn(nh, rank, d, device=dev) * d ** -0.5).to(bf)
        uv = (torch.randn(nh, d, rank, device=dev) * rank ** -0.5).to(bf)
        q_plain = lpacked[:, :lq].view(T, nh, d + r)[:, :, :d].transpose(0, 1)
        q_lat = ops.head_products(q_plain, uk_t)
        put(f"{phase}.mukenex.head_products_uk", timed_alone(lambda: ops.head_products(q_plain, uk_t), flush),
            flops=2.0 * T * nh * d * rank, of="bf16")
        lqo = torch.empty(T, nh * (rank + r), dtype=bf, device=dev)
        inv_freq = torch.pow(torch.tensor(1e6), -torch.arange(0, r, 2) / r).to(dev)
        lw = torch.ones(rank, device=dev)
        put(f"{phase}.mukenex.latent_prepare", timed_alone(lambda: ops.latent_prepare(
            lpacked, q_lat, lqo, lk, None, lw, 1e-5, c.positions, c.slots, nh, d, r, rank, inv_freq=inv_freq, rot_dims=r),
            flush), T * (nh * (rank * 2 + r * 2) * 2 + (rank + r) * 2 * 2))      # (the latent is stored once: key and value)
        # --- attention
        o = torch.empty(T, nh * d, dtype=bf, device=dev)
        lo = torch.empty(T, nh * rank, dtype=bf, device=dev)
        sinks = torch.zeros(nh, device=dev)
        if phase == "prefill":
            put("prefill.mukenex.attention_blocks", timed_alone(lambda: ops.prefill_attention(
                q, k_cache, v_cache, o, c.table, c.cu_q, c.kv_len, c.prefix_len, c.rows, 1, T, nh, nkv, d, page, None,
                d ** -0.5, v_head_dim=d, precise_weights=True, chunk=window), flush, repeats=3),
                flops=4.0 * nh * d * seen(T, window, True), of="bf16")
            put("prefill.mukenex.attention_latent", timed_alone(lambda: ops.prefill_attention(
                lqo, lk, None, lo, c.table, c.cu_q, c.kv_len, c.prefix_len, c.rows, 1, T, nh, 1, rank + r, page, window,
                (d + r) ** -0.5, v_head_dim=rank, precise_weights=True, sinks=sinks, shared_values=True), flush, repeats=3),
                flops=2.0 * nh * (2 * rank + r) * seen(T, window, False), of="bf16")
            put("prefill.qwen3.attention", timed_alone(lambda: ops.prefill_attention(
                q, k_cache, v_cache, o, c.table, c.cu_q, c.kv_len, c.prefix_len, c.rows, 1, T, nh, nkv, d, page, None,
                d ** -0.5), flush), flops=4.0 * nh * d * T * (T + 1) / 2, of="bf16")
        else:
            def decode(name, qq, kk, vv, oo, heads, kvh, dk, dv_, bound, nbytes, **kw):
                plain = dk == dv_
                per_split = ops.decode_ctas_per_split(bf, rows_dec, heads, kvh, dk, page, plain)
                if kw.get("shared_values"):
                    per_split = rows_dec * (heads // ops.latent_head_group(heads))
                splits = decode_splits(per_split, bound, 148)
                need = ops.decode_scratch_floats(rows_dec, heads, max(dk, dv_), splits)
                scratch = torch.empty(max(need, 1), device=dev)
                win, scale = kw.pop("window_", None), kw.pop("scale_", dk ** -0.5)
                put(name, timed_alone(lambda: ops.decode_attention(
                    qq, kk, vv, oo, scratch, c.table, c.cu_q, c.kv_len, c.rows, rows_dec, heads, kvh, dk, page,
                    win, scale, splits, **kw), flush), nbytes)
            kv_all = rows_dec * ctx_len * nkv * d * 2 * 2
            decode("decode.mukenex.attention_blocks", q, k_cache, v_cache, o, nh, nkv, d, d, window,
                   rows_dec * window * nkv * d * 2 * 2, v_head_dim=d, precise_weights=True, chunk=window)
            decode("decode.mukenex.attention_latent", lqo, lk, None, lo, nh, 1, rank + r, rank, window,
                   rows_dec * window * (rank + r) * 2, v_head_dim=rank, precise_weights=True, sinks=sinks,
                   window_=window, shared_values=True)
            decode("decode.qwen3.attention", q, k_cache, v_cache, o, nh, nkv, d, d, ctx_len, kv_all)
        lo_t = lo.view(T, nh, rank).transpose(0, 1)
        lout = torch.empty(T, nh * d, dtype=bf, device=dev)
        put(f"{phase}.mukenex.head_products_uv", timed_alone(lambda: ops.head_products(
            lo_t, uv, out=lout.view(T, nh, d).transpose(0, 1)), flush), flops=2.0 * T * nh * d * rank, of="bf16")
        # --- gates and activations
        gp = (torch.randn(T, 2 * nh * d, device=dev)).to(bf)
        put(f"{phase}.mukenex.sigmoid_gate_mul", timed_alone(lambda: ops.sigmoid_gate_mul(o, gp, nh * d), flush), T * nh * d * 6)
        zf = torch.randn(T, I * 3 // 2, device=dev).to(bf)
        put(f"{phase}.mukenex.gelu", timed_alone(lambda: ops.activate(zf, "gelu_erf", in_place=True), flush), T * I * 3 // 2 * 4)
        gu = torch.randn(T, 2 * I, device=dev).to(bf)
        put(f"{phase}.qwen3.silu_mul", timed_alone(lambda: ops.silu_mul(gu), flush), T * I * 6)
        # --- lightning: activation of q, k, v, the recurrence, the joint norm with its gate
        rp = (torch.randn(T, nh * 4 * d, device=dev) * 0.3).to(bf)
        put(f"{phase}.mukenex.silu_qkv", timed_alone(lambda: ops.activate(rp, "silu", columns=nh * 3 * d, in_place=True),
                                                     flush), T * nh * 3 * d * 4)
        rstate = torch.zeros(rows_dec + 1, nh, d, d, device=dev)
        decay = torch.full((nh,), 0.99, device=dev)
        us = timed_alone(lambda: ops.retention(rp, rstate, decay, None, 0, 1.0, c, nh, d, d), flush,
                         repeats=3 if phase == "prefill" else 7)
        if phase == "prefill":
            put("prefill.mukenex.retention", us, flops=4.0 * T * nh * d * d, of="fp32")
        else:
            put("decode.mukenex.retention", us, rows_dec * nh * d * d * 8)
        ro = torch.randn(T, nh * d, device=dev)
        nw = torch.ones(nh * d, device=dev)
        put(f"{phase}.mukenex.row_norm_gate", timed_alone(lambda: ops.row_norm_gate(ro, nw, rp, nh * 3 * d, 1e-5), flush),
            T * nh * d * 8)
        # --- experts beside Qwen3's feed-forward with the same active parameters
        xe = torch.randn(T, W, device=dev).to(bf)
        ids = torch.randint(0, 4096, (T,), device=dev, dtype=torch.int32)
        table = torch.stack([torch.randperm(E)[:top] for _ in range(4096)]).to(torch.int32).to(dev)
        gate_up = (torch.randn(E, 2 * ffe, W, device=dev) * W ** -0.5).to(bf)
        down = (torch.randn(E, W, ffe, device=dev) * ffe ** -0.5).to(bf)
        fl = 6.0 * T * top * W * ffe
        us = timed_alone(lambda: ops.table_experts(xe, ids, table, gate_up, down), flush)
        if phase == "prefill":
            put("prefill.mukenex.table_experts", us, flops=fl, of="bf16")
        else:
            put("decode.mukenex.table_experts", us, min(E, T * top) * 3 * W * ffe * 2)
        wgu = (torch.randn(2 * I, W, device=dev) * W ** -0.5).to(bf)
        wdn = (torch.randn(W, I, device=dev) * I ** -0.5).to(bf)
        us = timed_alone(lambda: ops.linear(ops.silu_mul(ops.linear(xe, wgu)), wdn), flush)
        if phase == "prefill":
            put("prefill.qwen3.feed_forward", us, flops=6.0 * T * W * I, of="bf16")
        else:
            put("decode.qwen3.feed_forward", us, 3 * W * I * 2)
    return out


# ----------------------------------------------------------------------------- --design torinex
TORINEX_EXPERTS = dict(experts=16, top=4, groups=4, keep=2)


def torinex_config(size, layers):
    """Attention layers over blocks of 1,024 positions; every second layer reads the keys and values of the layer
    before it; dense feed-forwards of 1.5 x Qwen3's intermediate size (two matrices with the parameters of Qwen3's
    three) in turn with 16 routed experts (4 a token out of 2 of 4 groups) and a shared expert which together take a
    token through as many parameters as Qwen3's feed-forward; a per-layer token input 64 wide."""
    z = DESIGN_SIZES[size]
    I = z["inter"]

    def layer(i):
        mixer = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["head_dim"], "vdim": z["head_dim"],
                 "scale": z["head_dim"] ** -0.5, "mask": {"size": 1024}, "rot": {"base": 1e6, "dims": z["head_dim"]}}
        if i % 2 == 1:
            mixer["kv_from"] = i - 1
        r = TORINEX_EXPERTS
        mlp = {"kind": "dense", "ff": I * 3 // 2} if i % 2 == 0 else {
            "kind": "moe", "expert": {"ff": I // 8, "limit": 7.0}, "shared": {"ff": I // 2, "limit": 7.0},
            "router": {"experts": r["experts"], "top": r["top"], "groups": {"count": r["groups"], "keep": r["keep"]}}}
        return {"type": "attention", "mixer": mixer, "mlp": mlp}

    return {"architecture": "Torinex", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5},
            "token_side": {"dim": 64}, "layers": [layer(i) for i in range(layers)]}


def torinex_kernel_table(size, peak):
    """Every kernel of Torinex alone, beside the like kernel of Qwen3's path (and of Mukenex's experts, the closest
    routed feed-forward), at one layer's sizes: a prompt portion of 2,048 tokens and a decode step of 8 rows at 2,048
    tokens (``frac`` as in ``kernel_table``)."""
    import types
    import torch
    from llm_infer_rust_b200.kernels import ops
    from llm_infer_rust_b200.parts.attention import decode_splits
    z = DESIGN_SIZES[size]
    W, nh, nkv, d, I = z["width"], z["heads"], z["kv_heads"], z["head_dim"], z["inter"]
    r = TORINEX_EXPERTS
    E, top, groups, keep, ffe, side, block = r["experts"], r["top"], r["groups"], r["keep"], I // 8, 64, 1024
    dev, bf = torch.device("cuda"), torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    page, ctx_len, rows_dec = 16, 2048, 8
    out = {}

    def put(name, us, nbytes=None, flops=None, of="hbm"):
        rec = {"us": round(us, 2)}
        if nbytes is not None:
            rec["gb_s"] = round(nbytes / us / 1e3, 1)
            rec["frac"] = round(nbytes / us / 1e3 / peak["hbm_gbs"], 3)
        if flops is not None:
            rec["tflops"] = round(flops / us / 1e6, 2)
            rec["frac"] = round(flops / us / 1e6 / peak["bf16_tflops"], 3)
            rec["of"] = of
        out[name] = rec

    def step(rows):
        cu, pos = [0], []
        for prefix, n in rows:
            cu.append(cu[-1] + n)
            pos += list(range(prefix, prefix + n))
        R = len(rows)
        width = -(-max(p + n for p, n in rows) // page)
        table = torch.arange(1, R * width + 1, dtype=torch.int32, device=dev).view(R, width).contiguous()
        slots = [int(table[r_, (p + i) // page]) * page + (p + i) % page for r_, (p, n) in enumerate(rows) for i in range(n)]
        return types.SimpleNamespace(
            num_rows=R, cu_q=i32(cu), positions=i32(pos), prefix_len=i32([p for p, _ in rows]),
            kv_len=i32([p + n for p, n in rows]), slots=i32(slots), table=table, rows=i32(list(range(R))),
            tokens=cu[-1], pages=R * width + 1)

    for phase, c in (("prefill", step([(0, ctx_len)])), ("decode", step([(ctx_len - 1, 1)] * rows_dec))):
        T = c.tokens
        # --- the residual: a sublayer's output normed and added into the float stream, rounded for the next product
        stream = torch.randn(T, W, device=dev)
        y = torch.randn(T, W, device=dev).to(bf)
        wn, ob = torch.ones(W, device=dev), torch.zeros(W, device=dev)
        put(f"{phase}.torinex.norm_add", timed_alone(lambda: ops.norm_add(stream, y, wn, 1e-5, bias=ob, cast_to=bf), flush),
            T * W * 12)
        res_b, xb = torch.randn(T, W, device=dev).to(bf), torch.randn(T, W, device=dev).to(bf)
        wb = torch.ones(W, dtype=bf, device=dev)
        put(f"{phase}.qwen3.add_rms_norm", timed_alone(lambda: ops.add_rms_norm(xb, res_b, wb, 1e-6), flush), T * W * 8)
        # --- between the projection and attention: bias, one norm over all of q and one over all of k, rotation, store
        cq = (nh + 2 * nkv) * d
        packed = (torch.randn(T, cq, device=dev) * 0.5).to(bf)
        k_cache = torch.zeros(c.pages, nkv, page, d, dtype=bf, device=dev).normal_()
        v_cache = torch.zeros(c.pages, nkv, page, d, dtype=bf, device=dev).normal_()
        q = torch.empty(T, nh * d, dtype=bf, device=dev)
        bias, qw, kw = torch.zeros(cq, device=dev), torch.ones(nh * d, device=dev), torch.ones(nkv * d, device=dev)
        inv_freq = torch.pow(torch.tensor(1e6), -torch.arange(0, d, 2) / d).to(dev)
        put(f"{phase}.torinex.joint_heads_prepare", timed_alone(lambda: ops.joint_heads_prepare(
            packed, q, k_cache, v_cache, c.positions, c.slots, nh, nkv, d, d, bias=bias, q_weight=qw, k_weight=kw,
            eps=1e-5, inv_freq=inv_freq, rot_dims=d, interleaved=True), flush), T * cq * 4)
        q_only = packed[:, :nh * d].contiguous()
        put(f"{phase}.torinex.joint_heads_prepare_q", timed_alone(lambda: ops.joint_heads_prepare(
            q_only, q, None, None, c.positions, None, nh, nkv, d, d, bias=bias[:nh * d], q_weight=qw, k_weight=None,
            eps=1e-5, inv_freq=inv_freq, rot_dims=d, interleaved=True, has_kv=False), flush), T * nh * d * 4)
        cos, sin = torch.ones(4096, d // 2, device=dev), torch.zeros(4096, d // 2, device=dev)
        hn = torch.ones(d, dtype=bf, device=dev)
        put(f"{phase}.qwen3.qkv_post", timed_alone(lambda: ops.qkv_post(
            packed, q, k_cache, v_cache, hn, hn, 1e-6, cos, sin, d, c.positions, c.slots, nh, nkv, d), flush), T * cq * 4)
        # --- attention over blocks of positions with one added to the denominator
        o = torch.empty(T, nh * d, dtype=bf, device=dev)
        sinks = torch.zeros(nh, device=dev)
        if phase == "prefill":
            pairs_seen = sum(p % block + 1 for p in range(T))
            put("prefill.torinex.attention_blocks_sink", timed_alone(lambda: ops.prefill_attention(
                q, k_cache, v_cache, o, c.table, c.cu_q, c.kv_len, c.prefix_len, c.rows, 1, T, nh, nkv, d, page, None,
                d ** -0.5, v_head_dim=d, precise_weights=True, chunk=block, sinks=sinks), flush, repeats=3),
                flops=4.0 * nh * d * pairs_seen, of="bf16")
            put("prefill.qwen3.attention", timed_alone(lambda: ops.prefill_attention(
                q, k_cache, v_cache, o, c.table, c.cu_q, c.kv_len, c.prefix_len, c.rows, 1, T, nh, nkv, d, page, None,
                d ** -0.5), flush), flops=4.0 * nh * d * T * (T + 1) / 2, of="bf16")
        else:
            def decode(name, bound, nbytes, **kw):
                per_split = ops.decode_ctas_per_split(bf, rows_dec, nh, nkv, d, page, True)
                splits = decode_splits(per_split, bound, 148)
                need = ops.decode_scratch_floats(rows_dec, nh, d, splits)
                scratch = torch.empty(max(need, 1), device=dev)
                put(name, timed_alone(lambda: ops.decode_attention(
                    q, k_cache, v_cache, o, scratch, c.table, c.cu_q, c.kv_len, c.rows, rows_dec, nh, nkv, d, page,
                    None, d ** -0.5, splits, **kw), flush), nbytes)
            decode("decode.torinex.attention_blocks_sink", block, rows_dec * block * nkv * d * 2 * 2,
                   v_head_dim=d, precise_weights=True, chunk=block, sinks=sinks)
            decode("decode.qwen3.attention", ctx_len, rows_dec * ctx_len * nkv * d * 2 * 2)
        # --- activations
        zf = torch.randn(T, I * 3 // 2, device=dev).to(bf)
        put(f"{phase}.torinex.relu_squared", timed_alone(lambda: ops.activate(zf, "relu_squared", in_place=True), flush),
            T * I * 3 // 2 * 4)
        gs = torch.randn(T, I, device=dev).to(bf)                   # the shared expert's gate and up columns
        put(f"{phase}.torinex.glu_clamped_swish", timed_alone(lambda: ops.glu_columns(gs, "clamped_swish", 7.0, 1.702), flush),
            T * I // 2 * 6)
        gu = torch.randn(T, 2 * I, device=dev).to(bf)
        put(f"{phase}.qwen3.silu_mul", timed_alone(lambda: ops.silu_mul(gu), flush), T * I * 6)
        # --- the per-layer token input: the gate on a row of the second table
        zs = torch.randn(T, side, device=dev).to(bf)
        table2 = torch.randn(4096, 8 * side, device=dev).to(bf)
        ids = torch.randint(0, 4096, (T,), device=dev, dtype=torch.int32)
        put(f"{phase}.torinex.act_table_mul", timed_alone(lambda: ops.act_table_mul(zs, "gelu_tanh", table2, ids, 3 * side),
                                                          flush), T * side * 6)
        if phase == "decode":                                      # the whole read in one kernel for a step of few tokens
            sg = (torch.randn(side, W, device=dev) * W ** -0.5).to(bf)
            sp = torch.randn(W, side, device=dev).to(bf)
            xs = stream.to(bf)
            put("decode.torinex.token_side_few", timed_alone(lambda: ops.token_side_few(
                stream, xs, sg, table2, ids, 3 * side, sp, wn, 1e-5, "gelu_tanh", cast_to=bf), flush),
                2 * side * W * 2 + T * W * 14)
        # --- router and experts beside Mukenex's experts and Qwen3's feed-forward with the same active parameters
        xe = torch.randn(T, W, device=dev).to(bf)
        wr = (torch.randn(E, W, device=dev) * W ** -0.5).to(bf)
        put(f"{phase}.torinex.expert_router", timed_alone(lambda: ops.expert_router(xe, wr, top, groups, keep), flush),
            T * W * 2 + E * W * 2 + T * top * 8)
        choice, gains = ops.expert_router(xe, wr, top, groups, keep)
        gate_up = (torch.randn(E, 2 * ffe, W, device=dev) * W ** -0.5).to(bf)
        down = (torch.randn(E, W, ffe, device=dev) * ffe ** -0.5).to(bf)
        share = torch.randn(T, W, device=dev).to(bf)
        us = timed_alone(lambda: ops.routed_experts(xe, choice, gains, gate_up, down, "clamped_swish", 7.0, 1.702,
                                                    add=share), flush)
        used = int(torch.unique(choice).numel())
        if phase == "prefill":
            put("prefill.torinex.routed_experts", us, flops=6.0 * T * top * W * ffe, of="bf16")
        else:
            put("decode.torinex.routed_experts", us, used * 3 * W * ffe * 2)
        E2, top2, ffe2 = 8, 2, I // 4                               # Mukenex's experts at the same active parameters
        tbl = torch.stack([torch.randperm(E2)[:top2] for _ in range(4096)]).to(torch.int32).to(dev)
        gate_up2 = (torch.randn(E2, 2 * ffe2, W, device=dev) * W ** -0.5).to(bf)
        down2 = (torch.randn(E2, W, ffe2, device=dev) * ffe2 ** -0.5).to(bf)
        us = timed_alone(lambda: ops.table_experts(xe, ids, tbl, gate_up2, down2), flush)
        if phase == "prefill":
            put("prefill.mukenex.table_experts", us, flops=6.0 * T * top2 * W * ffe2, of="bf16")
        else:
            put("decode.mukenex.table_experts", us, min(E2, T * top2) * 3 * W * ffe2 * 2)
        wgu = (torch.randn(2 * I, W, device=dev) * W ** -0.5).to(bf)
        wdn = (torch.randn(W, I, device=dev) * I ** -0.5).to(bf)
        us = timed_alone(lambda: ops.linear(ops.silu_mul(ops.linear(xe, wgu)), wdn), flush)
        if phase == "prefill":
            put("prefill.qwen3.feed_forward", us, flops=6.0 * T * W * I, of="bf16")
        else:
            put("decode.qwen3.feed_forward", us, 3 * W * I * 2)
    return out


# ----------------------------------------------------------------------------- --design lufizen
LUFIZEN_EXPERTS = dict(experts=16, top=4, groups=4, keep=2)


def lufizen_ranks(size):
    """(kv_rank, q_rank, rot_dim) of the latent layers: the key rows (kv_rank + rot_dim) stay within the attention
    kernels' 512 columns."""
    W = DESIGN_SIZES[size]["width"]
    return (256, 768, 64) if W <= 1024 else (384, 1536, 64)


def lufizen_config(size, layers):
    """Three attention layers (values that are the projected keys, a rotation of half of every head with stretched
    frequencies, learned sinks) and then a latent-attention layer (queries through a latent, a gate a head), in turn;
    every layer with 16 routed experts (4 a token out of 2 of 4 groups, each an eighth of Qwen3's intermediate size)
    and a gated shared expert of half that size: together the active parameters of Qwen3's feed-forward."""
    z = DESIGN_SIZES[size]
    H, G, d, I = z["heads"], z["kv_heads"], z["head_dim"], z["inter"]
    rank, q_rank, r = lufizen_ranks(size)
    e = LUFIZEN_EXPERTS
    mlp = {"kind": "moe", "expert": {"ff": I // 8}, "shared": {"ff": I // 2},
           "router": {"experts": e["experts"], "top": e["top"], "scale": 1.75,
                      "groups": {"count": e["groups"], "keep": e["keep"]}}}
    attn = {"type": "attention", "mlp": mlp,
            "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5,
                      "rot": {"base": 1e6, "dims": d // 2,
                              "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    latent = {"type": "latent_attention", "mlp": mlp,
              "mixer": {"heads": H, "dim": d, "rot_dim": r, "vdim": d, "kv_rank": rank, "q_rank": q_rank,
                        "scale": (d + r) ** -0.5, "rot": {"base": 1e6, "dims": r}}}
    return {"architecture": "Lufizen", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5},
            "embedding": {"scale": 8.0}, "logit_scale": 0.25,
            "layers": [latent if i % 4 == 2 else attn for i in range(layers)]}


def lufizen_kernel_table(size, peak):
    """Every kernel of Lufizen alone, beside the like kernel of the closest designs (Torinex's prepare kernel, attention
    with a sink, router and experts; Mukenex's latent attention; Qwen3's where there is no closer one), at one layer's
    sizes: a prompt portion of 2,048 tokens and a decode step of 8 rows at 2,048 tokens (``frac`` as in
    ``kernel_table``)."""
    import types
    import torch
    from llm_infer_rust_b200.kernels import ops
    from llm_infer_rust_b200.parts.attention import decode_splits
    z = DESIGN_SIZES[size]
    W, nh, nkv, d, I = z["width"], z["heads"], z["kv_heads"], z["head_dim"], z["inter"]
    rank, q_rank, r = lufizen_ranks(size)
    e = LUFIZEN_EXPERTS
    E, top, groups, keep, ffe = e["experts"], e["top"], e["groups"], e["keep"], I // 8
    dev, bf = torch.device("cuda"), torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    page, ctx_len, rows_dec = 16, 2048, 8
    out = {}

    def put(name, us, nbytes=None, flops=None, of="hbm"):
        rec = {"us": round(us, 2)}
        if nbytes is not None:
            rec["gb_s"] = round(nbytes / us / 1e3, 1)
            rec["frac"] = round(nbytes / us / 1e3 / peak["hbm_gbs"], 3)
        if flops is not None:
            rec["tflops"] = round(flops / us / 1e6, 2)
            rec["frac"] = round(flops / us / 1e6 / peak["bf16_tflops"], 3)
            rec["of"] = of
        out[name] = rec

    def step(rows):
        cu, pos = [0], []
        for prefix, n in rows:
            cu.append(cu[-1] + n)
            pos += list(range(prefix, prefix + n))
        R = len(rows)
        width = -(-max(p + n for p, n in rows) // page)
        table = torch.arange(1, R * width + 1, dtype=torch.int32, device=dev).view(R, width).contiguous()
        slots = [int(table[r_, (p + i) // page]) * page + (p + i) % page for r_, (p, n) in enumerate(rows) for i in range(n)]
        return types.SimpleNamespace(
            num_rows=R, cu_q=i32(cu), positions=i32(pos), prefix_len=i32([p for p, _ in rows]),
            kv_len=i32([p + n for p, n in rows]), slots=i32(slots), table=table, rows=i32(list(range(R))),
            tokens=cu[-1], pages=R * width + 1)

    for phase, c in (("prefill", step([(0, ctx_len)])), ("decode", step([(ctx_len - 1, 1)] * rows_dec))):
        T = c.tokens
        # --- between the projection and attention: rotation, a plain norm a head, the projected key kept as the value
        cq = (nh + nkv) * d
        packed = (torch.randn(T, cq, device=dev) * 0.5).to(bf)
        k_cache = torch.zeros(c.pages, nkv, page, d, dtype=bf, device=dev).normal_()
        v_cache = torch.zeros(c.pages, nkv, page, d, dtype=bf, device=dev).normal_()
        q = torch.empty(T, nh * d, dtype=bf, device=dev)
        inv_half = torch.pow(torch.tensor(1e6), -torch.arange(0, d // 2, 2) / (d // 2)).to(dev)
        moved = T * (cq * 2 + (nh + 2 * nkv) * d * 2)
        put(f"{phase}.lufizen.heads_prepare", timed_alone(lambda: ops.heads_prepare(
            packed, q, k_cache, v_cache, c.positions, c.slots, nh, nkv, d, d, eps=1e-5, inv_freq=inv_half,
            rot_dims=d // 2, interleaved=False, plain_norm=True, norm_after_rotation=True, values_are_keys=True),
            flush), moved)
        cq3 = (nh + 2 * nkv) * d
        packed3 = (torch.randn(T, cq3, device=dev) * 0.5).to(bf)
        bias, qw, kw = torch.zeros(cq3, device=dev), torch.ones(nh * d, device=dev), torch.ones(nkv * d, device=dev)
        inv_freq = torch.pow(torch.tensor(1e6), -torch.arange(0, d, 2) / d).to(dev)
        put(f"{phase}.torinex.joint_heads_prepare", timed_alone(lambda: ops.joint_heads_prepare(
            packed3, q, k_cache, v_cache, c.positions, c.slots, nh, nkv, d, d, bias=bias, q_weight=qw, k_weight=kw,
            eps=1e-5, inv_freq=inv_freq, rot_dims=d, interleaved=True), flush), T * cq3 * 4)
        cos, sin = torch.ones(4096, d // 2, device=dev), torch.zeros(4096, d // 2, device=dev)
        hn = torch.ones(d, dtype=bf, device=dev)
        put(f"{phase}.qwen3.qkv_post", timed_alone(lambda: ops.qkv_post(
            packed3, q, k_cache, v_cache, hn, hn, 1e-6, cos, sin, d, c.positions, c.slots, nh, nkv, d), flush), T * cq3 * 4)
        # --- the latent layer: the query latent's norm, the heads' small products, the prepare kernel
        lq = nh * (d + r)
        first = (torch.randn(T, q_rank + rank + r + nh, device=dev) * 0.5).to(bf)
        qn = torch.ones(q_rank, device=dev)
        put(f"{phase}.lufizen.columns_rms_norm", timed_alone(lambda: ops.columns_rms_norm(first, q_rank, qn, 1e-5), flush),
            T * q_rank * 4)
        xq = torch.randn(T, q_rank, device=dev).to(bf)
        wq = torch.ones(q_rank, dtype=bf, device=dev)
        put(f"{phase}.qwen3.rms_norm", timed_alone(lambda: ops.rms_norm(xq, wq, 1e-6), flush), T * q_rank * 4)
        queries = (torch.randn(T, lq, device=dev) * 0.5).to(bf)
        lk = torch.zeros(c.pages, 1, page, rank + r, dtype=bf, device=dev).normal_()
        uk_t = (torch.randn(nh, rank, d, device=dev) * d ** -0.5).to(bf)
        uv = (torch.randn(nh, d, rank, device=dev) * rank ** -0.5).to(bf)
        q_plain = queries.view(T, nh, d + r)[:, :, :d].transpose(0, 1)
        q_lat = ops.head_products(q_plain, uk_t)
        put(f"{phase}.lufizen.head_products_uk", timed_alone(lambda: ops.head_products(q_plain, uk_t), flush),
            flops=2.0 * T * nh * d * rank, of="bf16")
        lqo = torch.empty(T, nh * (rank + r), dtype=bf, device=dev)
        inv_r = torch.pow(torch.tensor(1e6), -torch.arange(0, r, 2) / r).to(dev)
        lw = torch.ones(rank, device=dev)
        put(f"{phase}.lufizen.latent_prepare", timed_alone(lambda: ops.latent_prepare(
            queries, q_lat, lqo, lk, None, lw, 1e-5, c.positions, c.slots, nh, d, r, rank, inv_freq=inv_r, rot_dims=r,
            down=first[:, q_rank:]), flush), T * (nh * (rank * 2 + r * 2) * 2 + (rank + r) * 2 * 2))
        # --- attention: every earlier key with a learned sink; the latent's rows without one
        o = torch.empty(T, nh * d, dtype=bf, device=dev)
        lo = torch.empty(T, nh * rank, dtype=bf, device=dev)
        sinks = torch.randn(nh, device=dev)
        pairs_all = T * (T + 1) / 2
        window = 1024                                              # Mukenex's latent layers read a window of that many
        if phase == "prefill":
            put("prefill.lufizen.attention_sink", timed_alone(lambda: ops.prefill_attention(
                q, k_cache, v_cache, o, c.table, c.cu_q, c.kv_len, c.prefix_len, c.rows, 1, T, nh, nkv, d, page, None,
                d ** -0.5, v_head_dim=d, precise_weights=True, sinks=sinks), flush, repeats=3),
                flops=4.0 * nh * d * pairs_all, of="bf16")
            put("prefill.torinex.attention_blocks_sink", timed_alone(lambda: ops.prefill_attention(
                q, k_cache, v_cache, o, c.table, c.cu_q, c.kv_len, c.prefix_len, c.rows, 1, T, nh, nkv, d, page, None,
                d ** -0.5, v_head_dim=d, precise_weights=True, chunk=window, sinks=sinks), flush, repeats=3),
                flops=4.0 * nh * d * sum(p % window + 1 for p in range(T)), of="bf16")
            put("prefill.qwen3.attention", timed_alone(lambda: ops.prefill_attention(
                q, k_cache, v_cache, o, c.table, c.cu_q, c.kv_len, c.prefix_len, c.rows, 1, T, nh, nkv, d, page, None,
                d ** -0.5), flush), flops=4.0 * nh * d * pairs_all, of="bf16")
            put("prefill.lufizen.attention_latent", timed_alone(lambda: ops.prefill_attention(
                lqo, lk, None, lo, c.table, c.cu_q, c.kv_len, c.prefix_len, c.rows, 1, T, nh, 1, rank + r, page, None,
                (d + r) ** -0.5, v_head_dim=rank, precise_weights=True, shared_values=True), flush, repeats=3),
                flops=2.0 * nh * (2 * rank + r) * pairs_all, of="bf16")
            put("prefill.mukenex.attention_latent", timed_alone(lambda: ops.prefill_attention(
                lqo, lk, None, lo, c.table, c.cu_q, c.kv_len, c.prefix_len, c.rows, 1, T, nh, 1, rank + r, page, window,
                (d + r) ** -0.5, v_head_dim=rank, precise_weights=True, sinks=sinks, shared_values=True), flush, repeats=3),
                flops=2.0 * nh * (2 * rank + r) * sum(min(p, window - 1) + 1 for p in range(T)), of="bf16")
        else:
            def decode(name, qq, kk, vv, oo, heads, kvh, dk, dv_, bound, nbytes, **kw):
                plain = dk == dv_
                per_split = ops.decode_ctas_per_split(bf, rows_dec, heads, kvh, dk, page, plain)
                keys = 512
                if kw.get("shared_values"):
                    per_split = rows_dec * (heads // ops.latent_head_group(heads))
                    keys = 128                                     # the engine's rule for latent rows
                splits = decode_splits(per_split, bound, 148, keys)
                need = ops.decode_scratch_floats(rows_dec, heads, max(dk, dv_), splits)
                scratch = torch.empty(max(need, 1), device=dev)
                win, scale = kw.pop("window_", None), kw.pop("scale_", dk ** -0.5)
                put(name, timed_alone(lambda: ops.decode_attention(
                    qq, kk, vv, oo, scratch, c.table, c.cu_q, c.kv_len, c.rows, rows_dec, heads, kvh, dk, page,
                    win, scale, splits, **kw), flush), nbytes)
            kv_all = rows_dec * ctx_len * nkv * d * 2 * 2
            decode("decode.lufizen.attention_sink", q, k_cache, v_cache, o, nh, nkv, d, d, ctx_len, kv_all,
                   v_head_dim=d, precise_weights=True, sinks=sinks)
            decode("decode.torinex.attention_blocks_sink", q, k_cache, v_cache, o, nh, nkv, d, d, window,
                   rows_dec * window * nkv * d * 2 * 2, v_head_dim=d, precise_weights=True, chunk=window, sinks=sinks)
            decode("decode.qwen3.attention", q, k_cache, v_cache, o, nh, nkv, d, d, ctx_len, kv_all)
            decode("decode.lufizen.attention_latent", lqo, lk, None, lo, nh, 1, rank + r, rank, ctx_len,
                   rows_dec * ctx_len * (rank + r) * 2, v_head_dim=rank, precise_weights=True, shared_values=True)
            decode("decode.mukenex.attention_latent", lqo, lk, None, lo, nh, 1, rank + r, rank, window,
                   rows_dec * window * (rank + r) * 2, v_head_dim=rank, precise_weights=True, sinks=sinks,
                   window_=window, shared_values=True)
        lo_t = lo.view(T, nh, rank).transpose(0, 1)
        lout = torch.empty(T, nh * d, dtype=bf, device=dev)
        put(f"{phase}.lufizen.head_products_uv", timed_alone(lambda: ops.head_products(
            lo_t, uv, out=lout.view(T, nh, d).transpose(0, 1)), flush), flops=2.0 * T * nh * d * rank, of="bf16")
        # --- the gate: one a head, beside one a column
        put(f"{phase}.lufizen.head_gate_mul", timed_alone(lambda: ops.sigmoid_gate_mul(
            lout, first, q_rank + rank + r, per=d), flush), T * nh * d * 4)
        gp = (torch.randn(T, 2 * nh * d, device=dev)).to(bf)
        put(f"{phase}.mukenex.sigmoid_gate_mul", timed_alone(lambda: ops.sigmoid_gate_mul(o, gp, nh * d), flush), T * nh * d * 6)
        # --- the residual (Torinex's kernel, unchanged) and the factor on the logits
        stream = torch.randn(T, W, device=dev)
        y = torch.randn(T, W, device=dev).to(bf)
        wn = torch.ones(W, device=dev)
        put(f"{phase}.lufizen.norm_add", timed_alone(lambda: ops.norm_add(stream, y, wn, 1e-5, cast_to=bf), flush), T * W * 12)
        if phase == "decode":
            lg = torch.randn(rows_dec, z["vocab"], device=dev)
            put("decode.lufizen.scale_logits", timed_alone(lambda: ops.scale_floats(lg, 0.25), flush), rows_dec * z["vocab"] * 8)
        # --- router and experts beside Torinex's and Qwen3's feed-forward with the same active parameters
        xe = torch.randn(T, W, device=dev).to(bf)
        wr = (torch.randn(E, W, device=dev) * W ** -0.5).to(bf)
        sg = (torch.randn(1, W, device=dev) * W ** -0.5).to(bf)
        corr = torch.randn(E, device=dev) * 0.1
        route = lambda: ops.expert_router(xe, wr, top, groups, keep, "sigmoid", False, correction=corr, group_members=2,
                                          gain_scale=1.75, gate=sg)
        put(f"{phase}.lufizen.expert_router", timed_alone(route, flush), T * W * 2 + (E + 1) * W * 2 + T * (top * 8 + 4))
        put(f"{phase}.torinex.expert_router", timed_alone(lambda: ops.expert_router(xe, wr, top, groups, keep), flush),
            T * W * 2 + E * W * 2 + T * top * 8)
        choice, gains, share_gate = route()
        gate_up = (torch.randn(E, 2 * ffe, W, device=dev) * W ** -0.5).to(bf)
        down = (torch.randn(E, W, ffe, device=dev) * ffe ** -0.5).to(bf)
        share = torch.randn(T, W, device=dev).to(bf)
        used = int(torch.unique(choice).numel())
        for name, fn in (("lufizen", lambda: ops.routed_experts(xe, choice, gains, gate_up, down, "silu", add=share,
                                                               add_scale=share_gate)),
                         ("torinex", lambda: ops.routed_experts(xe, choice, gains, gate_up, down, "clamped_swish", 7.0,
                                                               1.702, add=share))):
            us = timed_alone(fn, flush)
            if phase == "prefill":
                put(f"prefill.{name}.routed_experts", us, flops=6.0 * T * top * W * ffe, of="bf16")
            else:
                put(f"decode.{name}.routed_experts", us, used * 3 * W * ffe * 2)
        gs = torch.randn(T, I, device=dev).to(bf)                   # the shared expert's gate and up columns
        put(f"{phase}.lufizen.glu_silu", timed_alone(lambda: ops.glu_columns(gs, "silu"), flush), T * I // 2 * 6)
        put(f"{phase}.torinex.glu_clamped_swish", timed_alone(lambda: ops.glu_columns(gs, "clamped_swish", 7.0, 1.702), flush),
            T * I // 2 * 6)
        wgu = (torch.randn(2 * I, W, device=dev) * W ** -0.5).to(bf)
        wdn = (torch.randn(W, I, device=dev) * I ** -0.5).to(bf)
        us = timed_alone(lambda: ops.linear(ops.silu_mul(ops.linear(xe, wgu)), wdn), flush)
        if phase == "prefill":
            put("prefill.qwen3.feed_forward", us, flops=6.0 * T * W * I, of="bf16")
        else:
            put("decode.qwen3.feed_forward", us, 3 * W * I * 2)
    return out


DESIGNS = {"kefetar": (kefetar_config, kernel_table), "mukenex": (mukenex_config, mukenex_kernel_table),
           "torinex": (torinex_config, torinex_kernel_table), "lufizen": (lufizen_config, lufizen_kernel_table)}
# The closest earlier design, which stands beside the new one and Qwen3 at equal sizes.
BESIDE = {"lufizen": ("torinex", torinex_config)}


def design_main(args) -> int:
    import torch
    peak, peak_source = peaks()
    # float32 FMA throughput of the device: SMs x 128 lanes x 2 x the highest SM clock
    props = torch.cuda.get_device_properties(0)
    peak["fp32_tflops"] = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12
    make_config, make_table = DESIGNS[args.design]
    context, line = args.context, {"design": args.design, "layers": args.layers or 8, "context": args.context,
                                   "dtype": "bf16", "data": "synthetic token ids, random weights", "peaks": peak_source,
                                   "sizes": {}, "kernels": {}}
    for size in [n for n in args.design_sizes.split(",") if n]:
        rec = {}
        arms = [(args.design, make_config(size, args.layers or 8))]
        if args.design in BESIDE:
            arms.append((BESIDE[args.design][0], BESIDE[args.design][1](size, args.layers or 8)))
        arms.append(("qwen3", qwen3_config(size, args.layers or 8)))
        for name, raw in arms:
            engine = design_engine(raw, 8, context)
            vocab = raw.get("vocab", raw.get("vocab_size"))
            ms = prefill_timed(engine, 2048, vocab)
            one = {"params_m": round(engine.model.parameter_bytes() / 2e6, 1), "prefill_tok_s": round(2048e3 / ms, 1),
                   "prefill_ms": round(ms, 3)}
            for b in (1, 8):
                run = decode_device_timed(engine, b, context, max(8, args.steps // 4), args.warmup, vocab)
                one[f"decode_b{b}_tok_s"] = round(run["tokens_per_s"], 1)
                one[f"decode_b{b}_ms"] = round(run["ms_per_step"], 4)
                one[f"decode_b{b}_launches_per_step"] = run["launches"] // max(8, args.steps // 4)
            rec[name] = one
            del engine
            release()
        line["sizes"][size] = rec
        if not args.no_kernels:
            line["kernels"][size] = make_table(size, peak)
            release()
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="0.6b", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the shape has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--no-points", action="store_true", help="only the headline shape at the headline batch")
    ap.add_argument("--point-shapes", default="8b,32b",
                    help="other shapes measured into `points` (decode at batch 1 / 8 / 64, prefill), comma separated")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one phase alone and print a short line (for profiling)")
    ap.add_argument("--design", choices=["qwen3", "kefetar", "mukenex", "torinex", "lufizen"], default="qwen3",
                    help="kefetar, mukenex, torinex, lufizen: that design beside Qwen3 at equal sizes, and its kernels alone (another line)")
    ap.add_argument("--design-sizes", default="1k,4k", help="layer sizes of --design kefetar / mukenex / torinex / lufizen, comma separated")
    ap.add_argument("--no-kernels", action="store_true", help="--design ... without the table of single kernels")
    args = ap.parse_args()
    if args.design in DESIGNS and args.impl == "ours":
        if args.gpus != 1:
            print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
            return 2
        args.warmup = max(args.warmup, 3)
        if args.context == 4096:
            args.context = 2048
        return design_main(args)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    biggest = args.batch if (args.no_points or args.only) else max(64, args.batch)
    engine, raw, full_layers = build_engine(args.shape, args.layers, biggest, args.context)
    vocab = raw["vocab_size"]
    numbers = model_numbers(raw)
    peak, peak_source = peaks()

    if args.only == "decode":
        run = decode_device_timed(engine, args.batch, args.context, args.steps, args.warmup, vocab)
        print(json.dumps({"only": "decode", "batch": args.batch, **{k: round(v, 4) for k, v in run.items()}}))
        return 0
    if args.only == "prefill":
        ms = prefill_timed(engine, 2048, vocab, repeats=max(1, args.steps))
        print(json.dumps({"only": "prefill", "tokens": 2048, "ms": round(ms, 3)}))
        return 0
    prefill_ms = prefill_timed(engine, 2048, vocab)
    flops = prefill_flops(raw, 2048)
    points = {}

    def fraction(batch, run):
        return round(step_bytes(numbers, batch, run["mean_context"]) / (run["ms_per_step"] * 1e-3) / 1e9 / peak["hbm_gbs"], 4)

    if not args.no_points:
        for b in (1, 64):
            run = decode_device_timed(engine, b, args.context, args.steps, args.warmup, vocab)
            points[f"decode_b{b}"] = round(run["tokens_per_s"], 1)
            points[f"decode_b{b}_frac"] = fraction(b, run)
        # the same batch at half the context (the decode of a 2,048-token prompt starts there and ends at the headline's)
        half = decode_device_timed(engine, args.batch, args.context // 2, args.steps, args.warmup, vocab)
        points[f"decode_b{args.batch}_c{args.context // 2}"] = round(half["tokens_per_s"], 1)
        points[f"decode_b{args.batch}_c{args.context // 2}_frac"] = fraction(args.batch, half)
    e2e = decode_end_to_end(engine, args.batch, args.context, args.steps, args.warmup, vocab)
    clocks = ClockSampler()
    clocks.start()
    main_run = decode_device_timed(engine, args.batch, args.context, args.steps, args.warmup, vocab)
    clock_record = clocks.stop()
    routing = [f"{args.shape}: {routing_of(engine, args.batch)}"]
    del engine
    release()
    if not args.no_points:
        for name in [n for n in args.point_shapes.split(",") if n and n != args.shape]:
            more, way = measure_point_shape(name, args.context, max(8, args.steps // 4), args.warmup, peak)
            points.update(more)
            routing.append(way)

    achieved = step_bytes(numbers, args.batch, main_run["mean_context"]) / (main_run["ms_per_step"] * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s", "value": round(main_run["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random weights", "impl": "ours",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": raw["num_hidden_layers"],
                   "layers_of_shape": full_layers, "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"],
                   "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"],
                   "intermediate": raw["intermediate_size"], "vocab": vocab, "tied": raw["tie_word_embeddings"],
                   "global_batch": args.batch, "seq_len": args.context,
                   "prompt_len": args.context - args.steps - args.warmup, "page_size": 16,
                   "parallelism": "single GPU", "decode_graphs": True, "prefill_graph": True,
                   "l2": "inputs exceed L2: every step reads all weights and the live cache",
                   "peaks": peak_source},
        "clocks": clock_record,
        "e2e": {"value": round(e2e["tokens_per_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": main_run["launches"],
        "prefill": {"value": round(2048 * 1000.0 / prefill_ms, 1), "tokens": 2048, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
        "routing": "; ".join(routing),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
