"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch B] [--layers L] [--impl ours|reference]

The default run has the layer sizes of Qwen3-4B (BASELINE.json configs[2]) with
random weights in bfloat16, a batch of 8 requests that each hold a 2,048-token
prefix in a cache laid out for 4,096-token contexts with 16-token pages, and
prints one JSON line:

  value     decoded tokens a second, timed on the device: K replays of the captured
            decode step (model + sampling, the sampled token fed back on the device)
            between two CUDA events;
  e2e       the same through Engine.generate(): host token ids in, host token ids
            out, every step's inputs copied from pinned memory and its tokens read back;
  prefill   one 2,048-token prompt through the step function;
  roofline  the bytes a decode step has to read (every weight once, the cache of
            the live requests) over its time, against the measured copy bandwidth;
  points    the device-timed value at batch 1 and 64.

Every decode step reads the whole model (8 GB at full size), far more than the
126 MB L2, so no flush is needed between steps ("l2": "inputs_exceed_l2").

``--workload serving`` measures something else and prints a line of its own: a
mixed continuous batch through Engine.generate() (BASELINE.json configs[3]: 32
requests, prompts of 128 to 2,048 tokens cut into portions of 512 beside the
running decodes, 256 tokens each), as generated tokens a second by the wall clock.
``--workload pabelix`` and ``--workload kolisun`` put that design beside Qwen3 dense at equal
layer sizes (random weights): prefill and decode steps, and the design's kernels beside their
like, each a line of its own; ``--workload nedesun`` and ``--workload pepolorn`` do so beside Kolisun and
Qwen3 dense.
None of them changes the default run or its line.
"""
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

QWEN3_4B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=2560,
                intermediate_size=9728, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, max_position_embeddings=40960, rope_theta=1000000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=True, attention_bias=False, use_sliding_window=False, hidden_act="silu")
# the layer sizes of the other two Qwen3 dense models, for --model-size (the default run is the 4B model)
OTHER_SIZES = {
    "8b": dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, tie_word_embeddings=False),
    "32b": dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                num_key_value_heads=8, head_dim=128, tie_word_embeddings=False),
}
CONTEXT_LEN, PREFIX_LEN, PAGE_SIZE, PREFILL_TOKENS = 4096, 2048, 16, 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
        out = dict(FALLBACK_PEAKS, source="measured")
        for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            v = raw.get(k)
            if isinstance(v, dict):                          # a record around the figure
                v = v.get("value")
            if isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0:
                out[k] = float(v)
        return out
    except (OSError, ValueError, AttributeError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), [p.strip() for p in line.split(",")]))

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows):
        rows = [p for t, p in self.samples if any(a <= t <= b for a, b in windows) and len(p) >= 6]
        if not rows:
            rows = [p for _, p in self.samples if len(p) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        mhz = [int(float(p[0])) for p in rows if p[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for p in rows for n, v in zip(names, p[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None,
                "sm_max_mhz": int(float(rows[0][1])) if rows[0][1].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(rows)}


MODEL = QWEN3_4B            # what --model-size chose


def build_engine(layers, max_running, num_pages, prefill_chunk=0):
    import torch
    from prelude_b200 import Engine
    from prelude_b200.config import load_model_config
    from prelude_b200.engine.loading import build_model
    from prelude_b200.weights.loader import WeightStore
    from prelude_b200.weights.random_init import random_tensors
    cfg = dict(MODEL, num_hidden_layers=layers)
    tensors = random_tensors(cfg, seed=0, std=0.02, norm_jitter=0.05, dtype=torch.bfloat16, device="cuda:0")
    model = build_model(load_model_config(cfg).to_model_spec(), WeightStore.from_tensors(tensors), "bf16", "cuda:0")
    del tensors
    torch.cuda.empty_cache()
    return Engine(model, page_size=PAGE_SIZE, num_pages=num_pages, max_running_requests=max_running,
                  max_num_batched_tokens=max(8192, PREFILL_TOKENS), long_prefill_token_threshold=prefill_chunk,
                  max_model_len=CONTEXT_LEN, cuda_graph=True, cuda_graph_max_bs=64), cfg


def weight_bytes_per_step(cfg):
    """Bytes of weights one decode step reads: every matrix once (the tied
    embedding table once, as the output head), norm scales in float32."""
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    per_layer = 2 * (qkv * H + H * cfg["num_attention_heads"] * cfg["head_dim"] + 3 * I * H) + 4 * (2 * H + 2 * cfg["head_dim"])
    head = 2 * cfg["vocab_size"] * H          # tied or not: the head once; a separate table only at the step's token rows
    return L * per_layer + head + 4 * H


def kv_bytes_per_token(cfg):
    return 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, T):
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    nH, D = cfg["num_attention_heads"], cfg["head_dim"]
    qkv = (nH + 2 * cfg["num_key_value_heads"]) * D
    gemm = 2 * T * L * (qkv * H + H * nH * D + 3 * I * H) + 2 * 1 * cfg["vocab_size"] * H
    attn = L * 4 * nH * D * (T * (T + 1) // 2)          # QK^T and PV over the causal half
    return gemm + attn


def time_decode(engine, cfg, batch, steps, warmup, seed):
    """Device time of ``steps`` decode steps at ``batch`` requests with PREFIX_LEN-token prefixes."""
    import torch
    from prelude_b200.engine.graph import DecodeGraph
    from prelude_b200.engine.runner import StepEntry
    from prelude_b200.ops import library
    runner, cache = engine.runner, engine.cache
    g = torch.Generator().manual_seed(seed)
    rids = [f"bench{seed}_{i}" for i in range(batch)]
    for rid in rids:                                     # real prefill fills the cache
        ids = torch.randint(0, cfg["vocab_size"], (PREFIX_LEN,), generator=g).tolist()
        runner.step([StepEntry(rid, ids, [])], check_status=False)
    total = PREFIX_LEN + warmup + steps + 1
    for rid in rids:                                     # room for every token the loop will write
        cache.grow(rid, total)
    cache.flush_table_updates()
    graph = DecodeGraph(runner, batch, self_feeding=True)
    tokens = torch.randint(0, cfg["vocab_size"], (batch,), generator=g).tolist()
    graph.load(tokens, [PREFIX_LEN] * batch, [cache.slot_of(r) for r in rids], [0.0] * batch, [0] * batch, [0] * batch)
    graph.capture()
    graph.load(tokens, [PREFIX_LEN] * batch, [cache.slot_of(r) for r in rids], [0.0] * batch, [0] * batch, [0] * batch)
    for _ in range(warmup):
        graph.replay()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.time()
    start.record()
    torch.cuda.nvtx.range_push("timed_decode")          # lets a profiler pick these launches out
    for _ in range(steps):
        graph.replay()
    torch.cuda.nvtx.range_pop()
    end.record()
    torch.cuda.synchronize()
    t1 = time.time()
    ms = start.elapsed_time(end)
    status = int(graph.status.item())
    if status != 0:
        raise RuntimeError(f"decode loop raised kernel status {status}")
    if TIMELINE:
        print_timeline(graph)
    for rid in rids:
        runner.finish(rid)
    del graph
    avg_ctx = PREFIX_LEN + warmup + (steps + 1) / 2.0
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches_per_step": None,
            "avg_ctx": avg_ctx, "window": (t0, t1)}, library


TIMELINE = False


def print_timeline(graph):
    """One more replay of the captured step with the kernels' timeline marks on (a library built with
    PRELUDE_TIMELINE=1): for every kernel of the step's second layer, when its first block started, when the kernel
    before it had finished, when its input had arrived and when its first and last block were done, in
    microseconds from the layer's first mark."""
    import torch
    from prelude_b200.ops import timeline
    timeline.enable()
    timeline.reset()
    graph.replay()
    torch.cuda.synchronize()
    marks = timeline.read()
    # a layer begins with the add+norm that precedes the qkv product: cut the step at every second norm entry
    starts = [i for i, m in enumerate(marks) if m.kernel == "add_rmsnorm" and m.mark == "entry" and not m.last_block]
    if len(starts) < 5:
        print(f"timeline: {len(marks)} marks, too few to show a layer", file=sys.stderr)
        return
    lo, hi = starts[2], starts[4]                           # the second layer's two norms and what lies between
    t0 = marks[lo].ns
    print("timeline of one layer of the captured decode step (us from the layer's first mark):", file=sys.stderr)
    for m in marks[lo:hi]:
        print(f"  {(m.ns - t0) / 1e3:8.2f}  {m.kernel:22s} {m.mark:10s} {'last block' if m.last_block else 'first block'}", file=sys.stderr)
    print(f"  {(marks[hi].ns - t0) / 1e3:8.2f}  next layer begins", file=sys.stderr)


def time_prefill(engine, cfg, warmup, reps=3):
    import torch
    from prelude_b200.engine.runner import StepEntry
    runner = engine.runner
    g = torch.Generator().manual_seed(7)
    times = []
    t0 = time.time()
    for i in range(warmup + reps):
        ids = torch.randint(0, cfg["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        if i >= warmup:
            torch.cuda.nvtx.range_push("timed_prefill")
        runner.step([StepEntry(f"prefill{i}", ids, [PREFILL_TOKENS - 1])], check_status=False)
        if i >= warmup:
            torch.cuda.nvtx.range_pop()
        e.record()
        torch.cuda.synchronize()
        runner.finish(f"prefill{i}")
        if i >= warmup:
            times.append(s.elapsed_time(e))
    return min(times), (t0, time.time())


def time_e2e(engine, cfg, batch, steps):
    """Decoded tokens a second through Engine.generate(): after each request's first token."""
    import torch
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg["vocab_size"], (PREFIX_LEN,), generator=g).tolist() for _ in range(batch)]
    # warm up outside the timed call: the decode step is captured per batch size at its first use, and
    # requests that finish a step apart leave smaller batches behind
    engine.warmup(range(1, batch + 1))
    engine.generate([p[:32] for p in prompts], temperature=0.0, max_new_tokens=4, ignore_eos=True)
    import copy
    before = copy.copy(engine.stats())
    t0 = time.time()
    res = engine.generate(prompts, temperature=0.0, max_new_tokens=steps + 1, ignore_eos=True)
    t1 = time.time()
    decode_ms = max(r.total_ms for r in res) - max(r.ttft_ms for r in res)
    toks = sum(r.completion_tokens - 1 for r in res)
    # bytes that the timed call copied, counted by the engine from the tensors it copied, over the steps it ran
    # (a run of queued decode steps loads its inputs once and reads every step's tokens back)
    st = engine.stats()
    n_steps = max(1, st.steps - before.steps)
    return {"value": toks / (decode_ms / 1e3), "unit": "tok/s",
            "h2d_bytes_per_step": round((st.h2d_bytes - before.h2d_bytes) / n_steps, 1),
            "d2h_bytes_per_step": round((st.d2h_bytes - before.d2h_bytes) / n_steps, 1), "decode_ms": decode_ms}, (t0, t1)


# ---------------------------------------------------------------------------------------------------------------
# --workload pabelix: the Pabelix design beside Qwen3 dense at equal layer sizes
# ---------------------------------------------------------------------------------------------------------------
def pabelix_config(width, heads, kv_heads, dim, vdim, ff, experts, top, expert_ff, layers, vocab):
    """Layers that resemble a real model's: differential attention everywhere; the first layer's feed-forward dense,
    the others routed (top * expert_ff = ff, so a token does the dense layer's work); every third layer reads the
    keys and values of the layer before it."""
    out = []
    for i in range(layers):
        m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "diff": 0.5,
             "q_temp": {"coef": 0.1, "every": 512}}
        if i % 3 == 2:
            m["kv_from"] = i - 1
        mlp = ({"kind": "dense", "ff": ff, "limit": 7.0} if i == 0 else
               {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top, "groups": {"count": 4, "keep": 2}}})
        out.append({"type": "attention", "mixer": m, "mlp": mlp})
    return {"architecture": "Pabelix", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": out}


PABELIX_SIZES = {
    # name: (width, heads, kv heads, dim, vdim, ff, experts, top, expert ff); Qwen3 at the same width has `heads` heads of
    # 2 * dim = vdim, the same key/value heads and the same feed-forward width
    "2k": (2048, 16, 4, 64, 128, 8192, 32, 4, 2048),
    "4k": (4096, 32, 8, 64, 128, 12288, 64, 6, 2048),
}


def _engine_for(cfg, num_pages, max_running):
    import torch
    from prelude_b200 import Engine
    from prelude_b200.config import load_model_config
    from prelude_b200.engine.loading import build_model
    from prelude_b200.weights.loader import WeightStore
    from prelude_b200.weights.random_init import random_tensors
    tensors = random_tensors(cfg, seed=0, std=0.02, norm_jitter=0.05, dtype=torch.bfloat16, device="cuda:0")
    model = build_model(load_model_config(cfg).to_model_spec(), WeightStore.from_tensors(tensors), "bf16", "cuda:0")
    del tensors
    torch.cuda.empty_cache()
    return Engine(model, page_size=PAGE_SIZE, num_pages=num_pages, max_running_requests=max_running,
                  max_num_batched_tokens=max(8192, PREFILL_TOKENS), max_model_len=CONTEXT_LEN, cuda_graph=True, cuda_graph_max_bs=64)


def _event_ms(fn, warmup=3, reps=10, flush=None):
    """Median device time of fn() in milliseconds, CUDA events on the launching stream; ``flush`` (a tensor larger than
    the L2 cache) is overwritten between repetitions."""
    import torch
    for _ in range(warmup):
        fn()
    # one launch costs the host more than a small kernel takes: replay it from a captured graph, so that the events
    # bracket device work only
    try:
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        fn = graph.replay
        fn()
    except Exception:
        torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return statistics.median(times)


def pabelix_kernels(pk, size):
    """The new design's kernels beside their like of the closest model, one launch each, as fractions of the
    measured peaks: prompt attention over one 2,048-token request, decode attention of 8 tokens at 2,048 keys, the
    routed feed-forward's two grouped products beside one library product of the same work."""
    import torch
    from prelude_b200.cache.manager import CacheManager
    from prelude_b200.config.spec import DiffAttentionSpec, QueryTemperatureSpec
    from prelude_b200.engine.batch import StepItem, build_step_batch
    from prelude_b200.ops import kernels as K
    from prelude_b200.ops.attention import paged_attention
    from prelude_b200.ops.diff_attention import diff_attention
    from prelude_b200.parts.registry import KvPagesNeed
    width, H, G, dim, vdim, ff, E, top, eff = PABELIX_SIZES[size]
    dev = torch.device("cuda:0")
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    bf = torch.bfloat16
    out = {}
    T, ctx, B = 2048, 2048, 8
    spec = DiffAttentionSpec(width, H, G, dim, vdim, dim ** -0.5, 0.5, 1e-6, QueryTemperatureSpec(0.1, 512))
    needs = [KvPagesNeed(2 * G, dim, None, G, vdim), KvPagesNeed(G, vdim)]
    cache = CacheManager(needs, PAGE_SIZE, (B * (ctx + 16) + T) // PAGE_SIZE + 8, B + 1, dev, bf)
    for n in (0, 1):
        lc = cache.layer_cache(n)
        lc.k_pages.normal_()
        lc.v_pages.normal_()
    # prompt attention: one request of T tokens
    cache.add_request("p")
    cache.grow("p", T)
    batch = build_step_batch([StepItem("p", [0] * T, 0, [])], cache.block_tables(["p"]), [cache.slot_of("p")], dev, 10, 1 << 20)
    proj = torch.randn(T, H * 2 * dim + H * vdim, device=dev).to(bf)
    q, gate = proj[:, :H * 2 * dim], proj[:, H * 2 * dim:]
    lc0, lc1 = cache.layer_cache(0), cache.layer_cache(1)
    ms = _event_ms(lambda: diff_attention(q, gate, lc0.k_pages, lc0.v_pages, batch, cache.group_of[0], spec, 0.6), flush=flush)
    pairs = T * (T + 1) // 2
    flops = 2 * H * pairs * 2 * (dim + vdim)
    out["prefill_attention"] = {"pabelix_ms": round(ms, 4), "pabelix_tflops": round(flops / ms / 1e9, 1)}
    q3 = torch.randn(T, H, vdim, device=dev).to(bf)
    ms = _event_ms(lambda: paged_attention(q3, lc1.k_pages, lc1.v_pages, batch, cache.group_of[1], vdim ** -0.5, None), flush=flush)
    out["prefill_attention"].update(qwen3_ms=round(ms, 4), qwen3_tflops=round(H * pairs * 4 * vdim / ms / 1e9, 1))
    cache.release("p")
    # decode attention: B tokens at ctx keys
    rids = [f"d{i}" for i in range(B)]
    for r in rids:
        cache.add_request(r)
        cache.grow(r, ctx + 1)
    batch = build_step_batch([StepItem(r, [0], ctx, []) for r in rids], cache.block_tables(rids), [cache.slot_of(r) for r in rids], dev, 10, 1 << 20)
    proj = torch.randn(B, H * 2 * dim + H * vdim, device=dev).to(bf)
    q, gate = proj[:, :H * 2 * dim], proj[:, H * 2 * dim:]
    ms = _event_ms(lambda: diff_attention(q, gate, lc0.k_pages, lc0.v_pages, batch, cache.group_of[0], spec, 0.6), flush=flush, reps=20)
    nbytes = B * (ctx + 1) * G * (2 * dim + vdim) * 2
    out["decode_attention"] = {"pabelix_us": round(ms * 1e3, 2), "pabelix_gbs": round(nbytes / ms / 1e6, 1)}
    q3 = torch.randn(B, H, vdim, device=dev).to(bf)
    ms = _event_ms(lambda: paged_attention(q3, lc1.k_pages, lc1.v_pages, batch, cache.group_of[1], vdim ** -0.5, None), flush=flush, reps=20)
    out["decode_attention"].update(qwen3_us=round(ms * 1e3, 2), qwen3_gbs=round(B * (ctx + 1) * G * 2 * vdim * 2 / ms / 1e6, 1))
    # the routed feed-forward's products beside library products of the same work
    for rows, name in ((T, "prefill"), (B, "decode")):
        x = torch.randn(rows, width, device=dev).to(bf)
        ids = torch.stack([torch.randperm(E, device=dev)[:top] for _ in range(rows)]).to(torch.int32)
        w1 = (torch.randn(E, 2 * eff, width, device=dev) * 0.02).to(bf)
        w2 = (torch.randn(E, width, eff, device=dev) * 0.02).to(bf)
        from prelude_b200.ops import linear as L
        st = L.tc_status(dev)
        if rows * top >= 192 * E:
            # as the part runs a long prompt step: rows sorted by expert, both products on the paired-block tcgen05 kernel
            plan = K.moe_sort(ids, E, 256)
            h = K.moe_gemm_pair(K.moe_gather_rows(x, plan, top), w1, plan, True, st)
            ms1 = _event_ms(lambda: K.moe_gemm_pair(K.moe_gather_rows(x, plan, top), w1, plan, True, st), flush=flush)
            ms2 = _event_ms(lambda: K.moe_gemm_pair(h, w2, plan, False, st), flush=flush)
        else:
            few = rows * top <= 6 * E                        # as the part runs a decode step: the kernel that streams the weights
            plan = K.moe_sort(ids, E, 64 if few else None)
            h = K.moe_gemm(x, w1, plan, gated=True, gather_div=top, few_rows=few)
            ms1 = _event_ms(lambda: K.moe_gemm(x, w1, plan, gated=True, gather_div=top, few_rows=few), flush=flush)
            ms2 = _event_ms(lambda: K.moe_gemm(h, w2, plan, gated=False, out_dtype=torch.float32, few_rows=few), flush=flush)
        if int(st.item()) != 0:
            raise RuntimeError("a routed product raised the status word")
        flops = 2 * rows * top * 3 * eff * width
        d1 = (torch.randn(2 * top * eff, width, device=dev) * 0.02).to(bf)
        d2 = (torch.randn(width, top * eff, device=dev) * 0.02).to(bf)
        from prelude_b200.ops.linear import linear
        hd = K.silu_mul(linear(x, d1))
        msd = _event_ms(lambda: linear(K.silu_mul(linear(x, d1)), d2), flush=flush)
        touched = min(E, rows * top) * 3 * eff * width * 2
        out[f"routed_products_{name}"] = {"pabelix_ms": round(ms1 + ms2, 4), "pabelix_tflops": round(flops / (ms1 + ms2) / 1e9, 1),
                                           "pabelix_weight_gbs": round(touched / (ms1 + ms2) / 1e6, 1),
                                           "dense_same_work_ms": round(msd, 4), "dense_tflops": round(flops / msd / 1e9, 1),
                                           "dense_weight_gbs": round(3 * top * eff * width * 2 / msd / 1e6, 1)}
        del w1, w2, d1, d2
    out["peaks"] = {"bf16_tflops": pk["bf16_tflops"], "hbm_gbs": pk["hbm_gbs"], "source": pk["source"]}
    return out


def pabelix_compare(args):
    """Prefill and decode throughput of Pabelix beside Qwen3 dense at equal layer sizes (random weights, bfloat16):
    one prompt of --prefill-tokens through the step function, and --batch requests decoding behind --prefix-len
    tokens on the captured step, both timed on the device.  One JSON line of its own."""
    import torch
    pk = peaks()
    clocks = ClockSampler()
    clocks.start()
    t_begin = time.time()
    points = []
    vocab = 32768
    for size in args.sizes.split(","):
        width, H, G, dim, vdim, ff, E, top, eff = PABELIX_SIZES[size]
        layers = args.layers or 6
        arms = {
            "pabelix": pabelix_config(width, H, G, dim, vdim, ff, E, top, eff, layers, vocab),
            "qwen3": dict(QWEN3_4B, vocab_size=vocab, hidden_size=width, intermediate_size=ff, num_hidden_layers=layers,
                          num_attention_heads=H, num_key_value_heads=G, head_dim=vdim, tie_word_embeddings=True),
        }
        point = {"size": size, "layers": layers, "width": width}
        for name, cfg in arms.items():
            pages_per_req = -(-(PREFIX_LEN + args.warmup + args.steps + 2) // PAGE_SIZE)
            engine = _engine_for(cfg, args.batch * pages_per_req + 2 * (PREFILL_TOKENS // PAGE_SIZE) + 8, args.batch + 2)
            shim = {"vocab_size": vocab}
            prefill_ms, _ = time_prefill(engine, shim, args.warmup)
            dec, _ = time_decode(engine, shim, args.batch, args.steps, args.warmup, seed=1)
            point[name] = {"prefill_tok_s": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 3),
                           "decode_tok_s": round(dec["tok_s"], 1), "decode_ms_per_step": round(dec["ms_per_step"], 4),
                           "weight_gb": round(engine.model.weight_bytes() / 1e9, 3)}
            del engine
            torch.cuda.empty_cache()
        point["kernels"] = pabelix_kernels(pk, size)
        points.append(point)
    clocks.stop()
    print(json.dumps({"metric": "Pabelix beside Qwen3 dense at equal layer sizes: prefill and decode tokens a second, device-timed",
                      "unit": "tok/s", "n_gpus": 1, "dtype": "bf16", "data": "synthetic", "impl": "ours", "steps": args.steps,
                      "warmup": args.warmup, "config": {"batch": args.batch, "prefix_len": PREFIX_LEN, "prefill_tokens": PREFILL_TOKENS,
                                                        "page_size": PAGE_SIZE, "l2": "inputs_exceed_l2 (steps), flushed (kernels)"},
                      "points": points, "clocks": clocks.summary([(t_begin, time.time())])}))
    return 0


# ---------------------------------------------------------------------------------------------------------------
# --workload kolisun: the Kolisun design beside Qwen3 dense at equal layer sizes
# ---------------------------------------------------------------------------------------------------------------
KOLISUN_SIZES = {
    # width; window attention: heads, key/value heads, head size, window; state-space mixer: heads, head size, state, groups;
    # latent attention: heads, plain and rotated query/key sizes, value size, latent sizes; feed-forward width.
    # Qwen3 at the same width has the window attention's heads and head size and the same feed-forward width.
    "2k": dict(width=2048, heads=16, kv=4, dim=128, window=1024, ss_heads=64, ss_dim=64, state=128, groups=8,
               lat_heads=16, lat_dim=128, rot=64, vdim=128, kv_rank=512, q_rank=1536, ff=8192),
    "4k": dict(width=4096, heads=32, kv=8, dim=128, window=1024, ss_heads=128, ss_dim=64, state=128, groups=8,
               lat_heads=32, lat_dim=128, rot=64, vdim=128, kv_rank=512, q_rank=1536, ff=12288),
}


def kolisun_config(z, layers, vocab):
    """Layers that resemble a real model's: one layer with window attention and a state-space mixer side by side, then two
    with latent attention, and so on; every layer with a SiLU-gated feed-forward."""
    par = {"left": {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
                    "mask": {"size": z["window"]},
                    "rot": {"dims": z["dim"], "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}},
           "right": {"heads": z["ss_heads"], "vdim": z["ss_dim"], "state": z["state"], "groups": z["groups"], "conv": 4, "norm_groups": z["groups"]},
           "left_scale": 1.0, "right_scale": 1.0}
    lat = {"heads": z["lat_heads"], "dim": z["lat_dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "kv_rank": z["kv_rank"], "q_rank": z["q_rank"],
           "scale": (z["lat_dim"] + z["rot"]) ** -0.5,
           "rot": {"dims": z["rot"], "base": 10000.0, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    mlp = {"kind": "dense", "ff": z["ff"]}
    out = [{"type": "parallel", "mixer": par, "mlp": mlp} if i % 3 == 0 else {"type": "latent_attention", "mixer": lat, "mlp": mlp}
           for i in range(layers)]
    return {"architecture": "Kolisun", "vocab": vocab, "width": z["width"], "norm": {"eps": 1e-6}, "layers": out}


def kolisun_kernels(pk, size):
    """The new design's kernels beside their like of the closest model, one launch each: latent attention over a prompt of
    2,048 tokens and for 8 decoded tokens at 2,048 keys beside Qwen3's attention kernels; the kernel between projection and
    attention beside Qwen3's; the state-space mixer's kernels against the bytes they must move."""
    import torch
    from prelude_b200.cache.manager import CacheManager
    from prelude_b200.engine.batch import StepItem, build_step_batch
    from prelude_b200.ops import kernels as K
    from prelude_b200.ops.attention import paged_attention
    from prelude_b200.ops.paged_general import attention_general
    from prelude_b200.parts.registry import CombinedNeed, KvPagesNeed, StateNeed
    z = KOLISUN_SIZES[size]
    dev = torch.device("cuda:0")
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    bf = torch.bfloat16
    out = {}
    T, ctx, B = 2048, 2048, 8
    H, G, D = z["heads"], z["kv"], z["dim"]
    LH, row, rank = z["lat_heads"], z["kv_rank"] + z["rot"], z["kv_rank"]
    SH, P, N, SG = z["ss_heads"], z["ss_dim"], z["state"], z["groups"]
    inner, channels = SH * P, SH * P + 2 * SG * N
    needs = [KvPagesNeed(1, row, None, 0, 0), KvPagesNeed(G, D),
             CombinedNeed((StateNeed((SH, N, P), torch.float32), StateNeed((3, channels), None)))]
    cache = CacheManager(needs, PAGE_SIZE, (B * (ctx + 16) + T) // PAGE_SIZE + 8, B + 1, dev, bf)
    lat, plain = cache.layer_cache(0), cache.layer_cache(1)
    lat.k_pages.normal_()
    plain.k_pages.normal_()
    plain.v_pages.normal_()
    sink = torch.zeros(LH, device=dev)
    # -- one request of T prompt tokens
    cache.add_request("p")
    cache.grow("p", T)
    batch = build_step_batch([StepItem("p", [0] * T, 0, [])], cache.block_tables(["p"]), [cache.slot_of("p")], dev, 10, 1 << 20)
    cache.zero_fresh_state()
    pairs = T * (T + 1) // 2
    q = torch.randn(T, LH, row, device=dev).to(bf)
    ms = _event_ms(lambda: attention_general(q, lat.k_pages, None, rank, batch, cache.group_of[0], row ** -0.5, None, sink), flush=flush)
    out["prefill_attention"] = {"latent_ms": round(ms, 4), "latent_tflops": round(2 * LH * pairs * (row + rank) / ms / 1e9, 1)}
    q3 = torch.randn(T, H, D, device=dev).to(bf)
    ms = _event_ms(lambda: paged_attention(q3, plain.k_pages, plain.v_pages, batch, cache.group_of[1], D ** -0.5, None), flush=flush)
    out["prefill_attention"].update(qwen3_ms=round(ms, 4), qwen3_tflops=round(H * pairs * 4 * D / ms / 1e9, 1))
    # the kernel between projection and attention
    proj = torch.randn(T, (H + 2 * G) * D, device=dev).to(bf)
    wq, wk = torch.ones(H * D, device=dev), torch.ones(G * D, device=dev)
    rates = torch.rand(D // 2, device=dev)
    qo = torch.empty(T, H, D, dtype=bf, device=dev)
    ms = _event_ms(lambda: K.qkv_prepare(proj[:, :H * D], proj[:, H * D:(H + G) * D], proj[:, (H + G) * D:], n_heads=H, q_dim=D, q_weight=wq,
                                         k_weight=wk, k_norm_cols=G * D, eps=1e-6, rates=rates, rot_dims=D, adjacent=True,
                                         positions=batch.positions, table_row=batch.table_row_of_token,
                                         block_table=batch.block_tables[cache.group_of[1]], q_out=qo, k_pages=plain.k_pages,
                                         v_pages=plain.v_pages, swizzle_k=True, swizzle_v=True, status=batch.status), flush=flush)
    moved = T * (H + 2 * G) * D * 2 * 2
    out["projection_to_pages"] = {"kolisun_us": round(ms * 1e3, 2), "kolisun_gbs": round(moved / ms / 1e6, 1)}
    ang = torch.arange(T, device=dev, dtype=torch.float32).reshape(-1, 1) * rates.reshape(1, -1)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    hw = torch.ones(D, device=dev)
    ms = _event_ms(lambda: K.qknorm_rope_kvwrite(proj, H, G, D, hw, hw, 1e-6, cos, sin, D, batch.positions, batch.table_row_of_token,
                                                 batch.block_tables[cache.group_of[1]], plain.k_pages, plain.v_pages, True, batch.status,
                                                 out=qo), flush=flush)
    out["projection_to_pages"].update(qwen3_us=round(ms * 1e3, 2), qwen3_gbs=round(moved / ms / 1e6, 1))
    # the state-space mixer's kernels over the prompt
    sc = cache.layer_cache(2)
    state, carried = sc.children[0].state, sc.children[1].state
    sproj = (torch.randn(T, 2 * inner + 2 * SG * N + SH, device=dev) * 0.5).to(bf)
    xbc, dt, zz = sproj[:, inner:inner + channels], sproj[:, inner + channels:], sproj[:, :inner]
    conv_w, conv_b = torch.randn(channels, 4, device=dev) * 0.5, torch.zeros(channels, device=dev)
    hb, al, dd, nw = torch.zeros(SH, device=dev), torch.zeros(SH, device=dev), torch.ones(SH, device=dev), torch.ones(inner, device=dev)
    u = K.causal_conv_silu(xbc, conv_w, conv_b, carried, batch)
    y = K.ssm_scan(u, dt, hb, al, dd, state, batch, SG)
    ms_c = _event_ms(lambda: K.causal_conv_silu(xbc, conv_w, conv_b, carried, batch, out=u), flush=flush)
    ms_s = _event_ms(lambda: K.ssm_scan(u, dt, hb, al, dd, state, batch, SG, out=y), flush=flush)
    ms_n = _event_ms(lambda: K.gated_group_rmsnorm(y, zz, nw, SG, 1e-6), flush=flush)
    out["state_space_prefill"] = {
        "conv_us": round(ms_c * 1e3, 2), "conv_gbs": round(T * channels * 2 * 2 / ms_c / 1e6, 1),
        "scan_us": round(ms_s * 1e3, 2), "scan_gbs": round((T * channels * 2 + T * inner * 4) / ms_s / 1e6, 1),
        "scan_gflops": round(T * SH * N * P * 6 / ms_s / 1e6, 1),
        "gated_norm_us": round(ms_n * 1e3, 2), "gated_norm_gbs": round(T * inner * (4 + 2 + 2) / ms_n / 1e6, 1)}
    cache.release("p")
    # -- B single tokens at ctx keys
    rids = [f"d{i}" for i in range(B)]
    for r in rids:
        cache.add_request(r)
        cache.grow(r, ctx + 1)
    batch = build_step_batch([StepItem(r, [0], ctx, []) for r in rids], cache.block_tables(rids), [cache.slot_of(r) for r in rids], dev, 10, 1 << 20)
    cache.zero_fresh_state()
    q = torch.randn(B, LH, row, device=dev).to(bf)
    ms = _event_ms(lambda: attention_general(q, lat.k_pages, None, rank, batch, cache.group_of[0], row ** -0.5, None, sink), flush=flush, reps=20)
    out["decode_attention"] = {"latent_us": round(ms * 1e3, 2), "latent_gbs": round(B * (ctx + 1) * row * 2 / ms / 1e6, 1)}
    q3 = torch.randn(B, H, D, device=dev).to(bf)
    ms = _event_ms(lambda: paged_attention(q3, plain.k_pages, plain.v_pages, batch, cache.group_of[1], D ** -0.5, None), flush=flush, reps=20)
    out["decode_attention"].update(qwen3_us=round(ms * 1e3, 2), qwen3_gbs=round(B * (ctx + 1) * G * 2 * D * 2 / ms / 1e6, 1))
    u8, y8 = u[:B], y[:B]
    ms_s = _event_ms(lambda: K.ssm_scan(u8, dt[:B], hb, al, dd, state, batch, SG, out=y8), flush=flush, reps=20)
    out["state_space_decode"] = {"scan_us": round(ms_s * 1e3, 2), "scan_state_gbs": round(B * SH * N * P * 4 * 2 / ms_s / 1e6, 1)}
    out["peaks"] = {"bf16_tflops": pk["bf16_tflops"], "hbm_gbs": pk["hbm_gbs"], "source": pk["source"]}
    return out


def kolisun_compare(args):
    """Prefill and decode throughput of Kolisun beside Qwen3 dense at equal layer sizes (random weights, bfloat16):
    one prompt of --prefill-tokens through the step function, and --batch requests decoding behind --prefix-len
    tokens on the captured step, both timed on the device.  One JSON line of its own."""
    import torch
    pk = peaks()
    clocks = ClockSampler()
    clocks.start()
    t_begin = time.time()
    points = []
    vocab = 32768
    for size in args.sizes.split(","):
        z = KOLISUN_SIZES[size]
        layers = args.layers or 6
        arms = {
            "kolisun": kolisun_config(z, layers, vocab),
            "qwen3": dict(QWEN3_4B, vocab_size=vocab, hidden_size=z["width"], intermediate_size=z["ff"], num_hidden_layers=layers,
                          num_attention_heads=z["heads"], num_key_value_heads=z["kv"], head_dim=z["dim"], tie_word_embeddings=True),
        }
        point = {"size": size, "layers": layers, "width": z["width"]}
        for name, cfg in arms.items():
            pages_per_req = -(-(PREFIX_LEN + args.warmup + args.steps + 2) // PAGE_SIZE)
            engine = _engine_for(cfg, args.batch * pages_per_req + 2 * (PREFILL_TOKENS // PAGE_SIZE) + 8, args.batch + 2)
            shim = {"vocab_size": vocab}
            prefill_ms, _ = time_prefill(engine, shim, args.warmup)
            dec, _ = time_decode(engine, shim, args.batch, args.steps, args.warmup, seed=1)
            point[name] = {"prefill_tok_s": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 3),
                           "decode_tok_s": round(dec["tok_s"], 1), "decode_ms_per_step": round(dec["ms_per_step"], 4),
                           "weight_gb": round(engine.model.weight_bytes() / 1e9, 3)}
            del engine
            torch.cuda.empty_cache()
        point["kernels"] = kolisun_kernels(pk, size)
        points.append(point)
    clocks.stop()
    print(json.dumps({"metric": "Kolisun beside Qwen3 dense at equal layer sizes: prefill and decode tokens a second, device-timed",
                      "unit": "tok/s", "n_gpus": 1, "dtype": "bf16", "data": "synthetic", "impl": "ours", "steps": args.steps,
                      "warmup": args.warmup, "config": {"batch": args.batch, "prefix_len": PREFIX_LEN, "prefill_tokens": PREFILL_TOKENS,
                                                        "page_size": PAGE_SIZE, "l2": "inputs_exceed_l2 (steps), flushed (kernels)"},
                      "points": points, "clocks": clocks.summary([(t_begin, time.time())])}))
    return 0


# ---------------------------------------------------------------------------------------------------------------
# --workload nedesun: the Nedesun design beside Kolisun (the closest design: attention beside a recurrent mixer, state
# slots) and Qwen3 dense at equal layer sizes
# ---------------------------------------------------------------------------------------------------------------
NEDESUN_SIZES = {
    # width; attention (both kinds): heads, key/value heads, head size; window and kept first tokens; chunk; gated delta
    # rule: heads, query/key heads, key and value sizes; time mixing: heads of 64; feed-forward width
    "2k": dict(width=2048, heads=16, kv=4, dim=128, window=1024, keep=64, chunk=1024, d_heads=16, d_kv=8, d_dim=128, d_vdim=128,
               w_dim=64, ff=8192),
    "4k": dict(width=4096, heads=32, kv=8, dim=128, window=1024, keep=64, chunk=1024, d_heads=32, d_kv=16, d_dim=128, d_vdim=128,
               w_dim=64, ff=12288),
}


def nedesun_config(z, layers, vocab):
    """Layers that resemble a real model's: window attention beside the gated delta rule, then chunked attention with blended
    values, then time mixing, and so on; every layer with a SiLU-gated feed-forward."""
    par = {"left": {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
                    "mask": {"size": z["window"], "keep_first": z["keep"]}},
           "right": {"heads": z["d_heads"], "kv_heads": z["d_kv"], "dim": z["d_dim"], "vdim": z["d_vdim"], "conv": 4}}
    att = {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
           "mask": {"size": z["chunk"]}, "rot": {"dims": z["dim"], "base": 500000.0}, "softcap": 30.0, "v_mix": True}
    wkv = {"heads": z["width"] // z["w_dim"], "dim": z["w_dim"]}
    mlp = {"kind": "dense", "ff": z["ff"]}
    kinds = [("parallel", par), ("attention", att), ("wkv", wkv)]
    out = [{"type": kinds[i % 3][0], "mixer": kinds[i % 3][1], "mlp": mlp} for i in range(layers)]
    return {"architecture": "Nedesun", "vocab": vocab, "width": z["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "embedding": {"scale": 1.0}, "layers": out}


def nedesun_kernels(pk, size):
    """The new design's kernels beside their like of the closest model, one launch each: chunked, capped, gated attention
    and window attention with kept first tokens and a sink beside Kolisun's window attention, over a prompt of 2,048 tokens
    and for 8 decoded tokens; the kernel between projection and attention beside Kolisun's; the two recurrences and the
    token blend beside Kolisun's state-space scan, against the bytes and operations they must do."""
    import torch
    from prelude_b200.cache.manager import CacheManager
    from prelude_b200.engine.batch import StepItem, build_step_batch
    from prelude_b200.ops import kernels as K
    from prelude_b200.ops.attention import paged_attention
    from prelude_b200.ops.paged_general import attention_general
    from prelude_b200.parts.registry import CombinedNeed, KvPagesNeed, StateNeed
    z, kz = NEDESUN_SIZES[size], KOLISUN_SIZES[size]
    dev = torch.device("cuda:0")
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    bf = torch.bfloat16
    out = {}
    T, B = 2048, 8
    H, G, D = z["heads"], z["kv"], z["dim"]
    window, keep, chunk = z["window"], z["keep"], z["chunk"]
    ctx = 2 * chunk - 1                                      # the decoded token is the last of its chunk
    DH, DG, DD, DE = z["d_heads"], z["d_kv"], z["d_dim"], z["d_vdim"]
    WH, WD = z["width"] // z["w_dim"], z["w_dim"]
    SH, P, N, SG = kz["ss_heads"], kz["ss_dim"], kz["state"], kz["groups"]
    d_channels, d_inner = 2 * DG * DD + DH * DE, DH * DE
    s_inner, s_channels = SH * P, SH * P + 2 * SG * N
    needs = [KvPagesNeed(G, D), KvPagesNeed(G, D),
             CombinedNeed((StateNeed((DH, DD, DE), torch.float32), StateNeed((3, d_channels), None))),
             CombinedNeed((StateNeed((WH, WD, WD), torch.float32), StateNeed((1, z["width"]), None))),
             CombinedNeed((StateNeed((SH, N, P), torch.float32), StateNeed((3, s_channels), None)))]
    cache = CacheManager(needs, PAGE_SIZE, (B * (ctx + 16) + T) // PAGE_SIZE + 8, B + 1, dev, bf)
    gen, plain = cache.layer_cache(0), cache.layer_cache(1)
    for lc in (gen, plain):
        lc.k_pages.normal_()
        lc.v_pages.normal_()
    sink = torch.zeros(H, device=dev)
    scale = D ** -0.5

    def visible_pairs(n, first=0):
        w = sum(min(i + 1, window) + max(0, min(keep, i + 1 - window)) for i in range(first, first + n))
        c = sum(i % chunk + 1 for i in range(first, first + n))
        return w, c

    # -- one request of T prompt tokens
    cache.add_request("p")
    cache.grow("p", T)
    batch = build_step_batch([StepItem("p", [0] * T, 0, [])], cache.block_tables(["p"]), [cache.slot_of("p")], dev, 10, 1 << 20)
    cache.zero_fresh_state()
    w_pairs, c_pairs = visible_pairs(T)
    q = torch.randn(T, H, D, device=dev).to(bf)
    gate = torch.randn(T, H, device=dev).to(bf)
    g0 = cache.group_of[0]
    ms = _event_ms(lambda: attention_general(q, gen.k_pages, gen.v_pages, D, batch, g0, scale, None, None, chunk=chunk, softcap=30.0, gate=gate),
                   flush=flush)
    out["prefill_attention"] = {"chunked_ms": round(ms, 4), "chunked_tflops": round(H * c_pairs * 4 * D / ms / 1e9, 1)}
    ms = _event_ms(lambda: attention_general(q, gen.k_pages, gen.v_pages, D, batch, g0, scale, window, sink, keep_first=keep), flush=flush)
    out["prefill_attention"].update(window_kept_ms=round(ms, 4), window_kept_tflops=round(H * w_pairs * 4 * D / ms / 1e9, 1))
    k_pairs = sum(min(i + 1, kz["window"]) for i in range(T))
    ms = _event_ms(lambda: paged_attention(q, plain.k_pages, plain.v_pages, batch, cache.group_of[1], scale, kz["window"]), flush=flush)
    out["prefill_attention"].update(kolisun_window_ms=round(ms, 4), kolisun_window_tflops=round(H * k_pairs * 4 * D / ms / 1e9, 1))
    # the kernel between projection and attention
    proj = torch.randn(T, (H + 2 * G) * D, device=dev).to(bf)
    rates = torch.rand(D // 2, device=dev)
    qo = torch.empty(T, H, D, dtype=bf, device=dev)
    v_first = torch.randn(T, G * D, device=dev).to(bf)
    ms = _event_ms(lambda: K.heads_prepare(proj[:, :H * D], proj[:, H * D:(H + G) * D], proj[:, (H + G) * D:], n_heads=H, q_dim=D, rates=rates,
                                           rot_dims=D, v_other=v_first, mix=0.3, positions=batch.positions,
                                           table_row=batch.table_row_of_token, block_table=batch.block_tables[g0], q_out=qo,
                                           k_pages=gen.k_pages, v_pages=gen.v_pages, status=batch.status), flush=flush)
    moved = T * (H + 2 * G) * D * 2 * 2
    out["projection_to_pages"] = {"rotate_blend_us": round(ms * 1e3, 2), "rotate_blend_gbs": round((moved + T * G * D * 2) / ms / 1e6, 1)}
    hw = torch.ones(D, device=dev)
    ms = _event_ms(lambda: K.heads_prepare(proj[:, :H * D], proj[:, H * D:(H + G) * D], proj[:, (H + G) * D:], n_heads=H, q_dim=D, q_weight=hw,
                                           k_weight=hw, eps=1e-6, positions=batch.positions, table_row=batch.table_row_of_token,
                                           block_table=batch.block_tables[g0], q_out=qo, k_pages=gen.k_pages, v_pages=gen.v_pages,
                                           status=batch.status), flush=flush)
    out["projection_to_pages"].update(head_norm_us=round(ms * 1e3, 2), head_norm_gbs=round(moved / ms / 1e6, 1))
    wq, wk = torch.ones(H * D, device=dev), torch.ones(G * D, device=dev)
    ms = _event_ms(lambda: K.qkv_prepare(proj[:, :H * D], proj[:, H * D:(H + G) * D], proj[:, (H + G) * D:], n_heads=H, q_dim=D, q_weight=wq,
                                         k_weight=wk, k_norm_cols=G * D, eps=1e-6, rates=rates, rot_dims=D, adjacent=True,
                                         positions=batch.positions, table_row=batch.table_row_of_token,
                                         block_table=batch.block_tables[cache.group_of[1]], q_out=qo, k_pages=plain.k_pages,
                                         v_pages=plain.v_pages, swizzle_k=True, swizzle_v=True, status=batch.status), flush=flush)
    out["projection_to_pages"].update(kolisun_us=round(ms * 1e3, 2), kolisun_gbs=round(moved / ms / 1e6, 1))
    # the recurrences over the prompt
    dc, wc, sc = cache.layer_cache(2), cache.layer_cache(3), cache.layer_cache(4)
    d_state, d_carried = dc.children[0].state, dc.children[1].state
    dproj = (torch.randn(T, d_channels + d_inner + 2 * DH, device=dev) * 0.5).to(bf)
    qkv, dgate = dproj[:, :d_channels], dproj[:, d_channels:d_channels + d_inner]
    beta, a = dproj[:, d_channels + d_inner:d_channels + d_inner + DH], dproj[:, d_channels + d_inner + DH:]
    d_conv = torch.randn(d_channels, 4, device=dev) * 0.5
    al, hb, nw = torch.zeros(DH, device=dev), torch.zeros(DH, device=dev), torch.ones(d_inner, device=dev)
    u = K.causal_conv_silu(qkv, d_conv, None, d_carried, batch)
    y = K.gated_delta_scan(u, beta, a, al, hb, d_state, batch, DG)
    ms_c = _event_ms(lambda: K.causal_conv_silu(qkv, d_conv, None, d_carried, batch, out=u), flush=flush)
    ms_s = _event_ms(lambda: K.gated_delta_scan(u, beta, a, al, hb, d_state, batch, DG, out=y), flush=flush)
    ms_n = _event_ms(lambda: K.gated_group_rmsnorm(y, dgate, nw, DH, 1e-6, gate_after=True), flush=flush)
    out["gated_delta_prefill"] = {
        "conv_us": round(ms_c * 1e3, 2), "conv_gbs": round(T * d_channels * 2 * 2 / ms_c / 1e6, 1),
        "scan_us": round(ms_s * 1e3, 2), "scan_gbs": round((T * d_channels * 2 + T * d_inner * 4) / ms_s / 1e6, 1),
        "scan_gflops": round(T * DH * DD * DE * 9 / ms_s / 1e6, 1),
        "gated_norm_us": round(ms_n * 1e3, 2), "gated_norm_gbs": round(T * d_inner * (4 + 2 + 2) / ms_n / 1e6, 1)}
    w_state, w_carried = wc.children[0].state, wc.children[1].state
    w_inner = WH * WD
    x = (torch.randn(T, z["width"], device=dev) * 0.5).to(bf)
    mu = torch.rand(5, z["width"], device=dev)
    blends = K.token_shift_mix(x, w_carried.view(w_carried.shape[0], z["width"]), mu, batch)
    ms_b = _event_ms(lambda: K.token_shift_mix(x, w_carried.view(w_carried.shape[0], z["width"]), mu, batch, out=blends), flush=flush)
    rkvw = (torch.randn(4, T, w_inner, device=dev) * 0.5).to(bf)
    w0, bonus = torch.full((w_inner,), -1.0, device=dev), torch.zeros(w_inner, device=dev)
    yw = K.wkv_scan(rkvw[0], rkvw[1], rkvw[2], rkvw[3], w0, bonus, w_state, batch)
    ms_w = _event_ms(lambda: K.wkv_scan(rkvw[0], rkvw[1], rkvw[2], rkvw[3], w0, bonus, w_state, batch, out=yw), flush=flush)
    out["time_mixing_prefill"] = {
        "blend_us": round(ms_b * 1e3, 2), "blend_gbs": round(T * z["width"] * 2 * 6 / ms_b / 1e6, 1),
        "scan_us": round(ms_w * 1e3, 2), "scan_gbs": round((4 * T * w_inner * 2 + T * w_inner * 4) / ms_w / 1e6, 1),
        "scan_gflops": round(T * WH * WD * WD * 5 / ms_w / 1e6, 1)}
    s_state, s_carried = sc.children[0].state, sc.children[1].state
    sproj = (torch.randn(T, 2 * s_inner + 2 * SG * N + SH, device=dev) * 0.5).to(bf)
    xbc, dt = sproj[:, s_inner:s_inner + s_channels], sproj[:, s_inner + s_channels:]
    s_conv, s_b = torch.randn(s_channels, 4, device=dev) * 0.5, torch.zeros(s_channels, device=dev)
    shb, sal, sdd = torch.zeros(SH, device=dev), torch.zeros(SH, device=dev), torch.ones(SH, device=dev)
    su = K.causal_conv_silu(xbc, s_conv, s_b, s_carried, batch)
    sy = K.ssm_scan(su, dt, shb, sal, sdd, s_state, batch, SG)
    ms_k = _event_ms(lambda: K.ssm_scan(su, dt, shb, sal, sdd, s_state, batch, SG, out=sy), flush=flush)
    out["kolisun_state_space_prefill"] = {"scan_us": round(ms_k * 1e3, 2),
                                          "scan_gbs": round((T * s_channels * 2 + T * s_inner * 4) / ms_k / 1e6, 1),
                                          "scan_gflops": round(T * SH * N * P * 6 / ms_k / 1e6, 1)}
    cache.release("p")
    # -- B single tokens at ctx keys
    rids = [f"d{i}" for i in range(B)]
    for r in rids:
        cache.add_request(r)
        cache.grow(r, ctx + 1)
    batch = build_step_batch([StepItem(r, [0], ctx, []) for r in rids], cache.block_tables(rids), [cache.slot_of(r) for r in rids], dev, 10, 1 << 20)
    cache.zero_fresh_state()
    q = torch.randn(B, H, D, device=dev).to(bf)
    gate = torch.randn(B, H, device=dev).to(bf)
    row_bytes = G * 2 * D * 2
    ms = _event_ms(lambda: attention_general(q, gen.k_pages, gen.v_pages, D, batch, g0, scale, None, None, chunk=chunk, softcap=30.0, gate=gate),
                   flush=flush, reps=20)
    out["decode_attention"] = {"chunked_us": round(ms * 1e3, 2), "chunked_gbs": round(B * chunk * row_bytes / ms / 1e6, 1)}
    ms = _event_ms(lambda: attention_general(q, gen.k_pages, gen.v_pages, D, batch, g0, scale, window, sink, keep_first=keep), flush=flush, reps=20)
    out["decode_attention"].update(window_kept_us=round(ms * 1e3, 2), window_kept_gbs=round(B * (window + keep) * row_bytes / ms / 1e6, 1))
    ms = _event_ms(lambda: paged_attention(q, plain.k_pages, plain.v_pages, batch, cache.group_of[1], scale, kz["window"]), flush=flush, reps=20)
    out["decode_attention"].update(kolisun_window_us=round(ms * 1e3, 2), kolisun_window_gbs=round(B * kz["window"] * row_bytes / ms / 1e6, 1))
    ms = _event_ms(lambda: K.gated_delta_scan(u[:B], beta[:B], a[:B], al, hb, d_state, batch, DG, out=y[:B]), flush=flush, reps=20)
    out["gated_delta_decode"] = {"scan_us": round(ms * 1e3, 2), "scan_state_gbs": round(B * DH * DD * DE * 4 * 2 / ms / 1e6, 1)}
    ms = _event_ms(lambda: K.wkv_scan(rkvw[0, :B], rkvw[1, :B], rkvw[2, :B], rkvw[3, :B], w0, bonus, w_state, batch, out=yw[:B]), flush=flush, reps=20)
    out["time_mixing_decode"] = {"scan_us": round(ms * 1e3, 2), "scan_state_gbs": round(B * WH * WD * WD * 4 * 2 / ms / 1e6, 1)}
    ms = _event_ms(lambda: K.ssm_scan(su[:B], dt[:B], shb, sal, sdd, s_state, batch, SG, out=sy[:B]), flush=flush, reps=20)
    out["kolisun_state_space_decode"] = {"scan_us": round(ms * 1e3, 2), "scan_state_gbs": round(B * SH * N * P * 4 * 2 / ms / 1e6, 1)}
    out["peaks"] = {"bf16_tflops": pk["bf16_tflops"], "hbm_gbs": pk["hbm_gbs"], "source": pk["source"]}
    return out


def nedesun_compare(args):
    """Prefill and decode throughput of Nedesun beside Kolisun and Qwen3 dense at equal layer sizes (random weights,
    bfloat16): one prompt of --prefill-tokens through the step function, and --batch requests decoding behind
    --prefix-len tokens on the captured step, both timed on the device.  One JSON line of its own."""
    import torch
    pk = peaks()
    clocks = ClockSampler()
    clocks.start()
    t_begin = time.time()
    points = []
    vocab = 32768
    for size in args.sizes.split(","):
        z = NEDESUN_SIZES[size]
        layers = args.layers or 6
        arms = {
            "nedesun": nedesun_config(z, layers, vocab),
            "kolisun": kolisun_config(KOLISUN_SIZES[size], layers, vocab),
            "qwen3": dict(QWEN3_4B, vocab_size=vocab, hidden_size=z["width"], intermediate_size=z["ff"], num_hidden_layers=layers,
                          num_attention_heads=z["heads"], num_key_value_heads=z["kv"], head_dim=z["dim"], tie_word_embeddings=True),
        }
        point = {"size": size, "layers": layers, "width": z["width"]}
        for name, cfg in arms.items():
            pages_per_req = -(-(PREFIX_LEN + args.warmup + args.steps + 2) // PAGE_SIZE)
            engine = _engine_for(cfg, args.batch * pages_per_req + 2 * (PREFILL_TOKENS // PAGE_SIZE) + 8, args.batch + 2)
            shim = {"vocab_size": vocab}
            prefill_ms, _ = time_prefill(engine, shim, args.warmup)
            dec, _ = time_decode(engine, shim, args.batch, args.steps, args.warmup, seed=1)
            point[name] = {"prefill_tok_s": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 3),
                           "decode_tok_s": round(dec["tok_s"], 1), "decode_ms_per_step": round(dec["ms_per_step"], 4),
                           "weight_gb": round(engine.model.weight_bytes() / 1e9, 3)}
            del engine
            torch.cuda.empty_cache()
        point["kernels"] = nedesun_kernels(pk, size)
        points.append(point)
    clocks.stop()
    print(json.dumps({"metric": "Nedesun beside Kolisun and Qwen3 dense at equal layer sizes: prefill and decode tokens a second, device-timed",
                      "unit": "tok/s", "n_gpus": 1, "dtype": "bf16", "data": "synthetic", "impl": "ours", "steps": args.steps,
                      "warmup": args.warmup, "config": {"batch": args.batch, "prefix_len": PREFIX_LEN, "prefill_tokens": PREFILL_TOKENS,
                                                        "page_size": PAGE_SIZE, "l2": "inputs_exceed_l2 (steps), flushed (kernels)"},
                      "points": points, "clocks": clocks.summary([(t_begin, time.time())])}))
    return 0


# ---------------------------------------------------------------------------------------------------------------
# --workload pepolorn: the Pepolorn design beside Kolisun (the closest design: attention beside a recurrent mixer in one
# layer, a state-space mixer, norms on the sublayers' outputs, state slots) and Qwen3 dense at equal layer sizes
# ---------------------------------------------------------------------------------------------------------------
PEPOLORN_SIZES = {
    # width; chunked attention: heads, key/value heads, head size, chunk, rotated elements; linear attention with a decaying
    # state: heads, key and value sizes; state-space mixer: heads, head size, state, groups; dense feed-forward width; routed
    # experts: how many, how many per token, their width (top * expert_ff = ff: a token does the dense layer's work)
    "2k": dict(width=2048, heads=16, kv=4, dim=128, chunk=1024, rot=64, l_heads=16, l_dim=128, l_vdim=128, ss_heads=64, ss_dim=64,
               state=128, groups=8, ff=8192, experts=32, top=4, expert_ff=2048),
    "4k": dict(width=4096, heads=32, kv=8, dim=128, chunk=1024, rot=64, l_heads=32, l_dim=128, l_vdim=128, ss_heads=128, ss_dim=64,
               state=128, groups=8, ff=12288, experts=64, top=6, expert_ff=2048),
}


def pepolorn_config(z, layers, vocab):
    """Layers that resemble a real model's: a state-space layer with a dense feed-forward first, then chunked attention
    beside linear attention, then state-space layers, all with routed experts; the fifth layer runs the second's weights."""
    par = {"left": {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["dim"], "vdim": z["dim"], "scale": 8.0 * z["dim"] ** -0.5,
                    "mask": {"size": z["chunk"]},
                    "rot": {"dims": z["rot"], "base": 500000.0, "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}},
           "right": {"heads": z["l_heads"], "dim": z["l_dim"], "vdim": z["l_vdim"],
                     "decay": [1.0 - 2.0 ** -(3 + 6 * h / max(1, z["l_heads"] - 1)) for h in range(z["l_heads"])]},
           "left_scale": 1.0, "right_scale": 1.0}
    ssm = {"heads": z["ss_heads"], "vdim": z["ss_dim"], "state": z["state"], "groups": z["groups"], "conv": 4, "norm_groups": z["groups"]}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": 4, "keep": 2}}}
    out = []
    for i in range(layers):
        layer = {"type": "parallel", "mixer": par, "mlp": moe} if i % 3 == 1 else \
                {"type": "mamba2", "mixer": ssm, "mlp": {"kind": "dense", "ff": z["ff"]} if i == 0 else moe}
        if i == 4:
            layer = dict(layer, weights_of=1)
        out.append(layer)
    return {"architecture": "Pepolorn", "vocab": vocab, "width": z["width"], "norm": {"eps": 1e-6}, "layers": out}


def pepolorn_kernels(pk, size):
    """The new design's kernels beside their like of the closest model, one launch each: chunked attention beside Kolisun's
    window attention, over a prompt of 2,048 tokens and for 8 decoded tokens; the kernel between projection and attention
    (rotation, then the norm per head) beside Kolisun's; the decaying-state scan beside the state-space scan, against the
    bytes and operations they must do; the gate and norm behind it; the router's choice; the GELU-gated product beside the
    SiLU-gated one."""
    import torch
    from prelude_b200.cache.manager import CacheManager
    from prelude_b200.engine.batch import StepItem, build_step_batch
    from prelude_b200.ops import kernels as K
    from prelude_b200.ops import linear as L
    from prelude_b200.ops.attention import paged_attention
    from prelude_b200.ops.paged_general import attention_general
    from prelude_b200.parts.registry import CombinedNeed, KvPagesNeed, StateNeed
    z, kz = PEPOLORN_SIZES[size], KOLISUN_SIZES[size]
    dev = torch.device("cuda:0")
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    bf = torch.bfloat16
    out = {}
    T, B = 2048, 8
    H, G, D, chunk = z["heads"], z["kv"], z["dim"], z["chunk"]
    ctx = 2 * chunk - 1                                      # the decoded token is the last of its chunk
    LH, LN, LP = z["l_heads"], z["l_dim"], z["l_vdim"]
    SH, P, N, SG = kz["ss_heads"], kz["ss_dim"], kz["state"], kz["groups"]
    s_inner, s_channels = SH * P, SH * P + 2 * SG * N
    l_cols = LH * (LP + 2 * LN)
    needs = [KvPagesNeed(G, D, chunk=chunk), KvPagesNeed(G, D), StateNeed((LH, LN, LP), torch.float32),
             CombinedNeed((StateNeed((SH, N, P), torch.float32), StateNeed((3, s_channels), None)))]
    cache = CacheManager(needs, PAGE_SIZE, (B * (ctx + 16) + T) // PAGE_SIZE + 8, B + 1, dev, bf)
    gen, plain = cache.layer_cache(0), cache.layer_cache(1)
    for lc in (gen, plain):
        lc.k_pages.normal_()
        lc.v_pages.normal_()
    scale = D ** -0.5
    # -- one request of T prompt tokens
    cache.add_request("p")
    cache.grow("p", T)
    batch = build_step_batch([StepItem("p", [0] * T, 0, [])], cache.block_tables(["p"]), [cache.slot_of("p")], dev, 10, 1 << 20)
    cache.zero_fresh_state()
    c_pairs = sum(i % chunk + 1 for i in range(T))
    k_pairs = sum(min(i + 1, kz["window"]) for i in range(T))
    q = torch.randn(T, H, D, device=dev).to(bf)
    g0, g1 = cache.group_of[0], cache.group_of[1]
    ms = _event_ms(lambda: attention_general(q, gen.k_pages, gen.v_pages, D, batch, g0, scale, None, None, chunk=chunk), flush=flush)
    out["prefill_attention"] = {"chunked_ms": round(ms, 4), "chunked_tflops": round(H * c_pairs * 4 * D / ms / 1e9, 1)}
    ms = _event_ms(lambda: paged_attention(q, plain.k_pages, plain.v_pages, batch, g1, scale, kz["window"]), flush=flush)
    out["prefill_attention"].update(kolisun_window_ms=round(ms, 4), kolisun_window_tflops=round(H * k_pairs * 4 * D / ms / 1e9, 1))
    # the kernel between projection and attention
    proj = torch.randn(T, (H + 2 * G) * D, device=dev).to(bf)
    rates = torch.rand(z["rot"] // 2, device=dev)
    qo = torch.empty(T, H, D, dtype=bf, device=dev)
    moved = T * (H + 2 * G) * D * 2 * 2
    ms = _event_ms(lambda: K.heads_prepare(proj[:, :H * D], proj[:, H * D:(H + G) * D], proj[:, (H + G) * D:], n_heads=H, q_dim=D, eps=1e-6,
                                           norm="after", rates=rates, amplitude=1.2, rot_dims=z["rot"], positions=batch.positions,
                                           table_row=batch.table_row_of_token, block_table=batch.block_tables[g0], q_out=qo,
                                           k_pages=gen.k_pages, v_pages=gen.v_pages, status=batch.status), flush=flush)
    out["projection_to_pages"] = {"rotate_norm_us": round(ms * 1e3, 2), "rotate_norm_gbs": round(moved / ms / 1e6, 1)}
    wq, wk = torch.ones(H * D, device=dev), torch.ones(G * D, device=dev)
    full = torch.rand(D // 2, device=dev)
    ms = _event_ms(lambda: K.qkv_prepare(proj[:, :H * D], proj[:, H * D:(H + G) * D], proj[:, (H + G) * D:], n_heads=H, q_dim=D, q_weight=wq,
                                         k_weight=wk, k_norm_cols=G * D, eps=1e-6, rates=full, rot_dims=D, adjacent=True,
                                         positions=batch.positions, table_row=batch.table_row_of_token, block_table=batch.block_tables[g1],
                                         q_out=qo, k_pages=plain.k_pages, v_pages=plain.v_pages, swizzle_k=True, swizzle_v=True,
                                         status=batch.status), flush=flush)
    out["projection_to_pages"].update(kolisun_us=round(ms * 1e3, 2), kolisun_gbs=round(moved / ms / 1e6, 1))
    # the recurrences over the prompt
    l_state = cache.layer_cache(2).state
    lproj = (torch.randn(T, l_cols + LH * LP, device=dev) * 0.5).to(bf)
    decay = torch.linspace(0.9, 0.999, LH, device=dev)
    ly = K.decay_scan(lproj, decay, l_state, batch)
    ms_l = _event_ms(lambda: K.decay_scan(lproj, decay, l_state, batch, out=ly), flush=flush)
    nw = torch.ones(LH * LP, device=dev)
    ms_n = _event_ms(lambda: K.gated_group_rmsnorm(ly, lproj[:, l_cols:], nw, 1, 1e-6, gate_after=True, sigmoid_gate=True), flush=flush)
    out["linear_attention_prefill"] = {
        "scan_us": round(ms_l * 1e3, 2), "scan_gbs": round((T * l_cols * 2 + T * LH * LP * 4) / ms_l / 1e6, 1),
        "scan_gflops": round(T * LH * LN * LP * 4 / ms_l / 1e6, 1), "us_per_token": round(ms_l * 1e3 / T, 3),
        "gated_norm_us": round(ms_n * 1e3, 2), "gated_norm_gbs": round(T * LH * LP * (4 + 2 + 2) / ms_n / 1e6, 1)}
    sc = cache.layer_cache(3)
    s_state, s_carried = sc.children[0].state, sc.children[1].state
    sproj = (torch.randn(T, 2 * s_inner + 2 * SG * N + SH, device=dev) * 0.5).to(bf)
    xbc, dt = sproj[:, s_inner:s_inner + s_channels], sproj[:, s_inner + s_channels:]
    s_conv, s_b = torch.randn(s_channels, 4, device=dev) * 0.5, torch.zeros(s_channels, device=dev)
    shb, sal, sdd = torch.zeros(SH, device=dev), torch.zeros(SH, device=dev), torch.ones(SH, device=dev)
    su = K.causal_conv_silu(xbc, s_conv, s_b, s_carried, batch)
    sy = K.ssm_scan(su, dt, shb, sal, sdd, s_state, batch, SG)
    ms_k = _event_ms(lambda: K.ssm_scan(su, dt, shb, sal, sdd, s_state, batch, SG, out=sy), flush=flush)
    out["state_space_prefill"] = {"scan_us": round(ms_k * 1e3, 2), "scan_gbs": round((T * s_channels * 2 + T * s_inner * 4) / ms_k / 1e6, 1),
                                  "scan_gflops": round(T * SH * N * P * 6 / ms_k / 1e6, 1), "us_per_token": round(ms_k * 1e3 / T, 3)}
    # the router's choice, with and without the correction, and the GELU-gated product beside the SiLU-gated one
    logits = torch.randn(T, z["experts"], device=dev)
    corr = torch.randn(z["experts"], device=dev) * 0.3
    ms_r = _event_ms(lambda: K.moe_route(logits, z["top"], 4, 2, 2, False, corr), flush=flush)
    ms_p = _event_ms(lambda: K.moe_route(logits, z["top"], 4, 2, 2, False, None), flush=flush)
    out["router_choice"] = {"corrected_us": round(ms_r * 1e3, 2), "plain_us": round(ms_p * 1e3, 2)}
    x = (torch.randn(T, z["width"], device=dev) * 0.5).to(bf)
    w_gu = (torch.randn(2 * z["ff"], z["width"], device=dev) * 0.02).to(bf)
    fl = 2.0 * T * 2 * z["ff"] * z["width"]
    ms_g = _event_ms(lambda: L.gated_linear_gelu_tanh(x, w_gu), flush=flush)
    ms_s = _event_ms(lambda: L.gated_linear_silu(x, w_gu), flush=flush)
    out["gated_product_prefill"] = {"gelu_us": round(ms_g * 1e3, 2), "gelu_tflops": round(fl / ms_g / 1e9, 1),
                                    "silu_us": round(ms_s * 1e3, 2), "silu_tflops": round(fl / ms_s / 1e9, 1)}
    cache.release("p")
    # -- B single tokens at ctx keys
    rids = [f"d{i}" for i in range(B)]
    for r in rids:
        cache.add_request(r)
        cache.grow(r, ctx + 1)
        cache.trim(r)
    batch = build_step_batch([StepItem(r, [0], ctx, []) for r in rids], cache.block_tables(rids), [cache.slot_of(r) for r in rids], dev, 10, 1 << 20)
    cache.zero_fresh_state()
    q = torch.randn(B, H, D, device=dev).to(bf)
    row_bytes = G * 2 * D * 2
    ms = _event_ms(lambda: attention_general(q, gen.k_pages, gen.v_pages, D, batch, g0, scale, None, None, chunk=chunk), flush=flush, reps=20)
    out["decode_attention"] = {"chunked_us": round(ms * 1e3, 2), "chunked_gbs": round(B * chunk * row_bytes / ms / 1e6, 1)}
    ms = _event_ms(lambda: paged_attention(q, plain.k_pages, plain.v_pages, batch, g1, scale, kz["window"]), flush=flush, reps=20)
    out["decode_attention"].update(kolisun_window_us=round(ms * 1e3, 2), kolisun_window_gbs=round(B * kz["window"] * row_bytes / ms / 1e6, 1))
    ms = _event_ms(lambda: K.decay_scan(lproj[:B], decay, l_state, batch, out=ly[:B]), flush=flush, reps=20)
    out["linear_attention_decode"] = {"scan_us": round(ms * 1e3, 2), "scan_state_gbs": round(B * LH * LN * LP * 4 * 2 / ms / 1e6, 1)}
    ms = _event_ms(lambda: K.ssm_scan(su[:B], dt[:B], shb, sal, sdd, s_state, batch, SG, out=sy[:B]), flush=flush, reps=20)
    out["state_space_decode"] = {"scan_us": round(ms * 1e3, 2), "scan_state_gbs": round(B * SH * N * P * 4 * 2 / ms / 1e6, 1)}
    xs = x[:B].contiguous()
    wb = 2 * z["ff"] * z["width"] * 2
    ms_g = _event_ms(lambda: L.gated_linear_gelu_tanh(xs, w_gu), flush=flush, reps=20)
    ms_s = _event_ms(lambda: L.gated_linear_silu(xs, w_gu), flush=flush, reps=20)
    out["gated_product_decode"] = {"gelu_us": round(ms_g * 1e3, 2), "gelu_gbs": round(wb / ms_g / 1e6, 1),
                                   "silu_us": round(ms_s * 1e3, 2), "silu_gbs": round(wb / ms_s / 1e6, 1)}
    out["peaks"] = {"bf16_tflops": pk["bf16_tflops"], "hbm_gbs": pk["hbm_gbs"], "source": pk["source"]}
    return out


def pepolorn_compare(args):
    """Prefill and decode throughput of Pepolorn beside Kolisun and Qwen3 dense at equal layer sizes (random weights,
    bfloat16): one prompt of --prefill-tokens through the step function, and --batch requests decoding behind
    --prefix-len tokens on the captured step, both timed on the device.  One JSON line of its own."""
    import torch
    pk = peaks()
    clocks = ClockSampler()
    clocks.start()
    t_begin = time.time()
    points = []
    vocab = 32768
    for size in args.sizes.split(","):
        z = PEPOLORN_SIZES[size]
        layers = args.layers or 6
        arms = {
            "pepolorn": pepolorn_config(z, layers, vocab),
            "kolisun": kolisun_config(KOLISUN_SIZES[size], layers, vocab),
            "qwen3": dict(QWEN3_4B, vocab_size=vocab, hidden_size=z["width"], intermediate_size=z["ff"], num_hidden_layers=layers,
                          num_attention_heads=z["heads"], num_key_value_heads=z["kv"], head_dim=z["dim"], tie_word_embeddings=True),
        }
        point = {"size": size, "layers": layers, "width": z["width"]}
        for name, cfg in arms.items():
            pages_per_req = -(-(PREFIX_LEN + args.warmup + args.steps + 2) // PAGE_SIZE)
            engine = _engine_for(cfg, args.batch * pages_per_req + 2 * (PREFILL_TOKENS // PAGE_SIZE) + 8, args.batch + 2)
            shim = {"vocab_size": vocab}
            prefill_ms, _ = time_prefill(engine, shim, args.warmup)
            dec, _ = time_decode(engine, shim, args.batch, args.steps, args.warmup, seed=1)
            point[name] = {"prefill_tok_s": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 3),
                           "decode_tok_s": round(dec["tok_s"], 1), "decode_ms_per_step": round(dec["ms_per_step"], 4),
                           "weight_gb": round(engine.model.weight_bytes() / 1e9, 3)}
            del engine
            torch.cuda.empty_cache()
        point["kernels"] = pepolorn_kernels(pk, size)
        points.append(point)
    clocks.stop()
    print(json.dumps({"metric": "Pepolorn beside Kolisun and Qwen3 dense at equal layer sizes: prefill and decode tokens a second, device-timed",
                      "unit": "tok/s", "n_gpus": 1, "dtype": "bf16", "data": "synthetic", "impl": "ours", "steps": args.steps,
                      "warmup": args.warmup, "config": {"batch": args.batch, "prefix_len": PREFIX_LEN, "prefill_tokens": PREFILL_TOKENS,
                                                        "page_size": PAGE_SIZE, "l2": "inputs_exceed_l2 (steps), flushed (kernels)"},
                      "points": points, "clocks": clocks.summary([(t_begin, time.time())])}))
    return 0


def serve(args):
    """A mixed continuous batch through ``Engine.generate`` (host tokens in, host tokens out): ``--requests`` prompts
    of uniform random ids with lengths uniform in [128, 2048], prompts cut into portions of ``--prefill-chunk``
    tokens beside the running decodes, ``--new-tokens`` greedy tokens each.  One JSON line of its own."""
    import copy
    import random
    import time
    import torch
    rng = random.Random(7)
    lens = [rng.randint(128, 2048) for _ in range(args.requests)]
    pages = sum(-(-(n + args.new_tokens + 1) // PAGE_SIZE) for n in lens) + 64
    engine, cfg = build_engine(args.layers, args.requests, pages, prefill_chunk=args.prefill_chunk)
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    engine.warmup(range(1, args.requests + 1))
    engine.warmup_prompt_steps([args.prefill_chunk])
    engine.generate(prompts[:2], temperature=0.0, max_new_tokens=4, ignore_eos=True)
    before = copy.copy(engine.stats())
    torch.cuda.synchronize()
    clocks = ClockSampler()
    clocks.start()
    t0 = time.time()
    results = engine.generate(prompts, temperature=0.0, max_new_tokens=args.new_tokens, ignore_eos=True)
    torch.cuda.synchronize()
    t1 = time.time()
    clocks.stop()
    st = engine.stats()
    out_tokens = sum(r.completion_tokens for r in results)
    ttft = sorted(r.ttft_ms for r in results)
    line = {
        "metric": f"serving: {args.requests} requests, prompts of 128 to 2,048 tokens in portions of {args.prefill_chunk}, "
                  f"{args.new_tokens} greedy tokens each (Qwen3-{args.model_size.upper()} sizes, random weights, bf16)",
        "value": round(out_tokens / (t1 - t0), 1), "unit": "generated tok/s", "n_gpus": 1, "higher_is_better": True,
        "dtype": "bf16", "data": "synthetic", "impl": "ours", "seconds": round(t1 - t0, 3),
        "prompt_tokens": sum(lens), "generated_tokens": out_tokens,
        "total_tok_s": round((sum(lens) + out_tokens) / (t1 - t0), 1),
        "ttft_ms": {"p50": round(statistics.median(ttft), 1), "p95": round(ttft[int(0.95 * (len(ttft) - 1))], 1), "max": round(ttft[-1], 1)},
        "steps": st.steps - before.steps, "decode_steps": st.decode_steps - before.decode_steps,
        "captured_steps": st.graph_steps - before.graph_steps, "preemptions": st.preemptions - before.preemptions,
        "config": {"model": f"qwen3-{args.model_size}-sizes", "layers": args.layers, "layers_full": MODEL["num_hidden_layers"],
                   "requests": args.requests, "prefill_chunk": args.prefill_chunk, "new_tokens": args.new_tokens, "page_size": PAGE_SIZE},
        "clocks": clocks.summary([(t0, t1)]),
    }
    print(json.dumps(line))
    return 0


def main():
    global MODEL, PREFIX_LEN, CONTEXT_LEN, PAGE_SIZE, PREFILL_TOKENS, TIMELINE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    ap.add_argument("--model-size", default="4b", choices=["4b", "8b", "32b"],
                    help="layer sizes of another Qwen3 dense model (the headline run is 4b)")
    ap.add_argument("--prefix-len", type=int, default=PREFIX_LEN, help="tokens every request holds before the timed decode steps")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="length of the timed prompt (the contract's is 2,048)")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per page of the key/value cache")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--timeline", action="store_true",
                    help="print the kernels' timeline of one layer of the decode step to stderr (needs PRELUDE_TIMELINE=1 in the environment)")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving", "pabelix", "kolisun", "nedesun", "pepolorn"],
                    help="serving: a mixed continuous batch through Engine.generate instead of the decode step (a line of its own); "
                         "pabelix, kolisun: that design beside Qwen3 dense at equal layer sizes (a line of its own); "
                         "nedesun, pepolorn: that design beside Kolisun and Qwen3 dense at equal layer sizes (a line of its own)")
    ap.add_argument("--sizes", default="2k,4k", help="pabelix, kolisun, nedesun, pepolorn: which layer sizes to run (2k, 4k)")
    ap.add_argument("--requests", type=int, default=32, help="serving: number of requests")
    ap.add_argument("--prefill-chunk", type=int, default=512, help="serving: tokens per portion of a prompt")
    ap.add_argument("--new-tokens", type=int, default=256, help="serving: generated tokens per request")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pip install of the reference fails (not installable: neither setup.py nor pyproject.toml; a Rust workspace with git-only "
                          "dependencies, no cargo or rustc and no network here)"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus N with N > 1 is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    TIMELINE = args.timeline
    if args.model_size != "4b":
        MODEL = dict(QWEN3_4B, **OTHER_SIZES[args.model_size])
    PREFIX_LEN = args.prefix_len
    PAGE_SIZE = args.page_size
    PREFILL_TOKENS = args.prefill_tokens
    CONTEXT_LEN = max(CONTEXT_LEN, PREFIX_LEN + args.steps + args.warmup + 64, PREFILL_TOKENS + 64)
    args.layers = args.layers or MODEL["num_hidden_layers"]
    if args.workload == "serving":
        CONTEXT_LEN = max(CONTEXT_LEN, 2048 + args.new_tokens + 64)
        return serve(args)
    if args.workload == "pabelix":
        args.layers = 0 if args.layers == MODEL["num_hidden_layers"] else args.layers
        return pabelix_compare(args)
    if args.workload == "kolisun":
        args.layers = 0 if args.layers == MODEL["num_hidden_layers"] else args.layers
        return kolisun_compare(args)
    if args.workload == "nedesun":
        args.layers = 0 if args.layers == MODEL["num_hidden_layers"] else args.layers
        return nedesun_compare(args)
    if args.workload == "pepolorn":
        args.layers = 0 if args.layers == MODEL["num_hidden_layers"] else args.layers
        return pepolorn_compare(args)
    import torch
    pk = peaks()
    # cache: the largest point (64 requests) with room for prefix + generated tokens, in whole pages
    biggest = 64 if not args.no_points else args.batch
    pages_per_req = -(-(PREFIX_LEN + args.warmup + args.steps + 2) // PAGE_SIZE)
    num_pages = max(biggest, args.batch) * pages_per_req + 2 * (PREFILL_TOKENS // PAGE_SIZE) + 8
    engine, cfg = build_engine(args.layers, max(64, args.batch) + 2, num_pages)
    clocks = ClockSampler()
    clocks.start()
    windows = []

    prefill_ms, w = time_prefill(engine, cfg, args.warmup)
    windows.append(w)
    dec, library = time_decode(engine, cfg, args.batch, args.steps, args.warmup, seed=1)
    windows.append(dec["window"])
    points = {}
    if not args.no_points:
        for b, k in ((1, min(args.steps, 128)), (64, min(args.steps, 64))):
            if b == args.batch:
                points[f"decode_b{b}"] = round(dec["tok_s"], 1)
                continue
            d, _ = time_decode(engine, cfg, b, k, args.warmup, seed=100 + b)
            windows.append(d["window"])
            points[f"decode_b{b}"] = round(d["tok_s"], 1)
    e2e, w = time_e2e(engine, cfg, args.batch, args.steps)
    windows.append(w)
    clocks.stop()

    launches_per_step = engine.graphs.get(args.batch).launches
    step_bytes = weight_bytes_per_step(cfg) + args.batch * dec["avg_ctx"] * kv_bytes_per_token(cfg)
    achieved = step_bytes / (dec["ms_per_step"] / 1e3) / 1e9
    pf = prefill_flops(cfg, PREFILL_TOKENS)
    line = {
        "metric": f"decode tok/s (Qwen3-{args.model_size.upper()} sizes, random weights, bf16, batch {args.batch}, "
                  f"{PREFIX_LEN:,}-token prefixes)",
        "value": round(dec["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dec["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": f"qwen3-{args.model_size}-sizes", "layers": args.layers, "layers_full": MODEL["num_hidden_layers"],
                   "hidden_size": cfg["hidden_size"], "intermediate_size": cfg["intermediate_size"],
                   "num_attention_heads": cfg["num_attention_heads"], "num_key_value_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "vocab_size": cfg["vocab_size"], "tie_word_embeddings": cfg["tie_word_embeddings"],
                   "global_batch": args.batch, "seq_len": PREFIX_LEN, "context_len": CONTEXT_LEN,
                   "page_size": PAGE_SIZE, "prefill_tokens": PREFILL_TOKENS, "parallelism": "single",
                   "l2": "inputs_exceed_l2", "peaks": pk["source"]},
        "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items() if k != "decode_ms"},
        "gpu_launches": int(launches_per_step * args.steps),
        "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(pf / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks.summary(windows),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
