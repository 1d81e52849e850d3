"""Benchmark of the int8 weight-only LLaMA-7B-architecture decode path (batch 8, prompt 512, greedy decode) plus
the W8A16 GEMM sweep over the LLaMA-7B projection shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one greedy decode step of the whole batch (B = 8 sequences, prompt 512, random-init weights
quantized to int8 on the fly, synthetic token ids).  The timed region of K steps is repeated (same range of
cache lengths every time, W warm-up steps before each repeat) until the clock sampler has seen at least a second
of load, at least five times; the MEDIAN repeat is reported, the per-repeat list is kept in the line.  Rank 0
prints ONE JSON line:

  value      tokens/s over K timed decode steps with the token ids already on the device (CUDA events)
  e2e        tokens/s through the public model API with the ids coming from pinned host memory and the
             chosen tokens read back to the host every step
  roofline   the W8A16 skinny GEMM (dominant kernel): algorithmic bytes / measured kernel time vs the
             measured HBM copy bandwidth
  gemm_sweep GB/s and TFLOP/s of the GEMM for the LLaMA-7B projection shapes over M (N = 1 only)
  tp_parity  after the timing: a 2-layer model of the same architecture and the same tensor-parallel degree,
             prompt + decode steps, rank 0's logits against the CPU oracle (a check, not a measurement)
  cpu_baseline  the CPU oracle (a port of the reference's arithmetic; the reference has no CPU path) on a
             bounded sample, on this host's cores

`--impl reference` times that CPU port alone and prints the same line shape with "impl": "reference".
For N > 1 launch with torchrun; the model is sharded Megatron-style (strong scaling).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
import types

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "int8_llama7b_decode_tokens_per_s"
UNIT = "tokens/s"
CFG = dict(hidden_size=4096, num_attention_heads=32, num_hidden_layers=32, intermediate_size=11008, vocab_size=32000,
           rms_norm_eps=1e-6, hidden_act="silu", pad_token_id=None)
BATCH, PROMPT = 8, 512
WORKLOAD, FAMILY = "llama7b_arch_int8_decode_b8_prompt512", "llama"
# The lm_head runs through the W8A16 path as well, its vocabulary sharded over the tensor-parallel ranks
# (--lm-head fp16 keeps the reference's replicated fp16 torch.nn.Linear instead).
LM_HEAD_INT8 = True

# The headline configuration above is what a run without --workload measures.  The two other model-level
# configurations of the reference's latency scripts are selectable for additional lines:
WORKLOADS = {
    "llama7b": None,
    # Baichuan-13B architecture (ALiBi attention op), batch 32, prompt 256
    "baichuan13b": dict(metric="int8_baichuan13b_decode_tokens_per_s", workload="baichuan13b_arch_int8_decode_b32_prompt256",
                        family="baichuan", batch=32, prompt=256,
                        cfg=dict(hidden_size=5120, num_attention_heads=40, num_hidden_layers=40, intermediate_size=13696,
                                 vocab_size=64000)),
    # LLaMA-65B architecture, batch 64, prompt 1024: weights + KV cache need at least two GPUs
    "llama65b": dict(metric="int8_llama65b_decode_tokens_per_s", workload="llama65b_arch_int8_decode_b64_prompt1024",
                     family="llama", batch=64, prompt=1024,
                     cfg=dict(hidden_size=8192, num_attention_heads=64, num_hidden_layers=80, intermediate_size=22016,
                              vocab_size=32000)),
}


def select_workload(name):
    global METRIC, BATCH, PROMPT, WORKLOAD, FAMILY
    w = WORKLOADS[name]
    if w is None:
        return
    METRIC, WORKLOAD, FAMILY, BATCH, PROMPT = w["metric"], w["workload"], w["family"], w["batch"], w["prompt"]
    CFG.update(w["cfg"])


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                mhz.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


# ------------------------------------------------------------------------------------------------ model
def random_eet_dict(cfg, dev):
    """Random-init weights of the architecture `cfg` (N(0, 0.02^2), fp16) generated on the GPU and quantized by the
    library's quantizer, as the dictionary from_eet() takes.  Every rank draws the same full matrices (same seed)."""
    from eet_b200 import EET
    gen = torch.Generator(device=dev).manual_seed(0)
    h, f, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size

    def qw(k, n):
        w = (torch.randn(n, k, generator=gen, device=dev, dtype=torch.float32) * 0.02).half().t().contiguous()
        return EET.quant_weights(w, torch.int8, False)

    d = {"embed_tokens.weight": (torch.randn(v, h, generator=gen, device=dev) * 0.02).half(),
         "norm.weight": torch.ones(h, device=dev).half(),
         "lm_head.weight": (torch.randn(v, h, generator=gen, device=dev) * 0.02).half()}
    for i in range(cfg.num_hidden_layers):
        p = f"layer.{i}."
        for name, (k, n) in (("self_attn.qkv_proj", (h, 3 * h)), ("self_attn.out_proj", (h, h)),
                             ("ffn.intermediate_0", (h, f)), ("ffn.intermediate_1", (h, f)), ("ffn.output", (f, h))):
            d[p + name + ".weight"], d[p + name + ".scale"] = qw(k, n)
        d[p + "self_attn.layernorm.weight"] = torch.ones(h, device=dev).half()
        d[p + "ffn.layernorm.weight"] = torch.ones(h, device=dev).half()
    return d


def build_model(tp, device_index, t_max, layers=None, batch=None, prompt=None, keep_dict=False):
    """The selected architecture with random weights, assembled through the public from_eet() entry point; every
    rank keeps its shard."""
    from eet_b200 import modeling
    cfg = types.SimpleNamespace(**CFG)
    if layers:
        cfg.num_hidden_layers = layers
    dev = torch.device("cuda", device_index)
    d = random_eet_dict(cfg, dev)
    cls = modeling.EETBaichuanForCausalLM if FAMILY == "baichuan" else modeling.EETLlamaForCausalLM
    model = cls.from_eet(d, cfg, batch or BATCH, prompt or PROMPT, t_max, torch.int8, device_id=device_index, tp=tp,
                         lm_head_int8=LM_HEAD_INT8)
    return (model, cfg, d) if keep_dict else (model, cfg)


def rewind(model, step):
    """Puts every attention op back to a history of `step` tokens (the cache contents beyond it are simply
    overwritten again), so that every repeat of a timed region walks the same range of cache lengths.  A
    captured decode graph stays valid: only the device-resident step counters are set back."""
    model.model.past_kv_length = step
    for layer in model.model.layers:
        layer.attention.step_ = step
        if layer.attention.use_device_step:
            layer.attention.sync_device_step()


def kernel_launches_per_step(n_layers, batch, world):
    """Launches of this library's kernels in one decode step (NCCL and torch kernels are not counted)."""
    head = 2 if LM_HEAD_INT8 else 1   # int8: lm_head GEMM + fused argmax; fp16: argmax (the GEMM is cuBLAS, not counted)
    if batch <= 64:
        # per layer: rmsnorm(+finalize), qkv gemm, decode attention, out gemm, rmsnorm(+finalize), gate+up gemm,
        # swiglu(+finalize), down gemm; per step: advance_steps, embedding gather, final rmsnorm(+finalize), lm_head
        return 8 * n_layers + 3 + head
    # larger batches: every projection is an accumulate + finalize pair, gate and up are separate launches
    # (and with tensor parallelism the residual is added by its own kernel after the NCCL all-reduce)
    per_layer = 14 + (2 if world > 1 else 0)
    return per_layer * n_layers + 3 + head


# ------------------------------------------------------------------------------------------------ GEMM timing
def _time_graph(fn, iters_in_graph, reps=5):
    """Captures `fn` (which enqueues iters_in_graph launches) into a CUDA graph and returns the best time per
    launch over `reps` replays: kernel time without the host cost of a Python/ctypes launch."""
    fn()  # eager once: sizes pooled scratch, sets function attributes
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    best = None
    for _ in range(reps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        e1.synchronize()
        t = e0.elapsed_time(e1) * 1e-3 / iters_in_graph
        best = t if best is None else min(best, t)
    return best


def time_gemm_shapes(model, batch):
    """Times the skinny GEMM kernel alone (the accumulate kernel, without the epilogue that the next kernel
    of a decode step performs) on the real weights of the model: for each of the five projection shapes, all
    layers' launches back to back inside one CUDA graph between two CUDA events (one distinct weight buffer
    per layer, GBs in total, so nothing is served from L2).  Returns per-shape results."""
    from eet_b200 import EET
    dev = model.model.desc.device
    per = {}
    layers = model.model.layers
    shapes = (("qkv", "qkv_w", "qkv_s"), ("out", "out_w", "out_s"), ("gate", "w0", "s0"), ("up", "w1", "s1"),
              ("down", "w2", "s2"))
    for name, wn, sn in shapes:
        K, N = getattr(layers[0], wn).shape
        x = torch.randn(batch, K, device=dev).half()
        sums = torch.zeros(batch, N, device=dev, dtype=torch.float32)

        def run():
            for layer in layers:
                EET.gemm_w8a16_accum(x, getattr(layer, wn), sums)

        t = _time_graph(run, len(layers))
        nbytes = N * K + 2 * N + 2 * batch * K + 2 * batch * N
        per[name] = {"K": K, "N": N, "M": batch, "us": t * 1e6, "bytes": nbytes, "gbs": nbytes / t / 1e9}
    return per


def skinny_steady_state(device, batch, hbm_peak):
    """The decode GEMM kernel on a matrix large enough to leave its launch ramp behind: K=8192, N=22016 (the
    FFN shape of configs[4], 180 MB per buffer, 3 rotating buffers), M = the workload's batch capped at 8."""
    from eet_b200 import EET
    K, N, M = 8192, 22016, min(batch, 8)
    ws = [torch.randint(-128, 128, (K, N), dtype=torch.int8, device=device) for _ in range(3)]
    x = torch.randn(M, K, device=device).half()
    sums = torch.zeros(M, N, device=device, dtype=torch.float32)

    def run():
        for i in range(12):
            EET.gemm_w8a16_accum(x, ws[i % 3], sums)

    t = _time_graph(run, 12)
    nbytes = N * K + 2 * N + 2 * M * K + 2 * M * N
    return {"K": K, "N": N, "M": M, "us": round(t * 1e6, 2), "achieved": round(nbytes / t / 1e9, 1),
            "frac": round(nbytes / t / 1e9 / hbm_peak, 4)}


def gemm_sweep(device, hbm_peak, tflops_peak):
    """configs[1]: K x N in {4096x4096, 4096x11008, 11008x4096}, M in {1..4096}; 8 rotating weight buffers
    (134-360 MB per shape, more than the 126 MB L2), launches replayed from a CUDA graph."""
    from eet_b200 import EET
    res = []
    for K, N in ((4096, 4096), (4096, 11008), (11008, 4096)):
        nbuf = 8
        ws = [torch.randint(-128, 128, (K, N), dtype=torch.int8, device=device) for _ in range(nbuf)]
        s = (torch.rand(N, device=device) * 1e-3).half()
        for M in (1, 2, 4, 8, 16, 64, 256, 1024, 4096):
            x = torch.randn(M, K, device=device).half()
            out = torch.empty(M, N, device=device, dtype=torch.float16)
            iters = 32 if M <= 64 else 8

            def run():
                for i in range(iters):
                    EET.gemm_w8a16(x, ws[i % nbuf], s, out=out)

            t = _time_graph(run, iters, reps=3)
            nbytes = N * K + 2 * N + 2 * M * K + 2 * M * N
            flops = 2.0 * M * N * K
            t_roof = max(nbytes / (hbm_peak * 1e9), flops / (tflops_peak * 1e12))
            res.append({"K": K, "N": N, "M": M, "us": round(t * 1e6, 2), "gbs": round(nbytes / t / 1e9, 1),
                        "tflops": round(flops / t / 1e12, 2), "frac_of_roofline": round(t_roof / t, 4)})
        del ws
    return res


# ------------------------------------------------------------------------------------------------ CPU port
def cpu_decode_sample(steps, warmup=1, budget_s=15.0, threads=None):
    """Times the CPU oracle on the workload's decode step: fp32 torch ops on all host cores, batch and history of
    the workload, synthetic int8 weights (distinct buffers per layer).  As many of the architecture's layers as fit
    `budget_s` for `warmup + steps` steps are run - all of them when they fit - and the step time is scaled to the
    full depth otherwise (decoder layers are identical in cost).  Returns a dict with tokens/s, the measured and
    the scaled step time, layers run, cores and a description."""
    from oracle import ops
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    cfg = types.SimpleNamespace(**CFG)
    h, f, H, D, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, 128, cfg.num_hidden_layers
    gen = torch.Generator().manual_seed(0)
    shapes = ((h, 3 * h), (h, h), (h, f), (h, f), (f, h))
    base = [torch.randint(-128, 128, kn, generator=gen, dtype=torch.int8) for kn in shapes]
    scales = [(torch.rand(n, generator=gen) * 3e-4 + 1e-4).half() for _, n in shapes]

    def layer(i):
        # same value distribution in every layer, its own memory: rotated copies of the first layer's matrices
        args = []
        for q, sc in zip(base, scales):
            args.extend((q if i == 0 else torch.roll(q, i, 0), sc))
        return ops.LayerWeights(*args, torch.ones(h).half(), torch.ones(h).half())

    def make(n_layers):
        dec = ops.DecoderOracle([layer(i) for i in range(n_layers)], H, D, cfg.rms_norm_eps, PROMPT + warmup + steps + 2, BATCH)
        for c in dec.kc + dec.vc:
            c[:, :, :PROMPT] = torch.randn(BATCH, H, PROMPT, D, generator=gen).half()
        dec.step = PROMPT
        return dec

    x = torch.randn(BATCH, 1, h, generator=gen).half()
    probe = make(1)
    probe.forward(x, False)
    t0 = time.perf_counter()
    probe.forward(x, False)
    t_layer = time.perf_counter() - t0
    n_layers = int(max(1, min(L, budget_s / ((warmup + steps) * t_layer))))
    dec = probe if n_layers == 1 else make(n_layers)
    dec.step = PROMPT
    for _ in range(warmup):
        dec.forward(x, False)
    t0 = time.perf_counter()
    for _ in range(steps):
        dec.forward(x, False)
    dt = (time.perf_counter() - t0) / steps
    factor = L / n_layers
    sample = (f"{steps} decode steps (+{warmup} warm-up) of {n_layers} of {L} layers (batch {BATCH}, history {PROMPT}); "
              f"torch fp32 ops on {threads} threads" + ("" if n_layers == L else f"; step time scaled by {L}/{n_layers}"))
    return {"tok_s": BATCH / (dt * factor), "threads": threads, "sample": sample, "step_s_measured": dt,
            "step_s": dt * factor, "layers_run": n_layers, "layers": L, "steps": steps}


def profile_kernels():
    """A handful of launches for profiler captures of the tensor-core kernels (`--profile-kernels`): the stream-K
    kernel at M = 32 and M = 256 on K=8192, N=22016, the 256 x 256 tile kernel at M = 4096 on K=4096, N=11008
    (persistent CTAs) and at M = 1024 on K=11008, N=4096 (split-K over clusters of two), the stream-K kernel on
    a LLaMA-7B shape (K=N=4096, M = 256), and the prefill attention at B=8, H=32, S=512.  The working sets of the
    first three GEMMs and of the attention exceed L2; nothing is timed or printed but the device status."""
    from eet_b200 import EET, _lib
    from eet_b200._lib import check, lib
    dev = torch.device("cuda", 0)

    def gemm(K, N, M, reps=2):
        w = torch.randint(-128, 128, (K, N), dtype=torch.int8, device=dev)
        s = (torch.rand(N, device=dev) * 1e-3).half()
        x = torch.randn(M, K, device=dev).half()
        out = torch.empty(M, N, device=dev, dtype=torch.float16)
        for _ in range(reps):
            EET.gemm_w8a16(x, w, s, out=out)
        torch.cuda.synchronize()

    gemm(8192, 22016, 32)
    gemm(8192, 22016, 256)
    gemm(4096, 11008, 4096)
    gemm(11008, 4096, 1024)
    gemm(4096, 4096, 256)
    B, H, S, D, T = 8, 32, 512, 128, 640
    q = torch.randn(B, H, S, D, device=dev).half()
    k = torch.randn(B, H, T, D, device=dev).half()
    v = torch.randn(B, H, T, D, device=dev).half()
    ctx = torch.empty(B, S, H * D, device=dev, dtype=torch.float16)
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        check(lib.eet_prefill_mha(q.data_ptr(), k.data_ptr(), v.data_ptr(), ctx.data_ptr(), B, S, H, D, T, None, None, S, st))
    torch.cuda.synchronize()
    print(json.dumps({"profile_kernels": "done", "device_status": _lib.device_status()}))


# ------------------------------------------------------------------------------------------------ arms
def bench_config(n_layers, world, cuda_graph, warmup, steps):
    """The `config` object of the JSON line: both arms print the same keys."""
    return {"workload": WORKLOAD, "layers": n_layers, "global_batch": BATCH, "seq_len": PROMPT,
            "lm_head": "int8, vocabulary-sharded over the ranks" if LM_HEAD_INT8 else "fp16, replicated (torch.nn.Linear)",
            "cache_len_during_timing": [PROMPT + warmup + 1, PROMPT + warmup + steps],
            "parallelism": f"tp{world}", "cuda_graph": cuda_graph,
            "l2": "weights (GBs per step) and KV cache exceed L2; no flush needed"}


def run_reference(args):
    """The reference arm: the CPU port of the path on this host's cores (rank 0 only).  With the driver's step
    counts all 32 layers run for every step; a run that would not end within a few minutes runs fewer layers per
    step and says so in `extrapolated`."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    r = cpu_decode_sample(args.steps, warmup=min(args.warmup, 2), budget_s=150.0)
    tok_s = round(r["tok_s"], 3)
    line = {"impl": "reference", "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(r["step_s"] * 1e3, 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32 (cpu port of f16 path)",
            "data": "synthetic",
            "config": bench_config(CFG["num_hidden_layers"], args.gpus, not getattr(args, "no_graph", False),
                                   args.warmup, args.steps),
            "cpu_baseline": {"value": tok_s, "unit": UNIT, "cores": r["threads"], "kind": "port", "sample": r["sample"]},
            "e2e": {"value": tok_s, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "extrapolated": None if r["layers_run"] == r["layers"] else
            {"layers_run": r["layers_run"], "factor": r["layers"] / r["layers_run"],
             "ms_per_step_measured": round(r["step_s_measured"] * 1e3, 3)},
            "note": "the reference has no CPU implementation of this path and its GPU kernels refuse sm_90+; this "
                    "arm times the CPU restatement (oracle/ops.py) of the reference's arithmetic",
            "wall_s": round(time.perf_counter() - t0, 1)}
    print(json.dumps(line))


def parity_check(tp, local, world, rank):
    """Not a measurement: a 2-layer model of the benchmark's architecture under the same tensor-parallel degree
    runs a 64-token prompt and four decode steps (the chain that the timed region used), and rank 0 compares its
    logits with the CPU oracle.  Returns the `tp_parity` object (None on other ranks)."""
    from eet_b200 import EET
    S, NEW = 64, 4
    model, cfg, d = build_model(tp, local, S + NEW + 2, layers=2, prompt=S, keep_dict=True)
    dev = torch.device("cuda", local)
    gen = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab_size, (BATCH, S + NEW), generator=gen)
    outs = [model(ids[:, :S].to(dev), first_pass=True).logits[:, -1:].float().cpu()]
    for t in range(S, S + NEW):
        outs.append(model.decode_logits(ids[:, t:t + 1].to(dev)).float().cpu())
    torch.cuda.synchronize()
    if rank != 0:
        return None
    from oracle import ops
    torch.set_num_threads(os.cpu_count() or 1)   # torchrun starts its workers with one OpenMP thread
    names = ("self_attn.qkv_proj", "self_attn.out_proj", "ffn.intermediate_0", "ffn.intermediate_1", "ffn.output")
    layers = []
    for i in range(2):
        args = []
        for n in names:
            args.extend((EET.unpack_weights(d[f"layer.{i}.{n}.weight"]).cpu(), d[f"layer.{i}.{n}.scale"].cpu()))
        layers.append(ops.LayerWeights(*args, d[f"layer.{i}.self_attn.layernorm.weight"].cpu(),
                                       d[f"layer.{i}.ffn.layernorm.weight"].cpu()))
    H = cfg.num_attention_heads
    dec = ops.DecoderOracle(layers, H, cfg.hidden_size // H, cfg.rms_norm_eps, S + NEW + 2, BATCH,
                            rope=(FAMILY != "baichuan"))
    emb, gamma = d["embed_tokens.weight"].cpu(), d["norm.weight"].cpu()
    if LM_HEAD_INT8:
        hq, _, hs = EET.quant_weights(d["lm_head.weight"].t().contiguous(), torch.int8, True)
        hq, hs = hq.cpu(), hs.cpu()
    else:
        head = d["lm_head.weight"].cpu().float()

    def oracle(tok, first):
        x = ops.rmsnorm(dec.forward(emb[tok], first), gamma, cfg.rms_norm_eps)[:, -1]
        if LM_HEAD_INT8:
            return ops.gemm_w8a16(x, hq, hs).float().unsqueeze(1)
        return (x.float() @ head.t()).unsqueeze(1)

    want = [oracle(ids[:, :S], True)] + [oracle(ids[:, t:t + 1], False) for t in range(S, S + NEW)]
    worst, worst_ratio = 0.0, 0.0
    for a, b in zip(outs, want):
        err = (a - b).abs()
        worst = max(worst, float(err.max()))
        worst_ratio = max(worst_ratio, float((err / (2e-2 + 2e-2 * b.abs())).max()))
    return {"max_abs_err": round(worst, 5), "tol": "2e-2 + 2e-2*|ref| on fp32 logits", "max_err_over_tol": round(worst_ratio, 4),
            "ok": worst_ratio <= 1.0, "layers": 2, "prompt": S, "decode_steps": NEW, "world": world,
            "checked_against": "oracle/ops.py on the host (rank 0)"}


def run_ours(args):
    from eet_b200 import tp as tp_mod
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    tp = tp_mod.init_from_env("nccl") if world > 1 else None
    dev = torch.device("cuda", local)
    K, W = args.steps, args.warmup
    t_max = PROMPT + W + K + 4
    model, cfg = build_model(tp, local, t_max, layers=args.layers)
    n_layers = cfg.num_hidden_layers
    model.use_cuda_graph = not args.no_graph

    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (BATCH, PROMPT), generator=gen)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # prefill (untimed set-up of the 512-token history)
    prefill_ms = None
    if args.skip_prefill:
        for layer in model.model.layers:   # profiling runs: a random history instead of a real prefill
            layer.attention.k_cache.normal_()
            layer.attention.v_cache.normal_()
        rewind(model, PROMPT)
        first = prompt[:, -1:].to(dev)
    else:
        pe0, pe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dev_prompt = prompt.to(dev)
        for _ in range(2):                                # sizes the pooled buffers and the allocator's cache
            out = model(dev_prompt, first_pass=True)
            del out                                       # (a live result would force a fresh 262 MB cudaMalloc
            torch.cuda.synchronize()                      # for the logits inside the timed call)
        pe0.record()
        out = model(dev_prompt, first_pass=True)          # same prompt again: identical state, timed
        pe1.record()
        first = torch.argmax(out.logits[:, -1, :], dim=-1, keepdim=True)
        del out
        torch.cuda.synchronize()
        prefill_ms = pe0.elapsed_time(pe1)
    torch.cuda.synchronize()

    host_ids = torch.empty((BATCH, 1), dtype=torch.long).pin_memory()
    host_next = torch.empty((BATCH, 1), dtype=torch.long).pin_memory()

    def e2e_steps(n):
        # through the public API: ids from pinned host memory, the chosen tokens read back every step
        for _ in range(n):
            nxt = model.decode_step(host_ids)
            host_next.copy_(nxt, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            host_ids.copy_(host_next)

    dev_ids = [first.clone()]

    def dev_steps(n):
        # ids resident on the device
        for _ in range(n):
            dev_ids[0] = model.decode_step(dev_ids[0])

    def timed_region(run_steps, reset):
        """One repeat: back to the prompt's history, W warm-up steps, then EXACTLY K steps between two CUDA events,
        a barrier and a device synchronisation on both sides; the maximum over the ranks, in seconds."""
        rewind(model, PROMPT)
        reset()
        run_steps(W)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run_steps(K)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) * 1e-3)

    def repeated(run_steps, reset):
        """Repeats the region until the clock sampler has seen at least a second of load (at least 5 repeats, at
        most 40); every rank takes the same decisions because the times are maxima over the ranks."""
        times = [timed_region(run_steps, reset)]   # untimed in effect: captures the graph, sizes buffers
        with ClockSampler(local) as clk:
            times = [timed_region(run_steps, reset)]
            repeats = args.repeats or int(min(40, max(5, -(-1.0 // max(times[0], 1e-4)))))
            while len(times) < repeats:
                times.append(timed_region(run_steps, reset))
        return times, clk

    def reset_host():
        host_ids.copy_(first.cpu())

    def reset_dev():
        dev_ids[0] = first.clone()

    e2e_times, clk_e2e = repeated(e2e_steps, reset_host)
    dev_times, clk = repeated(dev_steps, reset_dev)
    t_e2e, t_dev = statistics.median(e2e_times), statistics.median(dev_times)

    from eet_b200 import _lib
    status = _lib.device_status()

    pk = peaks()
    gemms = time_gemm_shapes(model, BATCH)
    g_bytes = sum(v["bytes"] for v in gemms.values())
    g_time = sum(v["us"] for v in gemms.values()) * 1e-6
    dom = gemms["qkv"]   # the largest single launch of a layer: fused QKV projection
    # `traffic` is NOT measured by this run: it is dram__bytes_read.sum + dram__bytes_write.sum of one launch of
    # this kernel at K=4096, N=12288, M=8 from an ncu capture (50.81 MB against 50.62 MB algorithmic), scaled by
    # the algorithmic bytes of the launch timed here; `traffic_source` says so in the line.  No capture exists
    # for the other workloads' shapes: null there.
    traffic = 50.81e6 * dom["bytes"] / 50620416.0 if WORKLOAD.startswith("llama7b") else None
    line = {"metric": METRIC, "value": round(BATCH * K / t_dev, 2), "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": round(t_dev / K * 1e3, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 activations x int8 weights, f32 accumulate", "data": "synthetic",
            "config": bench_config(n_layers, world, model.use_cuda_graph, W, K),
            "timing": {"repeats": len(dev_times), "statistic": "median of the repeats, each the max over ranks",
                       "ms_per_step_each": [round(t / K * 1e3, 4) for t in dev_times],
                       "ms_per_step_min": round(min(dev_times) / K * 1e3, 4),
                       "ms_per_step_max": round(max(dev_times) / K * 1e3, 4)},
            "e2e": {"value": round(BATCH * K / t_e2e, 2), "unit": UNIT, "h2d_bytes_per_step": BATCH * 8,
                    "d2h_bytes_per_step": BATCH * 8, "ms_per_step": round(t_e2e / K * 1e3, 4),
                    "repeats": len(e2e_times), "ms_per_step_each": [round(t / K * 1e3, 4) for t in e2e_times],
                    # the end-to-end step contains the device step plus copies and a synchronisation
                    "consistent": t_e2e >= t_dev * 0.98},
            "prefill": None if prefill_ms is None else {"ms": round(prefill_ms, 2), "tokens": BATCH * PROMPT,
                                                         "tokens_per_s": round(BATCH * PROMPT / prefill_ms * 1e3)},
            "gpu_launches": kernel_launches_per_step(n_layers, BATCH, world) * K,
            "clocks": clk.summary(), "clocks_e2e": clk_e2e.summary(), "device_status": status,
            "roofline": {"bound": "hbm",
                         "kernel": f"gemm_skinny_kernel<{1 if BATCH <= 8 else 2}>, fused QKV projection "
                                   f"K={dom['K']} N={dom['N']} M={BATCH}",
                         "achieved": round(dom["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(dom["gbs"] / pk["hbm_gbs"], 4), "peak_source": pk["source"],
                         "traffic": None if traffic is None else round(traffic),
                         "traffic_source": None if traffic is None else
                         "not measured by this run: one ncu capture of this kernel at K=4096 N=12288 M=8 "
                         "(50.81 MB read+written for 50.62 MB algorithmic), scaled by this launch's algorithmic bytes",
                         "algorithmic_bytes": dom["bytes"],
                         "launch_us": round(dom["us"], 2),
                         "all_gemm_launches_of_a_layer": {"achieved": round(g_bytes / g_time / 1e9, 1),
                                                          "frac": round(g_bytes / g_time / 1e9 / pk["hbm_gbs"], 4)},
                         "per_shape": {k: {"K": v["K"], "N": v["N"], "us": round(v["us"], 2), "gbs": round(v["gbs"], 1)}
                                       for k, v in gemms.items()}}}
    if world == 1 and not args.no_sweep:
        # the same kernel where the ~2 us launch ramp no longer matters: its steady-state rate
        line["roofline"]["same_kernel_on_a_180MB_matrix"] = skinny_steady_state(dev, BATCH, pk["hbm_gbs"])
        line["gemm_sweep"] = gemm_sweep(dev, pk["hbm_gbs"], pk["tflops"])
    if not args.no_parity and FAMILY == "llama":
        par = parity_check(tp, local, world, rank)
        if rank == 0:
            line["tp_parity"] = par
    if rank == 0 and world == 1 and not args.no_cpu:
        r = cpu_decode_sample(4, warmup=1, budget_s=15.0)
        line["cpu_baseline"] = {"value": round(r["tok_s"], 3), "unit": UNIT, "cores": r["threads"], "kind": "port",
                                "sample": r["sample"],
                                "extrapolated": None if r["layers_run"] == r["layers"] else
                                {"layers_run": r["layers_run"], "factor": r["layers"] / r["layers_run"]}}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # CUDA graphs that captured NCCL kernels keep the communicator busy: drop them before tearing the
        # process group down, and never let the teardown outlive the measurement by more than a few seconds
        threading.Timer(20.0, lambda: os._exit(0)).start()
        model.end_graph()
        del model
        import gc
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama7b", choices=sorted(WORKLOADS),
                    help="model-level configuration; the default is the headline one")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the architecture has (profiling runs only)")
    ap.add_argument("--no-graph", action="store_true", help="launch the decode step eagerly")
    ap.add_argument("--no-sweep", action="store_true", help="skip the GEMM sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    ap.add_argument("--repeats", type=int, default=0,
                    help="repeats of the timed region (default: at least 5 and at least a second of load; "
                         "profiling runs pass 1)")
    ap.add_argument("--lm-head", default="int8", choices=["int8", "fp16"],
                    help="int8: lm_head through the W8A16 GEMM, vocabulary-sharded under tensor parallelism (default); "
                         "fp16: the reference's replicated fp16 torch.nn.Linear")
    ap.add_argument("--no-parity", action="store_true", help="skip the 2-layer parity check against the CPU oracle")
    ap.add_argument("--profile-kernels", action="store_true",
                    help="run a few launches of the tensor-core kernels for a profiler capture and exit")
    ap.add_argument("--skip-prefill", action="store_true",
                    help="fill the KV cache with random data instead of running the prompt (profiling runs only)")
    args = ap.parse_args()
    select_workload(args.workload)
    global LM_HEAD_INT8
    LM_HEAD_INT8 = args.lm_head == "int8"
    if args.warmup < 3:
        args.warmup = 3
    if args.profile_kernels:
        profile_kernels()
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
