"""Decode and prefill throughput at the Llama-3.1-8B shape with random weights, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--repeats R] [--batch 8] [--layers 32] [--impl reference]

Prints ONE JSON line.  `value` is decoded tokens per second at the default batch (8 requests,
each with 1,024 tokens of context): after W warm-up steps, R repeats of K decode steps are timed
on the device with CUDA events and the median repeat is reported (`ms_per_step_min_max` gives the
spread).  `e2e` is the same workload through the Python entry point (`Engine.step`), with every
step's token ids going from pinned host memory to the device and the sampled tokens read back,
timed on the host clock.  `prefill` is one step of 2,048 prompt tokens; `roofline` sets the decode
step's bytes (every weight it uses once plus the cache of the live requests) against the measured
copy bandwidth.  `points` holds decode at batch 1 and 64 and two further workloads, each with its
time set against the roofline of its steps (a step's bound is the slower of its flops over the
tensor peak and its bytes over the copy peak): continuous batching of 64 requests at the
Llama-3.2-3B shape (prompts of 16 to 2,048 tokens, 256 new tokens each) and, at the Llama-3.2-1B
shape, 8 prompts of 8,192 tokens prefilled in portions of 512 beside 128 requests that decode
with temperature 1.0 and fixed seeds.  SM clocks are sampled during every point (`clocks` for the
headline point, `clocks_points` for the others).  The weights of every step are larger than L2,
so nothing is flushed between timed iterations.  Peaks come from MEASURED_PEAKS.json beside this
file when present.

`--impl reference` runs the same workloads on the unmodified reference engine (baseline/reference_arm.py).

`--design dezolorn` measures another thing and leaves the above alone: prefill and decode throughput of Dezolorn models
(windowed attention with kept first keys, retention, gated delta rule; random weights) at two sizes that resemble real
layers, each beside a Llama model of equal width, feed-forward, heads and layer count, and every kernel of one prefill
step and one decode step of both, timed alone and set against its own bound (bytes over the copy peak, tensor flops over
the tensor peak, CUDA-core flops over the nominal float32 rate).  `--design sorizen` does the same for Sorizen models (attention
over a cached latent with a sink or a gate, hyper-connections, dense and routed feed-forwards) beside Dezolorn models of
windowed attention layers alone, and `--design debuvik` for Debuvik models (latent attention with a gate on every output
feature, chunked attention with capped scores and biases, partly on an earlier layer's keys and values, norms on the sublayers'
outputs, the token's side input) beside Dezolorn layers of windowed attention and Sorizen layers of latent attention; `like`
sets every Debuvik kernel's fraction of its bound over that of the sibling's kernel that does the like work.  `--design fubolix`:
Fubolix models (one dynamic-tanh norm a layer whose output the mixer and a squared-relu feed-forward both read; attention with a
sink in the denominator - windowed with kept first keys, gated heads and keys as values; with a query temperature; behind a short
convolution) beside Dezolorn layers of windowed attention.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# every size of the benchmark's third, fourth and fifth configuration
SHAPES = {
    "8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192),
    "3b": dict(vocab_size=128256, hidden_size=3072, intermediate_size=8192, num_hidden_layers=28, num_attention_heads=24,
               num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=4096,
               tie_word_embeddings=True),
    "1b": dict(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_hidden_layers=16, num_attention_heads=32,
               num_key_value_heads=8, head_dim=64, rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=16384,
               tie_word_embeddings=True),
}
ROPES = {"8b": (8.0, 1.0, 4.0, 8192), "3b": (32.0, 1.0, 4.0, 8192), "1b": (32.0, 1.0, 4.0, 8192)}
SHAPE, ROPE = SHAPES["8b"], ROPES["8b"]
CONTEXT = 1024        # tokens each request holds when decoding is timed
PREFILL_TOKENS = 2048
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            p = json.load(open(path))
            out = dict(FALLBACK_PEAKS)

            def find(node, key):  # the key at the top level, or in a nested object
                if isinstance(node, dict):
                    if isinstance(node.get(key), (int, float)) and not isinstance(node.get(key), bool):
                        return float(node[key])
                    for v in node.values():
                        hit = find(v, key)
                        if hit is not None:
                            return hit
                return None

            found = {k: find(p, k) for k in out}
            if found["hbm_gbs"] is not None or found["bf16_tflops"] is not None:
                out.update({k: v for k, v in found.items() if v is not None and v > 0})
                return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.rows: list[list[str]] = []
        self.proc = None
        self.first = 0

    def mark(self) -> None:
        """The timed region begins: samples taken before now (nvidia-smi needs a moment to start, so it is started
        ahead of the warm-up) do not count, except the last one when no later sample exists."""
        self.first = len(self.rows)

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = self.rows[self.first:] or self.rows[-1:]
        sm = sorted(int(r[0]) for r in rows if len(r) >= 6 and r[0].isdigit())
        mx = [int(r[1]) for r in rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


class Sizes:
    """Elements, bytes and flops of a shape, for setting times against the roofline."""

    def __init__(self, cfg: dict, layers: int) -> None:
        H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
        nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        self.layers, self.H, self.V, self.nq, self.d = layers, H, V, nq, d
        self.per_layer = (nq + 2 * nkv) * d * H + H * nq * d + 3 * I * H  # matrix elements of one layer
        self.head = V * H
        self.norms = (2 * layers + 1) * H
        self.kv_per_token = 2 * layers * nkv * d * 2                      # bytes, bf16

    def decode_bytes(self, batch: int, context: int) -> float:
        return 2 * (self.layers * self.per_layer + self.head) + 4 * self.norms + batch * self.H * 2 \
            + batch * context * self.kv_per_token

    def step_flops(self, tokens: int, sampled: int, pairs: int) -> float:
        """Products over `tokens` rows, the head over `sampled` rows, q k^T and p v over `pairs` query-key pairs."""
        return 2.0 * tokens * self.layers * self.per_layer + 2.0 * sampled * self.head + 4.0 * self.layers * self.nq * self.d * pairs

    def step_bytes(self, kv_positions: int, sampled: int) -> float:
        return 2.0 * (self.layers * self.per_layer + (self.head if sampled else 0)) + kv_positions * self.kv_per_token

    def step_bound_s(self, log_row: tuple, pk: dict) -> float:
        tokens, kv_positions, sampled, pairs = log_row
        return max(self.step_flops(tokens, sampled, pairs) / (pk["bf16_tflops_sustained"] * 1e12),
                   self.step_bytes(kv_positions, sampled) / (pk["hbm_gbs"] * 1e9))


def build_engine(shape: str, layers: int | None, max_running: int, num_blocks: int, **kw):
    import torch

    from nanospec_b200 import Engine, EngineConfig, LlamaConfig, random_model
    from nanospec_b200.config import Llama3RopeScaling

    sh = dict(SHAPES[shape])
    if layers:
        sh["num_hidden_layers"] = layers
    cfg = LlamaConfig(**sh, rope_scaling=Llama3RopeScaling(*ROPES[shape]))
    model = random_model(cfg, seed=0, device="cuda", dtype=torch.bfloat16)
    opts = dict(num_blocks=num_blocks, block_size=PAGE, max_running=max_running, max_admit=64, max_step_tokens=8192,
                prefill_chunk=PREFILL_TOKENS)
    opts.update(kw)
    return model, Engine(model, EngineConfig(**opts))


def prime(eng, batch: int, context: int, max_tokens: int, seed: int = 0):
    """Adds `batch` requests of `context` random tokens and runs steps until all of them decode."""
    import torch

    from nanospec_b200 import SamplingParams

    g = torch.Generator().manual_seed(seed)
    vocab = eng.model.vocab_size
    reqs = [eng.add(torch.randint(0, vocab, (context - 1,), generator=g).tolist(),
                    SamplingParams(max_tokens=max_tokens, ignore_eos=True)) for _ in range(batch)]
    while any(r.state == "waiting" or (r.state == "running" and r.pending > 1) for r in reqs):
        eng.step()
    return reqs


def median(xs: list[float]) -> float:
    xs = sorted(xs)
    return xs[len(xs) // 2]


def time_decode(eng, batch: int, steps: int, warmup: int, repeats: int) -> dict:
    """`repeats` x `steps` decode steps of `batch` requests after `warmup` steps.  Device time: every step is
    one graph launch with its own pair of events around copy-in, replay and copy-out; a repeat's figure is the
    mean over the launches made during it (steps may be launched one ahead of their predecessor's results, so a
    repeat's launches can differ from its calls by one).  Host time: the clock around the repeat's `step()` calls."""
    import torch

    from nanospec_b200.ops import lib

    sampler = ClockSampler()
    sampler.start()
    reqs = prime(eng, batch, CONTEXT, max_tokens=warmup + repeats * steps + 8)
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    bucket = eng.graphs.buckets[eng.graphs.bucket_size(batch)]
    launches0, replays0 = lib.launch_count(), eng.graphs.replays
    sampler.mark()
    dev_ms, host_s = [], []
    for _ in range(repeats):
        eng.graphs.timing = []
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            eng.step()          # host ids -> pinned -> device, graph replay, sampled tokens back to the host
        torch.cuda.synchronize()
        host_s.append((time.perf_counter() - t0) / steps)
        launched = len(eng.graphs.timing)
        assert abs(launched - steps) <= 1, f"{launched} graph launches in {steps} timed steps"
        dev_ms.append(sum(s.elapsed_time(e) for s, e in eng.graphs.timing) / launched)
    clocks = sampler.stop()
    eng.graphs.timing = None
    launches = lib.launch_count() - launches0 + (eng.graphs.replays - replays0) * bucket.kernels
    h2d = eng.runner.h2d_bytes_last
    for r in reqs:
        if r.state == "running":
            eng.sched.finish(r)
    return {"ms": median(dev_ms), "ms_min": min(dev_ms), "ms_max": max(dev_ms), "host_s": median(host_s), "clocks": clocks,
            "launches": launches, "h2d": h2d, "d2h": 3 * 4 * batch}


def time_prefill(eng, warmup: int, iters: int) -> tuple[float, dict]:
    import torch

    from nanospec_b200 import SamplingParams

    g = torch.Generator().manual_seed(123)
    times = []
    sampler = ClockSampler()
    sampler.start()
    for i in range(warmup + iters):
        if i == warmup:
            sampler.mark()
        ids = torch.randint(0, eng.model.vocab_size, (PREFILL_TOKENS,), generator=g).tolist()
        req = eng.add(ids, SamplingParams(max_tokens=1, ignore_eos=True))
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step()
        b.record()
        torch.cuda.synchronize()
        assert req.state == "done"
        if i >= warmup:
            times.append(a.elapsed_time(b))
    return median(times), sampler.stop()


def _workload_record(eng, sizes: Sizes, pk: dict, seconds: float, out_tokens: int, all_tokens: int, live: int, clocks: dict) -> dict:
    bound = sum(sizes.step_bound_s(row, pk) for row in eng.step_log)
    return {"out_tok_s": round(out_tokens / seconds, 1), "total_tok_s": round(all_tokens / seconds, 1),
            "tpot_ms": round(1000.0 * seconds / (out_tokens / live), 3), "seconds": round(seconds, 4), "steps": len(eng.step_log),
            "roofline_s": round(bound, 4), "frac": round(bound / seconds, 4), "sm_mhz": clocks.get("sm_mhz"),
            "reasons": clocks.get("reasons")}


def workload_continuous_batching(pk: dict, runs: int) -> dict:
    """Llama-3.2-3B shape: 64 requests with prompts of 16 to 2,048 seeded random tokens and 256 new tokens each,
    all admitted at once, continuous batching until the last one ends.  The reference's definitions
    (bench/run.py:43-44, bench/table.py:19 there): tok_s = output tokens / seconds, tpot_ms = 1000 * seconds /
    (output tokens / batch), the median over the runs; the first run also loads the library's kernels for these
    shapes and does not count."""
    import torch

    from nanospec_b200 import SamplingParams

    n_req, new = 64, 256
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(16, 2048 + 1, (n_req,), generator=g).tolist()
    prompts = [torch.randint(0, SHAPES["3b"]["vocab_size"], (n,), generator=g).tolist() for n in lens]
    pages = sum(-(-(n + new) // PAGE) + 1 for n in lens) + 16
    model, eng = build_engine("3b", None, n_req, pages)
    sizes = Sizes(SHAPES["3b"], SHAPES["3b"]["num_hidden_layers"])
    recs = []
    for run in range(runs + 1):
        eng.step_log = []
        sampler = ClockSampler()
        sampler.start()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = eng.generate(prompts, SamplingParams(max_tokens=new, ignore_eos=True))
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        n_out = sum(len(o) for o in outs)
        recs.append(_workload_record(eng, sizes, pk, dt, n_out, n_out + sum(lens), n_req, sampler.stop()))
    recs = sorted(recs[1:], key=lambda r: r["seconds"])
    rec = recs[len(recs) // 2]
    rec.update(requests=n_req, prompt_tokens=sum(lens), new_tokens_each=new, runs=runs, context=4096)
    del eng, model
    torch.cuda.empty_cache()
    return rec


def workload_mixed(pk: dict, runs: int) -> dict:
    """Llama-3.2-1B shape, contexts of up to 16,384: 128 requests decode (temperature 1.0, fixed seeds) while 8
    prompts of 8,192 tokens are prefilled in portions of 512.  Timed from the step that admits the prompts to the
    step that ends the last of them; the decoders run throughout."""
    import torch

    from nanospec_b200 import SamplingParams

    n_dec, n_long, long_len, portion = 128, 8, 8192, 512
    vocab = SHAPES["1b"]["vocab_size"]
    g = torch.Generator().manual_seed(0)
    dec = [torch.randint(0, vocab, (int(n),), generator=g).tolist() for n in torch.randint(32, 512, (n_dec,), generator=g)]
    longs = [torch.randint(0, vocab, (long_len,), generator=g).tolist() for _ in range(n_long)]
    budget = (runs + 1) * (long_len // portion + 8) + 32   # the decoders outlive every run's prompts
    pages = sum(-(-(len(p) + budget) // PAGE) + 1 for p in dec) + n_long * (long_len // PAGE + 8) + 16
    model, eng = build_engine("1b", None, n_dec + n_long, pages, prefill_chunk=portion)
    sizes = Sizes(SHAPES["1b"], SHAPES["1b"]["num_hidden_layers"])
    reqs = [eng.add(p, SamplingParams(max_tokens=budget, temperature=1.0, seed=7 + i, ignore_eos=True)) for i, p in enumerate(dec)]
    while any(r.state == "waiting" or (r.state == "running" and r.pending > 1) for r in reqs):
        eng.step()
    recs = []
    for run in range(runs + 1):
        lreqs = [eng.add(p, SamplingParams(max_tokens=2, temperature=1.0, seed=99 + i, ignore_eos=True)) for i, p in enumerate(longs)]
        eng.step_log = []
        sampler = ClockSampler()
        sampler.start()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while any(r.state != "done" for r in lreqs):
            eng.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        steps = len(eng.step_log)
        n_out = steps * n_dec + 2 * n_long
        rec = _workload_record(eng, sizes, pk, dt, n_out, n_out + n_long * long_len, n_dec, sampler.stop())
        rec["prefill_tok_s"] = round(n_long * long_len / dt, 1)
        rec["ms_per_step"] = round(1000.0 * dt / steps, 3)
        recs.append(rec)
    assert all(r.state == "running" for r in reqs)
    recs = sorted(recs[1:], key=lambda r: r["seconds"])
    rec = recs[len(recs) // 2]
    rec.update(decoding_requests=n_dec, long_prompts=n_long, prompt_tokens_each=long_len, portion=portion, temperature=1.0,
               runs=runs, context=16384)
    del eng, model
    torch.cuda.empty_cache()
    return rec


def run_ours(args) -> dict:
    import torch

    pk, pk_src = peaks()
    layers = args.layers
    sizes = Sizes(SHAPE, layers)
    pages_per_req = -(-(CONTEXT + args.repeats * args.steps + args.warmup + 64) // PAGE)
    num_blocks = max(64 * pages_per_req, -(-PREFILL_TOKENS // PAGE) + 8) + 8
    model, eng = build_engine("8b", layers, 64, num_blocks)
    torch.cuda.synchronize()

    head = time_decode(eng, args.batch, args.steps, args.warmup, args.repeats)
    dev_ms = head["ms"]
    value = args.batch * 1000.0 / dev_ms
    e2e = args.batch / head["host_s"]

    points, clocks_points = {}, {}
    for b in (1, 64):
        pt = time_decode(eng, b, args.steps, args.warmup, args.repeats)
        points[f"decode_b{b}"] = round(b * 1000.0 / pt["ms"], 1)
        points[f"decode_b{b}_frac"] = round(sizes.decode_bytes(b, CONTEXT) / (pt["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        clocks_points[f"decode_b{b}"] = {"sm_mhz": pt["clocks"].get("sm_mhz"), "reasons": pt["clocks"].get("reasons"),
                                         "ms": round(pt["ms"], 4), "ms_min_max": [round(pt["ms_min"], 4), round(pt["ms_max"], 4)]}
    pre_ms, pre_clocks = time_prefill(eng, warmup=3, iters=5)
    clocks_points["prefill"] = {"sm_mhz": pre_clocks.get("sm_mhz"), "reasons": pre_clocks.get("reasons")}
    prefill_flops = sizes.step_flops(PREFILL_TOKENS, 1, PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2)
    del eng, model
    torch.cuda.empty_cache()

    workloads = {}
    if not args.no_workloads and layers == SHAPE["num_hidden_layers"]:
        workloads["continuous_batching_3b"] = workload_continuous_batching(pk, runs=3)
        workloads["mixed_1b"] = workload_mixed(pk, runs=3)
        for name, short in (("continuous_batching_3b", "cb3b"), ("mixed_1b", "mixed1b")):
            for key in ("out_tok_s", "total_tok_s", "tpot_ms", "frac"):
                points[f"{short}_{key}"] = workloads[name][key]

    achieved = sizes.decode_bytes(args.batch, CONTEXT) / (dev_ms * 1e-3) / 1e9
    mhz = head["clocks"].get("sm_mhz")
    return {
        "metric": "decode tok/s (Llama-3.1-8B shape, batch 8, 1,024-token context)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform random token ids, random N(0, 0.02) weights",
        "config": {"model": "Llama-3.1-8B shape", "layers": layers, "layers_of_config": SHAPE["num_hidden_layers"],
                   "hidden": SHAPE["hidden_size"], "heads": SHAPE["num_attention_heads"],
                   "kv_heads": SHAPE["num_key_value_heads"], "head_dim": SHAPE["head_dim"],
                   "intermediate": SHAPE["intermediate_size"], "vocab": SHAPE["vocab_size"], "global_batch": args.batch,
                   "seq_len": CONTEXT, "max_context": SHAPE["max_position_embeddings"], "page": PAGE,
                   "parallelism": "single GPU", "cuda_graphs": True, "repeats": args.repeats,
                   "l2": "inputs larger than L2 (16 GB of weights per step)",
                   "peaks": pk_src},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": head["h2d"], "d2h_bytes_per_step": head["d2h"]},
        "gpu_launches": head["launches"],
        "ms_per_step_min_max": [round(head["ms_min"], 4), round(head["ms_max"], 4)],
        "ms_x_sm_mhz": round(dev_ms * mhz, 1) if mhz else None,
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(prefill_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "frac_of_sustained": round(prefill_flops / (pre_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "workloads": workloads,
        # the one number the reference publishes for this architecture: 137 tok/s at batch 1 on an H100
        # (its README.md:76); the headline metric here (batch 8) has no published counterpart
        "vs_published_b1_h100": round(points["decode_b1"] / 137.0, 2),
        "clocks": head["clocks"],
        "clocks_points": clocks_points,
    }


# ---- another design beside its closest sibling (--design) ---------------------------------------------------------------

DESIGN_SIZES = {
    # width, feed-forward, attention heads / kv heads / head size, state mixers' heads / q-k heads / head sizes, layers
    "w2048": dict(width=2048, ff=8192, heads=32, kv_heads=8, dim=64, s_heads=16, s_kv=8, s_dim=128, s_vdim=128, layers=8),
    "w4096": dict(width=4096, ff=14336, heads=32, kv_heads=8, dim=128, s_heads=32, s_kv=16, s_dim=128, s_vdim=128, layers=4),
}
DESIGN_VOCAB, DESIGN_WINDOW, DESIGN_KEEP = 32768, 1024, 8
FP32_TFLOPS_NOMINAL = 148 * 128 * 2 * 1.965e9 / 1e12  # CUDA cores: 148 SMs x 128 lanes x 2 flops x the top clock


def dezolorn_config(sz: dict) -> dict:
    attention = {"type": "attention", "mlp": {"kind": "dense", "ff": sz["ff"]}, "mixer": {
        "heads": sz["heads"], "kv_heads": sz["kv_heads"], "dim": sz["dim"], "vdim": sz["dim"], "scale": sz["dim"] ** -0.5,
        "mask": {"size": DESIGN_WINDOW, "keep_first": DESIGN_KEEP},
        "rot": {"dims": sz["dim"], "base": 1000000.0, "scaling": {"factor": 8.0, "original": 8192, "fast": 16.0, "slow": 2.0}}}}
    retention = {"type": "retention", "mlp": {"kind": "dense", "ff": sz["ff"]}, "mixer": {
        "heads": sz["s_heads"], "dim": sz["s_dim"], "vdim": sz["s_vdim"],
        "decay": [1.0 - 2.0 ** -(5 + h % 8) for h in range(sz["s_heads"])], "rot": {"dims": sz["s_dim"], "base": 10000.0}}}
    delta = {"type": "delta", "mlp": {"kind": "dense", "ff": sz["ff"]}, "mixer": {
        "heads": sz["s_heads"], "kv_heads": sz["s_kv"], "dim": sz["s_dim"], "vdim": sz["s_vdim"], "conv": 4}}
    pattern = [attention, retention, delta, attention]
    return {"architecture": "Dezolorn", "vocab": DESIGN_VOCAB, "width": sz["width"], "norm": {"eps": 1e-6},
            "layers": [pattern[i % 4] for i in range(sz["layers"])], "loop": {"start": 0, "stop": 0, "times": 1},
            "logit_scale": 1.0, "logit_softcap": 20.0}


def llama_sibling(sz: dict):
    from nanospec_b200 import LlamaConfig

    return LlamaConfig(vocab_size=DESIGN_VOCAB, hidden_size=sz["width"], intermediate_size=sz["ff"], num_hidden_layers=sz["layers"],
                       num_attention_heads=sz["heads"], num_key_value_heads=sz["kv_heads"], head_dim=sz["dim"], rms_norm_eps=1e-6,
                       rope_theta=500000.0, max_position_embeddings=8192, rope_scaling=None, tie_word_embeddings=False, eos_token_ids=())


def kernel_bounds(kind: str, sz: dict, tokens: int, batch: int, context: int, pk: dict) -> dict[str, float]:
    """Seconds that every kernel of one step needs at least, summed over the step's calls of it.  `tokens` > 0: a prompt of that
    many tokens; otherwise `batch` requests decoding at `context` tokens."""
    N = tokens or batch
    H, L = sz["width"], sz["layers"]
    bw, tc, cc = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12, FP32_TFLOPS_NOMINAL * 1e12
    nq, nkv, d = sz["heads"], sz["kv_heads"], sz["dim"]
    norm = 12.0 * N * H / bw  # stream read and written in float32, branch read and result written in bfloat16
    qkv = 2.0 * N * ((nq + nkv) * d * 2 + nkv * d + 2 * nkv * d) / bw
    out: dict[str, float] = {}
    if kind == "llama":
        pairs = tokens * (tokens + 1) // 2 if tokens else 0
        out["ns_add_rmsnorm"] = 2 * L * norm
        out["ns_rope_kv_write"] = L * qkv
        out["ns_attention_prefill_tc" if tokens else "ns_attention_decode_tma"] = \
            L * (4.0 * nq * d * pairs / tc if tokens else 4.0 * batch * context * nkv * d / bw)
        out["ns_swiglu"] = L * 6.0 * N * sz["ff"] / bw
        return out
    n_att, n_ret, n_del = (sum(1 for i in range(L) if i % 4 in kinds) for kinds in ((0, 3), (1,), (2,)))
    sh, sk, sd, sv = sz["s_heads"], sz["s_kv"], sz["s_dim"], sz["s_vdim"]
    seen = lambda p: min(p + 1, DESIGN_WINDOW) + max(0, min(DESIGN_KEEP, p + 1 - DESIGN_WINDOW))  # keys position p sees
    out["ns_add_layernorm"] = 2 * L * norm
    out["ns_qk_norm_rope_store"] = n_att * qkv
    if tokens:
        out["ns_attention_prefill_kept"] = n_att * 4.0 * nq * d * sum(seen(p) for p in range(tokens)) / tc
    else:
        out["ns_attention_decode_kept"] = n_att * 4.0 * batch * seen(context) * nkv * d / bw
    out["ns_swiglu"] = L * 6.0 * N * sz["ff"] / bw
    out["ns_rotary_prepare"] = n_ret * N * ((2 * sh * sd + sh * sv) * 2 + (2 * sh * sd + sh * sv) * 4) / bw
    chan = 2 * sk * sd + sh * sv
    out["ns_delta_prepare"] = n_del * N * (chan * 2 + (chan + 2 * sh) * 4) / bw
    rec_in = lambda g: (2 * g * sd + sh * sv) * 4.0  # the float32 operands of one token
    if tokens:  # the recurrence on CUDA cores: per token, head and state entry 5 flops (plain) or 7 (delta rule)
        out["ns_linear_scan"] = (n_ret * 5.0 + n_del * 7.0) * tokens * sh * sd * sv / cc
    else:       # the state read and written once per request
        out["ns_linear_scan"] = (n_ret + n_del) * batch * (8.0 * sh * sd * sv) / bw + batch * (n_ret * rec_in(sh) + n_del * rec_in(sk)) / bw
    out["ns_head_norm_gate"] = (n_ret + n_del) * N * sh * sv * 8.0 / bw
    return out


def design_engine(model, max_running: int, num_blocks: int, **kw):
    from nanospec_b200 import Engine, EngineConfig

    opts = dict(num_blocks=num_blocks, block_size=PAGE, max_running=max_running, max_admit=64, max_step_tokens=8192,
                prefill_chunk=PREFILL_TOKENS)
    opts.update(kw)
    return Engine(model, EngineConfig(**opts))


def time_kernels(model, tokens: int, batch: int, context: int) -> dict[str, tuple[int, float]]:
    """Every entry point of one eager step, bracketed by events: a prompt of `tokens`, or `batch` requests that decode at `context`."""
    import torch

    from nanospec_b200.engine.step import ModelRunner, StepEntry
    from nanospec_b200.ops import lib

    runner = ModelRunner(model, num_blocks=max(batch, 1) * (-(-(context + PREFILL_TOKENS) // PAGE) + 2), block_size=PAGE, max_requests=max(batch, 1))
    g = torch.Generator().manual_seed(5)
    ids = lambda n: torch.randint(0, model.vocab_size, (n,), generator=g).tolist()
    best: dict[str, tuple[int, float]] = {}
    if tokens:
        for it in range(4):
            runner.begin(it)
            if it:
                lib.start_kernel_timing()
            runner.step([StepEntry(it, ids(tokens), [tokens - 1])])
            if it:
                got = lib.stop_kernel_timing()
                best = {k: (v[0], min(v[1], best.get(k, v)[1])) for k, v in got.items()}
            runner.end(it)
        return best
    for b in range(batch):
        runner.begin(b)
    for at in range(0, context, PREFILL_TOKENS):  # the contexts, eight requests to a step
        for b0 in range(0, batch, 8):
            runner.step([StepEntry(b, ids(min(PREFILL_TOKENS, context - at)), []) for b in range(b0, min(batch, b0 + 8))])
    for it in range(4):
        if it:
            lib.start_kernel_timing()
        runner.step([StepEntry(b, ids(1), [0]) for b in range(batch)])
        if it:
            got = lib.stop_kernel_timing()
            best = {k: (v[0], min(v[1], best.get(k, v)[1])) for k, v in got.items()}
    return best


def run_design(args) -> dict:
    import torch

    from nanospec_b200 import random_model

    pk, pk_src = peaks()
    out_sizes = {}
    for name, sz in DESIGN_SIZES.items():
        row = {}
        for kind in ("dezolorn", "llama"):
            cfg = dezolorn_config(sz) if kind == "dezolorn" else llama_sibling(sz)
            model = random_model(cfg, seed=1, device="cuda", dtype=torch.bfloat16)
            pages_per_req = -(-(CONTEXT + args.repeats * args.steps + args.warmup + 64) // PAGE)
            eng = design_engine(model, 64, max(64 * pages_per_req, -(-PREFILL_TOKENS // PAGE) + 8) + 8)
            rec = {}
            for b in (8, 64):
                pt = time_decode(eng, b, args.steps, args.warmup, args.repeats)
                rec[f"decode_b{b}_tok_s"] = round(b * 1000.0 / pt["ms"], 1)
                rec[f"decode_b{b}_ms"] = round(pt["ms"], 4)
                rec[f"decode_b{b}_clocks"] = {"sm_mhz": pt["clocks"].get("sm_mhz"), "reasons": pt["clocks"].get("reasons")}
                if b == 8 and kind == "dezolorn" and name == "w4096":
                    headline = pt
            pre_ms, pre_clocks = time_prefill(eng, warmup=3, iters=5)
            rec["prefill_tok_s"] = round(PREFILL_TOKENS * 1000.0 / pre_ms, 1)
            rec["prefill_ms"] = round(pre_ms, 3)
            rec["prefill_clocks"] = {"sm_mhz": pre_clocks.get("sm_mhz"), "reasons": pre_clocks.get("reasons")}
            del eng
            torch.cuda.empty_cache()
            kernels = {}
            for what, tokens, batch in (("prefill", PREFILL_TOKENS, 0), ("decode_b64", 0, 64)):
                timed = time_kernels(model, tokens, batch, CONTEXT)
                bounds = kernel_bounds(kind, sz, tokens, batch, CONTEXT, pk)
                kernels[what] = {k: {"calls": n, "ms": round(ms, 4), "bound_ms": round(bounds[k] * 1e3, 4) if k in bounds else None,
                                     "frac": round(bounds[k] * 1e3 / ms, 4) if k in bounds and ms > 0 else None}
                                 for k, (n, ms) in sorted(timed.items(), key=lambda kv: -kv[1][1])}
            rec["kernels"] = kernels
            row[kind] = rec
            del model
            torch.cuda.empty_cache()
        out_sizes[name] = row
    value = out_sizes["w4096"]["dezolorn"]["decode_b8_tok_s"]
    return {
        "metric": "decode tok/s (Dezolorn, width 4,096, 4 layers, batch 8, 1,024-token context)", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": out_sizes["w4096"]["dezolorn"]["decode_b8_ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform random token ids, random weights",
        "config": {"design": "dezolorn beside llama", "sizes": DESIGN_SIZES, "vocab": DESIGN_VOCAB, "window": DESIGN_WINDOW,
                   "keep_first": DESIGN_KEEP, "seq_len": CONTEXT, "prefill_tokens": PREFILL_TOKENS, "page": PAGE, "cuda_graphs": True,
                   "peaks": pk_src, "fp32_tflops_nominal": round(FP32_TFLOPS_NOMINAL, 1),
                   "l2": "the weights of every step are larger than L2"},
        "gpu_launches": headline["launches"], "clocks": headline["clocks"], "sizes": out_sizes,
    }


# ---- Sorizen beside a Dezolorn model of attention layers alone (--design sorizen) -------------------------------------------

SORIZEN_SIZES = {
    # width, dense feed-forward, heads, plain / rotated / value head sizes, latent, experts (count, chosen, width, groups, kept), layers
    "w2048": dict(width=2048, ff=8192, heads=16, kv_heads=8, dim=128, rot_dim=64, vdim=128, rank=512, experts=32, top=4, eff=1024,
                  groups=4, keep=2, streams=2, layers=8),
    "w4096": dict(width=4096, ff=14336, heads=32, kv_heads=8, dim=128, rot_dim=64, vdim=128, rank=512, experts=32, top=4, eff=2048,
                  groups=4, keep=2, streams=2, layers=4),
}
SORIZEN_WINDOW = 1024


def sorizen_config(sz: dict) -> dict:
    def mixer():
        return {"heads": sz["heads"], "dim": sz["dim"], "rot_dim": sz["rot_dim"], "vdim": sz["vdim"], "kv_rank": sz["rank"],
                "scale": (sz["dim"] + sz["rot_dim"]) ** -0.5, "mask": {"size": SORIZEN_WINDOW},
                "rot": {"dims": sz["rot_dim"], "base": 1000000.0, "scaling": {"factor": 8.0, "original": 8192, "fast": 16.0, "slow": 2.0}}}
    dense = {"type": "latent_attention_2", "mixer": mixer(), "mlp": {"kind": "dense", "ff": sz["ff"]}}
    routed = {"type": "latent_attention", "mixer": mixer(), "mlp": {"kind": "moe", "expert": {"ff": sz["eff"]}, "router": {
        "experts": sz["experts"], "top": sz["top"], "scale": 2.0, "groups": {"count": sz["groups"], "keep": sz["keep"]}}}}
    return {"architecture": "Sorizen", "vocab": DESIGN_VOCAB, "width": sz["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "streams": sz["streams"], "layers": [dense if i % 2 == 0 else routed for i in range(sz["layers"])]}


def windowed_sibling(sz: dict) -> dict:
    """The closest model the framework had: Dezolorn layers of windowed attention alone (layer norm, rotation with scaling, a
    gated feed-forward), at the same width, feed-forward, heads and layer count."""
    attention = {"type": "attention", "mlp": {"kind": "dense", "ff": sz["ff"]}, "mixer": {
        "heads": sz["heads"], "kv_heads": sz["kv_heads"], "dim": sz["dim"], "vdim": sz["dim"], "scale": sz["dim"] ** -0.5,
        "mask": {"size": SORIZEN_WINDOW, "keep_first": 0},
        "rot": {"dims": sz["dim"], "base": 1000000.0, "scaling": {"factor": 8.0, "original": 8192, "fast": 16.0, "slow": 2.0}}}}
    return {"architecture": "Dezolorn", "vocab": DESIGN_VOCAB, "width": sz["width"], "norm": {"eps": 1e-6},
            "layers": [attention] * sz["layers"], "loop": {"start": 0, "stop": 0, "times": 1}, "logit_scale": 1.0, "logit_softcap": 0.0}


def sorizen_bounds(kind: str, sz: dict, tokens: int, batch: int, context: int, pk: dict) -> dict[str, float]:
    """Seconds that every kernel of one step needs at least, over all its calls (see kernel_bounds)."""
    N = tokens or batch
    W, L, H = sz["width"], sz["layers"], sz["heads"]
    bw, tc = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    seen = lambda p: min(p + 1, SORIZEN_WINDOW)
    pairs = sum(seen(p) for p in range(tokens)) if tokens else batch * seen(context)
    out: dict[str, float] = {}
    if kind == "dezolorn":
        nkv, d = sz["kv_heads"], sz["dim"]
        out["ns_add_layernorm"] = 2 * L * 12.0 * N * W / bw
        out["ns_qk_norm_rope_store"] = L * 2.0 * N * ((H + nkv) * d * 2 + nkv * d + 2 * nkv * d) / bw
        if tokens:
            out["ns_attention_prefill_kept"] = L * 4.0 * H * d * pairs / tc
        else:
            out["ns_attention_decode_kept"] = L * 4.0 * pairs * nkv * d / bw
        out["ns_swiglu"] = L * 6.0 * N * sz["ff"] / bw
        return out
    S, R, r, d = sz["streams"], sz["rank"], sz["rot_dim"], sz["dim"]
    n_dense, n_moe = (L + 1) // 2, L // 2
    # the copies read and written in float32, the branch read and the normed row written in bfloat16 (the last call of a step
    # reads only); one call per sublayer and one at the end
    out["ns_stream_mix_norm"] = (2 * L + 1) * N * (8.0 * S * W + 4.0 * W) / bw
    out["ns_embed_streams"] = N * (2.0 * W + 4.0 * S * W) / bw
    out["ns_latent_rope_store"] = L * N * 2.0 * (2 * H * r + 2 * (R + r)) / bw
    if tokens:  # scores over R + r features and sums over R per (query, key, head), on the tensor cores
        out["ns_attention_latent_tc"] = L * 2.0 * H * (2 * R + r) * pairs / tc
    else:       # every visible latent once per request: the heads share it
        out["ns_attention_latent_tc"] = L * 2.0 * pairs * (R + r) / bw
    out["ns_activation"] = n_dense * 4.0 * N * sz["ff"] / bw
    E, top, eff = sz["experts"], sz["top"], sz["eff"]
    out["ns_router_logits"] = n_moe * (2.0 * N * W + 4.0 * E * W) / bw
    if tokens:
        out["ns_moe_gather"] = n_moe * 4.0 * N * top * W / bw
        out["ns_moe_combine"] = n_moe * 2.0 * N * (top + 1) * W / bw
        out["ns_swiglu"] = n_moe * 6.0 * N * top * eff / bw
    else:       # the weights of the experts that the step's tokens chose, once
        out["ns_moe_expert_rows"] = n_moe * min(E, batch * top) * 6.0 * eff * W / bw
    return out


def run_design_sorizen(args) -> dict:
    import torch

    from nanospec_b200 import random_model

    pk, pk_src = peaks()
    out_sizes = {}
    for name, sz in SORIZEN_SIZES.items():
        row = {}
        for kind in ("sorizen", "dezolorn"):
            cfg = sorizen_config(sz) if kind == "sorizen" else windowed_sibling(sz)
            model = random_model(cfg, seed=1, device="cuda", dtype=torch.bfloat16)
            pages_per_req = -(-(CONTEXT + args.repeats * args.steps + args.warmup + 64) // PAGE)
            eng = design_engine(model, 64, max(64 * pages_per_req, -(-PREFILL_TOKENS // PAGE) + 8) + 8)
            rec = {}
            for b in (8, 64):
                pt = time_decode(eng, b, args.steps, args.warmup, args.repeats)
                rec[f"decode_b{b}_tok_s"] = round(b * 1000.0 / pt["ms"], 1)
                rec[f"decode_b{b}_ms"] = round(pt["ms"], 4)
                rec[f"decode_b{b}_clocks"] = {"sm_mhz": pt["clocks"].get("sm_mhz"), "reasons": pt["clocks"].get("reasons")}
                if b == 8 and kind == "sorizen" and name == "w4096":
                    headline = pt
            pre_ms, pre_clocks = time_prefill(eng, warmup=3, iters=5)
            rec["prefill_tok_s"] = round(PREFILL_TOKENS * 1000.0 / pre_ms, 1)
            rec["prefill_ms"] = round(pre_ms, 3)
            rec["prefill_clocks"] = {"sm_mhz": pre_clocks.get("sm_mhz"), "reasons": pre_clocks.get("reasons")}
            del eng
            torch.cuda.empty_cache()
            kernels = {}
            for what, tokens, batch in (("prefill", PREFILL_TOKENS, 0), ("decode_b64", 0, 64)):
                timed = time_kernels(model, tokens, batch, CONTEXT)
                bounds = sorizen_bounds(kind, sz, tokens, batch, CONTEXT, pk)
                kernels[what] = {k: {"calls": n, "ms": round(ms, 4), "bound_ms": round(bounds[k] * 1e3, 4) if k in bounds else None,
                                     "frac": round(bounds[k] * 1e3 / ms, 4) if k in bounds and ms > 0 else None}
                                 for k, (n, ms) in sorted(timed.items(), key=lambda kv: -kv[1][1])}
            rec["kernels"] = kernels
            row[kind] = rec
            del model
            torch.cuda.empty_cache()
        out_sizes[name] = row
    value = out_sizes["w4096"]["sorizen"]["decode_b8_tok_s"]
    return {
        "metric": "decode tok/s (Sorizen, width 4,096, 4 layers, batch 8, 1,024-token context)", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": out_sizes["w4096"]["sorizen"]["decode_b8_ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform random token ids, random weights",
        "config": {"design": "sorizen beside dezolorn (attention layers)", "sizes": SORIZEN_SIZES, "vocab": DESIGN_VOCAB,
                   "window": SORIZEN_WINDOW, "seq_len": CONTEXT, "prefill_tokens": PREFILL_TOKENS, "page": PAGE, "cuda_graphs": True,
                   "peaks": pk_src, "l2": "the weights of every step are larger than L2"},
        "gpu_launches": headline["launches"], "clocks": headline["clocks"], "sizes": out_sizes,
    }


# ---- Debuvik beside Dezolorn attention layers and Sorizen latent layers (--design debuvik) --------------------------------

DEBUVIK_SIZES = {
    # width, feed-forward; chunked attention: heads / kv heads / key and value head sizes / rotated features; latent attention:
    # heads, head sizes, latent; columns of the token's side table per layer; layers (latent, attention, latent, attention
    # on the keys and values of the attention layer two before it, and so on)
    "w2048": dict(width=2048, ff=8192, heads=32, kv_heads=8, dim=128, vdim=64, rot=64, l_heads=16, l_dim=128, l_vdim=128, rank=512,
                  side=64, layers=8),
    "w4096": dict(width=4096, ff=14336, heads=32, kv_heads=8, dim=128, vdim=128, rot=64, l_heads=32, l_dim=128, l_vdim=128, rank=512,
                  side=128, layers=4),
}
DEBUVIK_CHUNK, DEBUVIK_CAP = 1536, 30.0  # chunks that the decoding context (1,024 tokens and the timed steps) stays inside
DEBUVIK_SIBLING_WINDOW = 1024


def debuvik_config(sz: dict) -> dict:
    mlp = {"kind": "dense", "ff": sz["ff"]}
    latent = {"type": "latent_attention", "mlp": mlp, "mixer": {
        "heads": sz["l_heads"], "dim": sz["l_dim"], "vdim": sz["l_vdim"], "kv_rank": sz["rank"], "scale": sz["l_dim"] ** -0.5}}

    def attention(i: int) -> dict:
        m = {"heads": sz["heads"], "kv_heads": sz["kv_heads"], "dim": sz["dim"], "vdim": sz["vdim"], "scale": sz["dim"] ** -0.5,
             "softcap": DEBUVIK_CAP, "mask": {"size": DEBUVIK_CHUNK},
             "rot": {"dims": sz["rot"], "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
        if i % 4 == 3:
            m["kv_from"] = i - 2
        return {"type": "attention", "mlp": mlp, "mixer": m}
    return {"architecture": "Debuvik", "vocab": DESIGN_VOCAB, "width": sz["width"], "norm": {"eps": 1e-6}, "token_side": {"dim": sz["side"]},
            "layers": [latent if i % 2 == 0 else attention(i) for i in range(sz["layers"])]}


def debuvik_attention_sibling(sz: dict) -> dict:
    """Dezolorn layers of windowed attention alone at the same width, feed-forward, heads and layer count: the closest model
    the framework had for the chunked attention layers (the same m16n8k16 kernels, a window where Debuvik has chunks)."""
    return windowed_sibling(dict(sz, dim=sz["dim"]))


def debuvik_latent_sibling(sz: dict) -> dict:
    """Sorizen layers of latent attention with a gate per head and a dense feed-forward, one plain stream, every key visible:
    the closest model the framework had for the latent layers (the same attention kernel, plus a rotated key part)."""
    mixer = {"heads": sz["l_heads"], "dim": sz["l_dim"], "rot_dim": 64, "vdim": sz["l_vdim"], "kv_rank": sz["rank"],
             "scale": (sz["l_dim"] + 64) ** -0.5, "mask": {"size": 1 << 16},
             "rot": {"dims": 64, "base": 1000000.0, "scaling": {"factor": 8.0, "original": 8192, "fast": 16.0, "slow": 2.0}}}
    layer = {"type": "latent_attention_2", "mixer": mixer, "mlp": {"kind": "dense", "ff": sz["ff"]}}
    return {"architecture": "Sorizen", "vocab": DESIGN_VOCAB, "width": sz["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "layers": [layer] * sz["layers"]}


def debuvik_bounds(kind: str, sz: dict, tokens: int, batch: int, context: int, pk: dict) -> dict[str, float]:
    """Seconds that every kernel of one step needs at least, over all its calls (see kernel_bounds)."""
    N = tokens or batch
    W, L = sz["width"], sz["layers"]
    bw, tc = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    out: dict[str, float] = {}
    if kind == "dezolorn":
        return sorizen_bounds("dezolorn", dict(sz, rot_dim=0, streams=1, experts=1, top=1, eff=1), tokens, batch, context, pk)
    R, Hl, dvl = sz["rank"], sz["l_heads"], sz["l_vdim"]
    causal = tokens * (tokens + 1) // 2 if tokens else batch * (context + 1)
    if kind == "sorizen":
        r = 64
        out["ns_add_layernorm"] = 2 * L * 12.0 * N * W / bw
        out["ns_latent_rope_store"] = L * N * 2.0 * (2 * Hl * r + 2 * (R + r)) / bw
        out["ns_attention_latent_tc"] = L * (2.0 * Hl * (2 * R + r) * causal / tc if tokens else 2.0 * causal * (R + r) / bw)
        out["ns_activation"] = L * 4.0 * N * sz["ff"] / bw
        return out
    n_lat, n_att, n_own = (L + 1) // 2, L // 2, sum(1 for i in range(L) if i % 4 == 1)
    nq, nkv, d, dv = sz["heads"], sz["kv_heads"], sz["dim"], sz["vdim"]
    seen = lambda p: p % DEBUVIK_CHUNK + 1  # keys of its own chunk that position p sees
    pairs = sum(seen(p) for p in range(tokens)) if tokens else batch * seen(context)
    # the stream read and written in float32, the branch read and the stream's copy written in bfloat16: after the mixer, the
    # feed-forward and the side input of every layer
    out["ns_norm_add"] = 3 * L * 12.0 * N * W / bw
    # q read and written, k and v read and stored (layers with projections of their own)
    out["ns_qk_norm_rope_store"] = (n_att * 4.0 * N * nq * d + n_own * 4.0 * N * nkv * (d + dv)) / bw
    if tokens:
        out["ns_attention_prefill_kept"] = n_att * 2.0 * nq * (d + dv) * pairs / tc
    else:
        out["ns_attention_decode_kept"] = n_att * 2.0 * pairs * nkv * (d + dv) / bw
    out["ns_latent_rope_store"] = n_lat * N * 4.0 * R / bw
    out["ns_attention_latent_tc"] = n_lat * (4.0 * Hl * R * causal / tc if tokens else 2.0 * causal * R / bw)
    out["ns_sigmoid_mul"] = n_lat * 6.0 * N * Hl * dvl / bw
    out["ns_swiglu"] = L * 6.0 * N * sz["ff"] / bw
    out["ns_token_gate"] = L * 6.0 * N * sz["side"] / bw
    return out


# a Debuvik kernel and the kernel of a sibling that does the like work
DEBUVIK_LIKE = {"ns_norm_add": ("dezolorn", "ns_add_layernorm"), "ns_qk_norm_rope_store": ("dezolorn", "ns_qk_norm_rope_store"),
                "ns_attention_prefill_kept": ("dezolorn", "ns_attention_prefill_kept"),
                "ns_attention_decode_kept": ("dezolorn", "ns_attention_decode_kept"), "ns_swiglu": ("dezolorn", "ns_swiglu"),
                "ns_latent_rope_store": ("sorizen", "ns_latent_rope_store"), "ns_attention_latent_tc": ("sorizen", "ns_attention_latent_tc"),
                "ns_sigmoid_mul": ("sorizen", "ns_activation"), "ns_token_gate": ("sorizen", "ns_activation")}


def run_design_debuvik(args) -> dict:
    import torch

    from nanospec_b200 import random_model

    pk, pk_src = peaks()
    makers = {"debuvik": debuvik_config, "dezolorn": debuvik_attention_sibling, "sorizen": debuvik_latent_sibling}
    out_sizes = {}
    for name, sz in DEBUVIK_SIZES.items():
        row = {}
        for kind, maker in makers.items():
            model = random_model(maker(sz), seed=1, device="cuda", dtype=torch.bfloat16)
            pages_per_req = -(-(CONTEXT + args.repeats * args.steps + args.warmup + 64) // PAGE)
            eng = design_engine(model, 64, max(64 * pages_per_req, -(-PREFILL_TOKENS // PAGE) + 8) + 8)
            rec = {}
            for b in (8, 64):
                pt = time_decode(eng, b, args.steps, args.warmup, args.repeats)
                rec[f"decode_b{b}_tok_s"] = round(b * 1000.0 / pt["ms"], 1)
                rec[f"decode_b{b}_ms"] = round(pt["ms"], 4)
                rec[f"decode_b{b}_clocks"] = {"sm_mhz": pt["clocks"].get("sm_mhz"), "reasons": pt["clocks"].get("reasons")}
                if b == 8 and kind == "debuvik" and name == "w4096":
                    headline = pt
            pre_ms, pre_clocks = time_prefill(eng, warmup=3, iters=5)
            rec["prefill_tok_s"] = round(PREFILL_TOKENS * 1000.0 / pre_ms, 1)
            rec["prefill_ms"] = round(pre_ms, 3)
            rec["prefill_clocks"] = {"sm_mhz": pre_clocks.get("sm_mhz"), "reasons": pre_clocks.get("reasons")}
            del eng
            torch.cuda.empty_cache()
            kernels = {}
            for what, tokens, batch in (("prefill", PREFILL_TOKENS, 0), ("decode_b64", 0, 64)):
                timed = time_kernels(model, tokens, batch, CONTEXT)
                bounds = debuvik_bounds(kind, sz, tokens, batch, CONTEXT, pk)
                kernels[what] = {k: {"calls": n, "ms": round(ms, 4), "bound_ms": round(bounds[k] * 1e3, 4) if k in bounds else None,
                                     "frac": round(bounds[k] * 1e3 / ms, 4) if k in bounds and ms > 0 else None}
                                 for k, (n, ms) in sorted(timed.items(), key=lambda kv: -kv[1][1])}
            rec["kernels"] = kernels
            row[kind] = rec
            del model
            torch.cuda.empty_cache()
        # every Debuvik kernel's fraction of its bound over the like kernel's of a sibling (below 0.5: more than twice as far)
        like = {}
        for what in ("prefill", "decode_b64"):
            for k, v in row["debuvik"]["kernels"][what].items():
                other = row[DEBUVIK_LIKE[k][0]]["kernels"][what].get(DEBUVIK_LIKE[k][1]) if k in DEBUVIK_LIKE else None
                if v["frac"] and other and other["frac"]:
                    like[f"{what}:{k}"] = {"frac": v["frac"], "like": "/".join(DEBUVIK_LIKE[k]), "like_frac": other["frac"],
                                           "ratio": round(v["frac"] / other["frac"], 3)}
        row["like"] = like
        out_sizes[name] = row
    value = out_sizes["w4096"]["debuvik"]["decode_b8_tok_s"]
    return {
        "metric": "decode tok/s (Debuvik, width 4,096, 4 layers, batch 8, 1,024-token context)", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": out_sizes["w4096"]["debuvik"]["decode_b8_ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform random token ids, random weights",
        "config": {"design": "debuvik beside dezolorn (attention layers) and sorizen (latent layers)", "sizes": DEBUVIK_SIZES,
                   "vocab": DESIGN_VOCAB, "chunk": DEBUVIK_CHUNK, "softcap": DEBUVIK_CAP, "sibling_window": DEBUVIK_SIBLING_WINDOW,
                   "seq_len": CONTEXT, "prefill_tokens": PREFILL_TOKENS, "page": PAGE, "cuda_graphs": True, "peaks": pk_src,
                   "l2": "the weights of every step are larger than L2"},
        "gpu_launches": headline["launches"], "clocks": headline["clocks"], "sizes": out_sizes,
    }


# ---- Fubolix beside Dezolorn attention layers (--design fubolix) -------------------------------------------------------------

FUBOLIX_SIZES = {
    # width, feed-forward, heads / kv heads / head size, layers (in the pattern windowed, convolved, windowed, tempered)
    "w2048": dict(width=2048, ff=8192, heads=32, kv_heads=8, dim=64, layers=8),
    "w4096": dict(width=4096, ff=14336, heads=32, kv_heads=8, dim=128, layers=4),
}
FUBOLIX_CONV, FUBOLIX_TEMP_EVERY = 4, 128


def fubolix_config(sz: dict) -> dict:
    d = sz["dim"]
    yarn = {"factor": 8.0, "original": 8192, "fast": 16.0, "slow": 2.0}
    base = {"heads": sz["heads"], "kv_heads": sz["kv_heads"], "dim": d, "vdim": d, "scale": d ** -0.5}
    mlp = {"kind": "dense", "ff": sz["ff"]}
    windowed = {"type": "attention", "mlp": mlp, "mixer": {**base, "mask": {"size": DESIGN_WINDOW, "keep_first": DESIGN_KEEP},
                                                            "rot": {"dims": d // 2, "base": 1000000.0, "scaling": yarn}}}
    convolved = {"type": "attention_3", "mlp": mlp, "mixer": {**base, "conv": FUBOLIX_CONV, "rot": {"dims": d, "base": 1000000.0, "scaling": yarn}}}
    tempered = {"type": "attention_2", "mlp": mlp, "mixer": {**base, "q_temp": {"coef": 0.25, "every": FUBOLIX_TEMP_EVERY}}}
    pattern = [windowed, convolved, windowed, tempered]
    return {"architecture": "Fubolix", "vocab": DESIGN_VOCAB, "width": sz["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0},
            "layers": [pattern[i % 4] for i in range(sz["layers"])]}


def fubolix_sibling(sz: dict) -> dict:
    """The closest model the framework had: Dezolorn layers of windowed attention with kept first keys alone (layer norm, q/k norm,
    rotation with scaling, the same m16n8k16 attention kernels), at the same width, feed-forward width, heads and layer count."""
    cfg = windowed_sibling(sz)
    for layer in cfg["layers"]:
        layer["mixer"] = {**layer["mixer"], "mask": {"size": DESIGN_WINDOW, "keep_first": DESIGN_KEEP}}
    return cfg


def fubolix_bounds(kind: str, sz: dict, tokens: int, batch: int, context: int, pk: dict) -> dict[str, float]:
    """Seconds that every kernel of one step needs at least, over all its calls (see kernel_bounds)."""
    N = tokens or batch
    W, L, H, nkv, d = sz["width"], sz["layers"], sz["heads"], sz["kv_heads"], sz["dim"]
    bw, tc = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    seen_w = lambda p: min(p + 1, DESIGN_WINDOW) + max(0, min(DESIGN_KEEP, p + 1 - DESIGN_WINDOW))
    pairs_w = sum(seen_w(p) for p in range(tokens)) if tokens else batch * seen_w(context)
    pairs_all = tokens * (tokens + 1) // 2 if tokens else batch * (context + 1)
    out: dict[str, float] = {}
    if kind == "dezolorn":
        out["ns_add_layernorm"] = 2 * L * 12.0 * N * W / bw
        out["ns_qk_norm_rope_store"] = L * 2.0 * N * ((H + nkv) * d * 2 + nkv * d + 2 * nkv * d) / bw
        if tokens:
            out["ns_attention_prefill_kept"] = L * 4.0 * H * d * pairs_w / tc
        else:
            out["ns_attention_decode_kept"] = L * 4.0 * pairs_w * nkv * d / bw
        out["ns_swiglu"] = L * 6.0 * N * sz["ff"] / bw
        return out
    n_win = sum(1 for i in range(L) if i % 4 in (0, 2))
    n_all = L - n_win
    # one norm a layer: the stream read and written in float32, two branches read and the result written in bfloat16 (the first
    # has no branches yet); the model's last norm reads the wanted rows only
    out["ns_add_dyt"] = ((L - 1) * 14.0 + 6.0) * N * W / bw
    # projections read and q, k written back, k and v to the cache; a windowed layer has no v to read
    out["ns_head_prepare_store"] = 2.0 * N * (L * ((H + nkv) * d * 2 + 2 * nkv * d) + n_all * nkv * d) / bw
    if tokens:
        out["ns_attention_prefill_kept"] = 4.0 * H * d * (n_win * pairs_w + n_all * pairs_all) / tc
    else:
        out["ns_attention_decode_kept"] = 4.0 * (n_win * pairs_w + n_all * pairs_all) * nkv * d / bw
    out["ns_activation"] = out["ns_activation_rows"] = L * 4.0 * N * sz["ff"] / bw  # (rows of a wider buffer when the block packs its products)
    out["ns_residual_add"] = 10.0 * N * W / bw
    out["ns_embed_streams"] = 6.0 * N * W / bw
    return out


def run_design_fubolix(args) -> dict:
    import torch

    from nanospec_b200 import random_model

    pk, pk_src = peaks()
    out_sizes = {}
    for name, sz in FUBOLIX_SIZES.items():
        row = {}
        for kind in ("fubolix", "dezolorn"):
            cfg = fubolix_config(sz) if kind == "fubolix" else fubolix_sibling(sz)
            model = random_model(cfg, seed=1, device="cuda", dtype=torch.bfloat16)
            pages_per_req = -(-(CONTEXT + args.repeats * args.steps + args.warmup + 64) // PAGE)
            eng = design_engine(model, 64, max(64 * pages_per_req, -(-PREFILL_TOKENS // PAGE) + 8) + 8)
            rec = {}
            for b in (8, 64):
                pt = time_decode(eng, b, args.steps, args.warmup, args.repeats)
                rec[f"decode_b{b}_tok_s"] = round(b * 1000.0 / pt["ms"], 1)
                rec[f"decode_b{b}_ms"] = round(pt["ms"], 4)
                rec[f"decode_b{b}_clocks"] = {"sm_mhz": pt["clocks"].get("sm_mhz"), "reasons": pt["clocks"].get("reasons")}
                if b == 8 and kind == "fubolix" and name == "w4096":
                    headline = pt
            pre_ms, pre_clocks = time_prefill(eng, warmup=3, iters=5)
            rec["prefill_tok_s"] = round(PREFILL_TOKENS * 1000.0 / pre_ms, 1)
            rec["prefill_ms"] = round(pre_ms, 3)
            rec["prefill_clocks"] = {"sm_mhz": pre_clocks.get("sm_mhz"), "reasons": pre_clocks.get("reasons")}
            del eng
            torch.cuda.empty_cache()
            kernels = {}
            for what, tokens, batch in (("prefill", PREFILL_TOKENS, 0), ("decode_b64", 0, 64)):
                timed = time_kernels(model, tokens, batch, CONTEXT)
                bounds = fubolix_bounds(kind, sz, tokens, batch, CONTEXT, pk)
                kernels[what] = {k: {"calls": n, "ms": round(ms, 4), "bound_ms": round(bounds[k] * 1e3, 4) if k in bounds else None,
                                     "frac": round(bounds[k] * 1e3 / ms, 4) if k in bounds and ms > 0 else None}
                                 for k, (n, ms) in sorted(timed.items(), key=lambda kv: -kv[1][1])}
            rec["kernels"] = kernels
            row[kind] = rec
            del model
            torch.cuda.empty_cache()
        out_sizes[name] = row
    value = out_sizes["w4096"]["fubolix"]["decode_b8_tok_s"]
    return {
        "metric": "decode tok/s (Fubolix, width 4,096, 4 layers, batch 8, 1,024-token context)", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": out_sizes["w4096"]["fubolix"]["decode_b8_ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform random token ids, random weights",
        "config": {"design": "fubolix beside dezolorn (attention layers)", "sizes": FUBOLIX_SIZES, "vocab": DESIGN_VOCAB,
                   "window": DESIGN_WINDOW, "keep_first": DESIGN_KEEP, "conv": FUBOLIX_CONV, "seq_len": CONTEXT,
                   "prefill_tokens": PREFILL_TOKENS, "page": PAGE, "cuda_graphs": True, "peaks": pk_src,
                   "l2": "the weights of every step are larger than L2"},
        "gpu_launches": headline["launches"], "clocks": headline["clocks"], "sizes": out_sizes,
    }


def run_reference(args) -> dict:
    from baseline import reference_arm

    return reference_arm.run(args, SHAPE, ROPE, CONTEXT, PREFILL_TOKENS, PAGE, ClockSampler)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--repeats", type=int, default=5, help="the timed steps are run this many times; the median repeat is reported")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=SHAPE["num_hidden_layers"])
    ap.add_argument("--no-workloads", action="store_true", help="leave out the 3B continuous-batching and 1B mixed workloads")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--design", choices=["dezolorn", "sorizen", "debuvik", "fubolix"], help="measure this design beside its closest sibling of equal size instead")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    args.repeats = max(1, args.repeats)
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    out = run_reference(args) if args.impl == "reference" else run_design_fubolix(args) if args.design == "fubolix" else run_design_sorizen(args) if args.design == "sorizen" else run_design_debuvik(args) if args.design == "debuvik" else run_design(args) if args.design else run_ours(args)
    print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
