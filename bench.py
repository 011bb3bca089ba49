#!/usr/bin/env python3
"""Headline benchmark: decode tokens/s of the Orpheus-3B-sized Llama decoder (random
weights, bfloat16) at batch 8 with 2,048-token cached prompts and pages of 16 tokens, on
one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--rounds R] [--page-size P]
                    [--impl ours|reference] [--workloads all|none|mixed64|long8]
    python bench.py --arch tifosun|vudivik|relurax|mokotar [--arch-size small|medium]   (another architecture)

One JSON line on stdout.  ``value``: decoded tokens per second of the engine's step
function plus greedy sampling, timed on the device with CUDA events: W warm-up steps, then
R rounds of exactly K steps each; ``ms_per_step`` is the median round, the fastest and
slowest are beside it.  ``e2e``: the same through the Python entry point (``LLM.step``),
host token ids in and out.  ``prefill``: one 2,048-token prompt in one step.
``roofline``: bytes a decode step has to read (every weight once, and the cache of the
live requests) over its time, against the measured copy bandwidth.  ``points``: decode at
batch 1 and 64, batch 8 with pages of 64 tokens, and two serving workloads through the
entry point at other sizes of the architecture (64 mixed requests at the Llama 3.2 1B
sizes, 8 long prompts in portions at the Llama 3.1 8B sizes), each as generated tokens per
second and median time to the first token.  A step is one decode step; every step reads
all weights (6.6 GB), far more than the 126 MB L2, so no L2 flush is needed.
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Layer sizes of the benchmark model: Orpheus 3B / Llama 3.2 3B
# (mstar/model/orpheus/config.py:4-23).
ORPHEUS_3B = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=28, hidden_size=3072,
    num_attention_heads=24, num_key_value_heads=8, head_dim=128, intermediate_size=8192,
    vocab_size=156940, tie_word_embeddings=True, rope_theta=500000.0,
    rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                  "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    rms_norm_eps=1e-5, max_position_embeddings=131072, hidden_act="silu",
    torch_dtype="bfloat16",
)
# Further sizes of the same architecture (--sizes): Llama 3.2 1B and Llama 3.1 8B.
LLAMA_1B = dict(ORPHEUS_3B, num_hidden_layers=16, hidden_size=2048, num_attention_heads=32,
                head_dim=64, vocab_size=128256)
LLAMA_8B = dict(ORPHEUS_3B, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                intermediate_size=14336, vocab_size=128256, tie_word_embeddings=False,
                rope_scaling=dict(ORPHEUS_3B["rope_scaling"], factor=8.0))
SIZES = {"orpheus-3b": ("Orpheus 3B / Llama 3.2 3B", ORPHEUS_3B),
         "llama-1b": ("Llama 3.2 1B", LLAMA_1B), "llama-8b": ("Llama 3.1 8B", LLAMA_8B)}
PROMPT_LEN = 2048
CONTEXT = 4096
PAGE_SIZE = 16          # the default of --page-size; kernel_bench reads the global
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                     "--format=csv,noheader,nounits"], capture_output=True, text=True,
                    timeout=5).stdout.strip().splitlines()[0]
                parts = [p.strip() for p in out.split(",")]
                self.samples.append(float(parts[0]))
                self.max_mhz = float(parts[1])
                for name, val in zip(self.NAMES, parts[2:]):
                    if val.lower().startswith("active"):
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def flops_of_step(cfg: dict, q_lens, kv_lens, rows: int) -> float:
    """Matrix and attention FLOPs of one step (2 per multiply-add)."""
    L, H, I, V = (cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"],
                  cfg["vocab_size"])
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = sum(q_lens)
    per_token = (H * (nq + 2 * nkv) * hd) + (nq * hd * H) + 3 * H * I
    linear = 2.0 * T * L * per_token + 2.0 * rows * H * V
    attn = 0.0
    for q, kv in zip(q_lens, kv_lens):
        keys = sum(kv - q + i + 1 for i in range(q))     # causal: token i sees kv-q+i+1 keys
        attn += 4.0 * nq * hd * keys
    return linear + L * attn


def bytes_of_decode_step(cfg: dict, model, kv_lens) -> float:
    """Every weight used once (tied head counted once) plus keys and values read."""
    nkv, hd, L = cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    kv = sum(kv_lens) * 2 * nkv * hd * 2 * L
    return float(model.parameter_bytes() + kv)


def build_model(cfg_raw: dict, seed: int = 0):
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.engine.model import load_model
    from mstar_b200.weights.random_init import random_checkpoint

    cfg = config_from_dict(cfg_raw)
    tensors = random_checkpoint(cfg, seed, std=0.02, device="cuda:0")
    model = load_model(None, dtype="bfloat16", device="cuda:0", config=cfg, tensors=tensors)
    del tensors
    return model


def prompts(batch: int, vocab: int, length: int, seed: int = 1) -> list:
    import torch

    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=g).tolist()


def time_decode(stepper, batch: int, cfg: dict, steps: int, warmup: int, rounds: int = 1) -> dict:
    """B requests with PROMPT_LEN cached tokens each; W warm-up decode steps of the step
    function plus greedy sampling, then ``rounds`` rounds of exactly K steps, each round timed
    with CUDA events.  The median round is the result; fastest and slowest are reported."""
    import torch

    from mstar_b200 import ops
    from mstar_b200.engine.step import StepEntry
    from mstar_b200.ops import lib

    ids = [f"d{batch}-{i}" for i in range(batch)]
    total = warmup + rounds * steps
    toks = prompts(batch, cfg["vocab_size"], PROMPT_LEN + total + 1, seed=batch)
    for rid, t in zip(ids, toks):
        stepper.add_request(rid)
        stepper.step([StepEntry(rid, t[:PROMPT_LEN], ())])
    torch.cuda.synchronize()

    def one(k: int):
        logits = stepper.step([StepEntry(rid, [t[PROMPT_LEN + k]], (0,))
                               for rid, t in zip(ids, toks)])
        return ops.argmax(logits)

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    times, launches = [], 0
    for r in range(rounds):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = lib.launch_count()
        start.record()
        for k in range(warmup + r * steps, warmup + (r + 1) * steps):
            one(k)
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / steps)
        launches = lib.launch_count() - launches0
    ops.check_error_word(stepper.device)
    ms = statistics.median(times)
    kv_lens = [PROMPT_LEN + warmup + (rounds * steps) // 2] * batch
    for rid in ids:
        stepper.free_request(rid)
    return {"ms_per_step": ms, "ms_min": min(times), "ms_max": max(times),
            "tokens_per_s": batch / (ms / 1e3), "launches": launches, "kv_lens": kv_lens}


def time_prefill(stepper, cfg: dict, reps: int = 5) -> dict:
    import torch

    from mstar_b200.engine.step import StepEntry

    toks = prompts(reps + 2, cfg["vocab_size"], PROMPT_LEN, seed=99)
    times = []
    for i, t in enumerate(toks):
        rid = f"p{i}"
        stepper.add_request(rid)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        stepper.step([StepEntry(rid, t, (PROMPT_LEN - 1,))])
        end.record()
        torch.cuda.synchronize()
        stepper.free_request(rid)
        if i >= 2:                                   # two warm-up prompts
            times.append(start.elapsed_time(end))
    ms = statistics.median(times)
    return {"ms": ms, "tokens_per_s": PROMPT_LEN / (ms / 1e3),
            "flops": flops_of_step(cfg, [PROMPT_LEN], [PROMPT_LEN], 1)}


def time_e2e(model, batch: int, cfg: dict, steps: int, warmup: int, num_pages: int,
             page_size: int, rounds: int = 1) -> dict:
    """The same decode steps through the public entry point: host token ids in (pinned
    index buffer copied to the device every step) and sampled token ids read back; wall
    clock around ``rounds`` rounds of K steps, the median round reported."""
    import torch

    from mstar_b200 import LLM, SamplingParams

    llm = LLM(model, page_size=page_size, max_num_pages=num_pages,
              max_num_batched_tokens=PROMPT_LEN, max_concurrent_requests=max(batch, 1),
              max_batch_size=max(batch, 1))
    params = SamplingParams(temperature=0.0, ignore_eos=True,
                            max_output_tokens=warmup + rounds * steps + batch + 8)
    for i, t in enumerate(prompts(batch, cfg["vocab_size"], PROMPT_LEN, seed=7 + batch)):
        llm.add_request(t, params, request_id=f"e{i}")
    while any(r.num_pending() > 1 for r in llm.scheduler.running) or llm.scheduler.waiting:
        llm.step()                                   # prompts, one per step
    for _ in range(warmup):
        llm.step()
    times = []
    for _ in range(rounds):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            llm.step()
        torch.cuda.synchronize()
        times.append((time.perf_counter() - t0) / steps * 1e3)
    ms = statistics.median(times)
    h2d = llm.stepper.last_h2d_bytes
    for r in list(llm.scheduler.running):
        llm.scheduler.abort(r.request_id)
    # tokens out: 4 bytes a request, and the 4-byte word kernels report a given-up wait in
    return {"tokens_per_s": batch / (ms / 1e3), "ms_per_step": ms, "ms_min": min(times),
            "ms_max": max(times), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch + 4}


# ------------------------------------------------------------------ serving workloads
WORKLOADS = {
    # 64 requests at once, prompts of 16 to 2,048 tokens, 256 new tokens each
    "mixed64": dict(sizes="llama-1b", requests=64, prompt=(16, 2048), new_tokens=256,
                    budget=2048),
    # 8 prompts of 8,192 tokens, computed in portions of 2,048, 128 new tokens each
    "long8": dict(sizes="llama-8b", requests=8, prompt=(8192, 8192), new_tokens=128,
                  budget=2048),
}


def run_workload(name: str, page_size: int) -> dict:
    """A whole serving run through the entry point: all requests are handed over at time
    zero, the scheduler admits, cuts prompts into portions under its token budget, decodes
    and frees.  Run twice (the first run captures the decode graphs and compiles nothing
    else); the second is timed by the wall clock.  Greedy sampling, no stop token."""
    import numpy as np
    import torch

    from mstar_b200 import LLM, SamplingParams

    w = WORKLOADS[name]
    model_name, cfg = SIZES[w["sizes"]]
    print(f"[bench] workload {name}: {w['requests']} requests at the {model_name} sizes ...",
          file=sys.stderr, flush=True)
    model = build_model(dict(cfg), seed=2)
    rng = np.random.default_rng(5)
    lens = rng.integers(w["prompt"][0], w["prompt"][1] + 1, size=w["requests"]).tolist()
    g = torch.Generator().manual_seed(11)
    prompt_ids = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    pages = sum(-(-(n + w["new_tokens"]) // page_size) for n in lens) + 64
    llm = LLM(model, page_size=page_size, max_num_pages=pages,
              max_num_batched_tokens=w["budget"], max_concurrent_requests=w["requests"],
              max_batch_size=w["requests"])
    params = SamplingParams(temperature=0.0, ignore_eos=True, max_output_tokens=w["new_tokens"])
    result, before = {}, None
    for run in ("warm-up", "timed"):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ids = [llm.add_request(p, params, request_id=f"{name}-{run}-{i}")
               for i, p in enumerate(prompt_ids)]
        waiting = {r.request_id: r for r in llm.scheduler.waiting}
        first: dict = {}
        done = 0
        while llm.has_unfinished():
            done += len(llm.step())
            if len(first) < len(ids):
                now = time.perf_counter() - t0
                for rid, r in waiting.items():
                    if rid not in first and r.output and r.output[0] is not None:
                        first[rid] = now
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        assert done == len(ids) and len(first) == len(ids)
        generated = w["requests"] * w["new_tokens"]
        # the two runs decode the same prompts greedily: the same tokens, whatever the
        # batches were that the scheduler formed
        tokens = [list(waiting[rid].output) for rid in ids]
        agree = None if run == "warm-up" else tokens == before
        before = tokens
        result = {"tokens_per_s": generated / seconds, "seconds": seconds, "runs_agree": agree,
                  "ttft_ms_median": statistics.median(first.values()) * 1e3,
                  "ttft_ms_max": max(first.values()) * 1e3,
                  "prompt_tokens": sum(lens), "generated_tokens": generated,
                  "steps": llm.stats.steps, "preemptions": llm.stats.preemptions}
        llm.stats.steps = 0
    del llm, model
    torch.cuda.empty_cache()
    return result


# ------------------------------------------------------------------ another architecture
def tifosun_sizes(name: str) -> tuple:
    """(Tifosun config, Llama config of equal size) at layer sizes that resemble a real
    model's: three matrix-memory layers to one windowed latent-attention layer, routed
    experts with a shared one in most layers and a dense feed-forward in the first.  The
    Llama beside it has the same width, depth and vocabulary, heads of 128, and a
    feed-forward as wide as the experts a Tifosun token uses (top experts + shared)."""
    if name == "small":
        width, depth, vocab = 1024, 8, 32000
        mem = dict(heads=4, dim=128, vdim=256, gate_cap=15.0)
        att = dict(heads=8, dim=64, rot_dim=32, vdim=128, kv_rank=256, mask={"size": 512},
                   rot={"base": 10000.0, "dims": 32}, scale=96 ** -0.5)
        experts, top, ff, shared, dense = 16, 2, 512, 1024, 3072
    elif name == "medium":
        width, depth, vocab = 2048, 12, 64000
        mem = dict(heads=4, dim=256, vdim=512, gate_cap=15.0)
        att = dict(heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, mask={"size": 1024},
                   rot={"base": 10000.0, "dims": 64}, scale=192 ** -0.5)
        experts, top, ff, shared, dense = 32, 4, 768, 2048, 6144
    else:
        raise ValueError(f"unknown size {name!r} (small, medium)")
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
           "shared": {"ff": shared}}
    layers = []
    for i in range(depth):
        kind = "latent_attention" if i % 4 == 2 else ("mlstm_2" if i % 4 == 3 else "mlstm")
        layers.append({"type": kind, "mixer": dict(att if kind == "latent_attention" else mem),
                       "mlp": {"kind": "dense", "ff": dense} if i == 0 else moe})
    tifosun = {"architecture": "Tifosun", "width": width, "vocab": vocab, "norm": {"eps": 1e-6},
               "layers": layers}
    llama = dict(ORPHEUS_3B, num_hidden_layers=depth, hidden_size=width,
                 num_attention_heads=width // 128, num_key_value_heads=max(width // 512, 1),
                 head_dim=128, intermediate_size=top * ff + shared, vocab_size=vocab,
                 tie_word_embeddings=False)
    return tifosun, llama


def _time_models(args, models, out: dict) -> None:
    """Prefill of one prompt and a decode step at ``args.batch`` for each (name, raw config),
    through the step function, into ``out["models"]``."""
    import torch

    from mstar_b200.engine.step import StepEntry, make_stepper

    page, batch = args.page_size, args.batch
    for name, raw in models:
        print(f"[bench] {name} at the {args.arch_size} sizes ...", file=sys.stderr, flush=True)
        model = build_model(raw)
        cfg = {"vocab_size": model.vocab_size}
        stepper = make_stepper(model, page_size=page, num_pages=batch * (CONTEXT // page) + 64,
                               num_slots=batch + 4)
        toks = prompts(7, model.vocab_size, PROMPT_LEN, seed=99)
        times = []
        for i, t in enumerate(toks):
            stepper.add_request(f"p{i}")
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            stepper.step([StepEntry(f"p{i}", t, (PROMPT_LEN - 1,))])
            end.record()
            torch.cuda.synchronize()
            stepper.free_request(f"p{i}")
            if i >= 2:
                times.append(start.elapsed_time(end))
        pre_ms = statistics.median(times)
        dec = time_decode(stepper, batch, cfg, args.steps, max(args.warmup, 3), min(args.rounds, 3))
        out["models"][name] = {
            "parameters_gb": round(model.parameter_bytes() / 1e9, 3),
            "prefill_ms": round(pre_ms, 3), "prefill_tok_s": round(PROMPT_LEN / pre_ms * 1e3, 1),
            "decode_ms_per_step": round(dec["ms_per_step"], 4),
            "decode_tok_s": round(dec["tokens_per_s"], 1), "launches_per_step": dec["launches"] // args.steps}
        del stepper, model
        torch.cuda.empty_cache()


def arch_bench(args) -> int:
    """``--arch tifosun``: prefill and decode throughput of the Tifosun decoder (random
    weights, bfloat16) at ``--arch-size``, beside the Llama decoder at equal size, through the
    same step function; and its own kernels alone at those sizes with what each has to move
    or compute, against the measured peaks.  One JSON line."""
    import torch

    from mstar_b200 import ops

    if args.arch == "vudivik":
        return vudivik_bench(args)
    if args.arch == "relurax":
        return relurax_bench(args)
    if args.arch == "mokotar":
        return mokotar_bench(args)
    pk = peaks()
    t_cfg, l_cfg = tifosun_sizes(args.arch_size)
    page, batch = args.page_size, args.batch
    out = {"arch": "Tifosun", "size": args.arch_size, "batch": batch, "prompt_len": PROMPT_LEN,
           "peaks": pk["source"], "models": {}, "kernels": {}}
    _time_models(args, (("tifosun", t_cfg), ("llama", l_cfg)), out)

    # ---- the new kernels alone, at the sizes of one layer
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (scale * torch.randn(*shape, generator=g, device=dev)).to(torch.bfloat16)

    def i32(v):
        return torch.tensor(v, dtype=torch.int32, device=dev)

    width = t_cfg["width"]
    mem = next(l["mixer"] for l in t_cfg["layers"] if l["type"] == "mlstm")
    att = next(l["mixer"] for l in t_cfg["layers"] if l["type"] == "latent_attention")
    moe = next(l["mlp"] for l in t_cfg["layers"] if l["mlp"]["kind"] == "moe")
    K = out["kernels"]
    H, dim, vdim = mem["heads"], mem["dim"], mem["vdim"]
    size = ops.matrix_memory_state_size(H, dim, vdim)
    copies = max(1, -(-(160 << 20) // (size * 4 * batch)))          # states larger than L2
    state = torch.zeros(copies * batch + 1, size, device=dev)
    for tokens, entries, label in ((batch, batch, "decode"), (PROMPT_LEN, 1, "prefill")):
        proj = rnd(tokens, 2 * H * dim + 2 * H * vdim)
        gates = torch.randn(tokens, 2 * H, device=dev)
        bias = torch.zeros(2 * H, device=dev)
        per = tokens // entries
        indptr = i32([k * per for k in range(entries + 1)])
        turn = {"i": 0}

        def scan():
            base = (turn["i"] % copies) * batch
            turn["i"] += 1
            return ops.matrix_memory_scan(proj, gates, bias, indptr, slot_sets[base // batch],
                                          state, entries, H, dim, vdim, 15.0, dim ** -0.5, 1e-6)

        slot_sets = [i32([c * batch + k for k in range(entries)]) for c in range(copies)]
        ms = _time_graph(scan, reps=max(copies, 4) if label == "decode" else 2)
        nbytes = 2.0 * entries * size * 4
        K[f"matrix_memory_scan_{label}"] = {
            "ms": round(ms, 4), "state_gbs": round(nbytes / ms / 1e6, 1),
            "frac_hbm": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4),
            "tokens_per_chain_us": round(per / (ms * 1e3), 3)}
    heads, rank, rot, window = att["heads"], att["kv_rank"], att["rot_dim"], att["mask"]["size"]
    for tokens, reqs, label in ((batch, batch, "decode"), (PROMPT_LEN, 1, "prefill")):
        ctx = PROMPT_LEN
        pages_per = -(-ctx // page)
        copies = 1 if label == "prefill" else max(1, -(-(160 << 20) // (reqs * window * (rank + rot) * 2)))
        caches = [rnd(reqs * pages_per + 1, 1, 1, page, rank + rot) for _ in range(copies)]
        table = torch.randperm(reqs * pages_per, device=dev).to(torch.int32).view(reqs, pages_per)
        per = tokens // reqs
        token_req = i32([r for r in range(reqs) for _ in range(per)])
        cache_pos = i32([ctx - per + k for _ in range(reqs) for k in range(per)])
        q_abs = torch.randn(tokens, heads, rank, device=dev)
        q_rot = rnd(tokens, heads, rot)
        turn = {"i": 0}

        def attend():
            c = caches[turn["i"] % copies]
            turn["i"] += 1
            return ops.latent_attention(q_abs, q_rot, c, table, token_req, cache_pos, heads, rank,
                                        rot, page, window, att["scale"], entries=reqs)

        ms = _time_graph(attend, reps=max(copies, 4) if label == "decode" else 2)
        keys = sum(min(ctx - per + k + 1, window) for k in range(per)) * reqs
        flops = 2.0 * heads * keys * (2 * rank + rot)
        nbytes = reqs * min(ctx, window + per) * (rank + rot) * 2.0
        K[f"latent_attention_{label}"] = {
            "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 2),
            "frac_bf16": round(flops / ms / 1e9 / pk["bf16_tflops"], 5),
            "gbs": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4)}
    E, top, ff = moe["router"]["experts"], moe["router"]["top"], moe["expert"]["ff"]
    copies = max(1, -(-(160 << 20) // (E * 3 * ff * width * 2)))
    w_gu = [rnd(E * 2 * ff, width, scale=0.02) for _ in range(copies)]
    w_dn = [rnd(E * width, ff, scale=0.02) for _ in range(copies)]
    for tokens, label in ((batch, "decode"), (PROMPT_LEN, "prefill")):
        x = rnd(tokens, width)
        chosen, weight = ops.route_topk(torch.randn(tokens, E, device=dev), top)
        turn = {"i": 0}

        def experts():
            k = turn["i"] % copies
            turn["i"] += 1
            return ops.routed_experts(x, w_gu[k], w_dn[k], chosen, weight, E, ff, True)

        ms = _time_graph(experts, reps=max(copies * 2, 4) if label == "decode" else 2)
        used = len(set(chosen.flatten().tolist()))
        nbytes = used * 3.0 * ff * width * 2
        flops = 2.0 * tokens * top * 3 * ff * width
        K[f"routed_experts_{label}"] = {
            "ms": round(ms, 4), "experts_used": used, "gbs": round(nbytes / ms / 1e6, 1),
            "frac_hbm": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4),
            "tflops": round(flops / ms / 1e9, 2),
            "frac_bf16": round(flops / ms / 1e9 / pk["bf16_tflops"], 5)}
    for tokens, label in ((batch, "decode"), (PROMPT_LEN, "prefill")):
        resid = torch.randn(tokens, width, device=dev)
        delta, w = rnd(tokens, width), rnd(width)
        wb = torch.randn(width, device=dev)
        ms = _time_graph(lambda: ops.add_postnorm_rmsnorm(resid, delta, wb, 1e-6, 1.0, w, 1e-6, 1.0,
                                                          torch.bfloat16), reps=20)
        nbytes = tokens * width * (4 + 4 + 2 + 2.0)
        K[f"postnorm_add_norm_{label}"] = {"ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
                                           "frac_hbm": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4)}
    ops.check_error_word(dev)
    print(json.dumps(out))
    return 0


# ------------------------------------------------------------------ a third architecture
def vudivik_sizes(name: str) -> tuple:
    """(Vudivik config, Llama config of equal size) at layer sizes that resemble a real
    model's: every layer a windowed attention with four kept first keys beside a selective
    scan, feed-forwards dense and routed in turn.  The Llama beside it has the same width,
    depth, vocabulary, heads and key/value heads, and a gated feed-forward with as many
    weights as the dense relu-squared one."""
    if name == "small":
        width, depth, vocab = 1024, 8, 32000
        left = dict(heads=8, kv_heads=2, dim=128, vdim=128, scale=128 ** -0.5)
        right = dict(inner=2048, state=16, dt_rank=64, conv=4)
        window, dense, experts, top, ff = 1024, 4096, 16, 2, 1024
    elif name == "medium":
        width, depth, vocab = 2048, 12, 64000
        left = dict(heads=16, kv_heads=4, dim=128, vdim=128, scale=128 ** -0.5)
        right = dict(inner=4096, state=16, dt_rank=128, conv=4)
        window, dense, experts, top, ff = 1024, 8192, 32, 4, 1024
    else:
        raise ValueError(f"unknown size {name!r} (small, medium)")
    left.update(mask={"size": window, "keep_first": 4},
                rot={"base": 1000000.0, "dims": 128,
                     "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}})
    moe = {"kind": "moe", "router": {"experts": experts, "identity": 2, "top": top},
           "expert": {"ff": ff}}
    layers = [{"type": "parallel", "mixer": {"left": dict(left), "right": dict(right)},
               "mlp": moe if i % 2 else {"kind": "dense", "ff": dense}} for i in range(depth)]
    vudivik = {"architecture": "Vudivik", "width": width, "vocab": vocab, "norm": {"eps": 1e-6},
               "residual_mult": 0.5, "layers": layers}
    llama = dict(ORPHEUS_3B, num_hidden_layers=depth, hidden_size=width,
                 num_attention_heads=left["heads"], num_key_value_heads=left["kv_heads"],
                 head_dim=128, intermediate_size=dense * 2 // 3 // 256 * 256, vocab_size=vocab,
                 tie_word_embeddings=False)
    return vudivik, llama


def vudivik_bench(args) -> int:
    """``--arch vudivik``: prefill and decode throughput of the Vudivik decoder (random
    weights, bfloat16) beside the Llama decoder at equal size, through the same step
    function; then its own kernels alone at the sizes of one layer, each beside the like
    kernel of the Llama (attention) or Tifosun (recurrence, experts) decoder where there is
    one, with what each has to move or compute against the measured peaks.  One JSON line."""
    import torch

    from mstar_b200 import ops
    from mstar_b200.parts.base import StepContext

    pk = peaks()
    v_cfg, l_cfg = vudivik_sizes(args.arch_size)
    page, batch = args.page_size, args.batch
    out = {"arch": "Vudivik", "size": args.arch_size, "batch": batch, "prompt_len": PROMPT_LEN,
           "peaks": pk["source"], "models": {}, "kernels": {}}
    _time_models(args, (("vudivik", v_cfg), ("llama", l_cfg)), out)

    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (scale * torch.randn(*shape, generator=g, device=dev)).to(torch.bfloat16)

    def i32(v):
        return torch.tensor(v, dtype=torch.int32, device=dev)

    def record(name, ms, nbytes=None, flops=None, **more):
        row = {"ms": round(ms, 4)}
        if nbytes is not None:
            row["gbs"] = round(nbytes / ms / 1e6, 1)
            row["frac_hbm"] = round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4)
        if flops is not None:
            row["tflops"] = round(flops / ms / 1e9, 2)
            row["frac_bf16"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 5)
        row.update(more)
        out["kernels"][name] = row

    width = v_cfg["width"]
    left, right = v_cfg["layers"][0]["mixer"]["left"], v_cfg["layers"][0]["mixer"]["right"]
    moe = v_cfg["layers"][1]["mlp"]
    H, G, hd = left["heads"], left["kv_heads"], left["dim"]
    window, keep = left["mask"]["size"], left["mask"]["keep_first"]
    ctx_len = PROMPT_LEN
    pages_per = -(-ctx_len // page)
    for tokens, reqs, label in ((batch, batch, "decode"), (PROMPT_LEN, 1, "prefill")):
        per = tokens // reqs
        seen = min(ctx_len, window + keep + per)
        copies = 1 if label == "prefill" else max(1, -(-(160 << 20) // (reqs * seen * G * hd * 4)))
        caches = [rnd(reqs * pages_per + 1, 2, G, page, hd) for _ in range(copies)]
        table = torch.randperm(reqs * pages_per, device=dev).to(torch.int32).view(reqs, pages_per)
        token_req = i32([r for r in range(reqs) for _ in range(per)])
        cache_pos = i32([ctx_len - per + k for _ in range(reqs) for k in range(per)])
        indptr = i32([k * per for k in range(reqs + 1)])
        kv_len = i32([ctx_len] * reqs)
        q = rnd(tokens, H * hd)
        sc = StepContext(num_tokens=tokens, num_entries=reqs, token_req=token_req,
                         positions=cache_pos, cache_pos=cache_pos, qo_indptr=indptr, kv_len=kv_len,
                         slots=i32(list(range(reqs))), q_lens=[per] * reqs, kv_lens=[ctx_len] * reqs,
                         host_slots=list(range(reqs)), max_q_len=per, max_kv_len=ctx_len,
                         num_decode=reqs if per == 1 else 0)
        turn = {"i": 0}

        def attend():
            c = caches[turn["i"] % copies].view(reqs * pages_per + 1, -1)
            turn["i"] += 1
            return ops.sink_attention(q, c, table, token_req, cache_pos, H, G, hd, hd, page, window,
                                      keep, left["scale"], ctx=sc)

        reps = max(copies, 4) if label == "decode" else 2
        ms = _time_graph(attend, reps=reps)
        keys = sum(min(ctx_len - per + k + 1, window + keep) for k in range(per)) * reqs
        record(f"window_attention_{label}", ms, nbytes=reqs * seen * G * hd * 4.0,
               flops=4.0 * H * keys * hd)
        # the Llama decoder's attention on the same cache: every key (no window)
        out_l = torch.empty(tokens, H * hd, dtype=torch.bfloat16, device=dev)
        turn["i"] = 0
        if label == "decode":
            def llama_attend():
                c = caches[turn["i"] % copies]
                turn["i"] += 1
                ops.paged_decode_attention(q, q.stride(0), out_l, c, table, token_req, cache_pos,
                                           tokens, H, G, hd, page, 0, left["scale"], ctx_len)
            all_keys, all_bytes = reqs * ctx_len, reqs * ctx_len * G * hd * 4.0
        else:
            def llama_attend():
                ops.paged_prefill_attention(q, q.stride(0), out_l, caches[0], table, indptr, kv_len,
                                            0, reqs, per, H, G, hd, page, 0, left["scale"])
            all_keys, all_bytes = per * (per + 1) // 2, ctx_len * G * hd * 4.0
        ms = _time_graph(llama_attend, reps=reps)
        record(f"llama_attention_{label}", ms, nbytes=all_bytes, flops=4.0 * H * all_keys * hd)

    inner, N, R, taps = right["inner"], right["state"], right["dt_rank"], right["conv"]
    size = ops.selective_scan_state_size(inner, N, taps)
    copies = max(1, -(-(160 << 20) // (size * 4 * batch)))
    state = torch.zeros(copies * batch + 1, size, device=dev)
    w_dt = torch.randn(inner, R, device=dev) * R ** -0.5
    dt_bias = torch.full((inner,), -3.0, device=dev)
    a_neg = -torch.rand(inner, N, device=dev) * 4 - 0.5
    d_skip = torch.ones(inner, device=dev)
    conv_w, conv_b = rnd(inner, taps), rnd(inner)
    for tokens, entries, label in ((batch, batch, "decode"), (PROMPT_LEN, 1, "prefill")):
        per = tokens // entries
        xz, xc = rnd(tokens, 2 * inner), rnd(tokens, inner)
        proj = torch.randn(tokens, R + 2 * N, device=dev)
        indptr = i32([k * per for k in range(entries + 1)])
        token_req = i32([r for r in range(entries) for _ in range(per)])
        slot_sets = [i32([c * batch + k for k in range(entries)]) for c in range(copies)]
        turn = {"i": 0}

        def scan():
            sl = slot_sets[turn["i"] % copies]
            turn["i"] += 1
            return ops.selective_scan(xc, xz, proj, w_dt, dt_bias, a_neg, d_skip, indptr, sl, state,
                                      entries, inner, N, R, taps, max_q_len=per)

        ms = _time_graph(scan, reps=max(copies, 4) if label == "decode" else 2)
        nbytes = 2.0 * entries * size * 4 + tokens * (inner * 3 * 2 + (R + 2 * N) * 4.0)
        record(f"selective_scan_{label}", ms, nbytes=nbytes,
               tokens_per_chain_us=round(per / (ms * 1e3), 3))
        conv_wt, conv_bf = conv_w.float().t().contiguous(), conv_b.float()
        ms = _time_graph(lambda: ops.conv_silu(xz, conv_w, conv_b, token_req, indptr, slot_sets[0],
                                               state, inner, taps, weight_t=conv_wt,
                                               bias_f32=conv_bf), reps=8)
        record(f"conv_silu_{label}", ms, nbytes=tokens * inner * 4.0)

    E, ident, top, ff = (moe["router"]["experts"], moe["router"]["identity"], moe["router"]["top"],
                         moe["expert"]["ff"])
    copies = max(1, -(-(160 << 20) // (E * 2 * ff * width * 2)))
    w_up = [rnd(E * ff, width, scale=0.02) for _ in range(copies)]
    w_dn = [rnd(E * width, ff, scale=0.02) for _ in range(copies)]
    for tokens, label in ((batch, "decode"), (PROMPT_LEN, "prefill")):
        x = rnd(tokens, width)
        chosen, weight = ops.route_topk(torch.randn(tokens, E + ident, device=dev), top, softmax=True,
                                        choice_bias=torch.zeros(E + ident, device=dev))
        turn = {"i": 0}

        def experts():
            k = turn["i"] % copies
            turn["i"] += 1
            return ops.routed_experts(x, w_up[k], w_dn[k], chosen, weight, E, ff, False, gated=False,
                                      identity=ident)

        ms = _time_graph(experts, reps=max(copies * 2, 4) if label == "decode" else 2)
        picks = [e for e in chosen.flatten().tolist() if e < E]
        record(f"routed_experts_{label}", ms, nbytes=len(set(picks)) * 2.0 * ff * width * 2,
               flops=2.0 * len(picks) * 2 * ff * width, experts_used=len(set(picks)))
    for tokens, label in ((batch, "decode"), (PROMPT_LEN, "prefill")):
        resid = torch.randn(tokens, width, device=dev)
        a, b = rnd(tokens, width), rnd(tokens, width)
        wa, wb = torch.randn(width, device=dev), torch.randn(width, device=dev)
        ms = _time_graph(lambda: ops.mean_of_norms([a, b], [wa, wb], 1e-6), reps=20)
        record(f"mean_of_norms_{label}", ms, nbytes=tokens * width * (2 + 2 + 4.0))
        delta = torch.randn(tokens, width, device=dev)
        ms = _time_graph(lambda: ops.add_postnorm_rmsnorm(resid, delta, wa, 1e-6, 0.0,
                                                          out_dtype=torch.bfloat16, post_scale=0.5,
                                                          plain_out=True), reps=20)
        record(f"postnorm_add_{label}", ms, nbytes=tokens * width * (4 + 4 + 4 + 2.0))
    ops.check_error_word(dev)
    print(json.dumps(out))
    return 0


def relurax_sizes(name: str) -> tuple:
    """(Relurax config, Llama config of equal size) at layer sizes that resemble a real model's: three sliding-window layers (keys
    through a four-tap convolution, values that are the keys, a gate a head) to one latent
    layer with queries through a latent of their own, the second latent layer reading the
    first one's rows; gelu-gated feed-forwards.  The Llama beside it has the same width,
    depth, vocabulary, heads, key/value heads and feed-forward size."""
    if name == "small":
        width, depth, vocab, ff = 1024, 8, 32000, 2816
        att = dict(heads=8, kv_heads=2, dim=128, vdim=128, conv=4, mask={"size": 1024},
                   scale=128 ** -0.5)
        lat = dict(heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=256, q_rank=384,
                   rot={"base": 500000.0, "dims": 32}, scale=96 ** -0.5)
    elif name == "medium":
        width, depth, vocab, ff = 2048, 12, 64000, 5632
        att = dict(heads=16, kv_heads=4, dim=128, vdim=128, conv=4, mask={"size": 1024},
                   scale=128 ** -0.5)
        lat = dict(heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=1024,
                   rot={"base": 500000.0, "dims": 64}, scale=192 ** -0.5)
    else:
        raise ValueError(f"unknown size {name!r} (small, medium)")
    layers, first_latent = [], None
    for i in range(depth):
        if i % 4 == 2:
            m = dict(lat)
            if first_latent is None:
                first_latent = i
            else:
                m["kv_from"] = first_latent
            layers.append({"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff}})
        else:
            layers.append({"type": "attention", "mixer": dict(att), "mlp": {"kind": "dense", "ff": ff}})
    relurax = {"architecture": "Relurax", "width": width, "vocab": vocab, "norm": {"eps": 1e-5},
               "layers": layers}
    llama = dict(ORPHEUS_3B, num_hidden_layers=depth, hidden_size=width,
                 num_attention_heads=att["heads"], num_key_value_heads=att["kv_heads"],
                 head_dim=128, intermediate_size=ff, vocab_size=vocab, tie_word_embeddings=False)
    return relurax, llama


def relurax_bench(args) -> int:
    """``--arch relurax``: prefill and decode throughput of the Relurax decoder (random
    weights, bfloat16) beside the Llama decoder at equal size, through the same step
    function; then the kernels of its two mixers alone at the sizes of one layer, each beside
    the like kernel of the decoder that is closest to it (window attention and its input
    kernel: Vudivik's form of the same kernels and the Llama attention; latent attention:
    Tifosun's windowed form), with what each has to move or compute against the measured
    peaks.  One JSON line."""
    import torch

    from mstar_b200 import ops
    from mstar_b200.parts.base import StepContext

    pk = peaks()
    r_cfg, l_cfg = relurax_sizes(args.arch_size)
    page, batch = args.page_size, args.batch
    out = {"arch": "Relurax", "size": args.arch_size, "batch": batch, "prompt_len": PROMPT_LEN,
           "peaks": pk["source"], "models": {}, "kernels": {}}
    _time_models(args, (("relurax", r_cfg), ("llama", l_cfg)), out)

    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (scale * torch.randn(*shape, generator=g, device=dev)).to(torch.bfloat16)

    def i32(v):
        return torch.tensor(v, dtype=torch.int32, device=dev)

    def record(name, ms, nbytes=None, flops=None, **more):
        row = {"ms": round(ms, 4)}
        if nbytes is not None:
            row["gbs"] = round(nbytes / ms / 1e6, 1)
            row["frac_hbm"] = round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4)
        if flops is not None:
            row["tflops"] = round(flops / ms / 1e9, 2)
            row["frac_bf16"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 5)
        row.update(more)
        out["kernels"][name] = row

    width = r_cfg["width"]
    att = next(l["mixer"] for l in r_cfg["layers"] if l["type"] == "attention")
    lat = next(l["mixer"] for l in r_cfg["layers"] if l["type"] == "latent_attention")
    H, G, hd, taps, window = att["heads"], att["kv_heads"], att["dim"], att["conv"], att["mask"]["size"]
    ctx_len = PROMPT_LEN
    pages_per = -(-ctx_len // page)
    channels = (H + G) * hd
    for tokens, reqs, label in ((batch, batch, "decode"), (PROMPT_LEN, 1, "prefill")):
        per = tokens // reqs
        seen = min(ctx_len, window + per)
        copies = 1 if label == "prefill" else max(1, -(-(160 << 20) // (reqs * seen * G * hd * 4)))
        caches = [rnd(reqs * pages_per + 1, 2, G, page, hd) for _ in range(copies)]
        table = torch.randperm(reqs * pages_per, device=dev).to(torch.int32).view(reqs, pages_per)
        token_req = i32([r for r in range(reqs) for _ in range(per)])
        cache_pos = i32([ctx_len - per + k for _ in range(reqs) for k in range(per)])
        indptr = i32([k * per for k in range(reqs + 1)])
        kv_len = i32([ctx_len] * reqs)
        slots = i32(list(range(reqs)))
        q = rnd(tokens, H * hd)
        sc = StepContext(num_tokens=tokens, num_entries=reqs, token_req=token_req,
                         positions=cache_pos, cache_pos=cache_pos, qo_indptr=indptr, kv_len=kv_len,
                         slots=slots, q_lens=[per] * reqs, kv_lens=[ctx_len] * reqs,
                         host_slots=list(range(reqs)), max_q_len=per, max_kv_len=ctx_len,
                         num_decode=reqs if per == 1 else 0)
        turn = {"i": 0}
        qkv = torch.randn(tokens, channels + H, device=dev)     # the first product: [q | k | gate]

        def attend(keep=0):
            c = caches[turn["i"] % copies].view(reqs * pages_per + 1, -1)
            turn["i"] += 1
            # the Relurax form gates every head where the output is written
            return ops.sink_attention(q, c, table, token_req, cache_pos, H, G, hd, hd, page, window,
                                      keep, att["scale"], ctx=sc,
                                      gate=None if keep else qkv[:, channels:])

        reps = max(copies, 4) if label == "decode" else 2
        keys = sum(min(ctx_len - per + k + 1, window) for k in range(per)) * reqs
        ms = _time_graph(attend, reps=reps)
        record(f"window_attention_{label}", ms, nbytes=reqs * seen * G * hd * 4.0,
               flops=4.0 * H * keys * hd)
        # the same kernel as the Vudivik decoder runs it: four kept first keys beside the window
        ms = _time_graph(lambda: attend(4), reps=reps)
        record(f"vudivik_window_attention_{label}", ms, nbytes=reqs * (seen + 4) * G * hd * 4.0,
               flops=4.0 * H * (keys + 4 * tokens) * hd)
        # what comes before it: convolution over q and k, head norms, cache write (values are
        # the keys before their norm) ...
        state = torch.zeros(reqs, (taps - 1) * channels, device=dev)
        wq, wk = rnd(H * hd, taps), rnd(G * hd, taps)
        nq, nk = rnd(hd), rnd(hd)
        c0 = caches[0].view(reqs * pages_per + 1, -1)
        ms = _time_graph(lambda: ops.sink_prepare(
            qkv, None, nq, nk, None, cache_pos, cache_pos, token_req, table, c0, H, G, hd, hd, 0,
            page, 1e-5, torch.bfloat16, conv=(wq, wk, indptr, slots, state), value_from_key=True),
            reps=8)
        record(f"conv_norm_cache_{label}", ms,
               nbytes=tokens * (channels * 4 + H * hd * 2 + 2 * G * hd * 2.0))
        ms = _time_graph(lambda: ops.conv_state_advance(qkv, channels, taps, indptr, slots, state,
                                                        reqs), reps=8)
        record(f"conv_rows_advance_{label}", ms, nbytes=reqs * (taps - 1) * channels * 8.0)
        # ... beside the Vudivik decoder's form of that kernel: bias, head norms, rotation,
        # separate values
        qkv_v = torch.randn(tokens, (H + 2 * G) * hd, device=dev)
        bias = rnd((H + 2 * G) * hd)
        freq = torch.rand(hd // 2, dtype=torch.float64, device=dev)
        ms = _time_graph(lambda: ops.sink_prepare(
            qkv_v, bias, nq, nk, freq, cache_pos, cache_pos, token_req, table, c0, H, G, hd, hd,
            hd, page, 1e-5, torch.bfloat16), reps=8)
        record(f"vudivik_bias_norm_rope_cache_{label}", ms,
               nbytes=tokens * ((H + 2 * G) * hd * 4 + H * hd * 2 + 2 * G * hd * 2.0))
        # the Llama decoder's attention on the same cache: every key (no window)
        out_l = torch.empty(tokens, H * hd, dtype=torch.bfloat16, device=dev)
        turn["i"] = 0
        if label == "decode":
            def llama_attend():
                c = caches[turn["i"] % copies]
                turn["i"] += 1
                ops.paged_decode_attention(q, q.stride(0), out_l, c, table, token_req, cache_pos,
                                           tokens, H, G, hd, page, 0, att["scale"], ctx_len)
            all_keys, all_bytes = reqs * ctx_len, reqs * ctx_len * G * hd * 4.0
        else:
            def llama_attend():
                ops.paged_prefill_attention(q, q.stride(0), out_l, caches[0], table, indptr, kv_len,
                                            0, reqs, per, H, G, hd, page, 0, att["scale"])
            all_keys, all_bytes = per * (per + 1) // 2, ctx_len * G * hd * 4.0
        ms = _time_graph(llama_attend, reps=reps)
        record(f"llama_attention_{label}", ms, nbytes=all_bytes, flops=4.0 * H * all_keys * hd)

    heads, rank, rot, q_rank = lat["heads"], lat["kv_rank"], lat["rot_dim"], lat["q_rank"]
    dim = lat["dim"]
    for tokens, reqs, label in ((batch, batch, "decode"), (PROMPT_LEN, 1, "prefill")):
        per = tokens // reqs
        copies = 1 if label == "prefill" else max(1, -(-(160 << 20) // (reqs * ctx_len * (rank + rot) * 2)))
        caches = [rnd(reqs * pages_per + 1, 1, 1, page, rank + rot) for _ in range(copies)]
        table = torch.randperm(reqs * pages_per, device=dev).to(torch.int32).view(reqs, pages_per)
        token_req = i32([r for r in range(reqs) for _ in range(per)])
        cache_pos = i32([ctx_len - per + k for _ in range(reqs) for k in range(per)])
        q_abs = torch.randn(tokens, heads, rank, device=dev)
        q_rot = rnd(tokens, heads, rot)
        turn = {"i": 0}

        def latent(win=0):
            c = caches[turn["i"] % copies]
            turn["i"] += 1
            return ops.latent_attention(q_abs, q_rot, c, table, token_req, cache_pos, heads, rank,
                                        rot, page, win, lat["scale"], max_keys=ctx_len,
                                        entries=reqs)

        reps = max(copies, 4) if label == "decode" else 2
        for name, win in (("latent_attention", 0), ("tifosun_latent_attention_window_512", 512)):
            seen = ctx_len if not win else min(ctx_len, win + per)
            keys = sum(min(ctx_len - per + k + 1, win or ctx_len) for k in range(per)) * reqs
            ms = _time_graph(lambda: latent(win), reps=reps)
            record(f"{name}_{label}", ms, nbytes=reqs * seen * (rank + rot) * 2.0,
                   flops=2.0 * heads * keys * (2 * rank + rot))
        # the elementwise work around the products: both latents normed, the shared key part
        # rotated, the cache row written; then the rotation of the queries
        down = torch.randn(tokens, q_rank + rank + rot + heads, device=dev)
        wn, wqn = torch.randn(rank, device=dev), torch.randn(q_rank, device=dev)
        freq = torch.rand(rot // 2, dtype=torch.float64, device=dev)
        fill = dict(positions=cache_pos, cache_pos=cache_pos, token_req=token_req,
                    block_table=table, heads=heads, qk_dim=dim, rot=rot, rot_dims=rot, rank=rank,
                    page_size=page, eps=1e-5, interleaved=False)
        ms = _time_graph(lambda: ops.latent_fill(None, down[:, q_rank:q_rank + rank + rot], wn, freq,
                                                 cache=caches[0], q_latent=down[:, :q_rank],
                                                 q_latent_weight=wqn, **fill), reps=8)
        record(f"latent_norms_rope_cache_{label}", ms,
               nbytes=tokens * ((q_rank + rank + rot) * 4 + (q_rank + rank + rot) * 2.0))
        qs = rnd(tokens, heads * (dim + rot))
        ms = _time_graph(lambda: ops.latent_fill(qs, None, None, freq, cache=caches[0], **fill), reps=8)
        record(f"latent_query_rope_{label}", ms, nbytes=tokens * heads * rot * 4.0)
    ff = r_cfg["layers"][0]["mlp"]["ff"]
    w_gu = rnd(2 * ff, width, scale=0.02)
    for tokens, label in ((batch, "decode"), (PROMPT_LEN, "prefill")):
        x = rnd(tokens, width)
        for kind in ("gelu_tanh", "silu"):
            ms = _time_graph(lambda: ops.gated_up(x, w_gu, static_weights=True, kind=kind), reps=8)
            record(f"gated_up_{kind}_{label}", ms, nbytes=2.0 * ff * width * 2,
                   flops=2.0 * tokens * 2 * ff * width)
        resid = torch.randn(tokens, width, device=dev)
        delta, w = rnd(tokens, width), rnd(width)
        wb = torch.randn(width, device=dev)
        ms = _time_graph(lambda: ops.add_postnorm_rmsnorm(resid, delta, wb, 1e-5, 0.0, w, 1e-5, 0.0,
                                                          torch.bfloat16), reps=20)
        record(f"postnorm_add_norm_{label}", ms, nbytes=tokens * width * (4 + 4 + 2 + 2.0))
    ops.check_error_word(dev)
    print(json.dumps(out))
    return 0


def mokotar_sizes(name: str) -> tuple:
    """(Mokotar config, Vudivik config, Llama config) at layer sizes that resemble a real
    model's: the four layer kinds in turn (an attention with soft cap, temperature and sink; one
    normed over the whole projection with rotary pairs; an attention beside a gated delta
    rule; the first kind again), two copies of the residual, biased gated feed-forwards.  The
    Vudivik beside it, the closest decoder of this engine (an attention of the same kernel
    family beside a recurrent scan in every layer), and the Llama have the same width, depth,
    vocabulary, heads and key/value heads."""
    if name == "small":
        width, depth, vocab, ff = 1024, 8, 32000, 2816
        heads, kv_heads, rank = 8, 2, 64
    elif name == "medium":
        width, depth, vocab, ff = 2048, 12, 64000, 5632
        heads, kv_heads, rank = 16, 4, 128
    else:
        raise ValueError(f"unknown size {name!r} (small, medium)")
    base = dict(heads=heads, kv_heads=kv_heads, dim=128, vdim=128, scale=128 ** -0.5)
    att = dict(base, q_temp={"coef": 0.3, "every": 512}, softcap=30.0)
    att2 = dict(base, rot={"base": 500000.0, "dims": 64})
    par = {"left": dict(base, rot={"base": 500000.0, "dims": 64}),
           "right": dict(heads=heads, kv_heads=heads, dim=128, vdim=128, conv=4, decay_rank=rank,
                         gate_rank=rank),
           "left_scale": 1.0, "right_scale": 1.0}
    kinds = [("attention", att), ("attention_2", att2), ("parallel", par), ("attention", att)]
    layers = [{"type": kinds[i % 4][0], "mixer": json.loads(json.dumps(kinds[i % 4][1])),
               "mlp": {"kind": "dense", "ff": ff}} for i in range(depth)]
    mokotar = {"architecture": "Mokotar", "width": width, "vocab": vocab, "norm": {"eps": 1e-6},
               "residual_mult": 0.5, "streams": 2, "layers": layers}
    vudivik, _ = vudivik_sizes(name)
    llama = dict(ORPHEUS_3B, num_hidden_layers=depth, hidden_size=width,
                 num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=128,
                 intermediate_size=ff, vocab_size=vocab, tie_word_embeddings=False)
    return mokotar, vudivik, llama


def mokotar_bench(args) -> int:
    """``--arch mokotar``: prefill and decode throughput of the Mokotar decoder (random
    weights, bfloat16) beside the Vudivik and Llama decoders at equal size, through the same
    step function; then its kernels alone at the sizes of one layer, each beside the like
    kernel of the closest decoder (attention with sink, soft cap and feature gate: Vudivik's
    window attention and the Llama attention; its input kernel: Vudivik's; the delta rule:
    Vudivik's selective scan and the matrix-memory scan; the hyper-connection kernel: the
    fused post-norm, add and norm), with what each has to move against the measured peaks.
    One JSON line."""
    import torch

    from mstar_b200 import ops
    from mstar_b200.parts.base import StepContext

    pk = peaks()
    m_cfg, v_cfg, l_cfg = mokotar_sizes(args.arch_size)
    page, batch = args.page_size, args.batch
    out = {"arch": "Mokotar", "size": args.arch_size, "batch": batch, "prompt_len": PROMPT_LEN,
           "peaks": pk["source"], "models": {}, "kernels": {}}
    _time_models(args, (("mokotar", m_cfg), ("vudivik", v_cfg), ("llama", l_cfg)), out)

    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (scale * torch.randn(*shape, generator=g, device=dev)).to(torch.bfloat16)

    def i32(v):
        return torch.tensor(v, dtype=torch.int32, device=dev)

    def record(name, ms, nbytes=None, flops=None, **more):
        row = {"ms": round(ms, 4)}
        if nbytes is not None:
            row["gbs"] = round(nbytes / ms / 1e6, 1)
            row["frac_hbm"] = round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4)
        if flops is not None:
            row["tflops"] = round(flops / ms / 1e9, 2)
            row["frac_bf16"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 5)
        row.update(more)
        out["kernels"][name] = row

    width = m_cfg["width"]
    att = m_cfg["layers"][0]["mixer"]
    par = m_cfg["layers"][2]["mixer"]
    H, G, hd = att["heads"], att["kv_heads"], att["dim"]
    ctx_len = PROMPT_LEN
    pages_per = -(-ctx_len // page)
    for tokens, reqs, label in ((batch, batch, "decode"), (PROMPT_LEN, 1, "prefill")):
        per = tokens // reqs
        copies = 1 if label == "prefill" else max(1, -(-(160 << 20) // (reqs * ctx_len * G * hd * 4)))
        caches = [rnd(reqs * pages_per + 1, 2, G, page, hd) for _ in range(copies)]
        table = torch.randperm(reqs * pages_per, device=dev).to(torch.int32).view(reqs, pages_per)
        token_req = i32([r for r in range(reqs) for _ in range(per)])
        cache_pos = i32([ctx_len - per + k for _ in range(reqs) for k in range(per)])
        indptr = i32([k * per for k in range(reqs + 1)])
        kv_len = i32([ctx_len] * reqs)
        slots = i32(list(range(reqs)))
        q = rnd(tokens, H * hd)
        sc = StepContext(num_tokens=tokens, num_entries=reqs, token_req=token_req,
                         positions=cache_pos, cache_pos=cache_pos, qo_indptr=indptr, kv_len=kv_len,
                         slots=slots, q_lens=[per] * reqs, kv_lens=[ctx_len] * reqs,
                         host_slots=list(range(reqs)), max_q_len=per, max_kv_len=ctx_len,
                         num_decode=reqs if per == 1 else 0)
        turn = {"i": 0}
        rows = (H + 2 * G) * hd
        qkv = torch.randn(tokens, rows + H * hd, device=dev)     # [q | k | v | gate]
        sink = torch.randn(H, device=dev)
        keys = sum(ctx_len - per + k + 1 for k in range(per)) * reqs
        all_bytes = reqs * ctx_len * G * hd * 4.0

        def attend(form):
            c = caches[turn["i"] % copies].view(reqs * pages_per + 1, -1)
            turn["i"] += 1
            if form == "mokotar":       # every key, soft cap, sink, a gate a feature
                return ops.sink_attention(q, c, table, token_req, cache_pos, H, G, hd, hd, page, 0,
                                          0, att["scale"], ctx=sc, gate=qkv[:, rows:],
                                          softcap=att["softcap"], sink=sink)
            if form == "plain":         # the same kernel without the three options
                return ops.sink_attention(q, c, table, token_req, cache_pos, H, G, hd, hd, page, 0,
                                          0, att["scale"], ctx=sc)
            return ops.sink_attention(q, c, table, token_req, cache_pos, H, G, hd, hd, page, 1024,
                                      4, att["scale"], ctx=sc)

        reps = max(copies, 4) if label == "decode" else 2
        ms = _time_graph(lambda: attend("mokotar"), reps=reps)
        record(f"sink_attention_{label}", ms, nbytes=all_bytes, flops=4.0 * H * keys * hd)
        ms = _time_graph(lambda: attend("plain"), reps=reps)
        record(f"same_kernel_without_cap_sink_gate_{label}", ms, nbytes=all_bytes,
               flops=4.0 * H * keys * hd)
        seen = min(ctx_len, 1024 + per)
        wkeys = sum(min(ctx_len - per + k + 1, 1024) + 4 for k in range(per)) * reqs
        ms = _time_graph(lambda: attend("vudivik"), reps=reps)
        record(f"vudivik_window_attention_{label}", ms, nbytes=reqs * (seen + 4) * G * hd * 4.0,
               flops=4.0 * H * wkeys * hd)
        out_l = torch.empty(tokens, H * hd, dtype=torch.bfloat16, device=dev)
        turn["i"] = 0
        if label == "decode":
            def llama_attend():
                c = caches[turn["i"] % copies]
                turn["i"] += 1
                ops.paged_decode_attention(q, q.stride(0), out_l, c, table, token_req, cache_pos,
                                           tokens, H, G, hd, page, 0, att["scale"], ctx_len)
        else:
            def llama_attend():
                ops.paged_prefill_attention(q, q.stride(0), out_l, caches[0], table, indptr, kv_len,
                                            0, reqs, per, H, G, hd, page, 0, att["scale"])
        ms = _time_graph(llama_attend, reps=reps)
        record(f"llama_attention_{label}", ms, nbytes=all_bytes, flops=4.0 * H * keys * hd)
        # the input kernels: head norm + temperature; whole-projection norm + rotary pairs;
        # beside Vudivik's bias + head norm + split-half rotation
        c0 = caches[0].view(reqs * pages_per + 1, -1)
        nq, nk = rnd(hd), rnd(hd)
        nqw, nkw = rnd(H * hd), rnd(G * hd)
        freq = torch.rand(32, dtype=torch.float64, device=dev)
        io_bytes = tokens * (rows * 4 + H * hd * 2 + 2 * G * hd * 2.0)
        ms = _time_graph(lambda: ops.sink_prepare(
            qkv, None, nq, nk, None, cache_pos, cache_pos, token_req, table, c0, H, G, hd, hd, 0,
            page, 1e-6, torch.bfloat16, q_temp=(0.3, 512)), reps=8)
        record(f"norm_temperature_cache_{label}", ms, nbytes=io_bytes)
        ms = _time_graph(lambda: ops.sink_prepare(
            qkv, None, nqw, nkw, freq, cache_pos, cache_pos, token_req, table, c0, H, G, hd, hd, 64,
            page, 1e-6, torch.bfloat16, interleaved=True, norm_whole=True), reps=8)
        record(f"whole_norm_rope_pairs_cache_{label}", ms, nbytes=io_bytes)
        bias = rnd(rows)
        freq_v = torch.rand(hd // 2, dtype=torch.float64, device=dev)
        ms = _time_graph(lambda: ops.sink_prepare(
            qkv, bias, nq, nk, freq_v, cache_pos, cache_pos, token_req, table, c0, H, G, hd, hd, hd,
            page, 1e-6, torch.bfloat16), reps=8)
        record(f"vudivik_bias_norm_rope_cache_{label}", ms, nbytes=io_bytes)

        # the gated delta rule of one layer
        r = par["right"]
        DH, DG, D, VD, taps = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
        channels = 2 * DG * D + DH * VD
        size = ops.gated_delta_state_size(DH, DG, D, VD, taps)
        n_state = max(1, -(-(160 << 20) // (reqs * size * 4))) if label == "decode" else 1
        states = [torch.zeros(reqs, size, device=dev) for _ in range(n_state)]
        proj = torch.randn(tokens, channels + DH + 2 * r["decay_rank"], device=dev)
        conv_w = rnd(channels, taps)
        a_proj = torch.randn(tokens, DH * D, device=dev)
        dt_bias, a_exp = torch.randn(DH * D, device=dev) - 4.0, torch.rand(DH, device=dev) + 0.5
        pre = ops.delta_prepare(proj, conv_w, a_proj, dt_bias, a_exp, token_req, indptr, slots,
                                states[0], DH, DG, D, VD, taps, 1e-6)
        ms = _time_graph(lambda: ops.delta_prepare(proj, conv_w, a_proj, dt_bias, a_exp, token_req,
                                                   indptr, slots, states[0], DH, DG, D, VD, taps,
                                                   1e-6), reps=8)
        record(f"delta_conv_unit_decay_{label}", ms,
               nbytes=tokens * ((channels + DH + DH * D) * 4 + (channels + DH + DH * D) * 4.0))
        turn["i"] = 0

        def scan():
            st = states[turn["i"] % n_state]
            turn["i"] += 1
            return ops.delta_scan(*pre, indptr, slots, st, reqs, DH, DG, D, VD, taps, max_q_len=per)

        ms = _time_graph(scan, reps=max(n_state, 4) if label == "decode" else 2)
        record(f"delta_scan_{label}", ms, nbytes=reqs * DH * D * VD * 8.0,
               tokens_per_us=round(per / ms / 1e3, 3))
        o = torch.randn(tokens, DH * VD, device=dev)
        gate, nw = rnd(tokens, DH * VD), torch.randn(VD, device=dev)
        ms = _time_graph(lambda: ops.delta_finish(o, gate, nw, DH, VD, 1e-6, torch.bfloat16), reps=8)
        record(f"delta_head_norm_gate_{label}", ms, nbytes=tokens * DH * VD * 8.0)
        # Vudivik's recurrent branch at its sizes: convolution and scan
        vr = v_cfg["layers"][0]["mixer"]["right"]
        inner, n_st, rank, vt = vr["inner"], vr["state"], vr["dt_rank"], vr["conv"]
        vsize = ops.selective_scan_state_size(inner, n_st, vt)
        vstate = torch.zeros(reqs, vsize, device=dev)
        xz = rnd(tokens, 2 * inner)
        cw, cb = rnd(inner, vt), rnd(inner)
        xc = ops.conv_silu(xz, cw, cb, token_req, indptr, slots, vstate, inner, vt,
                           weight_t=cw.float().t().contiguous(), bias_f32=cb.float())
        ms = _time_graph(lambda: ops.conv_silu(xz, cw, cb, token_req, indptr, slots, vstate, inner,
                                               vt, weight_t=cw.float().t().contiguous(),
                                               bias_f32=cb.float()), reps=8)
        record(f"vudivik_conv_silu_{label}", ms, nbytes=tokens * inner * 4.0)
        vproj = torch.randn(tokens, rank + 2 * n_st, device=dev)
        w_dt, b_dt = torch.randn(inner, rank, device=dev) * 0.1, torch.randn(inner, device=dev) - 4.0
        a_neg, d_skip = -torch.rand(inner, n_st, device=dev) - 0.5, torch.ones(inner, device=dev)
        ms = _time_graph(lambda: ops.selective_scan(xc, xz, vproj, w_dt, b_dt, a_neg, d_skip, indptr,
                                                    slots, vstate, reqs, inner, n_st, rank, vt,
                                                    max_q_len=per), reps=4 if label == "decode" else 2)
        record(f"vudivik_selective_scan_{label}", ms, nbytes=reqs * inner * n_st * 8.0,
               tokens_per_us=round(per / ms / 1e3, 3))

    # between the sublayers: write of the copies, read and norm; beside the fused post-norm,
    # add and norm of the sandwich blocks; the biased gate beside the plain one
    ff = m_cfg["layers"][0]["mlp"]["ff"]
    S = m_cfg["streams"]
    for tokens, label in ((batch, "decode"), (PROMPT_LEN, "prefill")):
        x = torch.randn(tokens, S, width, device=dev)
        y1, y2, w = rnd(tokens, width), rnd(tokens, width), rnd(width)
        mix = torch.eye(S, device=dev).contiguous()
        t_out, t_in = torch.ones(S, device=dev), torch.full((S,), 1.0 / S, device=dev)
        ms = _time_graph(lambda: ops.hyper_step(x, y=y1, y2=y2, mix=mix, out=t_out, read=t_in,
                                                norm_weight=w, eps=1e-6, out_dtype=torch.bfloat16),
                         reps=20)
        record(f"hyper_write_read_norm_{label}", ms, nbytes=tokens * width * (8.0 * S + 2 + 2 + 2))
        resid = torch.randn(tokens, width, device=dev)
        wb = torch.randn(width, device=dev)
        ms = _time_graph(lambda: ops.add_postnorm_rmsnorm(resid, y1, wb, 1e-5, 0.0, w, 1e-5, 0.0,
                                                          torch.bfloat16), reps=20)
        record(f"postnorm_add_norm_{label}", ms, nbytes=tokens * width * (4 + 4 + 2 + 2.0))
        gu = torch.randn(tokens, 2 * ff, device=dev)
        bias = rnd(2 * ff)
        ms = _time_graph(lambda: ops.bias_act_mul(gu, bias, torch.bfloat16), reps=20)
        record(f"bias_silu_mul_{label}", ms, nbytes=tokens * ff * (8.0 + 2))
        gub = rnd(tokens, 2 * ff)
        ms = _time_graph(lambda: ops.silu_mul(gub), reps=20)
        record(f"silu_mul_{label}", ms, nbytes=tokens * ff * (4.0 + 2))
    ops.check_error_word(dev)
    print(json.dumps(out))
    return 0


# --------------------------------------------------------------- single kernels
def _time_graph(fn, reps: int = 20, rounds: int = 5) -> float:
    """Median milliseconds of one call of ``fn`` when ``reps`` calls are replayed as one
    CUDA graph (so that launch gaps are what they are inside a captured step)."""
    import torch

    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    # MSTAR_BENCH_WARM_MS=N replays for N ms first: short kernels then see the clocks of a busy
    # GPU (a little faster), long ones its power cap (8,192-token attention 0.41 instead of
    # 0.37 ms); the figures in profiles/ are taken without, like the burst peak they are
    # compared with
    warm = float(os.environ.get("MSTAR_BENCH_WARM_MS", "0"))
    t0 = time.perf_counter()
    while (time.perf_counter() - t0) * 1e3 < warm:
        for _ in range(10):
            graph.replay()
        torch.cuda.synchronize()
    times = []
    for _ in range(rounds):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / reps)
    return statistics.median(times)


def kernel_bench(name: str, batch: int, ctx: int, small: bool, cfg: dict) -> int:
    """Time one kernel alone at the benchmark model's shapes: ``--kernel NAME``.  Inputs
    rotate over copies larger than L2 where the kernel is memory-bound.  ``--small``
    shrinks the case for profiler captures (still larger than L2 where it matters)."""
    import torch

    from mstar_b200 import ops

    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    dev = "cuda:0"
    pk = peaks()
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (scale * torch.randn(*shape, generator=g, device=dev)).to(torch.bfloat16)

    out = {"kernel": name, "batch": batch, "ctx": ctx}
    if name in ("decode_attention", "prefill_attention"):
        page = PAGE_SIZE
        reqs = batch
        pages_per = -(-ctx // page)
        kv = rnd(reqs * pages_per + 1, 2, nkv, page, hd)
        table = torch.randperm(reqs * pages_per, device=dev).to(torch.int32).view(reqs, pages_per)
        if name == "decode_attention":
            q = rnd(reqs, (nq + 2 * nkv) * hd)
            o = torch.empty(reqs, nq * hd, dtype=torch.bfloat16, device=dev)
            token_req = torch.arange(reqs, dtype=torch.int32, device=dev)
            cache_pos = torch.full((reqs,), ctx - 1, dtype=torch.int32, device=dev)
            fn = lambda: ops.paged_decode_attention(q, q.stride(0), o, kv, table, token_req,
                                                    cache_pos, reqs, nq, nkv, hd, page, 0,
                                                    hd ** -0.5, ctx)
            ms = _time_graph(fn)
            nbytes = reqs * ctx * 2 * nkv * hd * 2
            out.update(ms=ms, gbs=nbytes / ms / 1e6, frac_hbm=nbytes / ms / 1e6 / pk["hbm_gbs"],
                       split=ops.decode_split(reqs, nkv, ctx, ring=os.environ.get("MSTAR_DECODE_ATTENTION") != "per_item"))
        else:
            q = rnd(reqs * ctx, (nq + 2 * nkv) * hd)
            o = torch.empty(reqs * ctx, nq * hd, dtype=torch.bfloat16, device=dev)
            indptr = torch.arange(0, (reqs + 1) * ctx, ctx, dtype=torch.int32, device=dev)
            kvl = torch.full((reqs,), ctx, dtype=torch.int32, device=dev)
            fn = lambda: ops.paged_prefill_attention(q, q.stride(0), o, kv, table, indptr, kvl, 0,
                                                     reqs, ctx, nq, nkv, hd, page, 0, hd ** -0.5)
            ms = _time_graph(fn, reps=5)
            flops = reqs * 4.0 * nq * hd * ctx * (ctx + 1) / 2
            out.update(ms=ms, tflops=flops / ms / 1e9,
                       frac_bf16=flops / ms / 1e9 / pk["bf16_tflops"])
    elif name in ("gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down", "gemm_lm_head"):
        n, k = {"gemm_qkv": ((nq + 2 * nkv) * hd, H), "gemm_o": (H, nq * hd),
                "gemm_gate_up": (2 * I, H), "gemm_down": (H, I), "gemm_lm_head": (V, H)}[name]
        if small and name == "gemm_lm_head":
            n = 65536
        copies = max(1, -(-(160 << 20) // (n * k * 2)))          # rotate over > L2 bytes
        ws = [rnd(n, k, scale=0.02) for _ in range(copies)]
        x = rnd(batch, k)
        state = {"i": 0}

        def fn():
            w = ws[state["i"] % copies]
            state["i"] += 1
            if name == "gemm_gate_up":
                return ops.gated_up(x, w)
            return ops.linear(x, w, out_dtype=torch.float32 if name == "gemm_lm_head" else None)

        ms = _time_graph(fn, reps=max(copies * 2, 8))
        nbytes = n * k * 2
        flops = 2.0 * batch * n * k
        out.update(ms=ms, n=n, k=k, gbs=nbytes / ms / 1e6,
                   frac_hbm=nbytes / ms / 1e6 / pk["hbm_gbs"], tflops=flops / ms / 1e9)
    elif name == "qkv_rope":
        # the decode form of the mixer's first product: product, rotation and cache write
        n, k = (nq + 2 * nkv) * hd, H
        copies = max(1, -(-(160 << 20) // (n * k * 2)))
        ws = [rnd(n, k, scale=0.02) for _ in range(copies)]
        x = rnd(batch, k)
        pages_per = -(-ctx // PAGE_SIZE)
        kv = rnd(batch * pages_per + 1, 2, nkv, PAGE_SIZE, hd)
        table = torch.arange(batch * pages_per, dtype=torch.int32, device=dev).view(batch, -1)
        pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device=dev)
        req = torch.arange(batch, dtype=torch.int32, device=dev)
        inv = torch.rand(hd // 2, device=dev)
        state = {"i": 0}

        def fn():
            w = ws[state["i"] % copies]
            state["i"] += 1
            return ops.qkv_rope_write(x, w, pos, pos, req, table, inv, kv, nq, nkv, hd, PAGE_SIZE,
                                      static_weights=True)

        ms = _time_graph(fn, reps=max(copies * 2, 8))
        out.update(ms=ms, n=n, k=k, gbs=n * k * 2 / ms / 1e6,
                   frac_hbm=n * k * 2 / ms / 1e6 / pk["hbm_gbs"])
    elif name in ("add_rmsnorm", "rope_kv_write"):
        rows = batch
        if name == "add_rmsnorm":
            resid = torch.randn(rows, H, device=dev)
            delta = rnd(rows, H)
            w = rnd(H)
            fn = lambda: ops.add_rmsnorm(resid, delta, w, 1e-5, torch.bfloat16)
        else:
            qkv = rnd(rows, (nq + 2 * nkv) * hd)
            pos = torch.full((rows,), ctx - 1, dtype=torch.int32, device=dev)
            req = torch.arange(rows, dtype=torch.int32, device=dev)
            kv = rnd(rows * (-(-ctx // PAGE_SIZE)) + 1, 2, nkv, PAGE_SIZE, hd)
            table = torch.arange(rows * (-(-ctx // PAGE_SIZE)), dtype=torch.int32,
                                 device=dev).view(rows, -1)
            inv = torch.rand(hd // 2, device=dev)
            fn = lambda: ops.rope_kv_write(qkv, pos, pos, req, table, inv, kv, nq, nkv, hd, hd,
                                           False, PAGE_SIZE)
        out.update(ms=_time_graph(fn, reps=50))
    elif name in ("matrix_memory_scan", "latent_attention"):
        # kernels of the Tifosun decoder at its medium layer sizes: --batch sequences of --ctx
        # new tokens each (the scan), or --batch requests whose last --ctx tokens attend over a
        # cache of max(--ctx, 2,048) rows (the attention); --ctx 1 is a decode step
        t_cfg, _ = tifosun_sizes("small" if small else "medium")
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        per = ctx
        if name == "matrix_memory_scan":
            m = next(l["mixer"] for l in t_cfg["layers"] if l["type"] == "mlstm")
            Hm, dim, vdim = m["heads"], m["dim"], m["vdim"]
            size = ops.matrix_memory_state_size(Hm, dim, vdim)
            state = torch.zeros(batch + 1, size, device=dev)
            proj = rnd(batch * per, 2 * Hm * dim + 2 * Hm * vdim)
            gates = torch.randn(batch * per, 2 * Hm, device=dev)
            bias = torch.zeros(2 * Hm, device=dev)
            indptr, slots = i32([k * per for k in range(batch + 1)]), i32(list(range(batch)))
            fn = lambda: ops.matrix_memory_scan(proj, gates, bias, indptr, slots, state, batch, Hm,
                                                dim, vdim, 15.0, dim ** -0.5, 1e-6)
            ms = _time_graph(fn, reps=4)
            out.update(ms=ms, heads=Hm, dim=dim, vdim=vdim, tokens_per_us_per_chain=per / ms / 1e3,
                       state_gbs=2.0 * batch * size * 4 / ms / 1e6)
        else:
            m = next(l["mixer"] for l in t_cfg["layers"] if l["type"] == "latent_attention")
            heads, rank, rot, window = m["heads"], m["kv_rank"], m["rot_dim"], m["mask"]["size"]
            length = max(ctx, PROMPT_LEN)
            pages_per = -(-length // PAGE_SIZE)
            cache = rnd(batch * pages_per + 1, 1, 1, PAGE_SIZE, rank + rot)
            table = torch.randperm(batch * pages_per, device=dev).to(torch.int32).view(batch, -1)
            token_req = i32([r for r in range(batch) for _ in range(per)])
            cache_pos = i32([length - per + k for _ in range(batch) for k in range(per)])
            q_abs = torch.randn(batch * per, heads, rank, device=dev)
            q_rot = rnd(batch * per, heads, rot)
            fn = lambda: ops.latent_attention(q_abs, q_rot, cache, table, token_req, cache_pos, heads,
                                              rank, rot, PAGE_SIZE, window, m["scale"],
                                              max_keys=length, entries=batch)
            ms = _time_graph(fn, reps=4)
            keys = sum(min(length - per + k + 1, window) for k in range(per)) * batch
            flops = 2.0 * heads * keys * (2 * rank + rot)
            out.update(ms=ms, heads=heads, rank=rank, rot=rot, window=window,
                       tflops=flops / ms / 1e9, frac_bf16=flops / ms / 1e9 / pk["bf16_tflops"])
    else:
        print(f"unknown kernel {name!r}")
        return 2
    out["peaks"] = pk["source"]
    print(json.dumps(out))
    return 0


def reference_arm(args) -> int:
    """The reference's own engine on the same workload, in a process of its own that
    imports nothing of this package (baseline/run_reference.py); its JSON line is passed
    on.  If that process dies without a line, the reason is printed as ``unavailable``."""
    cmd = [sys.executable, str(ROOT / "baseline" / "run_reference.py"), "--steps", str(args.steps),
           "--warmup", str(args.warmup), "--rounds", str(args.rounds), "--batch", str(args.batch),
           "--page-size", str(args.page_size)]
    if args.layers:
        cmd += ["--layers", str(args.layers)]
    try:
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, text=True, timeout=3000)
        lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
        if lines:
            print(lines[-1])
            return 0
        why = f"baseline/run_reference.py exited with {proc.returncode} and printed no record"
    except subprocess.TimeoutExpired:
        why = "baseline/run_reference.py did not finish within 3000 s"
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main() -> int:
    global PAGE_SIZE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--rounds", type=int, default=5,
                    help="rounds of --steps timed steps; the median round is reported")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per cache page")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the model has (named in the record)")
    ap.add_argument("--workloads", default="all", choices=["all", "none", *sorted(WORKLOADS)],
                    help="serving workloads through the entry point, reported under points")
    ap.add_argument("--kernel", default=None,
                    help="time one kernel alone (decode_attention, prefill_attention, gemm_qkv, "
                         "gemm_o, gemm_gate_up, gemm_down, gemm_lm_head, qkv_rope, add_rmsnorm, "
                         "rope_kv_write, matrix_memory_scan, latent_attention) at --batch rows / "
                         "requests and --ctx keys")
    ap.add_argument("--ctx", type=int, default=PROMPT_LEN)
    ap.add_argument("--small", action="store_true", help="a smaller case, for profiler captures")
    ap.add_argument("--sizes", default="orpheus-3b", choices=sorted(SIZES),
                    help="layer sizes; the default is the benchmark model")
    ap.add_argument("--arch", default=None, choices=["tifosun", "vudivik", "relurax", "mokotar"],
                    help="measure another architecture beside the Llama decoder at equal size "
                         "(prefill, decode, its own kernels) instead of the headline workload")
    ap.add_argument("--arch-size", default="small", choices=["small", "medium"])
    args = ap.parse_args()
    model_name, sizes = SIZES[args.sizes]
    PAGE_SIZE = page = args.page_size
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported")
        return 2
    if args.arch:
        return arch_bench(args)
    if args.kernel:
        return kernel_bench(args.kernel, args.batch, args.ctx, args.small, sizes)
    if args.impl == "reference":
        return reference_arm(args)
    warmup = max(args.warmup, 3)
    rounds = max(args.rounds, 1)

    import torch

    from mstar_b200.engine.step import make_stepper
    from mstar_b200.ops import lib

    cfg = dict(sizes)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    print("[bench] building the random-weight model ...", file=sys.stderr, flush=True)
    model = build_model(cfg)
    max_batch = max(64, args.batch)
    pages = max_batch * (CONTEXT // page) + 64
    stepper = make_stepper(model, page_size=page, num_pages=pages, num_slots=max_batch + 4)

    print("[bench] prefill ...", file=sys.stderr, flush=True)
    pre = time_prefill(stepper, cfg)
    print("[bench] decode ...", file=sys.stderr, flush=True)
    with ClockSampler() as clocks:
        head = time_decode(stepper, args.batch, cfg, args.steps, warmup, rounds)
    # the same steps through the entry point, directly after the device-timed ones (the
    # long batch-64 run below leaves the GPU under its power cap)
    print("[bench] end to end ...", file=sys.stderr, flush=True)
    e2e = time_e2e(model, args.batch, cfg, args.steps, warmup,
                   args.batch * (CONTEXT // page) + 64, page, rounds)
    print("[bench] decode at batch 1 and 64 ...", file=sys.stderr, flush=True)
    points = {}
    for b in (1, 64):
        r = time_decode(stepper, b, cfg, max(args.steps // 2, 8), warmup, min(rounds, 3))
        points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
    del stepper
    torch.cuda.empty_cache()
    other = 64 if page != 64 else 16
    print(f"[bench] decode with pages of {other} ...", file=sys.stderr, flush=True)
    stepper = make_stepper(model, page_size=other,
                           num_pages=args.batch * (CONTEXT // other) + 64,
                           num_slots=args.batch + 4)
    r = time_decode(stepper, args.batch, cfg, args.steps, warmup, min(rounds, 3))
    points[f"decode_b{args.batch}_page{other}"] = round(r["tokens_per_s"], 1)
    del stepper
    torch.cuda.empty_cache()

    step_bytes = bytes_of_decode_step(cfg, model, head["kv_lens"])
    achieved = step_bytes / (head["ms_per_step"] / 1e3) / 1e9
    parameter_gb = model.parameter_bytes() / 1e9
    del model
    torch.cuda.empty_cache()
    chosen = sorted(WORKLOADS) if args.workloads == "all" else (
        [] if args.workloads == "none" else [args.workloads])
    for name in chosen:
        w = run_workload(name, page)
        tag = f"{name}_{WORKLOADS[name]['sizes'].replace('-', '')}"
        points[f"{tag}_tok_s"] = round(w["tokens_per_s"], 1)
        points[f"{tag}_ttft_ms"] = round(w["ttft_ms_median"], 1)
        points[f"{tag}_seconds"] = round(w["seconds"], 3)
        points[f"{tag}_runs_agree"] = 1.0 if w["runs_agree"] else 0.0
        print(f"[bench] {name}: {json.dumps(w)}", file=sys.stderr, flush=True)

    record = {
        "metric": f"decode tok/s at batch {args.batch} ({model_name.split(' / ')[0]} bf16, "
                  "2,048-token cached prompts)",
        "value": round(head["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(head["ms_per_step"], 4),
        "rounds": rounds, "ms_per_step_min": round(head["ms_min"], 4),
        "ms_per_step_max": round(head["ms_max"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random-init weights N(0, 0.02)",
        "config": {
            "model": model_name, "global_batch": args.batch,
            "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "parallelism": "single GPU",
            "layers": cfg["num_hidden_layers"], "layers_of_model": full_layers,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "tied_embeddings": cfg["tie_word_embeddings"],
            "rope": f"theta 5e5, llama3 x{cfg['rope_scaling']['factor']:g} (1, 4, 8192)",
            "rms_eps": cfg["rms_norm_eps"], "page_size": page,
            "l2": f"inputs larger than L2 (weights {parameter_gb:.1f} GB per step)",
            "peaks": pk["source"]},
        "e2e": {"value": round(e2e["tokens_per_s"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                "d2h_bytes_per_step": e2e["d2h_bytes_per_step"],
                "ms_per_step": round(e2e["ms_per_step"], 4),
                "ms_per_step_min": round(e2e["ms_min"], 4),
                "ms_per_step_max": round(e2e["ms_max"], 4)},
        "gpu_launches": head["launches"],
        "clocks": clocks.summary(),
        "prefill": {"value": round(pre["tokens_per_s"], 1), "tokens": PROMPT_LEN,
                    "ms": round(pre["ms"], 3),
                    "frac": round(pre["flops"] / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "libraries": sorted(lib.loaded_libraries()),
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
