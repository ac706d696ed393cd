#!/usr/bin/env python3
"""Headline benchmark: decode tokens per second of the Llama-3-8B-sized model
(random weights, bfloat16) on one B200, plus prefill of 2,048 tokens and decode at
batch 1 and 64, and the two workloads of the larger configurations: continuous batching
of 128 requests at Llama-3.2-3B sizes, and 8 prompts of 30,000 tokens at Llama-3.1-8B sizes.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step of the whole batch.  Prints ONE JSON line.  The
decode steps are timed on the device with CUDA events; every request holds a
2,048-token prompt in the cache (put there by the engine's own prefill steps,
outside the timed region) and grows by one token per step.  A decode step reads
every weight once (15 GB, far beyond the 126 MB L2), so consecutive steps do not
reuse cached inputs.  ``e2e`` is the same workload through ``Engine.generate``
with host token ids in and out.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_LEN = 2048
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)) and d[k] > 0:
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [int(r[0]) for r in self.rows if r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=reasons, samples=len(sm))


def model_numbers(cfg, n_layers):
    """Bytes of weights one decode step reads, cache bytes per token, flops per token."""
    d, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_layer = d * (q + 2 * kv) + q * d + 2 * I * d + I * d + 2 * d
    weights = n_layers * per_layer + V * d + d                  # the head once; embedding rows are negligible
    return dict(weight_bytes=2 * weights, kv_bytes_per_token=n_layers * 2 * kv * 2,
                gemm_flops_per_token=2 * n_layers * (per_layer - 2 * d), head_flops_per_row=2 * V * d,
                attn_flops_per_pair=4 * n_layers * q)


def build_engine(layers, name="llama-3-8b"):
    import dataclasses
    import torch
    from batchspec_b200.config import get_config
    from batchspec_b200.engine import Engine
    cfg = get_config(name)
    full_layers = cfg.num_hidden_layers
    if layers and layers != full_layers:
        cfg = dataclasses.replace(cfg, num_hidden_layers=layers)
    eng = Engine(dtype="bfloat16", device="cuda:0")
    eng.load_model(config=cfg, random_seed=0, draw_on_device=True)
    eng.setup_sampling_params(temperature=0.0)
    return eng, cfg, full_layers


def prompts_for(batch, vocab, seed):
    import random
    rng = random.Random(seed)
    return [[rng.randrange(vocab) for _ in range(PROMPT_LEN)] for _ in range(batch)]


def run_decode(eng, cfg, batch, steps, warmup, page_size=16):
    """Device-timed decode: prefill the prompts through the engine, then
    ``warmup`` + ``steps`` decode steps; returns (ms per step, launches)."""
    import torch
    from batchspec_b200.engine import StepEntry
    from batchspec_b200.kernels import ops
    max_len = PROMPT_LEN + warmup + steps + 1
    eng.setup_caches(max_batch_size=batch, max_seq_length=max_len, page_size=page_size)
    prompts = prompts_for(batch, cfg.vocab_size, 1)
    last = []
    for i, p in enumerate(prompts):
        eng.admit(i)
        logits = eng.step([StepEntry(i, p, want=(len(p) - 1,))])
        last.append(int(ops.argmax(logits).cpu()[0]))
    session = eng.decode_session(list(range(batch)), last)
    for _ in range(warmup):
        session.step()
    torch.cuda.synchronize()
    l0 = session.launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        session.step()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launches = session.launches - l0
    session.close()
    for i in range(batch):
        eng.release(i)
    return ms, launches


def run_prefill(eng, cfg, warmup=2, iters=3, page_size=16):
    import torch
    from batchspec_b200.engine import StepEntry
    eng.setup_caches(max_batch_size=1, max_seq_length=PROMPT_LEN + 16, page_size=page_size)
    p = prompts_for(1, cfg.vocab_size, 2)[0]
    times = []
    for it in range(warmup + iters):
        eng.admit("p")
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        eng.step([StepEntry("p", p, want=(PROMPT_LEN - 1,))])
        e.record()
        torch.cuda.synchronize()
        eng.release("p")
        if it >= warmup:
            times.append(s.elapsed_time(e))
    return statistics.median(times)


def pct(values, q):
    v = sorted(values)
    return v[min(len(v) - 1, int(q * len(v)))] if v else None


E2E_WARMUP_STEPS = 32


def run_e2e(eng, cfg, batch, steps, warmup, page_size=16):
    """The same decode workload through Engine.generate: host token ids in, host token ids out.  Every request
    generates ``warm + steps + 1`` tokens; the value is decode tokens per second over the LAST ``steps`` decode
    steps (wall clock of each step, its host->device metadata copy and device->host token read included).  The
    first ``warm`` = max(warmup, 32) decode steps are warm-up, as in the device-timed region: for about 100 ms
    after the prompt step (a quarter of a second of tensor-core work under the power cap) the SM clock stays near
    1.4 GHz before it returns to 1.9 GHz, and a decode step takes 4.9 ms instead of 4.0 ms meanwhile (clock trace
    by NVML); ``value_from_first_step`` includes those steps."""
    from batchspec_b200.engine import Sequence
    warm = max(warmup, E2E_WARMUP_STEPS)
    # token budget of one step = all prompts, so the requests prefill together and then decode in lockstep
    eng.setup_caches(max_batch_size=batch, max_seq_length=PROMPT_LEN + warm + steps + 2, page_size=page_size,
                     prefill_chunk_size=PROMPT_LEN, max_tokens_per_step=batch * PROMPT_LEN)
    eng.ignore_eos = True
    prompts = prompts_for(batch, cfg.vocab_size, 3)
    # before that: the same call on the same prompts, a few tokens (loads kernels, captures the decode graph)
    eng.generate([Sequence(i, p, max_new_tokens=4) for i, p in enumerate(prompts)])
    eng.time_decode_on_device = True
    eng.generate([Sequence(i, p, max_new_tokens=warm + steps + 1) for i, p in enumerate(prompts)])
    eng.time_decode_on_device = False
    st = eng.last_stats
    ms = st["decode_step_ms"]
    assert len(ms) == warm + steps, (len(ms), warm, steps)
    timed = ms[warm:]
    # the same steps by CUDA events around each of them: what the GPU took for them at the clock it had then
    # (the clock moves between 1.3 and 1.9 GHz under the power cap and the step follows it), so that what the
    # host adds can be told from what the clock did between this region and the device-timed one
    on_device = st["decode_step_device_ms"][warm:]
    return dict(value=round(batch * steps / (sum(timed) * 1e-3), 2), unit="tok/s",
                same_steps_on_device_ms=round(sum(on_device) / len(on_device), 3),
                of_same_steps_on_device=round(sum(on_device) / sum(timed), 4),
                h2d_bytes_per_step=st["decode_h2d_bytes_per_step"], d2h_bytes_per_step=st["decode_d2h_bytes_per_step"],
                decode_steps=steps, warmup_steps=warm, step_p50_ms=round(pct(timed, 0.5), 3),
                step_mean_ms=round(sum(timed) / len(timed), 3), step_max_ms=round(max(timed), 3),
                first_step_ms=round(ms[0], 3), value_from_first_step=round(batch * len(ms) / (sum(ms) * 1e-3), 2))


def run_cfg4(pk):
    """Continuous batching at Llama-3.2-3B sizes: 128 seeded requests, prompts of 64..4096 tokens, 16..1024 new
    tokens each, sampled (temperature 0.6, top-k 20, top-p 0.95), at most 64 at a time, prompts in portions of 512
    tokens beside the decoding requests, through ``Engine.generate``."""
    import random
    import torch
    from batchspec_b200.engine import Sequence
    eng, cfg, full_layers = build_engine(0, "llama-3.2-3b")
    eng.setup_caches(max_batch_size=64, max_seq_length=4096 + 1024 + 1, page_size=16, prefill_chunk_size=512,
                     max_tokens_per_step=4096)
    eng.setup_sampling_params(temperature=0.6, top_k=20, top_p=0.95, seed=4)
    eng.ignore_eos = True
    rng = random.Random(44)

    def workload(n):
        return [Sequence(i, [rng.randrange(cfg.vocab_size) for _ in range(rng.randint(64, 4096))],
                         max_new_tokens=rng.randint(16, 1024)) for i in range(n)]
    eng.generate(workload(8)[:8])                      # warm-up: kernels and the first graphs
    seqs = workload(128)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    eng.generate(seqs)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = eng.last_stats
    out = {"cfg4_tok_s": round(st["generated"] / dt, 1), "cfg4_processed_tok_s": round((st["generated"] + st["tokens_fed"]) / dt, 1),
           "cfg4_seconds": round(dt, 3), "cfg4_steps": st["steps"], "cfg4_step_p50_ms": round(pct(st["step_ms"], 0.5), 3),
           "cfg4_step_p90_ms": round(pct(st["step_ms"], 0.9), 3), "cfg4_step_p99_ms": round(pct(st["step_ms"], 0.99), 3),
           "cfg4_pages_high_water": st["pages_high_water"][0], "cfg4_pages": eng.cache.groups[0].pool.num_pages,
           "cfg4_preemptions": st["preemptions"], "cfg4_layers": cfg.num_hidden_layers}
    del eng
    torch.cuda.empty_cache()
    return out


def run_cfg5(pk):
    """Long context at Llama-3.1-8B sizes: 8 prompts of 30,000 tokens in portions of 4,096, then 256 decode steps,
    through ``Engine.generate``.  Reports the prompt phase as a fraction of the tensor-core peak and the decode
    step against the time its bytes (weights once, 8 caches) take at the measured memory rate."""
    import torch
    from batchspec_b200.engine import Sequence
    eng, cfg, full_layers = build_engine(0, "llama-3.1-8b")
    nums = model_numbers(cfg, cfg.num_hidden_layers)
    B, T, NEW, CHUNK = 8, 30000, 257, 4096
    eng.setup_caches(max_batch_size=B, max_seq_length=T + NEW + 1, page_size=16, prefill_chunk_size=CHUNK,
                     max_tokens_per_step=CHUNK)
    eng.ignore_eos = True
    prompts = [[(7919 * i + 104729 * j) % cfg.vocab_size for j in range(T)] for i in range(B)]
    eng.generate([Sequence(0, prompts[0][:CHUNK + 7], max_new_tokens=4)])          # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    eng.generate([Sequence(i, p, max_new_tokens=NEW) for i, p in enumerate(prompts)])
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = eng.last_stats
    dec = st["decode_step_ms"]
    tail = dec[len(dec) // 4:]                               # the steps after the last prompt has joined
    prompt_ms = sum(st["step_ms"]) - sum(dec)
    flops = B * (T * nums["gemm_flops_per_token"] + nums["attn_flops_per_pair"] * T * (T + 1) / 2)
    step_bytes = nums["weight_bytes"] + B * (T + NEW / 2) * nums["kv_bytes_per_token"]
    p50 = pct(tail, 0.5)
    out = {"cfg5_seconds": round(dt, 3), "cfg5_prefill_tok_s": round(B * T / (prompt_ms * 1e-3), 1),
           "cfg5_prefill_tflops": round(flops / (prompt_ms * 1e-3) / 1e12, 1),
           "cfg5_prefill_frac": round(flops / (prompt_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
           "cfg5_decode_p50_ms": round(p50, 3), "cfg5_decode_steps": len(dec),
           "cfg5_decode_floor_ms": round(step_bytes / (pk["hbm_gbs"] * 1e9) * 1e3, 3),
           "cfg5_decode_frac": round(step_bytes / (p50 * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
           "cfg5_pages_per_request": -(-(T + NEW) // 16), "cfg5_layers": cfg.num_hidden_layers}
    del eng
    torch.cuda.empty_cache()
    return out


# ---- a second design beside the headline model (``--design vabanex``); the default workload does not run this

VABANEX_SIZES = {
    # width, heads, unrotated / rotated / value size per head, ranks, experts (count, chosen, ff, groups, kept), dense ff
    "w2048": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, q_rank=768, kv_rank=512,
                  experts=64, top=6, expert_ff=1408, groups=8, keep=4, dense_ff=8448, kv_heads=4),
    "w4096": dict(width=4096, heads=32, dim=128, rot=64, vdim=128, q_rank=1536, kv_rank=512,
                  experts=64, top=8, expert_ff=2048, groups=8, keep=4, dense_ff=14336, kv_heads=8),
}


def vabanex_config_json(z, layers, vocab=32000):
    mixer = dict(heads=z["heads"], dim=z["dim"], rot_dim=z["rot"], vdim=z["vdim"], q_rank=z["q_rank"],
                 kv_rank=z["kv_rank"], scale=(z["dim"] + z["rot"]) ** -0.5,
                 rot=dict(base=10000.0, dims=z["rot"], scaling=dict(factor=40.0, original=4096, fast=32.0, slow=1.0)))
    moe = dict(kind="moe", expert=dict(ff=z["expert_ff"]),
               router=dict(experts=z["experts"], top=z["top"], scale=2.5, groups=dict(count=z["groups"], keep=z["keep"])))
    dense = dict(kind="dense", ff=z["dense_ff"], limit=7.0)
    return dict(architecture="Vabanex", vocab=vocab, width=z["width"], embedding=dict(scale=1.0), norm=dict(eps=1e-5),
                logit_softcap=50.0,
                layers=[dict(type="latent_attention", mixer=mixer, mlp=dense if i == 0 else moe) for i in range(layers)])


def llama_config_json(z, layers, vocab=32000):
    """The closest existing model at equal size: same width, depth, heads and vocabulary; its feed-forward has the
    width of the first layer's dense one."""
    return dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", vocab_size=vocab,
                hidden_size=z["width"], num_hidden_layers=layers, num_attention_heads=z["heads"],
                num_key_value_heads=z["kv_heads"], head_dim=128, intermediate_size=z["dense_ff"], rms_norm_eps=1e-5,
                rope_theta=500000.0, rope_scaling=None, max_position_embeddings=131072, tie_word_embeddings=False)


def run_buckets(eng, cfg, n_tokens, page_size=16):
    """Device time of every part of one prompt step of ``n_tokens`` (CUDA events around each part's launches)."""
    import torch
    from batchspec_b200.engine import StepEntry
    from batchspec_b200.profiler import Profiler, register_active_profiler, release_active_profiler
    eng.setup_caches(max_batch_size=1, max_seq_length=n_tokens + 16, page_size=page_size)
    p = prompts_for(1, cfg.vocab_size, 2)[0][:n_tokens]
    prof = Profiler(warmup_runs=0, output_dir="/tmp/bspec_prof")
    register_active_profiler(prof)
    try:
        prof.begin_run()
        for it in range(3):
            eng.admit("p")
            with prof.step_timing_ctx():
                eng.step([StepEntry("p", p, want=(n_tokens - 1,))])
            eng.release("p")
        buckets = prof.steps[-1]["buckets"]
    finally:
        release_active_profiler()
    return {k: round(v, 3) for k, v in sorted(buckets.items())}


def latent_attention_alone(z, pk, iters=20):
    """The latent attention kernel by itself: a prompt of 4,096 tokens (FLOP/s against the measured product peak:
    scores over rank + rotated numbers, values over the rank) and a decode step of 64 requests x 4,096 entries
    (bytes of entries read once against the measured copy rate; 1.1 GB of entries, beyond the L2)."""
    import torch
    from types import SimpleNamespace
    from batchspec_b200.kernels import ops
    dev = "cuda:0"
    Hh, R, Pd, ps = z["heads"], z["kv_rank"], z["rot"], 16
    out = {}
    for name, q_lens, ctx_len in (("prompt_4096", [4096], 4096), ("decode_64x4096", [1] * 64, 4096)):
        n, B = sum(q_lens), len(q_lens)
        pages_per = -(-ctx_len // ps)
        cache = torch.randn(B * pages_per, 1, ps * (R + Pd), device=dev).bfloat16()
        ql = torch.randn(Hh, n, R, device=dev).bfloat16()
        qr = torch.randn(n, Hh, Pd, device=dev).bfloat16()
        o = torch.empty(Hh, n, R, device=dev, dtype=torch.bfloat16)
        qo = torch.tensor([0] + list(__import__("itertools").accumulate(q_lens)), dtype=torch.int32, device=dev)
        pos = torch.cat([torch.arange(ctx_len - q, ctx_len) for q in q_lens]).to(dev, torch.int32)
        ent = torch.cat([torch.full((q,), i) for i, q in enumerate(q_lens)]).to(dev, torch.int32)
        ctx = SimpleNamespace(qo_indptr=qo, positions=pos, tok_entry=ent, n_entries=B, n_tokens=n, max_q_len=max(q_lens),
                              max_kv_len=ctx_len, extras={})
        tables = SimpleNamespace(kv_indptr=torch.arange(B + 1, dtype=torch.int32, device=dev) * pages_per,
                                 kv_indices=torch.randperm(B * pages_per, device=dev).to(torch.int32), page_size=ps)
        run = lambda: ops.latent_attention(ql, qr, o, cache, ctx, tables, Hh, R, Pd, 0.05)
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            run()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / iters
        if name.startswith("prompt"):
            flops = 2.0 * Hh * (R + Pd + R) * ctx_len * (ctx_len + 1) / 2
            out[name] = dict(ms=round(ms, 4), tflops=round(flops / ms / 1e9, 1),
                             frac_of_measured=round(flops / ms / 1e9 / pk["bf16_tflops"], 4))
        else:
            nbytes = B * ctx_len * (R + Pd) * 2
            out[name] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1),
                             frac_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
    return out


LUPUSUN_SIZES = {
    # width, attention heads / kv heads, head size, chunk of the mask, delta rule heads / q-k heads, feed-forward
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, chunk=1024, delta_heads=16, delta_kv_heads=8, dense_ff=8448),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, chunk=1024, delta_heads=32, delta_kv_heads=16, dense_ff=14336),
}


def lupusun_config_json(z, layers, vocab=32000):
    """Attention and delta rule layers in turn, each with a feed-forward; no loop, so that the depth equals the
    Llama model's."""
    att = dict(type="attention", mlp=dict(kind="dense", ff=z["dense_ff"]),
               mixer=dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=z["dim"], vdim=z["dim"], scale=z["dim"] ** -0.5,
                          mask=dict(size=z["chunk"]),
                          rot=dict(base=500000.0, dims=z["dim"], scaling=dict(factor=8.0, original=8192, fast=32.0, slow=1.0))))
    dlt = dict(type="delta", mlp=dict(kind="dense", ff=z["dense_ff"]),
               mixer=dict(heads=z["delta_heads"], kv_heads=z["delta_kv_heads"], dim=z["dim"], vdim=z["dim"], conv=4))
    return dict(architecture="Lupusun", vocab=vocab, width=z["width"], norm=dict(eps=1e-5), residual_mult=0.7,
                layers=[att if i % 2 == 0 else dlt for i in range(layers)])


def _time(run, iters=20):
    import torch
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        run()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def lupusun_kernels_alone(z, pk, iters=20):
    """The design's own kernels by themselves, each beside the like kernel of the Llama model at equal sizes:
    attention with the chunk mask and the sink against plain causal attention (a prompt of 4,096 tokens: FLOP/s over
    the visible pairs against the measured product peak; a decode step of 64 requests x 4,096 keys: bytes of visible
    keys and values against the measured copy rate), the q/k/v preparation against the rotate-and-append kernel
    (bytes), and the delta rule's kernels (bytes of state read and written for decode; FLOP/s for a prompt)."""
    import torch
    from types import SimpleNamespace
    from batchspec_b200.kernels import ops
    dev = "cuda:0"
    Hq, G, hd, ps, chunk = z["heads"], z["kv_heads"], z["dim"], 16, z["chunk"]
    out = {}
    sink = torch.linspace(-1.0, 1.0, Hq, device=dev)
    sink_l2 = ops.sink_table(sink)

    def step_ctx(q_lens, ctx_len):
        n, B = sum(q_lens), len(q_lens)
        pages_per = -(-ctx_len // ps)
        qo = torch.tensor([0] + list(__import__("itertools").accumulate(q_lens)), dtype=torch.int32, device=dev)
        pos = torch.cat([torch.arange(ctx_len - q, ctx_len) for q in q_lens]).to(dev, torch.int32)
        ent = torch.cat([torch.full((q,), i) for i, q in enumerate(q_lens)]).to(dev, torch.int32)
        ctx = SimpleNamespace(qo_indptr=qo, positions=pos, tok_entry=ent, n_entries=B, n_tokens=n, max_q_len=max(q_lens),
                              max_kv_len=ctx_len, kv_len=torch.full((B,), ctx_len, dtype=torch.int32, device=dev),
                              state_slots=torch.arange(B, dtype=torch.int32, device=dev),
                              extras={"min_q_len": min(q_lens)})
        tables = SimpleNamespace(kv_indptr=torch.arange(B + 1, dtype=torch.int32, device=dev) * pages_per,
                                 kv_indices=torch.randperm(B * pages_per, device=dev).to(torch.int32), page_size=ps)
        return ctx, tables, n, B, pages_per

    for name, q_lens, ctx_len in (("prompt_4096", [4096], 4096), ("decode_64x4096", [1] * 64, 4096)):
        ctx, tables, n, B, pages_per = step_ctx(q_lens, ctx_len)
        cache = torch.randn(B * pages_per, 2, ps * G * hd, device=dev).bfloat16()
        q = torch.randn(n, Hq * hd, device=dev).bfloat16()
        o = torch.empty(n, Hq * hd, device=dev, dtype=torch.bfloat16)
        for label, ck, sk, sk2 in (("chunk_sink", chunk, sink, sink_l2), ("sink", 0, sink, sink_l2), ("causal", 0, None, None)):
            ctx.extras = {"min_q_len": min(q_lens)}
            ms = _time(lambda: ops.paged_attention(q, o, cache, ctx, tables, Hq, G, hd, hd ** -0.5, 0, ck, sk, sk2), iters)
            span = ck or (1 << 30)
            pairs = sum(p - (p // span) * span + 1 for p in range(ctx_len - q_lens[0], ctx_len)) * len(q_lens)
            if name.startswith("prompt"):
                flops = 4.0 * Hq * hd * pairs
                out[f"attention_{name}_{label}"] = dict(ms=round(ms, 4), tflops=round(flops / ms / 1e9, 1),
                                                        frac_of_measured=round(flops / ms / 1e9 / pk["bf16_tflops"], 4))
            else:
                nbytes = pairs * 2 * G * hd * 2
                out[f"attention_{name}_{label}"] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1),
                                                        frac_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
    # q/k/v preparation against rotate-and-append: bytes read and written per token
    ctx, tables, n, B, pages_per = step_ctx([4096], 4096)
    cache = torch.zeros(pages_per, 2, ps * G * hd, device=dev, dtype=torch.bfloat16)
    width = (Hq + 2 * G) * hd
    qkv32 = torch.randn(n, width, device=dev)
    qkv16 = torch.randn(n, width, device=dev).bfloat16()
    bias = torch.randn(width, device=dev)
    freq = ops.rope_frequency_table(torch.pow(torch.tensor(500000.0, dtype=torch.float64), -torch.arange(0, hd // 2, dtype=torch.float64) * 2 / hd), dev)
    ms = _time(lambda: ops.qkv_prepare(qkv32, Hq, G, hd, hd, bias, freq, hd, False, 1.2, 1e-5, ctx.positions, ctx.tok_entry,
                                       tables.kv_indptr, tables.kv_indices, cache, ps), iters)
    nbytes = n * width * (4 + 2)
    out["qkv_prepare_4096"] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1), frac_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
    ms = _time(lambda: ops.rope_kv_append(qkv16, Hq, G, hd, freq, hd, False, ctx.positions, ctx.tok_entry, tables.kv_indptr,
                                          tables.kv_indices, cache, ps), iters)
    nbytes = n * (width * 2 + Hq * hd * 2 + 2 * G * hd * 2)
    out["rope_kv_append_4096"] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1), frac_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
    # the delta rule's kernels
    Hd, Gd, dk, dv, taps = z["delta_heads"], z["delta_kv_heads"], z["dim"], z["dim"], 4
    C = 2 * Gd * dk + Hd * dv
    ld = C + Hd * dv + 2 * Hd
    tail_off = Hd * dv * dk
    conv = torch.randn(C, taps, device=dev) * 0.5
    a_log, dt_bias, norm_w = torch.zeros(Hd, device=dev), torch.zeros(Hd, device=dev), torch.ones(dv, device=dev)
    for name, q_lens in (("prompt_2048", [2048]), ("prompt_8x2048", [2048] * 8), ("decode_64", [1] * 64), ("decode_256", [1] * 256)):
        ctx, tables, n, B, _ = step_ctx(q_lens, q_lens[0])
        state = torch.zeros(B, tail_off + (taps - 1) * C, device=dev)
        proj = torch.randn(n, ld, device=dev)
        mix, gates = ops.delta_prepare(proj, ld - 2 * Hd, ld - Hd, conv, a_log, dt_bias, state, tail_off, ctx, Hd, Gd, dk, dv, taps, dk ** -0.5, 1e-6)
        ms_p = _time(lambda: ops.delta_prepare(proj, ld - 2 * Hd, ld - Hd, conv, a_log, dt_bias, state, tail_off, ctx, Hd, Gd, dk, dv, taps, dk ** -0.5, 1e-6), iters)
        ms_r = _time(lambda: ops.delta_recurrence(mix, gates, proj, state, tail_off, ctx, Hd, Gd, dk, dv, taps), iters)
        o32 = ops.delta_recurrence(mix, gates, proj, state, tail_off, ctx, Hd, Gd, dk, dv, taps)
        ms_n = _time(lambda: ops.gated_rmsnorm(o32, proj[:, C:C + Hd * dv], norm_w, 1e-5, Hd, dv, torch.bfloat16), iters)
        rec = dict(prepare_ms=round(ms_p, 4), recurrence_ms=round(ms_r, 4), out_norm_ms=round(ms_n, 4))
        b_prep = n * (C * 4 * 2 + 2 * Hd * 4 * 2)                       # rows read, mix and gates written
        rec["prepare_frac_of_measured"] = round(b_prep / ms_p / 1e6 / pk["hbm_gbs"], 4)
        b_norm = n * Hd * dv * (4 + 4 + 2)
        rec["out_norm_frac_of_measured"] = round(b_norm / ms_n / 1e6 / pk["hbm_gbs"], 4)
        if name.startswith("decode"):
            nbytes = B * Hd * dk * dv * 4 * 2                             # every state read and written once
            rec["recurrence_gbs"] = round(nbytes / ms_r / 1e6, 1)
            rec["recurrence_frac_of_measured"] = round(nbytes / ms_r / 1e6 / pk["hbm_gbs"], 4)
        else:
            flops = 7.0 * n * Hd * dk * dv                                # decay, S^T k, k u^T, S^T q in float32
            rec["recurrence_fp32_tflops"] = round(flops / ms_r / 1e9, 2)
        out[f"delta_{name}"] = rec
    return out


TOKOLORN_SIZES = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, chunk=1024, window=1024, inner=4096, state=16, dt_rank=128,
                  delta_heads=16, delta_kv_heads=8, dense_ff=8448),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, chunk=1024, window=1024, inner=8192, state=16, dt_rank=256,
                  delta_heads=32, delta_kv_heads=16, dense_ff=14336),
}


def tokolorn_config_json(z, layers, vocab=32000):
    """Chunk attention, lightning attention, window attention beside a selective scan, lightning attention, and so
    on in turn, each with a feed-forward; no loop, so that the depth equals the other models'."""
    H, hd = z["heads"], z["dim"]
    mlp = dict(kind="dense", ff=z["dense_ff"])
    att = dict(type="attention", mlp=mlp, mixer=dict(heads=H, kv_heads=z["kv_heads"], dim=hd, vdim=hd, scale=hd ** -0.5,
                                                     mask=dict(size=z["chunk"])))
    lit = dict(type="lightning", mlp=mlp,
               mixer=dict(heads=H, dim=hd, vdim=hd, decay=[1.0 - 2.0 ** (-(2.0 + 6.0 * i / (H - 1))) for i in range(H)]))
    par = dict(type="parallel", mlp=mlp, mixer=dict(
        left=dict(heads=H, kv_heads=z["kv_heads"], dim=hd, vdim=hd, scale=hd ** -0.5, softcap=30.0,
                  mask=dict(size=z["window"]), rot=dict(base=500000.0, dims=hd)),
        right=dict(inner=z["inner"], state=z["state"], dt_rank=z["dt_rank"], conv=4), left_scale=0.5, right_scale=0.5))
    return dict(architecture="Tokolorn", vocab=vocab, width=z["width"], norm=dict(eps=1e-5), logit_scale=1.0,
                embedding=dict(scale=1.0, bigram=dict(buckets=65521, mul_prev=31, mul_cur=7)),
                layers=[(att, lit, par, lit)[i % 4] for i in range(layers)])


def tokolorn_kernels_alone(z, pk, iters=20):
    """The design's own kernels by themselves.  Attention (a prompt of 4,096 tokens: FLOP/s over the visible pairs
    against the measured product peak; a decode step of 64 requests x 4,096 keys: bytes of visible keys and values
    against the measured copy rate) with a window and a soft cap, and with a chunk mask and a sink, beside plain
    causal attention; the lightning recurrence and the selective scan (decode: bytes of state read and written against
    the copy rate; prompts: time per token), their neighbours (output norm, convolution, gate), and the bigram rows."""
    import torch
    from types import SimpleNamespace
    from itertools import accumulate
    from batchspec_b200.kernels import ops
    ops.require("state_mixers")
    dev = "cuda:0"
    Hq, G, hd, ps = z["heads"], z["kv_heads"], z["dim"], 16
    out = {}
    sink = torch.zeros(Hq, device=dev)
    sink_l2 = ops.sink_table(sink)

    def step_ctx(q_lens, ctx_len):
        n, B = sum(q_lens), len(q_lens)
        pages_per = -(-ctx_len // ps)
        qo = torch.tensor([0] + list(accumulate(q_lens)), dtype=torch.int32, device=dev)
        pos = torch.cat([torch.arange(ctx_len - q, ctx_len) for q in q_lens]).to(dev, torch.int32)
        ent = torch.cat([torch.full((q,), i) for i, q in enumerate(q_lens)]).to(dev, torch.int32)
        ctx = SimpleNamespace(qo_indptr=qo, positions=pos, tok_entry=ent, n_entries=B, n_tokens=n, max_q_len=max(q_lens),
                              max_kv_len=ctx_len, kv_len=torch.full((B,), ctx_len, dtype=torch.int32, device=dev),
                              state_slots=torch.arange(B, dtype=torch.int32, device=dev),
                              token_ids=torch.randint(0, 32000, (n,), dtype=torch.int32, device=dev),
                              extras={"min_q_len": min(q_lens)})
        tables = SimpleNamespace(kv_indptr=torch.arange(B + 1, dtype=torch.int32, device=dev) * pages_per,
                                 kv_indices=torch.randperm(B * pages_per, device=dev).to(torch.int32), page_size=ps)
        return ctx, tables, n, B, pages_per

    for name, q_lens, ctx_len in (("prompt_4096", [4096], 4096), ("decode_64x4096", [1] * 64, 4096)):
        ctx, tables, n, B, pages_per = step_ctx(q_lens, ctx_len)
        cache = torch.randn(B * pages_per, 2, ps * G * hd, device=dev).bfloat16()
        q = torch.randn(n, Hq * hd, device=dev).bfloat16()
        o = torch.empty(n, Hq * hd, device=dev, dtype=torch.bfloat16)
        for label, win, ck, sk, sk2, cap in (("window_cap", z["window"], 0, None, None, 50.0),
                                             ("window", z["window"], 0, None, None, 0.0),
                                             ("chunk_sink", 0, z["chunk"], sink, sink_l2, 0.0), ("causal", 0, 0, None, None, 0.0)):
            ctx.extras = {"min_q_len": min(q_lens)}
            ms = _time(lambda: ops.paged_attention(q, o, cache, ctx, tables, Hq, G, hd, hd ** -0.5, win, ck, sk, sk2, cap), iters)
            first = lambda p: max(0, p - win + 1) if win else ((p // ck) * ck if ck else 0)
            pairs = sum(p - first(p) + 1 for p in range(ctx_len - q_lens[0], ctx_len)) * len(q_lens)
            if name.startswith("prompt"):
                flops = 4.0 * Hq * hd * pairs
                out[f"attention_{name}_{label}"] = dict(ms=round(ms, 4), tflops=round(flops / ms / 1e9, 1),
                                                        frac_of_measured=round(flops / ms / 1e9 / pk["bf16_tflops"], 4))
            else:
                nbytes = pairs * 2 * G * hd * 2
                out[f"attention_{name}_{label}"] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1),
                                                        frac_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
    # gate and factor after the attention, bigram rows after the embedding: bytes read and written
    n = 4096
    ctx, tables, _, _, _ = step_ctx([n], n)
    heads = torch.randn(n, Hq * hd, device=dev).bfloat16()
    gate = torch.randn(n, Hq * hd, device=dev)
    both = torch.empty(n, Hq * hd + z["inner"], device=dev, dtype=torch.bfloat16)
    ms = _time(lambda: ops.gate_mul(heads, gate, both[:, :Hq * hd], 0.5), iters)
    nbytes = n * Hq * hd * (2 + 4 + 2)
    out["gate_mul_4096"] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1), frac_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
    resid = torch.zeros(n, z["width"], device=dev)
    table = torch.randn(65522, z["width"], device=dev).bfloat16()
    prev = torch.zeros(4, 1, dtype=torch.int32, device=dev)
    ms = _time(lambda: ops.bigram_add(resid, table, prev, ctx, 65521, 1009, 17, 32000), iters)
    nbytes = n * z["width"] * (4 + 4 + 2)
    out["bigram_add_4096"] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1), frac_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
    # the two recurrences
    H, dk, dv = z["heads"], hd, hd
    inner, N, taps = z["inner"], z["state"], 4
    decay = torch.linspace(0.75, 0.999, H, device=dev)
    norm_w = torch.ones(H * dv, device=dev)
    conv, conv_b = torch.randn(inner, taps, device=dev) * 0.5, torch.zeros(inner, device=dev)
    a_log, d_skip, dt_b = torch.zeros(inner, N, device=dev), torch.ones(inner, device=dev), torch.zeros(inner, device=dev)
    for name, q_lens in (("prompt_2048", [2048]), ("prompt_8x2048", [2048] * 8), ("decode_64", [1] * 64), ("decode_256", [1] * 256)):
        ctx, tables, n, B, _ = step_ctx(q_lens, q_lens[0])
        ld = 2 * H * dk + 2 * H * dv
        proj = torch.randn(n, ld, device=dev)
        state = torch.zeros(B, H * dv * dk, device=dev)
        ms_r = _time(lambda: ops.lightning_recurrence(proj, 0, H * dk, 2 * H * dk, decay, state, ctx, H, dk, dv), iters)
        o32 = ops.lightning_recurrence(proj, 0, H * dk, 2 * H * dk, decay, state, ctx, H, dk, dv)
        ms_n = _time(lambda: ops.gated_rmsnorm(o32, proj[:, 2 * H * dk + H * dv:], norm_w, 1e-5, 1, H * dv, torch.bfloat16, "sigmoid"), iters)
        rec = dict(recurrence_ms=round(ms_r, 4), out_norm_ms=round(ms_n, 4),
                   out_norm_frac_of_measured=round(n * H * dv * (4 + 4 + 2) / ms_n / 1e6 / pk["hbm_gbs"], 4))
        if name.startswith("decode"):
            nbytes = B * H * dk * dv * 4 * 2                              # every state read and written once
            rec["recurrence_gbs"] = round(nbytes / ms_r / 1e6, 1)
            rec["recurrence_frac_of_measured"] = round(nbytes / ms_r / 1e6 / pk["hbm_gbs"], 4)
        else:
            rec["recurrence_ns_per_token"] = round(ms_r * 1e6 / q_lens[0], 1)
            rec["recurrence_fp32_tflops"] = round(5.0 * n * H * dk * dv / ms_r / 1e9, 2)     # decay, k v^T, S^T q
        out[f"lightning_{name}"] = rec
        xz = torch.randn(n, 2 * inner, device=dev)
        sstate = torch.zeros(B, N * inner + (taps - 1) * inner, device=dev)
        ms_c = _time(lambda: ops.scan_conv(xz, conv, conv_b, sstate, N * inner, ctx, inner, taps, torch.bfloat16), iters)
        xc, _ = ops.scan_conv(xz, conv, conv_b, sstate, N * inner, ctx, inner, taps, torch.bfloat16)
        dt_raw, bc = torch.randn(n, inner, device=dev), torch.randn(n, 2 * N, device=dev)
        y = torch.empty(n, inner, device=dev, dtype=torch.bfloat16)
        table = ops.scan_decay_table(a_log)
        ms_s = _time(lambda: ops.selective_scan(xz, xc, dt_raw, bc, a_log, d_skip, dt_b, sstate, N * inner, ctx, y, 0.5, inner, N, taps, table), iters)
        rec = dict(conv_ms=round(ms_c, 4), scan_ms=round(ms_s, 4),
                   conv_frac_of_measured=round(n * inner * (4 + 4 + 2) / ms_c / 1e6 / pk["hbm_gbs"], 4))
        nbytes = B * inner * N * 4 * 2 + n * inner * (4 * 4 + 2)          # state once; x, z, xc, dt read, y written
        rec["scan_gbs"] = round(nbytes / ms_s / 1e6, 1)
        rec["scan_frac_of_measured"] = round(nbytes / ms_s / 1e6 / pk["hbm_gbs"], 4)
        if not name.startswith("decode"):
            rec["scan_ns_per_token"] = round(ms_s * 1e6 / q_lens[0], 1)
        out[f"scan_{name}"] = rec
    return out


FINOLIX_SIZES = {
    # the Vabanex sizes (width, heads, head sizes, ranks, experts) with a window on the latent layers and four streams
    "w2048": dict(VABANEX_SIZES["w2048"], window=1024, streams=4),
    "w4096": dict(VABANEX_SIZES["w4096"], window=1024, streams=4),
}


def finolix_config_json(z, layers, vocab=32000):
    """Latent attention (window, sink) and gated grouped-query attention in turn; the first layer's feed-forward is
    the dense one, the others are routed (as in the Vabanex model of equal size, whose experts have two matrices
    where these have three)."""
    lat = dict(heads=z["heads"], dim=z["dim"], rot_dim=z["rot"], vdim=z["vdim"], q_rank=z["q_rank"],
               kv_rank=z["kv_rank"], scale=(z["dim"] + z["rot"]) ** -0.5, mask=dict(size=z["window"]),
               rot=dict(base=10000.0, dims=z["rot"], scaling=dict(factor=40.0, original=4096, fast=32.0, slow=1.0)))
    att = dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=128, vdim=128, scale=128 ** -0.5,
               rot=dict(base=500000.0, dims=64))
    moe = dict(kind="moe", expert=dict(ff=z["expert_ff"]), router=dict(experts=z["experts"], top=z["top"]))
    dense = dict(kind="dense", ff=z["dense_ff"])
    return dict(architecture="Finolix", vocab=vocab, width=z["width"], norm=dict(eps=1e-5), streams=z["streams"],
                layers=[dict(type="latent_attention" if i % 2 == 0 else "attention", mixer=lat if i % 2 == 0 else att,
                             mlp=dense if i == 0 else moe) for i in range(layers)])


def finolix_kernels_alone(z, pk, iters=20):
    """The design's own kernels by themselves, each beside its like at equal sizes: latent attention with the window
    and the sink against the same kernel without them (a prompt of 4,096 tokens: FLOP/s over the visible pairs
    against the measured product peak; a decode step of 64 requests x 4,096 entries: bytes of visible entries
    against the measured copy rate); the join, read and norm over the streams against add + RMS norm (bytes); the
    q/k/v preparation with weighted head norms against the one without; the gate per head; routed gated experts
    against routed GELU experts (FLOP/s of the two or three matrices of the chosen experts)."""
    import torch
    from types import SimpleNamespace
    from batchspec_b200.kernels import ops
    from batchspec_b200.parts.base import FEED_FORWARDS, PartSpec, Runtime, build_part
    dev = "cuda:0"
    Hh, R, Pd, ps, W, S, d = z["heads"], z["kv_rank"], z["rot"], 16, z["window"], z["streams"], z["width"]
    out = {}
    sinks = torch.linspace(-1.0, 1.0, Hh, device=dev)

    def step_ctx(q_lens, ctx_len):
        n, B = sum(q_lens), len(q_lens)
        pages_per = -(-ctx_len // ps)
        qo = torch.tensor([0] + list(__import__("itertools").accumulate(q_lens)), dtype=torch.int32, device=dev)
        pos = torch.cat([torch.arange(ctx_len - q, ctx_len) for q in q_lens]).to(dev, torch.int32)
        ent = torch.cat([torch.full((q,), i) for i, q in enumerate(q_lens)]).to(dev, torch.int32)
        ctx = SimpleNamespace(qo_indptr=qo, positions=pos, tok_entry=ent, n_entries=B, n_tokens=n, max_q_len=max(q_lens),
                              max_kv_len=ctx_len, kv_len=torch.full((B,), ctx_len, dtype=torch.int32, device=dev),
                              extras={"min_q_len": min(q_lens)})
        tables = SimpleNamespace(kv_indptr=torch.arange(B + 1, dtype=torch.int32, device=dev) * pages_per,
                                 kv_indices=torch.randperm(B * pages_per, device=dev).to(torch.int32), page_size=ps)
        return ctx, tables, n, B, pages_per

    for name, q_lens, ctx_len in (("prompt_4096", [4096], 4096), ("decode_64x4096", [1] * 64, 4096)):
        ctx, tables, n, B, pages_per = step_ctx(q_lens, ctx_len)
        cache = torch.randn(B * pages_per, 1, ps * (R + Pd), device=dev).bfloat16()
        ql = torch.randn(Hh, n, R, device=dev).bfloat16()
        qr = torch.randn(n, Hh, Pd, device=dev).bfloat16()
        o = torch.empty(Hh, n, R, device=dev, dtype=torch.bfloat16)
        for label, win, sk in (("window_sink", W, sinks), ("sink", 0, sinks), ("causal", 0, None)):
            ms = _time(lambda: ops.latent_attention(ql, qr, o, cache, ctx, tables, Hh, R, Pd, 0.05, window=win, sink=sk), iters)
            span = win or (1 << 30)
            pairs = sum(min(p + 1, span) for p in range(ctx_len - q_lens[0], ctx_len)) * len(q_lens)
            if name.startswith("prompt"):
                flops = 2.0 * Hh * (R + Pd + R) * pairs
                out[f"latent_{name}_{label}"] = dict(ms=round(ms, 4), tflops=round(flops / ms / 1e9, 1),
                                                     frac_of_measured=round(flops / ms / 1e9 / pk["bf16_tflops"], 4))
            else:
                nbytes = pairs * (R + Pd) * 2
                out[f"latent_{name}_{label}"] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1),
                                                     frac_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
    # the streams' join + read + norm against add + RMS norm, 4,096 rows and 64 rows
    for n in (4096, 64):
        x = torch.randn(n, S, d, device=dev)
        one = torch.randn(n, d, device=dev)
        y = torch.randn(n, d, device=dev).bfloat16()
        vec, w = torch.ones(d, device=dev), torch.ones(d, device=dev)
        mixw = torch.cat([torch.eye(S, device=dev).reshape(-1), torch.ones(S, device=dev)]).contiguous()
        rd = torch.full((S,), 1.0 / S, device=dev)
        o = torch.empty(n, d, device=dev, dtype=torch.bfloat16)
        ms = _time(lambda: ops.stream_norm(x, y, vec, mixw, rd, w, 1e-5, o), iters)
        nbytes = n * d * (S * 8 + 2 + 2)
        out[f"stream_norm_{n}"] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1),
                                       frac_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
        ms = _time(lambda: ops.add_rmsnorm(one, y, w, 1e-5, o, 1.0, True, vec), iters)
        nbytes = n * d * (8 + 2 + 2)
        out[f"add_rmsnorm_{n}"] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1),
                                       frac_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
    # q/k/v preparation with weighted head norms before the rotation against the one without; the gate per head
    Hq, G, hd = z["heads"], z["kv_heads"], 128
    ctx, tables, n, B, pages_per = step_ctx([4096], 4096)
    cache = torch.zeros(pages_per, 2, ps * G * hd, device=dev, dtype=torch.bfloat16)
    width = (Hq + 2 * G) * hd
    qkv32 = torch.randn(n, width, device=dev)
    nw = torch.ones(hd, device=dev, dtype=torch.bfloat16)
    freq = ops.rope_frequency_table(torch.pow(torch.tensor(500000.0, dtype=torch.float64), -torch.arange(0, 32, dtype=torch.float64) * 2 / 64), dev)
    nbytes = n * width * (4 + 2)
    for label, kw in (("qkv_prepare_weighted_norm_4096", dict(q_norm=nw, k_norm=nw, norm_first=True)), ("qkv_prepare_4096", {})):
        ms = _time(lambda: ops.qkv_prepare(qkv32, Hq, G, hd, hd, None, freq, 64, False, 1.0, 1e-5 if kw else 0.0, ctx.positions,
                                           ctx.tok_entry, tables.kv_indptr, tables.kv_indices, cache, ps, **kw), iters)
        out[label] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1), frac_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
    heads = torch.randn(n, Hq * hd, device=dev).bfloat16()
    gate = torch.randn(n, Hq, device=dev)
    gate_all = torch.randn(n, Hq * hd, device=dev)
    o = torch.empty_like(heads)
    ms = _time(lambda: ops.gate_heads(heads.view(n, Hq, hd).transpose(0, 1), gate, o), iters)
    out["gate_per_head_4096"] = dict(ms=round(ms, 4), frac_of_measured=round(n * Hq * hd * 4 / ms / 1e6 / pk["hbm_gbs"], 4))
    ms = _time(lambda: ops.gate_mul(heads, gate_all, o), iters)
    out["gate_per_number_4096"] = dict(ms=round(ms, 4), frac_of_measured=round(n * Hq * hd * 8 / ms / 1e6 / pk["hbm_gbs"], 4))
    # routed experts: gated (three matrices) against GELU (two), the router included
    rt = Runtime(torch.bfloat16, torch.device(dev))
    E, top, ff = z["experts"], z["top"], z["expert_ff"]
    glu = build_part(FEED_FORWARDS, PartSpec("routed_glu", dict(dim=d, intermediate=ff, n_experts=E, top=top)), rt)
    gelu = build_part(FEED_FORWARDS, PartSpec("routed_gelu", dict(dim=d, intermediate=ff, n_experts=E, top=top, n_groups=z["groups"],
                                                                  keep_groups=z["keep"])), rt)
    for part, mats in ((glu, 3), (gelu, 2)):
        part.bind({k: (torch.randn(ps_.shape, device=dev) * 0.02).bfloat16() for k, ps_ in part.param_specs().items()})
        for n in (4096, 64):
            x = torch.randn(n, d, device=dev).bfloat16()
            ms = _time(lambda: part.forward(x, None), iters)
            flops = 2.0 * n * top * mats * ff * d
            rec = dict(ms=round(ms, 4), tflops=round(flops / ms / 1e9, 1), frac_of_measured=round(flops / ms / 1e9 / pk["bf16_tflops"], 4))
            if n == 64:                     # decode: the weights of the experts that were chosen are read once
                nbytes = min(E, n * top) * mats * ff * d * 2
                rec["weights_frac_of_measured"] = round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4)
            out[f"{part.kind}_{n}"] = rec
        del part
    return out


DESIGNS = {
    "finolix": (FINOLIX_SIZES, finolix_config_json, finolix_kernels_alone, "kernels_alone"),
    "tokolorn": (TOKOLORN_SIZES, tokolorn_config_json, tokolorn_kernels_alone, "kernels_alone"),
    "vabanex": (VABANEX_SIZES, vabanex_config_json, latent_attention_alone, "latent_attention_alone"),
    "lupusun": (LUPUSUN_SIZES, lupusun_config_json, lupusun_kernels_alone, "kernels_alone"),
}


def run_design(a) -> int:
    """Prompt and decode throughput of a second design at layer sizes of real models (random weights, bfloat16)
    beside the Llama model of equal size, with the device time of every part of a prompt step and the design's own
    kernels by themselves.  One JSON line."""
    import torch
    from batchspec_b200.config import config_from_json_dict
    from batchspec_b200.engine import Engine
    pk = peaks()
    layers = a.layers or 4
    out = {"design": a.design, "layers": layers, "dtype": "bf16", "data": "synthetic", "prompt_len": PROMPT_LEN,
           "peaks": pk["source"], "sizes": {}}
    sizes, config_json, alone, alone_key = DESIGNS[a.design]
    for size, z in sizes.items():
        rec = {}
        models = [(a.design, config_json(z, layers)), ("llama", llama_config_json(z, layers))]
        if a.design == "tokolorn":        # its closest model, the other one with recurrent state beside attention
            models.append(("lupusun", lupusun_config_json(z, layers)))
        if a.design == "finolix":         # its closest model, the other one with latent attention and routed experts
            models.append(("vabanex", vabanex_config_json(z, layers)))
        for label, cj in models:
            cfg = config_from_json_dict(cj)
            eng = Engine(dtype="bfloat16", device="cuda:0")
            eng.load_model(config=cfg, random_seed=0, draw_on_device=True)
            eng.setup_sampling_params(temperature=0.0)
            r = {"prefill_ms": round(run_prefill(eng, cfg), 3)}
            r["prefill_tok_s"] = round(PROMPT_LEN / (r["prefill_ms"] * 1e-3), 1)
            for b in (8, 64):
                ms, launches = run_decode(eng, cfg, b, a.steps, max(a.warmup, 3))
                r[f"decode_b{b}_ms"] = round(ms, 4)
                r[f"decode_b{b}_tok_s"] = round(b * 1000.0 / ms, 1)
                r[f"decode_b{b}_launches_per_step"] = launches // a.steps
            r["prompt_step_parts_ms"] = run_buckets(eng, cfg, PROMPT_LEN)
            rec[label] = r
            del eng
            torch.cuda.empty_cache()
        rec[alone_key] = alone(z, pk)
        out["sizes"][size] = rec
    print(json.dumps(out))
    return 0


def reference_arm(a) -> int:
    """``--impl reference``: the unmodified reference through its own ``StandardEngine.generate`` (see
    baseline/reference_arm.py) on the same workload: batch, 2,048-token prompts, greedy decode steps.  If it cannot
    be imported or run, one line says why and the exit code is 0."""
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    cfg = json.loads((ROOT / "batchspec_b200" / "config" / "presets" / "llama-3-8b.json").read_text())
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    try:
        from baseline import reference_arm as RA
        clocks = ClockSampler()
        clocks.start()
        try:
            r = RA.bench(cfg, a.batch, PROMPT_LEN, a.steps, a.warmup)
        finally:
            clock_rec = clocks.stop()
    except BaseException as exc:                                    # noqa: BLE001  (the line must say what happened)
        if isinstance(exc, KeyboardInterrupt):
            raise
        why = " ".join(f"{type(exc).__name__}: {exc}".split())[:400]
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    out = {
        "metric": f"decode tok/s (Llama-3-8B sizes, bf16, batch {a.batch}, {PROMPT_LEN}-token prompts)",
        "value": round(a.batch * 1000.0 / r["ms_per_step"], 2), "unit": "tok/s", "n_gpus": 1, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": round(r["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"model": "llama-3-8b", "global_batch": a.batch, "seq_len": PROMPT_LEN, "parallelism": "single",
                   "layers": cfg["num_hidden_layers"], "layers_full": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": hd,
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "page_size": 16,
                   "weights": "random N(0,0.02)", "l2": "inputs_exceed_l2 (15 GB of weights per step)",
                   "prefill_chunk": r["chunk"],
                   "how": "StandardEngine.generate; CUDA events before each model call; tracer output discarded"},
        "clocks": clock_rec,
        "e2e": {"value": round(a.batch * 1000.0 / r["wall_ms_per_step"], 2), "unit": "tok/s",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": a.batch, "warmup_steps": r["warmup_steps"],
                "note": "generate keeps token ids on the device and reads one end-of-sequence flag per request"},
    }
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0: all)")
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (no prefill, b1, b64, e2e)")
    ap.add_argument("--skip-workloads", action="store_true",
                    help="leave out e2e at batch 64 and the 3B / long-context workloads (about a minute)")
    ap.add_argument("--design", default=None, choices=["vabanex", "lupusun", "tokolorn", "finolix"],
                    help="instead of the headline workload: this design at real layer sizes beside the Llama model of equal size")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    if a.design:
        return run_design(a)
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    import torch
    pk = peaks()
    eng, cfg, full_layers = build_engine(a.layers)
    L = cfg.num_hidden_layers
    nums = model_numbers(cfg, L)
    section_clocks = {}

    def timed_section(name, fn, *args):
        """Runs one section with its own record of the clocks."""
        clocks = ClockSampler()
        clocks.start()
        try:
            return fn(*args)
        finally:
            section_clocks[name] = clocks.stop()

    ms, launches = timed_section("decode", run_decode, eng, cfg, a.batch, a.steps, a.warmup)
    clock_rec = section_clocks["decode"]
    value = a.batch * 1000.0 / ms
    mean_ctx = PROMPT_LEN + a.warmup + (a.steps + 1) / 2.0
    step_bytes = nums["weight_bytes"] + a.batch * mean_ctx * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s (Llama-3-8B sizes, bf16, batch {a.batch}, {PROMPT_LEN}-token prompts)", "value": round(value, 2),
        "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": "llama-3-8b", "global_batch": a.batch, "seq_len": PROMPT_LEN, "parallelism": "single",
                   "layers": L, "layers_full": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "page_size": 16,
                   "weights": "random N(0,0.02)", "l2": "inputs_exceed_l2 (15 GB of weights per step)",
                   "peaks": pk["source"]},
        "gpu_launches": launches, "clocks": clock_rec,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if not a.skip_points:
        # the prompt step right after the (light) decode section: it is bound by the tensor cores under the power
        # cap, and what ran just before it moves its clocks
        pms = timed_section("prefill", run_prefill, eng, cfg)
        flops = (PROMPT_LEN * nums["gemm_flops_per_token"] + nums["head_flops_per_row"]
                 + nums["attn_flops_per_pair"] * PROMPT_LEN * (PROMPT_LEN + 1) / 2)
        out["prefill"] = {"value": round(PROMPT_LEN / (pms * 1e-3), 1), "tokens": PROMPT_LEN, "ms": round(pms, 3),
                          "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        out["e2e"] = timed_section("e2e", run_e2e, eng, cfg, a.batch, a.steps, a.warmup)
        out["e2e"]["of_device_timed"] = round(out["e2e"]["value"] / value, 4)
        points = {}
        for b in (1, 64):
            bms, _ = timed_section(f"decode_b{b}", run_decode, eng, cfg, b, a.steps, a.warmup)
            points[f"decode_b{b}"] = round(b * 1000.0 / bms, 2)
            ctx_bytes = nums["weight_bytes"] + b * mean_ctx * nums["kv_bytes_per_token"]
            points[f"decode_b{b}_hbm_frac"] = round(ctx_bytes / (bms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
            if b == 64 and not a.skip_workloads:
                e64 = timed_section("e2e_b64", run_e2e, eng, cfg, 64, a.steps, a.warmup)
                points["e2e_b64"] = e64["value"]
                points["e2e_b64_of_device_timed"] = round(e64["value"] / points["decode_b64"], 4)
        if not a.skip_workloads:
            del eng
            torch.cuda.empty_cache()
            points.update(timed_section("cfg4", run_cfg4, pk))
            points.update(timed_section("cfg5", run_cfg5, pk))
        out["points"] = points
        out["section_clocks"] = section_clocks
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
