"""The prefix-reuse workload and the admission-wave workload through the request scheduler on one GPU, on
synthetic token ids and seeded q/k/v tables (no model):

  shared   256 requests = common 1024-id prefix + unique 256-id suffix (Qwen3-8B attention
           shape, fp16, block 16), 128 decode steps each; request 0 is prefilled in full and
           registers the prefix, the others hit it.  `--unaligned` uses prefix 1000 + suffix 280
           so that the shared partial block is copied on first write.
  waves    decode requests with ctx ~ U{lo..hi} admitted in waves into a pool smaller than the
           whole set (fill the pool, decode, retire, refill).

    python tests/profiling/serving_case.py shared [--layers 4] [--unaligned] [--no-share]
    python tests/profiling/serving_case.py waves  [--layers 4] [--requests 96] [--lo 2048] [--hi 8192] \
                                                  [--blocks 20000] [--steps 16]

Prints pool usage, copy-on-write events, reuse, and the decode phase's algorithmic KV GB/s (device
time of the decode launches only, CUDA events around each step's layers).
"""
import argparse
import sys
import time
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from tests.serving_sim import ServingSim  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("case", choices=["shared", "waves"])
ap.add_argument("--layers", type=int, default=4)
ap.add_argument("--unaligned", action="store_true")
ap.add_argument("--no-share", action="store_true")
ap.add_argument("--requests", type=int, default=96)
ap.add_argument("--lo", type=int, default=2048)
ap.add_argument("--hi", type=int, default=8192)
ap.add_argument("--blocks", type=int, default=20000)
ap.add_argument("--steps", type=int, default=16)
a = ap.parse_args()
H, HKV = 32, 8


def timed_run(sim):
    """sim.run() with CUDA events around every decode step's launches."""
    events, bytes_per_step = [], []
    orig = sim.run_decode

    def wrapped(d):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = sim.kv_bytes_decoded
        e0.record()
        orig(d)
        e1.record()
        events.append((e0, e1))
        bytes_per_step.append(sim.kv_bytes_decoded - before)

    sim.run_decode = wrapped
    sim.decode_events = []
    t0 = time.perf_counter()
    sim.run()
    wall = time.perf_counter() - t0
    ms = [e0.elapsed_time(e1) for e0, e1 in events]
    return wall, ms, bytes_per_step


def kernel_line(sim, min_frac=0.9):
    """Device time of the decode launches alone (largest batches only: the steady state).  The
    median launch is reported: a launch that the host enqueues late (the device idle meanwhile)
    shows the host's delay inside its event bracket."""
    ev = [(e0.elapsed_time(e1), b) for e0, e1, b in sim.decode_events]
    top = max(b for _, b in ev)
    ev = [(m, b) for m, b in ev if b >= min_frac * top]
    rate = np.median([b / m for m, b in ev]) / 1e6
    return (f"  decode kernel alone: {len(ev)} launches of {np.mean([b for _, b in ev]) / 1e6:.1f} MB algorithmic, "
            f"median {np.median([m for m, _ in ev]) * 1e3:.1f} us = {rate:.1f} GB/s algorithmic")


if a.case == "shared":
    prefix, suffix = (1000, 280) if a.unaligned else (1024, 256)
    n_req, gen = 256, 129  # 129 sampled tokens = 128 cached decode positions
    sim = ServingSim(a.layers, H, HKV, num_blocks=24576, seed=7, max_positions=2048, prefill_chunk=512,
                     max_prefill_tokens=4096, max_decode_batch=256, use_prefix_cache=not a.no_share)
    rng = np.random.default_rng(4)
    common = rng.integers(0, 151936, prefix)
    first = sim.sched.submit(np.concatenate([common, rng.integers(0, 151936, suffix)]), 1, also_register=prefix)
    sim.run()
    for _ in range(n_req - 1):
        sim.sched.submit(np.concatenate([common, rng.integers(0, 151936, suffix)]), gen)
    wall, ms, nbytes = timed_run(sim)
    st = sim.sched.stats()
    print(f"shared-prefix workload: prefix {prefix} + suffix {suffix}, {n_req} requests, {gen - 1} decode steps, "
          f"{a.layers} layers, prefix cache {'off' if a.no_share else 'on'}")
    print(f"  peak blocks in use {st['peak_blocks_in_use']} (unshared: {n_req * ((prefix + suffix + gen - 1 + 15) // 16)}), "
          f"reused tokens {st['reused_tokens']}, prefilled {st['prefilled_tokens']}, "
          f"copy-on-write events {sim.manager.cow_events}")
    steady = [(m, b) for m, b in zip(ms, nbytes) if b == max(nbytes) or b > 0.9 * max(nbytes)]
    tot_ms, tot_b = sum(m for m, _ in steady), sum(b for _, b in steady)
    print(f"  decode phase: {len(ms)} steps, {sum(nbytes) / 1e9:.2f} GB algorithmic KV; full-batch steps: "
          f"{tot_b / tot_ms / 1e6:.1f} GB/s algorithmic over rope+append+decode of {a.layers} layers "
          f"({tot_ms / len(steady) * 1e3 / a.layers:.1f} us per layer-step, host work included)")
    print(kernel_line(sim))
    print(f"  wall {wall:.2f} s for {st['decoded_tokens']} decoded + {st['prefilled_tokens']} prefilled tokens")
else:
    sim = ServingSim(a.layers, H, HKV, num_blocks=a.blocks, seed=9, max_positions=a.hi + a.steps + 8,
                     prefill_chunk=2048, max_prefill_tokens=8192, max_decode_batch=256, use_prefix_cache=False)
    rng = np.random.default_rng(5)
    total_ctx = 0
    for _ in range(a.requests):
        n = int(rng.integers(a.lo, a.hi + 1))
        total_ctx += n
        sim.sched.submit(rng.integers(0, 151936, n), a.steps + 1)
    wall, ms, nbytes = timed_run(sim)
    st = sim.sched.stats()
    print(f"admission waves: {a.requests} requests, ctx U[{a.lo},{a.hi}] ({total_ctx} tokens = "
          f"{(total_ctx + 15) // 16} blocks) into a pool of {a.blocks} blocks, {a.steps} decode steps each, "
          f"{a.layers} layers")
    print(f"  admission stalls {st['admission_stalls']}, peak blocks in use {st['peak_blocks_in_use']}, "
          f"decode steps {st['decode_steps']}, prefill steps {st['prefill_steps']}")
    print(f"  decode launches: {sum(nbytes) / 1e9:.2f} GB algorithmic KV in {sum(ms):.1f} ms = "
          f"{sum(nbytes) / sum(ms) / 1e6:.1f} GB/s (rope+append+decode, host work of each step included)")
    print(kernel_line(sim, 0.5))
    print(f"  wall {wall:.2f} s; {st['decoded_tokens']} decoded tokens, {st['prefilled_tokens']} prefilled")
