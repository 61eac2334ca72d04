#!/usr/bin/env python
"""Headline benchmark: paged GQA decode attention at the Qwen3-8B attention shape.

Workload: 32 Q heads, 8 KV heads, head_dim 128, fp16 KV, block
size 16, batch 64, per-sequence context lengths uniform in [128, 4096] from a seed, block
pool = total blocks x 1.25 with a seeded random block table, Q/K/V ~ N(0,1).  One step =
one decode step of the KV-cache hot path over all 36 layers: per layer, RoPE the new Q/K
token of every sequence, append K/V into that layer's pool, then attend over the whole
context through the block table.  Every layer has its own 0.66 GB pool, so consecutive
launches never find their input in L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-graph]

Prints ONE JSON line (rank 0).  `value` is KV-read GB/s (algorithmic bytes / device time,
whole job); `e2e` is the same metric with the step's Q/K/V rows coming from pinned host
memory and the attention output going back to the host inside the timed region.
The step is captured once as a CUDA graph and replayed (the way the reference runs its decode
step); `--no-graph` launches every kernel separately.  The roofline's per-launch duration is
taken with CUDA events around every decode launch: inside the timed region with `--no-graph`,
otherwise over the same K steps launched one by one right after the timed replays.
`--impl reference` times the CPU restatement of the reference's fp32 MHA path (the oracle,
all host threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

Q_HEADS, KV_HEADS, HEAD, BLOCK = 32, 8, 128, 16
BATCH, CTX_LO, CTX_HI, LAYERS = 64, 128, 4096, 36
ROPE_THETA = 1e6
SEED = 2024
METRIC = "paged decode attn KV-read HBM GB/s"


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def tensor_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return float(d["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json bf16_tflops_sustained)"
    return 1400.0, "fallback (1.4 PFLOP/s sustained, earlier measurement on this pool)"


def make_lens(seed, batch=BATCH):
    rng = np.random.default_rng(seed)
    return rng.integers(CTX_LO, CTX_HI + 1, size=batch).astype(np.int32)


def kv_bytes_per_layer(lens_after_append):
    """Algorithmic KV bytes one decode launch must read: every cached token's K and V row."""
    return int(np.sum(lens_after_append)) * KV_HEADS * HEAD * 2 * 2


class ClockSampler(threading.Thread):
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self._halt = index, [], threading.Event()

    def run(self):
        while not self._halt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True,
                                     timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self._halt.wait(0.05)

    def stop(self):
        self._halt.set()
        self.join(timeout=6)
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for k, n in enumerate(names) if any(len(r) > 3 + k and r[3 + k].lower() == "active" for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


class DecodeWorkload:
    """Per-GPU state of the headline workload, resident in HBM."""

    def __init__(self, rank, total_steps, device, chains=1, fused=True, world=1, use_plan=False):
        import torch
        self.chains, self.fused = chains, fused
        self.use_plan = use_plan and not fused  # (the one-launch step takes no plan)
        self.per_layer = 1 if fused else 2
        from orinmllm_b200 import capi
        self.torch, self.capi, self.dev = torch, capi, device
        # weak scaling: one global draw of 64 x N requests, dealt to the ranks by KV bytes (longest
        # first to the least loaded rank, 64 requests each): every GPU gets the same batch size and
        # nearly the same bytes, but its own lengths.  N = 1 is the plain 64-request draw.
        from orinmllm_b200 import multigpu
        all_lens = make_lens(SEED, BATCH * world)
        mine = multigpu.deal_requests_by_load(all_lens, world, equal_counts=True)[rank]
        self.lens0 = np.ascontiguousarray(all_lens[mine])
        rng = np.random.default_rng(SEED + 1000 * rank + 1)
        final = self.lens0 + total_steps
        nblk = (final + BLOCK - 1) // BLOCK
        self.num_blocks = int(np.ceil(int(nblk.sum()) * 1.25))
        perm = rng.permutation(self.num_blocks).astype(np.int32)
        self.max_blocks = int(nblk.max())
        table = np.full((BATCH, self.max_blocks), -1, np.int32)
        c = 0
        for i, n in enumerate(nblk):
            table[i, :n] = perm[c:c + n]
            c += n
        steps = np.arange(total_steps, dtype=np.int64)
        pos = self.lens0[None, :].astype(np.int64) + steps[:, None]             # [T, B]
        blk = table[np.arange(BATCH)[None, :], pos // BLOCK].astype(np.int64)
        self.table = torch.from_numpy(table).to(device)
        self.slots = torch.from_numpy(blk * BLOCK + pos % BLOCK).to(device)     # [T, B] int64
        self.positions = torch.from_numpy(pos.astype(np.int32)).to(device)      # [T, B] int32
        self.layout = capi.layout_paged(capi.KPX_F16, KV_HEADS, HEAD, BLOCK, self.num_blocks)
        g = torch.Generator(device=device)
        g.manual_seed(SEED + rank)
        shape = (LAYERS, self.num_blocks, KV_HEADS, BLOCK, HEAD)
        self.k_pool = torch.empty(shape, dtype=torch.float16, device=device)
        self.v_pool = torch.empty(shape, dtype=torch.float16, device=device)
        for l in range(LAYERS):
            self.k_pool[l].normal_(generator=g)
            self.v_pool[l].normal_(generator=g)
        # a layer's new q, k and v rows lie one after the other (q block, k block, v block), on the
        # device and in the pinned host copy alike, so that a layer's rows arrive in one copy
        nq, nkv = BATCH * Q_HEADS * HEAD, BATCH * KV_HEADS * HEAD
        self.qkv = torch.randn(LAYERS, nq + 2 * nkv, generator=g, dtype=torch.float16, device=device)
        self.q = self.qkv[:, :nq].unflatten(1, (BATCH, Q_HEADS * HEAD))
        self.k = self.qkv[:, nq:nq + nkv].unflatten(1, (BATCH, KV_HEADS * HEAD))
        self.v = self.qkv[:, nq + nkv:].unflatten(1, (BATCH, KV_HEADS * HEAD))
        self.out = torch.empty_like(self.q)
        max_pos = int(final.max()) + 1
        self.sin = torch.empty(max_pos, HEAD, dtype=torch.float32, device=device)
        self.cos = torch.empty(max_pos, HEAD, dtype=torch.float32, device=device)
        capi.sin_cos_cache(self.sin, self.cos, HEAD, max_pos, ROPE_THETA)
        self.ws_bytes = capi.decode_workspace_bytes(BATCH, Q_HEADS, KV_HEADS, HEAD)
        # launches that may overlap on the GPU (layers captured on parallel chains) need a
        # workspace each
        self.wss = [torch.empty(self.ws_bytes, dtype=torch.uint8, device=device) for _ in range(max(1, chains))]
        for w in self.wss:
            capi.workspace_init(w, self.ws_bytes)
        self.ws = self.wss[0]
        self.plan = torch.zeros(capi.decode_plan_bytes(), dtype=torch.uint8, device=device)
        self.scale = 1.0 / float(np.sqrt(HEAD))
        self.launches = 0
        # host side of the end-to-end path
        self.h_qkv = self.qkv.cpu().pin_memory()
        self.h_out = torch.empty(LAYERS, BATCH, Q_HEADS * HEAD, dtype=torch.float16).pin_memory()
        self._prepare_pointers()
        torch.cuda.synchronize(device)

    def _prepare_pointers(self):
        """Raw device addresses, so the per-layer host work is two C calls and nothing else."""
        self.p_kpool = [self.k_pool[l].data_ptr() for l in range(LAYERS)]
        self.p_vpool = [self.v_pool[l].data_ptr() for l in range(LAYERS)]
        self.p_q = [self.q[l].data_ptr() for l in range(LAYERS)]
        self.p_k = [self.k[l].data_ptr() for l in range(LAYERS)]
        self.p_v = [self.v[l].data_ptr() for l in range(LAYERS)]
        self.p_out = [self.out[l].data_ptr() for l in range(LAYERS)]
        self.p_pos, self.p_slots = self.positions.data_ptr(), self.slots.data_ptr()
        self.p_sin, self.p_cos = self.sin.data_ptr(), self.cos.data_ptr()
        self.p_table, self.p_ws = self.table.data_ptr(), self.ws.data_ptr()
        self.stream = self.torch.cuda.current_stream().cuda_stream
        # the step a CUDA graph works on: positions and slots of the current step, refreshed by
        # two small device-to-device copies before each replay
        self.cur_pos = self.torch.empty(BATCH, dtype=self.torch.int32, device=self.dev)
        self.cur_slots = self.torch.empty(BATCH, dtype=self.torch.int64, device=self.dev)
        self.graph_resident = self.graph_e2e = None

    def layer(self, t, l, events=None, stream=None, ws=None, flags=0, plan=None):
        """RoPE + append + attend of layer l.  t: step index into the precomputed positions and
        slots, or None for the current-step buffers (graph capture)."""
        capi = self.capi
        stream = self.stream if stream is None else stream
        pos = self.cur_pos.data_ptr() if t is None else self.p_pos + t * BATCH * 4
        slots = self.cur_slots.data_ptr() if t is None else self.p_slots + t * BATCH * 8
        if self.fused:
            # one launch per layer: RoPE of the new rows, append, attention over cached + new
            if events is not None:
                events[0].record()
            capi.rope_append_decode(self.p_out[l], self.p_q[l], self.p_k[l], self.p_v[l], self.p_sin, self.p_cos,
                                    self.p_kpool[l], self.p_vpool[l], self.layout, self.p_table, self.max_blocks,
                                    pos, BATCH, Q_HEADS, self.scale, self.p_ws if ws is None else ws,
                                    self.ws_bytes, flags, stream=stream)
            if events is not None:
                events[1].record()
            self.launches += 1
            return
        capi.rope_append(self.p_q[l], self.p_k[l], self.p_v[l], Q_HEADS, pos, self.p_sin, self.p_cos,
                         self.p_kpool[l], self.p_vpool[l], self.layout, slots, BATCH, stream=stream)
        if events is not None:
            events[0].record()
        # tokens cached before the step + 1 appended = attended length (len_bias = 1)
        if plan is not None:
            # the step's plan (made once per step, see capture): the same launch, shorter prologue
            capi.paged_decode_planned(self.p_out[l], self.p_q[l], self.p_kpool[l], self.p_vpool[l], self.layout,
                                      self.p_table, self.max_blocks, pos, 1, BATCH, Q_HEADS, self.scale,
                                      self.p_ws if ws is None else ws, self.ws_bytes, plan, flags, stream=stream)
        else:
            decode = capi.paged_decode_overlapped if flags & capi.KPX_DECODE_OVERLAPPED else capi.paged_decode
            decode(self.p_out[l], self.p_q[l], self.p_kpool[l], self.p_vpool[l], self.layout,
                   self.p_table, self.max_blocks, pos, 1, BATCH, Q_HEADS, self.scale,
                   self.p_ws if ws is None else ws, self.ws_bytes, stream=stream)
        if events is not None:
            events[1].record()
        self.launches += 2

    def step_resident(self, t, event_sink=None):
        for l in range(LAYERS):
            ev = None
            if event_sink is not None:
                ev = (self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True))
                event_sink.append(ev)
            self.layer(t, l, ev)

    def step_e2e(self, t):
        # Q/K/V rows of the step come from pinned host memory, outputs return to it
        for l in range(LAYERS):
            self.qkv[l].copy_(self.h_qkv[l], non_blocking=True)
            self.layer(t, l)
            self.h_out[l].copy_(self.out[l], non_blocking=True)

    # ---- the same steps as CUDA graphs (captured once, replayed per step) ----
    def _set_step(self, t):
        self.cur_pos.copy_(self.positions[t], non_blocking=True)
        self.cur_slots.copy_(self.slots[t], non_blocking=True)

    def capture(self):
        """Captures the resident step and the end-to-end step (the same launches with every
        layer's host->device and device->host copies on side streams, so that copies of one
        layer run under the kernels of its neighbours).  Consecutive layers of this workload are
        independent (own pool, own rows, own output), so layer l is captured on chain l % chains
        with that chain's workspace: a layer's CTAs take over the SMs as the previous layer's
        CTAs retire instead of waiting for its last warp.  Capture executes nothing."""
        torch = self.torch
        main, h2d, d2h = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)
        side = [torch.cuda.Stream(self.dev) for _ in range(self.chains)] if self.chains > 1 else [main]
        flags = self.capi.KPX_DECODE_OVERLAPPED if self.chains > 1 else 0
        count = self.launches

        plan = self.plan.data_ptr() if self.use_plan else None

        def make_plan():
            # one small launch per step: lengths and table are the same for all 36 layers
            if plan is not None:
                self.capi.decode_plan(plan, self.plan.numel(), self.layout, self.p_table, self.max_blocks,
                                      self.cur_pos.data_ptr(), 1, BATCH, Q_HEADS, stream=main.cuda_stream)

        def run_layer(l):
            c = l % len(side)
            self.layer(None, l, stream=side[c].cuda_stream, ws=self.wss[c].data_ptr(), flags=flags, plan=plan)
            return side[c]

        self.graph_resident = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph_resident, stream=main):
            make_plan()
            for s_ in side:
                if s_ is not main:
                    s_.wait_stream(main)
            for l in range(LAYERS):
                run_layer(l)
            for s_ in side:
                if s_ is not main:
                    main.wait_stream(s_)
        self.graph_e2e = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph_e2e, stream=main):
            make_plan()
            for s_ in [h2d, d2h] + [x for x in side if x is not main]:
                s_.wait_stream(main)
            for l in range(LAYERS):
                with torch.cuda.stream(h2d):
                    self.qkv[l].copy_(self.h_qkv[l], non_blocking=True)
                side[l % len(side)].wait_stream(h2d)
                ran_on = run_layer(l)
                d2h.wait_stream(ran_on)
                with torch.cuda.stream(d2h):
                    self.h_out[l].copy_(self.out[l], non_blocking=True)
            for s_ in [h2d, d2h] + [x for x in side if x is not main]:
                main.wait_stream(s_)
        self.launches = count  # capture launched nothing

    def replay_resident(self, t):
        self._set_step(t)
        self.graph_resident.replay()
        self.launches += self.per_layer * LAYERS + (1 if self.use_plan else 0)

    def replay_e2e(self, t):
        self._set_step(t)
        self.graph_e2e.replay()
        self.launches += self.per_layer * LAYERS + (1 if self.use_plan else 0)

    def kv_bytes_step(self, t):
        return kv_bytes_per_layer(self.lens0 + t + 1) * LAYERS

    def h2d_bytes_per_step(self):
        return LAYERS * BATCH * (Q_HEADS + 2 * KV_HEADS) * HEAD * 2

    def d2h_bytes_per_step(self):
        return LAYERS * BATCH * Q_HEADS * HEAD * 2


# ------------------------------------------------- the path's other kernels, same run
def _median_ms(torch, fn, reps, flush=None):
    ms = []
    for _ in range(reps):
        if flush is not None:
            flush.sum()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    return float(np.median(ms))


def extra_prefill(torch, capi, dt=None):
    """Chunked prefill at the Qwen2.5-7B attention shape (28 Q / 4 KV heads, d 128, bf16, block 16):
    4 sequences of 2048-token prompts in 512-token chunks, seeded random block placement.  Device
    time of the four chunk calls of a layer (each queued several times back to back behind a
    filler kernel, CUDA events around the queue), FLOPs counted causal-exact.  The same with fp16
    pools (one 16-bit term for the softmax weights instead of two) is reported under "fp16"."""
    H, HKV, D, BS, B, PROMPT, CHUNK = 28, 4, HEAD, BLOCK, 4, 2048, 512
    rng = np.random.default_rng(3)
    nb = int(B * PROMPT / BS * 1.25)
    table = rng.permutation(nb).astype(np.int32)[:B * PROMPT // BS].reshape(B, PROMPT // BS).copy()
    first = dt is None
    dt = torch.bfloat16 if dt is None else dt
    kp = torch.randn(nb, HKV, BS, D, device="cuda", dtype=dt)
    vp = torch.randn(nb, HKV, BS, D, device="cuda", dtype=dt)
    q = torch.randn(B * CHUNK, H * D, device="cuda", dtype=dt)
    out = torch.empty_like(q)
    lay = capi.layout_paged(capi.dtype_code(dt), HKV, D, BS, nb)
    bt = torch.from_numpy(table).cuda()
    cu = (np.arange(B + 1) * CHUNK).astype(np.int32)
    nbytes = capi.prefill_workspace_bytes(B * CHUNK, H, HKV, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.workspace_init(ws, nbytes)
    nch = PROMPT // CHUNK
    flops = [B * 4.0 * H * D * sum(c * CHUNK + i + 1 for i in range(CHUNK)) for c in range(nch)]
    starts = [np.full(B, c * CHUNK, np.int32) for c in range(nch)]
    call = lambda c: capi.paged_prefill(out, q, kp, vp, lay, bt, table.shape[1], cu, starts[c], B, H,
                                        1 / np.sqrt(D), ws, nbytes)
    for c in range(nch):
        call(c)
    torch.cuda.synchronize()
    filler = torch.empty(1 << 27, dtype=torch.float32, device="cuda")
    queued, total_ms = 10, 0.0
    for c in range(nch):
        for _ in range(3):
            filler.add_(1.0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(queued):
            call(c)
        e1.record()
        torch.cuda.synchronize()
        total_ms += e0.elapsed_time(e1) / queued
    status = capi.workspace_status(ws)
    peak, src = tensor_peak()
    tflops = sum(flops) / total_ms / 1e9
    res = {"workload": "chunked prefill, 28 Q / 4 KV heads, %s, 4 x 2048 tokens in chunks of 512" % (
               "bf16" if dt == torch.bfloat16 else "fp16"),
           "kernel": "prefill_tc_kernel", "tflops": round(tflops, 1), "frac_of_sustained": round(tflops / peak, 4),
           "peak_tflops": peak, "peak_source": src, "us_per_layer": round(total_ms * 1e3, 1),
           "flops_per_layer": sum(flops), "launches": queued * nch, "status": status}
    if first:
        del kp, vp, q, out, ws, filler
        res["fp16"] = {k: v for k, v in extra_prefill(torch, capi, torch.float16).items()
                       if k in ("tflops", "frac_of_sustained", "us_per_layer", "status")}
    return res


def extra_append(torch, capi):
    """kpx_append and kpx_rope_append alone on 131 072 tokens at the Qwen3-8B shape (fp16, new rows
    filling whole blocks at seeded random places in the pool): bytes read + written / device time,
    L2 flushed before each launch."""
    n, HKV, H, D, BS = 131072, KV_HEADS, Q_HEADS, HEAD, BLOCK
    rng = np.random.default_rng(77)
    nb = int(np.ceil(n / BS * 1.25))
    kp = torch.zeros(nb, HKV, BS, D, device="cuda", dtype=torch.float16)
    vp = torch.zeros_like(kp)
    lay = capi.layout_paged(capi.KPX_F16, HKV, D, BS, nb)
    max_pos = 4096
    sin = torch.empty(max_pos * D, device="cuda", dtype=torch.float32)
    cos = torch.empty_like(sin)
    capi.sin_cos_cache(sin, cos, D, max_pos, ROPE_THETA)
    blocks = rng.permutation(nb)[:n // BS].astype(np.int64)
    slots = torch.from_numpy((blocks[:, None] * BS + np.arange(BS)[None, :]).reshape(-1)).cuda()
    pos = torch.from_numpy((np.arange(n) % max_pos).astype(np.int32)).cuda()
    q = torch.randn(n, H * D, device="cuda", dtype=torch.float16)
    k = torch.randn(n, HKV * D, device="cuda", dtype=torch.float16)
    v = torch.randn(n, HKV * D, device="cuda", dtype=torch.float16)
    flush = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")
    peak, src = peaks()
    t_plain = _median_ms(torch, lambda: capi.append(kp, vp, lay, k, v, slot_mapping=slots, num_tokens=n), 7, flush)
    b_plain = n * HKV * D * 2 * 2 * 2
    t_rope = _median_ms(torch, lambda: capi.rope_append(q, k, v, H, pos, sin, cos, kp, vp, lay, slots, n), 7, flush)
    b_rope = n * D * 2 * ((H + 2 * HKV) + (H + HKV) + 2 * HKV)
    return {"workload": "131072 tokens, 8 KV heads x 128, fp16, block 16, random block placement",
            "kernel": "append_token_kernel", "gbs": round(b_plain / t_plain / 1e6, 1),
            "frac": round(b_plain / t_plain / 1e6 / peak, 4), "us": round(t_plain * 1e3, 1), "bytes": b_plain,
            "rope_append": {"kernel": "rope_append_kernel", "gbs": round(b_rope / t_rope / 1e6, 1),
                            "frac": round(b_rope / t_rope / 1e6 / peak, 4), "us": round(t_rope * 1e3, 1),
                            "bytes": b_rope},
            "peak": peak, "peak_source": src}


def extra_prefix_reuse(torch, capi):
    """256 requests sharing a 1024-token prefix + 256 own tokens, 128 decode steps each, through
    the request scheduler on 2 layers (Qwen3-8B attention shape, fp16, block 16): pool usage with
    and without sharing, copy-on-write events, and the decode kernel's algorithmic KV GB/s on the
    full-batch steps (CUDA events around each decode launch; the median launch)."""
    from tests.serving_sim import ServingSim
    prefix, suffix, n_req, gen, layers = 1024, 256, 256, 129, 2
    sim = ServingSim(layers, Q_HEADS, KV_HEADS, num_blocks=8192, seed=7, max_positions=2048, prefill_chunk=512,
                     max_prefill_tokens=4096, max_decode_batch=256)
    rng = np.random.default_rng(4)
    common = rng.integers(0, 151936, prefix)
    sim.sched.submit(np.concatenate([common, rng.integers(0, 151936, suffix)]), 1, also_register=prefix)
    sim.run()
    for _ in range(n_req - 1):
        sim.sched.submit(np.concatenate([common, rng.integers(0, 151936, suffix)]), gen)
    sim.decode_events = []
    sim.run()
    st = sim.sched.stats()
    ev = [(e0.elapsed_time(e1), b) for e0, e1, b in sim.decode_events]
    top = max(b for _, b in ev)
    ev = [(m, b) for m, b in ev if b >= 0.9 * top]
    peak, _ = peaks()
    gbs = float(np.median([b / m for m, b in ev])) / 1e6
    return {"workload": "256 requests = 1024 shared + 256 own tokens, 128 decode steps, 2 layers, bs 255",
            "blocks_in_use": int(st["peak_blocks_in_use"]),
            "blocks_unshared": n_req * ((prefix + suffix + gen - 1 + BLOCK - 1) // BLOCK),
            "reused_tokens": int(st["reused_tokens"]), "cow_events": int(sim.manager.cow_events),
            "decode_gbs": round(gbs, 1), "decode_frac": round(gbs / peak, 4),
            "decode_launch_us": round(float(np.median([m for m, _ in ev])) * 1e3, 1),
            "decode_launches_timed": len(ev), "kv_bytes_per_launch": int(np.mean([b for _, b in ev]))}


# ------------------------------------------------------------------ CPU legs (oracle)
def cpu_decode_sample(threads, reps, seed=SEED):
    """Times the CPU restatement of the reference's fp32 MHA path (the oracle: test
    infrastructure, used here only as the reported baseline) on ONE layer of the workload:
    all 64 sequences, fp32 pools gathered through the block table.  Returns GB/s in the same
    algorithmic bytes as the GPU arm (fp16 K+V rows of every cached token)."""
    from tests import kvtest
    orc = kvtest.load_oracle()
    lens = make_lens(seed) + 1
    rng = np.random.default_rng(seed + 7)
    nblk = (lens + BLOCK - 1) // BLOCK
    num_blocks = int(np.ceil(int(nblk.sum()) * 1.25))
    perm = rng.permutation(num_blocks).astype(np.int32)
    table = np.zeros((BATCH, int(nblk.max())), np.int32)
    c = 0
    for i, n in enumerate(nblk):
        table[i, :n] = perm[c:c + n]
        c += n
    kp = rng.standard_normal((num_blocks, KV_HEADS, BLOCK, HEAD), np.float32)
    vp = rng.standard_normal((num_blocks, KV_HEADS, BLOCK, HEAD), np.float32)
    q = rng.standard_normal((BATCH, Q_HEADS * HEAD), np.float32)
    orc.paged_decode(q[:2], kp, vp, table[:2], lens[:2], Q_HEADS, KV_HEADS, HEAD, BLOCK, threads)  # warm
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        orc.paged_decode(q, kp, vp, table, lens, Q_HEADS, KV_HEADS, HEAD, BLOCK, threads)
        times.append(time.perf_counter() - t0)
    nbytes = kv_bytes_per_layer(lens)
    return nbytes / 1e9 / float(np.mean(times)), float(np.mean(times)), nbytes


def cpu_reference_sample(threads, reps, seed=SEED):
    """Times the REFERENCE's own CPU MHA (kernel::mha_kernel and the matmul / softmax / scale-sum
    kernels it calls, compiled unmodified into oracle/_ref/libref_cpu.so) on one layer of the
    workload.  The reference serves one sequence at a time from a contiguous fp32 cache, so every
    sequence's K/V is laid out that way beforehand (untimed) and the 64 single-sequence calls are
    spread over `threads` host threads.  Returns None where the library has not been built."""
    from concurrent.futures import ThreadPoolExecutor
    from tests import refcpu
    ref = refcpu.load(sequential=False)
    if ref is None:
        return None
    lens = make_lens(seed) + 1
    rng = np.random.default_rng(seed + 7)
    kv_dim = KV_HEADS * HEAD
    caches = [(rng.standard_normal((1, int(n), kv_dim), np.float32), rng.standard_normal((1, int(n), kv_dim), np.float32))
              for n in lens]
    q = rng.standard_normal((BATCH, Q_HEADS * HEAD), np.float32)

    def one(b):
        n = int(lens[b])
        return ref.mha(n - 1, Q_HEADS, 0, n, kv_dim, Q_HEADS // KV_HEADS, HEAD, 1, q[b], caches[b][0], caches[b][1])

    one(int(np.argmin(lens)))  # first call creates the reference's allocator singleton
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        if threads == 1:
            for b in range(BATCH):
                one(b)
        else:
            with ThreadPoolExecutor(max_workers=threads) as pool:
                list(pool.map(one, range(BATCH)))
        times.append(time.perf_counter() - t0)
    nbytes = kv_bytes_per_layer(lens)
    return nbytes / 1e9 / float(np.mean(times)), float(np.mean(times)), nbytes


def run_reference(args):
    """Reference arm: the reference's own CPU implementation of the path on the host cores.  Where
    oracle/_ref/libref_cpu.so exists (the reference's cpu/*.cpp compiled unmodified against the
    glog / Armadillo stand-ins) that is what is timed, else its plain-C restatement under
    oracle/.  One step = one layer of the workload (a bounded sample of the 36), all host
    threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # all host cores this process may run on (torchrun presets OMP_NUM_THREADS=1, so the OpenMP
    # default would be a single thread)
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    got = cpu_reference_sample(threads, max(1, args.steps))
    kind = "reference"
    if got is None:
        got, kind = cpu_decode_sample(threads, max(1, args.steps)), "port"
    gbs, sec, nbytes = got
    what = ("kernel::mha_kernel of the reference (compiled from its sources), one call per sequence over a "
            "contiguous fp32 cache") if kind == "reference" else "fp32 oracle (plain-C restatement)"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "paged GQA decode, Qwen3-8B attention shape, bs=64, ctx U[128,4096], block 16",
                   "sample": "1 of 36 layers per step, all 64 sequences"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": kind,
                         "sample": "one layer (all 64 sequences, %d KV bytes) per step; %s" % (nbytes, what)},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tokens_per_s": round(BATCH / (sec * LAYERS), 3),
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm
def run_gpu(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    from orinmllm_b200 import build
    if not (build.LIB / "libkpx.so").exists():
        build.build_all()
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    W, K = args.warmup, args.steps
    use_graph = not args.no_graph
    total_steps = 2 * (W + K) + K + 2
    wl = DecodeWorkload(rank, total_steps, device, chains=max(1, args.chains) if use_graph else 1,
                        fused=args.fused, world=world, use_plan=use_graph and not args.no_plan)
    if args.variant:
        wl.capi.lib().kpx_internal_set_decode_variant(args.variant)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    from orinmllm_b200 import multigpu

    def max_over_ranks(ms):
        return multigpu.max_over_ranks(ms, world, device)

    sampler = ClockSampler(local) if rank == 0 else None
    t = 0
    wl.step_resident(t)  # first-use work (attributes, module load) before any capture
    t += 1
    if use_graph:
        torch.cuda.synchronize(device)
        wl.capture()
    resident = wl.replay_resident if use_graph else wl.step_resident
    end_to_end = wl.replay_e2e if use_graph else wl.step_e2e
    # ---- device-resident phase ----
    for _ in range(W):
        resident(t)
        t += 1
    barrier()
    if sampler:
        sampler.start()
    wl.launches = 0
    pairs = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    bytes_resident = 0
    e0.record()
    for _ in range(K):
        if use_graph:
            resident(t)
        else:
            wl.step_resident(t, pairs)
        bytes_resident += wl.kv_bytes_step(t)
        t += 1
    e1.record()
    barrier()
    ms_resident = max_over_ranks(e0.elapsed_time(e1))
    launches = wl.launches
    if use_graph:
        # kernels inside a graph cannot be bracketed by events: the per-launch durations of the
        # roofline come from the same K steps launched one by one right after the timed replays
        for _ in range(K):
            wl.step_resident(t, pairs)
            t += 1
        barrier()
    decode_ms = [a.elapsed_time(b) for a, b in pairs]
    # ---- end-to-end phase (host buffers) ----
    wl.step_e2e(t)
    t += 1
    for _ in range(W):
        end_to_end(t)
        t += 1
    barrier()
    bytes_e2e = 0
    e0.record()
    for _ in range(K):
        end_to_end(t)
        bytes_e2e += wl.kv_bytes_step(t)
        t += 1
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if sampler else None
    for w in wl.wss:
        status = wl.capi.workspace_status(w)
        if status != 0:
            raise SystemExit(f"device status {status}: {wl.capi.status_string(status)}")
    # whole-job totals (every rank holds the same amount of work: weak scaling)
    tot = multigpu.sum_over_ranks([bytes_resident, bytes_e2e], world, device)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_src = peaks()
    value = tot[0] / 1e9 / (ms_resident / 1e3)
    e2e = tot[1] / 1e9 / (ms_e2e / 1e3)
    per_launch_bytes = bytes_resident / (K * LAYERS)
    # Per-launch duration inside the timed region: the region holds K x 36 decode launches (and
    # their small RoPE+append launches) and nothing else, so region time / launches is the
    # average a decode launch takes there.  Launches of neighbouring layers overlap, which
    # is why this is shorter than one launch timed alone (reported beside it).
    in_region_ms = ms_resident / (K * LAYERS)
    achieved = per_launch_bytes / 1e9 / (in_region_ms / 1e3)
    isolated_ms = float(np.mean(decode_ms))
    isolated = per_launch_bytes / 1e9 / (isolated_ms / 1e3)
    got = cpu_reference_sample(1, 1)
    cpu_kind = "reference"
    if got is None:
        got, cpu_kind = cpu_decode_sample(1, 3), "port"
    cpu_gbs, cpu_sec, cpu_bytes = got
    chains = wl.chains if use_graph else 1
    kernels = wl.per_layer * LAYERS + (1 if wl.use_plan else 0)
    launch = ("one CUDA graph replay per step: %d kernels%s, layer l on chain l %% %d (layers are independent: own pool, "
              "own rows, own workspace per chain), so a layer's CTAs take the SMs the previous layer's CTAs leave; "
              "end to end: plus 36 H2D and 36 D2H copies on side streams"
              % (kernels, " (the first one plans the step's 36 decode launches: kpx_decode_plan)" if wl.use_plan else "",
                 chains)) if use_graph \
        else "one launch per kernel, one stream"
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": round(ms_resident / K, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 storage, f32 arithmetic", "data": "synthetic",
        "config": {"workload": "paged GQA decode, Qwen3-8B attention shape (32 Q / 8 KV heads, d=128), "
                               "fp16 KV, block 16, bs=64 per GPU, ctx U[128,4096], pool x1.25, "
                               "seeded random block table; step = RoPE+append+attend over 36 layers",
                   "layers": LAYERS, "batch_per_gpu": BATCH,
                   "partition": "by request, no collective: one global draw of 64 x N requests dealt to the ranks "
                                "by KV bytes, 64 each",
                   "l2": "inputs larger than L2: every layer has its own 0.66 GB pool",
                   "launch": launch, "kernels_per_layer": wl.per_layer, "chains": chains},
        "tokens_per_s": round(world * BATCH / (ms_resident / K / 1e3), 1),
        "pct_of_8TBs_per_gpu": round(100 * value / world / 8000.0, 2),
        "e2e": {"value": round(e2e, 1), "unit": "GB/s", "h2d_bytes_per_step": wl.h2d_bytes_per_step(),
                "d2h_bytes_per_step": wl.d2h_bytes_per_step(), "ms_per_step": round(ms_e2e / K, 4),
                "tokens_per_s": round(world * BATCH / (ms_e2e / K / 1e3), 1)},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": "paged_decode_kernel", "achieved": round(achieved, 1),
                     "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "avg_launch_us": round(in_region_ms * 1e3, 2),
                     "timed": "CUDA events around the timed region / decode launches inside it (launches of "
                              "neighbouring layers overlap; the layer's RoPE+append launch is inside too)",
                     "isolated": {"launch_us": round(isolated_ms * 1e3, 2), "achieved": round(isolated, 1),
                                  "frac": round(isolated / peak, 4),
                                  "timed": ("CUDA events around each decode launch of K steps launched one by one, "
                                            "nothing else on the GPU, right after the timed region; launch latency "
                                            "included")},
                     "algorithmic_bytes_per_launch": int(per_launch_bytes),
                     "traffic": int(per_launch_bytes * TRAFFIC_RATIO), "traffic_note": TRAFFIC_NOTE},
        "cpu_baseline": {"value": round(cpu_gbs, 3), "unit": "GB/s", "cores": 1, "kind": cpu_kind,
                         "sample": "one layer of the workload (64 sequences, %d KV bytes), %s, %.2f s" % (
                             cpu_bytes, "the reference's own kernel::mha_kernel compiled from its sources, one "
                             "call per sequence" if cpu_kind == "reference" else "fp32 oracle, mean of 3 runs", cpu_sec)},
        "clocks": clocks,
    }
    if world == 1 and not args.no_extras:
        # the path's other kernels, measured in this same run after the headline
        del wl
        torch.cuda.empty_cache()
        from orinmllm_b200 import capi
        for key, fn in (("prefill", extra_prefill), ("append", extra_append), ("prefix_reuse", extra_prefix_reuse)):
            try:
                line[key] = fn(torch, capi)
            except Exception as exc:  # the headline stands on its own
                line[key] = {"error": repr(exc)[:200]}
            torch.cuda.empty_cache()
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# dram bytes (read+write) / algorithmic bytes of one decode launch, from the ncu capture
# summarised in profiles/ (same kernel, same shape, one layer)
TRAFFIC_RATIO = 1.020
TRAFFIC_NOTE = ("ncu dram__bytes_read+write of one launch of the overlapped form at this shape / algorithmic "
                "bytes = 534.90 MB / 524.59 MB = 1.020 (the one-CTA-per-SM form: 1.017)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--chains", type=int, default=3,
                    help="parallel chains the graph's independent layers are captured on")
    ap.add_argument("--fused", action="store_true",
                    help="one launch per layer (kpx_rope_append_decode) instead of kpx_rope_append + kpx_paged_decode")
    ap.add_argument("--no-plan", action="store_true",
                    help="decode launches work out their starting points themselves (no kpx_decode_plan per step)")
    ap.add_argument("--variant", type=int, default=0, help="decode tuning variant (experiments)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the prefill / append / prefix-reuse measurements after the headline")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel separately instead of replaying CUDA graphs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
