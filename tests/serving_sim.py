"""Synthetic serving loop over the C ABI: the request scheduler (kpx_sched.h) drives RoPE+append,
chunked prefill and batched decode on per-layer block pools, with prefix sharing and
copy-on-write mirrored on the device.  There is no model: the Q/K/V rows of a token come from
seeded per-layer tables indexed by token id, so two requests that share a token prefix share
bit-identical K/V rows, and the "sampled" token is a fixed function of (request, step).

Test / measurement driver only (torch supplies device memory and table lookups); the product is
the library it calls.
"""
from __future__ import annotations

import numpy as np
import torch

from orinmllm_b200 import capi, kvm, sched


class ServingSim:
    def __init__(self, num_layers, q_heads, kv_heads, num_blocks, dtype=torch.float16, vocab=4096, seed=0,
                 max_positions=8192, prefill_chunk=512, max_prefill_tokens=2048, max_decode_batch=256,
                 use_prefix_cache=True, record=False, theta=1e6, poison=False, record_ids=None):
        self.L, self.H, self.HKV, self.D, self.BS = num_layers, q_heads, kv_heads, 128, 16
        self.nb, self.dtype, self.vocab = num_blocks, dtype, vocab
        self.scale = 1.0 / np.sqrt(self.D)
        g = torch.Generator(device="cuda").manual_seed(seed)
        dim, kvd = q_heads * self.D, kv_heads * self.D
        # token-id tables of the layers' q/k/v rows
        self.Eq = torch.randn(num_layers, vocab, dim, generator=g, device="cuda", dtype=torch.float32).to(dtype)
        self.Ek = torch.randn(num_layers, vocab, kvd, generator=g, device="cuda", dtype=torch.float32).to(dtype)
        self.Ev = torch.randn(num_layers, vocab, kvd, generator=g, device="cuda", dtype=torch.float32).to(dtype)
        shape = (num_layers, num_blocks, kv_heads, self.BS, self.D)
        if poison:  # NaN everywhere: any read of a slot nobody wrote shows up in the outputs
            self.kp = torch.full(shape, float("nan"), device="cuda", dtype=dtype)
            self.vp = torch.full(shape, float("nan"), device="cuda", dtype=dtype)
        else:
            self.kp = torch.zeros(shape, device="cuda", dtype=dtype)
            self.vp = torch.zeros(shape, device="cuda", dtype=dtype)
        self.layer_stride = num_blocks * kv_heads * self.BS * self.D
        self.layout = capi.layout_paged(capi.dtype_code(dtype), kv_heads, self.D, self.BS, num_blocks)
        self.sin = torch.empty(max_positions * self.D, device="cuda", dtype=torch.float32)
        self.cos = torch.empty_like(self.sin)
        capi.sin_cos_cache(self.sin, self.cos, self.D, max_positions, theta)
        self.refc = torch.zeros(num_blocks, dtype=torch.int32, device="cuda")
        self.errc = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.staging = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
        self.manager = kvm.KvManager(num_blocks, self.BS, seed=seed + 1)
        self.sched = sched.Scheduler(self.manager, prefill_chunk=prefill_chunk, max_prefill_tokens=max_prefill_tokens,
                                     max_decode_batch=max_decode_batch, use_prefix_cache=use_prefix_cache)
        self.ws_bytes = max(capi.prefill_workspace_bytes(max_prefill_tokens, q_heads, kv_heads, self.D),
                            capi.decode_workspace_bytes(max_decode_batch, q_heads, kv_heads, self.D))
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device="cuda")
        capi.workspace_init(self.ws, self.ws_bytes)
        self.plan = torch.zeros(capi.decode_plan_bytes(), dtype=torch.uint8, device="cuda")
        self.record = record
        self.record_ids = None if record_ids is None else set(int(r) for r in record_ids)  # None: every request
        self.outputs = {}       # request id -> {position: [L, dim] output rows (host, float32)} when record
        self.kv_bytes_decoded = 0   # algorithmic K/V bytes the decode launches had to read
        self.decode_launches = 0
        self.prefill_launches = 0
        self.steps = 0
        self.decode_events = None   # set to a list to collect (start, stop, algorithmic bytes) per decode launch

    # ---- one step of each kind --------------------------------------------------------------
    def _flush(self):
        # copy-on-write copies and reference counts reach the device before new rows land
        self.manager.flush_device(self.refc, self.errc, self.kp, self.vp, self.layout, self.L, self.layer_stride,
                                  self.staging, self.staging.numel())

    def _rows(self, ids_dev):
        return self.Eq[:, ids_dev], self.Ek[:, ids_dev], self.Ev[:, ids_dev]

    def run_prefill(self, p: sched.PrefillStep):
        self._flush()
        ids = torch.from_numpy(p.token_ids.astype(np.int64) % self.vocab).cuda()
        pos = torch.from_numpy(p.positions).cuda()
        slots = torch.from_numpy(p.slot_mapping).cuda()
        table = torch.from_numpy(p.block_table).cuda()
        q_all, k_all, v_all = self._rows(ids)
        n, rows = len(p.positions), len(p.request_ids)
        outs = []
        for l in range(self.L):
            q, k, v = q_all[l].contiguous(), k_all[l].contiguous(), v_all[l].contiguous()
            capi.rope_append(q, k, v, self.H, pos, self.sin, self.cos, self.kp[l], self.vp[l], self.layout, slots, n)
            out = torch.empty_like(q)
            capi.paged_prefill(out, q, self.kp[l], self.vp[l], self.layout, table, table.shape[1], p.cu_q_lens,
                               p.start_pos, rows, self.H, self.scale, self.ws, self.ws_bytes)
            self.prefill_launches += 1
            if self.record:
                outs.append(out.float().cpu().numpy())
        if self.record:
            for i, rid in enumerate(p.request_ids):
                if self.record_ids is not None and int(rid) not in self.record_ids:
                    continue
                a, b = p.cu_q_lens[i], p.cu_q_lens[i + 1]
                store = self.outputs.setdefault(int(rid), {})
                for t in range(a, b):
                    store[int(p.positions[t])] = np.stack([o[t] for o in outs])

    def run_decode(self, d: sched.DecodeStep):
        self._flush()
        ids = torch.from_numpy(d.token_ids.astype(np.int64) % self.vocab).cuda()
        pos = torch.from_numpy(d.positions).cuda()
        slots = torch.from_numpy(d.slot_mapping).cuda()
        table = torch.from_numpy(d.block_table).cuda()
        lens = torch.from_numpy(d.seq_lens).cuda()
        q_all, k_all, v_all = self._rows(ids)
        rows = len(d.request_ids)
        outs = []
        # the step's plan: lengths and table are the same for every layer of the step
        capi.decode_plan(self.plan, self.plan.numel(), self.layout, table, table.shape[1], lens, 0, rows, self.H)
        for l in range(self.L):
            q, k, v = q_all[l].contiguous(), k_all[l].contiguous(), v_all[l].contiguous()
            capi.rope_append(q, k, v, self.H, pos, self.sin, self.cos, self.kp[l], self.vp[l], self.layout, slots,
                             rows)
            out = torch.empty_like(q)
            if self.decode_events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            capi.paged_decode_planned(out, q, self.kp[l], self.vp[l], self.layout, table, table.shape[1], lens, 0,
                                      rows, self.H, self.scale, self.ws, self.ws_bytes, self.plan)
            if self.decode_events is not None:
                e1.record()
                self.decode_events.append((e0, e1, int(d.seq_lens.sum()) * self.HKV * self.D * self.kp.element_size() * 2))
            self.decode_launches += 1
            if self.record:
                outs.append(out.float().cpu().numpy())
        self.kv_bytes_decoded += int(d.seq_lens.sum()) * self.HKV * self.D * self.kp.element_size() * 2 * self.L
        if self.record:
            for i, rid in enumerate(d.request_ids):
                if self.record_ids is not None and int(rid) not in self.record_ids:
                    continue
                self.outputs.setdefault(int(rid), {})[int(d.positions[i])] = np.stack([o[i] for o in outs])

    @staticmethod
    def sample(rid, n_generated):
        """The "sampled" token: a fixed function of the request and how many it has generated."""
        return (rid * 7919 + n_generated * 104729 + 13) % 151936

    # ---- the loop --------------------------------------------------------------------------
    def run(self, decode_hook=None):
        s = self.sched
        gen = {}
        while s.num_waiting or s.num_running:
            s.admit()
            while True:
                p = s.next_prefill()
                if p is None:
                    break
                self.run_prefill(p)
                sampled = []
                for rid in p.request_ids:
                    sampled.append(self.sample(int(rid), gen.get(int(rid), 0)))
                for rid, c in zip(p.request_ids, p.completes):
                    if c:
                        gen[int(rid)] = gen.get(int(rid), 0) + 1
                s.complete_prefill(sampled)
            d = s.next_decode()
            if d is not None:
                if decode_hook:
                    decode_hook(d)
                self.run_decode(d)
                sampled = [self.sample(int(rid), gen.get(int(rid), 0)) for rid in d.request_ids]
                for rid in d.request_ids:
                    gen[int(rid)] = gen.get(int(rid), 0) + 1
                s.complete_decode(sampled)
            self.steps += 1
        torch.cuda.synchronize()
        status = capi.workspace_status(self.ws)
        if status != 0:
            raise RuntimeError(f"workspace status {status}: {capi.status_string(status)}")
        if int(self.errc.item()) != 0:
            raise RuntimeError("device reference counts went negative")
