#!/usr/bin/env python
"""Benchmark of the Adamas decode hot path on B200.

A "step" is one decode token's pass through the attention hot path of every layer of a
Llama-2-7B-shaped stack (32 layers, 32 heads x 128) at a 32K-token context with a token budget of
1024 and page size 16: per layer, fused append (Hadamard + 2-bit code + KV write), distance
estimate over the layer's code cache, top-k, sparse paged attention.  Every layer has its own KV
and code cache, so one step streams ~1.6 GB of distinct data (inputs far larger than L2).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Every timed step ADVANCES the sequence: step i appends at position ctx - 1 + i.  The step is one CUDA
graph (the kernels take the sequence length from device memory, see utils.decode_step_dev) that is
replayed; per step the host only reserves cache room, which uploads one page number every page_size
tokens.  The K timed steps are repeated in several blocks and the median block is reported.

N > 1 is launched by torch.distributed.run; each rank owns the same number of KV heads of a model
N times as wide (head sharding, no collective inside the path; the per-step gather of the layer
outputs is part of the step graph).  The line then also carries a "strong" record: the 32-head model
split N ways.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "sparse_attn_decode_hbm_GBps_at_32k"
UNIT = "GB/s"


# --------------------------------------------------------------------------------------------
# algorithmic bytes of one layer-step (read + written bytes each stage cannot avoid)
# --------------------------------------------------------------------------------------------
def stage_bytes(L: int, H: int, B: int, b: int = 1) -> dict:
    n = L - 1
    est = b * H * (n * 32 + 32 + n * 2)            # codes + query code in, 16-bit distances out
    topk = b * H * (n * 2 + (B - 1) * 4)           # distances in, indices out
    attn = b * H * (B * 512 + (B - 1) * 4 + 256 + 256)   # K,V rows + indices + q in, o out
    return dict(estimate=est, topk=topk, attention=attn, total=est + topk + attn)


# --------------------------------------------------------------------------------------------
# clocks during the timed region (NVML, read-only)
# --------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting",
        0x100: "display_clock_setting", 0x10: "sync_boost",
    }

    def __init__(self, index: int, period_s: float = 0.02):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._h = None
        self._period = period_s

    def _once(self):
        nv = self._nv
        try:
            self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
            try:
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
            except Exception:
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self._once()
            self._stop.wait(self._period)

    def start(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self) -> dict:
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._once()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# --------------------------------------------------------------------------------------------
# CPU arm: the reference's PyTorch decode path restated (oracle), timed on the host cores
# --------------------------------------------------------------------------------------------
def cpu_layer_step_setup(L, H, B, seed=0):
    from oracle import adamas_ref as ref
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(H, 128, generator=g).to(torch.float16).float()
    k = torch.randn(H, L, 128, generator=g).to(torch.float16).float()
    v = torch.randn(H, L, 128, generator=g).to(torch.float16).float()
    thresholds = torch.tensor([-10, 0, 10])
    k_code = torch.bucketize(torch.from_numpy(ref.fwht(k.numpy())), thresholds, out_int32=True)
    return ref, q, k, v, k_code


def time_cpu_reference(L, H, B, steps, warmup, budget_s=25.0):
    """Times one layer-step of the reference's PyTorch path (bucketize of the query ->
    pairwise_distance(p=1) against cached key codes -> topk(largest=False) -> masked fp32 softmax
    -> @V) with all host threads.  Returns (seconds per layer-step, number of timed runs)."""
    torch.set_num_threads(os.cpu_count() or 1)
    ref, q, k, v, k_code = cpu_layer_step_setup(L, H, B)
    for _ in range(max(1, warmup)):
        ref.literal_reference_decode(q, k, v, B, k_code=k_code)
    times = []
    t_begin = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        ref.literal_reference_decode(q, k, v, B, k_code=k_code)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > budget_s:
            break
    return sum(times) / len(times), len(times)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    L, H, B = args.ctx, args.heads, args.budget
    sec, n = time_cpu_reference(L, H, B, args.steps, args.warmup, budget_s=120.0)
    by = stage_bytes(L, H, B)
    value = by["total"] / sec / 1e9
    cores = torch.get_num_threads()
    sample = (f"{n} timed runs of ONE layer-step (1 of {args.layers} layers) of the reference PyTorch decode path "
              f"(cached key codes), ctx {L}, budget {B}, {H} heads, fp32, torch CPU")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": n, "warmup": max(1, args.warmup), "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "us_per_layer": sec * 1e6,
        "config": workload_config(args, extra={"arm": "oracle port of evaluation/adamas_attention.py:214-241 on host cores"}),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def two_launch_step(args) -> bool:
    """decode_step folds the append (and a rotation) into the estimate launch for 16, 32 or 64 heads."""
    return (not args.unfused) and args.heads in (16, 32, 64) and os.environ.get("ADAMAS_FUSED_APPEND", "1") != "0"


def launches_per_layer(args) -> int:
    return 4 if args.unfused else (2 if two_launch_step(args) else 3)


def workload_config(args, extra=None):
    cfg = {
        "workload": (f"llama2-7b-shaped attention stack: {args.layers} layers x {args.heads} heads x 128, "
                     f"ctx {args.ctx} growing by one token per step, token budget {args.budget}, page size "
                     f"{args.page_size}, batch 1; per layer: fused append + estimate + top-k + sparse paged attention "
                     + ("(4 launches)" if args.unfused else
                        ("(decode_step: 2 launches, append inside the estimate kernel, top-k and attention in one kernel)"
                         if two_launch_step(args) else "(decode_step: 3 launches, top-k and attention in one kernel)"))),
        "layers": args.layers, "heads_per_gpu": args.heads, "ctx": args.ctx, "budget": args.budget,
        "page_size": args.page_size, "parallelism": f"head-sharded x{args.gpus}" if args.gpus > 1 else "single GPU",
        "l2": "inputs larger than L2 (each layer has its own caches; ~1.6 GB touched per step)",
        "launch": ("eager" if args.eager else
                   ("CUDA graph of the four operators at a fixed position" if args.unfused else
                    "one CUDA graph of the step, replayed; every step appends at the next position "
                    "(sequence length in device memory)")),
        "timing": "median of several blocks of `steps` steps, CUDA events, max over ranks",
        "appended_tokens": ("the same q/k/v at every step" if getattr(args, "repeat_token", False) else
                            "a different key at every step (device copy of k rotated by one dimension per step; "
                            "the end-to-end leg cycles through 64 pinned host buffers)"),
    }
    if extra:
        cfg.update(extra)
    return cfg


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
class Workload:
    """One sequence of `ctx` tokens in every layer's caches, ready to decode `room` more tokens."""

    def __init__(self, args, dev, seed_offset=0, room=0, heads=None, ctx=None, budget=None, layers=None, dtype=None):
        import adamas_b200.utils as U
        self.U = U
        self.args = args
        self.dev = dev
        self.H = H = heads or args.heads
        self.L = L = ctx or args.ctx
        self.B = B = budget or args.budget
        self.layers = layers = layers or args.layers
        ps = args.page_size
        dtype = dtype or (torch.bfloat16 if getattr(args, "dtype", "f16") == "bf16" else torch.float16)
        self.dtype = dtype
        self.c = c = U.InferenceController(layers, H, 128, ps, B // ps, L + room + ps, dtype, dev)
        gen = torch.Generator(device=dev).manual_seed(1234 + int(os.environ.get("RANK", "0")) + 1000 * seed_offset)
        c.prepare_hadamard(L - 1)
        c.begin_forward(L - 1)
        for layer in range(layers):
            k = torch.randn(L - 1, H, 128, device=dev, dtype=dtype, generator=gen)
            v = torch.randn(L - 1, H, 128, device=dev, dtype=dtype, generator=gen)
            U.append_kvh(k, v, None, c, layer)
            del k, v
        c.end_forward()
        c.prepare_hadamard(1)
        c.begin_forward(1)
        assert c.need_estimate()
        # this step's projections: pinned host copies (end-to-end path) and device copies
        hg = torch.Generator().manual_seed(99 + seed_offset)
        self.h_qkv = torch.randn(3, layers, 1, H, 128, generator=hg).to(dtype).pin_memory()
        self.d_qkv = self.h_qkv.to(dev)
        # Every appended token differs from the one before: the keys of the device copy are rotated by one
        # dimension at the end of a step (two small launches), and the end-to-end leg cycles through a ring of
        # host buffers.  (The same key appended
        # hundreds of times would put hundreds of equal distances into one histogram bin per head, a pile of
        # same-address atomics that no real sequence produces.)
        # --yarn F: q and k arrive un-rotated and the step rotates them with a YaRN frequency table (factor F over
        # an original context of 4096)
        self.rope = None
        if getattr(args, "yarn", 0.0) > 0:
            from adamas_b200.rope import yarn_inv_freq
            inv_freq, mscale = yarn_inv_freq(float(args.yarn), 4096)
            self.rope = {"inv_freq": inv_freq.to(dev), "mscale": mscale}
        self.vary = not getattr(args, "repeat_token", False)
        self.d_tmp = torch.empty_like(self.d_qkv[1]) if self.vary else None
        self.roll_idx = torch.roll(torch.arange(128, device=dev), 1)
        self.h_ring = [self.h_qkv]
        self.e2e_i = 0
        self.d_out = torch.zeros(layers, 1, H, 128, dtype=dtype, device=dev)
        self.h_out = torch.zeros(layers, 1, H, 128, dtype=dtype).pin_memory()
        self.q_code = torch.zeros(layers, 1, H, 16, dtype=dtype, device=dev)
        self.graph = None
        self.advancing = False
        self.after_layers = None      # e.g. the gather of the layer outputs over the ranks

    # ---- the step at a FIXED position (host lengths): four separate operators, or one kernel class alone
    def layer_step(self, layer):
        U, c = self.U, self.c
        q, k, v = self.d_qkv[0, layer], self.d_qkv[1, layer], self.d_qkv[2, layer]
        if not self.args.unfused:
            U.decode_step(q, k, v, c, layer, out=self.d_out[layer], record_indices=False, rope=self.rope)
            return
        q_code = U.append_qkv_fused(q, k, v, c, layer, out=self.q_code[layer])
        est = U.decode_estimate(q_code, c, layer)
        U.decode_topk(est, c)
        U.decode_sparse_attn(q, c, layer, c.topk_dindices_buffer, out=self.d_out[layer])

    def step_fixed(self):
        for layer in range(self.layers):
            self.layer_step(layer)
        if self.after_layers is not None:
            self.after_layers()

    # ---- the step that advances (device-resident length): the public fused API, graph-replayable
    def step_body_dev(self):
        U, c = self.U, self.c
        for layer in range(self.layers):
            U.decode_step_dev(self.d_qkv[0, layer], self.d_qkv[1, layer], self.d_qkv[2, layer], c, layer,
                              out=self.d_out[layer], rope=self.rope)
        if self.after_layers is not None:
            self.after_layers()
        U.seq_len_advance(c)
        if self.vary:      # the next token's projections
            torch.index_select(self.d_qkv[1], -1, self.roll_idx, out=self.d_tmp)
            self.d_qkv[1].copy_(self.d_tmp)

    def host_advance(self):
        """What the host does per token: reserve cache room (one page number travels to the device
        every page_size tokens)."""
        c = self.c
        c.prepare_hadamard(1)
        c.kv_cache.table_all()
        c.hadamard_cache.table_all()

    def capture(self):
        """Captures the step as one CUDA graph.  Fused step: the advancing, device-length form (the
        warm-up runs are real tokens).  --unfused: the four host-length operators at a fixed position."""
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        self.advancing = not self.args.unfused
        with torch.cuda.stream(s):
            if self.advancing:
                self.c.sync_seq_len()
                self.step_body_dev()          # token at position ctx - 1
                self.host_advance()
                self.step_body_dev()
            else:
                self.step_fixed()
                self.step_fixed()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        if self.args.eager:
            return
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            if self.advancing:
                self.step_body_dev()
            else:
                self.step_fixed()

    def step(self):
        if self.advancing:
            self.host_advance()
            if self.graph is not None:
                self.graph.replay()
            else:
                self.step_body_dev()
        elif self.graph is not None:
            self.graph.replay()
        else:
            self.step_fixed()

    def step_e2e(self):
        """Host buffers in, host buffers out: H2D of this step's q/k/v, the step, D2H of the outputs."""
        if self.vary and len(self.h_ring) < 64:      # built on first use: 64 different tokens' projections, pinned
            g = torch.Generator().manual_seed(1234)
            while len(self.h_ring) < 64:
                self.h_ring.append(torch.randn(self.h_qkv.shape, generator=g).to(self.h_qkv.dtype).pin_memory())
        self.d_qkv.copy_(self.h_ring[self.e2e_i % len(self.h_ring)], non_blocking=True)
        self.e2e_i += 1
        self.step()
        self.h_out.copy_(self.d_out, non_blocking=True)

    def stage_op(self, stage, layer):
        """One kernel class of one layer at the fixed position the host holds."""
        U, c = self.U, self.c
        from adamas_b200 import _kernels as K
        q, k, v = self.d_qkv[0, layer], self.d_qkv[1, layer], self.d_qkv[2, layer]
        n = c.hadamard_cache.seqlen - 1
        kk = c.inference_token_budget - 1
        if stage == "step":
            self.layer_step(layer)
        elif stage == "append":
            U.append_qkv_fused(q, k, v, c, layer, out=self.q_code[layer])
        elif stage == "append_estimate":   # first launch of the two-launch step (it also fills the histograms)
            K.append_estimate(q, k, v, self.q_code[layer], c.kv_cache.buf_layer(layer), c.kv_indices_with_last,
                              c.kv_cache.last_page_len, c.hadamard_cache.buf_layer(layer), c.hadamard_indices,
                              c.hadamard_cache.last_page_len, c.distance_scratch(n), hist=c.hist_scratch,
                              hist_slices=K.select_attend_slices(n, kk, self.H))
        elif stage == "estimate" and self.args.unfused:
            U.decode_estimate(self.q_code[layer], c, layer)
        elif stage == "estimate":      # fused step: integer distances + histograms, as decode_step asks for
            K.estimate_attn_score(self.q_code[layer], c.distance_scratch(n), c.hadamard_cache.buf_layer(layer),
                                  c.hadamard_indices, None, c.hadamard_cache.last_page_len,
                                  c.hadamard_last_page_idx, c.layout, hist=c.hist_scratch,
                                  hist_slices=K.select_attend_slices(n, kk, self.H))
        elif stage == "topk":
            U.decode_topk(c.estimate_buffer(n), c)
        elif stage == "attention":
            U.decode_sparse_attn(q, c, layer, c.topk_dindices_buffer, out=self.d_out[layer])
        elif stage == "select_attend":     # second launch of the step; the histograms are ready
            K.select_attend(c.distance_scratch(n), kk, q, self.d_out[layer], c.kv_cache.buf_layer(layer),
                            c.kv_indices_with_last, c.kv_cache.last_page_len, c.kv_last_page_idx,
                            hist=c.hist_scratch, hist_ready=True)
        else:
            raise ValueError(stage)


def capture_batch(wls, stage, pre_stage=None):
    """CUDA graph of `stage` for every layer of every sequence in `wls` (`pre_stage`, if given, runs in
    front of it in every layer).  The sequences are independent (each has its own controller, page tables
    and caches); within a layer they run on one stream each, forked from and joined to the capturing
    stream, the way a batched model step proceeds layer by layer."""
    layers = wls[0].layers

    def ops(wl, layer):
        if pre_stage is not None:
            wl.stage_op(pre_stage, layer)
        wl.stage_op(stage, layer)

    def body(main, streams):
        for layer in range(layers):
            if len(wls) == 1:
                ops(wls[0], layer)
                continue
            fork = torch.cuda.Event()
            fork.record(main)
            for wl, st in zip(wls, streams):
                st.wait_event(fork)
                with torch.cuda.stream(st):
                    ops(wl, layer)
                join = torch.cuda.Event()
                join.record(st)
                main.wait_event(join)

    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    streams = [torch.cuda.Stream() for _ in wls] if len(wls) > 1 else []
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        body(s, streams)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    with torch.cuda.graph(g, stream=s):
        body(s, streams)
    return g


def timed(fn, steps, dist_on, dev):
    """barrier + synchronize, CUDA events around exactly `steps` calls, max over ranks (ms)."""
    import torch.distributed as dist
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist_on:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    return ms


def timed_blocks(fn, steps, blocks, dist_on, dev):
    """`blocks` repetitions of timed(fn, steps): the median block (ms for `steps` calls) and all of them."""
    all_ms = sorted(timed(fn, steps, dist_on, dev) for _ in range(blocks))
    return all_ms[len(all_ms) // 2], all_ms


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def ncu_traffic(kernel, args):
    """DRAM bytes per launch of `kernel` from an ncu capture of this workload, if one is on record
    (profiles/ncu_traffic.json: a list of {kernel, ctx, heads, budget, page_size, dtype, bytes, source}),
    else None: the figure is never guessed."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            table = json.load(f)
    except Exception:
        return None, None
    for row in table:
        if (row.get("kernel"), row.get("ctx"), row.get("heads"), row.get("budget"), row.get("page_size"),
                row.get("dtype")) == (kernel, args.ctx, args.heads, args.budget, args.page_size, args.dtype):
            return float(row["bytes"]), row.get("source")
    return None, None


def strong_scaling_record(args, dev, world, dist_on):
    """The 32-head model split over the ranks (32 / N heads each; the configuration the head-sharded
    scaling is stated for), next to the whole model on one GPU, each as the advancing step graph:
    32K context / budget 1024 in fp16 and 128K / budget 2048 in bf16."""
    out = []
    for ctx, budget, dtype, name, layers in ((32768, 1024, torch.float16, "f16", 16), (131072, 2048, torch.bfloat16, "bf16", 4)):
        rec = {"ctx": ctx, "budget": budget, "dtype": name, "layers_timed": layers, "total_heads": 32, "n_gpus": world}
        for label, heads in (("one_gpu_32_heads", 32), ("sharded", 32 // world)):
            wl = Workload(args, dev, seed_offset=7, room=64, heads=heads, ctx=ctx, budget=budget, layers=layers, dtype=dtype)
            wl.capture()
            for _ in range(3):
                wl.step()
            ms, _ = timed_blocks(wl.step, 10, 3, dist_on, dev)
            rec[label + "_us_per_layer"] = ms / 10 * 1e3 / layers
            rec[label + "_heads_per_gpu"] = heads
            del wl
            torch.cuda.empty_cache()
        rec["speedup"] = rec["one_gpu_32_heads_us_per_layer"] / rec["sharded_us_per_layer"]
        rec["efficiency"] = rec["speedup"] / world
        peak, _ = measured_peak()
        rec["sharded_path_roofline_frac_per_gpu"] = (stage_bytes(ctx, 32 // world, budget)["total"] /
                                                     (rec["sharded_us_per_layer"] * 1e-6) / 1e9 / peak)
        out.append(rec)
    return out


def run_ours(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist_on = world > 1
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if dist_on:
        dist.init_process_group("nccl", device_id=dev)
    blocks = max(1, args.blocks)
    warm = max(3, args.warmup)
    # room for every token the run appends: warm-ups, the timed blocks of both legs, the eager leg
    room = 2 * (warm + blocks * args.steps) + 64 + 64
    wl = Workload(args, dev, room=room)
    if dist_on:
        gather_buf = torch.empty(world, *wl.d_out.shape, dtype=wl.d_out.dtype, device=dev)
        # the layer outputs of all ranks, gathered inside the step (NCCL collectives can be captured)
        wl.after_layers = lambda: dist.all_gather_into_tensor(gather_buf, wl.d_out)
        dist.all_gather_into_tensor(gather_buf, wl.d_out)     # communicator set-up outside any capture
        torch.cuda.synchronize()

    wl.capture()
    for _ in range(warm):
        wl.step()
    torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    ms, ms_blocks = timed_blocks(wl.step, args.steps, blocks, dist_on, dev)
    clocks = sampler.stop()

    for _ in range(3):
        wl.step_e2e()
    ms_e2e, _ = timed_blocks(wl.step_e2e, args.steps, blocks, dist_on, dev)

    # eager (no graph) end to end, for information: the same advancing step, launched call by call
    saved = wl.graph
    wl.graph = None
    for _ in range(2):
        wl.step_e2e()
    n_eager = max(1, min(args.steps, 20))
    ms_eager = timed(wl.step_e2e, n_eager, dist_on, dev)
    wl.graph = saved
    ctx_end = wl.c.kv_cache.seqlen

    # Every kernel class of the step alone (a graph with one launch per layer, so the data comes from HBM),
    # at the position the host holds now.  select_attend needs the estimate's distances and histograms in
    # front of it: it is timed as (estimate + select_attend) - estimate.
    c = wl.c
    c.begin_forward(1)
    stage_us = {}
    for layer in range(args.layers):   # query codes of every layer, for the estimate stage run alone
        wl.U.append_qkv_fused(wl.d_qkv[0, layer], wl.d_qkv[1, layer], wl.d_qkv[2, layer], c, layer, out=wl.q_code[layer])
    torch.cuda.synchronize()

    def stage_time(stage, pre=None):
        g_st = capture_batch([wl], stage, pre_stage=pre)
        for _ in range(3):
            g_st.replay()
        us = timed_blocks(g_st.replay, max(10, args.steps // 2), 3, False, dev)[0] * 1e3 / max(10, args.steps // 2) / args.layers
        del g_st
        return us

    if args.unfused:
        for stage in ("append", "estimate", "topk", "attention"):
            stage_us[stage] = stage_time(stage)
        kernels = {"append": "append_decode_kernel", "estimate": "estimate_kernel", "topk": "topk_cluster_kernel",
                   "attention": "sparse_decode_kernel"}
        kbytes = lambda by: {"append": 0, "estimate": by["estimate"], "topk": by["topk"], "attention": by["attention"]}
    else:
        first = "append_estimate" if two_launch_step(args) else "estimate"
        stage_us[first] = stage_time(first)
        if first != "estimate":
            stage_us["estimate"] = stage_time("estimate")
        else:
            stage_us["append"] = stage_time("append")
        both = stage_time("select_attend", pre="estimate")
        stage_us["estimate_then_select_attend"] = both
        stage_us["select_attend"] = both - stage_us["estimate"]
        kernels = {first: "estimate_append_kernel" if first == "append_estimate" else "estimate_kernel",
                   "select_attend": "select_attend_kernel"}
        if first == "estimate":
            kernels["append"] = "append_decode_kernel"
        kbytes = lambda by: {first: by["estimate"], "select_attend": by["topk"] + by["attention"], "append": 0}

    strong = None
    if dist_on and not args.no_strong and 32 % world == 0:
        del wl
        torch.cuda.empty_cache()
        strong = strong_scaling_record(args, dev, world, dist_on)

    if rank != 0:
        leave(dist_on)
        return

    L, H, B = args.ctx, args.heads, args.budget
    by = stage_bytes(L, H, B)
    step_bytes = by["total"] * args.layers * world
    ms_per_step = ms / args.steps
    value = step_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = step_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
    peak, peak_src = measured_peak()
    # roofline of every kernel of the step; the headline block is the one with the largest share of the time
    kb = kbytes(by)
    per_kernel = []
    for stage, kname in kernels.items():
        if stage not in stage_us or kb.get(stage, 0) == 0:
            continue
        traffic, src = ncu_traffic(kname, args)
        gbs = kb[stage] / (stage_us[stage] * 1e-6) / 1e9
        per_kernel.append({"kernel": kname, "bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s",
                           "frac": gbs / peak, "traffic": traffic, "traffic_source": src, "peak_source": peak_src,
                           "us_per_launch": stage_us[stage], "algorithmic_bytes_per_launch": kb[stage],
                           "share_of_step_time": stage_us[stage] / sum(stage_us[s] for s in kernels if s in stage_us)})
    per_kernel.sort(key=lambda r: -r["us_per_launch"])
    launches = launches_per_layer(args) * args.layers + (1 if not args.unfused else 0)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": getattr(args, "dtype", "f16"), "data": "synthetic",
        "us_per_layer": ms_per_step * 1e3 / args.layers,
        "us_per_layer_e2e": ms_e2e / args.steps * 1e3 / args.layers,
        "us_per_layer_e2e_eager": ms_eager / n_eager * 1e3 / args.layers,
        "path_roofline_frac": value / world / peak,
        "timed_blocks_ms": ms_blocks,
        "context_at_end": ctx_end,
        "config": workload_config(args),
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": args.layers * 3 * H * 128 * 2,
                "d2h_bytes_per_step": args.layers * H * 128 * 2},
        "gpu_launches": args.steps * blocks * launches,
        "roofline": per_kernel[0] if per_kernel else None,
        "roofline_other_kernels": per_kernel[1:],
        "stage_bytes_per_layer": by,
        "stage_us_alone": stage_us,
    }
    if strong is not None:
        line["strong"] = strong
    if not args.no_cpu and world == 1:      # (the CPU baseline is a single-GPU-run figure)
        sec, n = time_cpu_reference(L, H, B, steps=60, warmup=2, budget_s=15.0)
        line["cpu_baseline"] = {
            "value": by["total"] / sec / 1e9, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": (f"{n} timed runs of one layer-step (1 of {args.layers} layers) of the reference PyTorch "
                       f"decode path with cached key codes, ctx {L}, budget {B}, fp32 torch CPU; {sec * 1e3:.1f} ms each"),
        }
    print(json.dumps(line), flush=True)
    leave(dist_on)


def leave(dist_on):
    """End of a multi-rank run.  The process group is not torn down: CUDA graphs that hold captured
    collectives are still alive, and destroying the communicator under them has hung; every rank has
    passed its last collective when it gets here, so the processes simply exit."""
    if dist_on:
        sys.stdout.flush()
        sys.stderr.flush()
        torch.cuda.synchronize()
        os._exit(0)


def run_sweep(args):
    """Per-operator sweep (one GPU): context x budget, each stage timed alone in a CUDA graph with
    one launch per layer (distinct caches, so data comes from HBM).  Prints one JSON line per point.
    Batch > 1 (--sweep-batch) is b independent sequences, each with its own controller, page table
    and caches (the reference is batch-1 only): their launches run on one stream per sequence inside
    the graph, joined after every layer; GB/s figures are aggregates over the b sequences."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    for ctx in args.sweep_ctx:
        for batch in args.sweep_batch:
            # caches of all sequences and rotated layers stay under ~48 GB and well above L2
            layers = max(1, min(32, int(48e9 // (batch * ctx * args.heads * 544))))
            if batch == 1:
                layers = max(4, min(layers, int(6e9 // (ctx * args.heads * 544))))
            for budget in args.sweep_budget:
                if budget >= ctx:
                    continue
                a = argparse.Namespace(**vars(args))
                a.ctx, a.budget, a.layers, a.unfused = ctx, budget, layers, True
                from adamas_b200 import _kernels as K
                # several sequences in flight: fewer blocks per head so that their kernels overlap
                cluster = 8 if batch == 1 else 4      # measured: 4 is best from two sequences up
                if args.sweep_cluster:
                    cluster = args.sweep_cluster
                K.set_max_cluster(cluster)
                # several sequences: one estimate block per SM, so that other sequences' select+attend
                # blocks find room while an estimate streams
                K.set_estimate_blocks_per_sm(args.sweep_est_blocks or (1 if batch > 1 else 2))
                wls = [Workload(a, dev, seed_offset=i, room=(args.steps + 16 if batch > 1 else 0)) for i in range(batch)]
                for wl in wls:
                    wl.step_fixed()
                torch.cuda.synchronize()
                by = stage_bytes(ctx, args.heads, budget, batch)
                out = {"sweep": True, "batch": batch, "ctx": ctx, "budget": budget, "heads": args.heads,
                       "page_size": args.page_size, "layers_rotated": layers, "max_cluster": cluster,
                       "est_blocks_per_sm": args.sweep_est_blocks or (1 if batch > 1 else 2)}
                def sweep_time(stage, pre=None):
                    g = capture_batch(wls, stage, pre_stage=pre)
                    for _ in range(3):
                        g.replay()
                    us = timed(g.replay, args.steps, False, dev) * 1e3 / args.steps / layers
                    del g
                    return us

                for stage in ("estimate", "topk", "attention", "append"):     # the four separate operators
                    out[stage + "_us"] = round(sweep_time(stage), 2)
                    if stage in by:
                        out[stage + "_GBps"] = round(by[stage] / (out[stage + "_us"] * 1e-6) / 1e9, 1)
                # the fused step and its second kernel (timed behind the estimate that feeds it)
                a.unfused = False
                for wl in wls:
                    wl.step_fixed()
                est_fused = sweep_time("estimate")
                out["estimate_with_histograms_us"] = round(est_fused, 2)      # u16 distances + per-slice counts
                out["select_attend_us"] = round(sweep_time("select_attend", pre="estimate") - est_fused, 2)
                out["step_us"] = round(sweep_time("step"), 2)
                a.unfused = True
                out["select_attend_GBps"] = round((by["topk"] + by["attention"]) / (out["select_attend_us"] * 1e-6) / 1e9, 1)
                out["step_GBps"] = round(by["total"] / (out["step_us"] * 1e-6) / 1e9, 1)
                if batch > 1:
                    # all sequences through the SAME launches (utils.SequenceBatch), advancing one token per replay
                    import adamas_b200.utils as U
                    K.set_max_cluster(8)
                    K.set_estimate_blocks_per_sm(2)
                    sb = U.SequenceBatch([wl.c for wl in wls])
                    bq, bk, bv = ([torch.stack([wl.d_qkv[j, l, 0] for wl in wls]) for l in range(layers)] for j in range(3))
                    bo = [torch.zeros_like(t) for t in bq]

                    def batched_body():
                        for l in range(layers):
                            sb.decode_step_dev(bq[l], bk[l], bv[l], l, out=bo[l], rope=wls[0].rope)
                        sb.advance()

                    def batched_step():
                        sb.prepare(1)
                        gb.replay()

                    sb.sync_seq_lens()
                    batched_body()
                    torch.cuda.synchronize()
                    sb.prepare(1)
                    gb = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gb):
                        batched_body()
                    for _ in range(3):
                        batched_step()
                    out["step_one_launch_us"] = round(timed(batched_step, args.steps, False, dev) * 1e3 / args.steps / layers, 2)
                    out["step_one_launch_GBps"] = round(by["total"] / (out["step_one_launch_us"] * 1e-6) / 1e9, 1)
                    del sb, gb, bq, bk, bv, bo
                print(json.dumps(out), flush=True)
                del wls, wl
                torch.cuda.empty_cache()


def run_seqshard(args):
    """Sequence-sharded decode of one long context over the ranks (million-token configuration):
    rank g holds tokens [g*L/G, (g+1)*L/G) of every head and layer; per layer-step the ranks run the
    local estimate with its histograms, all-gather the histograms, derive the same cut and their own
    share of the ties, select and attend locally, all-gather the partial (o, lse) results and merge
    them (adamas_b200.sharding): two NCCL all-gathers per layer, everything else this library's
    kernels.  The whole step is one CUDA graph unless --eager.  Prints one JSON line on rank 0."""
    import torch.distributed as dist
    from adamas_b200 import _kernels as K, sharding
    import adamas_b200.utils as U
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    L, H, ps, B, layers = args.ctx, args.heads, args.page_size, args.budget, args.layers
    t0, t1 = sharding.token_range(L, world, rank, ps)
    n_local = t1 - t0
    owns_tail = t1 == L
    c = U.InferenceController(layers, H, 128, ps, 1 << 24, n_local + ps, dtype, dev)
    gen = torch.Generator(device=dev).manual_seed(4321 + rank)
    n_pre = n_local - 1 if owns_tail else n_local
    c.prepare_hadamard(n_pre)
    c.begin_forward(n_pre)
    chunk = 1 << 15
    for layer in range(layers):
        k = torch.randn(n_pre, H, 128, device=dev, dtype=dtype, generator=gen)
        v = torch.randn(n_pre, H, 128, device=dev, dtype=dtype, generator=gen)
        U.append_kvh(k, v, None, c, layer)
        del k, v
    c.end_forward()
    if owns_tail:
        c.prepare_hadamard(1)
        c.begin_forward(1)
    hg = torch.Generator().manual_seed(77)          # the same new token on every rank
    qkv = torch.randn(3, layers, 1, H, 128, generator=hg).to(dtype).to(dev)
    out = torch.zeros(layers, H, 128, dtype=dtype, device=dev)
    q_code = torch.empty(1, H, 16, dtype=dtype, device=dev)

    ops_of_layer = []
    codes = [torch.empty(1, H, 16, dtype=dtype, device=dev) for _ in range(layers)]

    def step():
        for layer in range(layers):
            q, k, v = qkv[0, layer], qkv[1, layer], qkv[2, layer]
            if owns_tail:
                U.append_qkv_fused(q, k, v, c, layer, out=codes[layer])      # (re-appends the same token every step)
            else:
                K.bucketize_pack(K.hadamard_transform(q), codes[layer])
            if len(ops_of_layer) <= layer:
                ops_of_layer.append(sharding.CudaOps(c, layer, codes[layer], owns_tail))
            o, _ = sharding.sequence_sharded_step(ops_of_layer[layer], q[0], B)
            out[layer].copy_(o)

    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    graph = None
    if not args.eager:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        for _ in range(2):
            graph.replay()
    ms = timed(graph.replay if graph is not None else step, args.steps, True, dev)
    if rank == 0:
        per_layer_us = ms * 1e3 / args.steps / layers
        by = stage_bytes(L, H, B)
        print(json.dumps({
            "mode": "sequence-sharded", "metric": METRIC, "value": by["total"] / (per_layer_us * 1e-6) / 1e9,
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms / args.steps, "us_per_layer": per_layer_us, "higher_is_better": True,
            "scaling": "strong", "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": f"one sequence of {L} tokens split over {world} GPUs, {layers} layers x {H} heads x 128, "
                                   f"budget {B}, page size {ps}; "
                                   + ("eager launches" if args.eager else "one CUDA graph per step")
                                   + ", 2 NCCL all-gathers per layer (histograms, partial results)",
                       "tokens_per_gpu": n_local}}), flush=True)
    leave(True)


def run_model(args):
    """End-to-end decode of a Llama-2-7B-shaped stack with random-init weights on one GPU: prefill
    `--ctx` seeded uniform-random token ids, then `--decode-tokens` greedy decode steps at token
    budget `--budget` (first two layers dense).  The timed region is the whole decode loop as a user
    runs it (host code included), bracketed by CUDA events; the sampled ids are read back once at the
    end.  Prints one JSON line with tokens/s and the share of the step spent in the attention path."""
    from adamas_b200 import llama_stack as S
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    cfg = S.StackConfig(num_layers=args.layers, num_heads=args.heads)
    st = S.LlamaStack(cfg, dev, dtype, seed=0)
    n_new = args.decode_tokens
    st.init_controller(args.page_size, args.budget, args.ctx + n_new + args.page_size)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (args.ctx,), generator=g).to(dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    ev[0].record()
    st.prefill(ids)
    ev[1].record()
    for _ in range(max(3, args.warmup)):       # the first token runs eagerly and captures the graph
        st.decode_one()
    out = torch.empty(n_new, dtype=torch.int64, device=dev)
    sampler = ClockSampler(0)
    torch.cuda.synchronize()
    sampler.start()
    t_host = time.perf_counter()
    ev[2].record()
    for i in range(n_new):
        st.decode_one()
        out[i:i + 1].copy_(st._tok)
    ev[3].record()
    t_issue = time.perf_counter() - t_host
    torch.cuda.synchronize()
    clocks = sampler.stop()
    toks = out.tolist()
    decode_ms = ev[2].elapsed_time(ev[3])

    # the same token without the attention path: what the dense rest of the model costs
    rest = st.capture_dense_rest()
    for _ in range(3):
        rest.replay()
    rest_ms = timed(rest.replay, 20, False, dev) / 20
    from adamas_b200 import _lib
    per_tok = decode_ms / n_new
    print(json.dumps({
        "mode": "model", "metric": "e2e_decode_tokens_per_s", "value": 1e3 / per_tok, "unit": "tokens/s",
        "n_gpus": 1, "steps": n_new, "warmup": max(3, args.warmup), "ms_per_step": per_tok,
        "higher_is_better": True, "dtype": args.dtype, "data": "synthetic",
        "prefill_s": ev[0].elapsed_time(ev[1]) / 1e3,
        "host_issue_ms_per_token": t_issue * 1e3 / n_new,
        "dense_rest_ms_per_token": rest_ms,
        "attention_path_ms_per_token": per_tok - rest_ms,
        "clocks": clocks, "device_error": _lib.device_error(),
        "distinct_tokens": len(set(toks)),
        "config": {"workload": f"Llama-2-7B-shaped stack ({cfg.num_layers} layers, hidden {cfg.hidden}, "
                               f"{cfg.num_heads}x128 heads, FFN {cfg.ffn}, vocab {cfg.vocab}, linear RoPE scale 8), "
                               f"random-init {args.dtype} weights, prefill {args.ctx} random ids, decode {n_new} tokens, "
                               f"token budget {args.budget}, page size {args.page_size}, first {cfg.skip_layers} layers dense; "
                               "GEMMs, norms and the dense prefill attention are torch library calls, the decode "
                               "attention path is this library; every token is ONE CUDA graph replay (sequence length "
                               "in device memory)"}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--budget", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--heads", type=int, default=32, help="KV heads per GPU")
    ap.add_argument("--page-size", dest="page_size", type=int, default=16)
    ap.add_argument("--eager", action="store_true", help="no CUDA graph")
    ap.add_argument("--unfused", action="store_true",
                    help="four launches per layer (append, estimate, top-k, sparse decode) instead of the fused step")
    ap.add_argument("--no-cpu", dest="no_cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--blocks", type=int, default=5, help="the timed steps are repeated this many times; the median block is reported")
    ap.add_argument("--yarn", type=float, default=0.0,
                    help="rotate q and k inside the step with a YaRN table of this factor (original context 4096)")
    ap.add_argument("--repeat-token", dest="repeat_token", action="store_true",
                    help="append the same token's q/k/v at every step instead of a different one")
    ap.add_argument("--no-strong", dest="no_strong", action="store_true",
                    help="N > 1: skip the strong-scaling record (the 32-head model split over the ranks)")
    ap.add_argument("--sweep", action="store_true", help="per-operator sweep over context x budget (one GPU)")
    ap.add_argument("--sweep-ctx", dest="sweep_ctx", type=int, nargs="+", default=[8192, 32768, 131072])
    ap.add_argument("--sweep-budget", dest="sweep_budget", type=int, nargs="+", default=[64, 128, 512, 2048])
    ap.add_argument("--sweep-cluster", dest="sweep_cluster", type=int, default=0,
                    help="force the select_attend cluster bound (default: 8 for one sequence, else 4)")
    ap.add_argument("--sweep-est-blocks", dest="sweep_est_blocks", type=int, default=0,
                    help="force the estimate's blocks per SM in the sweep (default: 2 for one sequence, else 1)")
    ap.add_argument("--sweep-batch", dest="sweep_batch", type=int, nargs="+", default=[1],
                    help="independent sequences per step, one stream each inside the graph")
    ap.add_argument("--seq-sharded", dest="seq_sharded", action="store_true",
                    help="one long sequence split over the ranks (torchrun); see run_seqshard")
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16"])
    ap.add_argument("--model", action="store_true",
                    help="end-to-end decode tokens/s of a Llama-2-7B-shaped stack (one GPU); see run_model")
    ap.add_argument("--decode-tokens", dest="decode_tokens", type=int, default=256)
    args = ap.parse_args()
    if args.model:
        run_model(args)
        return
    if args.seq_sharded:
        run_seqshard(args)
        return
    if args.sweep:
        run_sweep(args)
        return
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
