#!/usr/bin/env python
"""Benchmark of the Adamas decode hot path on B200.

A "step" is one decode token's pass through the attention hot path of every layer of a
Llama-2-7B-shaped stack (32 layers, 32 heads x 128) at a 32K-token context with a token budget of
1024 and page size 16: per layer, fused append (Hadamard + 2-bit code + KV write), distance
estimate over the layer's code cache, top-k, sparse paged attention.  Every layer has its own KV
and code cache, so one step streams ~1.6 GB of distinct data (inputs far larger than L2).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 is launched by torch.distributed.run; each rank owns the same number of KV heads of a model
N times as wide (head sharding, no collective inside the path; the per-step gather of the layer
outputs is included in the timed region).  Rank 0 prints one JSON line.
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
    """decode_step folds the append into the estimate launch for 32 or 64 heads."""
    return (not args.unfused) and args.heads in (32, 64) and os.environ.get("ADAMAS_FUSED_APPEND", "1") != "0"


def launches_per_layer(args) -> int:
    return 4 if args.unfused else (2 if two_launch_step(args) else 3)


def workload_config(args, extra=None):
    cfg = {
        "workload": (f"llama2-7b-shaped attention stack: {args.layers} layers x {args.heads} heads x 128, "
                     f"ctx {args.ctx}, token budget {args.budget}, page size {args.page_size}, batch 1; "
                     "per layer: fused append + estimate + top-k + sparse paged attention "
                     + ("(4 launches)" if args.unfused else
                        ("(decode_step: 2 launches, append inside the estimate kernel, top-k and attention in one kernel)"
                         if two_launch_step(args) else "(decode_step: 3 launches, top-k and attention in one kernel)"))),
        "layers": args.layers, "heads_per_gpu": args.heads, "ctx": args.ctx, "budget": args.budget,
        "page_size": args.page_size, "parallelism": f"head-sharded x{args.gpus}" if args.gpus > 1 else "single GPU",
        "l2": "inputs larger than L2 (each layer has its own caches; ~1.6 GB touched per step)",
        "launch": "CUDA graph of the step" if not args.eager else "eager",
    }
    if extra:
        cfg.update(extra)
    return cfg


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
class Workload:
    def __init__(self, args, dev, seed_offset=0):
        import adamas_b200.utils as U
        self.U = U
        self.args = args
        self.dev = dev
        L, H, ps, B, layers = args.ctx, args.heads, args.page_size, args.budget, args.layers
        dtype = torch.bfloat16 if getattr(args, "dtype", "f16") == "bf16" else torch.float16
        self.c = c = U.InferenceController(layers, H, 128, ps, B // ps, L, dtype, dev)
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
        self.d_out = torch.zeros(layers, 1, H, 128, dtype=dtype, device=dev)
        self.h_out = torch.zeros(layers, 1, H, 128, dtype=dtype).pin_memory()
        self.q_code = torch.zeros(layers, 1, H, 16, dtype=dtype, device=dev)
        self.graph = None

    def layer_step(self, layer):
        U, c = self.U, self.c
        q, k, v = self.d_qkv[0, layer], self.d_qkv[1, layer], self.d_qkv[2, layer]
        if not self.args.unfused:
            # public fused API: append + estimate + select/attend, two or three launches
            U.decode_step(q, k, v, c, layer, out=self.d_out[layer], record_indices=False)
            return
        q_code = U.append_qkv_fused(q, k, v, c, layer, out=self.q_code[layer])
        est = U.decode_estimate(q_code, c, layer)
        U.decode_topk(est, c)
        U.decode_sparse_attn(q, c, layer, c.topk_dindices_buffer, out=self.d_out[layer])

    def step_eager(self):
        for layer in range(self.args.layers):
            self.layer_step(layer)

    def capture(self):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self.step_eager()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.step_eager()

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step_eager()

    def step_e2e(self):
        """Host buffers in, host buffers out: H2D of this step's q/k/v, the step, D2H of the outputs."""
        self.d_qkv.copy_(self.h_qkv, non_blocking=True)
        self.step()
        self.h_out.copy_(self.d_out, non_blocking=True)

    def stage_op(self, stage, layer):
        """One kernel class of one layer ("step": the whole layer step)."""
        U, c = self.U, self.c
        from adamas_b200 import _kernels as K
        q, k, v = self.d_qkv[0, layer], self.d_qkv[1, layer], self.d_qkv[2, layer]
        if stage == "step":
            self.layer_step(layer)
        elif stage == "append":
            U.append_qkv_fused(q, k, v, c, layer, out=self.q_code[layer])
        elif stage == "append_estimate":   # first launch of the two-launch step
            n = c.hadamard_cache.seqlen - 1
            K.append_estimate(q, k, v, self.q_code[layer], c.kv_cache.buf_layer(layer), c.kv_indices_with_last,
                              c.kv_cache.last_page_len, c.hadamard_cache.buf_layer(layer), c.hadamard_indices,
                              c.hadamard_cache.last_page_len, c.distance_scratch(n))
        elif stage == "estimate" and self.args.unfused:
            U.decode_estimate(self.q_code[layer], c, layer)
        elif stage == "estimate":      # fused step: integer distances, as decode_step asks for
            n = c.hadamard_cache.seqlen - 1
            K.estimate_attn_score(self.q_code[layer], c.distance_scratch(n), c.hadamard_cache.buf_layer(layer),
                                  c.hadamard_indices, None, c.hadamard_cache.last_page_len,
                                  c.hadamard_last_page_idx, c.layout)
        elif stage == "topk":
            U.decode_topk(c.estimate_buffer(c.hadamard_cache.seqlen - 1), c)
        elif stage == "attention":
            U.decode_sparse_attn(q, c, layer, c.topk_dindices_buffer, out=self.d_out[layer])
        elif stage == "select_attend":
            n = c.hadamard_cache.seqlen - 1
            k = c.inference_token_budget - 1
            # first launch of the step without the append: leaves the distances and the histograms
            K.estimate_attn_score(self.q_code[layer], c.distance_scratch(n), c.hadamard_cache.buf_layer(layer),
                                  c.hadamard_indices, None, c.hadamard_cache.last_page_len,
                                  c.hadamard_last_page_idx, c.layout, hist=c.hist_scratch,
                                  hist_slices=K.select_attend_slices(n, k, self.args.heads))
            K.select_attend(c.distance_scratch(n), k, q, self.d_out[layer],
                            c.kv_cache.buf_layer(layer), c.kv_indices_with_last, c.kv_cache.last_page_len,
                            c.kv_last_page_idx, hist=c.hist_scratch, hist_ready=True)
        else:
            raise ValueError(stage)

    # one kernel class alone (a graph with one launch per layer, so the data comes from HBM)
    def capture_stage_only(self, stage):
        return capture_batch([self], stage)


def capture_batch(wls, stage):
    """CUDA graph of `stage` for every layer of every sequence in `wls`.  The sequences are
    independent (each has its own controller, page tables and caches); within a layer they run on
    one stream each, forked from and joined to the capturing stream, the way a batched model step
    proceeds layer by layer."""
    layers = wls[0].args.layers

    def body(main, streams):
        for layer in range(layers):
            if len(wls) == 1:
                wls[0].stage_op(stage, layer)
                continue
            fork = torch.cuda.Event()
            fork.record(main)
            for wl, st in zip(wls, streams):
                st.wait_event(fork)
                with torch.cuda.stream(st):
                    wl.stage_op(stage, layer)
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


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


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
    wl = Workload(args, dev)
    gather_buf = None
    if dist_on:
        gather_buf = torch.empty(world, *wl.d_out.shape, dtype=wl.d_out.dtype, device=dev)

    def step_dev():
        wl.step()
        if dist_on:
            dist.all_gather_into_tensor(gather_buf, wl.d_out)

    def step_e2e():
        wl.step_e2e()
        if dist_on:
            dist.all_gather_into_tensor(gather_buf, wl.d_out)

    if not args.eager:
        wl.capture()
    for _ in range(max(3, args.warmup)):
        step_dev()
    torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    ms = timed(step_dev, args.steps, dist_on, dev)
    clocks = sampler.stop()

    for _ in range(3):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps, dist_on, dev)

    # eager (no graph) end to end, for information
    saved = wl.graph
    wl.graph = None
    for _ in range(2):
        step_e2e()
    ms_eager = timed(step_e2e, max(1, min(args.steps, 20)), dist_on, dev)
    wl.graph = saved

    # dominant kernel alone (estimate), one launch per layer so the data comes from HBM
    stage_us = {}
    # leave integer distances of the last layer in the scratch for the select/attend stage
    wl.U.decode_step(wl.d_qkv[0, 0], wl.d_qkv[1, 0], wl.d_qkv[2, 0], wl.c, 0, out=wl.d_out[0], record_indices=True)
    for layer in range(args.layers):   # query codes of every layer, for the estimate stage run alone
        wl.U.append_qkv_fused(wl.d_qkv[0, layer], wl.d_qkv[1, layer], wl.d_qkv[2, layer], wl.c, layer, out=wl.q_code[layer])
    stage_list = ("estimate", "append", "select_attend") if not args.unfused else ("estimate", "append", "topk", "attention")
    if two_launch_step(args):
        stage_list = ("append_estimate",) + stage_list
    for stage in stage_list:
        g_st = wl.capture_stage_only(stage)
        for _ in range(3):
            g_st.replay()
        stage_us[stage] = timed(g_st.replay, args.steps, False, dev) * 1e3 / args.steps / args.layers
        del g_st
    # the dominant kernel of the timed region: the estimate, with the append inside in the two-launch step
    est_kernel = "estimate_append_kernel" if two_launch_step(args) else "estimate_kernel"
    est_us = stage_us["append_estimate" if two_launch_step(args) else "estimate"]

    if rank != 0:
        if dist_on:
            dist.destroy_process_group()
        return

    L, H, B = args.ctx, args.heads, args.budget
    by = stage_bytes(L, H, B)
    step_bytes = by["total"] * args.layers * world
    ms_per_step = ms / args.steps
    value = step_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = step_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
    peak, peak_src = measured_peak()
    est_gbs = by["estimate"] / (est_us * 1e-6) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": getattr(args, "dtype", "f16"), "data": "synthetic",
        "us_per_layer": ms_per_step * 1e3 / args.layers,
        "us_per_layer_e2e": ms_e2e / args.steps * 1e3 / args.layers,
        "us_per_layer_e2e_eager": ms_eager / max(1, min(args.steps, 20)) * 1e3 / args.layers,
        "path_roofline_frac": value / world / peak,
        "config": workload_config(args),
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": wl.h_qkv.numel() * wl.h_qkv.element_size(),
                "d2h_bytes_per_step": wl.h_out.numel() * wl.h_out.element_size()},
        "gpu_launches": args.steps * args.layers * launches_per_layer(args),
        "roofline": {"kernel": est_kernel, "bound": "hbm", "achieved": est_gbs, "peak": peak,
                     "unit": "GB/s", "frac": est_gbs / peak, "traffic": args.traffic,
                     "peak_source": peak_src, "us_per_launch": est_us,
                     "algorithmic_bytes_per_launch": by["estimate"]},
        "stage_bytes_per_layer": by,
        "stage_us_alone": stage_us,
        "stage_gbs_alone": {k: by[k] / (stage_us[k] * 1e-6) / 1e9 for k in ("estimate", "topk", "attention") if k in stage_us},
    }
    if not args.no_cpu and world >= 1:
        sec, n = time_cpu_reference(L, H, B, steps=60, warmup=2, budget_s=15.0)
        line["cpu_baseline"] = {
            "value": by["total"] / sec / 1e9, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": (f"{n} timed runs of one layer-step (1 of {args.layers} layers) of the reference PyTorch "
                       f"decode path with cached key codes, ctx {L}, budget {B}, fp32 torch CPU; {sec * 1e3:.1f} ms each"),
        }
    print(json.dumps(line), flush=True)
    if dist_on:
        dist.destroy_process_group()


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
                wls = [Workload(a, dev, seed_offset=i) for i in range(batch)]
                for wl in wls:
                    wl.step_eager()
                torch.cuda.synchronize()
                by = stage_bytes(ctx, args.heads, budget, batch)
                out = {"sweep": True, "batch": batch, "ctx": ctx, "budget": budget, "heads": args.heads,
                       "page_size": args.page_size, "layers_rotated": layers, "max_cluster": cluster,
                       "est_blocks_per_sm": args.sweep_est_blocks or (1 if batch > 1 else 2)}
                for stage in ("estimate", "topk", "attention", "select_attend", "append", "step"):
                    if stage in ("select_attend", "step"):
                        a.unfused = False      # the estimate must have left integer distances
                        for wl in wls:
                            wl.U.decode_step(wl.d_qkv[0, 0], wl.d_qkv[1, 0], wl.d_qkv[2, 0], wl.c, 0, out=wl.d_out[0])
                    g = capture_batch(wls, stage)
                    for _ in range(3):
                        g.replay()
                    us = timed(g.replay, args.steps, False, dev) * 1e3 / args.steps / layers
                    a.unfused = True
                    out[stage + "_us"] = round(us, 2)
                    if stage in by:
                        out[stage + "_GBps"] = round(by[stage] / (us * 1e-6) / 1e9, 1)
                    del g
                out["select_attend_GBps"] = round((by["topk"] + by["attention"]) / (out["select_attend_us"] * 1e-6) / 1e9, 1)
                out["step_GBps"] = round(by["total"] / (out["step_us"] * 1e-6) / 1e9, 1)
                print(json.dumps(out), flush=True)
                del wls, wl
                torch.cuda.empty_cache()


def run_seqshard(args):
    """Sequence-sharded decode of one long context over the ranks (million-token configuration):
    rank g holds tokens [g*L/G, (g+1)*L/G) of every head and layer; per layer-step the ranks run the
    local estimate and candidate selection, all-gather the candidate distances, pick the global
    winners, attend over their own winners and merge the partial results (adamas_b200.sharding).
    Eager launches (NCCL collectives between the kernels).  Prints one JSON line on rank 0."""
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

    def step():
        for layer in range(layers):
            q, k, v = qkv[0, layer], qkv[1, layer], qkv[2, layer]
            if owns_tail:
                U.append_qkv_fused(q, k, v, c, layer, out=q_code)
            else:
                K.bucketize_pack(K.hadamard_transform(q), q_code)
            ops = sharding.CudaOps(c, layer, q_code, owns_tail)
            o, _ = sharding.sequence_sharded_step(ops, q, B)
            out[layer].copy_(o)

    for _ in range(max(3, args.warmup)):
        step()
    ms = timed(step, args.steps, True, dev)
    if rank == 0:
        per_layer_us = ms * 1e3 / args.steps / layers
        by = stage_bytes(L, H, B)
        print(json.dumps({
            "mode": "sequence-sharded", "metric": METRIC, "value": by["total"] / (per_layer_us * 1e-6) / 1e9,
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms / args.steps, "us_per_layer": per_layer_us, "higher_is_better": True,
            "scaling": "strong", "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": f"one sequence of {L} tokens split over {world} GPUs, {layers} layers x {H} heads x 128, "
                                   f"budget {B}, page size {ps}; eager launches, 3 NCCL all-gathers per layer",
                       "tokens_per_gpu": n_local}}), flush=True)
    dist.destroy_process_group()


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
    for _ in range(max(3, args.warmup)):       # captures the graphs, warms the kernels
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

    # the same loop without the attention path: what the dense rest of the model costs
    def rest_only():
        st._graphs[0].replay()
        for layer in range(cfg.num_layers):
            st._graphs[layer + 1].replay()
    for _ in range(3):
        rest_only()
    rest_ms = timed(lambda: rest_only(), 20, False, dev) / 20
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
                               "attention path is this library"}}), flush=True)


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
    ap.add_argument("--traffic", type=float, default=None,
                    help="DRAM bytes per launch of the dominant kernel from an ncu capture; default: the figure in "
                         "profiles/fused_step_kernels_32k_b1024_ncu.md when the workload matches it")
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
    if args.traffic is None and (args.ctx, args.heads, args.page_size) == (32768, 32, 16):
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel (ncu, 32K
        # context, 32 heads): 33.62 MB for the estimate with the append inside
        # (profiles/fused_step_kernels_32k_b1024_ncu.md), 33.58 MB for the plain estimate
        args.traffic = 33.62e6 if two_launch_step(args) else 33.58e6 + 1.0e3
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
