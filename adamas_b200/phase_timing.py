"""Where a decode step spends its time, without a profiler.

    python adamas_b200/phase_timing.py [--ctx 32768] [--heads 32] [--budget 1024] [--layers 32]

Builds a variant of the library with -DADAMAS_PHASE_TIMING (one thread per block stamps the global
nanosecond timer at phase boundaries of the estimate and select+attend kernels; csrc/common.cuh), runs a
CUDA graph of `utils.decode_step` over `layers` layers with distinct caches a few times and prints,
for the last layer of the last replay, when each phase ended (median and maximum over the blocks) and,
for the whole replay, the period between successive layers.  The stamps cost about half a microsecond
per layer; the product library is not touched.  Run it as a script: it re-executes itself with
ADAMAS_B200_LIBRARY pointing at the variant.
"""
from __future__ import annotations

import argparse
import ctypes
import os
import subprocess
import sys
import tempfile

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)


def _build_variant() -> str:
    out = os.path.join(tempfile.gettempdir(), f"libadamas_b200_timing_{os.getuid()}.so")
    src = os.path.join(PKG_DIR, "csrc", "adamas_b200.cu")
    deps = [os.path.join(PKG_DIR, "csrc", f) for f in os.listdir(os.path.join(PKG_DIR, "csrc"))]
    if os.path.exists(out) and all(os.path.getmtime(d) <= os.path.getmtime(out) for d in deps):
        return out
    cmd = ["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-Xcompiler", "-fPIC", "-shared", "-DADAMAS_PHASE_TIMING", "-o", out, src]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    return out


def _stats(x):
    import numpy as np
    return f"median {np.median(x) / 1e3:7.2f}  max {x.max() / 1e3:7.2f}"


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--budget", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--page-size", dest="page_size", type=int, default=16)
    ap.add_argument("--replays", type=int, default=5)
    args = ap.parse_args()
    if "ADAMAS_B200_LIBRARY" not in os.environ:
        env = dict(os.environ, ADAMAS_B200_LIBRARY=_build_variant())
        os.execve(sys.executable, [sys.executable, os.path.abspath(__file__)] + sys.argv[1:], env)
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import numpy as np
    import torch
    import adamas_b200.utils as U
    from adamas_b200 import _lib
    if not hasattr(_lib.lib, "adamas_debug_read_timing"):
        raise SystemExit("the loaded library was not built with -DADAMAS_PHASE_TIMING")

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    L, H, ps = args.ctx, args.heads, args.page_size
    c = U.InferenceController(args.layers, H, 128, ps, args.budget // ps, L, torch.float16, dev)
    gen = torch.Generator(device=dev).manual_seed(1)
    c.prepare_hadamard(L - 1)
    c.begin_forward(L - 1)
    for layer in range(args.layers):
        k = torch.randn(L - 1, H, 128, device=dev, dtype=torch.float16, generator=gen)
        v = torch.randn(L - 1, H, 128, device=dev, dtype=torch.float16, generator=gen)
        U.append_kvh(k, v, None, c, layer)
        del k, v
    c.end_forward()
    c.prepare_hadamard(1)
    c.begin_forward(1)
    qkv = torch.randn(3, args.layers, 1, H, 128, device=dev, dtype=torch.float16, generator=gen)
    out = torch.zeros(args.layers, 1, H, 128, device=dev, dtype=torch.float16)

    def step():
        for layer in range(args.layers):
            U.decode_step(qkv[0, layer], qkv[1, layer], qkv[2, layer], c, layer, out=out[layer], record_indices=False)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(args.replays):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    print(f"ctx {L}, {H} heads, budget {args.budget}: {e0.elapsed_time(e1) * 1e3 / 20 / args.layers:.2f} us per layer "
          "(with the stamps)")

    tim = np.zeros((2, 512, 16), dtype=np.uint64)
    fn = _lib.lib.adamas_debug_read_timing
    fn.argtypes = [ctypes.c_void_p]
    fn.restype = ctypes.c_int
    assert fn(tim.ctypes.data) == 0
    tim = tim.astype(np.int64)
    est = tim[0][tim[0][:, 3] > 0]
    sa = tim[1][tim[1][:, 8] > 0]
    base = est[:, 0].min() if len(est) else sa[:, 0].min()
    print("last layer, microseconds after its first estimate block started:")
    for i, name in enumerate(["estimate block resident", "released by its predecessor", "query planes ready",
                              "consumer warps done"]):
        if len(est):
            print(f"  estimate       {name:32s} {_stats(est[:, i] - base)}")
    for i, name in enumerate(["block resident", "released by the estimate", "histogram done", "histograms exchanged",
                              "cut known", "winners compacted", "first tile gathered", "attention done",
                              "partials at rank 0"]):
        print(f"  select+attend  {name:32s} {_stats(sa[:, i] - base)}")
    print(f"  winners per block: min {sa[:, 11].min()} median {int(np.median(sa[:, 11]))} max {sa[:, 11].max()}; "
          f"blocks that needed a second tile: {int((sa[:, 10] > 0).sum())} of {len(sa)}")

    chain = np.zeros((3, 128, 4), dtype=np.uint64)
    seq = np.zeros(3, dtype=np.uint32)
    fn = _lib.lib.adamas_debug_read_chain
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    assert fn(chain.ctypes.data, seq.ctypes.data) == 0
    kid = 1   # the estimate's block 0
    n = min(int(seq[kid]), args.layers, 127)
    starts = sorted(int(chain[kid, (int(seq[kid]) - j) % 128, 1]) for j in range(1, n + 1))
    periods = [round((b - a) / 1e3, 1) for a, b in zip(starts, starts[1:])]
    print("period between the releases of successive layers' estimates (us):", periods)


if __name__ == "__main__":
    main()
