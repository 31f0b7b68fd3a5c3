"""Generate the golden fixtures in this directory from the reference's own Python code.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

What runs is the reference's code, unmodified, on the CPU:

* adamas/tests/test_estimate.py: ``pack_2bit`` (bit layout of the packed codes) and
  ``_ref_cpu_estimate`` (bucketize + pairwise_distance, newest token excluded);
* adamas/tests/test_approx_attention.py: ``_ref_self_approx_attention`` (top budget-1
  tokens plus the newest token, masked fp32 softmax, @ V);
* adamas/utils/{kv_cache,controller}.py: ``InferenceController`` page bookkeeping.

Two extension modules the reference imports are not available anywhere (their
sources are third-party and absent from the checkout), so they are stubbed:

* ``faster_hadamard_transform`` -> the oracle's Walsh-Hadamard transform
  (oracle/adamas_ref.py).  The reference's tests use that library on both sides of
  every comparison, so this stub leaves every other stage pinned by reference code.
* ``adamas._kernels`` -> an object whose decode-wrapper methods do nothing (only the
  controller's host bookkeeping is recorded; no kernel result is taken from it).

The package ``adamas`` itself is registered as an empty namespace so that its
``__init__`` (which pulls in a Llama model needing transformers 4.45) does not run.
"""
from __future__ import annotations

import importlib.util
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import adamas_ref as ref  # noqa: E402


def _install_stubs(ref_root: str):
    pkg = types.ModuleType("adamas")
    pkg.__path__ = [os.path.join(ref_root, "adamas")]
    sys.modules["adamas"] = pkg

    class _Wrapper:
        def __init__(self, layout):
            self.layout = layout

        def begin_forward(self, *a):
            pass

        def end_forward(self):
            pass

        def forward(self, *a):
            raise RuntimeError("kernel stub")

    k = types.ModuleType("adamas._kernels")
    k.BatchDecodeWithPagedKVCachePyTorchWrapper = _Wrapper
    sys.modules["adamas._kernels"] = k
    pkg._kernels = k

    fht = types.ModuleType("faster_hadamard_transform")

    def hadamard_transform(x, inplace=False):
        y = ref.hadamard_transform(x, scale=_SCALE[0])
        if inplace:
            x.copy_(y)
            return x
        return y

    fht.hadamard_transform = hadamard_transform
    sys.modules["faster_hadamard_transform"] = fht


_SCALE = [None]


def _load(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root: str):
    _install_stubs(ref_root)
    t_est = _load(os.path.join(ref_root, "adamas/tests/test_estimate.py"), "ref_test_estimate")
    t_att = _load(os.path.join(ref_root, "adamas/tests/test_approx_attention.py"), "ref_test_approx")
    import adamas.utils as ref_utils  # the reference's host runtime

    torch.set_num_threads(4)
    cases = {}
    # (name, kv_len, heads, budget, input sigma, hadamard scale)
    specs = [
        ("n27", 27, 4, 8, 1.0, None),
        ("n61", 61, 4, 16, 1.0, None),
        ("n113", 113, 4, 64, 1.0, None),
        ("n241", 241, 4, 112, 1.0, None),
        # wide inputs and an unnormalised transform: all four buckets and the
        # {1,2} code pairs (where L1 and the XOR metric differ) occur
        ("wide97", 97, 4, 32, 3.0, 1.0),
    ]
    for name, kv_len, heads, budget, sigma, scale in specs:
        _SCALE[0] = scale
        g = torch.Generator().manual_seed(1234 + kv_len)
        q = (torch.randn(1, heads, 128, generator=g) * sigma).to(torch.float16)
        k = (torch.randn(kv_len, heads, 128, generator=g) * sigma).to(torch.float16)
        v = torch.randn(kv_len, heads, 128, generator=g).to(torch.float16)

        thresholds = torch.tensor([-10, 0, 10])
        import faster_hadamard_transform as fht
        q_code_ref = t_est.pack_2bit(
            torch.bucketize(fht.hadamard_transform(q, inplace=False), thresholds, out_int32=True),
            torch.float16)
        est_ref = t_est._ref_cpu_estimate(q, k, v)                     # [H, kv_len-1] fp16
        o_ref, topk_ref = t_att._ref_self_approx_attention(q, k, v, budget)
        cases[name] = dict(
            q=q.view(torch.int16).numpy(), k=k.view(torch.int16).numpy(), v=v.view(torch.int16).numpy(),
            budget=np.int64(budget), scale=np.float64(-1.0 if scale is None else scale),
            q_code=q_code_ref.view(torch.int16).numpy(),
            est=est_ref.view(torch.int16).numpy(),
            o=o_ref.view(torch.int16).numpy(),
            topk=topk_ref.numpy().astype(np.int32),
        )
    flat = {f"{c}.{f}": a for c, d in cases.items() for f, a in d.items()}
    np.savez_compressed(os.path.join(HERE, "ref_python_path.npz"), **flat)

    # host bookkeeping trace of the reference InferenceController (CPU tensors)
    trace = []
    for page_size, prefill, steps, budget in [(1, 37, 6, 16), (1, 9, 4, 64)]:
        c = ref_utils.InferenceController(2, 4, 128, page_size, budget, 256, torch.float16, "cpu")
        rec = dict(page_size=page_size, prefill=prefill, steps=steps, budget=budget, states=[])

        def snap(c):
            return dict(
                kv_pages=list(c.kv_cache.indicies), code_pages=list(c.hadamard_cache.indicies),
                kv_seqlen=c.kv_cache.seqlen, code_seqlen=c.hadamard_cache.seqlen,
                kv_last_page_len=c.kv_cache.last_page_len, code_last_page_len=c.hadamard_cache.last_page_len,
                kv_last_page_idx=int(c.kv_last_page_idx), code_last_page_idx=int(c.hadamard_last_page_idx),
                kv_indptr_for_append=c.kv_indptr_for_append.tolist(),
                hadamard_indptr_for_append=c.hadamard_indptr_for_append.tolist(),
                kv_indices_with_last=c.kv_indices_with_last.tolist(),
                hadamard_indices=c.hadamard_indices.tolist(),
                kv_indices_without_last=None if c.kv_indices_without_last is None else c.kv_indices_without_last.tolist(),
                inference_page_budget=c.inference_page_budget,
                kv_indptr_for_approx_decode=None if c.kv_indptr_for_approx_decode is None else c.kv_indptr_for_approx_decode.tolist(),
                need_estimate=bool(c.need_estimate()),
                topk_shapes=None if c.topk_dout_buffer is None else [list(c.topk_dout_buffer.shape), list(c.topk_dindices_buffer.shape), list(c.topk_buf.shape)],
            )

        c.prepare_hadamard(prefill)
        c.begin_forward(prefill)
        rec["states"].append(snap(c))
        c.end_forward()
        for _ in range(steps):
            c.prepare_hadamard(1)
            c.begin_forward(1)
            rec["states"].append(snap(c))
            c.end_forward()
        trace.append(rec)
    with open(os.path.join(HERE, "ref_controller_trace.json"), "w") as f:
        json.dump(trace, f)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path of a checkout of the reference project>")
    main(sys.argv[1])
