"""The allocation-free decode entry point (adamas_decode_forward_static) against the handler-based
one.  Some users of this library cannot allocate device memory at the moment they need attention: a
server whose allocator has reserved the whole GPU, a latency-critical thread that must not trigger
the device-wide synchronisation of cudaMalloc/cudaFree.  For
them the library keeps a fixed scratch array on the device; this test calls that path through the C
ABI twice in a row (the array is reused and keeps the previous call's contents) and expects the same
output as the normal path.  The file name makes pytest collect it last.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

from oracle import adamas_ref as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL_TOL = 2e-3


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


@pytest.mark.parametrize("L,ps,budget,dtype", [(3000, 16, 512, torch.float16), (700, 1, 96, torch.bfloat16)])
def test_static_scratch_entry_point_matches_handler_path(L, ps, budget, dtype):
    import adamas_b200.utils as U
    from adamas_b200 import _lib

    H = 32
    g = torch.Generator().manual_seed(L)
    k = torch.randn(L, H, 128, generator=g).to(dtype)
    v = torch.randn(L, H, 128, generator=g).to(dtype)
    qs = [torch.randn(1, H, 128, generator=g).to(dtype) for _ in range(2)]

    c = U.InferenceController(1, H, 128, ps, budget // ps, L + ps, dtype, DEV)
    c.prepare_hadamard(L - 1)
    c.begin_forward(L - 1)
    U.append_kvh(k[: L - 1].to(DEV), v[: L - 1].to(DEV), None, c, 0)
    c.end_forward()
    c.prepare_hadamard(1)
    c.begin_forward(1)
    q_code = U.append_qkv_fused(qs[0].to(DEV), k[L - 1:].to(DEV), v[L - 1:].to(DEV), c, 0)
    U.decode_topk(U.decode_estimate(q_code, c, 0), c)
    idx = c.topk_dindices_buffer
    token_granular = ps > 1
    unit = 1 if token_granular else ps
    tail = 1 if token_granular else c.kv_cache.last_page_len
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = _lib.F16 if dtype == torch.float16 else _lib.BF16

    for q in qs:                      # two calls in a row on the shared scratch
        qd = q.to(DEV)
        want = U.decode_sparse_attn(qd, c, 0, idx)
        got = torch.full_like(qd, float("nan"))
        lse = torch.zeros(H, dtype=torch.float32, device=DEV)
        rc = _lib.lib.adamas_decode_forward_static(
            _ptr(qd), _ptr(got), _ptr(lse), _ptr(c.kv_cache.buf_layer(0)), _ptr(idx), idx.stride(0),
            idx.size(1), unit, H, 128, ps, code, int(c.kv_last_page_idx), int(c.kv_cache.last_page_len), tail,
            1.0 / math.sqrt(128.0), stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        atol = REL_TOL * float(want.float().abs().max())
        torch.testing.assert_close(got.float(), want.float(), rtol=REL_TOL, atol=atol)
        assert torch.isfinite(lse).all()
    # and against the oracle, so that both paths are not wrong together
    table = np.asarray(c.kv_cache.indicies)
    r = ref.decode_step(qs[0][0], k, v, budget)
    torch.testing.assert_close(got[0].float().cpu(), ref.sparse_attention(qs[1][0], k, v, r["idx"]),
                               rtol=REL_TOL, atol=REL_TOL * float(want.float().abs().max()))


def test_static_scratch_entry_point_rejects_oversized_requests():
    from adamas_b200 import _lib
    H, ps = 512, 16
    q = torch.zeros(1, H, 128, dtype=torch.float16, device=DEV)
    kv = torch.zeros(2, 2, ps, H, 128, dtype=torch.float16, device=DEV)
    idx = torch.zeros(H, 4, dtype=torch.int32, device=DEV)
    rc = _lib.lib.adamas_decode_forward_static(
        _ptr(q), _ptr(q), None, _ptr(kv), _ptr(idx), 4, 4, 1, H, 128, ps, _lib.F16, 1, 1, 1, 0.1,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == _lib.ERR_INVALID and "at most 256 heads" in _lib.last_error()
