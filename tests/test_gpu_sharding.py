"""Sequence- and head-sharded decode with the CUDA operators: all shards on one GPU driven by one
process (the collectives become concatenations), and, when two GPUs are visible, two NCCL ranks."""
import os

import numpy as np
import pytest
import torch

from oracle import adamas_ref as ref

pytestmark = pytest.mark.gpu
REL_TOL = 2e-3


def _inputs(L, H, seed, dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, H, 128, generator=g).to(dtype)
    k = torch.randn(L, H, 128, generator=g).to(dtype)
    v = torch.randn(L, H, 128, generator=g).to(dtype)
    return q, k, v


def _make_shard(dev, q, k, v, t0, t1, L, ps, dtype):
    """A controller holding tokens [t0, t1) and the CudaOps on it."""
    import adamas_b200.utils as U
    from adamas_b200 import _kernels as K, sharding
    H = k.shape[1]
    n = t1 - t0
    owns_tail = t1 == L
    c = U.InferenceController(1, H, 128, ps, 1 << 20, n + ps, dtype, dev)
    kd, vd, qd = k[t0:t1].to(dev), v[t0:t1].to(dev), q.to(dev)
    n_pre = n - 1 if owns_tail else n
    if n_pre > 1:
        c.prepare_hadamard(n_pre)
        c.begin_forward(n_pre)
        U.append_kvh(kd[:n_pre].contiguous(), vd[:n_pre].contiguous(), None, c, 0)
        c.end_forward()
    elif n_pre == 1:
        c.prepare_hadamard(1)
        c.begin_forward(2)
        h = K.hadamard_transform(torch.cat((qd, kd[:1]), 0))
        U.append_kvh(kd[:1].contiguous(), vd[:1].contiguous(), h, c, 0)
        c.end_forward()
    if owns_tail:
        c.prepare_hadamard(1)
        c.begin_forward(1)
        q_code = U.append_qkv_fused(qd, kd[n - 1:].contiguous(), vd[n - 1:].contiguous(), c, 0)
    else:
        q_code = torch.empty(1, H, 16, dtype=dtype, device=dev)
        K.bucketize_pack(K.hadamard_transform(qd), q_code)
    return sharding.CudaOps(c, 0, q_code, owns_tail), qd


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("L,budget,ps,dtype", [(3000, 257, 16, torch.float16), (1200, 1024, 16, torch.bfloat16),
                                                (500, 64, 1, torch.float16)])
def test_sequence_sharded_on_one_gpu(world, L, budget, ps, dtype):
    from adamas_b200 import sharding
    dev = "cuda:0"
    H = 8
    q, k, v = _inputs(L, H, L + world, dtype)
    ops, qd = [], None
    spans = []
    for rank in range(world):
        t0, t1 = sharding.token_range(L, world, rank, ps)
        if t1 > t0:
            o, qd = _make_shard(dev, q, k, v, t0, t1, L, ps, dtype)
            ops.append(o)
            spans.append(t0)
    out, idxs = sharding.sequence_sharded_step_local(ops, qd[0], budget)
    torch.cuda.synchronize()
    want = ref.decode_step(q[0], k, v, budget)
    got = out.float().cpu()
    atol = REL_TOL * float(want["out"].abs().max())
    torch.testing.assert_close(got, want["out"], rtol=REL_TOL, atol=atol)
    # winners: map each rank's local slots back to global token numbers
    union = [set() for _ in range(H)]
    for rank, (o, idx) in enumerate(zip(ops, idxs)):
        mine = idx.cpu().numpy()
        table = np.asarray(o.c.kv_cache.indicies)
        inv = np.full(table.max() + 1, -1)
        inv[table] = np.arange(len(table))
        for h in range(H):
            s = mine[h][mine[h] >= 0]
            logical = inv[s // ps] * ps + s % ps
            assert np.all(np.diff(logical) > 0)                      # ascending position order
            union[h] |= set((logical + spans[rank]).tolist())
    for h in range(H):
        assert union[h] == set(want["sel"][h].tolist())
    from adamas_b200 import _lib, _kernels as K
    assert _lib.device_error(clear=False) == 0
    for o in ops:
        assert int(K.histogram_counts(o.c.hist_scratch).abs().sum().item()) == 0


def test_holes_and_empty_lists_in_the_index_list():
    """negative entries are skipped; a head with nothing to attend gets zeros and lse = -inf"""
    import adamas_b200.utils as U
    dev = "cuda:0"
    L, H, ps = 400, 4, 16
    q, k, v = _inputs(L, H, 3)
    ops, qd = _make_shard(dev, q, k, v, 0, L, L + 1, ps, torch.float16)   # holds no "newest" token
    c = ops.c
    table = np.asarray(c.kv_cache.indicies)
    rng = np.random.default_rng(0)
    logical = np.stack([np.sort(rng.choice(L, size=100, replace=False)) for _ in range(H)])
    slots = table[logical // ps] * ps + logical % ps
    holes = rng.random((H, 100)) < 0.3
    holes[3, :] = True                                    # head 3: everything masked
    slots_t = torch.from_numpy(np.where(holes, -1, slots).astype(np.int32)).to(dev)
    o = torch.empty((H, 128), dtype=torch.float32, device=dev)
    lse = torch.empty(H, dtype=torch.float32, device=dev)
    w = c._decode_handler._wrapper
    if not w._started:
        c._decode_handler.begin_forward(torch.zeros(2, dtype=torch.int32), H, H, 128, ps, torch.float16)
    w.forward(qd, torch.empty(0), c.kv_cache.buf_layer(0), slots_t, None, c.kv_cache.last_page_len,
              c.kv_cache.indicies[-1], token_granular=True, lse=lse, tail_len=0, o_f32=o)
    for h in range(H):
        keep = logical[h][~holes[h]]
        if len(keep) == 0:
            assert float(o[h].abs().max()) == 0.0 and lse[h].item() == -float("inf")
        else:
            want = ref.sparse_attention(q[0, h:h + 1], k[:, h:h + 1], v[:, h:h + 1], keep[None])
            torch.testing.assert_close(o[h].cpu(), want[0], rtol=REL_TOL, atol=REL_TOL * float(want.abs().max()))


def _nccl_worker(rank, world, port, L, H, budget, ps, q_out):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from adamas_b200 import sharding
        q, k, v = _inputs(L, H, 21)
        t0, t1 = sharding.token_range(L, world, rank, ps)
        ops, qd = _make_shard(dev, q, k, v, t0, t1, L, ps, torch.float16)
        out, _ = sharding.sequence_sharded_step(ops, qd[0], budget)
        h0, h1 = sharding.head_range(H, world, rank)
        full = sharding.gather_heads(out[None, h0:h1].contiguous())
        torch.cuda.synchronize()
        q_out.put((rank, out.float().cpu().numpy(), full.float().cpu().numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_sharded_two_nccl_ranks():
    import torch.multiprocessing as mp
    L, H, budget, ps, world = 5000, 8, 513, 16, 2
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = 29600 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_nccl_worker, args=(r, world, port, L, H, budget, ps, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    q, k, v = _inputs(L, H, 21)
    want = ref.decode_step(q[0], k, v, budget)["out"].numpy()
    for rank, out, full in results:
        np.testing.assert_allclose(out, want, rtol=REL_TOL, atol=REL_TOL * np.abs(want).max())
        np.testing.assert_allclose(full[0], out, rtol=0, atol=0)
