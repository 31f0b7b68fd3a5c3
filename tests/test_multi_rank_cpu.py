"""Host-side logic of the multi-GPU partitionings, run as world_size-2 gloo ranks on CPU with the
oracle standing in for the CUDA operators (test-only stand-ins; the package itself never imports
the oracle)."""
import math
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import adamas_ref as ref

LN2 = math.log(2.0)


class OracleOps:
    """CPU stand-in with the interface adamas_b200.sharding expects, for one token shard."""

    def __init__(self, q, k_shard, v_shard, owns_tail):
        self.q, self.k, self.v, self.owns_tail = q, k_shard, v_shard, owns_tail
        self.q_code = ref.encode(q)
        self.k_codes = ref.encode(k_shard)
        self.dist = None

    def local_histograms(self, k):
        n = self.k.shape[0] - (1 if self.owns_tail else 0)
        h = self.q.shape[0]
        hist = np.zeros((h, 512), dtype=np.int32)
        self.dist = np.zeros((h, 0), dtype=np.int64)
        if n > 0:
            self.dist = ref.code_distance(self.q_code, self.k_codes[:n])
            for head in range(h):
                hist[head] = np.bincount(self.dist[head], minlength=512)
        return torch.from_numpy(hist)

    def cut(self, all_hists, rank, k):
        a = all_hists.numpy().astype(np.int64)                    # [G, H, 512]
        h = a.shape[1]
        out = np.zeros((h, 2), dtype=np.int32)
        for head in range(h):
            tot = a[:, head].sum(0)
            cum = np.cumsum(tot)
            if cum[-1] < k:
                out[head] = (512, 0)
                continue
            cut = int(np.searchsorted(cum, k))                    # first bin with cum >= k
            need = k - (cum[cut] - tot[cut])
            low = a[:rank, head, cut].sum()
            out[head] = (cut, max(0, min(need - low, a[rank, head, cut])))
        return torch.from_numpy(out)

    def select_attend(self, q, ext_cut, k):
        h, d = q.shape
        o = torch.zeros(h, d)
        lse = torch.full((h,), -float("inf"))
        idx = torch.full((h, k), -1, dtype=torch.int32)
        for head in range(h):
            cut, take = int(ext_cut[head, 0]), int(ext_cut[head, 1])
            row = self.dist[head]
            tok = np.sort(np.concatenate([np.flatnonzero(row < cut), np.flatnonzero(row == cut)[:take]])).tolist()
            idx[head, : len(tok)] = torch.tensor(tok, dtype=torch.int32)
            if self.owns_tail:
                tok = tok + [self.k.shape[0] - 1]
            if tok:
                oo, ll = ref.sparse_attention(q[head:head + 1], self.k[:, head:head + 1], self.v[:, head:head + 1],
                                              np.asarray([tok]), return_lse=True)
                o[head] = oo[0]
                lse[head] = ll[0] / LN2
        return o, lse, idx

    def merge(self, o_parts, lse_parts):
        return ref.merge_states(o_parts, lse_parts * LN2)[0]


def _inputs(L, H, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(H, 128, generator=g).to(torch.float16)
    k = torch.randn(L, H, 128, generator=g).to(torch.float16)
    v = torch.randn(L, H, 128, generator=g).to(torch.float16)
    return q, k, v


def _worker(rank, world, port, L, H, budget, page_size, q_out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from adamas_b200 import sharding
        q, k, v = _inputs(L, H, 11)
        t0, t1 = sharding.token_range(L, world, rank, page_size)
        ops = OracleOps(q, k[t0:t1], v[t0:t1], owns_tail=(t1 == L))
        o, mine = sharding.sequence_sharded_step(ops, q, budget)
        glob = torch.where(mine >= 0, mine + t0, mine)
        # head-sharded gather of a layer output
        h0, h1 = sharding.head_range(H, world, rank)
        full = sharding.gather_heads(o[None, h0:h1].contiguous())
        q_out.put((rank, o.numpy(), glob.numpy(), full.numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("L,budget,page_size", [(700, 65, 16), (300, 200, 1)])
def test_sequence_sharded_step_two_gloo_ranks(L, budget, page_size):
    H, world = 4, 2
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, L, H, budget, page_size, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    q, k, v = _inputs(L, H, 11)
    want = ref.decode_step(q, k, v, budget)
    union = [set() for _ in range(H)]
    for rank, o, glob, full in results:
        np.testing.assert_allclose(o, want["out"].numpy(), rtol=1e-4, atol=1e-5)     # every rank holds the result
        np.testing.assert_allclose(full[0], o, rtol=0, atol=0)                       # head gather reassembles it
        for h in range(H):
            union[h] |= {int(t) for t in glob[h] if t >= 0}
    for h in range(H):
        assert union[h] == set(want["sel"][h].tolist())                              # same winners as one GPU


def test_sequence_sharded_local_driver_matches_single_device():
    from adamas_b200 import sharding
    L, H, budget = 1000, 3, 129
    q, k, v = _inputs(L, H, 5)
    for world in (1, 2, 3, 8):
        ops = []
        for rank in range(world):
            t0, t1 = sharding.token_range(L, world, rank, 16)
            if t1 > t0:
                ops.append(OracleOps(q, k[t0:t1], v[t0:t1], owns_tail=(t1 == L)))
        o, _ = sharding.sequence_sharded_step_local(ops, q, budget)
        torch.testing.assert_close(o, ref.decode_step(q, k, v, budget)["out"], rtol=1e-4, atol=1e-5)


def test_partition_helpers():
    from adamas_b200 import sharding
    assert sharding.head_range(32, 8, 7) == (28, 32)
    with pytest.raises(ValueError):
        sharding.head_range(30, 8, 0)
    spans = [sharding.token_range(1000, 8, r, 16) for r in range(8)]
    assert spans[0][0] == 0 and spans[-1][1] == 1000
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert all(s[0] % 16 == 0 for s in spans)
    assert sharding.token_range(10, 4, 3, 16) == (10, 10)      # more ranks than pages: empty shards
