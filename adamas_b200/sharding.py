"""Multi-GPU partitioning of the decode path (one process per GPU, torch.distributed).

The reference is single-GPU (device fixed to cuda:0, adamas/models/llama.py:526; batch 1,
adamas/models/Adamas.py:83).  Two partitionings are provided on top of the single-GPU operators:

* by KV head: rank g owns heads [g*H/G, (g+1)*H/G) with its own KV and code caches and runs the
  unchanged single-GPU path on them; the only communication is the gather of the layer output
  (`gather_heads`).
* by sequence (million-token contexts): rank g owns a contiguous token range for all heads.  Per
  layer-step (`sequence_sharded_step`):
    1. local distances, counted into a 512-bin histogram per head (a distance is at most 384);
    2. all-gather of the histograms ([G, H, 512] int32, 64 KB per rank at 32 heads);
    3. every rank derives the same cut distance of the budget-1 smallest distances of the whole
       sequence and its own share of the cut-valued ones (ranks hold ascending token ranges, so
       "lower position wins a tie" means lower rank first, then lower local index: the single-GPU
       rule), and selects exactly its winners locally;
    4. local attention over them (the rank that owns the newest token adds it): a partial
       (o fp32, lse);
    5. all-gather of the partials ([G, H, 129] fp32) and a merge (same rule as the split-KV merge
       inside one GPU, kernels/include/decode/decode_attn.cuh:264-283, 1050-1059).
  Two collectives; no K/V, code or candidate bytes ever cross the link.

The numerical operators are injected (`ops`), so the protocol can be exercised on CPU ranks (gloo)
with stand-in operators and on GPUs with the CUDA ones (`CudaOps`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist


# ------------------------------------------------------------------------------------------------
# partitioning helpers
# ------------------------------------------------------------------------------------------------
def head_range(num_heads: int, world: int, rank: int) -> Tuple[int, int]:
    if num_heads % world != 0:
        raise ValueError(f"{num_heads} heads do not divide over {world} ranks")
    per = num_heads // world
    return rank * per, (rank + 1) * per


def token_range(seq_len: int, world: int, rank: int, page_size: int = 1) -> Tuple[int, int]:
    """Contiguous token range of `rank`, aligned to pages; the last rank takes the remainder."""
    pages = (seq_len + page_size - 1) // page_size
    per = (pages + world - 1) // world * page_size
    t0 = min(seq_len, rank * per)
    t1 = min(seq_len, (rank + 1) * per)
    return t0, t1


def gather_heads(o_local: torch.Tensor, group=None) -> torch.Tensor:
    """o_local [1, H/G, D] on every rank -> [1, H, D] on every rank (head-sharded layer output)."""
    world = dist.get_world_size(group)
    if world == 1:
        return o_local
    parts = [torch.empty_like(o_local) for _ in range(world)]
    dist.all_gather(parts, o_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)


# ------------------------------------------------------------------------------------------------
# sequence-sharded decode step
# ------------------------------------------------------------------------------------------------
def sequence_sharded_step(ops, q: torch.Tensor, budget: int, group=None):
    """One layer's decode step over a sequence split across the ranks of `group`.

    `ops` provides, for this rank's shard:
      ops.local_histograms(k) -> int32 [H, 512]: counts of the shard's distances per head (it also
          leaves the distances where ops.select_attend finds them);
      ops.cut(all_hists [G, H, 512], rank, k) -> int32 [H, 2]: (cut distance, cut-valued elements
          this rank takes);
      ops.select_attend(q, ext_cut, k) -> (o [H, D] fp32, lse [H] fp32 base 2, idx int32 [H, k]: the
          rank's winners as local token slots, ascending position, -1 beyond their number);
      ops.merge(o_parts [G, H, D], lse_parts [G, H]) -> o [H, D].
    Returns (o [H, D], idx).  The whole sequence must hold at least budget - 1 tokens besides the
    newest one.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    k = budget - 1
    hist = ops.local_histograms(k).contiguous()
    # (gathered along the first dimension, then viewed by rank: the layout every backend accepts)
    all_hists = torch.empty((world * hist.size(0), hist.size(1)), dtype=hist.dtype, device=hist.device)
    dist.all_gather_into_tensor(all_hists, hist, group=group)
    ext_cut = ops.cut(all_hists.view(world, hist.size(0), hist.size(1)), rank, k)
    o_part, lse_part, idx = ops.select_attend(q, ext_cut, k)
    packed = torch.cat((o_part, lse_part.unsqueeze(1)), dim=1).contiguous()          # [H, D + 1]
    gathered = torch.empty((world * packed.size(0), packed.size(1)), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(gathered, packed, group=group)
    gathered = gathered.view(world, packed.size(0), packed.size(1))
    d = o_part.size(1)
    o = ops.merge(gathered[:, :, :d].contiguous(), gathered[:, :, d].contiguous())
    return o, idx


def sequence_sharded_step_local(ops_list, q: torch.Tensor, budget: int):
    """The same protocol with all shards driven by one process (shards of one GPU, or CPU stand-ins):
    the collectives become stacks.  Returns (o [H, D], [idx of every shard])."""
    k = budget - 1
    all_hists = torch.stack([ops.local_histograms(k) for ops in ops_list]).contiguous()
    parts, idxs = [], []
    for rank, ops in enumerate(ops_list):
        o_part, lse_part, idx = ops.select_attend(q, ops.cut(all_hists, rank, k), k)
        parts.append((o_part, lse_part))
        idxs.append(idx)
    o = ops_list[0].merge(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]))
    return o, idxs


class CudaOps:
    """The CUDA operators of this package on one rank's shard (an InferenceController that holds
    the rank's token range as its own sequence).  The rank that owns the newest token has appended
    it like any decode step; the other ranks' controllers hold only past tokens.  A shard may be
    empty (more ranks than pages): it contributes empty histograms and an empty partial."""

    def __init__(self, controller, layer_idx: int, q_code: torch.Tensor, owns_tail: bool):
        from . import _kernels
        self.k = _kernels
        self.c = controller
        self.layer = layer_idx
        self.q_code = q_code
        self.owns_tail = owns_tail
        h, dev = controller.num_heads, q_code.device
        # buffers of the step, made once
        self._hist_out = torch.zeros(h, 512, dtype=torch.int32, device=dev)
        self._ext = torch.zeros(h, 2, dtype=torch.int32, device=dev)
        self._o = torch.zeros(h, controller.head_dim, dtype=torch.float32, device=dev)
        self._lse = torch.full((h,), -float("inf"), dtype=torch.float32, device=dev)
        self._slices = 0

    def _n_local(self) -> int:
        # the tail owner's newest token is excluded from the estimate, as on one GPU
        return self.c.hadamard_cache.seqlen - (1 if self.owns_tail else 0)

    def local_histograms(self, k: int) -> torch.Tensor:
        c = self.c
        n = self._n_local()
        if n <= 0:
            self._hist_out.zero_()
            return self._hist_out
        # (the slice count depends on the shard's length and on the upper bound of its winners)
        self._slices = self.k.select_attend_slices(n, max(1, min(k, n)), c.num_heads)
        # (from about 3 M distances per launch a counting launch of its own is cheaper than one L2 atomic
        # per distance from inside the estimate)
        count_apart = c.num_heads * n >= (3 << 20)
        dist = c.distance_scratch(n)
        self.k.estimate_attn_score(self.q_code, dist, c.hadamard_cache.buf_layer(self.layer),
                                   c.hadamard_indices, None, c.hadamard_cache.last_page_len,
                                   c.hadamard_last_page_idx, c.layout, exclude_last=self.owns_tail,
                                   hist=None if count_apart else c.hist_scratch, hist_slices=self._slices)
        if count_apart:
            self.k.dist_histograms(dist, c.hist_scratch, self._slices)
        self.k.hist_rowsum(c.hist_scratch, self._slices, self._hist_out)
        return self._hist_out

    def cut(self, all_hists: torch.Tensor, rank: int, k: int) -> torch.Tensor:
        self.k.global_cut(all_hists.contiguous(), rank, k, self._ext)
        return self._ext

    def select_attend(self, q: torch.Tensor, ext_cut: torch.Tensor, k: int):
        c = self.c
        n = self._n_local()
        idx = torch.full((c.num_heads, k), -1, dtype=torch.int32, device=q.device)
        if n <= 0:
            if not self.owns_tail:
                self._o.zero_()
                self._lse.fill_(-float("inf"))
                return self._o, self._lse, idx
            raise RuntimeError("the shard that owns the newest token must hold at least one older token")
        kk = max(1, min(k, n))
        assert self.k.select_attend_slices(n, kk, c.num_heads) == self._slices, "histograms were built for another shape"
        qq = q if q.dim() == 3 else q.unsqueeze(0)
        self.k.select_attend(c.distance_scratch(n), kk, qq, None, c.kv_cache.buf_layer(self.layer),
                             c.kv_cache.table_device(), c.kv_cache.last_page_len if self.owns_tail else 0,
                             c.kv_cache.indicies[-1], indices_out=idx[:, :kk],
                             lse=self._lse, hist=c.hist_scratch, hist_ready=True, ext_cut=ext_cut, o_f32=self._o)
        return self._o, self._lse, idx

    def merge(self, o_parts: torch.Tensor, lse_parts: torch.Tensor) -> torch.Tensor:
        h, d = o_parts.shape[1], o_parts.shape[2]
        out = torch.empty((h, d), dtype=self.c.dtype, device=o_parts.device)
        self.k.merge_states(o_parts.contiguous(), lse_parts.contiguous(), out)
        return out
