"""Multi-GPU partitioning of the decode path (one process per GPU, torch.distributed).

The reference is single-GPU (device fixed to cuda:0, adamas/models/llama.py:526; batch 1,
adamas/models/Adamas.py:83).  Two partitionings are provided on top of the single-GPU operators:

* by KV head: rank g owns heads [g*H/G, (g+1)*H/G) with its own KV and code caches and runs the
  unchanged single-GPU path on them; the only communication is the gather of the layer output
  (`gather_heads`).
* by sequence (million-token contexts): rank g owns a contiguous token range for all heads.  Per
  layer-step (`sequence_sharded_step`):
    1. local distances and a local top-(budget-1) (values + local slots, ascending position);
    2. all-gather of the candidate VALUES only ([G, H, budget-1] 16-bit);
    3. every rank selects the global budget-1 smallest among the G*(budget-1) candidates laid out
       rank-major, so that "lower position wins a tie" means lower rank, then lower local index:
       the same rule as on one GPU; each rank keeps its own winners (holes are -1);
    4. local attention over the winners (the rank that owns the newest token adds it), giving a
       partial (o, lse);
    5. all-gather of the partials and a merge (same rule as the split-KV merge inside one GPU).
  No K/V or code bytes ever cross the link.

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
@dataclass
class LocalCandidates:
    values: torch.Tensor   # [H, K] 16-bit distances (fp16 or int16), padded with the largest key
    slots: torch.Tensor    # [H, K] int32 local token slots of the candidates, -1 where padded
    count: int             # valid candidates per head (same for all heads)


def pad_value(dtype: torch.dtype):
    """A value that sorts after every real distance."""
    return float("inf") if dtype == torch.float16 else 0x7FFF


def sequence_sharded_step(ops, q: torch.Tensor, budget: int, group=None):
    """One layer's decode step over a sequence split across the ranks of `group`.

    `ops` provides, for this rank's shard:
      ops.local_candidates(k) -> LocalCandidates with K == k columns: the rank's k smallest distances
          (fewer if the shard is shorter; padded), ascending local position;
      ops.select(values [H, n], k) -> int64/int32 [H, k] positions of the k smallest, ties to the lower
          position, ascending;
      ops.attend(q, slots [H, m] with -1 holes, with_tail: bool) -> (o [H, D] fp32, lse [H] fp32 base 2);
      ops.merge(o_parts [G, H, D], lse_parts [G, H]) -> o [H, D];
      ops.owns_tail: this rank holds the newest token.
    Returns (o [H, D], selected [H, budget-1] int64 as rank * K + local candidate number).
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    k = budget - 1
    cand = ops.local_candidates(k)
    h = cand.values.size(0)

    # 16-bit integers travel as fp16 bit patterns (all-gather only copies; NCCL has no int16 type)
    wire = cand.values.contiguous()
    as_int = wire.dtype in (torch.int16, torch.uint16)
    if as_int:
        wire = wire.view(torch.float16)
    gathered = [torch.empty_like(wire) for _ in range(world)]
    dist.all_gather(gathered, wire, group=group)
    table = torch.stack(gathered, dim=1).reshape(h, world * k)        # rank-major candidate table
    if as_int:
        table = table.view(cand.values.dtype)
    sel = ops.select(table, k).to(torch.int64)                        # [H, k] positions in the table

    slots = winners_of_rank(sel, cand.slots, rank)

    o_part, lse_part = ops.attend(q, slots, ops.owns_tail)
    o_all = [torch.empty_like(o_part) for _ in range(world)]
    l_all = [torch.empty_like(lse_part) for _ in range(world)]
    dist.all_gather(o_all, o_part.contiguous(), group=group)
    dist.all_gather(l_all, lse_part.contiguous(), group=group)
    o = ops.merge(torch.stack(o_all), torch.stack(l_all))
    return o, sel


def winners_of_rank(sel: torch.Tensor, cand_slots: torch.Tensor, rank: int) -> torch.Tensor:
    """sel [H, k] positions in the rank-major candidate table, cand_slots [H, k] this rank's candidate
    slots -> int32 [H, k]: the rank's own winners' slots, -1 elsewhere."""
    k = cand_slots.size(1)
    sel = sel.to(torch.int64)
    mine = (sel // k) == rank
    local_no = (sel % k).clamp(0, k - 1)
    slots = torch.gather(cand_slots.to(torch.int64), 1, local_no)
    return torch.where(mine, slots, torch.full_like(slots, -1)).to(torch.int32).contiguous()


def sequence_sharded_step_local(ops_list, q: torch.Tensor, budget: int):
    """The same protocol with all shards driven by one process (shards of one GPU, or CPU stand-ins):
    the collectives become concatenations.  Returns (o [H, D], sel [H, budget-1])."""
    k = budget - 1
    cands = [ops.local_candidates(k) for ops in ops_list]
    h = cands[0].values.size(0)
    table = torch.stack([c.values for c in cands], dim=1).reshape(h, len(ops_list) * k)
    sel = ops_list[0].select(table, k).to(torch.int64)
    parts = []
    for rank, (ops, cand) in enumerate(zip(ops_list, cands)):
        parts.append(ops.attend(q, winners_of_rank(sel, cand.slots, rank), ops.owns_tail))
    o = ops_list[0].merge(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]))
    return o, sel


class CudaOps:
    """The CUDA operators of this package on one rank's shard (an InferenceController that holds
    the rank's token range as its own sequence).  The rank that owns the newest token has appended
    it like any decode step; the other ranks' controllers hold only past tokens."""

    def __init__(self, controller, layer_idx: int, q_code: torch.Tensor, owns_tail: bool):
        from . import _kernels
        self.k = _kernels
        self.c = controller
        self.layer = layer_idx
        self.q_code = q_code
        self.owns_tail = owns_tail
        w = controller._decode_handler._wrapper
        if not w._started:   # a shard without the newest token never went through a decode begin_forward
            controller._decode_handler.begin_forward(torch.zeros(2, dtype=torch.int32), controller.num_heads,
                                                     controller.num_heads, controller.head_dim,
                                                     controller.page_size, controller.dtype)

    def _n_local(self) -> int:
        # the tail owner's newest token is excluded from the estimate, as on one GPU
        return self.c.hadamard_cache.seqlen - (1 if self.owns_tail else 0)

    def local_candidates(self, k: int) -> LocalCandidates:
        c = self.c
        n = self._n_local()
        dev = self.q_code.device
        vdtype = torch.float16 if c.dtype == torch.float16 else torch.int16
        values = torch.full((c.num_heads, k), pad_value(vdtype), dtype=vdtype, device=dev)
        slots = torch.full((c.num_heads, k), -1, dtype=torch.int32, device=dev)
        kk = min(k, n)
        if kk > 0:
            dist_buf = c.estimate_buffer(n)
            self.k.estimate_attn_score(self.q_code, dist_buf, c.hadamard_cache.buf_layer(self.layer),
                                       c.hadamard_indices, None, c.hadamard_cache.last_page_len,
                                       c.hadamard_last_page_idx, c.layout, exclude_last=self.owns_tail)
            self.k.topk_select(dist_buf, kk, slots[:, :kk], values[:, :kk], page_table=c.kv_indices_with_last,
                               page_size=c.page_size)
        return LocalCandidates(values, slots, kk)

    def select(self, values: torch.Tensor, k: int) -> torch.Tensor:
        out = torch.empty((values.size(0), k), dtype=torch.int32, device=values.device)
        self.k.topk_select(values.contiguous(), k, out)
        return out

    def attend(self, q: torch.Tensor, slots: torch.Tensor, with_tail: bool):
        c = self.c
        o = torch.empty((c.num_heads, c.head_dim), dtype=torch.float32, device=q.device)
        lse = torch.empty(c.num_heads, dtype=torch.float32, device=q.device)
        w = c._decode_handler._wrapper
        w.forward(q, torch.empty(0), c.kv_cache.buf_layer(self.layer), slots, None, c.kv_cache.last_page_len,
                  c.kv_last_page_idx, token_granular=True, lse=lse, tail_len=1 if with_tail else 0, o_f32=o)
        return o, lse

    def merge(self, o_parts: torch.Tensor, lse_parts: torch.Tensor) -> torch.Tensor:
        h, d = o_parts.shape[1], o_parts.shape[2]
        out = torch.empty((h, d), dtype=self.c.dtype, device=o_parts.device)
        self.k.merge_states(o_parts.contiguous(), lse_parts.contiguous(), out)
        return out
