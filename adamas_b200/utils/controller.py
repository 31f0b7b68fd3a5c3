"""Per-sequence decode state: the surface of the reference's InferenceController
(adamas/utils/controller.py) on top of device-resident page tables.

Differences from the reference, none of which change what its callers see at page_size 1:

* page tables live in persistent device buffers that grow by the new entries only; the reference
  rebuilds three O(context) tensors from Python lists on every decode step (controller.py:86-111);
* ``kv_indices_without_last`` is a stride-0 view [H, pages-1] instead of H materialised copies;
* the small ``*_indptr_*`` tensors are created on first access (the kernels here take the page
  count as a host integer);
* for page_size > 1 the code cache holds one entry per token (the reference's layout is only
  consistent at page_size 1) and budgets are counted in tokens: budget = page_budget * page_size;
* the sequence length is also kept in device memory (``seq_len_dev``), for decode steps whose launches
  do not depend on the length and can therefore be replayed from one CUDA graph (utils.decode_step_dev).
"""
from __future__ import annotations

import torch

from .decode_wrapper import BatchDecodeWithPagedKVCacheWrapper
from .kv_cache import KvCache
from .utils import TensorLayout


class InferenceController:
    def __init__(self, num_layers, num_heads, head_dim, page_size,
                 page_budget,   # page budget including the last page
                 max_seq_len,   # capacity of the KV / code caches in tokens
                 dtype, device,
                 num_q_heads=None):   # query heads when they outnumber the cache's (grouped-query attention)
        self.kv_cache = KvCache(num_layers=num_layers, num_heads=num_heads, head_dim=head_dim,
                                max_seq_len=max_seq_len, page_size=page_size, items=2, dtype=dtype,
                                device=device)
        # 16-bit words of packed codes, head_dim/8 per (token, head); stored in `dtype` like the
        # reference so that buf_layer() views are interchangeable
        self.hadamard_cache = KvCache(num_layers=num_layers, num_heads=num_heads, head_dim=head_dim // 8,
                                      max_seq_len=max_seq_len, page_size=page_size, items=1, dtype=dtype,
                                      device=device)
        self.layout = TensorLayout.NHD
        self.device = device
        self.dtype = dtype
        self.num_heads = num_heads          # heads of the caches
        self.num_q_heads = num_heads if num_q_heads is None else int(num_q_heads)   # rows of q, o, distances, lists
        if self.num_q_heads < num_heads or self.num_q_heads % num_heads:
            raise ValueError("num_q_heads must be a multiple of num_heads")
        self.head_dim = head_dim
        self.page_size = page_size

        self._page_budget = page_budget
        self._decode_handler = BatchDecodeWithPagedKVCacheWrapper(kv_layout="NHD")

        self.kv_indices_with_last = None
        self.kv_indices_without_last = None
        self.hadamard_indices = None
        self.kv_last_page_idx = None
        self.hadamard_last_page_idx = None

        self._indptr_cache = {}
        self._indptr_vals = {}

        self.inference_page_budget = None
        self.inference_token_budget = None

        self.topk_dout_buffer = None
        self.topk_dindices_buffer = None
        self.topk_buf = None
        self._topk_store = None
        self._estimate_store = None

        self.max_seq_len = self.kv_cache.pool.capacity * page_size
        self._hist = None
        self._seq_len_dev = None
        self._q_code_scratch = None

    # ---- small index tensors, made on demand -------------------------------------------------
    def _indptr(self, name):
        vals = self._indptr_vals.get(name)
        if vals is None:
            return None
        t = self._indptr_cache.get(name)
        if t is None:
            t = torch.tensor(vals, dtype=torch.int32, device=self.device)
            self._indptr_cache[name] = t
        return t

    def _set_indptr(self, name, vals):
        if self._indptr_vals.get(name) != vals:
            self._indptr_vals[name] = vals
            self._indptr_cache.pop(name, None)

    kv_indptr_for_append = property(lambda self: self._indptr("kv_append"))
    hadamard_indptr_for_append = property(lambda self: self._indptr("code_append"))
    kv_indptr_for_approx_decode = property(lambda self: self._indptr("approx"))

    # ---- budget ------------------------------------------------------------------------------
    def set_page_budget(self, page_budget: int):
        """Used by the model to run the first layers dense (adamas/models/llama.py:428-439)."""
        self._page_budget = page_budget

    def prepare_hadamard(self, seq_len: int):
        """Reserve cache room for seq_len new tokens (once per forward, before the layers)."""
        self.kv_cache.append_seq(seq_len)
        self.hadamard_cache.append_seq(seq_len)

    def begin_forward(self, seq_len: int, updateTensor: bool = True):
        if updateTensor:
            self._set_indptr("kv_append", [0, len(self.kv_cache.indicies)])
            self._set_indptr("code_append", [0, len(self.hadamard_cache.indicies)])
            self.kv_last_page_idx = self.kv_cache.indicies[-1]
            self.hadamard_last_page_idx = self.hadamard_cache.indicies[-1]
            self.kv_indices_with_last = self.kv_cache.table_device()
            self.hadamard_indices = self.hadamard_cache.table_device()

        if seq_len > 1:
            return

        cur_page_nums = len(self.kv_cache.indicies)
        assert cur_page_nums > 1 or self.page_size > 1   # the newest token is always kept apart
        if updateTensor:
            n = cur_page_nums - 1
            self.kv_indices_without_last = self.kv_indices_with_last[:n].unsqueeze(0).expand(self.num_q_heads, n)

        if self.page_size == 1:
            self.inference_page_budget = min(self._page_budget, cur_page_nums)
            self.inference_token_budget = self.inference_page_budget
        else:
            self.inference_token_budget = min(self._page_budget * self.page_size, self.kv_cache.seqlen)
            self.inference_page_budget = min(self._page_budget, cur_page_nums)
        k = self.inference_token_budget - 1
        self._set_indptr("approx", [0, k])

        # top-k outputs: values and indices share one row stride; reused across steps
        if self._topk_store is None or self._topk_store[0].size(1) < k or self._topk_store[0].size(0) != self.num_q_heads:
            # grows geometrically: in the dense first layers k is the whole context, one more each step
            cap = max(k, 1) if self._topk_store is None else max(k, 2 * self._topk_store[0].size(1))
            cap = max(min(cap, self.kv_cache.pool.capacity * self.page_size), k, 1)
            vals = torch.zeros((self.num_q_heads, cap), dtype=torch.int16, device=self.device)
            idx = torch.zeros((self.num_q_heads, cap), dtype=torch.int32, device=self.device)
            self._topk_store = (vals, idx)
        vdtype = self.dtype if self.dtype == torch.float16 else torch.int16
        self.topk_dout_buffer = self._topk_store[0].view(vdtype)[:, :k]
        self.topk_dindices_buffer = self._topk_store[1][:, :k]
        if self.topk_buf is None:
            # the reference's radix-select scratch (controller.py:122); unused here, kept for callers
            self.topk_buf = torch.zeros((self.num_q_heads, 8192 * 2 * (2 + 4) // 2 // 48), dtype=self.dtype,
                                        device=self.device)

        self._decode_handler.begin_forward(torch.tensor([0, k], dtype=torch.int32), self.num_q_heads,
                                           self.num_heads, self.head_dim, self.page_size, self.dtype)

    def end_forward(self):
        self._decode_handler.end_forward()

    def need_estimate(self) -> bool:
        if self.inference_page_budget is None:
            return False
        if self.page_size == 1:
            return len(self.kv_cache.indicies) > self.inference_page_budget
        return self.kv_cache.seqlen > self.inference_token_budget

    def estimate_buffer(self, n: int) -> torch.Tensor:
        """[H, n] distance buffer (fp16 for fp16 models as in the reference, else int16), reused."""
        vdtype = self.dtype if self.dtype == torch.float16 else torch.int16
        if self._estimate_store is None or self._estimate_store.size(1) < n:
            cap = max(n, 1) if self._estimate_store is None else max(n, 2 * self._estimate_store.size(1))
            cap = max(min(cap, self.kv_cache.pool.capacity * self.page_size), n)
            cap = (cap + 7) // 8 * 8     # rows start on 16-byte boundaries (the top-k kernel's fast layout)
            self._estimate_store = torch.empty((self.num_q_heads, cap), dtype=torch.int16, device=self.device)
        return self._estimate_store.view(vdtype)[:, :n]

    def distance_scratch(self, n: int) -> torch.Tensor:
        """[H, n] int16 view of the same buffer, rows on 16-byte boundaries (fused decode step)."""
        self.estimate_buffer(n)
        return self._estimate_store[:, :n]

    # ---- state of the fused / graph-replayable decode step ------------------------------------
    @property
    def hist_scratch(self) -> torch.Tensor:
        """Scratch table of the fused decode step (_kernels.histogram_scratch; its histograms are zero
        between steps)."""
        if self._hist is None:
            from .. import _kernels
            self._hist = _kernels.histogram_scratch(self.num_q_heads, self.device)
        return self._hist

    @property
    def seq_len_dev(self) -> torch.Tensor:
        """One-element int32 device tensor with the sequence length the next device-state decode step
        sees (tokens in the caches, the one being appended included).  sync_seq_len() sets it from the
        host's count; utils.seq_len_advance adds one on the device."""
        if self._seq_len_dev is None:
            self._seq_len_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
        return self._seq_len_dev

    def sync_seq_len(self) -> None:
        """seq_len_dev := the host's sequence length (after prepare_hadamard(1): the length the coming
        decode step works on)."""
        self.seq_len_dev.fill_(self.kv_cache.seqlen)

    def q_code_scratch(self, dtype) -> torch.Tensor:
        """[1, H, D/8] packed query code of the step in flight (one per controller: the launches of one
        sequence are ordered on one stream)."""
        q = self._q_code_scratch
        if q is None or q.dtype != dtype:
            q = torch.empty(1, self.num_q_heads, self.head_dim // 8, dtype=dtype, device=self.device)
            self._q_code_scratch = q
        return q

    def token_budget(self) -> int:
        """The configured budget in tokens (not capped by the current length)."""
        return self._page_budget * self.page_size

    def clean_states(self):
        self.kv_cache.release()
        self.hadamard_cache.release()
