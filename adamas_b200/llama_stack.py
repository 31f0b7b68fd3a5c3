"""The caller of the decode path: a Llama-2-shaped decoder stack with random-init weights, used to
measure end-to-end decode tokens/s and to test the path where the reference runs it.

It follows the reference's model code for everything that touches the path
(adamas/models/llama.py:424-486: prepare_hadamard, dense budget for the first `skip_layers`
layers, then the sparse budget; adamas/models/Adamas.py:105-200: q/k/v projections, RoPE with
linear position scaling, append, estimate, top-k, sparse attention, o_proj).  Everything outside the
path is library code: torch GEMMs (cuBLAS), F.rms_norm, and scaled_dot_product_attention for the
dense causal prefill attention.

Decode runs without any host synchronisation per token: the sampled token stays on the device and
the WHOLE token (embedding, every layer's projections, attention path, MLP, the language-model head,
the argmax and the bump of the device-resident sequence length) is one CUDA graph, captured once
and replayed per token.  That is possible because the attention path takes the sequence length from
device memory (utils.decode_step_dev); per token the host only reserves cache room, which uploads one
page number every `page_size` tokens.  The graph is re-captured once, when the context outgrows the
token budget and the sparse layers switch from "attend to everything" to the sparse step.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional

import torch
import torch.nn.functional as F

from . import _kernels as K
from . import utils as U
from .rope import yarn_inv_freq

_DENSE_PAGE_LIMIT = 1 << 24     # "attend to everything" page budget for the first layers


@dataclasses.dataclass
class StackConfig:
    """Llama-2-7B by default (32 layers, hidden 4096, 32 heads x 128, FFN 11008, vocab 32000)."""
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 0         # heads of the K/V projections and caches; 0: as many as num_heads (multi-head
                                  # attention, all the reference supports); a divisor of num_heads: grouped queries
    head_dim: int = 128
    ffn: int = 11008
    vocab: int = 32000
    rope_scale: float = 8.0       # linear position scaling (adamas/models/Adamas.py:56-61)
    rope_theta: float = 1e4
    yarn_factor: float = 0.0      # > 0: YaRN frequencies (rope_scale is then unused) ...
    yarn_original_max_position: int = 4096      # ... stretched from this trained context
    rms_eps: float = 1e-5
    init_std: float = 0.02
    skip_layers: int = 2          # dense first layers (adamas/models/llama.py:538)

    @property
    def hidden(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_heads(self) -> int:
        return self.num_kv_heads or self.num_heads


class LlamaStack:
    def __init__(self, cfg: StackConfig, device, dtype=torch.float16, seed: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("LlamaStack runs the CUDA decode path; no GPU is visible")
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self._yarn = None
        g = torch.Generator(device=self.device).manual_seed(seed)

        def w(*shape):
            return (torch.randn(*shape, generator=g, device=self.device, dtype=torch.float32) * cfg.init_std).to(dtype)

        hd = cfg.hidden
        self.embed = w(cfg.vocab, hd)
        self.lm_head = w(cfg.vocab, hd)
        assert cfg.num_heads % cfg.kv_heads == 0, "num_kv_heads must divide num_heads"
        kvd = cfg.kv_heads * cfg.head_dim
        self.wqkv = [w(hd + 2 * kvd, hd) for _ in range(cfg.num_layers)]      # rows: q heads, k heads, v heads
        self.wo = [w(hd, hd) for _ in range(cfg.num_layers)]
        self.w_gate_up = [w(2 * cfg.ffn, hd) for _ in range(cfg.num_layers)]
        self.w_down = [w(hd, cfg.ffn) for _ in range(cfg.num_layers)]
        ones = torch.ones(hd, device=self.device, dtype=dtype)
        self.ln1 = [ones.clone() for _ in range(cfg.num_layers)]
        self.ln2 = [ones.clone() for _ in range(cfg.num_layers)]
        self.ln_f = ones.clone()

        self.controller: Optional[U.InferenceController] = None
        self._page_budget = None
        # static buffers of the decode step
        self._tok = torch.zeros(1, dtype=torch.int64, device=self.device)
        self._x = torch.zeros(1, hd, dtype=dtype, device=self.device)
        self._qkv_flat = torch.zeros(1, hd + 2 * kvd, dtype=dtype, device=self.device)
        self._qkv = (self._qkv_flat[:, :hd].view(1, cfg.num_heads, cfg.head_dim),              # q, k, v of the token
                     self._qkv_flat[:, hd:hd + kvd].view(1, cfg.kv_heads, cfg.head_dim),
                     self._qkv_flat[:, hd + kvd:].view(1, cfg.kv_heads, cfg.head_dim))
        self._o = torch.zeros(1, cfg.num_heads, cfg.head_dim, dtype=dtype, device=self.device)
        self._logits = torch.zeros(1, cfg.vocab, dtype=torch.float32, device=self.device)
        self._token_graphs = {}       # sparse layers dense / sparse -> graph of a whole token
        self._expected_dev_len = -1   # value seq_len_dev holds if nothing else has touched the caches

    # ---- controller (adamas/models/llama.py:528-560) -------------------------------------------
    def init_controller(self, page_size: int, token_budget: int, max_seq_len: int) -> None:
        assert self.controller is None, "controller already initialised"
        assert token_budget % page_size == 0, "the token budget must be a whole number of pages"
        self._page_budget = token_budget // page_size
        self.controller = U.InferenceController(
            num_layers=self.cfg.num_layers, num_heads=self.cfg.kv_heads, head_dim=self.cfg.head_dim,
            page_size=page_size, page_budget=self._page_budget, max_seq_len=max_seq_len,
            dtype=self.dtype, device=self.device, num_q_heads=self.cfg.num_heads)

    def clean_states(self) -> None:
        self.controller.clean_states()

    # ---- pieces -----------------------------------------------------------------------------
    def _norm(self, x, weight):
        return F.rms_norm(x, (self.cfg.hidden,), weight, self.cfg.rms_eps)

    def _mlp(self, x, layer):
        gu = F.linear(self._norm(x, self.ln2[layer]), self.w_gate_up[layer])
        gate, up = gu[:, :self.cfg.ffn], gu[:, self.cfg.ffn:]
        return F.linear(F.silu(gate) * up, self.w_down[layer])

    def _decode_attention(self, layer: int, q, k, v, out) -> None:
        """The hot path: un-rotated q, k, v [1,H,D] of the new token -> attention output in `out`."""
        U.decode_step(q, k, v, self.controller, layer, out=out, record_indices=False,
                      rope=self._rope())

    def _layer_loop(self, seq_len: int, body) -> None:
        """The controller protocol around the layers (adamas/models/llama.py:424-486)."""
        c, cfg = self.controller, self.cfg
        c.prepare_hadamard(seq_len)
        if cfg.skip_layers > 0:
            c.set_page_budget(_DENSE_PAGE_LIMIT)
            c.begin_forward(seq_len)
        for idx in range(cfg.num_layers):
            if idx == cfg.skip_layers:
                if idx > 0:
                    c.end_forward()
                c.set_page_budget(self._page_budget)
                c.begin_forward(seq_len, updateTensor=(idx == 0))
            body(idx)
        c.end_forward()

    # ---- prefill ------------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """ids int64 [N] on the device -> fills the caches, leaves the next token in the decode
        state and returns the last position's logits [1, vocab] (fp32)."""
        cfg, c = self.cfg, self.controller
        n = ids.numel()
        assert n > 1, "prefill needs at least two tokens"
        x = self.embed[ids]
        past = c.kv_cache.seqlen
        assert past == 0, "one prefill per sequence"

        def body(layer):
            nonlocal x
            qkv = F.linear(self._norm(x, self.ln1[layer]), self.wqkv[layer])
            kvd = cfg.kv_heads * cfg.head_dim
            q = qkv[:, :cfg.hidden].reshape(n, cfg.num_heads, cfg.head_dim).contiguous()
            k = qkv[:, cfg.hidden:cfg.hidden + kvd].reshape(n, cfg.kv_heads, cfg.head_dim).contiguous()
            v = qkv[:, cfg.hidden + kvd:].reshape(n, cfg.kv_heads, cfg.head_dim).contiguous()
            self._rope_prefill(q, k, past)
            U.append_kvh(k, v, None, c, layer)
            group = cfg.num_heads // cfg.kv_heads
            kk, vv = (k, v) if group == 1 else (k.repeat_interleave(group, 1), v.repeat_interleave(group, 1))
            attn = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), kk.transpose(0, 1).unsqueeze(0),
                                                  vv.transpose(0, 1).unsqueeze(0), is_causal=True)
            x = x + F.linear(attn.squeeze(0).transpose(0, 1).reshape(n, cfg.hidden), self.wo[layer])
            x = x + self._mlp(x, layer)

        self._layer_loop(n, body)
        logits = F.linear(self._norm(x[-1:], self.ln_f), self.lm_head).float()
        self._logits.copy_(logits)
        self._tok.copy_(logits.argmax(dim=-1))
        return logits

    # ---- decode -------------------------------------------------------------------------------
    def _segment_first(self):
        self._x.copy_(self.embed[self._tok])
        torch.matmul(self._norm(self._x, self.ln1[0]), self.wqkv[0].t(), out=self._qkv_flat)

    def _segment_after(self, layer: int):
        cfg = self.cfg
        self._x.addmm_(self._o.view(1, cfg.hidden), self.wo[layer].t())
        self._x.add_(self._mlp(self._x, layer))
        if layer + 1 < cfg.num_layers:
            torch.matmul(self._norm(self._x, self.ln1[layer + 1]), self.wqkv[layer + 1].t(),
                         out=self._qkv_flat)
        else:
            self._logits.copy_(F.linear(self._norm(self._x, self.ln_f), self.lm_head))
            self._tok.copy_(self._logits.argmax(dim=-1))

    def _rope(self):
        """The rotation the step operators take: (scale, theta), or the YaRN table."""
        cfg = self.cfg
        if cfg.yarn_factor > 0:
            if self._yarn is None:
                inv_freq, mscale = yarn_inv_freq(cfg.yarn_factor, cfg.yarn_original_max_position, cfg.rope_theta,
                                                 cfg.head_dim)
                self._yarn = {"inv_freq": inv_freq.to(self.device), "mscale": mscale}
            return self._yarn
        return (cfg.rope_scale, cfg.rope_theta)

    def _rope_prefill(self, q, k, past) -> None:
        r = self._rope()
        if isinstance(r, dict):
            K.apply_rope_table_in_place(q, k, past, r["inv_freq"], r["mscale"])
        else:
            U.apply_rope_in_place(q, k, past, rope_scale=r[0], rope_theta=r[1])

    def _token_body(self, sparse: bool) -> None:
        """One whole token with device-resident lengths: nothing in here depends on the host's view of
        the sequence, so it runs eagerly or under graph capture alike."""
        cfg, c = self.cfg, self.controller
        self._segment_first()
        q, k, v = self._qkv[0], self._qkv[1], self._qkv[2]
        for layer in range(cfg.num_layers):
            U.decode_step_dev(q, k, v, c, layer, out=self._o, dense=(layer < cfg.skip_layers or not sparse),
                              rope=self._rope())
            self._segment_after(layer)
        U.seq_len_advance(c)

    @torch.no_grad()
    def decode_one(self, token: Optional[int] = None, use_graphs: bool = True) -> None:
        """One decode step.  Consumes the token left on the device by the previous step (or
        `token`, to force it) and leaves the next one there; nothing is read back to the host.

        use_graphs=True: the whole token is one CUDA graph replay (captured the first time, after
        one eager run of the same launches).  use_graphs=False: eager launches through the
        host-length operators, the way the reference's model drives them."""
        if token is not None:
            self._tok.fill_(int(token))
        if not use_graphs:
            self._segment_first()
            q, k, v = self._qkv[0], self._qkv[1], self._qkv[2]

            def body(layer):
                self._decode_attention(layer, q, k, v, self._o)
                self._segment_after(layer)

            self._layer_loop(1, body)
            return
        c = self.controller
        c.prepare_hadamard(1)
        c.kv_cache.table_all()          # uploads the page number of a page that has just been opened
        c.hadamard_cache.table_all()
        if self._expected_dev_len != c.kv_cache.seqlen:
            c.sync_seq_len()
        sparse = c.kv_cache.seqlen > c.token_budget()
        g = self._token_graphs.get(sparse)
        if g is None:
            # first token in this mode: run it eagerly (it is a real token and warms up every library
            # call), then record the same launches for the tokens to come
            c.set_page_budget(self._page_budget)
            c.begin_forward(1)
            self._token_body(sparse)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._token_body(sparse)
            c.end_forward()
            self._token_graphs[sparse] = g
        else:
            g.replay()
        self._expected_dev_len = c.kv_cache.seqlen + 1

    @torch.no_grad()
    def capture_dense_rest(self) -> "torch.cuda.CUDAGraph":
        """A CUDA graph of everything in a token EXCEPT the attention path (embedding, projections, MLPs,
        head): what the dense rest of the model costs, for a breakdown of the token time.  Replaying it
        overwrites the decode state; use it after the run that is being measured."""
        def body():
            self._segment_first()
            for layer in range(self.cfg.num_layers):
                self._segment_after(layer)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            body()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            body()
        return g

    def last_logits(self) -> torch.Tensor:
        return self._logits

    @torch.no_grad()
    def generate(self, ids: torch.Tensor, new_tokens: int) -> List[int]:
        """Greedy decoding: prefill `ids`, then `new_tokens` decode steps; returns the sampled ids
        (one device->host read at the end)."""
        self.prefill(ids)
        out = torch.empty(new_tokens + 1, dtype=torch.int64, device=self.device)
        out[0:1].copy_(self._tok)
        for i in range(new_tokens):
            self.decode_one()
            out[i + 1:i + 2].copy_(self._tok)
        return out.tolist()
