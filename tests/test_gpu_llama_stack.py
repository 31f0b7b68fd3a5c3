"""The decode path inside its caller: a small Llama-shaped stack (adamas_b200/llama_stack.py) run
(1) densely against a plain fp32 torch model, (2) sparsely with every layer's selection and attention
output checked in place against the oracle on what the caches hold, (3) with and without CUDA graphs."""
import math

import numpy as np
import pytest
import torch

from oracle import adamas_ref as R

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
LOGIT_ATOL = 2e-2      # fp16 GEMM chain against fp32 (logits are O(0.5) here)


def _stack(cls=None, **over):
    from adamas_b200 import llama_stack as S
    kw = dict(num_layers=4, num_heads=4, head_dim=128, ffn=1024, vocab=512, skip_layers=1)
    kw.update(over)
    cfg = S.StackConfig(**kw)
    return (cls or S.LlamaStack)(cfg, DEV, torch.float16, seed=3)


def _ids(n, vocab=512, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).to(DEV)


def _rope_f32(x, rope_scale, theta):
    n, h, d = x.shape
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    pos = torch.arange(n, device=x.device, dtype=torch.float32) / rope_scale
    emb = torch.cat([torch.outer(pos, inv)] * 2, dim=-1)
    cos, sin = emb.cos()[:, None], emb.sin()[:, None]
    rot = torch.cat((-x[..., d // 2:], x[..., : d // 2]), dim=-1)
    return x * cos + rot * sin


def _reference_logits(st, ids):
    """Plain fp32 forward over the whole sequence with full causal attention."""
    cfg = st.cfg
    n = ids.numel()
    x = st.embed[ids].float()

    def norm(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * w.float()

    for l in range(cfg.num_layers):
        qkv = norm(x, st.ln1[l]) @ st.wqkv[l].float().t()
        kvd = cfg.kv_heads * cfg.head_dim
        group = cfg.num_heads // cfg.kv_heads
        q = _rope_f32(qkv[:, :cfg.hidden].reshape(n, cfg.num_heads, cfg.head_dim), cfg.rope_scale, cfg.rope_theta)
        k = _rope_f32(qkv[:, cfg.hidden:cfg.hidden + kvd].reshape(n, cfg.kv_heads, cfg.head_dim), cfg.rope_scale, cfg.rope_theta)
        v = qkv[:, cfg.hidden + kvd:].reshape(n, cfg.kv_heads, cfg.head_dim)
        k, v = k.repeat_interleave(group, 1), v.repeat_interleave(group, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(cfg.head_dim)
        s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool, device=x.device), 1), float("-inf"))
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(n, cfg.hidden)
        x = x + a @ st.wo[l].float().t()
        gu = norm(x, st.ln2[l]) @ st.w_gate_up[l].float().t()
        x = x + (torch.nn.functional.silu(gu[:, : cfg.ffn]) * gu[:, cfg.ffn:]) @ st.w_down[l].float().t()
    return norm(x[-1:], st.ln_f) @ st.lm_head.float().t()


@pytest.mark.parametrize("heads,kv_heads", [(4, 0), (8, 2)])
def test_dense_stack_matches_fp32_model(heads, kv_heads):
    st = _stack(num_heads=heads, num_kv_heads=kv_heads)
    ids = _ids(150)
    st.init_controller(page_size=16, token_budget=4096, max_seq_len=256)     # budget > context: every layer dense
    logits = st.prefill(ids[:140])
    ref = _reference_logits(st, ids[:140])
    assert torch.allclose(logits, ref, atol=LOGIT_ATOL), (logits - ref).abs().max().item()
    for t in range(140, 150):
        st.decode_one(token=int(ids[t]))
        ref = _reference_logits(st, ids[: t + 1])
        err = (st.last_logits() - ref).abs().max().item()
        assert err < LOGIT_ATOL, (t, err)
    from adamas_b200 import _lib
    assert _lib.device_error() == 0


def _checked_stack_class():
    from adamas_b200 import llama_stack as S
    from adamas_b200 import utils as U

    class CheckedAttention(S.LlamaStack):
        """Runs the fused CUDA decode step and, in place, recomputes distance, selection and
        attention on the CPU from what the caches then hold: same q, same keys, same codes."""
        checks = 0
        worst = 0.0

        def _decode_attention(self, layer, q, k, v, out):
            c = self.controller
            U.decode_step(q, k, v, c, layer, out=out, record_indices=True,
                          rope=(self.cfg.rope_scale, self.cfg.rope_theta))
            L, H, ps = c.kv_cache.seqlen, self.cfg.num_heads, c.page_size
            table = c.kv_indices_with_last.long()
            kv = c.kv_cache.buf_layer(layer)[table]                                    # [pages,2,ps,H,D]
            K = kv[:, 0].reshape(-1, H, 128)[:L].cpu()
            V = kv[:, 1].reshape(-1, H, 128)[:L].cpu()
            codes = c.hadamard_cache.buf_layer(layer)[c.hadamard_indices.long()][:, 0].reshape(-1, H, 16)[:L]
            codes = codes.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
            qr = q[0].cpu()                                                            # rotated in place
            budget = c.inference_token_budget
            assert np.array_equal(codes[L - 1], R.encode(K[L - 1]))
            if L <= budget:
                idx = np.tile(np.arange(L, dtype=np.int64), (H, 1))
            else:
                dist = R.code_distance(R.encode(qr), codes[: L - 1])
                sel = R.select_topk(dist, budget - 1)
                idx = np.concatenate([sel, np.full((H, 1), L - 1, dtype=np.int64)], axis=1)
                tab = table.cpu().numpy()
                want = tab[sel // ps] * ps + sel % ps
                got = c.topk_dindices_buffer.cpu().numpy()
                assert np.array_equal(np.sort(got, axis=1), np.sort(want, axis=1)), (layer, L)
                type(self).checks += 1
            ref = R.sparse_attention(qr, K, V, idx)
            err = ((out[0].float().cpu() - ref).abs().max() / ref.abs().max()).item()
            type(self).worst = max(type(self).worst, err)
            assert err < 2e-3, (layer, L, err)

    return CheckedAttention


@pytest.mark.parametrize("page_size,budget", [(16, 64), (1, 48)])
def test_sparse_stack_matches_oracle_layer_by_layer(page_size, budget):
    ids = _ids(330, seed=1)
    cls = _checked_stack_class()
    st = _stack(cls)
    st.init_controller(page_size=page_size, token_budget=budget, max_seq_len=352)
    st.prefill(ids[:320])
    for t in range(320, 330):
        st.decode_one(token=int(ids[t]), use_graphs=False)      # the eager, host-length path is the one checked in place
    assert cls.checks == 10 * (st.cfg.num_layers - st.cfg.skip_layers)      # every sparse layer, every step
    assert st.controller.need_estimate()
    from adamas_b200 import _lib
    assert _lib.device_error() == 0


@pytest.mark.parametrize("prefill,budget,new_tokens,yarn,kv_heads", [
    (200, 64, 40, 0.0, 0), (50, 64, 40, 0.0, 0), (120, 64, 24, 32.0, 0), (120, 64, 24, 0.0, 2)])
def test_whole_token_graph_equals_eager_loop(prefill, budget, new_tokens, yarn, kv_heads):
    """decode_one as ONE graph replay per token (device-resident sequence length) against the eager
    loop over the host-length operators: same sampled tokens, same logits, same caches.  The second
    case starts with every layer dense and crosses the token budget on the way (the graph is
    re-captured once), both cross several page boundaries; the third rotates with a YaRN table; the
    fourth has 8 query heads over 2 cache heads."""
    ids = _ids(prefill, seed=2)
    forced = _ids(new_tokens, seed=5).tolist()     # the same input token at every step of both runs
    runs = []
    for use_graphs in (True, False):
        st = _stack(yarn_factor=yarn, yarn_original_max_position=64, num_heads=8 if kv_heads else 4,
                    num_kv_heads=kv_heads)
        st.init_controller(page_size=16, token_budget=budget, max_seq_len=prefill + new_tokens + 16)
        st.prefill(ids)
        toks, logits = [], []
        for t in range(new_tokens):
            st.decode_one(token=forced[t], use_graphs=use_graphs)
            toks.append(st._tok.clone())
            logits.append(st.last_logits().clone())
        c = st.controller
        n_pages = len(c.kv_cache.indicies)
        table = torch.tensor(c.kv_cache.indicies, device=DEV)
        kv = c.kv_cache.pool.buf[:, table].clone()
        codes = c.hadamard_cache.pool.buf[:, torch.tensor(c.hadamard_cache.indicies, device=DEV)].clone()
        runs.append((torch.cat(toks).cpu(), torch.cat(logits).cpu(), kv.cpu(), codes.cpu(), c.kv_cache.seqlen, n_pages))
        if use_graphs:
            assert len(st._token_graphs) == (2 if prefill < budget else 1)
            assert int(c.seq_len_dev.item()) == c.kv_cache.seqlen + 1
    (tg, lg, kvg, cg, ng, pg), (te, le, kve, ce, ne, pe) = runs
    assert ng == ne == prefill + new_tokens and pg == pe
    assert torch.allclose(lg, le, atol=2e-3), (lg - le).abs().max().item()
    assert (tg == te).float().mean().item() > 0.9      # argmax of near-identical logits
    last = (ng - 1) % 16 + 1           # entries of the last page beyond the sequence are never written
    assert torch.equal(cg[:, :-1].view(torch.int16), ce[:, :-1].view(torch.int16))
    assert torch.equal(cg[:, -1, :, :last].view(torch.int16), ce[:, -1, :, :last].view(torch.int16))
    assert torch.allclose(kvg[:, :-1].float(), kve[:, :-1].float(), atol=2e-3)
    from adamas_b200 import _lib
    assert _lib.device_error() == 0


def test_generate_runs():
    ids = _ids(200, seed=2)
    st = _stack()
    st.init_controller(page_size=16, token_budget=64, max_seq_len=256)
    toks = st.generate(ids, 20)
    assert len(toks) == 21 and all(0 <= t < 512 for t in toks)
    assert st.controller.kv_cache.seqlen == 220
