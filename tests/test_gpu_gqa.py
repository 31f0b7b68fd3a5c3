"""Grouped-query attention through the decode path: Hq query heads over H cache heads, query head r
reading cache head r // (Hq // H).  The oracle states it as multi-head attention on repeated keys and
values (oracle.repeat_kv).  The reference's operators accept group 1 only
(kernels/include/decode/decode_handler.cuh:83); its CPU reference defines the mapping
(kernels/src/include/cpu_reference.h:83)."""
import numpy as np
import pytest
import torch

from oracle import adamas_ref as ref
from test_gpu_parity import DEV, _assert_attn_close, _codes_of, _mods, _randn

pytestmark = pytest.mark.gpu


class GqaState:
    """L-1 tokens prefilled into caches of H heads; q [1, Hq, 128], and k, v [1, H, 128] of the token to decode."""

    def __init__(self, L, Hq, H, ps, dtype=torch.float16, seed=0, budget_pages=64, max_seq_len=None, extra=0):
        _, K, U = _mods()
        self.L, self.Hq, self.H, self.ps, self.dtype = L, Hq, H, ps, dtype
        self.group = Hq // H
        self.q = _randn((1 + extra, Hq, 128), seed, dtype)
        self.k = _randn((L + extra, H, 128), seed + 1, dtype)
        self.v = _randn((L + extra, H, 128), seed + 2, dtype)
        cap = max_seq_len or (L + extra + 3 * ps + 5)
        self.c = c = U.InferenceController(1, H, 128, ps, budget_pages, cap, dtype, DEV, num_q_heads=Hq)
        c.prepare_hadamard(L - 1)
        c.begin_forward(L - 1)
        U.append_kvh(self.k[: L - 1].to(DEV), self.v[: L - 1].to(DEV), None, c, 0)
        c.end_forward()

    def oracle(self, budget, step=0, q=None, k=None):
        n = self.L + step
        kk = self.k if k is None else k
        return ref.decode_step((self.q[step] if q is None else q), ref.repeat_kv(kk[:n], self.group),
                               ref.repeat_kv(self.v[:n], self.group), budget)

    def slots(self, sel):
        table = np.asarray(self.c.kv_cache.indicies)
        return table[sel // self.ps] * self.ps + sel % self.ps


SHAPES = [(32, 8), (8, 2), (28, 4), (4, 1), (64, 8), (16, 16)]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("ps", [1, 16])
@pytest.mark.parametrize("Hq,H", SHAPES)
def test_gqa_stage_by_stage(Hq, H, ps, dtype):
    """append (codes of Hq query rows and H key rows), estimate [Hq, n], top-k, sparse attention through
    the decode wrapper planned with num_qo_heads != num_kv_heads."""
    _, K, U = _mods()
    L, budget = 700, 96 if ps == 1 else 6
    st = GqaState(L, Hq, H, ps, dtype, seed=Hq + H, budget_pages=budget)
    c = st.c
    tok_budget = budget * ps
    r = st.oracle(tok_budget)
    qd = st.q[:1].to(DEV)
    c.prepare_hadamard(1)
    c.begin_forward(1)
    q_code = U.append_qkv_fused(qd, st.k[L - 1:L].to(DEV), st.v[L - 1:L].to(DEV), c, 0)
    assert tuple(q_code.shape) == (1, Hq, 16)
    np.testing.assert_array_equal(_codes_of(q_code)[0], ref.encode(st.q[0]))
    table = np.asarray(c.hadamard_cache.indicies)
    codes = _codes_of(c.hadamard_cache.buf_layer(0))
    t = np.arange(L)
    np.testing.assert_array_equal(codes[table[t // ps], 0, t % ps], ref.encode(st.k[:L]))
    dist = U.decode_estimate(q_code, c, 0)
    assert tuple(dist.shape) == (Hq, L - 1)
    np.testing.assert_array_equal(dist.float().cpu().numpy().astype(np.int64), r["dist"])
    U.decode_topk(dist, c)
    got = c.topk_dindices_buffer.cpu().numpy()
    np.testing.assert_array_equal(got, st.slots(r["sel"]) if ps > 1 else table[r["sel"]])
    o = U.decode_sparse_attn(qd, c, 0, c.topk_dindices_buffer)
    _assert_attn_close(o[0], r["out"])
    # the dense form: every page "selected"
    o = U.decode_sparse_attn(qd, c, 0, c.kv_indices_without_last)
    full = np.tile(np.arange(L, dtype=np.int64), (Hq, 1))
    _assert_attn_close(o[0], ref.sparse_attention(st.q[0], ref.repeat_kv(st.k[:L], st.group),
                                                  ref.repeat_kv(st.v[:L], st.group), full))
    c.end_forward()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rope", [None, (8.0, 1e4)])
@pytest.mark.parametrize("L,ps,budget", [(700, 16, 6), (5000, 1, 256), (40000, 16, 64)])
@pytest.mark.parametrize("Hq,H", [(32, 8), (8, 2), (28, 4), (4, 1)])
def test_gqa_decode_step(Hq, H, L, ps, budget, rope, dtype):
    """The fused step (append, estimate with histograms, select + attend) with grouped queries."""
    _, K, U = _mods()
    st = GqaState(L, Hq, H, ps, dtype, seed=L + Hq, budget_pages=budget)
    c = st.c
    qd, kd, vd = st.q[:1].to(DEV), st.k[L - 1:L].to(DEV), st.v[L - 1:L].to(DEV)
    c.prepare_hadamard(1)
    c.begin_forward(1)
    o = U.decode_step(qd, kd, vd, c, 0, rope=rope)
    torch.cuda.synchronize()
    q_ref, k_ref = st.q[0], st.k
    if rope is not None:
        # the rotated rows as the kernel left them (the rotation has its own test): the rest must be exact on them
        q_ref = qd[0].cpu()
        k_ref = st.k.clone()
        k_ref[L - 1] = kd[0].cpu()
        torch.testing.assert_close(q_ref.float(), ref.rope(st.q[:1], L - 1, *rope)[0].float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(k_ref[L - 1].float(), ref.rope(st.k[L - 1:L], L - 1, *rope)[0].float(), rtol=2e-2, atol=2e-2)
    r = st.oracle(budget * ps, q=q_ref, k=k_ref)
    np.testing.assert_array_equal(c.topk_dindices_buffer.cpu().numpy(), st.slots(r["sel"]))
    _assert_attn_close(o[0], r["out"])
    assert int(K.histogram_counts(c.hist_scratch).abs().sum().item()) == 0
    from adamas_b200 import _lib
    assert _lib.device_error(clear=False) == 0
    c.end_forward()


@pytest.mark.parametrize("Hq,H,ps", [(32, 8, 16), (8, 2, 1), (12, 4, 16)])
def test_gqa_graph_replay_equals_eager_loop(Hq, H, ps):
    """Device-resident sequence length with grouped queries: one captured sparse step and one captured
    dense step, replayed over several tokens, against the host-length operators."""
    _, K, U = _mods()
    L, tokens, budget = 300, 20, 4 if ps == 16 else 64
    outs = {}
    for mode in ("graph", "eager"):
        st = GqaState(L, Hq, H, ps, torch.float16, seed=7, budget_pages=budget, max_seq_len=L + tokens + ps, extra=tokens)
        c = st.c
        qs = torch.zeros(1, Hq, 128, dtype=torch.float16, device=DEV)
        ks = torch.zeros(1, H, 128, dtype=torch.float16, device=DEV)
        vs = torch.zeros(1, H, 128, dtype=torch.float16, device=DEV)
        os_ = torch.zeros(2, 1, Hq, 128, dtype=torch.float16, device=DEV)
        res = []
        graph = None
        for t in range(tokens):
            c.prepare_hadamard(1)
            qs.copy_(st.q[t:t + 1]); ks.copy_(st.k[L - 1 + t:L + t]); vs.copy_(st.v[L - 1 + t:L + t])
            if mode == "graph":
                c.kv_cache.table_all()
                c.hadamard_cache.table_all()

                def body():
                    U.decode_step_dev(qs, ks, vs, c, 0, out=os_[0])
                    U.decode_step_dev(qs, ks, vs, c, 0, out=os_[1], dense=True)   # (appends the same token again)
                    U.seq_len_advance(c)

                if graph is None:
                    c.begin_forward(1)
                    c.sync_seq_len()
                    body()                       # the first token eagerly: one-time set-up happens outside the capture
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        body()
                else:
                    graph.replay()
            else:
                c.begin_forward(1)
                U.decode_step(qs, ks, vs, c, 0, out=os_[0])
                U.decode_sparse_attn(qs, c, 0, c.kv_indices_without_last, out=os_[1])
                c.end_forward()
            torch.cuda.synchronize()
            res.append(os_.clone().cpu())
        outs[mode] = torch.stack(res)
    assert torch.equal(outs["graph"][:, 0].view(torch.int16), outs["eager"][:, 0].view(torch.int16))
    torch.testing.assert_close(outs["graph"][:, 1].float(), outs["eager"][:, 1].float(), rtol=2e-3, atol=2e-3)
    from adamas_b200 import _lib
    assert _lib.device_error(clear=False) == 0


def test_gqa_rejects_a_query_head_count_that_is_no_multiple():
    _, K, U = _mods()
    with pytest.raises(ValueError):
        U.InferenceController(1, 8, 128, 16, 4, 256, torch.float16, DEV, num_q_heads=12)
    st = GqaState(100, 8, 4, 16, torch.float16, seed=1, budget_pages=2)
    c = st.c
    c.prepare_hadamard(1)
    c.begin_forward(1)
    bad_q = torch.zeros(1, 6, 128, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError):
        U.append_qkv_fused(bad_q, st.k[99:100].to(DEV), st.v[99:100].to(DEV), c, 0)
