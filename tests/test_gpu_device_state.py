"""Decode steps whose sequence length lives in device memory: one CUDA graph, captured once, is
replayed for consecutive tokens and must do exactly what the eager loop over the host-length
operators does (the loop the reference's controller drives, adamas/utils/controller.py:82-131)."""
import numpy as np
import pytest
import torch

from oracle import adamas_ref as ref
from test_gpu_parity import DEV, State, _assert_attn_close, _mods, _randn

pytestmark = pytest.mark.gpu


def _token_inputs(t, H, dtype):
    return (_randn((1, H, 128), 5000 + 3 * t, dtype), _randn((1, H, 128), 5001 + 3 * t, dtype),
            _randn((1, H, 128), 5002 + 3 * t, dtype))


def _gather_cache(c, L, ps):
    table = torch.tensor(c.kv_cache.indicies)
    t = torch.arange(L)
    kv = c.kv_cache.buf_layer(0).cpu()
    codes = c.hadamard_cache.buf_layer(0).cpu()
    ctab = torch.tensor(c.hadamard_cache.indicies)
    return kv[table[t // ps], 0, t % ps], kv[table[t // ps], 1, t % ps], codes[ctab[t // ps], 0, t % ps]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("L0,ps,budget,H,rope,tokens", [
    (300, 16, 64, 32, None, 64),            # two-launch step
    (300, 16, 64, 32, (8.0, 1e4), 64),      # rotary embedding inside the append-fused estimate
    (500, 1, 96, 16, None, 40),             # page size 1: a new page every token
    (2100, 16, 256, 4, (1.0, 1e4), 40),     # page-copy estimate (few heads)
    (32750, 16, 1024, 32, None, 40),        # crosses 32768 tokens: the row outgrows one granule per thread
])
def test_graph_replay_equals_eager_loop(dtype, L0, ps, budget, H, rope, tokens):
    _, K, U = _mods()
    cap = L0 + tokens + ps
    sa = State(L0, H, ps, dtype, seed=L0, budget_pages=max(1, budget // ps), fused=True, max_seq_len=cap)
    sb = State(L0, H, ps, dtype, seed=L0, budget_pages=max(1, budget // ps), fused=True, max_seq_len=cap)
    ca, cb = sa.c, sb.c
    ca.end_forward()
    cb.end_forward()
    tb = cb.token_budget()
    # static buffers of the captured step
    qs = torch.zeros(1, H, 128, dtype=dtype, device=DEV)
    ks, vs, ob = torch.zeros_like(qs), torch.zeros_like(qs), torch.zeros_like(qs)
    idx_b = torch.zeros(H, tb - 1, dtype=torch.int32, device=DEV)
    q_code = torch.zeros(1, H, 16, dtype=dtype, device=DEV)

    def step_b():
        K.decode_step_dev(qs, ks, vs, ob, q_code, cb.kv_cache.buf_layer(0), cb.kv_cache.table_all(),
                          cb.hadamard_cache.buf_layer(0), cb.hadamard_cache.table_all(), cb.seq_len_dev, cb.max_seq_len,
                          tb, cb.distance_scratch(cb.max_seq_len - 1), cb.hist_scratch, indices_out=idx_b, rope=rope)
        U.seq_len_advance(cb)

    graph = None
    q_last = None
    for t in range(tokens):
        q, k, v = _token_inputs(t, H, dtype)
        # eager, host lengths
        ca.prepare_hadamard(1)
        ca.begin_forward(1)
        qa, ka = q.to(DEV), k.to(DEV)
        oa = U.decode_step(qa, ka, v.to(DEV), ca, 0, rope=rope)
        idx_a = ca.topk_dindices_buffer.clone()
        ca.end_forward()
        # device lengths: the first token eagerly, then captured, then replays
        cb.prepare_hadamard(1)
        cb.kv_cache.table_all()
        cb.hadamard_cache.table_all()
        qs.copy_(q)
        ks.copy_(k)
        vs.copy_(v)
        if t == 0:
            cb.sync_seq_len()
            step_b()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step_b()
        else:
            graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(idx_a, idx_b), f"selected slots differ at token {t}"
        _assert_attn_close(ob[0], oa[0].float())
        assert torch.equal(qs.view(torch.int16), qa.view(torch.int16)), "rotated q"
        assert int(K.histogram_counts(cb.hist_scratch).abs().sum().item()) == 0
        q_last = qa
    L = L0 + tokens
    assert ca.kv_cache.seqlen == cb.kv_cache.seqlen == L and int(cb.seq_len_dev.item()) == L + 1
    for a, b, name in zip(_gather_cache(ca, L, ps), _gather_cache(cb, L, ps), ["K rows", "V rows", "codes"]):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), name
    # and the last token against the oracle, on what the caches hold
    kc, vc, _ = _gather_cache(cb, L, ps)
    r = ref.decode_step(q_last[0].cpu(), kc, vc, tb)
    table = np.asarray(cb.kv_cache.indicies)
    np.testing.assert_array_equal(idx_b.cpu().numpy(), table[r["sel"] // ps] * ps + r["sel"] % ps)
    _assert_attn_close(ob[0], r["out"])
    from adamas_b200 import _lib
    assert _lib.device_error(clear=False) == 0


@pytest.mark.parametrize("rope", [None, (8.0, 1e4)])
@pytest.mark.parametrize("H,ps", [(32, 16), (4, 1), (8, 16)])
def test_dense_graph_replay_equals_eager_loop(rope, H, ps):
    """The dense step (append + attention over every token) with the length on the device, replayed
    from one graph across page boundaries, against the eager dense decode_step."""
    _, K, U = _mods()
    L0, tokens, dtype = 150, 48, torch.float16
    cap = L0 + tokens + ps
    sa = State(L0, H, ps, dtype, seed=L0 + H, budget_pages=1 << 20, fused=True, max_seq_len=cap)
    sb = State(L0, H, ps, dtype, seed=L0 + H, budget_pages=1 << 20, fused=True, max_seq_len=cap)
    ca, cb = sa.c, sb.c
    ca.end_forward()
    qs = torch.zeros(1, H, 128, dtype=dtype, device=DEV)
    ks, vs, ob = torch.zeros_like(qs), torch.zeros_like(qs), torch.zeros_like(qs)

    def step_b():
        U.decode_step_dev(qs, ks, vs, cb, 0, out=ob, dense=True, rope=rope)
        U.seq_len_advance(cb)

    graph = None
    for t in range(tokens):
        q, k, v = _token_inputs(t, H, dtype)
        ca.prepare_hadamard(1)
        ca.begin_forward(1)
        assert not ca.need_estimate()
        qa = q.to(DEV)
        oa = U.decode_step(qa, k.to(DEV), v.to(DEV), ca, 0, rope=rope)
        ca.end_forward()
        cb.prepare_hadamard(1)
        cb.kv_cache.table_all()
        cb.hadamard_cache.table_all()
        qs.copy_(q)
        ks.copy_(k)
        vs.copy_(v)
        if t == 0:
            cb.sync_seq_len()
            step_b()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step_b()
        else:
            graph.replay()
        torch.cuda.synchronize()
        _assert_attn_close(ob[0], oa[0].float())
    L = L0 + tokens
    for a, b, name in zip(_gather_cache(ca, L, ps), _gather_cache(cb, L, ps), ["K rows", "V rows", "codes"]):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), name
    kc, vc, _ = _gather_cache(cb, L, ps)
    want = ref.sparse_attention(qs[0].cpu(), kc, vc, np.tile(np.arange(L), (H, 1)))
    _assert_attn_close(ob[0], want)


@pytest.mark.parametrize("H", [4, 32, 40])
def test_dense_step_with_rope_reads_the_rotated_query(H):
    """The dense branch of decode_step with the rotary embedding inside the append launch: the attention
    kernel must see the ROTATED query although it may become resident while the append still runs
    (programmatic dependent launch).  Many repeats, compared with the oracle on the rotated query."""
    _, K, U = _mods()
    L0, ps, dtype = 120, 16, torch.float16
    st = State(L0, H, ps, dtype, seed=H, budget_pages=1 << 20, fused=True, max_seq_len=L0 + 80)
    c = st.c
    c.end_forward()
    k_all, v_all = [st.k], [st.v]
    for t in range(60):
        q, k, v = _token_inputs(t, H, dtype)
        c.prepare_hadamard(1)
        c.begin_forward(1)
        qd, kd = q.to(DEV), k.to(DEV)
        o = U.decode_step(qd, kd, v.to(DEV), c, 0, rope=(8.0, 1e4))
        c.end_forward()
        L = c.kv_cache.seqlen
        # the rotation itself, at the reference's tolerance for that operator (adamas/tests/test_rope.py:10-15)
        torch.testing.assert_close(qd.cpu().float(), ref.rope(q, L - 1, 8.0, 1e4).float(), rtol=5e-3, atol=5e-3)
        q_rot, k_rot = qd.cpu(), kd.cpu()          # rotated in place by the append launch
        assert not torch.equal(q_rot, q)
        k_all.append(k_rot)
        v_all.append(v)
        want = ref.sparse_attention(q_rot[0], torch.cat(k_all, 0), torch.cat(v_all, 0), np.tile(np.arange(L), (H, 1)))
        _assert_attn_close(o[0], want)


def test_merge_states_with_every_part_empty():
    """A head whose parts are all empty (lse = -inf everywhere) gets zeros and lse = -inf, not NaN."""
    _, K, _ = _mods()
    P, H = 3, 4
    o_parts = torch.randn(P, H, 128)
    lse = torch.randn(P, H)
    lse[:, 1] = -float("inf")
    o_parts[:, 1] = float("nan")       # whatever an empty shard left behind must not leak
    o = torch.full((H, 128), 7.0, dtype=torch.float16, device=DEV)
    out_lse = torch.zeros(H, dtype=torch.float32, device=DEV)
    K.merge_states(o_parts.to(DEV), lse.to(DEV), o, out_lse)
    torch.cuda.synchronize()
    assert torch.all(o[1] == 0) and out_lse[1].item() == -float("inf")
    keep = [0, 2, 3]
    want, _ = ref.merge_states(o_parts[:, keep], lse[:, keep] * float(np.log(2.0)))
    _assert_attn_close(o[keep], want)
    assert torch.isfinite(o.float()).all()
