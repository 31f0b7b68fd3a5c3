"""Several sequences through the same launches (utils.SequenceBatch, adamas_decode_step_batch_dev /
adamas_dense_step_batch_dev): every sequence must get exactly what it gets when it is decoded alone,
and that against the oracle.  Sequences of different lengths, own caches and page tables each."""
import numpy as np
import pytest
import torch

from oracle import adamas_ref as ref
from test_gpu_parity import DEV, _assert_attn_close, _mods, _randn

pytestmark = pytest.mark.gpu


def _controllers(lengths, Hq, H, ps, budget_pages, dtype, cap, seed):
    """One controller per sequence, prefilled with lengths[i] - 1 tokens; returns (controllers, k, v per sequence)."""
    _, K, U = _mods()
    cs, ks, vs = [], [], []
    for i, L in enumerate(lengths):
        c = U.InferenceController(1, H, 128, ps, budget_pages, cap, dtype, DEV, num_q_heads=Hq)
        k = _randn((cap, H, 128), seed + 10 * i, dtype)
        v = _randn((cap, H, 128), seed + 10 * i + 1, dtype)
        c.prepare_hadamard(L - 1)
        c.begin_forward(L - 1)
        U.append_kvh(k[: L - 1].to(DEV), v[: L - 1].to(DEV), None, c, 0)
        c.end_forward()
        cs.append(c); ks.append(k); vs.append(v)
    return cs, ks, vs


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rope", [None, (8.0, 1e4)])
@pytest.mark.parametrize("lengths,Hq,H,ps,budget", [
    ([700, 300, 1500, 701], 32, 32, 16, 64),      # two-launch step (32 heads, no rotation) or three (with)
    ([40000, 33000], 32, 32, 16, 1024),           # beyond 32768 tokens: several granules per thread
    ([900, 2000, 500], 8, 8, 1, 96),              # page size 1, page-copy estimate
    ([700, 1300], 32, 8, 16, 64),                 # grouped queries
    ([350, 351, 352, 353, 354], 4, 4, 16, 32),    # five short sequences
])
def test_batched_step_equals_single_sequence_steps_and_oracle(lengths, Hq, H, ps, budget, rope, dtype):
    _, K, U = _mods()
    B = len(lengths)
    cap = max(lengths) + 2 * ps
    cs, ks, vs = _controllers(lengths, Hq, H, ps, budget // ps, dtype, cap, seed=sum(lengths))
    # reference run: each sequence alone through the host-length step, on caches of its own
    cs2, _, _ = _controllers(lengths, Hq, H, ps, budget // ps, dtype, cap, seed=sum(lengths))
    q = _randn((B, Hq, 128), 5, dtype)
    k_new = torch.stack([ks[i][L - 1] for i, L in enumerate(lengths)])
    v_new = torch.stack([vs[i][L - 1] for i, L in enumerate(lengths)])
    want_o, want_idx, q_rot = [], [], []
    for i, c in enumerate(cs2):
        c.prepare_hadamard(1)
        c.begin_forward(1)
        qi, ki = q[i:i + 1].to(DEV), k_new[i:i + 1].to(DEV)
        o = U.decode_step(qi, ki, v_new[i:i + 1].to(DEV), c, 0, rope=rope)
        want_o.append(o[0].clone()); want_idx.append(c.topk_dindices_buffer.clone()); q_rot.append((qi[0].cpu(), ki[0].cpu()))
        c.end_forward()
    batch = U.SequenceBatch(cs)
    batch.prepare(1)
    batch.sync_seq_lens()
    assert batch.all_sparse()
    qd, kd, vd = q.to(DEV), k_new.to(DEV), v_new.to(DEV)
    idx = torch.full((B * Hq, budget - 1), -1, dtype=torch.int32, device=DEV)
    o = batch.decode_step_dev(qd, kd, vd, 0, rope=rope, indices_out=idx)
    torch.cuda.synchronize()
    assert int(K.histogram_counts(batch._hist).abs().sum().item()) == 0
    for i, L in enumerate(lengths):
        # the physical slots differ between the two sets of caches only if the pools hand out pages differently: they do not
        assert torch.equal(idx[i * Hq:(i + 1) * Hq], want_idx[i]), f"sequence {i}: selected slots"
        _assert_attn_close(o[i], want_o[i])      # (the launch shapes differ, so the merge order may: not bit-equal)
        # and against the oracle, on the rows as rotated
        qr, kr = q_rot[i]
        kk = ks[i][:L].clone()
        kk[L - 1] = kr
        g = Hq // H
        r = ref.decode_step(qr, ref.repeat_kv(kk, g), ref.repeat_kv(vs[i][:L], g), budget)
        table = np.asarray(cs[i].kv_cache.indicies)
        np.testing.assert_array_equal(idx[i * Hq:(i + 1) * Hq].cpu().numpy(), table[r["sel"] // ps] * ps + r["sel"] % ps)
        _assert_attn_close(o[i], r["out"])
    from adamas_b200 import _lib
    assert _lib.device_error(clear=False) == 0


@pytest.mark.parametrize("lengths,Hq,H,ps", [([100, 37, 513], 32, 32, 16), ([64, 65], 8, 2, 1), ([3000, 10], 16, 16, 16)])
def test_batched_dense_step(lengths, Hq, H, ps):
    """Append and attention over every token, for several sequences in the same launches."""
    _, K, U = _mods()
    B, dtype = len(lengths), torch.float16
    cap = max(lengths) + 2 * ps
    cs, ks, vs = _controllers(lengths, Hq, H, ps, 4096, dtype, cap, seed=3)
    q = _randn((B, Hq, 128), 6, dtype)
    k_new = torch.stack([ks[i][L - 1] for i, L in enumerate(lengths)])
    v_new = torch.stack([vs[i][L - 1] for i, L in enumerate(lengths)])
    batch = U.SequenceBatch(cs)
    batch.prepare(1)
    batch.sync_seq_lens()
    o = batch.decode_step_dev(q.to(DEV), k_new.to(DEV), v_new.to(DEV), 0, dense=True)
    torch.cuda.synchronize()
    g = Hq // H
    for i, L in enumerate(lengths):
        full = np.tile(np.arange(L, dtype=np.int64), (Hq, 1))
        want = ref.sparse_attention(q[i], ref.repeat_kv(ks[i][:L], g), ref.repeat_kv(vs[i][:L], g), full)
        _assert_attn_close(o[i], want)
        # the appended token's codes
        c = cs[i]
        codes = c.hadamard_cache.buf_layer(0)[c.hadamard_cache.indicies[-1], 0, (L - 1) % ps]
        np.testing.assert_array_equal(codes.cpu().contiguous().view(torch.int16).numpy().view(np.uint16), ref.encode(k_new[i]))
    from adamas_b200 import _lib
    assert _lib.device_error(clear=False) == 0


def test_batched_graph_replay_over_tokens():
    """One captured graph (a sparse and a dense batched step, then the advance of all lengths) replayed
    for 24 tokens of three sequences that grow across page boundaries, against per-sequence eager steps."""
    _, K, U = _mods()
    lengths, Hq, H, ps, budget, tokens = [300, 420, 333], 32, 32, 16, 64, 24
    B, dtype = len(lengths), torch.float16
    cap = max(lengths) + tokens + ps
    cs, _, _ = _controllers(lengths, Hq, H, ps, budget // ps, dtype, cap, seed=9)
    cs2, _, _ = _controllers(lengths, Hq, H, ps, budget // ps, dtype, cap, seed=9)
    batch = U.SequenceBatch(cs)
    qs = torch.zeros(B, Hq, 128, dtype=dtype, device=DEV)
    ks, vs = torch.zeros(B, H, 128, dtype=dtype, device=DEV), torch.zeros(B, H, 128, dtype=dtype, device=DEV)
    o_sparse, o_dense = torch.zeros_like(qs), torch.zeros_like(qs)

    def body():
        batch.decode_step_dev(qs, ks, vs, 0, out=o_sparse)
        batch.decode_step_dev(qs, ks, vs, 0, out=o_dense, dense=True)      # (appends the same tokens again)
        batch.advance()

    graph = None
    for t in range(tokens):
        q = _randn((B, Hq, 128), 100 + t, dtype)
        k = _randn((B, H, 128), 200 + t, dtype)
        v = _randn((B, H, 128), 300 + t, dtype)
        want_s, want_d = [], []
        for i, c in enumerate(cs2):
            c.prepare_hadamard(1)
            c.begin_forward(1)
            qi = q[i:i + 1].to(DEV)
            want_s.append(U.decode_step(qi, k[i:i + 1].to(DEV), v[i:i + 1].to(DEV), c, 0)[0].clone())
            want_d.append(U.decode_sparse_attn(qi, c, 0, c.kv_indices_without_last)[0].clone())
            c.end_forward()
        batch.prepare(1)
        qs.copy_(q); ks.copy_(k); vs.copy_(v)
        if graph is None:
            batch.sync_seq_lens()
            body()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                body()
        else:
            graph.replay()
        torch.cuda.synchronize()
        for i in range(B):
            _assert_attn_close(o_sparse[i], want_s[i])
            torch.testing.assert_close(o_dense[i].float(), want_d[i].float(), rtol=2e-3, atol=2e-3)
    assert batch.seq_lens.cpu().tolist() == [L + tokens for L in lengths]
    from adamas_b200 import _lib
    assert _lib.device_error(clear=False) == 0


def test_large_launches_count_their_histograms_in_a_launch_of_their_own():
    """From 3 M distances per launch the fused step counts the histograms in a separate launch instead of
    inside the estimate.  Four sequences of 33K tokens x 32 heads cross that line as a batch and stay below
    it one by one: both forms must select the same slots; one 66K sequence of 64 heads is checked against
    the oracle."""
    _, K, U = _mods()
    lengths, Hq, H, ps, budget, dtype = [33100, 32900, 33500, 33001], 32, 32, 16, 1024, torch.float16
    B = len(lengths)
    cap = max(lengths) + 2 * ps
    cs, ks, vs = _controllers(lengths, Hq, H, ps, budget // ps, dtype, cap, seed=21)
    cs2, _, _ = _controllers(lengths, Hq, H, ps, budget // ps, dtype, cap, seed=21)
    q = _randn((B, Hq, 128), 5, dtype)
    k_new = torch.stack([ks[i][L - 1] for i, L in enumerate(lengths)])
    v_new = torch.stack([vs[i][L - 1] for i, L in enumerate(lengths)])
    want_o, want_idx = [], []
    for i, c in enumerate(cs2):
        c.prepare_hadamard(1)
        c.begin_forward(1)
        o = U.decode_step(q[i:i + 1].to(DEV), k_new[i:i + 1].to(DEV), v_new[i:i + 1].to(DEV), c, 0)
        want_o.append(o[0].clone()); want_idx.append(c.topk_dindices_buffer.clone())
        c.end_forward()
    batch = U.SequenceBatch(cs)
    batch.prepare(1)
    batch.sync_seq_lens()
    idx = torch.full((B * Hq, budget - 1), -1, dtype=torch.int32, device=DEV)
    o = batch.decode_step_dev(q.to(DEV), k_new.to(DEV), v_new.to(DEV), 0, indices_out=idx)
    torch.cuda.synchronize()
    assert int(K.histogram_counts(batch._hist).abs().sum().item()) == 0
    for i in range(B):
        assert torch.equal(idx[i * Hq:(i + 1) * Hq], want_idx[i]), f"sequence {i}: selected slots"
        _assert_attn_close(o[i], want_o[i])
    del cs, cs2, ks, vs, batch
    torch.cuda.empty_cache()
    # one long sequence of many heads, against the oracle
    L, H2 = 66000, 64
    cs, ks, vs = _controllers([L], H2, H2, ps, budget // ps, dtype, L + 2 * ps, seed=33)
    c = cs[0]
    q1 = _randn((1, H2, 128), 6, dtype)
    c.prepare_hadamard(1)
    c.begin_forward(1)
    o = U.decode_step(q1.to(DEV), ks[0][L - 1:L].to(DEV), vs[0][L - 1:L].to(DEV), c, 0)
    torch.cuda.synchronize()
    r = ref.decode_step(q1[0], ks[0][:L], vs[0][:L], budget)
    table = np.asarray(c.kv_cache.indicies)
    np.testing.assert_array_equal(c.topk_dindices_buffer.cpu().numpy(), table[r["sel"] // ps] * ps + r["sel"] % ps)
    _assert_attn_close(o[0], r["out"])
    from adamas_b200 import _lib
    assert _lib.device_error(clear=False) == 0
