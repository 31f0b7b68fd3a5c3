"""select_attend (top-k and sparse attention in one launch, the second kernel of the fused decode step)
on crafted distance rows, called directly through the C ABI: the selection is re-implemented inside
that kernel, so it gets the adversarial cases of the stand-alone top-k tests of its own.

Semantics as in the reference's operator tests (adamas/tests/test_approx_attention.py:66-86): the k
smallest distances over tokens [0, n) plus the newest token (position n), ties to the lower position.
"""
import numpy as np
import pytest
import torch

from oracle import adamas_ref as ref
from test_gpu_parity import DEV, State, _assert_attn_close, _mods

pytestmark = pytest.mark.gpu


def _rows(name: str, H: int, n: int, k: int, seed: int) -> np.ndarray:
    """[H, n] uint16 distance rows of one adversarial family."""
    rng = np.random.default_rng(seed)
    d = np.full((H, n), 200, dtype=np.uint16)
    if name == "first_slice":            # every winner at the very start of the row
        d[:, :k] = 10
    elif name == "last_slice":           # every winner at the very end
        d[:, n - k:] = 10
    elif name == "all_equal":            # every element ties: the first k positions win
        d[:] = 77
    elif name == "one_below_rest_tied":
        d[:] = 50
        d[np.arange(H), rng.integers(0, n, H)] = 3
    elif name == "random_ties":          # a narrow range: hundreds of ties at the cut
        d = rng.integers(40, 60, (H, n)).astype(np.uint16)
    elif name == "random_wide":
        d = rng.integers(0, 385, (H, n)).astype(np.uint16)
    elif name == "huge_values":          # beyond the largest possible distance: 511 and more count as equal
        d = rng.integers(300, 400, (H, n)).astype(np.uint16)
        d[:, ::3] = 600
        d[:, 1::7] = 511
        d[:, 2::11] = 65535
        d[:, 5::13] = 512
    elif name == "winners_in_one_block":  # a burst in the middle of the row
        lo = max(0, n // 2 - k // 2)
        d[:, lo:lo + k] = rng.integers(0, 5, (H, min(k, n - lo))).astype(np.uint16)
    else:
        raise ValueError(name)
    return d


def _check(st: State, dist: np.ndarray, k: int, with_idx: bool, K):
    H, n = dist.shape
    c = st.c
    stride = (n + 7) // 8 * 8
    dbuf = torch.zeros(H, stride, dtype=torch.int16, device=DEV)
    dbuf[:, :n] = torch.from_numpy(dist.view(np.int16)).to(DEV)
    d = dbuf[:, :n]
    o = torch.full((1, H, 128), float("nan"), dtype=st.dtype, device=DEV)
    idx = torch.full((H, k), -7, dtype=torch.int32, device=DEV) if with_idx else None
    hist = K.histogram_scratch(H, DEV)
    lse = torch.zeros(H, dtype=torch.float32, device=DEV)
    K.select_attend(d, k, st.qd, o, c.kv_cache.buf_layer(0), c.kv_indices_with_last, c.kv_cache.last_page_len,
                    c.kv_last_page_idx, indices_out=idx, lse=lse, hist=hist)
    torch.cuda.synchronize()
    assert int(K.histogram_counts(hist).abs().sum().item()) == 0, "the histogram table is left dirty"
    sel = ref.select_topk(np.minimum(dist, 511).astype(np.int64), k)
    if with_idx:
        table = np.asarray(c.kv_cache.indicies)
        np.testing.assert_array_equal(idx.cpu().numpy(), table[sel // st.ps] * st.ps + sel % st.ps)
    full = np.concatenate([sel, np.full((H, 1), n, dtype=np.int64)], axis=1)
    want, want_lse = ref.sparse_attention(st.q[0], st.k, st.v, full, return_lse=True)
    _assert_attn_close(o[0], want)
    torch.testing.assert_close(lse.cpu() * float(np.log(2.0)), want_lse, rtol=1e-3, atol=1e-3)


FAMILIES = ["first_slice", "last_slice", "all_equal", "one_below_rest_tied", "random_ties", "random_wide",
            "huge_values", "winners_in_one_block"]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("ps", [1, 3, 16])
@pytest.mark.parametrize("n,k", [(1, 1), (7, 7), (7, 1), (9, 4), (100, 100), (4097, 1), (4097, 1023), (4097, 4097),
                                 (20000, 640)])
def test_select_attend_adversarial_rows(dtype, ps, n, k):
    _, K, _ = _mods()
    H = 8
    st = State(n + 1, H, ps, dtype, seed=n + k, fused=True)
    for i, name in enumerate(FAMILIES):
        _check(st, _rows(name, H, n, k, seed=i + n), k, with_idx=(i % 2 == 0), K=K)
    from adamas_b200 import _lib
    assert _lib.device_error(clear=False) == 0


@pytest.mark.parametrize("blocks", [1, 2, 4, 8])
@pytest.mark.parametrize("n,k,H", [(4097, 1023, 32), (30000, 255, 8)])
def test_select_attend_every_cluster_shape(blocks, n, k, H):
    _, K, _ = _mods()
    st = State(n + 1, H, 16, torch.float16, seed=blocks + n, fused=True)
    K.set_max_cluster(blocks)
    try:
        assert K.select_attend_slices(n, k, H) <= blocks
        for i, name in enumerate(["first_slice", "last_slice", "all_equal", "random_ties", "winners_in_one_block"]):
            _check(st, _rows(name, H, n, k, seed=i), k, with_idx=True, K=K)
    finally:
        K.set_max_cluster(8)


@pytest.mark.parametrize("n,k,H", [(140000, 2047, 2), (262144, 100, 1)])
def test_select_attend_sixteen_block_clusters(n, k, H):
    """Long rows of few heads run with 16 thread blocks per head."""
    _, K, _ = _mods()
    st = State(n + 1, H, 16, torch.float16, seed=n, fused=True)
    for i, name in enumerate(["first_slice", "last_slice", "all_equal", "random_ties"]):
        _check(st, _rows(name, H, n, k, seed=i), k, with_idx=True, K=K)
    from adamas_b200 import _lib
    assert _lib.device_error(clear=False) == 0


def test_select_attend_with_prepared_histograms_and_without_newest_token():
    """The two-call form (estimate with hist, select_attend with hist_ready) and last_page_len = 0
    (no newest token: a sequence shard that does not hold it), with an fp32 partial output."""
    _, K, U = _mods()
    L, H, ps, k = 3000, 8, 16, 200
    st = State(L, H, ps, torch.float16, seed=4, fused=True)
    c = st.c
    n = L - 1
    slices = K.select_attend_slices(n, k, H)
    dist = c.distance_scratch(n)
    hist = K.histogram_scratch(H, DEV)
    K.estimate_attn_score(st.q_code, dist, c.hadamard_cache.buf_layer(0), c.hadamard_indices, None,
                          c.hadamard_cache.last_page_len, c.hadamard_last_page_idx, c.layout, hist=hist,
                          hist_slices=slices)
    torch.cuda.synchronize()
    r = ref.decode_step(st.q[0], st.k, st.v, k + 1)
    np.testing.assert_array_equal(dist.cpu().numpy().astype(np.int32), r["dist"])
    got_hist = K.histogram_counts(hist).cpu().numpy().sum(1)[:, :385]
    want_hist = np.stack([np.bincount(row, minlength=385) for row in r["dist"]])
    np.testing.assert_array_equal(got_hist, want_hist)
    # the counting launch of its own gives the same table, slice by slice
    hist2 = K.histogram_scratch(H, DEV)
    K.dist_histograms(dist, hist2, slices)
    assert torch.equal(K.histogram_counts(hist2), K.histogram_counts(hist))
    o32 = torch.zeros(H, 128, dtype=torch.float32, device=DEV)
    lse = torch.zeros(H, dtype=torch.float32, device=DEV)
    idx = torch.zeros(H, k, dtype=torch.int32, device=DEV)
    K.select_attend(dist, k, st.qd, None, c.kv_cache.buf_layer(0), c.kv_indices_with_last, 0, c.kv_last_page_idx,
                    indices_out=idx, lse=lse, hist=hist, hist_ready=True, o_f32=o32)
    torch.cuda.synchronize()
    assert int(K.histogram_counts(hist).abs().sum().item()) == 0
    table = np.asarray(c.kv_cache.indicies)
    np.testing.assert_array_equal(idx.cpu().numpy(), table[r["sel"] // ps] * ps + r["sel"] % ps)
    want, want_lse = ref.sparse_attention(st.q[0], st.k, st.v, r["sel"], return_lse=True)
    torch.testing.assert_close(o32.cpu(), want, rtol=2e-3, atol=2e-3 * float(want.abs().max()))
    torch.testing.assert_close(lse.cpu() * float(np.log(2.0)), want_lse, rtol=1e-3, atol=1e-3)


def test_select_attend_with_cut_decided_elsewhere():
    """ext_cut: the cut distance and this call's share of the cut-valued elements come from outside
    (the global cut of a sequence split over GPUs): everything below the cut and the first `take` ties."""
    _, K, _ = _mods()
    n, H, ps = 5000, 4, 16
    st = State(n + 1, H, ps, torch.float16, seed=8, fused=True)
    c = st.c
    rng = np.random.default_rng(1)
    dist = rng.integers(90, 110, (H, n)).astype(np.uint16)
    cut = np.array([95, 100, 90, 109])
    take = np.array([0, 17, 3, 250])
    sel = []
    for h in range(H):
        below = np.flatnonzero(dist[h] < cut[h])
        ties = np.flatnonzero(dist[h] == cut[h])[: take[h]]
        sel.append(np.sort(np.concatenate([below, ties])))
    kmax = max(len(s) for s in sel)
    dbuf = torch.zeros(H, (n + 7) // 8 * 8, dtype=torch.int16, device=DEV)
    dbuf[:, :n] = torch.from_numpy(dist.view(np.int16)).to(DEV)
    ext = torch.tensor(np.stack([cut, take], 1), dtype=torch.int32, device=DEV)
    idx = torch.full((H, kmax), -1, dtype=torch.int32, device=DEV)
    o = torch.zeros(1, H, 128, dtype=torch.float16, device=DEV)
    K.select_attend(dbuf[:, :n], kmax, st.qd, o, c.kv_cache.buf_layer(0), c.kv_indices_with_last,
                    c.kv_cache.last_page_len, c.kv_last_page_idx, indices_out=idx, ext_cut=ext)
    torch.cuda.synchronize()
    table = np.asarray(c.kv_cache.indicies)
    for h in range(H):
        np.testing.assert_array_equal(idx[h, : len(sel[h])].cpu().numpy(), table[sel[h] // ps] * ps + sel[h] % ps)
        full = np.concatenate([sel[h], [n]])[None, :]
        want = ref.sparse_attention(st.q[0, h:h + 1], st.k[:, h:h + 1], st.v[:, h:h + 1], full)
        _assert_attn_close(o[0, h:h + 1], want)


def test_stale_histogram_table_is_reported_not_followed():
    """A table that does not describe the rows (here: all zero although hist_ready is claimed) raises
    the device error flag; the call still ends and attends to the newest token only."""
    _, K, _ = _mods()
    from adamas_b200 import _lib
    n, H, k = 1000, 4, 10
    st = State(n + 1, H, 16, torch.float16, seed=2, fused=True)
    c = st.c
    _lib.device_error(clear=True)
    dist = torch.full((H, 1000), 5, dtype=torch.int16, device=DEV)
    o = torch.zeros(1, H, 128, dtype=torch.float16, device=DEV)
    K.select_attend(dist, k, st.qd, o, c.kv_cache.buf_layer(0), c.kv_indices_with_last, c.kv_cache.last_page_len,
                    c.kv_last_page_idx, hist=K.histogram_scratch(H, DEV), hist_ready=True)
    torch.cuda.synchronize()
    assert _lib.device_error(clear=True) == 8
    want = st.v[n].float()          # softmax over one token
    _assert_attn_close(o[0], want)
