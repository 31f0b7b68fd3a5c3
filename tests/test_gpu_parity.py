"""Parity of the CUDA path (called through the C ABI) with the CPU oracle on the same seeded
inputs.  Integer results (codes, distances, selected indices) must be bit-exact; attention outputs
must agree within 2e-3 relative (fp16 / bf16), the tolerance the task states.

Shape lists follow the reference's own tests: adamas/tests/test_estimate.py:66,
adamas/tests/test_topk.py:22, adamas/tests/test_approx_attention.py:100,
kernels/src/test/test_batch_decode.cu:215-257.
"""
import functools
import math
import os

import numpy as np
import pytest
import torch

from oracle import adamas_ref as ref

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
REL_TOL = 2e-3


def _mods():
    import adamas_b200
    from adamas_b200 import _kernels, utils
    return adamas_b200, _kernels, utils


def _randn(shape, seed, dtype=torch.float16, sigma=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * sigma).to(dtype)


def _assert_attn_close(got: torch.Tensor, want: torch.Tensor):
    got = got.detach().float().cpu()
    want = want.detach().float().cpu()
    atol = REL_TOL * float(want.abs().max())
    torch.testing.assert_close(got, want, rtol=REL_TOL, atol=atol)


def _codes_of(buf: torch.Tensor) -> np.ndarray:
    return buf.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


class State:
    """A sequence pushed through the host API the way the reference's tests do it: prefill of
    L-1 tokens (append_kvh), then one decode append."""

    def __init__(self, L, H=32, ps=1, dtype=torch.float16, seed=0, sigma=1.0, scale=None, budget_pages=64,
                 fused=False, layers=1, max_seq_len=None):
        _, K, U = _mods()
        self.L, self.H, self.ps, self.dtype, self.scale = L, H, ps, dtype, scale
        self.q = _randn((1, H, 128), seed, dtype, sigma)
        self.k = _randn((L, H, 128), seed + 1, dtype, sigma)
        self.v = _randn((L, H, 128), seed + 2, dtype)
        cap = max_seq_len or (L + 3 * ps + 5)
        self.c = U.InferenceController(layers, H, 128, ps, budget_pages, cap, dtype, DEV)
        # hand out physical pages in a shuffled order
        rng = np.random.default_rng(seed)
        for cache in (self.c.kv_cache, self.c.hadamard_cache):
            pool = cache.pool
            rng.shuffle(pool._free)
            pool.alloc_block = functools.partial(_pop_random, pool)
        qd, kd, vd = self.q.to(DEV), self.k.to(DEV), self.v.to(DEV)
        c = self.c
        if L > 1:
            c.prepare_hadamard(L - 1)
            c.begin_forward(max(L - 1, 2))      # prefill-style set-up even for a single token
            if L - 1 > 1:
                h = None if fused else K.hadamard_transform(kd[: L - 1], scale=scale)
                if fused and scale is not None:
                    K.append_kv_cache_prefill(kd[: L - 1].contiguous(), vd[: L - 1].contiguous(), None,
                                              c.kv_cache.buf_layer(0), c.kv_indices_with_last, None,
                                              c.kv_cache.last_page_len, c.kv_last_page_idx,
                                              c.hadamard_cache.buf_layer(0), c.hadamard_indices, None,
                                              c.hadamard_cache.last_page_len, c.hadamard_last_page_idx, c.layout,
                                              scale=scale)
                else:
                    U.append_kvh(kd[: L - 1].contiguous(), vd[: L - 1].contiguous(), h, c, 0)
            else:
                # a single prefill token goes through the decode append
                h = K.hadamard_transform(torch.cat((qd, kd[:1]), 0), scale=scale)
                U.append_kvh(kd[:1].contiguous(), vd[:1].contiguous(), h, c, 0)
            c.end_forward()
        c.prepare_hadamard(1)
        c.begin_forward(1)
        if fused:
            self.q_code = U.append_qkv_fused(qd, kd[L - 1:].contiguous(), vd[L - 1:].contiguous(), c, 0, scale=scale)
        else:
            h = K.hadamard_transform(torch.cat((qd, kd[L - 1:]), 0), scale=scale)
            self.q_code = U.append_kvh(kd[L - 1:].contiguous(), vd[L - 1:].contiguous(), h, c, 0)
        self.qd = qd

    def oracle_codes(self):
        return ref.encode(self.q[0], self.scale), ref.encode(self.k, self.scale)

    def cached_codes(self) -> np.ndarray:
        """[L, H, 16] uint16 read back from the paged code cache."""
        c = self.c
        buf = _codes_of(c.hadamard_cache.buf_layer(0))            # [P, 1, ps, H, 16]
        table = np.asarray(c.hadamard_cache.indicies)
        t = np.arange(self.L)
        return buf[table[t // self.ps], 0, t % self.ps]

    def cached_kv(self):
        c = self.c
        buf = c.kv_cache.buf_layer(0).cpu()
        table = torch.tensor(c.kv_cache.indicies)
        t = torch.arange(self.L)
        return buf[table[t // self.ps], 0, t % self.ps], buf[table[t // self.ps], 1, t % self.ps]


def _pop_random(pool):
    idx = pool._free.pop()
    pool._in_use.add(idx)
    return idx


# ------------------------------------------------------------------------------------------------
# stage 1
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,sigma,scale", [(1, 1.0, None), (37, 1.0, None), (64 * 33 + 5, 3.0, 1.0), (4096, 11.0, None)])
def test_hadamard_transform_bit_exact(dtype, rows, sigma, scale):
    _, K, _ = _mods()
    x = _randn((rows, 128), 11 + rows, dtype, sigma)
    y = K.hadamard_transform(x.to(DEV), scale=scale)
    want = ref.hadamard_transform(x, scale)
    assert torch.equal(y.cpu().view(torch.int16), want.view(torch.int16))
    # in place, 3-D input
    x3 = x[: (rows // 2) * 2].reshape(-1, 2, 128).contiguous().to(DEV) if rows >= 2 else x.reshape(1, 1, 128).to(DEV)
    ref3 = ref.hadamard_transform(x3.cpu(), scale)
    out = K.hadamard_transform(x3, inplace=True, scale=scale)
    assert out.data_ptr() == x3.data_ptr()
    assert torch.equal(x3.cpu().view(torch.int16), ref3.view(torch.int16))


def test_bucketize_pack_all_buckets_and_boundaries():
    _, K, _ = _mods()
    vals = torch.tensor([-65504.0, -11.0, -10.0, -9.99, -0.0, 0.0, 6e-8, 9.99, 10.0, 10.01, 65504.0, 1.0, -1.0, 5.0, -5.0, 0.5])
    h = vals.repeat(8).reshape(1, 1, 128).to(torch.float16)
    h = torch.cat([h, _randn((6, 1, 128), 3, torch.float16, 9.0)], 0)
    o = torch.zeros(7, 1, 16, dtype=torch.int16, device=DEV)
    K.bucketize_pack(h.to(DEV), o)
    want = ref.pack_2bit(ref.bucketize(h.float().numpy()))
    np.testing.assert_array_equal(_codes_of(o), want)
    # the reference's name for the same operator (adamas/ops/csrc/page.cu:271-298)
    o2 = torch.zeros_like(o)
    K.pack_2bit(h.to(DEV), o2, 0)
    assert torch.equal(o2, o)
    # custom thresholds
    K.bucketize_pack(h.to(DEV), o, thresholds=(-1.0, 0.25, 2.0))
    want = ref.pack_2bit(ref.bucketize(h.float().numpy(), (-1.0, 0.25, 2.0)))
    np.testing.assert_array_equal(_codes_of(o), want)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("L,H,ps,sigma,scale", [
    (2, 32, 1, 1.0, None), (27, 32, 1, 1.0, None), (61, 8, 16, 1.0, None), (113, 32, 3, 3.0, 1.0),
    (577, 32, 16, 3.0, 1.0), (1110, 4, 7, 1.0, None), (3330, 32, 1, 1.0, None), (2049, 40, 32, 3.0, 1.0),
])
def test_append_codes_and_kv_bit_exact(dtype, fused, L, H, ps, sigma, scale):
    st = State(L, H, ps, dtype, seed=L, sigma=sigma, scale=scale, fused=fused)
    q_code, k_codes = st.oracle_codes()
    np.testing.assert_array_equal(_codes_of(st.q_code)[0], q_code)
    np.testing.assert_array_equal(st.cached_codes(), k_codes)
    kk, vv = st.cached_kv()
    assert torch.equal(kk.view(torch.int16), st.k.view(torch.int16))
    assert torch.equal(vv.view(torch.int16), st.v.view(torch.int16))
    if sigma > 1.0:
        assert set(np.unique(ref.unpack_2bit(k_codes))) == {0, 1, 2, 3}


@pytest.mark.parametrize("past_kv_len", [13, 24, 51, 77, 244, 311, 502, 1110, 32760])   # adamas/tests/test_rope.py:33
@pytest.mark.parametrize("seq_len", [1, 2, 5, 19, 69, 251])
def test_rope_in_place(past_kv_len, seq_len):
    _, K, U = _mods()
    scale = 8.0 if past_kv_len > 2000 else 1.0
    q = _randn((seq_len, 32, 128), past_kv_len + seq_len, torch.float16)
    k = _randn((seq_len, 32, 128), past_kv_len + seq_len + 1, torch.float16)
    qd, kd = q.to(DEV), k.to(DEV)
    U.apply_rope_in_place(qd, kd, past_kv_len, rope_scale=scale)
    # the reference's tolerance for this operator (adamas/tests/test_rope.py:10-15)
    torch.testing.assert_close(qd.cpu().float(), ref.rope(q, past_kv_len, scale).float(), rtol=5e-3, atol=5e-3)
    torch.testing.assert_close(kd.cpu().float(), ref.rope(k, past_kv_len, scale).float(), rtol=5e-3, atol=5e-3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("past_kv_len,seq_len", [(0, 69), (4095, 3), (40000, 1), (131071, 1)])
def test_rope_table_in_place_yarn(dtype, past_kv_len, seq_len):
    """Per-dimension rotation frequencies and a factor on the rotated values (YaRN), against the
    oracle's restatement, at the reference's tolerance for its own RoPE operator scaled by the factor."""
    _, K, U = _mods()
    # the same table on both sides: at position 131071 one unit in the last place of a frequency moves the
    # angle by 0.008 rad (the table itself is compared with transformers' on the CPU)
    want_inv, want_scale = ref.yarn_parameters(32.0, 4096)
    mscale = want_scale
    q = _randn((seq_len, 32, 128), past_kv_len + seq_len, dtype)
    k = _randn((seq_len, 8, 128), past_kv_len + seq_len + 1, dtype)
    qd, kd = q.to(DEV), k.to(DEV)
    K.apply_rope_table_in_place(qd, kd, past_kv_len, want_inv.to(DEV), mscale)
    tol = 5e-3 * (4 if dtype == torch.bfloat16 else 1) * mscale
    torch.testing.assert_close(qd.cpu().float(), ref.rope_table(q, past_kv_len, want_inv, want_scale).float(), rtol=tol, atol=tol)
    torch.testing.assert_close(kd.cpu().float(), ref.rope_table(k, past_kv_len, want_inv, want_scale).float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_yarn_fused_append_equals_separate_launches(dtype):
    """The append launch with the frequency table rotates exactly as the stand-alone table operator."""
    _, K, U = _mods()
    from adamas_b200.rope import yarn_inv_freq
    inv_freq, mscale = yarn_inv_freq(32.0, 4096)
    rope = {"inv_freq": inv_freq.to(DEV), "mscale": mscale}
    L, H, ps = 9000, 32, 16
    outs = []
    for fused in (False, True):
        st = State(L - 1, H, ps, dtype, seed=4, fused=True, max_seq_len=L + ps)
        c = st.c
        c.end_forward()
        q = _randn((1, H, 128), 71, dtype).to(DEV)
        k = _randn((1, H, 128), 72, dtype).to(DEV)
        v = _randn((1, H, 128), 73, dtype).to(DEV)
        c.prepare_hadamard(1)
        c.begin_forward(1)
        if fused:
            code = U.append_qkv_fused(q, k, v, c, 0, rope=rope)
        else:
            K.apply_rope_table_in_place(q, k, L - 1, rope["inv_freq"], mscale)
            code = U.append_qkv_fused(q, k, v, c, 0)
        table = c.kv_cache.indicies
        kv = c.kv_cache.buf_layer(0)[table[-1], :, (L - 1) % ps].clone()
        outs.append((q.clone(), k.clone(), code.clone(), kv))
    for a, b in zip(*outs):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_rope_fused_append_equals_separate_launches(dtype):
    """rope + cat + hadamard + append in one launch gives the same bits as the separate operators."""
    _, K, U = _mods()
    L, H, ps = 500, 32, 16
    outs = []
    for fused in (False, True):
        st = State(L - 1, H, ps, dtype, seed=4, fused=True, max_seq_len=L + ps)
        c = st.c
        c.end_forward()
        q = _randn((1, H, 128), 71, dtype).to(DEV)
        k = _randn((1, H, 128), 72, dtype).to(DEV)
        v = _randn((1, H, 128), 73, dtype).to(DEV)
        c.prepare_hadamard(1)
        c.begin_forward(1)
        if fused:
            code = U.append_qkv_fused(q, k, v, c, 0, rope=(8.0, 1e4))
        else:
            U.apply_rope_in_place(q, k, L - 1, rope_scale=8.0)
            code = U.append_qkv_fused(q, k, v, c, 0)
        table = c.kv_cache.indicies
        kv = c.kv_cache.buf_layer(0)[table[-1], :, (L - 1) % ps].clone()
        codes = c.hadamard_cache.buf_layer(0)[c.hadamard_cache.indicies[-1], 0, (L - 1) % ps].clone()
        outs.append((q.clone(), k.clone(), code.clone(), kv, codes))
    for a, b in zip(*outs):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))


# ------------------------------------------------------------------------------------------------
# stage 2
# ------------------------------------------------------------------------------------------------
EST_LENS = [27, 61, 113, 482, 577, 1110, 1541, 2047, 3330]   # adamas/tests/test_estimate.py:66


@pytest.mark.parametrize("kv_len", EST_LENS + [2, 3, 33, 4096])
@pytest.mark.parametrize("ps", [1, 16])
def test_estimate_bit_exact(kv_len, ps):
    _, K, U = _mods()
    wide = kv_len % 2 == 1
    st = State(kv_len, 32, ps, seed=kv_len, sigma=3.0 if wide else 1.0, scale=1.0 if wide else None)
    q_code, k_codes = st.oracle_codes()
    for metric in ("l1", "xor"):
        want = ref.code_distance(q_code, k_codes[:-1], metric)
        got = U.decode_estimate(st.q_code, st.c, 0, metric=metric)
        assert got.dtype == torch.float16 and tuple(got.shape) == (32, kv_len - 1)
        np.testing.assert_array_equal(got.float().cpu().numpy().astype(np.int32), want)
        # integer output format
        o16 = torch.full((32, kv_len - 1), -1, dtype=torch.int16, device=DEV)
        K.estimate_attn_score(st.q_code, o16, st.c.hadamard_cache.buf_layer(0), st.c.hadamard_indices, None,
                              st.c.hadamard_cache.last_page_len, st.c.hadamard_last_page_idx, 0, metric)
        np.testing.assert_array_equal(o16.cpu().numpy().astype(np.int32), want)
    if wide:
        assert (ref.code_distance(q_code, k_codes[:-1], "xor") != ref.code_distance(q_code, k_codes[:-1], "l1")).any()


@pytest.mark.parametrize("H", [1, 4, 8, 40, 64])
def test_estimate_other_head_counts(H):
    _, _, U = _mods()
    st = State(300, H, 16, seed=H, sigma=3.0, scale=1.0)
    q_code, k_codes = st.oracle_codes()
    got = U.decode_estimate(st.q_code, st.c, 0)
    np.testing.assert_array_equal(got.float().cpu().numpy().astype(np.int32),
                                  ref.code_distance(q_code, k_codes[:-1], "l1"))


@pytest.mark.parametrize("H", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("L,ps", [(2, 16), (17, 16), (530, 16), (4099, 16), (9000, 32), (700, 3), (1000, 1)])
@pytest.mark.parametrize("metric", ["l1", "xor"])
def test_estimate_few_heads_page_copies(H, L, ps, metric):
    """Head-sharded shapes (16 heads or fewer): the estimate copies whole pages of codes when a page
    is at least 512 bytes, and token by token otherwise; both against the oracle, including rows
    that end inside a page and inside a tile."""
    _, _, U = _mods()
    st = State(L, H, ps, seed=3 * H + L, sigma=3.0, scale=1.0)
    q_code, k_codes = st.oracle_codes()
    got = U.decode_estimate(st.q_code, st.c, 0, metric=metric)
    np.testing.assert_array_equal(got.float().cpu().numpy().astype(np.int32),
                                  ref.code_distance(q_code, k_codes[:-1], metric))
    from adamas_b200 import _lib
    assert _lib.device_error(clear=False) == 0


def test_estimate_golden_reference_vectors():
    """Distances for the fixtures produced by the reference's own _ref_cpu_estimate."""
    _, K, U = _mods()
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_python_path.npz"))
    for name in sorted({k.split(".")[0] for k in gold.files}):
        f16 = lambda a: torch.from_numpy(a.copy()).view(torch.float16)
        q, k, v = f16(gold[name + ".q"]), f16(gold[name + ".k"]), f16(gold[name + ".v"])
        scale = None if gold[name + ".scale"] < 0 else float(gold[name + ".scale"])
        L, H, _ = k.shape
        c = U.InferenceController(1, H, 128, 1, 8, L + 8, torch.float16, DEV)
        c.prepare_hadamard(L - 1); c.begin_forward(L - 1)
        U.append_kvh(k[: L - 1].to(DEV), v[: L - 1].to(DEV), K.hadamard_transform(k[: L - 1].to(DEV), scale=scale), c, 0)
        c.end_forward()
        c.prepare_hadamard(1); c.begin_forward(1)
        h = K.hadamard_transform(torch.cat((q, k[L - 1:]), 0).to(DEV), scale=scale)
        q_code = U.append_kvh(k[L - 1:].to(DEV), v[L - 1:].to(DEV), h, c, 0)
        assert torch.equal(q_code.cpu().view(torch.int16), torch.from_numpy(gold[name + ".q_code"].copy()))
        est = U.decode_estimate(q_code, c, 0)
        assert torch.equal(est.cpu().view(torch.int16), torch.from_numpy(gold[name + ".est"].copy()))
        c.end_forward()


# ------------------------------------------------------------------------------------------------
# stage 3
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kv_len", [13, 24, 51, 77, 244, 311, 502, 1110])      # adamas/tests/test_topk.py:22
@pytest.mark.parametrize("k_budget", [2, 5, 7, 19, 31, 69, 111, 251])
def test_topk_reference_shapes(kv_len, k_budget):
    if k_budget > kv_len:
        pytest.skip("k should be less than kv_len")
    _, K, _ = _mods()
    q = _randn((32, 1, 128), kv_len, torch.float16)
    k = _randn((32, kv_len, 128), kv_len + 1, torch.float16)
    attn = (torch.matmul(q.float(), k.float().transpose(1, 2)) / math.sqrt(128)).squeeze(1).to(torch.float16)
    vals = attn.to(DEV).contiguous()
    in_idx = (torch.arange(kv_len, dtype=torch.int32) * 3 + 1).repeat(32, 1).to(DEV)
    d_out = torch.zeros(32, k_budget, dtype=torch.float16, device=DEV)
    i_out = torch.zeros(32, k_budget, dtype=torch.int32, device=DEV)
    buf = torch.zeros(32, 1024, dtype=torch.float16, device=DEV)
    K.topk_filtering(vals, in_idx, d_out, i_out, buf, k_budget)
    want = ref.select_topk(attn.numpy(), k_budget)
    np.testing.assert_array_equal(i_out.cpu().numpy(), want * 3 + 1)
    np.testing.assert_array_equal(d_out.cpu().numpy().view(np.uint16),
                                  np.take_along_axis(attn.numpy(), want, 1).view(np.uint16))
    # the reference's own check: sum of the selected values equals torch.topk's
    tsum = torch.topk(attn.float(), k=k_budget, dim=-1, largest=False).values.sum(-1)
    torch.testing.assert_close(d_out.float().cpu().sum(-1), tsum, rtol=5e-3, atol=5e-3)


@pytest.mark.parametrize("n,k", [(1, 1), (7, 7), (8, 1), (4095, 255), (4096, 4095), (32767, 1023), (32767, 63),
                                 (131071, 2047), (250000, 4095), (300001, 1000)])
@pytest.mark.parametrize("fmt", ["dist_f16", "dist_u16"])
def test_topk_distances_with_ties(n, k, fmt):
    """Binomial-like integer distances (the real input of this stage): massive ties at the cut."""
    _, K, _ = _mods()
    rng = np.random.default_rng(n + k)
    rows = 5 if n > 100000 else 32
    d = rng.binomial(128, 0.5, size=(rows, n)).astype(np.int32)
    if fmt == "dist_f16":
        vals = torch.from_numpy(d.astype(np.float16))
    else:
        vals = torch.from_numpy(d.astype(np.int16))
    # odd row stride: rows start at 2-byte-aligned addresses only
    store = torch.zeros(rows, n + 3, dtype=vals.dtype, device=DEV)
    store[:, 1:n + 1] = vals.to(DEV)
    view = store[:, 1:n + 1]
    i_out = torch.full((rows, k), -1, dtype=torch.int32, device=DEV)
    v_out = torch.zeros((rows, k), dtype=vals.dtype, device=DEV)
    K.topk_select(view, k, i_out, v_out)
    want = ref.select_topk(d, k)
    np.testing.assert_array_equal(i_out.cpu().numpy(), want)
    np.testing.assert_array_equal(v_out.cpu().numpy().astype(np.int32), np.take_along_axis(d, want, 1))
    # determinism: a second run gives the same bytes
    i2 = torch.full((rows, k), -1, dtype=torch.int32, device=DEV)
    K.topk_select(view, k, i2)
    assert torch.equal(i2, i_out)


def test_topk_adversarial_values():
    _, K, _ = _mods()
    rows = [
        np.full(1000, 7.0),                                   # all ties
        np.concatenate([np.zeros(500), -np.zeros(500)]),      # +0 / -0 are equal
        np.linspace(-100, 100, 1000),                          # negatives, ascending
        np.linspace(100, -100, 1000),                          # descending
        np.concatenate([np.full(999, 65504.0), [-65504.0]]),   # extreme values, winner last
    ]
    a = np.stack(rows).astype(np.float16)
    vals = torch.from_numpy(a).to(DEV)
    for k in (1, 2, 499, 500, 501, 999, 1000):
        i_out = torch.zeros((len(rows), k), dtype=torch.int32, device=DEV)
        K.topk_select(vals, k, i_out)
        np.testing.assert_array_equal(i_out.cpu().numpy(), ref.select_topk(a, k))


def test_topk_maps_positions_through_page_table():
    _, K, _ = _mods()
    n, ps, k = 1000, 16, 100
    d = np.random.default_rng(5).integers(0, 384, size=(4, n)).astype(np.int16)
    table = torch.from_numpy(np.random.default_rng(6).permutation(200)[: (n + ps - 1) // ps].astype(np.int32))
    i_out = torch.zeros((4, k), dtype=torch.int32, device=DEV)
    K.topk_select(torch.from_numpy(d).to(DEV), k, i_out, page_table=table.to(DEV), page_size=ps)
    want = ref.select_topk(d.astype(np.int32), k)
    np.testing.assert_array_equal(i_out.cpu().numpy(), table.numpy()[want // ps] * ps + want % ps)


def test_topk_rejects_bad_arguments():
    _, K, _ = _mods()
    vals = torch.zeros(2, 10, dtype=torch.float16, device=DEV)
    out = torch.zeros(2, 11, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):
        K.topk_select(vals, 11, out)
    with pytest.raises(RuntimeError):
        K.topk_select(vals, 0, out)
    with pytest.raises(RuntimeError):
        K.topk_select(vals.to(torch.bfloat16), 3, out)


# ------------------------------------------------------------------------------------------------
# stage 4
# ------------------------------------------------------------------------------------------------
def _attend(st, idx_tokens):
    """oracle output for per-head token positions idx_tokens [H, m]"""
    return ref.sparse_attention(st.q[0], st.k, st.v, idx_tokens)


@pytest.mark.parametrize("kv_len", [27, 61, 113, 482, 577, 1011, 1541])       # test_approx_attention.py:100
@pytest.mark.parametrize("token_budget", [64, 112, 240, 496, 880, 1136])
def test_sparse_attention_reference_shapes(kv_len, token_budget):
    """Page size 1, indices taken from the oracle's top-k, as the reference's test feeds its kernel."""
    _, K, U = _mods()
    st = State(kv_len, 32, 1, seed=kv_len + token_budget, budget_pages=token_budget)
    r = ref.decode_step(st.q[0], st.k, st.v, token_budget)
    c = st.c
    if not c.need_estimate():
        assert kv_len <= token_budget
        o = U.decode_sparse_attn(st.qd, c, 0, c.kv_indices_without_last)
    else:
        table = np.asarray(c.kv_cache.indicies)
        idx = torch.from_numpy(table[r["sel"]].astype(np.int32)).to(DEV)
        o = U.decode_sparse_attn(st.qd, c, 0, idx)
    _assert_attn_close(o[0], r["out"])


@pytest.mark.parametrize("seq_len", [63, 129, 1024, 7777, 28837])     # test_batch_decode.cu:215-257
@pytest.mark.parametrize("ps", [1, 3, 7, 16, 32])
@pytest.mark.parametrize("page_budget", [16, 128])
def test_sparse_attention_page_granular(seq_len, ps, page_budget):
    """Random per-head page lists plus the forced last page (the reference kernel's meaning of
    the index list), every page attended in full."""
    _, K, U = _mods()
    H = 8
    st = State(seq_len, H, ps, seed=seq_len + ps, budget_pages=page_budget)
    c = st.c
    n_pages = len(c.kv_cache.indicies)
    rng = np.random.default_rng(seq_len * 31 + ps)
    n_sel = min(page_budget - 1, n_pages - 1)
    if n_sel < 1:
        pytest.skip("needs at least two pages")
    logical = np.stack([np.sort(rng.choice(n_pages - 1, size=n_sel, replace=False)) for _ in range(H)])
    table = np.asarray(c.kv_cache.indicies)
    idx = torch.from_numpy(table[logical].astype(np.int32)).to(DEV)
    o = torch.empty_like(st.qd)
    lse = torch.zeros(H, dtype=torch.float32, device=DEV)
    c._decode_handler.forward(st.qd, o, c.kv_cache.buf_layer(0), idx, None, c.kv_cache.last_page_len,
                              c.kv_last_page_idx, lse=lse)
    tok = (logical[:, :, None] * ps + np.arange(ps)[None, None, :]).reshape(H, -1)
    last = np.arange((n_pages - 1) * ps, seq_len)
    tok = np.concatenate([tok, np.tile(last, (H, 1))], axis=1)
    want, want_lse = ref.sparse_attention(st.q[0], st.k, st.v, tok, return_lse=True)
    _assert_attn_close(o[0], want)
    torch.testing.assert_close(lse.cpu() * math.log(2.0), want_lse, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("L,ps,budget", [(300, 16, 64), (4096, 16, 256), (5000, 16, 1024), (9000, 32, 4096)])
def test_full_step_token_granular(dtype, L, ps, budget):
    """append -> estimate -> top-k -> sparse attention through the host API at page_size > 1."""
    _, K, U = _mods()
    H = 32
    st = State(L, H, ps, dtype, seed=L, budget_pages=budget // ps, fused=True)
    c = st.c
    assert c.need_estimate()
    r = ref.decode_step(st.q[0], st.k, st.v, budget)
    est = U.decode_estimate(st.q_code, c, 0)
    np.testing.assert_array_equal(est.cpu().numpy().astype(np.int32) if est.dtype == torch.int16
                                  else est.float().cpu().numpy().astype(np.int32), r["dist"])
    U.decode_topk(est, c)
    table = np.asarray(c.kv_cache.indicies)
    want_slots = table[r["sel"] // ps] * ps + r["sel"] % ps
    np.testing.assert_array_equal(c.topk_dindices_buffer.cpu().numpy(), want_slots)
    o = U.decode_sparse_attn(st.qd, c, 0, c.topk_dindices_buffer)
    _assert_attn_close(o[0], r["out"])
    # bytes are reproducible
    o2 = U.decode_sparse_attn(st.qd, c, 0, c.topk_dindices_buffer)
    assert torch.equal(o, o2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("L,ps,budget,H", [
    (70, 16, 8, 32), (300, 16, 64, 32), (700, 16, 128, 16), (700, 1, 128, 64), (2049, 16, 33, 8), (4096, 16, 256, 32), (5000, 1, 1024, 32),
    (9001, 32, 4096, 4), (8192, 16, 2048, 32), (32768, 16, 1024, 32), (70000, 16, 2048, 2), (131072, 16, 2048, 4),
    (150000, 16, 512, 1), (200000, 16, 1024, 8),      # 16-block clusters / 64 distances per thread
])
def test_fused_decode_step(dtype, L, ps, budget, H):
    """decode_step (append + estimate + select/attend in one call) against the oracle: codes and
    selected slots bit-exact, output within tolerance, and equal winners to the separate kernels."""
    _, K, U = _mods()
    st = State(L - 1, H, ps, dtype, seed=L + H, budget_pages=max(1, budget // ps), fused=True, max_seq_len=L + ps)
    # State holds L-1 tokens (its last one appended by a decode step); append one more with decode_step
    c = st.c
    c.end_forward()
    q = _randn((1, H, 128), 901 + L, dtype)
    k_new = _randn((1, H, 128), 902 + L, dtype)
    v_new = _randn((1, H, 128), 903 + L, dtype)
    c.prepare_hadamard(1)
    c.begin_forward(1)
    if ps > 1:
        assert c.inference_token_budget == min(max(1, budget // ps) * ps, L)
    bud = c.inference_token_budget
    o = U.decode_step(q.to(DEV), k_new.to(DEV), v_new.to(DEV), c, 0)
    k_all = torch.cat([st.k, k_new], 0)
    v_all = torch.cat([st.v, v_new], 0)
    r = ref.decode_step(q[0], k_all, v_all, bud)
    table = np.asarray(c.kv_cache.indicies)
    want_slots = table[r["sel"] // ps] * ps + r["sel"] % ps
    np.testing.assert_array_equal(c.topk_dindices_buffer.cpu().numpy(), want_slots)
    _assert_attn_close(o[0], r["out"])
    from adamas_b200 import _lib
    assert _lib.device_error(clear=False) == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rope", [None, (8.0, 1e4)])
@pytest.mark.parametrize("L,ps,budget,H", [(300, 16, 64, 32), (1500, 1, 128, 16), (2100, 16, 256, 64),
                                           (5000, 16, 1024, 32), (32768, 16, 1024, 32)])
def test_two_launch_step_equals_three_launch_step(dtype, rope, L, ps, budget, H):
    """decode_step with the append folded into the estimate launch writes the same bits as the
    three-launch step: rotated q and k, the new token's K/V rows and code, the query code, the
    distances, the selected slots and the output."""
    _, K, U = _mods()
    results = []
    for fused_append in (False, True):
        st = State(L - 1, H, ps, dtype, seed=L + 7, budget_pages=max(1, budget // ps), fused=True,
                   max_seq_len=L + ps)
        c = st.c
        c.end_forward()
        q = _randn((1, H, 128), 31 + L, dtype).to(DEV)
        k_new = _randn((1, H, 128), 32 + L, dtype).to(DEV)
        v_new = _randn((1, H, 128), 33 + L, dtype).to(DEV)
        c.prepare_hadamard(1)
        c.begin_forward(1)
        o = torch.full_like(q, float("nan"))
        q_code = torch.zeros(1, H, 16, dtype=dtype, device=DEV)
        n = c.hadamard_cache.seqlen - 1
        dist = c.distance_scratch(n)
        K.set_fused_append(fused_append)
        try:
            K.decode_step(q, k_new, v_new, o, q_code, c.kv_cache.buf_layer(0), c.kv_indices_with_last,
                          c.kv_cache.last_page_len, c.kv_last_page_idx, c.hadamard_cache.buf_layer(0),
                          c.hadamard_indices, c.hadamard_cache.last_page_len, c.inference_token_budget, dist,
                          c.hist_scratch, indices_out=c.topk_dindices_buffer, rope=rope)
            torch.cuda.synchronize()
        finally:
            K.set_fused_append(True)
        page = c.kv_cache.indicies[-1]
        kv_rows = c.kv_cache.buf_layer(0)[page, :, (L - 1) % ps].clone()
        code = c.hadamard_cache.buf_layer(0)[c.hadamard_cache.indicies[-1], 0, (L - 1) % ps].clone()
        results.append((q.clone(), k_new.clone(), kv_rows, code, q_code.clone(), dist[:, :n].clone(),
                        c.topk_dindices_buffer[:, : c.inference_token_budget - 1].clone(), o.clone()))
    names = ["q", "k", "kv rows", "key code", "query code", "distances", "selected slots", "output"]
    for name, a, b in zip(names, *results):
        a16 = a.view(torch.int16) if a.element_size() == 2 else a
        b16 = b.view(torch.int16) if b.element_size() == 2 else b
        assert torch.equal(a16, b16), name
    from adamas_b200 import _lib
    assert _lib.device_error(clear=False) == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("L,ps,H", [(500, 16, 32), (1300, 1, 16), (4100, 16, 64)])
def test_append_estimate_equals_separate_operators(dtype, L, ps, H):
    """append_estimate (one launch) leaves the same bits as append_kv_cache_decode_fused followed by
    estimate_attn_score: the new token's K/V rows and code, the query code and the integer distances."""
    _, K, U = _mods()
    results = []
    for one_launch in (False, True):
        st = State(L - 1, H, ps, dtype, seed=L + 3, fused=True, max_seq_len=L + ps)
        c = st.c
        c.end_forward()
        q = _randn((1, H, 128), 41 + L, dtype).to(DEV)
        k_new = _randn((1, H, 128), 42 + L, dtype).to(DEV)
        v_new = _randn((1, H, 128), 43 + L, dtype).to(DEV)
        c.prepare_hadamard(1)
        c.begin_forward(1)
        n = c.hadamard_cache.seqlen - 1
        dist = c.distance_scratch(n)
        dist.fill_(-1)
        q_code = torch.zeros(1, H, 16, dtype=dtype, device=DEV)
        if one_launch:
            K.append_estimate(q, k_new, v_new, q_code, c.kv_cache.buf_layer(0), c.kv_indices_with_last,
                              c.kv_cache.last_page_len, c.hadamard_cache.buf_layer(0), c.hadamard_indices,
                              c.hadamard_cache.last_page_len, dist)
        else:
            U.append_qkv_fused(q, k_new, v_new, c, 0, out=q_code)
            K.estimate_attn_score(q_code, dist, c.hadamard_cache.buf_layer(0), c.hadamard_indices, None,
                                  c.hadamard_cache.last_page_len, c.hadamard_last_page_idx, c.layout)
        torch.cuda.synchronize()
        kv_rows = c.kv_cache.buf_layer(0)[c.kv_cache.indicies[-1], :, (L - 1) % ps].clone()
        code = c.hadamard_cache.buf_layer(0)[c.hadamard_cache.indicies[-1], 0, (L - 1) % ps].clone()
        results.append((kv_rows, code, q_code.clone(), dist[:, :n].clone()))
    for name, a, b in zip(["kv rows", "key code", "query code", "distances"], *results):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), name
    # and the distances are the oracle's
    r = ref.decode_step(q[0].cpu(), torch.cat([st.k, k_new.cpu()], 0), torch.cat([st.v, v_new.cpu()], 0), 2)
    np.testing.assert_array_equal(results[1][3].cpu().numpy().astype(np.int32), r["dist"])


@pytest.mark.parametrize("blocks", [1, 2, 4])
@pytest.mark.parametrize("L,budget,H", [(32768, 1024, 8), (6000, 640, 32)])
def test_decode_step_with_smaller_clusters(blocks, L, budget, H):
    """set_max_cluster only changes how a head's row is split over thread blocks: same winners, same
    output (to tolerance) against the oracle for every bound."""
    _, K, U = _mods()
    ps = 16
    st = State(L - 1, H, ps, seed=L + blocks, budget_pages=budget // ps, fused=True, max_seq_len=L + ps)
    c = st.c
    c.end_forward()
    q, k_new, v_new = _randn((1, H, 128), 11 + L), _randn((1, H, 128), 12 + L), _randn((1, H, 128), 13 + L)
    c.prepare_hadamard(1)
    c.begin_forward(1)
    K.set_max_cluster(blocks)
    try:
        o = U.decode_step(q.to(DEV), k_new.to(DEV), v_new.to(DEV), c, 0)
        torch.cuda.synchronize()
    finally:
        K.set_max_cluster(8)
    r = ref.decode_step(q[0], torch.cat([st.k, k_new], 0), torch.cat([st.v, v_new], 0), c.inference_token_budget)
    table = np.asarray(c.kv_cache.indicies)
    np.testing.assert_array_equal(c.topk_dindices_buffer.cpu().numpy(), table[r["sel"] // ps] * ps + r["sel"] % ps)
    _assert_attn_close(o[0], r["out"])
    with pytest.raises(RuntimeError):
        K.set_max_cluster(3)


@pytest.mark.parametrize("ps", [1, 16])
def test_decode_step_dense_when_context_fits_budget(ps):
    """decode_step with a budget that covers the whole context (the reference's first two layers):
    append, then attention over every page."""
    _, K, U = _mods()
    L, H = 200, 32
    st = State(L - 1, H, ps, seed=12, budget_pages=1 << 20, fused=True, max_seq_len=L + ps)
    c = st.c
    c.end_forward()
    q, k_new, v_new = _randn((1, H, 128), 1), _randn((1, H, 128), 2), _randn((1, H, 128), 3)
    c.prepare_hadamard(1)
    c.begin_forward(1)
    assert not c.need_estimate()
    o = U.decode_step(q.to(DEV), k_new.to(DEV), v_new.to(DEV), c, 0)
    k_all, v_all = torch.cat([st.k, k_new], 0), torch.cat([st.v, v_new], 0)
    want = ref.sparse_attention(q[0], k_all, v_all, np.tile(np.arange(L), (H, 1)))
    _assert_attn_close(o[0], want)


def test_dense_layer_page_size_16():
    _, K, U = _mods()
    st = State(1000, 32, 16, seed=9, budget_pages=1 << 20)
    c = st.c
    assert not c.need_estimate()
    o = U.decode_sparse_attn(st.qd, c, 0, c.kv_indices_without_last)
    want = ref.sparse_attention(st.q[0], st.k, st.v, np.tile(np.arange(1000), (32, 1)))
    _assert_attn_close(o[0], want)


def test_config1_single_layer_decode_step():
    """batch 1, 32 heads, head_dim 128, KV length 4096, page size 16, budget 256, seed 0, N(0,1)
    fp16 inputs: codes and selected indices bit-exact, output vs attention restricted to the
    selection."""
    _, K, U = _mods()
    g = torch.Generator().manual_seed(0)
    L, H, ps, B = 4096, 32, 16, 256
    q = torch.randn(1, H, 128, generator=g, dtype=torch.float16)
    k = torch.randn(L, H, 128, generator=g, dtype=torch.float16)
    v = torch.randn(L, H, 128, generator=g, dtype=torch.float16)
    c = U.InferenceController(1, H, 128, ps, B // ps, L, torch.float16, DEV)
    c.prepare_hadamard(L - 1); c.begin_forward(L - 1)
    U.append_kvh(k[: L - 1].to(DEV), v[: L - 1].to(DEV), None, c, 0)
    c.end_forward()
    c.prepare_hadamard(1); c.begin_forward(1)
    q_code = U.append_qkv_fused(q.to(DEV), k[L - 1:].to(DEV), v[L - 1:].to(DEV), c, 0)
    r = ref.decode_step(q[0], k, v, B)
    np.testing.assert_array_equal(_codes_of(q_code)[0], r["q_code"])
    est = U.decode_estimate(q_code, c, 0)
    np.testing.assert_array_equal(est.float().cpu().numpy().astype(np.int32), r["dist"])
    U.decode_topk(est, c)
    table = np.asarray(c.kv_cache.indicies)
    np.testing.assert_array_equal(c.topk_dindices_buffer.cpu().numpy(), table[r["sel"] // ps] * ps + r["sel"] % ps)
    o = U.decode_sparse_attn(q.to(DEV), c, 0, c.topk_dindices_buffer)
    _assert_attn_close(o[0], r["out"])
    # ties at the cut were really exercised
    tau = np.take_along_axis(r["dist"], r["sel"], 1).max(1)
    assert ((r["dist"] == tau[:, None]).sum(1) > (np.take_along_axis(r["dist"], r["sel"], 1) == tau[:, None]).sum(1)).any()


def test_headline_size_properties_32k():
    """32K context, budget 1024, page size 16 (the benchmark's workload): full parity on the integer
    stages (the oracle takes a few seconds at this size) and the attention tolerance."""
    _, K, U = _mods()
    L, H, ps, B = 32768, 32, 16, 1024
    st = State(L, H, ps, seed=77, budget_pages=B // ps, fused=True, max_seq_len=L)
    c = st.c
    r = ref.decode_step(st.q[0], st.k, st.v, B)
    np.testing.assert_array_equal(st.cached_codes(), r["k_codes"])
    est = U.decode_estimate(st.q_code, c, 0)
    np.testing.assert_array_equal(est.float().cpu().numpy().astype(np.int32), r["dist"])
    U.decode_topk(est, c)
    table = np.asarray(c.kv_cache.indicies)
    np.testing.assert_array_equal(c.topk_dindices_buffer.cpu().numpy(), table[r["sel"] // ps] * ps + r["sel"] % ps)
    o = U.decode_sparse_attn(st.qd, c, 0, c.topk_dindices_buffer)
    _assert_attn_close(o[0], r["out"])


def test_no_kernel_gave_up_on_a_wait():
    """Runs after the estimate tests above: no bounded wait in a kernel has timed out."""
    from adamas_b200 import _lib
    st = State(5000, 32, 16, seed=5)
    _, _, U = _mods()
    U.decode_estimate(st.q_code, st.c, 0)
    assert _lib.device_error(clear=False) == 0


def test_merge_states_matches_oracle():
    _, K, _ = _mods()
    g = torch.Generator().manual_seed(3)
    P, H = 5, 32
    o_parts = torch.randn(P, H, 128, generator=g)
    lse = torch.randn(P, H, generator=g) * 3
    lse[2, 5] = -float("inf")                      # an empty shard
    want_o, want_lse = ref.merge_states(o_parts, lse * math.log(2.0))
    o = torch.zeros(H, 128, dtype=torch.float16, device=DEV)
    out_lse = torch.zeros(H, dtype=torch.float32, device=DEV)
    K.merge_states(o_parts.to(DEV), lse.to(DEV), o, out_lse)
    _assert_attn_close(o, want_o)
    torch.testing.assert_close(out_lse.cpu() * math.log(2.0), want_lse, rtol=1e-4, atol=1e-4)


def test_forward_before_begin_forward_raises():
    _, K, U = _mods()
    w = U.BatchDecodeWithPagedKVCacheWrapper("NHD")
    q = torch.zeros(1, 4, 128, dtype=torch.float16, device=DEV)
    kv = torch.zeros(4, 2, 1, 4, 128, dtype=torch.float16, device=DEV)
    idx = torch.zeros(4, 2, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):
        w.forward(q, torch.empty_like(q), kv, idx, None, 1, 3)
    with pytest.raises(KeyError):
        U.BatchDecodeWithPagedKVCacheWrapper("XYZ")
