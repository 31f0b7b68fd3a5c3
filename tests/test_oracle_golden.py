"""The CPU oracle against fixtures produced by the reference's own Python code
(tests/golden/make_golden.py) and against independent restatements."""
import os

import numpy as np
import pytest
import scipy.linalg
import torch

from oracle import adamas_ref as ref

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_python_path.npz"))
CASES = sorted({k.split(".")[0] for k in GOLD.files})


def _case(name):
    g = {k.split(".", 1)[1]: GOLD[k] for k in GOLD.files if k.startswith(name + ".")}
    f16 = lambda a: torch.from_numpy(a.copy()).view(torch.float16)
    scale = None if g["scale"] < 0 else float(g["scale"])
    return g, f16(g["q"]), f16(g["k"]), f16(g["v"]), int(g["budget"]), scale


def test_fwht_matches_sylvester_matrix():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 128)).astype(np.float32)
    want = x.astype(np.float64) @ scipy.linalg.hadamard(128).astype(np.float64) / np.sqrt(128.0)
    got = ref.fwht(x)
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-5)
    # unnormalised, small integers: exact
    xi = rng.integers(-8, 9, size=(3, 128)).astype(np.float32)
    np.testing.assert_array_equal(ref.fwht(xi, 1.0), xi @ scipy.linalg.hadamard(128).astype(np.float32))
    # involution: H(H(x)) = x with the orthonormal scale
    np.testing.assert_allclose(ref.fwht(ref.fwht(x)), x, atol=1e-5)


def test_bucketize_matches_torch():
    v = torch.tensor([-11.0, -10.0, -9.99, -0.0, 0.0, 1e-7, 9.99, 10.0, 10.01, 65504.0, -65504.0])
    want = torch.bucketize(v, torch.tensor([-10.0, 0.0, 10.0]), out_int32=True).numpy()
    np.testing.assert_array_equal(ref.bucketize(v.numpy()), want)


def test_pack_roundtrip():
    rng = np.random.default_rng(1)
    c = rng.integers(0, 4, size=(7, 3, 128)).astype(np.uint8)
    p = ref.pack_2bit(c)
    assert p.shape == (7, 3, 16) and p.dtype == np.uint16
    np.testing.assert_array_equal(ref.unpack_2bit(p), c)
    assert ref.pack_2bit(np.array([[1, 0, 0, 0, 0, 0, 0, 3]]))[0, 0] == 1 | (3 << 14)


@pytest.mark.parametrize("name", CASES)
def test_codes_bit_exact(name):
    g, q, k, v, budget, scale = _case(name)
    got = ref.encode(q, scale)
    np.testing.assert_array_equal(got, g["q_code"].view(np.uint16))


@pytest.mark.parametrize("name", CASES)
def test_distances_bit_exact(name):
    g, q, k, v, budget, scale = _case(name)
    qc = ref.encode(q[0], scale)
    kc = ref.encode(k, scale)
    dist = ref.code_distance(qc, kc[:-1], "l1")
    want = torch.from_numpy(g["est"].copy()).view(torch.float16).to(torch.float32).numpy()
    np.testing.assert_array_equal(dist.astype(np.float32), want)
    if name.startswith("wide"):
        codes = ref.unpack_2bit(kc)
        assert set(np.unique(codes)) == {0, 1, 2, 3}
        assert (ref.code_distance(qc, kc[:-1], "xor") != dist).any()


@pytest.mark.parametrize("name", CASES)
def test_topk_same_multiset_as_reference(name):
    g, q, k, v, budget, scale = _case(name)
    l = k.shape[0]
    if l <= budget:
        pytest.skip("dense case")
    dist = ref.code_distance(ref.encode(q[0], scale), ref.encode(k, scale)[:-1], "l1")
    mine = ref.select_topk(dist, budget - 1)
    theirs = g["topk"].astype(np.int64)
    assert mine.shape == theirs.shape
    for h in range(dist.shape[0]):
        dm = np.sort(dist[h, mine[h]])
        dt = np.sort(dist[h, theirs[h]])
        np.testing.assert_array_equal(dm, dt)            # same multiset of distances
        tau = dm[-1]
        strict_m = set(mine[h][dist[h, mine[h]] < tau].tolist())
        strict_t = set(theirs[h][dist[h, theirs[h]] < tau].tolist())
        assert strict_m == strict_t                       # identical below the cut
        ties = np.nonzero(dist[h] == tau)[0]
        need = budget - 1 - len(strict_m)
        assert set(mine[h][dist[h, mine[h]] == tau].tolist()) == set(ties[:need].tolist())


@pytest.mark.parametrize("name", CASES)
def test_attention_matches_reference(name):
    g, q, k, v, budget, scale = _case(name)
    l, h, d = k.shape
    idx = np.concatenate([g["topk"].astype(np.int64), np.full((h, 1), l - 1)], axis=1)
    o = ref.sparse_attention(q[0], k, v, idx)
    want = torch.from_numpy(g["o"].copy()).view(torch.float16).to(torch.float32)[0]
    # the reference's own tolerance for fp16 (adamas/tests/test_approx_attention.py:30-35)
    torch.testing.assert_close(o, want, rtol=5e-3, atol=5e-3)


def test_decode_step_semantics_and_merge():
    g = torch.Generator().manual_seed(7)
    q = torch.randn(4, 128, generator=g).to(torch.float16)
    k = torch.randn(300, 4, 128, generator=g).to(torch.float16)
    v = torch.randn(300, 4, 128, generator=g).to(torch.float16)
    r = ref.decode_step(q, k, v, 33)
    assert r["idx"].shape == (4, 33) and (r["idx"][:, -1] == 299).all()
    assert (np.diff(r["sel"], axis=1) > 0).all()
    # splitting the selected set in two and merging gives the same output
    o1, l1 = ref.sparse_attention(q, k, v, r["idx"][:, :10], return_lse=True)
    o2, l2 = ref.sparse_attention(q, k, v, r["idx"][:, 10:], return_lse=True)
    om, _ = ref.merge_states(torch.stack([o1, o2]), torch.stack([l1, l2]))
    torch.testing.assert_close(om, r["out"], rtol=1e-5, atol=1e-6)
    # dense fallback when the context fits in the budget
    r2 = ref.decode_step(q, k[:20], v[:20], 33)
    assert r2["idx"].shape == (4, 20) and r2["dist"] is None
    # literal reference expressions: same multiset of distances at the cut ("eval" semantics)
    kf = k.to(torch.float32).transpose(0, 1).contiguous()
    vf = v.to(torch.float32).transpose(0, 1).contiguous()
    out_lit, idx_lit, dist_lit = ref.literal_reference_decode(q.to(torch.float32), kf, vf, 33)
    re = ref.decode_step(q, k, v, 33, semantics="eval")
    np.testing.assert_array_equal(np.round(dist_lit.numpy()).astype(np.int32), re["dist"])
    for h in range(4):
        np.testing.assert_array_equal(np.sort(re["dist"][h, re["idx"][h]]),
                                      np.sort(re["dist"][h, idx_lit[h].numpy()]))


def test_topk_edge_cases():
    d = np.array([[5, 5, 5, 5, 5, 5]], dtype=np.int32)
    np.testing.assert_array_equal(ref.select_topk(d, 3), [[0, 1, 2]])
    np.testing.assert_array_equal(ref.select_topk(d, 6), [[0, 1, 2, 3, 4, 5]])
    d = np.array([[9, 1, 9, 1, 0, 9]], dtype=np.int32)
    np.testing.assert_array_equal(ref.select_topk(d, 1), [[4]])
    np.testing.assert_array_equal(ref.select_topk(d, 4), [[0, 1, 3, 4]])
    f = np.array([[0.5, -0.0, 0.0, -1.0, 2.0]], dtype=np.float16)
    np.testing.assert_array_equal(ref.select_topk(f, 2), [[1, 3]])


def test_rope_matches_hf_apply_rotary_pos_emb():
    """The rotate-half structure against transformers' own helper (the reference's test_rope.py uses it)."""
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
    g = torch.Generator().manual_seed(0)
    q = torch.randn(7, 4, 128, generator=g)
    k = torch.randn(7, 4, 128, generator=g)
    past, theta = 13, 1e4
    inv_freq = 1.0 / (theta ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
    pos = torch.arange(past, past + 7, dtype=torch.float32)
    emb = torch.cat((torch.outer(pos, inv_freq),) * 2, dim=-1)
    cos, sin = emb.cos()[None], emb.sin()[None]                    # [1, N, D]
    qh, kh = apply_rotary_pos_emb(q.transpose(0, 1)[None], k.transpose(0, 1)[None], cos, sin)
    torch.testing.assert_close(ref.rope(q, past), qh[0].transpose(0, 1), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(ref.rope(k, past), kh[0].transpose(0, 1), rtol=1e-5, atol=1e-5)
    # position scaling divides the position
    torch.testing.assert_close(ref.rope(q[:1], 16, rope_scale=8.0), ref.rope(q[:1], 2), rtol=1e-5, atol=1e-5)


def test_yarn_parameters_match_transformers_and_table_rope_reduces_to_linear():
    """The YaRN restatement against transformers' own rope initialiser, and rope_table against
    rope for the table that encodes linear scaling."""
    from transformers import LlamaConfig
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    for factor, orig in [(32.0, 4096), (4.0, 8192), (16.0, 2048)]:
        cfg = LlamaConfig(hidden_size=4096, num_attention_heads=32, max_position_embeddings=int(orig * factor),
                          rope_theta=1e4, rope_scaling={"rope_type": "yarn", "factor": factor,
                                                        "original_max_position_embeddings": orig})
        inv, att = ROPE_INIT_FUNCTIONS["yarn"](cfg, "cpu")
        mine, mscale = ref.yarn_parameters(factor, orig)
        torch.testing.assert_close(mine, inv, rtol=1e-6, atol=1e-9)
        assert abs(mscale - att) < 1e-12
        from adamas_b200.rope import yarn_inv_freq
        pkg, pkg_scale = yarn_inv_freq(factor, orig)
        torch.testing.assert_close(pkg, inv, rtol=1e-6, atol=1e-9)
        assert abs(pkg_scale - att) < 1e-12
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, 3, 128, generator=g)
    from adamas_b200.rope import linear_inv_freq
    torch.testing.assert_close(ref.rope_table(x, 1000, linear_inv_freq(8.0)), ref.rope(x, 1000, 8.0), rtol=1e-6, atol=1e-6)
