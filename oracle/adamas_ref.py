"""CPU oracle for the Adamas per-step decode path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU with numpy / torch, the arithmetic of the four
stages of the reference's decode hot path so that the CUDA kernels can be
checked against it.  Nothing in the shipped package imports it: only the test
suite, the smoke check and the CPU-baseline leg of the benchmark do.

What each function follows in the reference (paths relative to the reference
project root):

* Hadamard transform  -- the reference calls an external extension,
  ``faster_hadamard_transform.hadamard_transform`` (submodule
  kernels/3rdparty/applied-ai, directory empty, no pinned revision; call sites
  adamas/models/Adamas.py:120,150 and evaluation/adamas_attention.py:219-220).
  Its source is not available, so the transform itself is restated from the
  published definition: the Sylvester-ordered Walsh-Hadamard matrix
  H[i][j] = (-1)^popcount(i & j), scaled by 1/sqrt(D).  PARITY UNPINNED for
  this one stage (normalisation and element ordering cannot be checked against
  the absent library); it is checked against scipy.linalg.hadamard instead.
* bucketize / pack    -- kernels/include/decode/decode_page.cuh:380-398 and
  adamas/tests/test_estimate.py:12-24 (element 8w+i at bits [2i, 2i+1] of
  16-bit word w; bucket = (v > -10) + (v > 0) + (v > 10)).
* distance estimate   -- evaluation/adamas_attention.py:222 and
  adamas/tests/test_estimate.py:57-64 (L1 distance between 2-bit codes, newest
  token excluded); the shipped CUDA kernel's XOR-weighted variant
  (kernels/include/decode/decode_attn.cuh:192-193) is available as
  metric="xor".
* top-k               -- evaluation/adamas_attention.py:224-225 /
  adamas/tests/test_approx_attention.py:73-86 (k smallest distances).  The
  reference leaves the tie order open (torch.topk / raft radix select); the
  canonical rule here is "lower index wins", i.e. a stable sort by
  (distance, index).
* sparse attention    -- adamas/tests/test_approx_attention.py:37-98 and
  kernels/src/include/cpu_reference.h:161-292 (softmax in fp32 over the selected
  tokens plus the newest token, scale 1/sqrt(D)).

The restatement is pinned against outputs of the reference's own Python helper
functions (run on the CPU with the two absent extension modules stubbed): see
tests/golden/make_golden.py and tests/test_oracle_golden.py.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

THRESHOLDS = (-10.0, 0.0, 10.0)
HEAD_DIM = 128


# --------------------------------------------------------------------------
# stage 1: Hadamard transform, bucketize, pack
# --------------------------------------------------------------------------
def fwht(x: np.ndarray, scale: Optional[float] = None) -> np.ndarray:
    """Walsh-Hadamard transform (Sylvester order) over the last axis, in float32.

    Canonical arithmetic, shared bit for bit with the CUDA kernel: inputs are
    widened to float32; butterfly stages run with strides 1, 2, 4, ... D/2; in
    each stage the pair (a, b) = (x[i], x[i + stride]) with bit `stride` of i
    clear becomes (a + b, a - b); one final multiply by float32(scale).
    """
    x = np.ascontiguousarray(x, dtype=np.float32).copy()
    d = x.shape[-1]
    assert d & (d - 1) == 0, "last dimension must be a power of two"
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    lead = x.shape[:-1]
    stride = 1
    while stride < d:
        v = x.reshape(*lead, d // (2 * stride), 2, stride)
        a = v[..., 0, :].copy()
        b = v[..., 1, :].copy()
        v[..., 0, :] = a + b
        v[..., 1, :] = a - b
        stride *= 2
    return x * np.float32(scale)


def hadamard_transform(x: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """Drop-in for ``faster_hadamard_transform.hadamard_transform(x, inplace=False)``:
    the transform of the last dim, rounded (nearest-even) back to ``x.dtype``
    as the reference's extension returns its input dtype."""
    y = fwht(x.detach().cpu().to(torch.float32).numpy(), scale)
    return torch.from_numpy(y).to(x.dtype)


def bucketize(v: np.ndarray, thresholds: Sequence[float] = THRESHOLDS) -> np.ndarray:
    """bucket = #thresholds strictly below v (decode_page.cuh:385-392); equal to
    torch.bucketize(v, thresholds) with right=False."""
    v = np.asarray(v, dtype=np.float32)
    out = np.zeros(v.shape, dtype=np.uint8)
    for t in thresholds:
        out += (v > np.float32(t)).astype(np.uint8)
    return out


def pack_2bit(codes: np.ndarray) -> np.ndarray:
    """[..., D] codes in {0..3} -> [..., D/8] uint16; element 8w+i sits at bits
    [2i, 2i+1] of word w (decode_page.cuh:394, test_estimate.py:12-24)."""
    codes = np.asarray(codes)
    *lead, d = codes.shape
    assert d % 8 == 0
    c = codes.reshape(*lead, d // 8, 8).astype(np.uint16)
    out = np.zeros((*lead, d // 8), dtype=np.uint16)
    for i in range(8):
        out |= (c[..., i] & np.uint16(3)) << np.uint16(2 * i)
    return out


def unpack_2bit(packed: np.ndarray) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint16)
    *lead, w = packed.shape
    out = np.zeros((*lead, w, 8), dtype=np.uint8)
    for i in range(8):
        out[..., i] = ((packed >> np.uint16(2 * i)) & np.uint16(3)).astype(np.uint8)
    return out.reshape(*lead, w * 8)


def encode(x: torch.Tensor, scale: Optional[float] = None,
           thresholds: Sequence[float] = THRESHOLDS) -> np.ndarray:
    """x [..., D] (fp16 / bf16 / fp32) -> packed 2-bit codes [..., D/8] uint16.
    Transform in fp32, round to x.dtype, compare against the thresholds."""
    h = hadamard_transform(x, scale).to(torch.float32).numpy()
    return pack_2bit(bucketize(h, thresholds))


def rope(x: torch.Tensor, past_len: int, rope_scale: float = 1.0, rope_theta: float = 1e4) -> torch.Tensor:
    """Llama rotary embedding with linear position scaling of x [N, H, D]; token s has position
    past_len + s.  Same arithmetic as the HF module the reference's test compares against
    (adamas/tests/test_rope.py:17-31): fp32 inverse frequencies theta^(-2j/D), angle = position /
    rope_scale * inv_freq, out = x * cos + rotate_half(x) * sin; result in x.dtype."""
    n, h, d = x.shape
    inv_freq = 1.0 / (torch.tensor(rope_theta, dtype=torch.float32) ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    pos = torch.arange(past_len, past_len + n, dtype=torch.float32) / rope_scale
    freqs = torch.outer(pos, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    cos, sin = emb.cos()[:, None, :], emb.sin()[:, None, :]
    xf = x.to(torch.float32)
    rot = torch.cat((-xf[..., d // 2:], xf[..., : d // 2]), dim=-1)
    return (xf * cos + rot * sin).to(x.dtype)


def rope_table(x: torch.Tensor, past_len: int, inv_freq: torch.Tensor, mscale: float = 1.0) -> torch.Tensor:
    """Rotate-half RoPE of x [N, H, D] with one rotation frequency per dimension pair (inv_freq
    float32 [D/2], any position scaling folded in) and a factor on cos and sin: the form
    YaRN-scaled models use.  angle = position * inv_freq in float32; result in x.dtype."""
    n, h, d = x.shape
    pos = torch.arange(past_len, past_len + n, dtype=torch.float32)
    freqs = torch.outer(pos, inv_freq.to(torch.float32))
    emb = torch.cat((freqs, freqs), dim=-1)
    cos, sin = emb.cos()[:, None, :] * mscale, emb.sin()[:, None, :] * mscale
    xf = x.to(torch.float32)
    rot = torch.cat((-xf[..., d // 2:], xf[..., : d // 2]), dim=-1)
    return (xf * cos + rot * sin).to(x.dtype)


def yarn_parameters(factor: float, original_max_position: int, rope_theta: float = 1e4, dim: int = 128,
                    beta_fast: float = 32.0, beta_slow: float = 1.0):
    """The published YaRN rule (Peng et al., "YaRN: Efficient Context Window Extension of Large
    Language Models", sec. 3.2-3.4), restated: per dimension pair i with wavelength
    2*pi*theta^(2i/d), pairs that complete more than beta_fast rotations over the original
    context are left alone, pairs with fewer than beta_slow rotations are interpolated (divided by
    `factor`), a linear ramp over the pair index blends between the two; attention factor
    0.1 * ln(factor) + 1 multiplies cos and sin.  Returns (inv_freq float32 [dim/2], factor)."""
    i = np.arange(0, dim, 2, dtype=np.float64)
    pos_freqs = rope_theta ** (i / dim)

    def pair_index_for(rotations):
        return dim * math.log(original_max_position / (rotations * 2 * math.pi)) / (2 * math.log(rope_theta))

    low = max(math.floor(pair_index_for(beta_fast)), 0)
    high = min(math.ceil(pair_index_for(beta_slow)), dim - 1)
    if low == high:
        high += 0.001
    ramp = np.clip((np.arange(dim // 2, dtype=np.float64) - low) / (high - low), 0.0, 1.0)
    inv_freq = (1.0 / (factor * pos_freqs)) * ramp + (1.0 / pos_freqs) * (1.0 - ramp)
    return torch.from_numpy(inv_freq.astype(np.float32)), 0.1 * math.log(factor) + 1.0


# --------------------------------------------------------------------------
# stage 2: distance estimate
# --------------------------------------------------------------------------
def code_distance(q_packed: np.ndarray, k_packed: np.ndarray, metric: str = "l1") -> np.ndarray:
    """q_packed [H, W] uint16, k_packed [T, H, W] uint16 -> int32 [H, T].

    metric "l1": sum_d |qc[d] - kc[d]| (evaluation/adamas_attention.py:222).
    metric "xor": sum_d lowbit(x) + 2*highbit(x) with x = qc[d] ^ kc[d]
    (decode_attn.cuh:192-193).  They differ only on code pairs {1, 2}.
    """
    qc = unpack_2bit(q_packed).astype(np.int16)            # [H, D]
    kc = unpack_2bit(k_packed).astype(np.int16)            # [T, H, D]
    if metric == "l1":
        d = np.abs(kc - qc[None]).sum(-1, dtype=np.int32)
    elif metric == "xor":
        x = kc ^ qc[None]
        d = ((x & 1) + 2 * (x >> 1)).sum(-1, dtype=np.int32)
    else:
        raise ValueError(metric)
    return np.ascontiguousarray(d.T)                       # [H, T]


# --------------------------------------------------------------------------
# stage 3: top-k (k smallest, ties -> lower index)
# --------------------------------------------------------------------------
def sortable_key_fp16(v: np.ndarray) -> np.ndarray:
    """Order-preserving map fp16 -> uint16 used by the CUDA select: -0 is folded
    onto +0, negative values have all bits flipped, others the sign bit set."""
    b = np.asarray(v, dtype=np.float16).view(np.uint16).copy()
    b[b == 0x8000] = 0
    neg = (b & 0x8000) != 0
    return np.where(neg, ~b, b | np.uint16(0x8000)).astype(np.uint16)


def select_topk(values: np.ndarray, k: int) -> np.ndarray:
    """values [H, n] -> int64 [H, k]: positions of the k smallest values per row,
    ties resolved towards the lower position, returned in ascending position
    order (the order the CUDA kernel emits)."""
    values = np.asarray(values)
    if values.dtype == np.float16:
        keys = sortable_key_fp16(values).astype(np.int64)
    else:
        keys = values.astype(np.int64)
    order = np.argsort(keys, axis=-1, kind="stable")[:, :k]
    return np.sort(order, axis=-1)


# --------------------------------------------------------------------------
# stage 4: attention over the selected tokens
# --------------------------------------------------------------------------
def sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     idx: np.ndarray, return_lse: bool = False):
    """q [H, D], k/v [L, H, D], idx [H, m] token positions -> o [H, D] fp32.

    softmax(q . K_sel / sqrt(D)) @ V_sel in fp32 (test_approx_attention.py:56,
    93-96; cpu_reference.h:190-284).  lse is the natural-log sum of exponentials
    of the scaled logits."""
    qf = q.to(torch.float32)
    kf = k.to(torch.float32)
    vf = v.to(torch.float32)
    h, d = qf.shape
    idx_t = torch.as_tensor(np.asarray(idx), dtype=torch.long)
    heads = torch.arange(h).unsqueeze(1)
    ks = kf[idx_t, heads]                                   # [H, m, D]
    vs = vf[idx_t, heads]
    logits = torch.einsum("hd,hmd->hm", qf, ks) / math.sqrt(d)
    p = torch.softmax(logits, dim=-1)
    o = torch.einsum("hm,hmd->hd", p, vs)
    if return_lse:
        return o, torch.logsumexp(logits, dim=-1)
    return o


def merge_states(o_parts: torch.Tensor, lse_parts: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merge partial attention results over disjoint token sets.
    o_parts [P, H, D] fp32, lse_parts [P, H] (natural log) -> (o [H, D], lse [H]).
    Same rule as the reference's state merge (decode_attn.cuh:264-283)."""
    m = lse_parts.max(dim=0).values
    w = torch.exp(lse_parts - m)
    w = torch.where(torch.isfinite(lse_parts), w, torch.zeros_like(w))
    den = w.sum(0)
    o = (w.unsqueeze(-1) * o_parts).sum(0) / den.unsqueeze(-1)
    return o, m + torch.log(den)


# --------------------------------------------------------------------------
# whole decode step
# --------------------------------------------------------------------------
def repeat_kv(x: torch.Tensor, group: int) -> torch.Tensor:
    """Grouped-query attention stated as multi-head attention: x [L, H_kv, D] ->
    [L, H_kv * group, D] with query head r reading cache head r // group (the
    kv_head_idx = qo_head_idx / GROUP_SIZE of kernels/src/include/cpu_reference.h:83;
    the reference's operators themselves run group 1 only,
    kernels/include/decode/decode_handler.cuh:83)."""
    return x if group == 1 else x.repeat_interleave(group, dim=1)


def decode_step(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, budget: int,
                scale: Optional[float] = None, metric: str = "l1",
                semantics: str = "ops", thresholds: Sequence[float] = THRESHOLDS):
    """One layer's decode step on q [H, D], k/v [L, H, D] (token L-1 is the one
    being decoded).  Returns dict(q_code, k_codes, dist, idx, out).

    semantics "ops" (operator path, test_approx_attention.py:66-86): distances
    over tokens [0, L-1), the budget-1 smallest are selected and the newest
    token is always attended.  If L <= budget every token is attended.
    semantics "eval" (evaluation/adamas_attention.py:224-225): the min(budget, L)
    smallest over all L tokens, no forced inclusion.
    """
    l, h, d = k.shape
    q_code = encode(q, scale, thresholds)                   # [H, W]
    k_codes = encode(k, scale, thresholds)                  # [L, H, W]
    if semantics == "ops":
        if l <= budget:
            dist = None
            sel = np.tile(np.arange(l - 1, dtype=np.int64), (h, 1))
        else:
            dist = code_distance(q_code, k_codes[: l - 1], metric)
            sel = select_topk(dist, budget - 1)
        idx = np.concatenate([sel, np.full((h, 1), l - 1, dtype=np.int64)], axis=1)
    elif semantics == "eval":
        dist = code_distance(q_code, k_codes, metric)
        idx = sel = select_topk(dist, min(budget, l))
    else:
        raise ValueError(semantics)
    out = sparse_attention(q, k, v, idx)
    return dict(q_code=q_code, k_codes=k_codes, dist=dist, sel=sel, idx=idx, out=out)


def literal_reference_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, budget: int,
                             k_code: Optional[torch.Tensor] = None,
                             scale: Optional[float] = None):
    """The reference's PyTorch decode path written with the same torch calls it
    uses (evaluation/adamas_attention.py:214-241): bucketize -> pairwise_distance
    (p=1) -> topk(largest=False) -> scatter mask -> fp32 softmax -> @ V.

    q [H, D], k/v [H, L, D] fp32.  If `k_code` (int32 [H, L, D]) is given the key
    codes are taken as cached; otherwise all keys are re-transformed and
    re-bucketized, which is what the reference does every step.  Used as the
    timed CPU baseline and for multiset cross-checks; its tie order is torch's.
    """
    h, l, d = k.shape
    thresholds = torch.tensor([-10, 0, 10])
    attn = torch.matmul(q.unsqueeze(1), k.transpose(1, 2)) / math.sqrt(d)      # [H, 1, L]
    if k_code is None:
        kh = torch.from_numpy(fwht(k.numpy(), scale))
        k_code = torch.bucketize(kh, thresholds, out_int32=True)
    qh = torch.from_numpy(fwht(q.numpy(), scale))
    q_code = torch.bucketize(qh, thresholds, out_int32=True)
    dist = torch.nn.functional.pairwise_distance(q_code.unsqueeze(1), k_code, p=1).unsqueeze(1)
    kk = min(budget, l)
    _, topk_idx = dist.topk(k=kk, dim=-1, largest=False)
    mask = torch.zeros_like(attn, dtype=torch.bool)
    mask.scatter_(-1, topk_idx, True)
    attn = attn.masked_fill(~mask, torch.finfo(attn.dtype).min)
    p = torch.softmax(attn, dim=-1, dtype=torch.float32)
    out = torch.matmul(p, v).squeeze(1)
    return out, topk_idx.squeeze(1), dist.squeeze(1)


# --------------------------------------------------------------------------
# paged layout helpers (adamas/utils/kv_cache.py:21-24, decode_page.cuh:135-180)
# --------------------------------------------------------------------------
def build_paged_caches(k: torch.Tensor, v: torch.Tensor, codes: np.ndarray, page_size: int,
                       capacity_pages: int, seed: int = 0):
    """Scatter k/v [L, H, D] and packed codes [L, H, W] into NHD paged buffers with a
    random physical page permutation.  Returns (kv_buf [P,2,ps,H,D], code_buf
    [P,1,ps,H,W] int16, kv_table [n_pages] int32, code_table [n_pages] int32)."""
    l, h, d = k.shape
    w = codes.shape[-1]
    n_pages = (l + page_size - 1) // page_size
    assert capacity_pages >= n_pages
    rng = np.random.default_rng(seed)
    kv_table = rng.permutation(capacity_pages)[:n_pages].astype(np.int32)
    code_table = rng.permutation(capacity_pages)[:n_pages].astype(np.int32)
    kv_buf = torch.zeros(capacity_pages, 2, page_size, h, d, dtype=k.dtype)
    code_buf = np.zeros((capacity_pages, 1, page_size, h, w), dtype=np.uint16)
    for t in range(l):
        p, e = divmod(t, page_size)
        kv_buf[kv_table[p], 0, e] = k[t]
        kv_buf[kv_table[p], 1, e] = v[t]
        code_buf[code_table[p], 0, e] = codes[t]
    return kv_buf, torch.from_numpy(code_buf.view(np.int16)), torch.from_numpy(kv_table), torch.from_numpy(code_table)
