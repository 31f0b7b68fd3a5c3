"""CPU-only checks of the host side: the C-ABI library loads and exports what the header
declares, argument validation answers without a GPU, and the InferenceController mirror walks
through the same states as the reference's (trace recorded by tests/golden/make_golden.py)."""
import ctypes
import json
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from adamas_b200 import _lib
    header = open(os.path.join(ROOT, "include", "adamas_b200.h")).read()
    declared = set(re.findall(r"\b(adamas_[a-z0-9_]+)\s*\(", header))
    declared -= {"adamas_stream_t", "adamas_decode_handler_t"}
    assert len(declared) >= 15
    for name in sorted(declared):
        assert hasattr(_lib.lib, name), f"{name} declared in the header but not exported"
    assert set(_lib.SIGNATURES) | {"adamas_abi_version", "adamas_last_error"} == declared
    assert _lib.lib.adamas_abi_version() == _lib.ABI_VERSION == 4


def test_ctypes_signatures_match_the_header():
    """Every declaration's parameter list against the ctypes table: count, and pointer / integer /
    float kind of each parameter."""
    from adamas_b200 import _lib
    header = open(os.path.join(ROOT, "include", "adamas_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    decls = dict(re.findall(r"\bint\s+(adamas_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", header))
    assert set(decls) >= set(_lib.SIGNATURES)

    def kind(param: str) -> str:
        param = param.strip()
        if "*" in param or param.startswith("adamas_stream_t"):
            return "p"
        if param.startswith("float"):
            return "f"
        if param.startswith("int64_t"):
            return "l"
        assert param.startswith(("int ", "unsigned")), param
        return "i"

    ctype_kind = {ctypes.c_int: "i", ctypes.c_int64: "l", ctypes.c_float: "f", ctypes.c_void_p: "p"}
    for name, args in _lib.SIGNATURES.items():
        params = [p for p in decls[name].split(",") if p.strip() and p.strip() != "void"]
        got = "".join(ctype_kind.get(a, "p") for a in args)
        want = "".join(kind(p) for p in params)
        assert got == want, f"{name}: ctypes {got} vs header {want}"


def test_argument_validation_without_gpu():
    from adamas_b200 import _lib
    lib = _lib.lib
    null = ctypes.c_void_p(0)
    rc = lib.adamas_hadamard_transform(null, null, 4, 64, 1.0, 0, null)
    assert rc == _lib.ERR_INVALID and "head_dim" in _lib.last_error()
    rc = lib.adamas_topk(null, 0, 10, 10, null, 0, 1, 2, 11, null, null, 11, null)
    assert rc == _lib.ERR_INVALID
    h = ctypes.c_void_p()
    assert lib.adamas_decode_handler_create(ctypes.byref(h)) == 0
    rc = lib.adamas_decode_forward(h, null, null, null, null, null, 0, 0, 1, 0, 1, 1, 1.0, null)
    assert rc == _lib.ERR_STATE and "begin_forward" in _lib.last_error()
    assert lib.adamas_decode_handler_destroy(h) == 0
    with pytest.raises(RuntimeError):
        _lib.check(rc, "decode")
    assert lib.adamas_set_max_cluster(3) == _lib.ERR_INVALID and "power of two" in _lib.last_error()
    assert lib.adamas_set_max_cluster(16) == _lib.ERR_INVALID
    assert lib.adamas_set_max_cluster(8) == 0
    assert lib.adamas_set_estimate_blocks_per_sm(3) == _lib.ERR_INVALID and "1 or 2" in _lib.last_error()
    assert lib.adamas_set_estimate_blocks_per_sm(2) == 0
    assert lib.adamas_set_fused_append(1) == 0


def test_ops_reject_cpu_tensors():
    import adamas_b200
    x = torch.zeros(2, 4, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        adamas_b200.hadamard_transform(x)


def _snap(c):
    opt = lambda t: None if t is None else t.tolist()
    return dict(
        kv_pages=list(c.kv_cache.indicies), code_pages=list(c.hadamard_cache.indicies),
        kv_seqlen=c.kv_cache.seqlen, code_seqlen=c.hadamard_cache.seqlen,
        kv_last_page_len=c.kv_cache.last_page_len, code_last_page_len=c.hadamard_cache.last_page_len,
        kv_last_page_idx=int(c.kv_last_page_idx), code_last_page_idx=int(c.hadamard_last_page_idx),
        kv_indptr_for_append=opt(c.kv_indptr_for_append),
        hadamard_indptr_for_append=opt(c.hadamard_indptr_for_append),
        kv_indices_with_last=opt(c.kv_indices_with_last),
        hadamard_indices=opt(c.hadamard_indices),
        kv_indices_without_last=opt(c.kv_indices_without_last),
        inference_page_budget=c.inference_page_budget,
        kv_indptr_for_approx_decode=opt(c.kv_indptr_for_approx_decode),
        need_estimate=bool(c.need_estimate()),
        topk_shapes=None if c.topk_dout_buffer is None else [list(c.topk_dout_buffer.shape),
                                                              list(c.topk_dindices_buffer.shape),
                                                              list(c.topk_buf.shape)],
    )


def test_controller_follows_reference_trace():
    from adamas_b200.utils import InferenceController
    trace = json.load(open(os.path.join(ROOT, "tests", "golden", "ref_controller_trace.json")))
    for rec in trace:
        c = InferenceController(2, 4, 128, rec["page_size"], rec["budget"], 256, torch.float16, "cpu")
        states = []
        c.prepare_hadamard(rec["prefill"])
        c.begin_forward(rec["prefill"])
        states.append(_snap(c))
        c.end_forward()
        for _ in range(rec["steps"]):
            c.prepare_hadamard(1)
            c.begin_forward(1)
            states.append(_snap(c))
            c.end_forward()
        assert len(states) == len(rec["states"])
        for got, want in zip(states, rec["states"]):
            assert got == want


def test_controller_page_size_16_counts_tokens():
    from adamas_b200.utils import InferenceController
    c = InferenceController(1, 2, 128, 16, 4, 512, torch.float16, "cpu")   # budget 4 pages = 64 tokens
    c.prepare_hadamard(100)
    c.begin_forward(100)
    assert c.kv_cache.seqlen == c.hadamard_cache.seqlen == 100
    assert len(c.kv_cache.indicies) == len(c.hadamard_cache.indicies) == 7
    c.end_forward()
    c.prepare_hadamard(1)
    c.begin_forward(1)
    assert c.inference_token_budget == 64 and c.need_estimate()
    assert tuple(c.topk_dindices_buffer.shape) == (2, 63)
    assert c.kv_cache.last_page_len == 5 and c.kv_last_page_idx == 6
    c.end_forward()
    c.clean_states()
    assert c.kv_cache.seqlen == 0 and c.kv_cache.pool.num_free_blocks == 32


def test_kv_pool_reuses_lowest_page_first():
    from adamas_b200.utils import KvCache
    kc = KvCache(1, 1, 8, 8, 2, 1, torch.float16, "cpu")
    assert kc.append_seq(5) == 3 and kc.indicies == [0, 1, 2] and kc.last_page_len == 1
    assert kc.append_seq(1) == 0 and kc.last_page_len == 2
    kc.release()
    assert kc.append_seq(1) == 1 and kc.indicies == [0]
    assert kc.append_seq(0) == 0
    with pytest.raises(RuntimeError):
        kc.append_seq(100)


def test_header_is_plain_c_and_a_c_program_links(tmp_path):
    """include/adamas_b200.h compiles as C99 and a C program linked against the library sees the same
    ABI version: the boundary needs neither C++ nor Python."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    from adamas_b200 import _lib
    src = tmp_path / "abi_check.c"
    src.write_text('#include "adamas_b200.h"\n'
                   "int main(void) {\n"
                   "  adamas_seq_desc_t d = {0, 0, 0, 0};\n"
                   "  (void)d;\n"
                   "  return adamas_abi_version() == ADAMAS_ABI_VERSION ? 0 : 1;\n"
                   "}\n")
    exe = tmp_path / "abi_check"
    lib_dir = os.path.dirname(_lib.LIB_PATH)
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(ROOT, "include"),
                    str(src), "-o", str(exe), "-L", lib_dir, "-ladamas_b200", f"-Wl,-rpath,{lib_dir}"], check=True)
    assert subprocess.run([str(exe)]).returncode == 0
