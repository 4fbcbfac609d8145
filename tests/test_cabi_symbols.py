"""The C-ABI library loads without a GPU and exports every symbol the header
declares (no compute calls here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "pam_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(pamc?_[a-z0-9_]+)\s*\(", text))
    names.discard("pamc_available_fn")
    return sorted(names)


def test_header_declares_reference_abi():
    # the thirteen entry points of PagedAttentionCABI.swift:71-337
    ref = {"pam_create_context", "pam_destroy_context", "pam_last_error", "pam_create_cache", "pam_destroy_cache",
           "pam_reserve_sequence", "pam_append_tokens", "pam_free_sequence", "pam_available_blocks",
           "pam_sequence_length", "pam_append_kv", "pam_prefill", "pam_decode"}
    assert ref <= set(declared_symbols())


def test_library_exports_every_declared_symbol():
    from pagedattentionmetal_b200 import _cabi
    handle = ctypes.CDLL(_cabi.LIB_PATH)
    missing = [n for n in declared_symbols() if not hasattr(handle, n)]
    assert not missing, missing
    # and the Python binding covers the same set
    assert set(declared_symbols()) == set(_cabi.SIGNATURES)


def test_null_handles_follow_reference_conventions():
    from pagedattentionmetal_b200._cabi import lib
    assert lib.pam_available_blocks(None) == -1               # CABI.swift:183
    assert lib.pam_reserve_sequence(None, None, 1) == -1      # CABI.swift:146
    assert lib.pam_last_error(None) is None
    lib.pam_free_sequence(None, 3)                            # no-op, CABI.swift:178
    lib.pam_destroy_cache(None)
    lib.pam_destroy_context(None)
    assert lib.pamc_device_count() >= 0


def test_host_context_refuses_gpu_work():
    from pagedattentionmetal_b200._cabi import lib
    ctx = lib.pamc_create_host_context()
    assert ctx
    assert lib.pam_create_cache(ctx, 8, 16, 64, 2, 1) is None
    assert lib.pamc_last_error_code(ctx) == 1
    assert b"could not be initialized" in lib.pam_last_error(ctx)
    lib.pam_destroy_context(ctx)
