"""CPU checks of the boundary: the library builds for sm_100a without a GPU, loads, exports every
symbol the header declares, and the Python layer validates arguments like the reference."""

from __future__ import annotations

import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from flashloop_b200 import _native, build_kernels

    build_kernels.build()
    return _native.load()


def test_header_and_library_agree(lib):
    from flashloop_b200 import _native

    header = (ROOT / "include" / "flashloop_b200.h").read_text()
    declared = set(re.findall(r"\b(fl_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_native.SIGNATURES), declared ^ set(_native.SIGNATURES)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.fl_version() == 1
    # every declaration cites the reference interface it replaces (or says it has none)
    for block in re.findall(r"/\*((?:(?!\*/).)*)\*/\s*(?:int|size_t|const char\*)\s+fl_", header, flags=re.S):
        assert re.search(r"flashloop/|kivi_outer_gemv|reference", block), block[:80]


def test_workspace_size_is_monotonic(lib):
    small = lib.fl_reader_workspace_bytes(16, 4096)
    large = lib.fl_reader_workspace_bytes(512, 32768)
    assert 0 < small <= large
    assert lib.fl_reader_workspace_bytes(0, 100) == 0


def test_argument_errors_without_a_gpu(lib):
    from flashloop_b200 import _native

    assert lib.fl_pack_k_rows(None, 0, 1, 64, 4, None, None, None, None) == -1
    assert b"null pointer" in lib.fl_last_error()
    assert lib.fl_select_decode_keys(None, 0, 1, 1, 8, None, 0.1, 0, None, None, 64, None, None, None, None) == -1
    with pytest.raises(RuntimeError):
        _native.check(-1, "probe")


def test_python_layer_rejects_cpu_tensors_and_bad_shapes():
    from flashloop_b200 import kivi_backend, packing, selection

    with pytest.raises(RuntimeError):  # no CPU fallback
        packing.pack_k_per_channel(torch.zeros(1, 1, 64, 128, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        packing.pack_v_per_token(torch.zeros(1, 64, 128))
    with pytest.raises(ValueError):
        kivi_backend.pack_kivi_k_per_channel(torch.zeros(1, 1, 64, 64))
    with pytest.raises(ValueError):
        selection.select_decode_keys(torch.ones(1, 1, 2, 8), fraction=0.1)
    with pytest.raises(ValueError):
        selection.select_decode_keys(torch.ones(1, 1, 1, 8), fraction=0.0)
    with pytest.raises(TypeError):
        kivi_backend.KiviPacked4Bit(payload=torch.zeros(1, 1, 8, 128), minimum=torch.zeros(1, 1, 1, 128).half(),
                                    scale=torch.zeros(1, 1, 1, 128).half(), original_shape=(1, 1, 64, 128),
                                    original_dtype=torch.bfloat16, axis="per_channel", group_size=64)


def test_select_prefill_tokens_matches_reference_vectors(golden):
    from flashloop_b200 import selection

    m3 = selection.select_prefill_tokens(torch.from_numpy(golden["retain.score3"]), fraction=0.25)
    assert torch.equal(m3, torch.from_numpy(golden["retain.mask3"]))
    m4 = selection.select_prefill_tokens(torch.from_numpy(golden["retain.score4"]), fraction=0.10, eligible=m3)
    assert torch.equal(m4, torch.from_numpy(golden["retain.mask4"]))
    with pytest.raises(ValueError):
        selection.select_prefill_tokens(torch.zeros(1, 4), fraction=0.5,
                                        eligible=torch.tensor([[True, True, True, False]]))
