"""The kernel libraries as built: every C function the Python side declares is exported.
Needs the CUDA compiler but no GPU (nvcc cross-compiles; the libraries load without a device)."""

from __future__ import annotations

import ctypes
import shutil

import pytest


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="no CUDA compiler")
def test_every_declared_entry_point_is_exported():
    from inference_engine_b200.kernels.build import build_attention, build_core
    from inference_engine_b200.kernels.cuda_ops import CudaOps

    core = ctypes.CDLL(str(build_core()))
    fake = type("Declared", (), {"lib": core})()
    CudaOps._declare(fake)  # looks every core entry point up by name
    assert hasattr(core, "ie_set_pdl")
    attention = ctypes.CDLL(str(build_attention(64)))
    for name in ("ie_set_pdl", "ie_set_decode_pair", "ie_attention_decode", "ie_attention_decode_balanced", "ie_attention_prefill",
                 "ie_attention_prefill_tc5", "ie_attention_prefill_tc5_ok", "ie_attention_prefill_rows",
                 "ie_attention_decode_scratch_floats", "ie_attention_decode_balanced_scratch_floats",
                 "ie_attention_decode_balanced_max_seqs", "ie_attention_prefill_tc5_scratch_floats",
                 "ie_attention_decode_static", "ie_attention_decode_static_capacity_floats"):
        assert hasattr(attention, name), name


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="no CUDA compiler")
def test_part_libraries_export_what_is_declared():
    """The libraries that single mixers and feed-forwards need (built on first use) and the
    tensor-core sigmoid attention, built for one pair of sizes."""
    from inference_engine_b200.kernels.build import PART_LIBRARIES, build_part_library, build_sigmoid_attention
    from inference_engine_b200.kernels.cuda_ops import CudaOps

    assert set(CudaOps._PART_SIGNATURES) == set(PART_LIBRARIES)
    for name, functions in CudaOps._PART_SIGNATURES.items():
        lib = ctypes.CDLL(str(build_part_library(name)))
        for fn in functions:
            assert hasattr(lib, fn), (name, fn)
    lib = ctypes.CDLL(str(build_sigmoid_attention(32, 48)))
    d, dv = ctypes.c_int(), ctypes.c_int()
    lib.ie_sigmoid_attention_dims(ctypes.byref(d), ctypes.byref(dv))
    assert (d.value, dv.value) == (32, 48) and hasattr(lib, "ie_sigmoid_attention_mma")
