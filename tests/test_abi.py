"""CPU checks of the drop-in boundary: the shared library loads without a GPU, exports every
symbol include/sgattn.h declares, lists the registry the reference's callers expect, and refuses
to pretend when there is no device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def sg():
    from super_gemma_b200 import build

    build.build()
    import super_gemma_b200 as sg

    return sg


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "sgattn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sgb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(sg):
    L = ctypes.CDLL(sg.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/sgattn.h but not exported"
    assert sorted(sg.ABI) == names, "the Python mirror binds exactly the declared ABI"


def test_registry_keeps_the_reference_contract(sg):
    """Names, binding counts and push sizes of the reference's variants
    (crates/sg-gpu/build.rs:253-437, 2207-2287): a caller written against sg-gpu binds them unchanged."""
    reg = {k.name: k for k in sg.kernels()}
    ref = {
        "attn_decode_sliding": (5, 8), "attn_decode_global": (5, 8), "attn_decode_global_q8k": (6, 8),
        "attn_reduce_d256": (2, 4), "attn_reduce_d512": (2, 4), "attn_prefill_sliding": (5, 4),
        "attn_prefill_sliding_ring": (7, 4), "attn_prefill_global": (5, 4), "kv_append_sliding": (3, 0),
        "kv_append_global": (3, 0), "kv_append_global_q8": (4, 0), "kv_quant_q8": (3, 0), "kv_dequant_q8": (3, 0),
        # the tiled global-prefill variants (build.rs:2207-2287); sg-model dispatches ..._flash_sp_iq (graph.rs:1210-1223)
        "attn_prefill_global_flash": (5, 4), "attn_prefill_global_flash_sp": (5, 4), "attn_prefill_global_flash_sp_q8": (7, 4),
        "attn_prefill_global_flash_sp_iq": (7, 4),
    }
    for name, (bindings, push) in ref.items():
        assert name in reg, name
        assert (reg[name].bindings, reg[name].push_bytes) == (bindings, push), name
    for name in ("attn_decode_paged_q8kv_d128", "attn_verify_paged_q8kv_d128", "attn_reduce_f32_d128", "attn_combine_ranks_d128",
                 "attn_prefill_flash_f16_d128", "attn_prefill_sliding_ring_flash_d128", "attn_prefill_paged_q8kv_flash_d128",
                 "attn_verify_sliding_ring_d128", "kv_append_paged_q8_d128", "kv_dequant_paged_q8_d128"):
        assert name in reg, name
    assert sg.kernel_blob("no_such_kernel") is None
    for k in reg.values():
        assert k.signature and all(w > 0 for w in k.workgroup)


def test_no_device_is_an_error_not_a_fallback(sg):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(sg.NoDevice):
        sg.GpuContext(0)


def test_product_does_not_reach_into_the_oracle():
    """The shipped package and library must not import, link or run anything under oracle/."""
    pkg = os.path.join(ROOT, "super_gemma_b200")
    for dirpath, _, files in os.walk(pkg):
        if os.path.basename(dirpath) == "build":
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "sg_oracle" not in text and "libsgoracle" not in text and "from oracle" not in text, f
