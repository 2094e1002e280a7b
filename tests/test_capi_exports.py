"""CPU-only checks of the boundary: the shared library loads without a GPU, exports every symbol
that include/fgattn_b200.h declares, and rejects bad arguments before touching a device."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "fgattn_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fgattn_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from fgattn_tk_cuda_b200 import _build, capi
    _build.build_library()
    lib = capi.lib()
    names = declared_symbols()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), n
        assert n in capi.PROTOTYPES, f"{n} has no ctypes prototype"
    assert set(capi.PROTOTYPES) == set(names)


def test_status_strings_and_host_only_entry_points():
    from fgattn_tk_cuda_b200 import capi
    lib = capi.lib()
    assert lib.fgattn_status_string(0) == b"ok"
    assert b"aligned" in lib.fgattn_status_string(3)
    # scratch size is pure host arithmetic: B*H * nkb * S_pad * 4
    assert capi.block_scratch_bytes(1, 32, 16384) == 32 * 256 * 16384 * 4
    assert capi.block_scratch_bytes(4, 24, 12345) == 96 * 193 * 12416 * 4
    assert capi.block_scratch_bytes(1, 1, 0) == 0


def test_argument_validation_needs_no_device():
    from fgattn_tk_cuda_b200 import capi
    lib = capi.lib()
    null = ctypes.c_void_p(0)
    buf = ctypes.c_void_p(0x1000)
    assert lib.fgattn_full_attn(null, buf, buf, buf, 1, 1, 64, 64, 64, 64, 0.0, null) == 1  # null output
    assert lib.fgattn_full_attn(buf, buf, buf, buf, 1, 1, 64, 96, 64, 64, 0.0, null) == 2   # head dim
    assert lib.fgattn_full_attn(buf, buf, buf, buf, 1, 1, 64, 64, 64, 65, 0.0, null) == 1   # kv_seq_len > kv_rows
    assert lib.fgattn_full_attn(buf, buf, buf, buf, 1, 1, 64, 64, 0, 0, 0.0, null) == 1     # no key rows
    assert lib.fgattn_full_attn(buf, ctypes.c_void_p(0x1008), buf, buf, 1, 1, 64, 64, 64, 64, 0.0, null) == 3
    assert lib.fgattn_maxq_denom(null, null, buf, buf, 1, 1, 64, 64, 64, 64, 0.0, null) == 1
    assert lib.fgattn_booleanmask_to_indexmask(buf, buf, buf, 1, 1, 64, 0, 128, null) == 1
    assert lib.fgattn_sp_attn_blocks_ml(buf, buf, buf, buf, buf, buf, 4, null, null, 1, 1, 64, 64, 64, 64, 0.0, buf, 64, null) == 1
    assert lib.fgattn_booleanmask_128_listed(buf, 1e-3, 128, buf, buf, buf, buf, null, buf, 4, 1, 1, 64, 64, 64, 64, 0.0,
                                             null, 0, null) == 1
    assert lib.fgattn_booleanmask_128_listed(buf, 1e-3, 128, buf, buf, buf, buf, buf, buf, 4, 1, 1, 64, 64, 64, 64, 0.0,
                                             buf, 8, null) == 7
    assert lib.fgattn_block_lists_from_maxima(buf, buf, 4, null, buf, buf, 1e-3, 1, 1, 64, 64, 64, 0.0, null) == 1
    assert lib.fgattn_block_lists_from_maxima(buf, buf, 0, buf, buf, buf, 1e-3, 1, 1, 64, 64, 64, 0.0, null) == 1   # list too narrow
    assert lib.fgattn_sp_attn(buf, buf, buf, buf, buf, null, 128, 1, 1, 64, 64, 64, 0.0, null, 0, null) == 1
    assert lib.fgattn_sp_attn(buf, buf, buf, buf, buf, buf, 128, 1, 1, 64, 64, 64, 0.0, buf, 8, null) == 7
    assert lib.fgattn_sp_attn_blocks(buf, buf, buf, buf, null, buf, 4, 1, 1, 64, 64, 64, 64, 0.0, null, 0, null) == 1
    assert lib.fgattn_sp_attn_blocks(buf, buf, buf, buf, buf, buf, 4, 1, 1, 64, 64, 64, 64, 0.0, buf, 8, null) == 7
    # one-bit-per-entry masks
    assert lib.fgattn_pack_mask(null, buf, 4, 8, 64, null) == 1                             # null output
    assert lib.fgattn_pack_mask(buf, buf, 2, 8, 64, null) == 2                              # element size
    assert lib.fgattn_pack_mask(buf, buf, 4, 8, 60, null) == 1                              # width % 8
    assert lib.fgattn_pack_mask(buf, ctypes.c_void_p(0x1004), 4, 8, 64, null) == 3          # int32 mask, 16-byte rule
    assert lib.fgattn_unpack_mask(buf, 1, null, 8, 64, null) == 1
    assert lib.fgattn_packedmask_to_indexmask(buf, buf, buf, 8, 64, 0, 64, 64, null) == 1   # list stride
    assert lib.fgattn_indexmask_to_packedmask(buf, buf, buf, 8, 64, 8 * 64 * 1024, null) == 2   # row too wide
    # top-k selector
    assert lib.fgattn_topk_indices(buf, buf, 128, buf, buf, 0, 1, 1, 256, 64, 128, 256, 256, 0.0, buf, 1 << 30, null) == 1
    assert lib.fgattn_topk_indices(buf, buf, 128, buf, buf, 129, 1, 1, 256, 64, 128, 256, 256, 0.0, buf, 1 << 30, null) == 1
    assert lib.fgattn_topk_indices(buf, buf, 16384, buf, buf, 9000, 1, 1, 16384, 64, 128, 16384, 16384, 0.0, buf, 1 << 40, null) == 2
    assert lib.fgattn_topk_indices(buf, buf, 128, buf, buf, 64, 1, 1, 256, 64, 128, 256, 256, 0.0, buf, 16, null) == 7
    assert capi.topk_scratch_bytes(1, 12, 32760, 128, 128) == 2 * 12 * 256 * 128 * 2 + 12 * 256 * 32768 * 4


def test_python_layer_refuses_cpu_tensors():
    import torch
    from fgattn_tk_cuda_b200 import capi
    q = torch.zeros(1, 1, 64, 64, dtype=torch.bfloat16)
    with pytest.raises(capi.FgattnError):
        capi.full_attn(torch.empty_like(q), q, q, q)


def test_operator_schemas_match_reference():
    """The seven reference schemas are registered verbatim under torch.ops.cuda_attn."""
    import torch
    import fgattn_tk_cuda_b200.spattn  # noqa: F401
    want = {
        "full_attn": "cuda_attn::full_attn(Tensor(o!) o, Tensor q, Tensor k, Tensor v) -> ()",
        "all_index_mask": "cuda_attn::all_index_mask(Tensor(kv_indices!) kv_indices, Tensor(kv_num_indices!) kv_num_indices, int batch, int heads, int seqblocks, int seq) -> ()",
        "sp_attn": "cuda_attn::sp_attn(Tensor(o!) o, Tensor q, Tensor k, Tensor v, Tensor kv_indices, Tensor kv_num_indices) -> ()",
        "fullattn_maxq_denom": "cuda_attn::fullattn_maxq_denom(Tensor(o!) o, Tensor(o_max_q!) o_max_q, Tensor(o_denom!) o_denom, Tensor q, Tensor k, Tensor v) -> ()",
        "maxq_denom": "cuda_attn::maxq_denom(Tensor(o_max_q!) o_max_q, Tensor(o_denom!) o_denom, Tensor q, Tensor k) -> ()",
        "booleanmask_128": "cuda_attn::booleanmask_128(Tensor(booleanmask!) booleanmask, Tensor o_max_q, Tensor o_denom, Tensor q, Tensor k, float threshold) -> ()",
        "booleanmask_to_indexmask": "cuda_attn::booleanmask_to_indexmask(Tensor(kv_indices!) kv_indices, Tensor(kv_numindices!) kv_numindices, Tensor booleanmask, int seq) -> ()",
    }
    for name, schema in want.items():
        op = getattr(torch.ops.cuda_attn, name)
        assert str(op.default._schema) == schema, str(op.default._schema)
    from fgattn_tk_cuda_b200.spattn import cuda_attn
    for name in want:
        assert hasattr(cuda_attn, name)
    # meta dispatch (shape propagation only) works without a device
    q = torch.empty(1, 1, 64, 64, dtype=torch.bfloat16, device="meta")
    assert torch.ops.cuda_attn.full_attn(q, q, q, q) is None
