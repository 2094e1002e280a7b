"""ctypes binding of the C ABI declared in include/fgattn_b200.h.

This is the only route from Python to the kernels; there is no fallback.  Importing works without a
GPU (so the symbol table can be checked), calling needs one.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

import os

# FGATTN_B200_LIB overrides the library file (A/B builds of the same C ABI)
_LIB_PATH = Path(os.environ.get("FGATTN_B200_LIB") or Path(__file__).resolve().parent / "libfgattn_b200.so")

OK = 0
STATUS_NAMES = {0: "OK", 1: "INVALID_ARGUMENT", 2: "UNSUPPORTED", 3: "MISALIGNED", 4: "CUDA_ERROR", 5: "NO_DRIVER",
                6: "DEVICE_TIMEOUT", 7: "SCRATCH_TOO_SMALL"}

_vp, _i, _f, _sz, _ll = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_longlong

# name -> (restype, argtypes); mirrors include/fgattn_b200.h one to one
PROTOTYPES = {
    "fgattn_status_string": (C.c_char_p, [_i]),
    "fgattn_last_cuda_error": (_i, []),
    "fgattn_check": (_i, [_vp, C.POINTER(_i)]),
    "fgattn_set_tuning": (_i, [C.c_char_p, _i]),
    "fgattn_full_attn": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "fgattn_fullattn_maxq_denom": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "fgattn_maxq_denom": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "fgattn_booleanmask_128": (_i, [_vp, _f, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "fgattn_booleanmask_128_listed": (_i, [_vp, _f, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f,
                                           _vp, _sz, _vp]),
    "fgattn_booleanmask_to_indexmask": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "fgattn_all_index_mask": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "fgattn_sp_attn": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp]),
    "fgattn_block_scratch_bytes": (_sz, [_i, _i, _i, _i]),
    "fgattn_block_index_lists": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i, _i, _i, _i, _i, _f, _vp,
                                      _sz, _vp]),
    "fgattn_block_lists_from_maxima": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _f, _i, _i, _i, _i, _i, _f, _vp]),
    "fgattn_block_index_lists_noalloc": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i, _i, _i, _i, _f,
                                              _vp]),
    "fgattn_sp_attn_blocks_ml": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _sz,
                                      _vp]),
    "fgattn_sp_attn_workspace_bytes": (_sz, [_i, _i, _i]),
    "fgattn_sp_attn_token_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "fgattn_sp_attn_blocks_hint": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _sz,
                                        _vp]),
    "fgattn_selftest_bounded_wait": (_i, [_ll, _vp]),
    "fgattn_sp_attn_blocks": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp]),
    "fgattn_topk_scratch_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "fgattn_topk_indices": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp]),
    "fgattn_pack_mask": (_i, [_vp, _vp, _i, _ll, _i, _vp]),
    "fgattn_unpack_mask": (_i, [_vp, _i, _vp, _ll, _i, _vp]),
    "fgattn_packedmask_to_indexmask": (_i, [_vp, _vp, _vp, _ll, _i, _i, _i, _i, _vp]),
    "fgattn_indexmask_to_packedmask": (_i, [_vp, _vp, _vp, _ll, _i, _i, _vp]),
}

_lib = None


class FgattnError(RuntimeError):
    def __init__(self, fn: str, status: int, detail: str = ""):
        self.status = status
        super().__init__(f"{fn} failed: {STATUS_NAMES.get(status, status)} {detail}".strip())


def lib() -> C.CDLL:
    """Load libfgattn_b200.so (built in-tree by fgattn_tk_cuda_b200._build).  Raises if absent."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(f"{_LIB_PATH} is missing: build it with `python -m fgattn_tk_cuda_b200._build` "
                              "(there is no CPU or PyTorch fallback)")
        l = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(t: torch.Tensor):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _call(name: str, *args):
    st = getattr(lib(), name)(*args)
    if st != OK:
        detail = lib().fgattn_status_string(st).decode()
        if st == 4:
            detail += f" (cudaError {lib().fgattn_last_cuda_error()})"
        raise FgattnError(name, st, detail)


def _check_qkv(*ts):
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise FgattnError("argument check", 1, "tensors must live on a CUDA device")
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or t.dim() != 4:
            raise FgattnError("argument check", 1, "q/k/v/o must be contiguous bf16 [B,H,S,D]")


def check(device=None) -> None:
    """Synchronise the current stream and raise if a kernel gave up on a bounded wait."""
    code = _i(0)
    with torch.cuda.device(device):
        st = lib().fgattn_check(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(code))
    if st != OK:
        e = FgattnError("fgattn_check", st, f"wait id {code.value}")
        e.code = code.value
        raise e


def set_tuning(name: str, value: int) -> None:
    """Scheduling knobs ("group_heads", "dense_persist"); see fgattn_set_tuning in the header."""
    _call("fgattn_set_tuning", name.encode(), int(value))


def full_attn(o, q, k, v, kv_seq_len=None, scale=0.0):
    _check_qkv(o, q, k, v)
    B, H, S, D = q.shape
    with torch.cuda.device(q.device):
        _call("fgattn_full_attn", _ptr(o), _ptr(q), _ptr(k), _ptr(v), B, H, S, D, k.shape[2],
              kv_seq_len or k.shape[2], scale, _stream(q))


def fullattn_maxq_denom(o, max_q, denom, q, k, v, kv_seq_len=None, scale=0.0):
    _check_qkv(o, q, k, v)
    B, H, S, D = q.shape
    with torch.cuda.device(q.device):
        _call("fgattn_fullattn_maxq_denom", _ptr(o), _ptr(max_q), _ptr(denom), _ptr(q), _ptr(k), _ptr(v), B, H, S, D,
              k.shape[2], kv_seq_len or k.shape[2], scale, _stream(q))


def maxq_denom(max_q, denom, q, k, kv_seq_len=None, scale=0.0):
    _check_qkv(q, k)
    B, H, S, D = q.shape
    with torch.cuda.device(q.device):
        _call("fgattn_maxq_denom", _ptr(max_q), _ptr(denom), _ptr(q), _ptr(k), B, H, S, D, k.shape[2],
              kv_seq_len or k.shape[2], scale, _stream(q))


def booleanmask_128(booleanmask, max_q, denom, q, k, threshold, kv_seq_len=None, scale=0.0):
    _check_qkv(q, k)
    B, H, S, D = q.shape
    with torch.cuda.device(q.device):
        _call("fgattn_booleanmask_128", _ptr(booleanmask), float(threshold), booleanmask.shape[3], _ptr(max_q),
              _ptr(denom), _ptr(q), _ptr(k), B, H, S, D, k.shape[2], kv_seq_len or k.shape[2], scale, _stream(q))


def booleanmask_128_listed(booleanmask, max_q, denom, q, k, threshold, kb_indices, kb_counts, kv_seq_len=None,
                           scale=0.0, workspace=None, ordered=True):
    """booleanmask_128 restricted to the 64x64 blocks that block_index_lists kept for the same inputs.
    ordered: thread blocks take the longest lists first (workspace allocated here when not given)."""
    _check_qkv(q, k)
    B, H, S, D = q.shape
    if ordered and workspace is None:
        workspace = torch.empty(sp_attn_workspace_bytes(B, H, S), dtype=torch.uint8, device=q.device)
    ws_ptr = _ptr(workspace) if ordered else None
    ws_bytes = workspace.numel() * workspace.element_size() if ordered else 0
    with torch.cuda.device(q.device):
        _call("fgattn_booleanmask_128_listed", _ptr(booleanmask), float(threshold), booleanmask.shape[3], _ptr(max_q),
              _ptr(denom), _ptr(q), _ptr(k), _ptr(kb_indices), _ptr(kb_counts), kb_indices.shape[3], B, H, S, D,
              k.shape[2], kv_seq_len or k.shape[2], scale, ws_ptr, ws_bytes, _stream(q))


def booleanmask_to_indexmask(kv_indices, kv_num_indices, booleanmask, seq):
    B, H, SB, stride = booleanmask.shape
    with torch.cuda.device(booleanmask.device):
        _call("fgattn_booleanmask_to_indexmask", _ptr(kv_indices), _ptr(kv_num_indices), _ptr(booleanmask), B, H,
              int(seq), SB, stride, _stream(booleanmask))


def all_index_mask(kv_indices, kv_num_indices, batch, heads, seqblocks, seq):
    with torch.cuda.device(kv_indices.device):
        _call("fgattn_all_index_mask", _ptr(kv_indices), _ptr(kv_num_indices), batch, heads, seqblocks, seq,
              kv_indices.shape[3], _stream(kv_indices))


def sp_attn_token_workspace_bytes(B, H, S, kv_rows) -> int:
    return int(lib().fgattn_sp_attn_token_workspace_bytes(B, H, S, kv_rows))


def sp_attn(o, q, k, v, kv_indices, kv_num_indices, scale=0.0, workspace=None, ordered=True, block_route=False):
    """ordered: thread blocks take the longest lists first (needs the workspace, allocated here when not
    given); ordered=False runs them in storage order with no workspace.  block_route (with ordered):
    allocate the large workspace, with which -- once set_tuning("token_block_route", 1) is on -- query
    blocks whose lists fill the key blocks they touch load whole K/V tiles instead of gathering rows."""
    _check_qkv(o, q, k, v)
    B, H, S, D = q.shape
    if ordered and workspace is None:
        nbytes = sp_attn_token_workspace_bytes(B, H, S, k.shape[2]) if block_route else sp_attn_workspace_bytes(B, H, S)
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    ws_ptr = _ptr(workspace) if ordered else None
    ws_bytes = workspace.numel() * workspace.element_size() if ordered else 0
    with torch.cuda.device(q.device):
        _call("fgattn_sp_attn", _ptr(o), _ptr(q), _ptr(k), _ptr(v), _ptr(kv_indices), _ptr(kv_num_indices),
              kv_indices.shape[3], B, H, S, D, k.shape[2], scale, ws_ptr, ws_bytes, _stream(q))


def block_scratch_bytes(B, H, S, kv_seq_len=None) -> int:
    return int(lib().fgattn_block_scratch_bytes(B, H, S, kv_seq_len or S))


def block_index_lists(kb_indices, kb_counts, max_q, denom, q, k, threshold, scratch, o=None, v=None, kv_seq_len=None,
                      scale=0.0):
    _check_qkv(q, k, o, v)
    B, H, S, D = q.shape
    with torch.cuda.device(q.device):
        _call("fgattn_block_index_lists", _ptr(kb_indices), _ptr(kb_counts), kb_indices.shape[3], _ptr(max_q),
              _ptr(denom), _ptr(o), _ptr(q), _ptr(k), _ptr(v), float(threshold), B, H, S, D, k.shape[2],
              kv_seq_len or k.shape[2], scale, _ptr(scratch), scratch.numel() * scratch.element_size(), _stream(q))


def block_lists_from_maxima(kb_indices, kb_counts, block_maxima, max_q, denom, q_shape, threshold, kv_seq_len=None,
                            scale=0.0):
    """The threshold step alone on the block maxima that block_index_lists left in a scratch sized for all units
    (q_shape = (B, H, S, D) of that call): lists for another threshold without a new pass over the keys."""
    B, H, S, D = q_shape
    with torch.cuda.device(kb_indices.device):
        _call("fgattn_block_lists_from_maxima", _ptr(kb_indices), _ptr(kb_counts), kb_indices.shape[3],
              _ptr(block_maxima), _ptr(max_q), _ptr(denom), float(threshold), B, H, S, D, kv_seq_len or S, scale,
              _stream(kb_indices))


NOALLOC_SCRATCH_BYTES = 64 << 20


def block_index_lists_noalloc(kb_indices, kb_counts, max_q, denom, q, k, threshold, o=None, v=None, kv_seq_len=None,
                              scale=0.0):
    """fgattn_block_index_lists_noalloc: same results as block_index_lists, scratch built into the
    library (no allocation anywhere on this path; one (batch, head) unit must fit in 64 MiB)."""
    # this entry point has no kv_rows argument: it reads k / v as [B, H, S, D]
    if k.shape != q.shape or (v is not None and v.shape != q.shape) or (o is not None and o.shape != q.shape):
        raise FgattnError("fgattn_block_index_lists_noalloc", 1, "k, v and o must have exactly the shape of q")
    _check_qkv(q, k, o, v)
    B, H, S, D = q.shape
    with torch.cuda.device(q.device):
        _call("fgattn_block_index_lists_noalloc", _ptr(kb_indices), _ptr(kb_counts), kb_indices.shape[3], _ptr(max_q),
              _ptr(denom), _ptr(o), _ptr(q), _ptr(k), _ptr(v), float(threshold), B, H, S, D, kv_seq_len or S, scale,
              _stream(q))


def sp_attn_workspace_bytes(B, H, S) -> int:
    return int(lib().fgattn_sp_attn_workspace_bytes(B, H, S))


def sp_attn_blocks_ml(o, q, k, v, kb_indices, kb_counts, max_q, denom, kv_seq_len=None, scale=0.0, workspace=None):
    _check_qkv(o, q, k, v)
    B, H, S, D = q.shape
    if workspace is None:                                # stream-ordered scratch from torch's caching allocator
        workspace = torch.empty(sp_attn_workspace_bytes(B, H, S), dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        _call("fgattn_sp_attn_blocks_ml", _ptr(o), _ptr(q), _ptr(k), _ptr(v), _ptr(kb_indices), _ptr(kb_counts),
              kb_indices.shape[3], _ptr(max_q), _ptr(denom), B, H, S, D, k.shape[2], kv_seq_len or k.shape[2], scale,
              _ptr(workspace),
              workspace.numel() * workspace.element_size(), _stream(q))


def sp_attn_blocks_hint(o, q, k, v, kb_indices, kb_counts, max_q_hint, kv_seq_len=None, scale=0.0, workspace=None):
    """Renormalising block-sparse attention on the persistent kernel; max_q_hint [B,H,1,S_pad] is a
    per-row estimate of the row maximum (e.g. the max_q of the pass that built the lists)."""
    _check_qkv(o, q, k, v)
    B, H, S, D = q.shape
    if workspace is None:
        workspace = torch.empty(sp_attn_workspace_bytes(B, H, S), dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        _call("fgattn_sp_attn_blocks_hint", _ptr(o), _ptr(q), _ptr(k), _ptr(v), _ptr(kb_indices), _ptr(kb_counts),
              kb_indices.shape[3], _ptr(max_q_hint), B, H, S, D, k.shape[2], kv_seq_len or k.shape[2], scale,
              _ptr(workspace), workspace.numel() * workspace.element_size(), _stream(q))
    return workspace


def selftest_bounded_wait(budget_cycles: int = 100000, device=None) -> None:
    """Launch the one-warp probe whose bounded wait is left to run out; the next check() raises
    FgattnError(DEVICE_TIMEOUT) with wait id 9001."""
    with torch.cuda.device(device):
        _call("fgattn_selftest_bounded_wait", int(budget_cycles), C.c_void_p(torch.cuda.current_stream().cuda_stream))


def sp_attn_blocks(o, q, k, v, kb_indices, kb_counts, kv_seq_len=None, scale=0.0, workspace=None, ordered=True):
    """ordered: thread blocks take the longest lists first (needs the workspace, allocated here when not
    given); ordered=False runs them in storage order with no workspace."""
    _check_qkv(o, q, k, v)
    B, H, S, D = q.shape
    if ordered and workspace is None:
        workspace = torch.empty(sp_attn_workspace_bytes(B, H, S), dtype=torch.uint8, device=q.device)
    ws_ptr = _ptr(workspace) if ordered else None
    ws_bytes = workspace.numel() * workspace.element_size() if ordered else 0
    with torch.cuda.device(q.device):
        _call("fgattn_sp_attn_blocks", _ptr(o), _ptr(q), _ptr(k), _ptr(v), _ptr(kb_indices), _ptr(kb_counts),
              kb_indices.shape[3], B, H, S, D, k.shape[2], kv_seq_len or k.shape[2], scale, ws_ptr, ws_bytes,
              _stream(q))


# ---- one-bit-per-entry masks ----------------------------------------------------------------------
def _mask_elem_size(t: torch.Tensor) -> int:
    if not t.is_cuda or not t.is_contiguous():
        raise FgattnError("argument check", 1, "mask tensors must be contiguous CUDA tensors")
    if t.dtype in (torch.bool, torch.uint8):
        return 1
    if t.dtype == torch.int32:
        return 4
    raise FgattnError("argument check", 1, "masks are bool, uint8 or int32")


def pack_mask(packed, mask):
    """mask [..., W] (bool / uint8 / int32, kept iff > 0) -> packed uint8 [..., W/8]."""
    W = mask.shape[-1]
    with torch.cuda.device(mask.device):
        _call("fgattn_pack_mask", _ptr(packed), _ptr(mask), _mask_elem_size(mask), mask.numel() // W, W, _stream(mask))


def unpack_mask(mask, packed):
    """packed uint8 [..., W/8] -> mask [..., W] of 0 / 1 (bool / uint8 / int32)."""
    W = mask.shape[-1]
    with torch.cuda.device(mask.device):
        _call("fgattn_unpack_mask", _ptr(mask), _mask_elem_size(mask), _ptr(packed), mask.numel() // W, W,
              _stream(mask))


def packedmask_to_indexmask(indices, num_indices, packed, n_valid, sentinel=None):
    """packed uint8 [..., W/8] -> ascending lists `indices` int32 [..., stride] + counts [...]."""
    W = packed.shape[-1] * 8
    stride = indices.shape[-1]
    with torch.cuda.device(packed.device):
        _call("fgattn_packedmask_to_indexmask", _ptr(indices), _ptr(num_indices), _ptr(packed),
              packed.numel() // packed.shape[-1], W, stride, int(n_valid), stride if sentinel is None else int(sentinel),
              _stream(packed))


def indexmask_to_packedmask(packed, indices, num_indices):
    """lists int32 [..., stride] + counts [...] -> packed uint8 [..., W/8]."""
    W = packed.shape[-1] * 8
    with torch.cuda.device(packed.device):
        _call("fgattn_indexmask_to_packedmask", _ptr(packed), _ptr(indices), _ptr(num_indices),
              packed.numel() // packed.shape[-1], indices.shape[-1], W, _stream(packed))


# ---- top-k selector ---------------------------------------------------------------------------------
def topk_scratch_bytes(B, H, S, D, blocksz, kv_seq_len=None) -> int:
    return int(lib().fgattn_topk_scratch_bytes(B, H, S, D, blocksz, kv_seq_len or S))


def topk_indices(kv_indices, kv_num_indices, q, k, select_k, blocksz=128, kv_seq_len=None, scale=0.0, scratch=None):
    """Per query block the select_k keys with the largest (block-mean query . key) score."""
    _check_qkv(q, k)
    B, H, S, D = q.shape
    if scratch is None:
        scratch = torch.empty(topk_scratch_bytes(B, H, S, D, blocksz, kv_seq_len or k.shape[2]), dtype=torch.uint8,
                              device=q.device)
    with torch.cuda.device(q.device):
        _call("fgattn_topk_indices", _ptr(kv_indices), _ptr(kv_num_indices), kv_indices.shape[3], _ptr(q), _ptr(k),
              int(select_k), B, H, S, D, int(blocksz), k.shape[2], kv_seq_len or k.shape[2], scale, _ptr(scratch),
              scratch.numel() * scratch.element_size(), _stream(q))
