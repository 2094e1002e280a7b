"""Mask pipeline wrappers and mask caches, mirroring python/spattn/mask_utils.py of the reference.

`blocksz=128` keeps the reference's granularity (128 query rows x 1 key token, token lists);
`blocksz=64` is the 64x64 block mode: key-BLOCK lists plus the per-row (max_q, denom) that the
block-sparse kernel needs, produced in ONE pass over the keys.

The reference's pure-PyTorch functions of the same module (qk_bitmask, qk_indexmask, attnmapor,
boolean_to_index_mask_2d, bitmask_to_indexmask) are its CPU path; they are deliberately not part of
this package (no CPU route exists here) and live, restated, in the test oracle.
"""
from __future__ import annotations

import torch

from . import cuda_attn  # noqa: F401  registers torch.ops.cuda_attn

spattn_interface = torch.ops.cuda_attn


def _pad128(n: int) -> int:
    return 128 * ((n + 127) // 128)


class nvtx_range:
    """NVTX range around one stage of the path (max_q / denom + lists, token mask, compaction, sparse
    attention, dense attention), so that a timeline shows the stages by name; the reference's profiling
    recipe picks kernels by name instead (profile.sh:5).  Costs nothing measurable without a profiler."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        torch.cuda.nvtx.range_pop()
        return False


# ------------------------------------------------------------------------------------------------
# mask caches (python/spattn/mask_utils.py:17-98): decide on which diffusion runs the mask is
# rebuilt and hand the cached lists to the sparse steps in between
# ------------------------------------------------------------------------------------------------
class NaiveMaskCache:
    """Keeps whatever the build step produced, per layer, on the device."""

    def __init__(self, compute_cache_at):
        self.cache = {}
        self.compute_cache_at = compute_cache_at

    def run_fullattn(self, ditrun) -> bool:
        return ditrun in self.compute_cache_at

    def get_mask_from_cache(self, layer):
        return self.cache[layer]

    def update_cache(self, layer, *mask):
        self.cache[layer] = tuple(mask)


class OffloadMaskCache(NaiveMaskCache):
    """Index lists live in host memory between uses; counts (and m/l in block mode) stay on the GPU."""

    def get_mask_from_cache(self, layer, ditrun=0):
        first, *rest = self.cache[layer]
        return (first.to("cuda", non_blocking=True), *rest)

    def update_cache(self, layer, first, *rest):
        self.cache[layer] = (first.cpu(), *rest)


class BitMaskCache(NaiveMaskCache):
    """Stores the int mask [B,H,SB,stride] and rebuilds the lists on every read."""

    def get_mask_from_cache(self, layer):
        mask, seq_len = self.cache[layer]
        return bitmask_to_indexmask_cuda(mask, seq_len)

    def update_cache(self, layer, mask, seq_len):
        self.cache[layer] = (mask, seq_len)


class CompressedBitMaskCache(BitMaskCache):
    """Same, with the mask packed to one bit per entry (python/spattn/mask_utils.py:87-98).  Reading
    goes from the packed bits straight to the lists in one kernel; the int32 mask is never rebuilt."""

    def get_mask_from_cache(self, layer):
        packed, seq_len = self.cache[layer]
        return packedmask_to_indexmask_cuda(packed, seq_len)

    def update_cache(self, layer, mask, seq_len):
        self.cache[layer] = (pack(mask), seq_len)


class CompressedListCache(NaiveMaskCache):
    """Caches index lists (key tokens or 64-key blocks) as one bit per entry: 1/32 of the int32 lists.
    `width` = number of list targets (keys or key blocks); lists come back ascending, unused slots
    filled with the list stride.  Tensors handed over after the counts (the max_q hint of the block mode)
    are kept as they are and come back behind the lists."""

    def get_mask_from_cache(self, layer):
        packed, width, stride, extra = self.cache[layer]
        return (*packedmask_to_indexmask_cuda(packed, width, stride=stride), *extra)

    def update_cache(self, layer, indices, num_indices, *extra, width=None):
        if extra and isinstance(extra[0], int):
            width, extra = extra[0], extra[1:]
        width = indices.shape[-1] if width is None else width
        self.cache[layer] = (indexmask_to_packedmask_cuda(indices, num_indices, width), width, indices.shape[-1],
                             tuple(extra))


def pack(mask: torch.Tensor) -> torch.Tensor:
    """[..., W] (bool / uint8 / int32, kept iff > 0; W % 8 == 0) -> uint8 [..., W/8], least significant
    bit first (python/spattn/mask_utils.py:421-430)."""
    mask = mask.contiguous()
    packed = torch.empty((*mask.shape[:-1], mask.shape[-1] // 8), dtype=torch.uint8, device=mask.device)
    spattn_interface.pack_mask(packed, mask)
    return packed


def unpack(packed: torch.Tensor, dtype=torch.bool) -> torch.Tensor:
    """Inverse of pack (python/spattn/mask_utils.py:433-440): bool [..., 8 * W8] (or uint8 / int32 of
    0 / 1 when `dtype` says so)."""
    packed = packed.contiguous()
    mask = torch.empty((*packed.shape[:-1], packed.shape[-1] * 8), dtype=dtype, device=packed.device)
    spattn_interface.unpack_mask(mask, packed)
    return mask


def packedmask_to_indexmask_cuda(packed: torch.Tensor, seq=None, stride=None):
    """Packed mask [..., W/8] -> ascending lists int32 [..., stride] (default stride = W) + counts
    [...]; entries >= `seq` are ignored; unused slots = stride."""
    W = packed.shape[-1] * 8
    stride = W if stride is None else stride
    indices = torch.empty((*packed.shape[:-1], stride), dtype=torch.int32, device=packed.device)
    num = torch.empty(packed.shape[:-1], dtype=torch.int32, device=packed.device)
    spattn_interface.packedmask_to_indexmask(indices, num, packed.contiguous(), W if seq is None else seq, stride)
    return indices, num


def indexmask_to_packedmask_cuda(indices: torch.Tensor, num_indices: torch.Tensor, width: int) -> torch.Tensor:
    """Lists int32 [..., stride] + counts -> packed mask uint8 [..., ceil(width / 32) * 4]."""
    packed = torch.empty((*indices.shape[:-1], 4 * ((width + 31) // 32)), dtype=torch.uint8, device=indices.device)
    spattn_interface.indexmask_to_packedmask(packed, indices.contiguous(), num_indices.contiguous())
    return packed


# ------------------------------------------------------------------------------------------------
# synthetic lists (python/spattn/mask_utils.py:175-203)
# ------------------------------------------------------------------------------------------------
def allindex_mask(B: int, H: int, max_stride: int, S: int, BLOCKSZ: int, device="cuda"):
    nb = (S + BLOCKSZ - 1) // BLOCKSZ
    kv_indices = torch.empty(B, H, nb, max_stride, device=device, dtype=torch.int32)
    kv_num_indices = torch.empty(B, H, nb, device=device, dtype=torch.int32)
    spattn_interface.all_index_mask(kv_indices, kv_num_indices, B, H, nb, S)
    return kv_indices, kv_num_indices


def halfindex_mask(B: int, H: int, S: int, BLOCKSZ: int, device="cuda"):
    nb = (S + BLOCKSZ - 1) // BLOCKSZ
    idx = (2 * torch.arange(S // 2, device=device, dtype=torch.int32)).expand(B, H, nb, S // 2).contiguous()
    return idx, torch.full((B, H, nb), S // 2, device=device, dtype=torch.int32)


def allindex_randompermutation_mask(B: int, H: int, max_stride: int, S: int, BLOCKSZ: int, device="cuda"):
    nb = (S + BLOCKSZ - 1) // BLOCKSZ
    perm = torch.randperm(S, device=device).to(torch.int32)
    if max_stride > S:
        perm = torch.cat([perm, torch.full((max_stride - S,), max_stride, device=device, dtype=torch.int32)])
    return perm.expand(B, H, nb, max_stride).contiguous(), torch.full((B, H, nb), S, device=device, dtype=torch.int32)


# ------------------------------------------------------------------------------------------------
# CUDA mask pipeline
# ------------------------------------------------------------------------------------------------
def _maxq_denom(q, k):
    B, H, S, _ = q.shape
    max_q = torch.empty((B, H, 1, _pad128(S)), dtype=torch.float32, device=q.device)
    denom = torch.empty_like(max_q)
    with nvtx_range("fgattn.maxq_denom"):
        spattn_interface.maxq_denom(max_q, denom, q.contiguous(), k.contiguous())
    return max_q, denom


def qk_bitmask_from_maxq_denom_cuda(max_q, denom, q, k, thresh, blocksz=128):
    """int32 [B,H,ceil(S/128),S_pad] token mask (python/spattn/mask_utils.py:337-354)."""
    assert blocksz == 128
    B, H, S, _ = q.shape
    mask = torch.empty((B, H, (S + 127) // 128, max_q.shape[3]), device=q.device, dtype=torch.int32)
    with nvtx_range("fgattn.token_mask"):
        spattn_interface.booleanmask_128(mask, max_q.contiguous(), denom.contiguous(), q.contiguous(), k.contiguous(),
                                         thresh)
    return mask


def qk_token_mask_cuda(q, k, thresh, v=None):
    """Token mask int32 [B,H,ceil(S/128),pad128(S_kv)] of the reference granularity in two cheap passes:
    the one-pass 64x64 block pipeline (max_q, denom, key-block lists, and the dense output when v is
    given), then the threshold test of python/spattn/mask_utils.py:337-354 only inside the kept blocks --
    a token can pass only there.  Returns (mask, max_q, denom[, out])."""
    kb_idx, kb_cnt, max_q, denom, *out = qk_block_indexmask_cuda(q, k, thresh, v=v)
    B, H, S, _ = q.shape
    mask = torch.empty((B, H, (S + 127) // 128, _pad128(k.shape[2])), device=q.device, dtype=torch.int32)
    with nvtx_range("fgattn.token_mask_in_kept_blocks"):
        spattn_interface.booleanmask_128_listed(mask, max_q, denom, q.contiguous(), k.contiguous(), thresh, kb_idx,
                                                kb_cnt)
    return (mask, max_q, denom, *out)


def qk_bitmask_cuda(q, k, thresh, blocksz=128):
    """bool token mask (python/spattn/mask_utils.py:248-269)."""
    assert blocksz == 128
    return qk_token_mask_cuda(q, k, thresh)[0] > 0


def bitmask_to_indexmask_cuda(booleanmask, seq=None):
    """Mask -> ascending token lists + counts (python/spattn/mask_utils.py:293-303); `seq` bounds
    the key index (default: the mask width)."""
    B, H, SB, stride = booleanmask.shape
    kv_indices = torch.empty((B, H, SB, stride), device=booleanmask.device, dtype=torch.int32)
    num_kv_indices = torch.empty((B, H, SB), device=booleanmask.device, dtype=torch.int32)
    with nvtx_range("fgattn.mask_to_lists"):
        spattn_interface.booleanmask_to_indexmask(kv_indices, num_kv_indices,
                                                  booleanmask.to(torch.int32).contiguous(),
                                                  stride if seq is None else seq)
    return kv_indices, num_kv_indices


def qk_indexmask_from_maxq_denom_cuda(max_q, denom, q, k, thresh, blocksz=128):
    """Token lists from an existing (max_q, denom) (python/spattn/mask_utils.py:358-382)."""
    mask = qk_bitmask_from_maxq_denom_cuda(max_q, denom, q, k, thresh, blocksz)
    return bitmask_to_indexmask_cuda(mask, q.shape[2])


_scratch = {}


def _block_scratch(q, k=None):
    """Block-maxima scratch of the one-pass list builder, cached per (device, current stream): calls on
    one stream are serialised by it and share the buffer, calls on different streams (or host threads
    working on different streams) get their own.  release_block_scratch() drops the buffers."""
    B, H, S, _ = q.shape
    need = cuda_attn.block_scratch_bytes(B, H, S, S if k is None else k.shape[2])
    per_head = need // (B * H)
    key = (q.device, torch.cuda.current_stream(q.device).cuda_stream)
    have = _scratch.get(key)
    if have is not None and have.numel() * 4 >= need:
        return have
    free, _total = torch.cuda.mem_get_info(q.device)
    heads_fit = max(1, min(B * H, int(free * 0.5) // per_head))     # fewer heads -> the op loops over chunks
    want = per_head * heads_fit
    if have is None or have.numel() * 4 < want:
        _scratch.pop(key, None)
        have = None
        _scratch[key] = have = torch.empty(want // 4, dtype=torch.float32, device=q.device)
    return have


def release_block_scratch():
    """Free the cached scratch buffers of qk_block_indexmask_cuda (and the operators' work-queue scratch)."""
    _scratch.clear()
    cuda_attn.release_workspaces()


def qk_block_indexmask_cuda(q, k, thresh, v=None):
    """64x64 block mode, one pass: returns (kb_indices [B,H,nqb,nkb], kb_counts [B,H,nqb], max_q,
    denom) and, when v is given, the dense attention output as a fifth element."""
    B, H, S, D = q.shape
    nqb, nkb = (S + 63) // 64, (k.shape[2] + 63) // 64
    kb_indices = torch.empty((B, H, nqb, nkb), device=q.device, dtype=torch.int32)
    kb_counts = torch.empty((B, H, nqb), device=q.device, dtype=torch.int32)
    max_q = torch.empty((B, H, 1, _pad128(S)), dtype=torch.float32, device=q.device)
    denom = torch.empty_like(max_q)
    o = torch.empty((B, H, S, D), device=q.device, dtype=torch.bfloat16) if v is not None else None
    with nvtx_range("fgattn.maxq_denom+block_lists" + ("+full_attn" if v is not None else "")):
        spattn_interface.block_index_lists(kb_indices, kb_counts, max_q, denom, o, q.contiguous(), k.contiguous(),
                                           None if v is None else v.contiguous(), thresh, _block_scratch(q, k))
    return (kb_indices, kb_counts, max_q, denom) + ((o,) if v is not None else ())


def qk_indexmask_cuda(q, k, thresh, blocksz=128):
    """python/spattn/mask_utils.py:306-334.  blocksz=128: token lists; blocksz=64: see
    qk_block_indexmask_cuda (returns four tensors)."""
    if blocksz == 64:
        return qk_block_indexmask_cuda(q, k, thresh)
    assert blocksz == 128
    return bitmask_to_indexmask_cuda(qk_token_mask_cuda(q, k, thresh)[0], k.shape[2])


# ------------------------------------------------------------------------------------------------
# alternative selectors (python/spattn/mask_utils.py:385-417)
# ------------------------------------------------------------------------------------------------
def qk_lshmask_indices(query, key, thresh, blocksz=128):
    """Not implemented in the reference either (python/spattn/mask_utils.py:385-386)."""
    raise NotImplementedError


def qk_topkmask_indices(q, k, select_k, B=None, H=None, S=None, D=None, BLOCKSZ=128, blocksz=None, max_stride=None):
    """Per block of BLOCKSZ query rows the select_k keys with the largest (block-mean query . key)/sqrt(D),
    descending (python/spattn/mask_utils.py:389-417; B, H, S, D are taken from q when omitted).  The
    list stride is select_k rounded up to a multiple of 128 (unused slots = stride), the form the
    sp_attn operator takes."""
    BLOCKSZ = BLOCKSZ if blocksz is None else blocksz
    Bq, Hq, Sq, _ = q.shape
    nblk = (Sq + BLOCKSZ - 1) // BLOCKSZ
    stride = _pad128(select_k) if max_stride is None else max_stride
    kv_indices = torch.empty((Bq, Hq, nblk, stride), dtype=torch.int32, device=q.device)
    kv_num_indices = torch.empty((Bq, Hq, nblk), dtype=torch.int32, device=q.device)
    spattn_interface.topk_indices(kv_indices, kv_num_indices, q.contiguous(), k.contiguous(), int(select_k),
                                  int(BLOCKSZ))
    return kv_indices, kv_num_indices
