"""Model-facing attention entry points, mirroring python/spattn/sparseattn_functionals.py of the
reference: same names, same `(query, key, value, current_layer, ditrun, **kwargs)` calling
convention, same kwargs (`thresh`, `blocksz`, `mask_cache`).  `blocksz=128` runs the reference
granularity (token lists, renormalising sp_attn); `blocksz=64` runs the 64x64 block mode (key-block
lists, probabilities from the full softmax's max_q / denom)."""
from __future__ import annotations

import torch

from . import mask_utils

spattn_interface = torch.ops.cuda_attn


def _out(query):
    return torch.empty(query.shape, device=query.device, dtype=torch.bfloat16)


def _ml(query):
    B, H, S, _ = query.shape
    m = torch.empty((B, H, 1, 128 * ((S + 127) // 128)), dtype=torch.float32, device=query.device)
    return m, torch.empty_like(m)


def baseline_attn(query, key, value, current_layer=None, ditrun=None, *args, **kwargs):
    """Dense attention (sparseattn_functionals.py:10-15)."""
    out = _out(query)
    with mask_utils.nvtx_range("fgattn.full_attn"):
        spattn_interface.full_attn(out, query.contiguous(), key.contiguous(), value.contiguous())
    return out


def baseline_attn_maxq_denom(query, key, value, current_layer=None, ditrun=None, *args, **kwargs):
    """Dense attention that also computes max_q / denom (sparseattn_functionals.py:18-26)."""
    out = _out(query)
    max_q, denom = _ml(query)
    with mask_utils.nvtx_range("fgattn.full_attn+maxq_denom"):
        spattn_interface.fullattn_maxq_denom(out, max_q, denom, query.contiguous(), key.contiguous(),
                                             value.contiguous())
    return out


def _sparse(out, query, key, value, mask, blocksz=128):
    """One sparse step.  A 4-tuple (kb_indices, kb_counts, max_q, denom) carries the max_q / denom of
    THESE query / key tensors and runs the non-renormalising block kernel; a pair of lists runs the
    renormalising kernel of its granularity (key blocks for blocksz 64, key tokens otherwise), which is
    what a mask cached from an earlier diffusion run needs; a 3-tuple (kb_indices, kb_counts, max_q) is
    such a cached block mask together with the max_q of the run that built it, which the renormalising
    persistent kernel takes as its per-row exponent hint."""
    q, k, v = query.contiguous(), key.contiguous(), value.contiguous()
    with mask_utils.nvtx_range("fgattn.sparse_attention"):
        if len(mask) == 4:
            spattn_interface.sp_attn_blocks_ml(out, q, k, v, mask[0].contiguous(), mask[1].contiguous(), mask[2],
                                               mask[3])
        elif len(mask) == 3:
            spattn_interface.sp_attn_blocks_hint(out, q, k, v, mask[0].contiguous(), mask[1].contiguous(), mask[2])
        elif blocksz == 64:
            spattn_interface.sp_attn_blocks(out, q, k, v, mask[0].contiguous(), mask[1].contiguous())
        else:
            spattn_interface.sp_attn(out, q, k, v, mask[0].contiguous(), mask[1].contiguous())
    return out


def attn_computed_with_sparse_mask_cuda(query, key, value, *args, **kwargs):
    """Build the mask from (query, key) and run the sparse kernel with it
    (sparseattn_functionals.py:61-69)."""
    mask = mask_utils.qk_indexmask_cuda(query, key, kwargs["thresh"], blocksz=kwargs["blocksz"])
    return _sparse(_out(query), query, key, value, mask)


def attn_topkmask_cuda(query, key, value, current_layer=None, ditrun=None, *args, **kwargs):
    """Top-k key selection per 128-row query block, then the token-list sparse kernel
    (sparseattn_functionals.py:39-48)."""
    select_k = kwargs.get("select_k") or query.shape[2]
    mask = mask_utils.qk_topkmask_indices(query, key, select_k, blocksz=kwargs.get("blocksz", 128))
    return _sparse(_out(query), query, key, value, mask)


def attn_lshmask_cuda(query, key, value, current_layer=None, ditrun=None, *args, **kwargs):
    """The LSH selector is a stub in the reference (mask_utils.py:385-386); it stays one."""
    raise NotImplementedError


def compute_cache_and_attn_cuda(query, key, value, *args, **kwargs):
    """Dense attention + mask in one go (sparseattn_functionals.py:74-84).  Returns
    (out, kv_indices, kv_num_indices) and, in block mode, additionally (max_q, denom)."""
    thresh, blocksz = kwargs["thresh"], kwargs["blocksz"]
    if blocksz == 64:
        idx, cnt, max_q, denom, out = mask_utils.qk_block_indexmask_cuda(query, key, thresh, v=value)
        return out, idx, cnt, max_q, denom
    # reference granularity: dense output, max_q / denom and the 64x64 block lists in one pass, then the
    # token mask only inside the kept blocks, then the compaction
    mask, _, _, out = mask_utils.qk_token_mask_cuda(query, key, thresh, v=value)
    idx, cnt = mask_utils.bitmask_to_indexmask_cuda(mask, key.shape[2])
    return out, idx, cnt


def sparse_attn_from_cache_cuda(query, key, value, *args, **kwargs):
    """Sparse step from a cached mask (sparseattn_functionals.py:87-93)."""
    mask = kwargs["mask_cache"].get_mask_from_cache(kwargs.get("current_layer", 0))
    blocksz = kwargs.get("blocksz", 128)
    return _sparse(_out(query), query, key, value, mask[:3] if blocksz == 64 else mask[:2], blocksz)


def cached_attn_cuda(query, key, value, current_layer, ditrun, *args, **kwargs):
    """Dense + mask build on the runs the cache names, sparse from the cache otherwise
    (sparseattn_functionals.py:95-113)."""
    mask_cache = kwargs["mask_cache"]
    if mask_cache.run_fullattn(ditrun):
        out, *mask = compute_cache_and_attn_cuda(query, key, value, thresh=kwargs["thresh"], blocksz=kwargs["blocksz"])
        # block mode keeps max_q with the lists: it belongs to this run's q, k, but on later runs it still
        # places the exponent range of the renormalising kernel (denom is of no use there)
        mask_cache.update_cache(current_layer, *mask[:3])
        return out
    mask = mask_cache.get_mask_from_cache(current_layer)
    blocksz = kwargs["blocksz"]
    return _sparse(_out(query), query, key, value, mask[:3] if blocksz == 64 else mask[:2], blocksz)


def bitmaskcached_attn_cuda(query, key, value, current_layer, ditrun, *args, **kwargs):
    """Like cached_attn_cuda with the int mask cached instead of the lists
    (sparseattn_functionals.py:116-134); reference granularity only."""
    mask_cache = kwargs["mask_cache"]
    if mask_cache.run_fullattn(ditrun):
        mask, _, _, out = mask_utils.qk_token_mask_cuda(query, key, kwargs["thresh"], v=value)
        mask_cache.update_cache(current_layer, mask, key.shape[2])
        return out
    return _sparse(_out(query), query, key, value, mask_cache.get_mask_from_cache(current_layer)[:2])


def attn_2xmask_cuda(query, key, value, current_layer=None, ditrun=None, *args, **kwargs):
    """Every other key, for every query block (sparseattn_functionals.py:137-153): the token-list kernel
    at exactly half density, lists built on the fly."""
    B, H, S, _ = query.shape
    idx, cnt = mask_utils.halfindex_mask(B, H, S, kwargs.get("blocksz", 128), device=query.device)
    return _sparse(_out(query), query, key, value, (idx, cnt))
