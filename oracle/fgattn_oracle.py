"""CPU oracle for the threshold block-sparse attention forward path.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain fp32 torch on the CPU, the pure-PyTorch
reference functions of sankeerth95/fgattn_tk_cuda.  Only the test-suite, the smoke check and the
benchmark's cpu_baseline / reference legs may import it; the product (the CUDA library and its
Python host layer) never does.

Parity status: PINNED.  tests/golden/ holds outputs of the reference's own functions
(python/spattn/mask_utils.py and python/test_mask.py, imported unmodified on the CPU by
tests/golden/make_golden.py); tests/test_oracle_golden.py checks every function here against them.

Every function cites the reference file:line it follows (paths inside the reference project).
Because the reference materialises an S x S map per head, the restatements here walk the query
rows in chunks; the arithmetic per row is the same (row softmax over ALL keys in fp32).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

__all__ = [
    "maxq_denom", "full_attn", "attnmapor", "boolean_to_index_mask_2d", "bitmask_to_indexmask",
    "qk_bitmask", "qk_token_pmax", "qk_indexmask", "qk_block_pmax", "qk_block_bitmask", "qk_block_indexmask",
    "qkattn_masked", "block_masked_attn", "sp_attn_tokens", "sp_attn_blocks", "allindex_mask",
    "near_threshold",
]


def _f32(x: torch.Tensor) -> torch.Tensor:
    return x.detach().to(device="cpu", dtype=torch.float32)


def _row_chunks(n_rows: int, block: int, max_rows: int = 2048):
    """Yield (start, stop) row ranges that are whole multiples of `block` (last may be ragged)."""
    step = max(block, (max_rows // block) * block)
    for s in range(0, n_rows, step):
        yield s, min(n_rows, s + step)


# ------------------------------------------------------------------------------------------------
# m / l : per-row raw maximum and softmax denominator
# ------------------------------------------------------------------------------------------------
def maxq_denom(q: torch.Tensor, k: torch.Tensor, kv_seq_len: Optional[int] = None,
               scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """m_i = max_j q_i.k_j (raw, unscaled) and l_i = sum_j exp((q_i.k_j - m_i) * scale).

    Follows python/test/spattn/test_mask_utils.py:42-52 (definition the CUDA pass is checked
    against) and include/maxq_denom.cuh:169-206.  Outputs have the reference's storage shape
    [B, H, 1, ceil(S/128)*128] with tail max = 0 and tail denom = -inf
    (include/maxq_denom.cuh:202-206).  scale defaults to 1/sqrt(D).
    """
    q, k = _f32(q), _f32(k)
    B, H, S, D = q.shape
    n_kv = k.shape[2] if kv_seq_len is None else kv_seq_len
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    s_pad = 128 * ((S + 127) // 128)
    m = torch.zeros(B, H, 1, s_pad, dtype=torch.float32)
    l = torch.full((B, H, 1, s_pad), float("-inf"), dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            kk = k[b, h, :n_kv]
            for r0, r1 in _row_chunks(S, 128):
                qk = q[b, h, r0:r1] @ kk.T
                mx = qk.max(dim=-1).values
                m[b, h, 0, r0:r1] = mx
                l[b, h, 0, r0:r1] = torch.exp((qk - mx[:, None]) * scale).sum(dim=-1)
    return m, l


def full_attn(q, k, v, kv_seq_len: Optional[int] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Dense softmax(q k^T * scale) v in fp32.  The reference checks its dense kernels against
    F.scaled_dot_product_attention (python/test/test_extension.py:15-30); this is the same math."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, H, S, D = q.shape
    n_kv = k.shape[2] if kv_seq_len is None else kv_seq_len
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    o = torch.empty(B, H, S, v.shape[3], dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            kk, vv = k[b, h, :n_kv], v[b, h, :n_kv]
            for r0, r1 in _row_chunks(S, 128):
                p = torch.softmax((q[b, h, r0:r1] @ kk.T) * scale, dim=-1)
                o[b, h, r0:r1] = p @ vv
    return o


# ------------------------------------------------------------------------------------------------
# 2-D map helpers
# ------------------------------------------------------------------------------------------------
def attnmapor(attnmap: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Row-block OR / max of an [M, N] map, ragged last block included.
    Follows python/spattn/mask_utils.py:126-142."""
    M, N = attnmap.shape
    nb = (M + block - 1) // block
    out = torch.empty(nb, N, dtype=attnmap.dtype)
    for i in range(nb):
        out[i] = attnmap[i * block:min(M, (i + 1) * block)].max(dim=0).values
    return out


def boolean_to_index_mask_2d(boolean_mask) -> Tuple[torch.Tensor, torch.Tensor]:
    """Each row of a [R, N] boolean map -> ascending column indices, unused slots = N, plus the
    per-row count; both int32.  Follows python/spattn/mask_utils.py:152-167."""
    bm = np.asarray(torch.as_tensor(boolean_mask).to(torch.bool).cpu().numpy())
    R, N = bm.shape
    idx = np.full((R, N), N, dtype=np.int32)
    cnt = bm.sum(axis=1).astype(np.int32)
    for r in range(R):
        nz = np.flatnonzero(bm[r]).astype(np.int32)
        idx[r, :nz.size] = nz
    return torch.from_numpy(idx), torch.from_numpy(cnt)


def bitmask_to_indexmask(booleanmask) -> Tuple[torch.Tensor, torch.Tensor]:
    """[B, H, R, N] boolean (or int, > 0 = keep) map -> index lists + counts.
    Follows python/spattn/mask_utils.py:272-289."""
    bm = torch.as_tensor(booleanmask)
    bm = (bm > 0) if bm.dtype != torch.bool else bm
    B, H, R, N = bm.shape
    idx = torch.empty(B, H, R, N, dtype=torch.int32)
    cnt = torch.empty(B, H, R, dtype=torch.int32)
    for b in range(B):
        for h in range(H):
            idx[b, h], cnt[b, h] = boolean_to_index_mask_2d(bm[b, h])
    return idx, cnt


def pack_mask(mask) -> np.ndarray:
    """[..., W] map (bool, or numeric with > 0 = keep; W % 8 == 0) -> uint8 [..., W/8]: entry e of a
    row sits in byte e // 8 at bit e % 8 (sum of bit * 2^(e % 8) over groups of eight).
    Follows python/spattn/mask_utils.py:421-430."""
    m = np.asarray(torch.as_tensor(mask).cpu().numpy())
    m = m if m.dtype == np.bool_ else (m > 0)
    assert m.shape[-1] % 8 == 0
    g = m.reshape(*m.shape[:-1], m.shape[-1] // 8, 8).astype(np.uint16)
    w = np.array([1, 2, 4, 8, 16, 32, 64, 128], dtype=np.uint16)
    return (g * w).sum(axis=-1).astype(np.uint8)


def unpack_mask(packed) -> np.ndarray:
    """uint8 [..., W8] -> bool [..., 8 * W8]; inverse of pack_mask.
    Follows python/spattn/mask_utils.py:433-440."""
    p = np.asarray(torch.as_tensor(packed).cpu().numpy()).astype(np.uint8)
    w = np.array([1, 2, 4, 8, 16, 32, 64, 128], dtype=np.uint8)
    bits = (p[..., None] & w) != 0
    return bits.reshape(*p.shape[:-1], p.shape[-1] * 8)


def packedmask_to_indexmask(packed, n_valid: Optional[int] = None, stride: Optional[int] = None,
                            sentinel: Optional[int] = None) -> Tuple[np.ndarray, np.ndarray]:
    """What a compressed mask cache hands back (python/spattn/mask_utils.py:89-93: unpack, then the
    row compaction of :152-167): ascending positions < n_valid of the set bits of every row, unused
    slots = sentinel (default: the list stride, default: the row width), counts; both int32."""
    bits = unpack_mask(packed)
    W = bits.shape[-1]
    n_valid = W if n_valid is None else min(n_valid, W)
    stride = W if stride is None else stride
    sentinel = stride if sentinel is None else sentinel
    rows = bits.reshape(-1, W)
    idx = np.full((rows.shape[0], stride), sentinel, dtype=np.int32)
    cnt = np.zeros(rows.shape[0], dtype=np.int32)
    for r in range(rows.shape[0]):
        nz = np.flatnonzero(rows[r, :n_valid]).astype(np.int32)
        cnt[r] = nz.size
        idx[r, :min(nz.size, stride)] = nz[:stride]
    return idx.reshape(*bits.shape[:-1], stride), cnt.reshape(bits.shape[:-1])


def indexmask_to_packedmask(indices, num_indices, width: int) -> np.ndarray:
    """Index lists + counts -> packed rows of ceil(width / 32) * 4 bytes: bit e set iff e < width is
    among the first num_indices entries of the row (inverse of packedmask_to_indexmask)."""
    idx = np.asarray(torch.as_tensor(indices).cpu().numpy())
    cnt = np.asarray(torch.as_tensor(num_indices).cpu().numpy()).reshape(-1)
    rows = idx.reshape(-1, idx.shape[-1])
    Wp = 32 * ((width + 31) // 32)
    bits = np.zeros((rows.shape[0], Wp), dtype=bool)
    for r in range(rows.shape[0]):
        e = rows[r, :min(int(cnt[r]), rows.shape[1])]
        e = e[(e >= 0) & (e < width)]
        bits[r, e] = True
    return pack_mask(bits).reshape(*idx.shape[:-1], Wp // 8)


def topk_scores(q, k, blocksz: int = 128, kv_seq_len: Optional[int] = None,
                scale: Optional[float] = None) -> torch.Tensor:
    """[B, H, ceil(S/blocksz), n_kv] fp32: mean of each block of query rows (the last block may be
    shorter), times scale, dotted with every key.  Follows python/spattn/mask_utils.py:390-411."""
    q, k = _f32(q), _f32(k)
    B, H, S, D = q.shape
    n_kv = k.shape[2] if kv_seq_len is None else kv_seq_len
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    nblk = (S + blocksz - 1) // blocksz
    qmean = torch.stack([q[:, :, i * blocksz:min(S, (i + 1) * blocksz)].mean(dim=2) for i in range(nblk)], dim=2)
    return torch.einsum("bhmd,bhnd->bhmn", qmean * scale, k[:, :, :n_kv])


def topk_indices(q, k, select_k: int, blocksz: int = 128, kv_seq_len: Optional[int] = None,
                 scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """The select_k keys with the largest topk_scores per query block, descending (equal scores:
    smaller index first), int32, and counts = select_k.  Follows python/spattn/mask_utils.py:412-417."""
    sc = topk_scores(q, k, blocksz, kv_seq_len, scale)
    order = torch.sort(sc, dim=-1, descending=True, stable=True).indices[..., :select_k]
    cnt = torch.full(sc.shape[:3], select_k, dtype=torch.int32)
    return order.to(torch.int32), cnt


def allindex_mask(B: int, H: int, max_stride: int, S: int, block: int):
    """Identity key lists: every key kept, in order.  Follows python/spattn/mask_utils.py:175-180
    and include/utils.cuh:73-93 (the all_index_mask operator)."""
    nb = (S + block - 1) // block
    cnt = torch.full((B, H, nb), S, dtype=torch.int32)
    idx = torch.arange(max_stride, dtype=torch.int32).expand(B, H, nb, max_stride).contiguous()
    return idx, cnt


# ------------------------------------------------------------------------------------------------
# threshold masks
# ------------------------------------------------------------------------------------------------
def _head_probs_rows(qh, kh, r0, r1, scale):
    return torch.softmax((qh[r0:r1] @ kh.T) * scale, dim=-1)


def qk_bitmask(q, k, thresh: float = 0.001, blocksz: int = 128, kv_seq_len: Optional[int] = None,
               scale: Optional[float] = None) -> torch.Tensor:
    """bool [B, H, ceil(S/blocksz), N]: key TOKEN j kept for a query block iff any of the block's
    rows has softmax probability > thresh (strict).  Follows python/spattn/mask_utils.py:206-222."""
    q, k = _f32(q), _f32(k)
    B, H, S, D = q.shape
    n_kv = k.shape[2] if kv_seq_len is None else kv_seq_len
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    nqb = (S + blocksz - 1) // blocksz
    out = torch.zeros(B, H, nqb, n_kv, dtype=torch.bool)
    for b in range(B):
        for h in range(H):
            kh = k[b, h, :n_kv]
            for r0, r1 in _row_chunks(S, blocksz):
                p = _head_probs_rows(q[b, h], kh, r0, r1, scale)
                out[b, h, r0 // blocksz:(r1 + blocksz - 1) // blocksz] = attnmapor(p > thresh, blocksz)
    return out


def qk_token_pmax(q, k, blocksz: int = 128, kv_seq_len: Optional[int] = None,
                  scale: Optional[float] = None) -> torch.Tensor:
    """fp32 [B, H, ceil(S/blocksz), N]: for each query block and key token the largest softmax
    probability over the block's rows (attnmapor of the float map, python/spattn/mask_utils.py:126-142);
    qk_bitmask is this map compared with the threshold."""
    q, k = _f32(q), _f32(k)
    B, H, S, D = q.shape
    n_kv = k.shape[2] if kv_seq_len is None else kv_seq_len
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    nqb = (S + blocksz - 1) // blocksz
    out = torch.zeros(B, H, nqb, n_kv, dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            kh = k[b, h, :n_kv]
            for r0, r1 in _row_chunks(S, blocksz):
                p = _head_probs_rows(q[b, h], kh, r0, r1, scale)
                out[b, h, r0 // blocksz:(r1 + blocksz - 1) // blocksz] = attnmapor(p, blocksz)
    return out


def qk_indexmask(q, k, thresh: float = 0.001, blocksz: int = 128, kv_seq_len: Optional[int] = None,
                 scale: Optional[float] = None):
    """Token index lists + counts.  Follows python/spattn/mask_utils.py:225-245."""
    return bitmask_to_indexmask(qk_bitmask(q, k, thresh, blocksz, kv_seq_len, scale))


def qk_block_pmax(q, k, bq: int = 64, bk: int = 64, kv_seq_len: Optional[int] = None,
                  scale: Optional[float] = None) -> torch.Tensor:
    """fp32 [B, H, nqb, nkb]: the largest softmax probability inside each (query block, key block).
    This is the 'score' that the threshold is compared with; a block is kept iff score > tau, which
    equals attnmapor over the block's rows (python/spattn/mask_utils.py:126-142, :218) followed by
    an OR over each group of bk key columns."""
    q, k = _f32(q), _f32(k)
    B, H, S, D = q.shape
    n_kv = k.shape[2] if kv_seq_len is None else kv_seq_len
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    nqb, nkb = (S + bq - 1) // bq, (n_kv + bk - 1) // bk
    out = torch.zeros(B, H, nqb, nkb, dtype=torch.float32)
    pad = nkb * bk - n_kv
    for b in range(B):
        for h in range(H):
            kh = k[b, h, :n_kv]
            for r0, r1 in _row_chunks(S, bq):
                p = _head_probs_rows(q[b, h], kh, r0, r1, scale)
                colmax = attnmapor(p, bq)                                  # [blocks, n_kv]
                if pad:
                    colmax = torch.nn.functional.pad(colmax, (0, pad), value=0.0)
                out[b, h, r0 // bq:(r1 + bq - 1) // bq] = colmax.view(colmax.shape[0], nkb, bk).max(dim=-1).values
    return out


def qk_block_bitmask(q, k, thresh: float, bq: int = 64, bk: int = 64, kv_seq_len=None, scale=None):
    """bool [B, H, nqb, nkb], strict '>' as in python/spattn/mask_utils.py:218,238."""
    return qk_block_pmax(q, k, bq, bk, kv_seq_len, scale) > thresh


def qk_block_indexmask(q, k, thresh: float, bq: int = 64, bk: int = 64, kv_seq_len=None, scale=None):
    """Per-query-block ascending key-BLOCK lists (fill = number of key blocks) and counts; the
    list format of python/spattn/mask_utils.py:152-167 applied to the block map."""
    return bitmask_to_indexmask(qk_block_bitmask(q, k, thresh, bq, bk, kv_seq_len, scale))


def near_threshold(pmax: torch.Tensor, thresh: float, rel: float = 1e-3) -> torch.Tensor:
    """Blocks whose score lies within rel*tau of tau: exempt from the bit-exactness requirement."""
    return (pmax - thresh).abs() <= rel * thresh


# ------------------------------------------------------------------------------------------------
# masked / sparse attention
# ------------------------------------------------------------------------------------------------
def qkattn_masked(q, k, v, thresh: float, blocksz: int = 128, scale: Optional[float] = None) -> torch.Tensor:
    """Full-softmax probabilities, zeroed outside the kept (query block x key token) set, times v;
    NO renormalisation.  Follows python/test_mask.py:37-54 (which hard-codes 1/sqrt(128) at :5-6;
    here the scale is 1/sqrt(D) unless given)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, H, S, D = q.shape
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    o = torch.empty(B, H, S, v.shape[3], dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            for r0, r1 in _row_chunks(S, blocksz):
                p = _head_probs_rows(q[b, h], k[b, h], r0, r1, scale)
                keep = attnmapor(p > thresh, blocksz)                      # [blocks, N]
                keep_rows = keep.repeat_interleave(blocksz, dim=0)[: r1 - r0]
                o[b, h, r0:r1] = (p * keep_rows) @ v[b, h]
    return o


def block_masked_attn(q, k, v, block_mask, bq: int = 64, bk: int = 64, kv_seq_len=None,
                      scale: Optional[float] = None) -> torch.Tensor:
    """python/test_mask.py:37-54 with a given [B, H, nqb, nkb] block map: probabilities come from
    the softmax over ALL keys (precomputed m, l in the CUDA path), dropped blocks contribute 0."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, H, S, D = q.shape
    n_kv = k.shape[2] if kv_seq_len is None else kv_seq_len
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    bm = torch.as_tensor(block_mask).to(torch.bool).cpu()
    o = torch.empty(B, H, S, v.shape[3], dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            kh, vh = k[b, h, :n_kv], v[b, h, :n_kv]
            for r0, r1 in _row_chunks(S, bq):
                p = _head_probs_rows(q[b, h], kh, r0, r1, scale)
                keep = bm[b, h, r0 // bq:(r1 + bq - 1) // bq]              # [blocks, nkb]
                keep = keep.repeat_interleave(bk, dim=1)[:, :n_kv].repeat_interleave(bq, dim=0)[: r1 - r0]
                o[b, h, r0:r1] = (p * keep) @ vh
    return o


def sp_attn_tokens(q, k, v, kv_indices, kv_num_indices, blocksz: int = 128,
                   scale: Optional[float] = None) -> torch.Tensor:
    """The sp_attn operator: for each query block, softmax restricted to (renormalised over) the
    listed key tokens, times the listed v rows.  Follows
    include/sparseattn_asyncgatherload_padded.cuh:198-249 (online softmax over gathered keys only)
    and the identity-list test test/test_sparseattn_asyncgatherload_padded.cu:37-62."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, H, S, D = q.shape
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    idx = torch.as_tensor(kv_indices).cpu().long()
    cnt = torch.as_tensor(kv_num_indices).cpu().long()
    o = torch.zeros(B, H, S, v.shape[3], dtype=torch.float32)
    nqb = (S + blocksz - 1) // blocksz
    for b in range(B):
        for h in range(H):
            for qb in range(nqb):
                n = int(cnt[b, h, qb])
                sel = idx[b, h, qb, :n]
                sel = sel[sel < k.shape[2]]
                r0, r1 = qb * blocksz, min(S, (qb + 1) * blocksz)
                if sel.numel() == 0:
                    continue
                p = torch.softmax((q[b, h, r0:r1] @ k[b, h, sel].T) * scale, dim=-1)
                o[b, h, r0:r1] = p @ v[b, h, sel]
    return o


def sp_attn_blocks(q, k, v, kb_indices, kb_counts, bq: int = 64, bk: int = 64, kv_seq_len=None,
                   scale: Optional[float] = None) -> torch.Tensor:
    """Renormalising sparse attention over key-BLOCK lists (same semantics as sp_attn_tokens with
    every token of each listed block kept)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, H, S, D = q.shape
    n_kv = k.shape[2] if kv_seq_len is None else kv_seq_len
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    idx = torch.as_tensor(kb_indices).cpu().long()
    cnt = torch.as_tensor(kb_counts).cpu().long()
    o = torch.zeros(B, H, S, v.shape[3], dtype=torch.float32)
    nqb = (S + bq - 1) // bq
    ar = torch.arange(bk)
    for b in range(B):
        for h in range(H):
            for qb in range(nqb):
                n = int(cnt[b, h, qb])
                if n == 0:
                    continue
                sel = (idx[b, h, qb, :n, None] * bk + ar[None, :]).reshape(-1)
                sel = sel[sel < n_kv]
                r0, r1 = qb * bq, min(S, (qb + 1) * bq)
                p = torch.softmax((q[b, h, r0:r1] @ k[b, h, sel].T) * scale, dim=-1)
                o[b, h, r0:r1] = p @ v[b, h, sel]
    return o
