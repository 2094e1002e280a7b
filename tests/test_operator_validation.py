"""Shape and dtype validation of the torch operators, on meta tensors (no GPU needed): the Meta
kernel of every operator is the same check that its CUDA kernel runs first, so a wrong-shaped tensor
is an error before anything reaches the device."""
import pytest
import torch

import fgattn_tk_cuda_b200.spattn  # noqa: F401  (registers torch.ops.cuda_attn)

ops = torch.ops.cuda_attn
B, H, S, D, SKV = 2, 3, 300, 64, 200
NQB, NKB, NQB128, SPAD = 5, 4, 3, 384


def t(*shape, dtype=torch.bfloat16):
    return torch.empty(*shape, dtype=dtype, device="meta")


def good():
    return dict(q=t(B, H, S, D), k=t(B, H, SKV, D), v=t(B, H, SKV, D), o=t(B, H, S, D),
                m=t(B, H, 1, SPAD, dtype=torch.float32), l=t(B, H, 1, SPAD, dtype=torch.float32),
                kb=t(B, H, NQB, NKB, dtype=torch.int32), kc=t(B, H, NQB, dtype=torch.int32),
                ti=t(B, H, NQB128, 256, dtype=torch.int32), tc=t(B, H, NQB128, dtype=torch.int32),
                mask=t(B, H, NQB128, 256, dtype=torch.int32), scratch=t(1024, dtype=torch.float32))


CALLS = {
    "full_attn": lambda a: ops.full_attn(a["o"], a["q"], a["k"], a["v"]),
    "fullattn_maxq_denom": lambda a: ops.fullattn_maxq_denom(a["o"], a["m"], a["l"], a["q"], a["k"], a["v"]),
    "maxq_denom": lambda a: ops.maxq_denom(a["m"], a["l"], a["q"], a["k"]),
    "sp_attn": lambda a: ops.sp_attn(a["o"], a["q"], a["k"], a["v"], a["ti"], a["tc"]),
    "booleanmask_128": lambda a: ops.booleanmask_128(a["mask"], a["m"], a["l"], a["q"], a["k"], 1e-3),
    "booleanmask_128_listed": lambda a: ops.booleanmask_128_listed(a["mask"], a["m"], a["l"], a["q"], a["k"], 1e-3,
                                                                   a["kb"], a["kc"]),
    "booleanmask_to_indexmask": lambda a: ops.booleanmask_to_indexmask(a["ti"], a["tc"], a["mask"], SKV),
    "block_index_lists": lambda a: ops.block_index_lists(a["kb"], a["kc"], a["m"], a["l"], a["o"], a["q"], a["k"],
                                                         a["v"], 1e-3, a["scratch"]),
    "sp_attn_blocks_ml": lambda a: ops.sp_attn_blocks_ml(a["o"], a["q"], a["k"], a["v"], a["kb"], a["kc"], a["m"], a["l"]),
    "sp_attn_blocks": lambda a: ops.sp_attn_blocks(a["o"], a["q"], a["k"], a["v"], a["kb"], a["kc"]),
    "sp_attn_blocks_hint": lambda a: ops.sp_attn_blocks_hint(a["o"], a["q"], a["k"], a["v"], a["kb"], a["kc"], a["m"]),
}

# (operators that take the tensor, replacement that must be refused)
BAD = [
    ("k", t(B, H + 1, SKV, D), None),                             # heads differ from q
    ("k", t(B, H, SKV, 128), None),                               # head dimension differs from q
    ("k", t(B, H, SKV, D, dtype=torch.float16), None),            # dtype
    ("v", t(B, H, SKV - 8, D), None),                             # fewer rows than k
    ("o", t(B, H, S - 1, D), None),                               # not the shape of q
    ("m", t(B, H, 1, S, dtype=torch.float32), None),              # [B,H,1,S] instead of the padded length
    ("l", t(B, H, 1, SPAD, dtype=torch.float16), None),           # dtype
    ("kb", t(B, H, NQB - 1, NKB, dtype=torch.int32), None),       # rows != ceil(S/64)
    ("kb", t(B, H, NQB, NKB - 1, dtype=torch.int32), None),       # stride < number of key blocks
    ("kc", t(B, H, NQB - 1, dtype=torch.int32), None),
    ("ti", t(B, H, NQB128 + 1, 256, dtype=torch.int32), None),    # rows != ceil(S/128)
    ("tc", t(B, H, NQB128 + 2, dtype=torch.int32), None),
    ("mask", t(B, H, NQB128, SKV - 8, dtype=torch.int32), None),  # narrower than the key sequence
    ("mask", t(B, H - 1, NQB128, 256, dtype=torch.int32), None),
]
USES = {
    "full_attn": "qkvo", "fullattn_maxq_denom": ("q", "k", "v", "o", "m", "l"), "maxq_denom": ("q", "k", "m", "l"),
    "sp_attn": ("q", "k", "v", "o", "ti", "tc"), "booleanmask_128": ("q", "k", "m", "l", "mask"),
    "booleanmask_128_listed": ("q", "k", "m", "l", "mask", "kb", "kc"),
    "booleanmask_to_indexmask": ("ti", "tc", "mask"),
    "block_index_lists": ("q", "k", "v", "o", "m", "l", "kb", "kc"),
    "sp_attn_blocks_ml": ("q", "k", "v", "o", "m", "l", "kb", "kc"),
    "sp_attn_blocks": ("q", "k", "v", "o", "kb", "kc"), "sp_attn_blocks_hint": ("q", "k", "v", "o", "m", "kb", "kc"),
}


@pytest.mark.parametrize("name", sorted(CALLS))
def test_well_formed_arguments_pass(name):
    assert CALLS[name](good()) is None


@pytest.mark.parametrize("name", sorted(CALLS))
def test_every_wrong_shape_is_refused(name):
    n = 0
    for key, bad, _ in BAD:
        if key not in USES[name]:
            continue
        if name == "booleanmask_to_indexmask" and key == "mask":
            continue                                  # there the mask defines the shapes; covered below
        args = good()
        args[key] = bad
        with pytest.raises(RuntimeError):
            CALLS[name](args)
        n += 1
    assert n >= 2


def test_compaction_and_packed_mask_shapes():
    a = good()
    with pytest.raises(RuntimeError):
        ops.booleanmask_to_indexmask(t(B, H, NQB128, 128, dtype=torch.int32), a["tc"], a["mask"], SKV)
    with pytest.raises(RuntimeError):
        ops.pack_mask(t(B, 5, dtype=torch.uint8), t(B, 48, dtype=torch.int32))
    assert ops.pack_mask(t(B, 6, dtype=torch.uint8), t(B, 48, dtype=torch.int32)) is None
    with pytest.raises(RuntimeError):
        ops.all_index_mask(a["ti"], a["tc"], B, H, NQB128 + 1, S)
    with pytest.raises(RuntimeError):
        ops.topk_indices(t(B, H, NQB128, 64, dtype=torch.int32), a["tc"], a["q"], a["k"], 100, 128)   # stride < select_k
    assert ops.topk_indices(t(B, H, NQB128, 128, dtype=torch.int32), a["tc"], a["q"], a["k"], 100, 128) is None


def test_noalloc_wrapper_refuses_k_of_another_length():
    """fgattn_block_index_lists_noalloc has no kv_rows argument: the Python layer must not let a k / v of
    another length through (it would be read past its end, or at the wrong per-head stride)."""
    from fgattn_tk_cuda_b200 import capi
    q = torch.zeros(1, 1, 128, 64, dtype=torch.bfloat16)
    k_short = torch.zeros(1, 1, 64, 64, dtype=torch.bfloat16)
    i32 = torch.zeros(1, 1, 2, 2, dtype=torch.int32)
    f32 = torch.zeros(1, 1, 1, 128)
    with pytest.raises(capi.FgattnError, match="shape of q"):
        capi.block_index_lists_noalloc(i32, i32, f32, f32, q, k_short, 1e-3)
    with pytest.raises(capi.FgattnError, match="shape of q"):
        capi.block_index_lists_noalloc(i32, i32, f32, f32, q, q, 1e-3, o=q, v=k_short)
