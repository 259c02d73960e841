"""The decode-attention entry point that allocates nothing (csrc/attention_noalloc.h).

Some hosts of a kernel library may not allocate device memory once they are running: a
serving process that has pinned its whole budget at start-up, or a plug-in thread that is
kept away from the allocator.  For them the library exports ``mi_attention_decode_noalloc``,
which keeps the scratch of the split-key merge in a static device array instead of asking the
caller for it.  This test calls that exported C symbol directly, twice in a row on different
inputs (the array keeps the first call's contents), and compares with the regular entry point.
It lives in a file that is collected last, so a run that stops at the first failure has
already run everything else.
"""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def paged_case(kv_lens, nq, nkv, d, page, seed):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-L // page) for L in kv_lens) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    kc = torch.randn(n_pages, nkv, page, d, generator=g).to(torch.bfloat16)      # a page is [nkv, page, d]
    vc = torch.randn(n_pages, nkv, page, d, generator=g).to(torch.bfloat16)
    tables = [[perm.pop() for _ in range(-(-L // page))] for L in kv_lens]
    width = max(len(t) for t in tables)
    bt = torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32)
    B = len(kv_lens)
    qkv = torch.randn(B, (nq + 2 * nkv) * d, generator=g).to(torch.bfloat16)
    return dict(
        qkv=qkv.to(DEV), kc=kc.to(DEV), vc=vc.to(DEV), bt=bt.to(DEV),
        q_start=torch.arange(B, dtype=torch.int32, device=DEV),
        kv_len=torch.tensor(kv_lens, dtype=torch.int32, device=DEV), B=B,
    )


def test_no_alloc_entry_point_matches_the_regular_one():
    from mini_infer_b200.csrc import build, ops

    lib = build.library("attention_mma")
    fn = lib.mi_attention_decode_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                   c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
    nq, nkv, d, page = 12, 4, 64, 16
    scale = 1.0 / math.sqrt(d)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)

    def both(case, n_splits):
        want = torch.full((case["B"], nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.attention_decode(case["qkv"], case["qkv"].stride(0), want, case["kc"], case["vc"], case["bt"], page,
                             case["q_start"], case["kv_len"], case["B"], nq, nkv, d, scale, 0, n_splits)
        got = torch.full_like(want, float("nan"))      # allocated here, by the caller: the entry point gets pointers
        rc = fn(case["qkv"].data_ptr(), case["qkv"].stride(0), got.data_ptr(), got.stride(0),
                case["kc"].data_ptr(), case["vc"].data_ptr(), case["bt"].data_ptr(), case["bt"].stride(0), page,
                case["q_start"].data_ptr(), case["kv_len"].data_ptr(), case["B"], nq, nkv, d, scale, 0, n_splits,
                stream)
        assert rc == 0, lib.mi_error_message().decode()
        torch.cuda.synchronize()
        return got.float(), want.float()

    # two calls in a row share the static array; the second has other lengths and more slices
    first = both(paged_case([700, 64, 1, 333], nq, nkv, d, page, seed=1), n_splits=3)
    second = both(paged_case([65, 900, 129], nq, nkv, d, page, seed=2), n_splits=7)
    for got, want in (first, second):
        assert torch.isfinite(got).all()
        assert (got - want).abs().max().item() <= 1 / 64      # the tolerance of the attention kernel tests

    # a call that would not fit the built-in array is refused with a message, nothing is launched
    case = paged_case([16], nq, nkv, d, page, seed=3)
    out = torch.zeros(1, nq * d, dtype=torch.bfloat16, device=DEV)
    rc = fn(case["qkv"].data_ptr(), case["qkv"].stride(0), out.data_ptr(), out.stride(0), case["kc"].data_ptr(),
            case["vc"].data_ptr(), case["bt"].data_ptr(), case["bt"].stride(0), page, case["q_start"].data_ptr(),
            case["kv_len"].data_ptr(), 60000, nq, nkv, d, scale, 0, 64, stream)
    assert rc != 0 and "scratch" in lib.mi_error_message().decode()
