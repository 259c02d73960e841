"""The decode-attention entry point that allocates nothing (csrc/attention_noalloc.h).

Some hosts of a kernel library may not allocate device memory once they are running: a
serving process that has pinned its whole budget at start-up, or a plug-in thread that is
kept away from the allocator.  For them the library exports ``mi_attention_decode_noalloc``,
which keeps the scratch of the split-key merge in a static device array instead of asking the
caller for it.  This test calls that exported C symbol directly, several times in a row on
different inputs (the array keeps the previous call's contents), and compares it both with the
regular entry point and with the plain float64 attention of ``plain_impl``.  The cases include
counts of arrival counters that are odd (the scratch behind them must stay aligned for the
8-byte loads of the merge), a window, and a request that holds no key at all.
It lives in a file that is collected last, so a run that stops at the first failure has
already run everything else.
"""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

import plain_impl as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BOUND = 1 / 64      # the tolerance of the attention kernel tests (two bfloat16 roundings)


def paged_case(kv_lens, nq, nkv, d, page, seed):
    """Random keys and values of several requests on shuffled pages (never-written slots hold
    NaN), one query token each; returns device tensors and the per-request keys and values."""
    from mini_infer_b200.csrc import ops

    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-L // page) for L in kv_lens) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    kc = torch.full((n_pages * page, nkv, d), float("nan"), dtype=torch.bfloat16)
    vc = torch.full((n_pages * page, nkv, d), float("nan"), dtype=torch.bfloat16)
    tables, ks, vs = [], [], []
    for L in kv_lens:
        k = torch.randn(L, nkv, d, generator=g).to(torch.bfloat16)
        v = torch.randn(L, nkv, d, generator=g).to(torch.bfloat16)
        t = [perm.pop() for _ in range(-(-L // page))]
        for p in range(L):
            kc[t[p // page] * page + p % page] = k[p]
            vc[t[p // page] * page + p % page] = v[p]
        tables.append(t)
        ks.append(k)
        vs.append(v)
    width = max(1, max(len(t) for t in tables))
    bt = torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32)
    B = len(kv_lens)
    q = torch.randn(B, nq, d, generator=g).to(torch.bfloat16)
    qkv = torch.zeros(B, (nq + 2 * nkv) * d, dtype=torch.bfloat16)
    qkv[:, : nq * d] = q.view(B, nq * d)
    return dict(
        qkv=qkv.to(DEV), kc=ops.pack_cache_pages(kc, page).to(DEV), vc=ops.pack_cache_pages(vc, page).to(DEV),
        bt=bt.to(DEV), q_start=torch.arange(B, dtype=torch.int32, device=DEV),
        kv_len=torch.tensor(kv_lens, dtype=torch.int32, device=DEV), B=B, q=q, ks=ks, vs=vs, kv_lens=kv_lens,
    )


def plain(case, nq, d, window):
    want = torch.zeros(case["B"], nq, d, dtype=torch.float64)
    for i, L in enumerate(case["kv_lens"]):
        if L == 0:
            continue                                     # no key: the kernel writes zeros
        want[i:i + 1] = P.causal_attention(case["q"][i:i + 1].double(), case["ks"][i].double(),
                                           case["vs"][i].double(), 1.0 / math.sqrt(d), window or None,
                                           q_offset=L - 1)
    return want.view(case["B"], nq * d)


def test_no_alloc_entry_point_matches_the_regular_one_and_the_plain_attention():
    from mini_infer_b200.csrc import build, ops

    lib = build.library("attention_mma")
    fn = lib.mi_attention_decode_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                   c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
    page = 16
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)

    def check(kv_lens, nq, nkv, d, n_splits, seed, window=0, regular=True):
        case = paged_case(kv_lens, nq, nkv, d, page, seed)
        scale = 1.0 / math.sqrt(d)
        got = torch.full((case["B"], nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        # `got` is allocated here, by the caller: the entry point receives pointers only
        rc = fn(case["qkv"].data_ptr(), case["qkv"].stride(0), got.data_ptr(), got.stride(0),
                case["kc"].data_ptr(), case["vc"].data_ptr(), case["bt"].data_ptr(), case["bt"].stride(0), page,
                case["q_start"].data_ptr(), case["kv_len"].data_ptr(), case["B"], nq, nkv, d, scale, window,
                n_splits, stream)
        assert rc == 0, lib.mi_error_message().decode()
        torch.cuda.synchronize()
        assert ops.attention_wait_status() == 0
        got = got.double().cpu()
        assert torch.isfinite(got).all()
        want = plain(case, nq, d, window)
        assert (got - want).abs().max().item() <= BOUND, (kv_lens, nq, nkv, d, n_splits, window)
        if regular:
            ref = torch.full((case["B"], nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
            ops.attention_decode(case["qkv"], case["qkv"].stride(0), ref, case["kc"], case["vc"], case["bt"], page,
                                 case["q_start"], case["kv_len"], case["B"], nq, nkv, d, scale, window, n_splits)
            torch.cuda.synchronize()
            assert (got - ref.double().cpu()).abs().max().item() <= BOUND

    # calls in a row share the static array; lengths, head counts and slice counts change
    check([700, 64, 1, 333], 12, 4, 64, n_splits=3, seed=1)          # 16 arrival counters
    check([65, 900, 129], 12, 4, 64, n_splits=7, seed=2)             # 12
    # odd numbers of arrival counters: 1, 3 and 3
    check([300], 8, 1, 64, n_splits=2, seed=3)
    check([200, 77, 513], 4, 1, 32, n_splits=5, seed=4)
    check([1000], 24, 3, 128, n_splits=9, seed=5)
    # a window, with slices that end up empty for the short request
    check([500, 64, 7], 8, 1, 64, n_splits=4, seed=6, window=100)
    # one slice (no scratch is touched), and a request without any key among normal ones
    check([130, 0, 17], 6, 3, 48, n_splits=1, seed=7)
    check([130, 0, 400], 6, 3, 48, n_splits=3, seed=8)

    # a call that would not fit the built-in array is refused with a message, nothing is launched
    case = paged_case([16], 12, 4, 64, page, seed=9)
    out = torch.zeros(1, 12 * 64, dtype=torch.bfloat16, device=DEV)
    rc = fn(case["qkv"].data_ptr(), case["qkv"].stride(0), out.data_ptr(), out.stride(0), case["kc"].data_ptr(),
            case["vc"].data_ptr(), case["bt"].data_ptr(), case["bt"].stride(0), page, case["q_start"].data_ptr(),
            case["kv_len"].data_ptr(), 60000, 12, 4, 64, 0.125, 0, 64, stream)
    assert rc != 0 and "scratch" in lib.mi_error_message().decode()


def test_regular_entry_point_refuses_misaligned_scratch():
    """The merge reads (max, sum) pairs with one 8-byte load: scratch that is only 4-byte
    aligned is refused on the host, nothing is launched."""
    from mini_infer_b200.csrc import build

    lib = build.library("attention_mma")
    fn = lib.mi_attention_decode
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                   c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p,
                   c_void_p]
    nq, nkv, d, page = 4, 1, 32, 16
    case = paged_case([100], nq, nkv, d, page, seed=10)
    out = torch.zeros(1, nq * d, dtype=torch.bfloat16, device=DEV)
    scratch = torch.zeros(4096, dtype=torch.float32, device=DEV)
    counters = torch.zeros(16, dtype=torch.int32, device=DEV)
    rc = fn(case["qkv"].data_ptr(), case["qkv"].stride(0), out.data_ptr(), out.stride(0), case["kc"].data_ptr(),
            case["vc"].data_ptr(), case["bt"].data_ptr(), case["bt"].stride(0), page, case["q_start"].data_ptr(),
            case["kv_len"].data_ptr(), 1, nq, nkv, d, 0.2, 0, 2,
            scratch.data_ptr(), scratch.data_ptr() + 4 * (1 * nq * 2 * d + 1), counters.data_ptr(),
            c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0 and "aligned" in lib.mi_error_message().decode()
    torch.cuda.synchronize()
