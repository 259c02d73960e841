"""Each CUDA kernel alone against its plain reference, at sizes other than the engine's."""

import math

import numpy as np
import pytest
import torch

import plain_impl as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from mini_infer_b200.csrc import ops as _ops

    return _ops


def tol(dtype, fp32=2e-6, bf16=1.0 / 128):
    """Relative bound: a few fp32 roundings, or one bf16 rounding (2^-8) with margin."""
    return fp32 if dtype == torch.float32 else bf16


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


# ----------------------------------------------------------------------------- embedding


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [40, 96, 1030])
def test_embedding(dtype, H):
    table = rnd(77, H, dtype=dtype).to(DEV)
    ids = torch.tensor([0, 76, 5, 5, 33], dtype=torch.int32, device=DEV)
    out = ops().embedding(table, ids)
    assert torch.equal(out, table[ids.long()])


def test_embedding_bad_id_is_loud():
    table = rnd(10, 16).to(DEV)
    out = ops().embedding(table, torch.tensor([3, 10], dtype=torch.int32, device=DEV))
    assert torch.equal(out[0], table[3]) and torch.isnan(out[1]).all()


# ----------------------------------------------------------------------------- rms norm


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,H", [(5, 100), (3, 4096), (2, 50001), (7, 192)])
def test_add_rmsnorm(dtype, M, H):
    x = rnd(M, H, dtype=dtype, seed=1)
    res = rnd(M, H, seed=2)
    w = (1 + 0.1 * rnd(H, seed=3)).to(dtype)
    eps = 1e-5
    r64 = x.double() + res.double()
    want = P.rms_norm(r64, w.double(), eps)
    res_out = torch.empty(M, H, device=DEV)
    out = ops().add_rmsnorm(x.to(DEV), w.to(DEV), eps, residual_in=res.to(DEV), residual_out=res_out)
    assert torch.allclose(res_out.cpu().double(), r64, rtol=1e-6, atol=1e-6)
    err = (out.cpu().double() - want).abs().max().item()
    assert err <= tol(dtype, fp32=5e-6) * want.abs().max().item()
    # without a residual the stream starts as float(x)
    res_out2 = torch.empty(M, H, device=DEV)
    out2 = ops().add_rmsnorm(x.to(DEV), w.to(DEV), eps, residual_out=res_out2)
    assert torch.equal(res_out2.cpu(), x.float())
    want2 = P.rms_norm(x.double(), w.double(), eps)
    assert (out2.cpu().double() - want2).abs().max().item() <= tol(dtype, fp32=5e-6) * want2.abs().max().item()


def test_add_rmsnorm_rows_and_fp32_gain():
    M, H = 9, 136
    x = rnd(M, H, dtype=torch.bfloat16, seed=4)
    res = rnd(M, H, seed=5)
    w32 = 1 + 0.1 * rnd(H, seed=6)          # a gain stored in 32-bit stays 32-bit
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    out = ops().add_rmsnorm(x.to(DEV), w32.to(DEV), 1e-6, residual_in=res.to(DEV), rows=rows.to(DEV))
    want = P.rms_norm(x.double() + res.double(), w32.double(), 1e-6)[rows.long()]
    assert out.shape == (3, H)
    assert (out.cpu().double() - want).abs().max().item() <= want.abs().max().item() / 128


# ----------------------------------------------------------------------------- rope + store


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot", [(6, 2, 32, 32), (5, 5, 48, 48), (4, 1, 64, 32), (8, 2, 128, 128)])
def test_rope_write(dtype, nq, nkv, d, rot):
    M, n_slots = 11, 40
    qkv = rnd(M, (nq + 2 * nkv) * d, dtype=dtype, seed=7)
    pos = torch.tensor([0, 1, 2, 50, 51, 7, 1000, 30000, 3, 4, 131071], dtype=torch.int32)
    slots = torch.tensor([5, 6, 7, 39, 0, 17, 18, 19, 20, 33, 2], dtype=torch.int32)
    inv = P.rope_inv_freq(rot, 500000.0, None) if rot == d else (
        1.0 / (500000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / d)))
    page = 8                                   # 40 slots = 5 pages of 8; a page is [nkv, page, d]
    kc = torch.zeros(n_slots // page, nkv, page, d, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    buf = qkv.to(DEV).clone()
    ops().rope_write(buf, nq, nkv, d, positions=pos.to(DEV), inv_freq=inv.to(DEV), rotary_dim=rot,
                     slots=slots.to(DEV), kcache=kc, vcache=vc)
    x = qkv.double().view(M, nq + 2 * nkv, d)
    cos, sin = P.rope_cos_sin(pos.tolist(), inv, torch.float64)
    want = x.clone()
    want[:, : nq + nkv, :rot] = P.apply_rope(x[:, : nq + nkv, :rot], cos, sin)
    got = buf.cpu().double().view(M, nq + 2 * nkv, d)
    bound = tol(dtype, fp32=3e-5) * 4.0     # sine/cosine of angles up to 1.3e5 rad in fp32
    assert (got - want).abs().max().item() <= bound
    # the cache holds exactly what the buffer holds, at the given slots, and nothing else
    ks, vs = ops().unpack_cache_pages(kc), ops().unpack_cache_pages(vc)      # [slot, head, d]
    for t in range(M):
        assert torch.equal(ks[slots[t]].cpu(), buf[t].view(nq + 2 * nkv, d)[nq:nq + nkv].cpu())
        assert torch.equal(vs[slots[t]].cpu(), qkv[t].view(nq + 2 * nkv, d)[nq + nkv:])
    untouched = sorted(set(range(n_slots)) - set(slots.tolist()))
    assert ks[untouched].abs().sum().item() == 0 and vs[untouched].abs().sum().item() == 0


def test_rope_write_refuses_bad_rotary_width():
    buf = torch.zeros(2, 4 * 16, device=DEV)
    with pytest.raises(Exception):
        ops().rope_write(buf, 2, 1, 16, positions=torch.zeros(2, dtype=torch.int32, device=DEV),
                         inv_freq=torch.zeros(9, device=DEV), rotary_dim=18)


# ----------------------------------------------------------------------------- silu * up


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,I", [(3, 176), (5, 50), (2, 14336), (4, 33)])
def test_silu_mul(dtype, M, I):
    gu = rnd(M, 2 * I, dtype=dtype, seed=8, scale=3.0)
    gu[0, 0], gu[0, 1] = 60.0, -60.0      # large and tiny gates stay finite
    out = ops().silu_mul(gu.to(DEV))
    g, u = gu.double()[:, :I], gu.double()[:, I:]
    want = P.silu(g) * u
    assert torch.isfinite(out).all()
    assert (out.cpu().double() - want).abs().max().item() <= tol(dtype, fp32=3e-6) * want.abs().max().item()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,I", [(3, 176), (5, 50), (2, 14336), (4, 33)])
def test_silu_mul_pairs(dtype, M, I):
    """The same with gate and up interleaved column by column."""
    gu = rnd(M, 2 * I, dtype=dtype, seed=9, scale=3.0)
    gu[0, 0], gu[0, 2] = 60.0, -60.0
    out = ops().silu_mul(gu.to(DEV), pairs=True)
    g, u = gu.double()[:, 0::2], gu.double()[:, 1::2]
    want = P.silu(g) * u
    assert torch.isfinite(out).all()
    assert (out.cpu().double() - want).abs().max().item() <= tol(dtype, fp32=3e-6) * want.abs().max().item()


@pytest.mark.parametrize("M,I,K", [(1, 64, 64), (8, 7168, 512), (5, 1000, 264), (8, 100, 14336), (16, 513, 1032)])
def test_gemm_tma_gate_up_epilogue(M, I, K):
    """silu(x Wg^T) * (x Wu^T) from one kernel, rows of W alternating gate and up, against a
    float64 product; sizes whose tiles are cut across blocks (partial tiles are summed before
    the activation) and whose last tile is ragged."""
    x = rnd(M, K, dtype=torch.bfloat16, seed=40)
    wg = rnd(I, K, dtype=torch.bfloat16, seed=41, scale=0.1)
    wu = rnd(I, K, dtype=torch.bfloat16, seed=42, scale=0.1)
    w = torch.stack([wg, wu], dim=1).reshape(2 * I, K).contiguous()
    out = ops().gemm_tma(x.to(DEV), w.to(DEV), torch.bfloat16, swiglu=True)
    want = P.silu(x.double() @ wg.double().T) * (x.double() @ wu.double().T)
    assert out.shape == (M, I)
    assert (out.cpu().double() - want).abs().max().item() <= 1 / 128 * max(1.0, want.abs().max().item())
    assert ops().gemm_tma_status() == 0
    # the unfused route (library product, then the activation on the interleaved result) agrees
    big = ops().silu_mul(ops().linear(rnd(40, K, dtype=torch.bfloat16, seed=43).to(DEV), w.to(DEV)), pairs=True)
    assert big.shape == (40, I)


# ----------------------------------------------------------------------------- fp32 product


@pytest.mark.parametrize("M,N,K", [(1, 300, 77), (17, 130, 64), (200, 190, 1000), (64, 512, 176), (3, 5, 2)])
def test_gemm_f32(M, N, K):
    a, w = rnd(M, K, seed=9), rnd(N, K, seed=10)
    out = ops().gemm_f32(a.to(DEV), w.to(DEV))
    want = a.double() @ w.double().T
    assert (out.cpu().double() - want).abs().max().item() <= 1e-6 * math.sqrt(K) * want.abs().max().item() + 1e-6


def test_gemm_f32_rows_do_not_depend_on_the_batch():
    a, w = rnd(150, 333, seed=11), rnd(257, 333, seed=12)
    full = ops().gemm_f32(a.to(DEV), w.to(DEV))
    for rows in ([0], [5, 6, 7], list(range(40)), list(range(149, 70, -1))):
        part = ops().gemm_f32(a[rows].contiguous().to(DEV), w.to(DEV))
        assert torch.equal(part, full[rows])


def test_gemm_f32_is_not_reduced_precision():
    # products that a 10-bit (TF32) or 8-bit (bf16) mantissa would lose
    a = torch.tensor([[1.0 + 2.0 ** -20, 1.0]], device=DEV)
    w = torch.tensor([[1.0, -1.0]], device=DEV)
    assert ops().gemm_f32(a, w).item() == 2.0 ** -20


# ----------------------------------------------------------------------------- bf16 product, few rows


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 1000, 64), (3, 50, 176), (8, 4096, 4096), (9, 320, 192), (16, 513, 4104),
                                   (5, 128256, 256), (8, 16, 8), (17, 6144, 1024), (64, 264, 14336),
                                   (128, 520, 1032)])
def test_gemm_tma(M, N, K, out_dtype):
    """The tcgen05 weight-streaming product against a float64 product, at sizes that are no
    multiples of its tiles (128 rows of W, 64 of k, 16 tokens) and that cut tiles' k ranges
    across blocks."""
    x = rnd(M, K, dtype=torch.bfloat16, seed=30)
    w = rnd(N, K, dtype=torch.bfloat16, seed=31, scale=0.1)
    out = ops().gemm_tma(x.to(DEV), w.to(DEV), out_dtype)
    want = x.double() @ w.double().T
    bound = (1e-5 if out_dtype == torch.float32 else 1 / 128) * max(1.0, want.abs().max().item())
    assert out.dtype == out_dtype
    assert (out.cpu().double() - want).abs().max().item() <= bound
    assert ops().gemm_tma_status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 256, 64), (8, 4096, 4096), (5, 320, 176), (8, 192, 14336), (16, 1000, 520),
                                   (3, 4104, 1032)])
def test_gemm_tma_adds_to_the_stream_and_leaves_statistics(M, N, K):
    """The residual epilogue: the fp32 stream takes the product in place, the output is the new
    stream times the gain, and the sums of squares per 128 features add up to each row's; then
    the product that takes those statistics finishes an RMS norm.  Against float64; widths with
    a ragged last tile and k ranges cut across blocks."""
    x = rnd(M, K, dtype=torch.bfloat16, seed=50)
    w = rnd(N, K, dtype=torch.bfloat16, seed=51, scale=0.1)
    res = rnd(M, N, seed=52)
    gain = 1 + 0.1 * rnd(N, seed=53)
    eps = 1e-5
    stream = res.clone().to(DEV)
    y, stats = ops().gemm_tma(x.to(DEV), w.to(DEV), torch.bfloat16, residual=stream, gain=gain.to(DEV), eps=eps)
    want_stream = res.double() + x.double() @ w.double().T
    scale = max(1.0, want_stream.abs().max().item())
    assert (stream.cpu().double() - want_stream).abs().max().item() <= 1e-5 * scale
    want_y = want_stream * gain.double()
    assert (y.cpu().double() - want_y).abs().max().item() <= 1 / 128 * max(1.0, want_y.abs().max().item())
    assert stats.width == N and stats.eps == eps and stats.sums.shape == (-(-N // 128), 16)
    sums = stats.sums.cpu().double()
    want_sq = (want_stream ** 2).sum(dim=1)
    assert ((sums[:, :M].sum(dim=0) - want_sq).abs() <= 1e-5 * want_sq).all()
    for t in range(sums.shape[0]):      # tile by tile, so that no tile's share lands in another's slot
        part = (want_stream[:, t * 128:(t + 1) * 128] ** 2).sum(dim=1)
        assert ((sums[t, :M] - part).abs() <= 1e-5 * part + 1e-9).all()
    # the consumer: a product of the gained stream, scaled row by row in its epilogue
    w2 = rnd(264, N, dtype=torch.bfloat16, seed=54, scale=0.1)
    out = ops().gemm_tma(y, w2.to(DEV), torch.float32, row_stats=stats)
    rstd = 1.0 / torch.sqrt(want_sq / N + eps)
    want_out = (y.cpu().double() * rstd[:, None]) @ w2.double().T
    assert (out.cpu().double() - want_out).abs().max().item() <= 1e-5 * max(1.0, want_out.abs().max().item())
    # against the norm itself: gain * h * rstd, rounded once more on this route (y is bfloat16)
    normed = (want_stream * rstd[:, None] * gain.double()) @ w2.double().T
    assert (out.cpu().double() - normed).abs().max().item() <= 1 / 128 * max(1.0, normed.abs().max().item())
    # and with the gate/up epilogue behind the scaling
    wg, wu = rnd(100, N, dtype=torch.bfloat16, seed=55, scale=0.1), rnd(100, N, dtype=torch.bfloat16, seed=56, scale=0.1)
    pairs = torch.stack([wg, wu], dim=1).reshape(200, N).contiguous()
    act = ops().gemm_tma(y, pairs.to(DEV), torch.bfloat16, swiglu=True, row_stats=stats)
    xn = y.cpu().double() * rstd[:, None]
    want_act = P.silu(xn @ wg.double().T) * (xn @ wu.double().T)
    assert (act.cpu().double() - want_act).abs().max().item() <= 1 / 128 * max(1.0, want_act.abs().max().item())
    assert ops().gemm_tma_status() == 0


def test_gemm_tma_fused_forms_refuse_what_they_cannot_take():
    w = rnd(256, 64, dtype=torch.bfloat16, seed=57).to(DEV)
    x = rnd(17, 64, dtype=torch.bfloat16, seed=58).to(DEV)
    with pytest.raises(ops().KernelError, match="at most 16"):
        ops().gemm_tma(x, w, torch.bfloat16, residual=torch.zeros(17, 256, device=DEV),
                       gain=torch.ones(256, device=DEV), eps=1e-5)
    with pytest.raises(ops().KernelError, match="fp32"):
        ops().gemm_tma(x[:4].contiguous(), w, torch.bfloat16, residual=torch.zeros(4, 256, device=DEV),
                       gain=torch.ones(256, device=DEV, dtype=torch.bfloat16), eps=1e-5)
    stats = ops().RowStats(torch.zeros(2, 16, device=DEV), 200, 1e-5)
    with pytest.raises(ops().KernelError, match="do not fit"):
        ops().gemm_tma(x[:4].contiguous(), w, torch.bfloat16, row_stats=stats)
    assert not ops().linear_fusable(17, w) and ops().linear_fusable(16, w)


def test_gemm_tma_is_deterministic_and_independent_of_other_rows():
    """Partial tiles are added in block order whatever the arrival order, and a row of x gives
    the same result alone as among other rows."""
    N, K = 4096, 14336
    x = rnd(8, K, dtype=torch.bfloat16, seed=32).to(DEV)
    w = rnd(N, K, dtype=torch.bfloat16, seed=33, scale=0.05).to(DEV)
    first = ops().gemm_tma(x, w, torch.float32)
    for _ in range(5):
        assert torch.equal(ops().gemm_tma(x, w, torch.float32), first)
    alone = ops().gemm_tma(x[3:4].contiguous(), w, torch.float32)
    assert torch.equal(alone[0], first[3])
    assert ops().gemm_tma_status() == 0


def test_gemm_tma_refuses_what_it_cannot_take():
    w = rnd(64, 36, dtype=torch.bfloat16, seed=34).to(DEV)
    with pytest.raises(ops().KernelError, match="multiples of 8"):
        ops().gemm_tma(rnd(2, 36, dtype=torch.bfloat16, seed=35).to(DEV), w)
    w = rnd(64, 64, dtype=torch.bfloat16, seed=36).to(DEV)
    with pytest.raises(ops().KernelError, match="at most"):
        ops().gemm_tma(rnd(129, 64, dtype=torch.bfloat16, seed=37).to(DEV), w)
    assert not ops().gemm_tma_ok(rnd(2, 36, dtype=torch.bfloat16, seed=35).to(DEV), rnd(64, 36, dtype=torch.bfloat16).to(DEV))


def test_linear_library_and_streaming_kernels_agree():
    w = rnd(300, 264, dtype=torch.bfloat16, seed=22, scale=0.1).to(DEV)
    x = rnd(40, 264, dtype=torch.bfloat16, seed=23).to(DEV)
    big = ops().linear(x, w).float()              # library product
    small = torch.cat([ops().linear(x[i:i + 8].contiguous(), w).float() for i in range(0, 40, 8)])
    assert (big - small).abs().max().item() <= 1 / 64 * max(1.0, big.abs().max().item())
    assert ops().linear(x[:4].contiguous(), w, out_dtype=torch.float32).dtype == torch.float32
    assert ops().linear(x, w, out_dtype=torch.float32).dtype == torch.float32


# ----------------------------------------------------------------------------- attention


def build_paged(kv_lens, nkv, d, page, dtype, seed, n_extra_pages=3):
    """Random keys/values of several requests scattered over shuffled pages, addressed by
    slot ([pages * page, nkv, d]); ``as_pages`` gives the layout the kernels read."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-L // page) for L in kv_lens) + n_extra_pages
    perm = torch.randperm(n_pages, generator=g).tolist()
    kc = torch.full((n_pages * page, nkv, d), float("nan"), dtype=dtype)
    vc = torch.full((n_pages * page, nkv, d), float("nan"), dtype=dtype)
    tables, ks, vs = [], [], []
    for L in kv_lens:
        k = torch.randn(L, nkv, d, generator=g).to(dtype)
        v = torch.randn(L, nkv, d, generator=g).to(dtype)
        t = [perm.pop() for _ in range(-(-L // page))]
        for p in range(L):
            kc[t[p // page] * page + p % page] = k[p]
            vc[t[p // page] * page + p % page] = v[p]
        tables.append(t)
        ks.append(k)
        vs.append(v)
    width = max(len(t) for t in tables)
    bt = torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32)
    return kc, vc, bt, ks, vs


def as_pages(c, page):
    """[pages * page, nkv, d] by slot -> the cache layout (pages per head, rows chunk-permuted)."""
    return ops().pack_cache_pages(c, page)


def run_attention(q_lens, kv_lens, nq, nkv, d, page, dtype, window=0, seed=0, boost=None, kernel="generic",
                  n_splits=1, slice_chunks=None):
    o = ops()
    kc, vc, bt, ks, vs = build_paged(kv_lens, nkv, d, page, dtype, seed)
    M = sum(q_lens)
    g = torch.Generator().manual_seed(seed + 1)
    q = torch.randn(M, nq, d, generator=g).to(dtype)
    if boost is not None:
        boost(q, ks, kc, bt)
    q_start = [sum(q_lens[:i]) for i in range(len(q_lens))]
    T_ = {"generic": lambda: o.ATTENTION_TILE_TOKENS, "prefill_tc": lambda: o.prefill_tc_tile_tokens(nq // nkv)}.get(
        kernel, lambda: o.prefill_tile_tokens(nq // nkv))()
    treq = [i for i, n in enumerate(q_lens) for _ in range(0, n, T_)]
    ttok = [t0 for n in q_lens for t0 in range(0, n, T_)]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    # q lives inside a wider buffer, as it does in the engine (row stride > nq * d)
    wide = torch.zeros(M, nq * d + 24, dtype=dtype)
    wide[:, : nq * d] = q.view(M, nq * d)
    wide = wide.to(DEV)
    out = torch.full((M, nq * d), float("nan"), dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(d)
    kc, vc = as_pages(kc, page), as_pages(vc, page)
    if kernel == "generic":
        o.attention_generic(wide, wide.stride(0), out, kc.to(DEV), vc.to(DEV), bt.to(DEV), page, i32(q_start),
                            i32(q_lens), i32(kv_lens), i32(treq), i32(ttok), len(treq), nq, nkv, d, scale, window)
    elif kernel in ("prefill", "prefill_tc"):
        fn = o.attention_prefill if kernel == "prefill" else o.attention_prefill_tc
        fn(wide, wide.stride(0), out, kc.to(DEV), vc.to(DEV), bt.to(DEV), page, i32(q_start),
           i32(q_lens), i32(kv_lens), i32(treq), i32(ttok), len(treq), T_, nq, nkv, d, scale, window)
        if kernel == "prefill_tc":
            assert o.attention_tc_status() == 0, "a block of the tcgen05 kernel gave up a wait"
    elif kernel == "balanced":
        assert all(n == 1 for n in q_lens)
        # the requests' rows of the block table in another order than the requests, as in the engine
        order = list(reversed(range(len(q_lens))))
        table = torch.full((len(q_lens) + 2, bt.shape[1]), -1, dtype=torch.int32)
        for i, row in enumerate(order):
            table[row] = bt[i]
        o.attention_decode_balanced(wide, wide.stride(0), out, kc.to(DEV), vc.to(DEV), table.to(DEV), page, i32(q_start),
                                    i32(kv_lens), len(q_lens), nq, nkv, d, scale, window, table_rows=i32(order))
    else:
        assert all(n == 1 for n in q_lens)
        o.attention_decode(wide, wide.stride(0), out, kc.to(DEV), vc.to(DEV), bt.to(DEV), page, i32(q_start),
                           i32(kv_lens), len(q_lens), nq, nkv, d, scale, window, n_splits,
                           slice_chunks=None if slice_chunks is None else i32([slice_chunks]))
    if kernel != "generic":
        assert o.attention_wait_status() == 0, "a kernel gave up waiting for its copies"
    want = torch.empty(M, nq, d, dtype=torch.float64)
    for i, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        want[q_start[i]:q_start[i] + ql] = P.causal_attention(
            q[q_start[i]:q_start[i] + ql].double(), ks[i].double(), vs[i].double(), 1.0 / math.sqrt(d),
            window or None, q_offset=kl - ql)
    return out.cpu().double().view(M, nq, d), want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page", [(6, 2, 48, 8), (4, 4, 16, 16), (8, 1, 128, 16), (3, 1, 256, 4), (10, 5, 80, 32)])
def test_attention_mixed_batch(dtype, nq, nkv, d, page):
    q_lens = [1, 5, 37, 1, 16]
    kv_lens = [1, 5, 100, 131, 16]
    got, want = run_attention(q_lens, kv_lens, nq, nkv, d, page, dtype, seed=nq)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() <= tol(dtype, fp32=2e-5, bf16=1 / 64)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 20, 64])
def test_attention_window(dtype, window):
    got, want = run_attention([1, 40, 3], [90, 70, 3], 4, 2, 32, 8, dtype, window=window, seed=3)
    assert (got - want).abs().max().item() <= tol(dtype, fp32=2e-5, bf16=1 / 64)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key_among_hundreds(dtype):
    """One key far back is made to match the last query strongly; the output must be its
    value.  A kernel that skips, repeats or misplaces a page cannot pass."""
    nq, nkv, d, page = 2, 1, 32, 16
    for target in (0, 15, 16, 257, 700, 703):
        def boost(q, ks, kc, bt, target=target):
            ks[0][target] = 0
            ks[0][target, 0, 0] = 8.0
            kc[bt[0, target // page] * page + target % page] = ks[0][target]
            q[-1] = 0
            q[-1, :, 0] = 40.0
        got, want = run_attention([1], [704], nq, nkv, d, page, dtype, seed=5, boost=boost)
        assert (got - want).abs().max().item() <= tol(dtype, fp32=2e-5, bf16=1 / 64)


BF16_BOUND = 1 / 64      # probabilities and outputs are rounded to bfloat16 (2^-9 each)


@pytest.mark.parametrize("nq,nkv,d,page", [(6, 2, 48, 8), (4, 4, 16, 16), (32, 8, 128, 16), (3, 1, 256, 4),
                                            (10, 5, 80, 32), (40, 2, 64, 16), (70, 1, 32, 16)])
def test_attention_prefill_tensor_cores(nq, nkv, d, page):
    q_lens = [1, 5, 37, 1, 16, 130]
    kv_lens = [1, 5, 100, 131, 16, 257]
    got, want = run_attention(q_lens, kv_lens, nq, nkv, d, page, torch.bfloat16, seed=nq, kernel="prefill")
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() <= BF16_BOUND


@pytest.mark.parametrize("window", [1, 7, 20, 64, 100])
def test_attention_prefill_tensor_cores_window(window):
    got, want = run_attention([1, 90, 3, 150], [90, 170, 3, 150], 4, 2, 32, 8, torch.bfloat16, window=window,
                              seed=3, kernel="prefill")
    assert (got - want).abs().max().item() <= BF16_BOUND


@pytest.mark.parametrize("nq,nkv,d,page", [(32, 8, 128, 16), (8, 1, 128, 8), (4, 4, 64, 16), (16, 2, 64, 64),
                                            (2, 1, 128, 32), (64, 1, 64, 16)])
def test_attention_prefill_tcgen05(nq, nkv, d, page):
    """The tcgen05 prefill kernel at the sizes it takes: both head sizes, every page size, group
    sizes from 1 (128 tokens per tile) to 64 (2 tokens per tile); requests of one token, of
    lengths that end inside a page and inside a 64-key chunk, and portions that start deep in
    the cache.  Never-written cache slots hold NaN (build_paged), so a masked value row that is
    not cleared would show."""
    assert ops().prefill_tc_supported(nq, nkv, d, page)
    q_lens = [1, 5, 37, 1, 16, 130, 64]
    kv_lens = [1, 5, 100, 131, 16, 257, 320]
    got, want = run_attention(q_lens, kv_lens, nq, nkv, d, page, torch.bfloat16, seed=nq, kernel="prefill_tc")
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() <= BF16_BOUND


@pytest.mark.parametrize("window", [1, 7, 20, 64, 100])
def test_attention_prefill_tcgen05_window(window):
    got, want = run_attention([1, 90, 3, 150], [90, 170, 3, 150], 4, 2, 64, 8, torch.bfloat16, window=window,
                              seed=3, kernel="prefill_tc")
    assert (got - want).abs().max().item() <= BF16_BOUND


def test_attention_prefill_tcgen05_far_key_and_big_scores():
    """One key far back matches the last query strongly (its score is hundreds of units above
    the rest, far beyond the lazy-rescale threshold), in the first chunk, at a chunk's edge and
    in the last chunk; and the sizes the kernel does not take are refused."""
    nq, nkv, d, page = 2, 1, 64, 16
    for target in (0, 63, 64, 257, 700, 703):
        def boost(q, ks, kc, bt, target=target):
            ks[0][target] = 0
            ks[0][target, 0, 0] = 8.0
            kc[bt[0, target // page] * page + target % page] = ks[0][target]
            q[-1] = 0
            q[-1, :, 0] = 40.0
        got, want = run_attention([70], [704], nq, nkv, d, page, torch.bfloat16, seed=5, boost=boost,
                                  kernel="prefill_tc")
        assert (got - want).abs().max().item() <= BF16_BOUND
    assert not ops().prefill_tc_supported(6, 2, 48, 8)
    assert not ops().prefill_tc_supported(4, 4, 64, 4)
    assert not ops().prefill_tc_supported(3, 1, 128, 16)
    # the Python-side test and the library's own agree
    lib = ops()._lib("attention_tc")
    for nq, nkv in [(1, 1), (4, 2), (6, 2), (32, 8), (3, 1), (64, 1), (256, 1), (5, 5), (4, 3)]:
        for d in (16, 48, 64, 96, 128, 256):
            for page in (1, 4, 8, 12, 16, 32, 64, 128):
                assert ops().prefill_tc_supported(nq, nkv, d, page) == bool(
                    lib.mi_attention_prefill_tc_supported(nq, nkv, d, page)), (nq, nkv, d, page)


def test_attention_long_contexts():
    """Tens of thousands of keys: decode over 20,000 cached tokens with few and many key
    slices, and a 4,100-token portion through both prefill kernels (65 chunks per tile, many
    rounds of every ring of stages and of every barrier phase)."""
    got, want = run_attention([1, 1], [20000, 8191], 4, 2, 64, 16, torch.bfloat16, seed=21, kernel="decode", n_splits=3)
    assert (got - want).abs().max().item() <= BF16_BOUND
    got, want = run_attention([1, 1], [20000, 8191], 4, 2, 64, 16, torch.bfloat16, seed=21, kernel="decode", n_splits=64)
    assert (got - want).abs().max().item() <= BF16_BOUND
    for kernel in ("prefill", "prefill_tc"):
        got, want = run_attention([4100], [4100], 2, 1, 64, 16, torch.bfloat16, seed=22, kernel=kernel)
        assert torch.isfinite(got).all()
        assert (got - want).abs().max().item() <= BF16_BOUND


@pytest.mark.parametrize("n_splits", [1, 2, 5, 64])
@pytest.mark.parametrize("nq,nkv,d,page", [(32, 8, 128, 16), (6, 2, 48, 8), (3, 3, 16, 4), (40, 2, 64, 16), (5, 1, 256, 16)])
def test_attention_decode_split_keys(nq, nkv, d, page, n_splits):
    kv_lens = [1, 64, 65, 700, 17, 2048 if d <= 128 else 300]
    got, want = run_attention([1] * len(kv_lens), kv_lens, nq, nkv, d, page, torch.bfloat16, seed=nq + 7,
                              kernel="decode", n_splits=n_splits)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() <= BF16_BOUND


@pytest.mark.parametrize("n_splits,slice_chunks", [(4, 9), (8, 4), (5, 1), (64, 1), (3, 100), (12, 3)])
def test_attention_decode_slices_of_one_length(n_splits, slice_chunks):
    """Slices of the same number of chunks for every request: requests far shorter than the
    longest fill one slice and leave the others empty; a slice length too short to cover the
    longest request with the slices at hand is lengthened by the kernel, never obeyed."""
    kv_lens = [2100, 1, 64, 65, 300, 17, 640]
    got, want = run_attention([1] * len(kv_lens), kv_lens, 8, 2, 64, 16, torch.bfloat16, seed=31,
                              kernel="decode", n_splits=n_splits, slice_chunks=slice_chunks)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() <= BF16_BOUND
    got, want = run_attention([1, 1, 1], [500, 64, 7], 8, 2, 64, 16, torch.bfloat16, window=100, seed=9,
                              kernel="decode", n_splits=n_splits, slice_chunks=slice_chunks)
    assert (got - want).abs().max().item() <= BF16_BOUND


@pytest.mark.parametrize("nq,nkv,d,page", [(32, 8, 128, 16), (6, 2, 48, 8), (3, 3, 16, 4), (40, 2, 64, 16), (5, 1, 256, 16),
                                            (24, 1, 128, 32)])
def test_attention_decode_balanced(nq, nkv, d, page):
    """The balanced decode kernel: requests of very different lengths (one key, a chunk's edge,
    thousands), so that some blocks hold several whole units, some a stretch of one unit, and a
    long unit is merged from many stretches; a request without any key among them."""
    kv_lens = [1, 64, 65, 700, 17, 2048 if d <= 128 else 300, 3, 129, 5000 if d <= 64 else 130]
    got, want = run_attention([1] * len(kv_lens), kv_lens, nq, nkv, d, page, torch.bfloat16, seed=nq + 11, kernel="balanced")
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() <= BF16_BOUND
    # the same twice more with other lengths: the counters were left at zero
    for seed, lens in ((3, [40000 if d <= 64 else 9000]), (4, [300, 300, 300, 300]), (5, [5, 9, 2, 1, 1, 1, 130])):
        got, want = run_attention([1] * len(lens), lens, nq, nkv, d, page, torch.bfloat16, seed=seed, kernel="balanced")
        assert (got - want).abs().max().item() <= BF16_BOUND


@pytest.mark.parametrize("unit_cost", [0, 1, 2, 5, 40])
def test_attention_decode_balanced_whatever_a_unit_is_reckoned_to_cost(unit_cost):
    """The balanced kernel lengthens every unit by a number of positions that stand for no chunk
    before it cuts the row into stretches.  Whatever that number is, every chunk is read exactly
    once: many requests of one chunk beside a long one (stretches that begin and end inside the
    added positions, blocks that find no chunk in theirs), a window."""
    before = ops().decode_unit_cost(unit_cost)
    try:
        assert ops().decode_unit_cost() == unit_cost
        for seed, (nq, nkv, d, page), lens, window in (
                (1, (32, 8, 128, 16), [3000] + [5, 64, 1, 17, 63, 65, 2, 128] * 6 + [700], 0),
                (2, (8, 2, 64, 8), [1] * 40 + [9000] + [1] * 23, 0),
                (3, (6, 2, 48, 8), [130, 1, 200, 64, 7, 1000, 3], 100),
                (4, (4, 4, 64, 16), [2, 2, 2], 0)):
            got, want = run_attention([1] * len(lens), lens, nq, nkv, d, page, torch.bfloat16, seed=seed, window=window,
                                      kernel="balanced")
            assert torch.isfinite(got).all()
            assert (got - want).abs().max().item() <= BF16_BOUND
    finally:
        ops().decode_unit_cost(before)


@pytest.mark.parametrize("nq,nkv,d,page", [(32, 8, 128, 16), (8, 2, 64, 8), (6, 3, 128, 16), (5, 1, 256, 32), (4, 4, 64, 16),
                                            (24, 1, 128, 32)])
def test_attention_decode_rotates_and_stores_by_itself(nq, nkv, d, page):
    """The decode kernel given the projection's raw q, k, v and the step's rotary table against
    the two-kernel route (rotate and store, then attend): the same output and the same cache,
    bit for bit, with requests whose newest token lies at a page's first slot, at a chunk's edge,
    deep inside a long context, and alone."""
    o = ops()
    kv_lens = [1, 64, 65, 700, page + 1, 2048 if d <= 128 else 300, 129]
    B = len(kv_lens)
    kc, vc, bt, ks, vs = build_paged(kv_lens, nkv, d, page, torch.bfloat16, seed=nq + 50)
    g = torch.Generator().manual_seed(nq + 51)
    qkv = torch.randn(B, (nq + 2 * nkv) * d, generator=g).to(torch.bfloat16).to(DEV)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
    positions = torch.tensor([L - 1 for L in kv_lens], dtype=torch.int32, device=DEV)
    slots = torch.tensor([int(bt[i, (L - 1) // page]) * page + (L - 1) % page for i, L in enumerate(kv_lens)],
                         dtype=torch.int32, device=DEV)
    q_start = torch.arange(B, dtype=torch.int32, device=DEV)
    kv_len = torch.tensor(kv_lens, dtype=torch.int32, device=DEV)
    btd = bt.to(DEV)
    scale = d ** -0.5

    def caches():
        return as_pages(kc, page).to(DEV), as_pages(vc, page).to(DEV)

    # two kernels
    k1, v1 = caches()
    qkv1 = qkv.clone()
    o.rope_write(qkv1, nq, nkv, d, positions=positions, inv_freq=inv_freq, rotary_dim=d, slots=slots, kcache=k1, vcache=v1)
    out1 = torch.full((B, nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.attention_decode_balanced(qkv1, qkv1.stride(0), out1, k1, v1, btd, page, q_start, kv_len, B, nq, nkv, d, scale)
    # one kernel
    k2, v2 = caches()
    table = o.rope_table(positions, inv_freq)
    out2 = torch.full((B, nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.attention_decode_balanced(qkv.clone(), qkv.stride(0), out2, k2, v2, btd, page, q_start, kv_len, B, nq, nkv, d, scale,
                                rope_table=table, store_kv=True)
    torch.cuda.synchronize()
    assert o.attention_wait_status() == 0
    assert torch.isfinite(out2).all()
    assert torch.equal(out1, out2)
    # the written rows are the same (everything else in the pool is NaN or untouched and equal bit for bit)
    assert torch.equal(k1.view(torch.int16), k2.view(torch.int16))
    assert torch.equal(v1.view(torch.int16), v2.view(torch.int16))
    # without storing: q is rotated, the cache is left as it was (a layer that reads another layer's cache)
    k3, v3 = k1.clone(), v1.clone()
    out3 = torch.full((B, nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.attention_decode_balanced(qkv.clone(), qkv.stride(0), out3, k3, v3, btd, page, q_start, kv_len, B, nq, nkv, d, scale,
                                rope_table=table, store_kv=False)
    assert torch.equal(out3, out1) and torch.equal(k3.view(torch.int16), k1.view(torch.int16))


@pytest.mark.parametrize("window", [1, 30, 64, 200])
def test_attention_decode_balanced_window_and_far_key(window):
    got, want = run_attention([1, 1, 1], [500, 64, 7], 8, 2, 64, 16, torch.bfloat16, window=window, seed=9, kernel="balanced")
    assert (got - want).abs().max().item() <= BF16_BOUND
    nq, nkv, d, page = 4, 1, 32, 16
    for target in (0, 15, 16, 63, 64, 257, 700, 703):
        def boost(q, ks, kc, bt, target=target):
            ks[0][target] = 0
            ks[0][target, 0, 0] = 8.0
            kc[bt[0, target // page] * page + target % page] = ks[0][target]
            q[-1] = 0
            q[-1, :, 0] = 40.0
        got, want = run_attention([1], [704], nq, nkv, d, page, torch.bfloat16, seed=5, boost=boost, kernel="balanced")
        assert (got - want).abs().max().item() <= BF16_BOUND


@pytest.mark.parametrize("window", [1, 30, 64, 200])
def test_attention_decode_window(window):
    got, want = run_attention([1, 1, 1], [500, 64, 7], 8, 2, 64, 16, torch.bfloat16, window=window, seed=9,
                              kernel="decode", n_splits=4)
    assert (got - want).abs().max().item() <= BF16_BOUND


@pytest.mark.parametrize("kernel,n_splits", [("prefill", 1), ("decode", 1), ("decode", 7)])
def test_tensor_core_attention_finds_a_far_key(kernel, n_splits):
    nq, nkv, d, page = 4, 1, 32, 16
    for target in (0, 15, 16, 63, 64, 257, 700, 703):
        def boost(q, ks, kc, bt, target=target):
            ks[0][target] = 0
            ks[0][target, 0, 0] = 8.0
            kc[bt[0, target // page] * page + target % page] = ks[0][target]
            q[-1] = 0
            q[-1, :, 0] = 40.0
        got, want = run_attention([1], [704], nq, nkv, d, page, torch.bfloat16, seed=5, boost=boost,
                                  kernel=kernel, n_splits=n_splits)
        assert (got - want).abs().max().item() <= BF16_BOUND


def test_attention_refuses_bad_head_size():
    with pytest.raises(Exception):
        run_attention([1], [4], 2, 1, 24, 4, torch.float32)


# ----------------------------------------------------------------------------- sampling


def sample_rows(logits, temperature=None, top_k=None, top_p=None, seeds=None, draws=None):
    B = logits.shape[0]
    f32 = lambda x: torch.tensor(x, dtype=torch.float32, device=DEV)
    i32 = lambda x: torch.tensor(np.array(x, dtype=np.int64).astype(np.uint32).view(np.int32).tolist() if x is not None else [],
                                 dtype=torch.int32, device=DEV)
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    kw = {}
    if temperature is not None:
        kw = dict(temperature=f32(temperature), top_k=i32(top_k if top_k is not None else [0] * B),
                  top_p=f32(top_p if top_p is not None else [1.0] * B),
                  seed_lo=i32([s & 0xFFFFFFFF for s in seeds]), seed_hi=i32([(s >> 32) & 0xFFFFFFFF for s in seeds]),
                  draw_index=i32(draws))
    ops().sample(logits.to(DEV), out, **kw)
    return out.cpu().tolist()


def test_sample_greedy_is_argmax_with_lowest_index():
    logits = rnd(6, 1000, seed=13)
    logits[2, 17] = logits[2, 900] = 50.0
    got = sample_rows(logits)
    want = logits.argmax(dim=-1).tolist()
    want[2] = 17
    assert got == want


@pytest.mark.parametrize("V", [4096, 50001, 128256])
def test_sample_greedy_with_rows_cut_across_blocks(V):
    """Large vocabularies are scanned by several blocks per row; equal maxima in different
    slices still give the lowest index, and a vocabulary that is no multiple of the slices,
    or of four, loses no element."""
    logits = rnd(5, V, seed=15)
    logits[1, 3] = logits[1, V - 1] = 60.0          # a tie between the first and the last slice
    logits[2, V - 1] = 70.0                         # the very last element wins
    logits[3, V // 2 + 1] = logits[3, V // 2 + 2] = 65.0
    want = logits.argmax(dim=-1).tolist()
    want[1], want[3] = 3, V // 2 + 1
    for _ in range(3):                              # the arrival counters reset themselves
        assert sample_rows(logits) == want
    # a view whose rows are not 16-byte aligned takes the element-wise scan
    wide = torch.zeros(5, V + 3)
    wide[:, 1:V + 1] = logits
    assert sample_rows(wide.to(DEV)[:, 1:V + 1]) == want


def test_sample_matches_reference_draws():
    V = 1000
    logits = rnd(8, V, seed=14, scale=2.0)
    temps = [0.7, 1.0, 0.0, 1.3, 0.8, 0.8, 1.0, 0.5]
    top_k = [0, 5, 0, 50, 0, 3, 1, 0]
    top_p = [1.0, 1.0, 1.0, 1.0, 0.6, 0.9, 1.0, 0.05]
    seeds = [1, 2, 3, (7 << 32) | 9, 5, 6, 7, 8]
    draws = [0, 1, 2, 3, 4, 5, 6, 100000]
    got = sample_rows(logits, temps, top_k, top_p, seeds, draws)
    for b in range(8):
        tok, score, keep = P.sample_reference(logits[b].numpy(), temps[b], top_k[b], top_p[b], seeds[b], draws[b])
        if temps[b] == 0.0:
            assert got[b] == tok
            continue
        assert keep[got[b]], f"row {b}: token {got[b]} is outside the kept set"
        # the chosen token maximises the perturbed score up to fp32 rounding of the noise
        assert score[got[b]] >= score.max() - 1e-4 * max(1.0, abs(score.max()))


def test_sample_draws_follow_softmax_and_ignore_the_batch():
    logits_row = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, -30.0, 1.5, 0.2])
    B = 4000
    logits = logits_row.repeat(B, 1)
    got = sample_rows(logits, [0.9] * B, None, None, [42] * B, list(range(B)))
    freq = np.bincount(got, minlength=8) / B
    probs = torch.softmax(logits_row.double() / 0.9, dim=-1).numpy()
    assert np.abs(freq - probs).max() < 0.03
    # the same (seed, draw index) gives the same token whatever else is in the batch
    alone = sample_rows(logits[:1], [0.9], None, None, [42], [1234])
    mixed = sample_rows(logits[:3], [0.9, 0.0, 0.9], None, None, [7, 8, 42], [0, 0, 1234])
    assert alone[0] == mixed[2]
