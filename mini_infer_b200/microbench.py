"""Time one kernel of the engine alone, at sizes given on the command line.

    python -m mini_infer_b200.microbench attention_decode --batch 8 --context 2048
    python -m mini_infer_b200.microbench attention_prefill --tokens 2048 [--impl mma]
    python -m mini_infer_b200.microbench gemm_tma --rows 8 --n 28672 --k 4096 [--epilogue stream|stats]
    python -m mini_infer_b200.microbench add_rmsnorm --rows 8 --width 4096
    python -m mini_infer_b200.microbench rope_write --rows 2048
    python -m mini_infer_b200.microbench silu_mul --rows 2048 --width 14336
    python -m mini_infer_b200.microbench sample --rows 8 --vocab 128256

Before each iteration a buffer larger than the L2 cache is overwritten, so every run starts
cold.  The time is the device-side duration of the kernels the call launches (``--timer
events`` takes CUDA events around the call instead, which adds the host's launch work); the
line printed gives the median and the bytes (or flops) the kernel has to move divided by
it.  The same command with ``--timer events`` under ``ncu -k regex:<kernel>`` profiles
exactly these launches.
"""

from __future__ import annotations

import argparse
import math
import statistics
import sys

import torch


def _flush_buffer(device) -> torch.Tensor:
    return torch.empty(256 << 20, dtype=torch.uint8, device=device)


TIMER = "device"


def _time(fn, iters: int, warmup: int, flush: torch.Tensor) -> float:
    """Median microseconds of ``fn()``, L2 flushed before each call.

    ``TIMER == "device"``: the sum of the device-side durations of the kernels ``fn`` launches
    (from the profiler's activity records), which leaves out the host's launch work; that
    matters for kernels of a few microseconds.  ``"events"``: CUDA events around the call."""
    if TIMER == "events":
        times = []
        for i in range(warmup + iters):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            if i >= warmup:
                times.append(start.elapsed_time(end) * 1e3)
        return statistics.median(times)
    from torch.profiler import ProfilerActivity, profile

    for _ in range(warmup):
        flush.zero_()
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.zero_()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            fn()
            torch.cuda.synchronize()
        times.append(sum(ev.device_time for ev in prof.events()
                         if ev.device_type == torch.autograd.DeviceType.CUDA))
    return statistics.median(times)


def _paged_cache(batch: int, context: int, nkv: int, d: int, page: int, device):
    pages_per_request = -(-context // page)
    n_pages = batch * pages_per_request
    kcache = torch.randn(n_pages, nkv, page, d, device=device, dtype=torch.bfloat16)
    vcache = torch.randn_like(kcache)
    table = torch.randperm(n_pages, device=device).to(torch.int32).view(batch, pages_per_request).contiguous()
    return kcache, vcache, table


def _library_attention(q_lens, kv_lens, nq, nkv, d, page, device):
    """The same attention through FlashInfer's paged prefill wrapper, the library call the
    reference project makes for every attention layer (cache/flashinfer_backend.py:289-349:
    one ``plan`` per step, ``run`` per layer): a bar to compare with, never a product path.
    Returns ``run()`` or raises ImportError."""
    import flashinfer

    pages = [-(-n // page) for n in kv_lens]
    n_pages = sum(pages)
    kcache = torch.randn(n_pages, page, nkv, d, device=device, dtype=torch.bfloat16)
    vcache = torch.randn_like(kcache)
    q = torch.randn(sum(q_lens), nq, d, device=device, dtype=torch.bfloat16)
    qo_indptr = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=device)
    kv_indptr = torch.tensor([0] + list(torch.tensor(pages).cumsum(0)), dtype=torch.int32, device=device)
    kv_indices = torch.randperm(n_pages, device=device).to(torch.int32)
    last = torch.tensor([(n - 1) % page + 1 for n in kv_lens], dtype=torch.int32, device=device)
    workspace = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    wrapper = flashinfer.BatchPrefillWithPagedKVCacheWrapper(workspace, "NHD")
    wrapper.plan(qo_indptr, kv_indptr, kv_indices, last, nq, nkv, d, page, causal=True, pos_encoding_mode="NONE",
                 sm_scale=1.0 / math.sqrt(d), q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16)

    def run():
        wrapper.run(q, (kcache, vcache))

    return run


def attention_decode(args, ops, device, flush) -> tuple[float, str]:
    nq, nkv, d = args.heads, args.kv_heads, args.head_dim
    kcache, vcache, table = _paged_cache(args.batch, args.context, nkv, d, args.page, device)
    qkv = torch.randn(args.batch, (nq + 2 * nkv) * d, device=device, dtype=torch.bfloat16)
    out = torch.empty(args.batch, nq * d, device=device, dtype=torch.bfloat16)
    q_start = torch.arange(args.batch, device=device, dtype=torch.int32)
    kv_len = torch.full((args.batch,), args.context, device=device, dtype=torch.int32)
    if args.skew:      # lengths from context / skew up to context, so that requests differ widely
        lens = [max(1, int(args.context / args.skew ** (i / max(1, args.batch - 1)))) for i in range(args.batch)]
        kv_len = torch.tensor(lens, device=device, dtype=torch.int32)
    total = int(kv_len.sum().item())
    nbytes = 2 * total * nkv * d * 2
    if args.impl == "library":
        run = _library_attention([1] * args.batch, kv_len.tolist(), nq, nkv, d, args.page, device)
        us = _time(run, args.iters, args.warmup, flush)
        return us, f"FlashInfer's paged prefill wrapper on one query token per request, {nbytes / us / 1e6:.2f} TB/s of keys and values"
    if args.impl == "sliced":
        splits = args.splits or ops.decode_splits(args.batch, nq, nkv, args.context, 0, device)

        def run():
            ops.attention_decode(qkv, qkv.stride(0), out, kcache, vcache, table, args.page, q_start, kv_len,
                                 args.batch, nq, nkv, d, 1.0 / math.sqrt(d), 0, splits)

        us = _time(run, args.iters, args.warmup, flush)
        return us, f"{splits} key slices, {nbytes / us / 1e6:.2f} TB/s of keys and values"

    rope = None
    if args.rope:   # the kernel rotates q and stores the new key and value itself
        inv_freq = (1.0 / (10000.0 ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))).contiguous()
        rope = ops.rope_table((kv_len - 1).to(torch.int32), inv_freq)

    def run():
        ops.attention_decode_balanced(qkv, qkv.stride(0), out, kcache, vcache, table, args.page, q_start, kv_len,
                                      args.batch, nq, nkv, d, 1.0 / math.sqrt(d), 0, rope_table=rope)

    us = _time(run, args.iters, args.warmup, flush)
    return us, f"balanced over persistent blocks, {nbytes / us / 1e6:.2f} TB/s of keys and values"


def attention_prefill(args, ops, device, flush) -> tuple[float, str]:
    nq, nkv, d, T = args.heads, args.kv_heads, args.head_dim, args.tokens
    kcache, vcache, table = _paged_cache(1, T, nkv, d, args.page, device)
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=device, dtype=torch.bfloat16)
    out = torch.empty(T, nq * d, device=device, dtype=torch.bfloat16)
    q_start = torch.zeros(1, device=device, dtype=torch.int32)
    q_len = torch.full((1,), T, device=device, dtype=torch.int32)
    kv_len = torch.full((1,), T, device=device, dtype=torch.int32)
    tile = (ops.prefill_tc_tile_tokens if args.impl == "tc" else ops.prefill_tile_tokens)(nq // nkv)
    n_tiles = -(-T // tile)
    tile_req = torch.zeros(n_tiles, device=device, dtype=torch.int32)
    # the tiles with the most keys first, as the engine's step plan lists them
    tile_tok0 = (torch.arange(n_tiles - 1, -1, -1, device=device, dtype=torch.int32) * tile).contiguous()

    flops = 4.0 * nq * d * T * (T + 1) / 2     # causal: QK^T and PV over the visible half
    if args.impl == "library":
        us = _time(_library_attention([T], [T], nq, nkv, d, args.page, device), args.iters, args.warmup, flush)
        return us, f"FlashInfer's paged prefill wrapper, {flops / us / 1e6:.1f} TFLOP/s (causal flops)"
    kernel = ops.attention_prefill_tc if args.impl == "tc" else ops.attention_prefill

    def run():
        kernel(qkv, qkv.stride(0), out, kcache, vcache, table, args.page, q_start, q_len, kv_len,
               tile_req, tile_tok0, n_tiles, tile, nq, nkv, d, 1.0 / math.sqrt(d), 0)

    us = _time(run, args.iters, args.warmup, flush)
    return us, f"{flops / us / 1e6:.1f} TFLOP/s (causal flops)"


def gemm_tma(args, ops, device, flush) -> tuple[float, str]:
    x = torch.randn(args.rows, args.k, device=device, dtype=torch.bfloat16)
    w = torch.randn(args.n, args.k, device=device, dtype=torch.bfloat16)
    if args.epilogue == "stream":      # the product added to the fp32 stream, gain and statistics for the next norm
        stream = torch.randn(args.rows, args.n, device=device)
        gain = torch.ones(args.n, device=device)

        def run():
            ops.gemm_tma(x, w, residual=stream, gain=gain, eps=1e-5)
    elif args.epilogue == "stats":     # every row scaled by the statistics the product before left
        stats = ops.RowStats(torch.rand(-(-args.k // 128), 16, device=device) * 128, args.k, 1e-5)

        def run():
            ops.gemm_tma(x, w, row_stats=stats)
    else:
        def run():
            ops.gemm_tma(x, w)

    us = _time(run, args.iters, args.warmup, flush)
    status = ops.gemm_tma_status()
    return us, f"{args.n * args.k * 2 / us / 1e6:.2f} TB/s of weights, wait status {status}"


def add_rmsnorm(args, ops, device, flush) -> tuple[float, str]:
    x = torch.randn(args.rows, args.width, device=device, dtype=torch.bfloat16)
    res = torch.randn(args.rows, args.width, device=device, dtype=torch.float32)
    w = torch.ones(args.width, device=device, dtype=torch.bfloat16)

    def run():
        ops.add_rmsnorm(x, w, 1e-5, residual_in=res, residual_out=res)

    us = _time(run, args.iters, args.warmup, flush)
    nbytes = args.rows * args.width * (2 + 4 + 4 + 2)
    return us, f"{nbytes / us / 1e6:.2f} TB/s"


def silu_mul(args, ops, device, flush) -> tuple[float, str]:
    gu = torch.randn(args.rows, 2 * args.width, device=device, dtype=torch.bfloat16)

    def run():
        ops.silu_mul(gu, pairs=True)   # the layout the engine's merged gate/up projection has

    us = _time(run, args.iters, args.warmup, flush)
    return us, f"{args.rows * args.width * 6 / us / 1e6:.2f} TB/s"


def rope_write(args, ops, device, flush) -> tuple[float, str]:
    nq, nkv, d, T = args.heads, args.kv_heads, args.head_dim, args.rows
    kcache, vcache, _ = _paged_cache(1, T, nkv, d, args.page, device)
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=device, dtype=torch.bfloat16)
    pos = torch.arange(T, device=device, dtype=torch.int32)
    slots = torch.randperm(T, device=device).to(torch.int32)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))).contiguous()

    def run():
        ops.rope_write(qkv, nq, nkv, d, positions=pos, inv_freq=inv_freq, rotary_dim=d, slots=slots,
                       kcache=kcache, vcache=vcache)

    us = _time(run, args.iters, args.warmup, flush)
    nbytes = T * (nq + 2 * nkv) * d * 2 * 2
    return us, f"{nbytes / us / 1e6:.2f} TB/s"


def sample(args, ops, device, flush) -> tuple[float, str]:
    from .sampling import DeviceSampler, SamplingParams

    logits = torch.randn(args.rows, args.vocab, device=device, dtype=torch.float32)
    sampler = DeviceSampler(device)
    params = [SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p)] * args.rows

    def run():
        sampler.sample(logits, params, [1] * args.rows, [0] * args.rows)

    us = _time(run, args.iters, args.warmup, flush)
    return us, f"{args.rows * args.vocab * 4 / us / 1e6:.2f} TB/s of logits"


KERNELS = {
    "attention_decode": attention_decode,
    "attention_prefill": attention_prefill,
    "gemm_tma": gemm_tma,
    "add_rmsnorm": add_rmsnorm,
    "silu_mul": silu_mul,
    "rope_write": rope_write,
    "sample": sample,
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m mini_infer_b200.microbench", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=sorted(KERNELS))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--splits", type=int, default=0, help="key slices of decode attention (0: the engine's choice)")
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--width", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--impl", choices=["tc", "mma", "balanced", "sliced", "library"], default=None,
                    help="attention_prefill: the tcgen05 kernel (default) or the mma.sync kernel; attention_decode: "
                         "keys spread evenly over persistent blocks (default) or equal slices per request; "
                         "library: FlashInfer's paged prefill wrapper on the same shapes, for comparison")
    ap.add_argument("--epilogue", choices=["plain", "stream", "stats"], default="plain",
                    help="gemm_tma: the plain product, or one of its fused forms for up to 16 rows")
    ap.add_argument("--rope", action="store_true",
                    help="attention_decode: give the kernel un-rotated q, k, v and the rotary table (it rotates and stores itself)")
    ap.add_argument("--skew", type=float, default=0.0,
                    help="attention_decode: request lengths from context / skew up to context (0: all equal)")
    ap.add_argument("--timer", choices=["device", "events"], default="device",
                    help="device: kernel durations from the profiler's records; events: CUDA events around the call")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    if args.impl is None:
        args.impl = "balanced" if args.kernel == "attention_decode" else "tc"
    if not torch.cuda.is_available():
        print("microbench needs a GPU", file=sys.stderr)
        return 2
    from .csrc import ops

    global TIMER
    TIMER = args.timer
    device = torch.device("cuda:0")
    torch.manual_seed(0)
    flush = _flush_buffer(device)
    us, note = KERNELS[args.kernel](args, ops, device, flush)
    print(f"{args.kernel}: {us:.1f} us median of {args.iters} cold runs ({args.timer} timer); {note}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
