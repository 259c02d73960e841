"""The assembled engine at Llama 3.1 8B's layer sizes (two layers of them): hidden 4096, 32
query heads over 8 key/value heads of 128, intermediate 14336, vocabulary 128256, llama3
rotary scaling with an original context of 8192, pages of 16.

At these sizes the kernels take paths the tiny configurations never reach: decode attention's
stretches for 32/8 heads, the streaming product cut stream-K fashion over a
28672 x 4096 gate/up matrix with its activation epilogue, a 128256-row head, the tcgen05
prefill attention, and positions past the original context length.  The float32 engine is
compared with the plain implementation under the four cuttings, the bfloat16 engine with the
float32 engine, with and without captured decode steps.

The weights are drawn on the device (the generator gives the same numbers on a CPU, see
test_weights.py) and the plain implementation, unchanged, runs on the device too, in float64
(on the CPU a sequence of 8,000 tokens at these widths would take minutes); only its table of
rotary frequencies is computed on the CPU, as the engine's is, because a power function's
last bit differs between devices and positions in the thousands multiply that bit.
"""

import numpy as np
import pytest
import torch

import plain_impl as P
import trace_util as T

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 16
SEED = 41

RAW = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 4096,
    "intermediate_size": 14336, "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072, "tie_word_embeddings": False,
}
# queries and keys wide enough that single keys stand out (see tiny_configs.PEAKED)
WIDE = {"q_proj": (2.5 / 4096) ** 0.5, "k_proj": (2.5 / 4096) ** 0.5}
LENGTHS = [300, 77, 130, 33]


def ids(n, salt):
    g = torch.Generator().manual_seed(9000 + salt)
    return torch.randint(0, RAW["vocab_size"], (n,), generator=g).tolist()


def plain_on_device(state, tokens):
    """``plain_impl.llama_logits`` in float64 with its tensors on the device."""
    cpu_inv_freq = P.rope_inv_freq

    def inv_freq_from_the_cpu(*args):
        with torch.device("cpu"):
            return cpu_inv_freq(*args).to(DEV)

    P.rope_inv_freq = inv_freq_from_the_cpu
    try:
        with torch.device(DEV):
            return P.llama_logits(state, RAW, tokens, dtype=torch.float64)
    finally:
        P.rope_inv_freq = cpu_inv_freq


@pytest.fixture(scope="module")
def full(tmp_path_factory):
    from mini_infer_b200.engine import ModelRunner
    from mini_infer_b200.weights import random_state_dict

    requests = {f"r{i}": ids(n, i) for i, n in enumerate(LENGTHS)}
    state = random_state_dict(RAW, SEED, gain_std=0.1, std_overrides=WIDE, device=DEV)
    want = {r: plain_on_device(state, toks).float().cpu().numpy() for r, toks in requests.items()}
    long_ids = ids(8192 + 300, 77)
    long_want = plain_on_device(state, long_ids)[-40:].float().cpu().numpy()
    del state
    torch.cuda.empty_cache()
    pool = 4 * 512 // PAGE + (8192 + 512) // PAGE + 8

    def runner(dtype, cuda_graph=False):
        r = ModelRunner.from_random(RAW, SEED, dtype=dtype, gain_std=0.1, std_overrides=WIDE, device=DEV,
                                    num_blocks=pool, block_size=PAGE, max_requests=4, cuda_graph=cuda_graph)
        for st in r.cache.storage:
            st.fill_(float("nan"))
        return r

    out = {"requests": requests, "want": want, "long_ids": long_ids, "long_want": long_want,
           "float32": runner("float32"), "bfloat16": runner("bfloat16"), "bfloat16+graph": runner("bfloat16", True)}
    yield out
    out.clear()
    torch.cuda.empty_cache()


CUTTINGS = {"whole": T.cut_whole, "last_decoded": T.cut_last_decoded, "portions": T.cut_portions, "mixed": T.cut_mixed}


def replay(runner, steps):
    got = T.collect(steps, T.replay_in_process(runner, steps), RAW["vocab_size"])
    runner.cache.check()
    assert runner.cache.num_requests == 0
    return got


def check_status():
    from mini_infer_b200.csrc import ops

    assert ops.attention_wait_status() == 0 and ops.attention_tc_status() == 0 and ops.gemm_tma_status() == 0


@pytest.mark.parametrize("cutting", list(CUTTINGS))
def test_full_size_float32_matches_plain(cutting, full):
    steps = CUTTINGS[cutting](full["requests"])
    got = replay(full["float32"], steps)
    scale = max(float(np.abs(w).max()) for w in full["want"].values())
    for rid, want in full["want"].items():
        assert np.isfinite(got[rid]).all()
        bad = T.first_bad(got[rid], want, T.tolerance("float32", scale))
        assert bad is None, (f"float32/{cutting}: request {rid} first differs at position {bad}, "
                             f"|diff| = {np.abs(got[rid][bad] - want[bad]).max():.3e} at logit scale {scale:.2f}")


@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("cutting", list(CUTTINGS))
def test_full_size_bfloat16_matches_float32_engine(cutting, graph, full):
    from mini_infer_b200.csrc import build

    steps = CUTTINGS[cutting](full["requests"])
    if "float32 whole" not in full:
        full["float32 whole"] = replay(full["float32"], CUTTINGS["whole"](full["requests"]))
    reference = full["float32 whole"]
    runner = full["bfloat16+graph" if graph else "bfloat16"]
    got = replay(runner, steps)
    check_status()
    scale = max(float(np.abs(w).max()) for w in reference.values())
    for rid, want in reference.items():
        assert np.isfinite(got[rid]).all()
        bad = T.first_bad(got[rid], want, T.tolerance("bfloat16", scale))
        assert bad is None, (f"bfloat16/{cutting}: request {rid} first differs at position {bad}, "
                             f"|diff| = {np.abs(got[rid][bad] - want[bad]).max():.3e} at logit scale {scale:.2f}")
    # and against the plain implementation directly
    for rid, want in full["want"].items():
        assert T.first_bad(got[rid], want, T.tolerance("bfloat16", scale)) is None
    # the Blackwell kernels were on the path
    assert {"attention_tc", "gemm_tma", "attention_mma"} <= set(build._loaded)
    if graph and cutting in ("last_decoded", "mixed"):
        assert sum(slot.replays for slot in runner.stepper._graphs.values()) >= 20


@pytest.mark.parametrize("which", ["float32", "bfloat16", "bfloat16+graph"])
def test_full_size_positions_past_the_original_context(which, full):
    """A request whose last 40 tokens sit past position 8,192 + 260: most of it is fed without
    asking for logits (in portions of 2,048), then 8 tokens as a portion and 32 one by one."""
    toks = full["long_ids"]
    head = len(toks) - 40
    steps = []
    for s0 in range(0, head, 2048):
        steps.append({"step": len(steps), "end": [], "entries": [{"id": "long", "tokens": toks[s0:min(head, s0 + 2048)], "want": []}]})
    steps.append({"step": len(steps), "end": [], "entries": [{"id": "long", "tokens": toks[head:head + 8], "want": list(range(8))}]})
    for t in toks[head + 8:]:
        steps.append({"step": len(steps), "end": [], "entries": [{"id": "long", "tokens": [t], "want": [0]}]})
    steps[-1]["end"] = ["long"]
    got = replay(full[which], steps)["long"]
    check_status()
    want = full["long_want"]
    dtype = which.split("+")[0]
    bad = T.first_bad(got, want, T.tolerance(dtype, float(np.abs(want).max())))
    assert bad is None, (f"{which}: first differs at token {bad} of the last 40, "
                         f"|diff| = {np.abs(got[bad] - want[bad]).max():.3e}")
    # the comparison can fail: without the rescale these logits are somewhere else
    assert np.abs(want).max() > 1.0
