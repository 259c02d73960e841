"""Two tiny Llama configurations that differ in every size and option, and helpers to
make model folders from them in a temporary place."""

from __future__ import annotations

import os
import tempfile

import torch

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 512,
    "hidden_size": 64,
    "intermediate_size": 176,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 8.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 64,
    },
    "max_position_embeddings": 512,
    "tie_word_embeddings": False,
    "attention_bias": False,
    "mlp_bias": False,
    "hidden_act": "silu",
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 1000,
    "hidden_size": 192,
    "intermediate_size": 320,
    "num_hidden_layers": 3,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 32,
    "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": None,
    "max_position_embeddings": 1024,
    "tie_word_embeddings": True,
}

# A third one whose sizes put the Blackwell-specific kernels on the engine's path: head size
# 64 with a group of 4 and pages of 16 (the tcgen05 prefill kernel), widths that are multiples
# of 8 (the TMA / tcgen05 product for decode-sized inputs).
TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 640,
    "hidden_size": 256,
    "intermediate_size": 384,
    "num_hidden_layers": 2,
    "num_attention_heads": 8,
    "num_key_value_heads": 2,
    "head_dim": 64,
    "rms_norm_eps": 1e-5,
    "rope_theta": 100000.0,
    "rope_scaling": None,
    "max_position_embeddings": 2048,
    "tie_word_embeddings": False,
}

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
PAGE_SIZE = {"A": 16, "B": 8, "C": 16}
SEED = {"A": 11, "B": 23, "C": 37}

# Attention that is almost uniform hides position and cache faults; q and k projections
# drawn this wide make single keys stand out (the reference's own rope test widens them
# too, tests/unit/models/llama/test_llama_rope_scaling.py:83-92).
# The width is sqrt(2.5 / hidden_size): attention scores then have a standard deviation of
# about 2.5, peaked enough to show a wrong key, mild enough for bfloat16 to follow.
def peaked(which: str) -> dict:
    s = (2.5 / TINY[which]["hidden_size"]) ** 0.5
    return {"q_proj": s, "k_proj": s}


PEAKED = {w: peaked(w) for w in TINY}


def make_model_dir(which: str, root: str | None = None, peaked: bool = True) -> str:
    from mini_infer_b200.weights import write_random_model

    root = root or tempfile.mkdtemp(prefix="mini_infer_test_")
    out = os.path.join(root, f"tiny_{which}{'_peaked' if peaked else ''}")
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        write_random_model(TINY[which], out, SEED[which], std_overrides=PEAKED[which] if peaked else None)
    return out


def load_state(model_dir: str) -> dict[str, torch.Tensor]:
    from mini_infer_b200.weights import Checkpoint

    with Checkpoint(model_dir) as ck:
        return {n: ck.read(n) for n in ck.names()}


def prompt_ids(which: str, length: int, salt: int = 0) -> list[int]:
    g = torch.Generator().manual_seed(1000 * SEED[which] + 7 * length + salt)
    return torch.randint(0, TINY[which]["vocab_size"], (length,), generator=g).tolist()
