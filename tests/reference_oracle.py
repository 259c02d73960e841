"""Runs the reference project's own model code on the CPU in float32, for tests.

Used by ``tests/golden/make_golden.py`` (stored outputs) and by
``tests/test_reference_crosscheck.py`` (a live comparison that runs wherever the reference's
sources can be found and is skipped elsewhere).  Nothing of the package under test is used
here except the reader of its own model folders.

The reference is driven the way its own chunked-prefill test drives it
(``tests/unit/models/llama/test_llama_rope_scaling.py:99-121``): ``LlamaConfig.from_hf`` on
the raw ``config.json`` keys, ``LlamaForCausalLM.load_weights`` with Hugging Face tensor names,
a ``BlockPool`` / ``PagedKVCache`` with the torch attention backend, and
``ModelRunner.forward_step_packed`` portion by portion.
"""

from __future__ import annotations

import os
import sys
from types import SimpleNamespace

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def find_reference_src() -> str | None:
    """The reference's ``src`` folder: ``MINI_INFER_REFERENCE_SRC``, or a checkout named
    ``reference`` beside this repository."""
    candidates = [os.environ.get("MINI_INFER_REFERENCE_SRC"),
                  os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference", "src")]
    for c in candidates:
        if c and os.path.isfile(os.path.join(c, "mini_infer", "models", "llama", "llama.py")):
            return c
    return None


def reference_logits(ref_src: str, raw_config: dict, state: dict, ids: list[int], page_size: int,
                     cuts: list[int]):
    """``(logits [T, vocab] float32, the model's inv_freq table)`` of the reference's fp32 CPU
    path, the prompt fed in portions that end at ``cuts`` (and at its end)."""
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    if ref_src not in sys.path:
        sys.path.insert(0, ref_src)
    from mini_infer.cache.block_pool import BlockPool
    from mini_infer.cache.paged_kv_cache import PagedKVCache
    from mini_infer.engine.model_runner import ModelRunner
    from mini_infer.models.llama.llama import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig.from_hf(SimpleNamespace(**raw_config))
    model = LlamaForCausalLM(cfg).eval().float()
    LlamaForCausalLM.load_weights(model, {k: v.float() for k, v in state.items()})
    pool = BlockPool(num_blocks=-(-len(ids) // page_size) + 4, block_size=page_size,
                     num_layers=cfg.num_hidden_layers, num_kv_heads=cfg.num_key_value_heads,
                     head_dim=cfg.head_dim, dtype=torch.float32, device="cpu", attention_backend="torch")
    runner = ModelRunner(model=model, tokenizer=None, device="cpu", block_pool=pool)
    cache = PagedKVCache(pool)
    cache.add_request_slot()
    edges = sorted(set(c for c in cuts if 0 < c < len(ids))) + [len(ids)]
    out, start = [], 0
    with torch.no_grad():
        for end in edges:
            part = runner.forward_step_packed(cache, ids[start:end], [0, end - start], [start])
            out.append(part[0].float())
            start = end
    return torch.cat(out, dim=0), model.rotary_emb.inv_freq.detach().float().clone()
