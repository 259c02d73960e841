"""Makes ``tests/golden/tiny_{A,B}.npz`` from the reference project's own CPU fp32 code.

Run once, by hand, where the reference's sources are available:

    python tests/golden/make_golden.py /path/to/reference/src

For each tiny configuration it writes the seeded random model folder with this
package's random-weights mode, loads it into the reference's ``LlamaForCausalLM`` through
the reference's HF-name loader, runs a prompt through the reference's paged cache in two
portions (its cached path, ``attention_backend="torch"``, float32) and stores: the
prompt, the logits of every position, the reference's ``inv_freq`` table, and a checksum
of the weights (so a change of the random generator is noticed).  ``test_plain_impl.py``
compares the plain implementation with these files.
"""

import hashlib
import os
import sys
import tempfile
from types import SimpleNamespace

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tiny_configs import PAGE_SIZE, TINY, load_state, make_model_dir, prompt_ids  # noqa: E402


def weights_checksum(state):
    h = hashlib.sha256()
    for name in sorted(state):
        h.update(name.encode())
        h.update(state[name].float().numpy().tobytes())
    return h.hexdigest()


def main(ref_src: str) -> None:
    os.environ["HF_HUB_OFFLINE"] = "1"
    os.environ["TRANSFORMERS_OFFLINE"] = "1"
    sys.path.insert(0, ref_src)
    from mini_infer.cache.block_pool import BlockPool
    from mini_infer.cache.paged_kv_cache import PagedKVCache
    from mini_infer.engine.model_runner import ModelRunner
    from mini_infer.models.llama.llama import LlamaConfig, LlamaForCausalLM

    for which, length in (("A", 48), ("B", 63)):
        raw = TINY[which]
        folder = make_model_dir(which, tempfile.mkdtemp())
        state = load_state(folder)
        cfg = LlamaConfig.from_hf(SimpleNamespace(**raw))
        model = LlamaForCausalLM(cfg).eval().float()
        LlamaForCausalLM.load_weights(model, {k: v.float() for k, v in state.items()})
        pool = BlockPool(num_blocks=64, block_size=PAGE_SIZE[which], num_layers=cfg.num_hidden_layers,
                         num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                         dtype=torch.float32, device="cpu", attention_backend="torch")
        runner = ModelRunner(model=model, tokenizer=None, device="cpu", block_pool=pool)
        cache = PagedKVCache(pool)
        cache.add_request_slot()
        ids = prompt_ids(which, length)
        cut = length // 2 + 3
        first = runner.forward_step_packed(cache, ids[:cut], [0, cut], [0])
        second = runner.forward_step_packed(cache, ids[cut:], [0, length - cut], [cut])
        logits = torch.cat([first[0], second[0]], dim=0).float().numpy()
        out = os.path.join(HERE, f"tiny_{which}.npz")
        np.savez_compressed(
            out,
            prompt=np.array(ids, dtype=np.int32),
            logits=logits.astype(np.float32),
            inv_freq=model.rotary_emb.inv_freq.numpy().astype(np.float32),
            weights_sha256=np.array(weights_checksum(state)),
        )
        print(out, logits.shape, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <the reference project's src folder>")
    main(sys.argv[1])
