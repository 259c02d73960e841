"""Makes ``tests/golden/tiny_{A,B,C}.npz`` from the reference project's own CPU fp32 code.

Run once, by hand, where the reference's sources are available:

    python tests/golden/make_golden.py /path/to/reference/src

For each tiny configuration it writes the seeded random model folder with this
package's random-weights mode, loads it into the reference's ``LlamaForCausalLM`` through
the reference's HF-name loader, runs a prompt through the reference's paged cache in two
portions (its cached path, ``attention_backend="torch"``, float32; see
``tests/reference_oracle.py``) and stores: the prompt, the logits of every position, the
reference's ``inv_freq`` table, and a checksum of the weights (so a change of the random
generator is noticed).  Configuration A's prompt is longer than its
``original_max_position_embeddings``, so the rescaled frequencies matter.
``test_plain_impl.py`` compares the plain implementation with these files.
"""

import hashlib
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from reference_oracle import reference_logits  # noqa: E402
from tiny_configs import PAGE_SIZE, TINY, load_state, make_model_dir, prompt_ids  # noqa: E402

LENGTHS = {"A": 100, "B": 63, "C": 80}


def weights_checksum(state):
    h = hashlib.sha256()
    for name in sorted(state):
        h.update(name.encode())
        h.update(state[name].float().numpy().tobytes())
    return h.hexdigest()


def main(ref_src: str) -> None:
    for which, length in LENGTHS.items():
        folder = make_model_dir(which, tempfile.mkdtemp())
        state = load_state(folder)
        ids = prompt_ids(which, length)
        logits, inv_freq = reference_logits(ref_src, TINY[which], state, ids, PAGE_SIZE[which], [length // 2 + 3])
        out = os.path.join(HERE, f"tiny_{which}.npz")
        np.savez_compressed(
            out,
            prompt=np.array(ids, dtype=np.int32),
            logits=logits.numpy().astype(np.float32),
            inv_freq=inv_freq.numpy().astype(np.float32),
            weights_sha256=np.array(weights_checksum(state)),
        )
        print(out, tuple(logits.shape), os.path.getsize(out), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <the reference project's src folder>")
    main(sys.argv[1])
