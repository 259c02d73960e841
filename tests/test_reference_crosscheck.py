"""The plain implementation against the reference project's own model code, live.

Runs wherever the reference's sources can be found (``MINI_INFER_REFERENCE_SRC``, or a
checkout named ``reference`` beside this repository) and is skipped elsewhere; the stored
outputs under ``tests/golden`` cover the same ground where it cannot run.  Fresh prompts
(not the stored ones), all three tiny configurations, several ways of cutting the prompt
into portions, and for configuration A a prompt far past ``original_max_position_embeddings``
(64), so that the rescaled rotary frequencies decide the result.
"""

import numpy as np
import pytest
import torch

import plain_impl as P
from reference_oracle import find_reference_src, reference_logits
from tiny_configs import PAGE_SIZE, TINY, load_state, prompt_ids

REF = find_reference_src()
pytestmark = pytest.mark.skipif(REF is None, reason="the reference project's sources are not here")


@pytest.mark.parametrize("which,length,cuts", [
    ("A", 230, [64, 65, 130]),          # crosses the original context length inside and between portions
    ("A", 17, []),
    ("B", 41, [1, 9, 24]),
    ("C", 150, [100]),
])
def test_plain_matches_the_reference_live(which, length, cuts, model_dirs):
    state = load_state(model_dirs[which])
    ids = prompt_ids(which, length, salt=99)
    ref, inv_freq = reference_logits(REF, TINY[which], state, ids, PAGE_SIZE[which], cuts)
    cfg = P.normalise_config(TINY[which])
    assert np.array_equal(P.rope_inv_freq(cfg["head_dim"], cfg["_theta"], cfg["_scaling"]).numpy(), inv_freq.numpy())
    plain32 = P.llama_logits(state, TINY[which], ids, dtype=torch.float32)
    plain64 = P.llama_logits(state, TINY[which], ids, dtype=torch.float64)
    scale = max(1.0, ref.abs().max().item())
    assert (plain32 - ref).abs().max().item() <= 2e-5 * scale
    assert (plain64.float() - ref).abs().max().item() <= 1e-4 * scale
    # the comparison can fail: without the rescale the logits past the original length move
    if which == "A" and length > 64:
        raw = dict(TINY[which], rope_scaling=None)
        other = P.llama_logits(state, raw, ids, dtype=torch.float32)
        assert (other - ref).abs().max().item() > 1e-3 * scale
