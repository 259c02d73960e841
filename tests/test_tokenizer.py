"""The optional text front end: a tokenizer file in the model folder, the beginning-of-sequence
id prepended when the tokenizer does not add it (the reference's rule, ``engine/tokenizer.py:71-90``)."""

from __future__ import annotations

import json
import os

import pytest

tokenizers = pytest.importorskip("tokenizers")

from mini_infer_b200.engine.tokenizer import Tokenizer  # noqa: E402


def _folder(tmp_path, config):
    from tokenizers import Tokenizer as Backend
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    vocab = {"<s>": 0, "</s>": 1, "<unk>": 2, "the": 3, "cat": 4, "sat": 5}
    backend = Backend(WordLevel(vocab, unk_token="<unk>"))
    backend.pre_tokenizer = Whitespace()
    backend.add_special_tokens(["<s>", "</s>"])
    backend.save(os.path.join(tmp_path, "tokenizer.json"))
    with open(os.path.join(tmp_path, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config, f)
    return str(tmp_path)


def test_bos_is_prepended_once_and_text_comes_back(tmp_path):
    tk = Tokenizer.from_pretrained(_folder(tmp_path, {"bos_token_id": 0, "eos_token_id": [1, 7]}))
    assert tk.encode("the cat sat") == [0, 3, 4, 5]
    assert tk.encode("<s> the") == [0, 3]            # already there: not doubled
    assert tk.encode("") == [0]
    assert tk.decode([3, 4]) == "the cat"
    assert tk.eos_token_id == 1                      # the first of a list


def test_without_a_bos_id_nothing_is_added(tmp_path):
    tk = Tokenizer.from_pretrained(_folder(tmp_path, {}))
    assert tk.encode("the dog") == [3, 2]
    assert tk.bos_token_id is None and tk.eos_token_id is None


def test_a_folder_without_tokenizer_json_is_an_error(tmp_path):
    with pytest.raises(FileNotFoundError, match="tokenizer.json"):
        Tokenizer.from_pretrained(str(tmp_path))


def test_the_scheduler_takes_text_through_it(tmp_path):
    """A text prompt is encoded on submit and the result carries decoded text; without a
    tokenizer a text prompt is refused."""
    from test_scheduler import make

    from mini_infer_b200.engine import Request

    tk = Tokenizer.from_pretrained(_folder(tmp_path, {"bos_token_id": 0}))
    runner, sched = make(num_pages=16, tokenizer=tk)
    out = sched.generate([Request("the cat", max_tokens=3)])[0]
    assert out.prompt_tokens == 3 and len(out.tokens) == 3
    assert runner.fed[0][:3] == [0, 3, 4]            # what the step function was given
    assert out.text == tk.decode(out.tokens)
    _, plain = make(num_pages=16)
    with pytest.raises(ValueError, match="tokenizer"):
        plain.submit(Request("the cat"))
