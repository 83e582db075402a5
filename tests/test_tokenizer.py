"""The tokenizer glue: ``load_tokenizer`` (tokenizer.json + tokenizer_config.json, as llama4/llama4_jax/model.py:234-246
reads them), ``encode_chat`` (llama4/main.py:29-39) and the command line's ``--prompt``.  The tokenizer is a tiny
word-level one that the test writes itself."""

import json
import subprocess
import sys

import pytest

from tests import helpers as H

WORDS = "the quick brown fox jumps over lazy dog hello world what is your name tell me a story".split()
SPECIAL = ["<|begin_of_text|>", "<|header_start|>", "<|header_end|>", "<|eot|>", "<unk>"]
TEMPLATE = ("{{ bos_token }}{% for m in messages %}<|header_start|>{{ m['role'] }}<|header_end|> {{ m['content'] }} <|eot|>"
            "{% endfor %}")


def write_tokenizer(folder):
    from tokenizers import Tokenizer, models, pre_tokenizers

    names = SPECIAL + ["user", "assistant"] + WORDS
    names += [f"w{i}" for i in range(256 - len(names))]  # as many entries as the tiny models' vocabulary has
    vocab = {w: i for i, w in enumerate(names)}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.add_special_tokens(SPECIAL)
    tok.save(str(folder / "tokenizer.json"))
    added = {str(i): {"content": s, "lstrip": False, "normalized": False, "rstrip": False, "single_word": False, "special": True}
             for i, s in enumerate(SPECIAL)}
    (folder / "tokenizer_config.json").write_text(json.dumps({
        "added_tokens_decoder": added, "bos_token": "<|begin_of_text|>", "eos_token": "<|eot|>",
        "unk_token": {"content": "<unk>", "lstrip": False, "normalized": False, "rstrip": False, "single_word": False},
        "chat_template": TEMPLATE, "clean_up_tokenization_spaces": False, "model_max_length": 4096}))
    return vocab


def test_load_tokenizer_and_encode_chat(tmp_path):
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.tokenizer import encode_chat

    vocab = write_tokenizer(tmp_path)
    tok = J.load_tokenizer(tmp_path / "tokenizer.json", tmp_path / "tokenizer_config.json")
    assert tok.bos_token == "<|begin_of_text|>" and tok.eos_token == "<|eot|>" and tok.unk_token == "<unk>"
    assert tok.encode("hello world") == [vocab["hello"], vocab["world"]]
    ids = encode_chat(tok, "tell me a story")
    want = ["<|begin_of_text|>", "<|header_start|>", "user", "<|header_end|>", "tell", "me", "a", "story", "<|eot|>",
            "<|header_start|>", "assistant", "<|header_end|>"]  # the user's turn, then the assistant's header
    assert ids == [vocab[w] for w in want]
    assert tok.decode(ids[4:8]) == "tell me a story"


@pytest.mark.gpu
def test_command_line_with_a_text_prompt(tmp_path):
    folder = H.make_model_dir(tmp_path / "m", "tiny_a", seed=0)
    vocab = write_tokenizer(folder)
    cmd = [sys.executable, "-m", "jax_llm_examples_b200.main", "--model", str(folder), "--dtype", "float32",
           "--prompt", "what is your name", "--max-new-tokens", "5", "--page-size", "16"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=H.ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.tokenizer import encode_chat

    tok = J.load_tokenizer(folder / "tokenizer.json", folder / "tokenizer_config.json")
    prompt = encode_chat(tok, "what is your name")
    want = J.generate(J.load_model(folder, "float32"), [prompt], J.SamplingParams(max_new_tokens=5), page_size=16)[0]
    assert len(tok.decode(want).split()) >= 1 and tok.decode(want) in out.stdout, (tok.decode(want), out.stdout)
