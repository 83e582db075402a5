"""The tokenizer of a model folder, for callers that start from text.  Token ids are the engine's own
interface (a random-weights model has no tokenizer); this is the reference's helper under its name."""

from __future__ import annotations

import json
import os
from pathlib import Path


def load_tokenizer(tokenizer_path: "str | os.PathLike[str]", tokenizer_config_path: "str | os.PathLike[str]"):
    """tokenizer.json and tokenizer_config.json -> a fast tokenizer with the config's special tokens
    (llama4/llama4_jax/model.py:234-246).  Needs the `transformers` package (its tokenizer classes only)."""
    from transformers import AddedToken, PreTrainedTokenizerFast

    def token(v):
        return AddedToken(**v) if isinstance(v, dict) else v

    raw = json.loads(Path(tokenizer_config_path).read_text())
    config = {k: token(v) if str(k).endswith("token") else v for k, v in raw.items()}
    config["added_tokens_decoder"] = {int(k): AddedToken(**v) for k, v in raw.get("added_tokens_decoder", {}).items()}
    return PreTrainedTokenizerFast(tokenizer_file=str(tokenizer_path), **config)


def encode_chat(tokenizer, text: str) -> list[int]:
    """A user message through the chat template, followed by the assistant header, as the reference prepares
    its prompts (llama4/main.py:29-39, without the padding that a fixed batch shape needs there)."""
    ids = tokenizer.apply_chat_template([{"role": "user", "content": text}])
    ids = getattr(ids, "input_ids", ids)
    return list(ids) + list(tokenizer.encode("<|header_start|>assistant<|header_end|>"))
