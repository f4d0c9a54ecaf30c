"""Tokenizers: HuggingFace ``AutoTokenizer`` from a local directory, or the built-in character-level
``AlphaNumericTokenizer`` (selected with ``tokenizer_name: alpha_numeric``); lm_engine/tokenizers/__init__.py:10-20."""

from __future__ import annotations

from .alpha_numeric import AlphaNumericTokenizer

_CUSTOM = {"alpha_numeric": AlphaNumericTokenizer, "AlphaNumericTokenizer": AlphaNumericTokenizer}


def get_tokenizer(tokenizer_name: str, **kwargs):
    if tokenizer_name in _CUSTOM:
        return _CUSTOM[tokenizer_name]()
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(tokenizer_name, **kwargs)
