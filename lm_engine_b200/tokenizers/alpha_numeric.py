"""Character-level tokenizer over ``[0-9a-zA-Z]`` backed by the native host library
(lm_engine/tokenizers/alpha_numeric/__init__.py:14-64).  Ids: digits 0-9, lower case 10-35, upper case 36-61,
``<|endoftext|>`` (EOS and padding) 62."""

from __future__ import annotations

import ctypes

import numpy as np

from ..ops._lib import host_lib


class AlphaNumericTokenizer:
    eos_token = pad_token = bos_token = "<|endoftext|>"
    eos_token_id = pad_token_id = bos_token_id = 62
    vocab_size = 63
    padding_side = "left"

    def __init__(self) -> None:
        lib = host_lib()
        lib.lme_alnum_encode.restype = ctypes.c_int64
        lib.lme_alnum_encode.argtypes = [ctypes.c_char_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p,
                                         ctypes.c_void_p]
        lib.lme_alnum_encode_batch.restype = ctypes.c_int64
        lib.lme_alnum_encode_batch.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
        lib.lme_alnum_decode.restype = ctypes.c_int64
        lib.lme_alnum_decode.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p,
                                         ctypes.c_int64]
        self._lib = lib

    def __len__(self) -> int:
        return self.vocab_size

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        raw = text.encode("utf-8")
        out = np.empty(len(raw) + 1, dtype=np.int32)
        bad = ctypes.c_int64(0)
        n = self._lib.lme_alnum_encode(raw, len(raw), int(add_special_tokens), out.ctypes.data, ctypes.byref(bad))
        if n < 0:
            raise ValueError(f"unsupported character {text[bad.value]!r} at position {bad.value}")
        return out[:n].tolist()

    def __call__(self, text: str | list[str], add_special_tokens: bool = False, padding: bool = False,
                 return_tensors: str | None = None, **_unused) -> dict:
        if isinstance(text, str):
            ids = self.encode(text, add_special_tokens)
            out = {"input_ids": ids, "attention_mask": [1] * len(ids)}
        else:
            raws = [t.encode("utf-8") for t in text]
            if padding:
                max_len = max(len(self.encode(t, add_special_tokens)) for t in text) if text else 0
                arr = (ctypes.c_char_p * len(raws))(*raws)
                lens = np.array([len(r) for r in raws], dtype=np.int64)
                ids = np.empty((len(raws), max_len), dtype=np.int32)
                mask = np.empty((len(raws), max_len), dtype=np.int32)
                rc = self._lib.lme_alnum_encode_batch(ctypes.cast(arr, ctypes.c_void_p), lens.ctypes.data, len(raws),
                                                      int(add_special_tokens), 1, ids.ctypes.data, mask.ctypes.data,
                                                      max_len)
                if rc < 0:
                    raise ValueError("unsupported character in batch")
                out = {"input_ids": ids.tolist(), "attention_mask": mask.tolist()}
            else:
                enc = [self.encode(t, add_special_tokens) for t in text]
                out = {"input_ids": enc, "attention_mask": [[1] * len(e) for e in enc]}
        if return_tensors == "pt":
            import torch

            out = {k: torch.tensor(v) for k, v in out.items()}
        return out

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        arr = np.asarray(ids, dtype=np.int32).reshape(-1)
        cap = arr.size * 13 + 1
        buf = ctypes.create_string_buffer(cap)
        n = self._lib.lme_alnum_decode(arr.ctypes.data, arr.size, int(skip_special_tokens), buf, cap)
        if n < 0:
            raise ValueError("token id outside the alpha-numeric vocabulary")
        return buf.raw[:n].decode("utf-8")

    def batch_decode(self, batch, skip_special_tokens: bool = False) -> list[str]:
        return [self.decode(ids, skip_special_tokens) for ids in batch]

    def add_special_tokens(self, *_args, **_kwargs) -> int:
        return 0

    def save_pretrained(self, *_args, **_kwargs) -> None:
        return None
