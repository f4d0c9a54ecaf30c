"""Access to the unmodified reference package (installed under baseline/_ref) for parity tests; tests that need it
skip when it is absent."""

import os
import sys

import pytest

_REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


def reference():
    if not os.path.isdir(os.path.join(_REF, "lm_engine")):
        pytest.skip("reference package not installed under baseline/_ref")
    if _REF not in sys.path:
        sys.path.append(_REF)
    import lm_engine  # noqa: F401
    from lm_engine.hf_adapter import get_causal_lm_class
    from lm_engine.models import GPTBaseConfig

    return get_causal_lm_class, GPTBaseConfig


def build_reference_model(cfg_dict: dict, **kwargs):
    import warnings

    get_causal_lm_class, _ = reference()
    cls = get_causal_lm_class(cfg_dict["model_type"])
    cfg = cls.config_class(**cfg_dict)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        return cls(cfg, **kwargs)
