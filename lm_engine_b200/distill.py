"""``python -m lm_engine_b200.distill --config distill.yml``: training with a frozen teacher and a KL term
(lm_engine/distill.py:5-10)."""

from __future__ import annotations

from .arguments import DistillationArgs
from .train import main

if __name__ == "__main__":
    main(DistillationArgs)
