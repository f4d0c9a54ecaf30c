"""Template markers of the finetuning data formats and the multi-storage URL prefix (lm_engine/defaults.py:5-8)."""

INPUT_FORMAT = "__input__"
OUTPUT_FORMAT = "__output__"
MSC_PREFIX = "msc://"
