#!/bin/bash
# Tokenises a directory of jsonl / parquet shards into .bin/.idx pairs and merges them into shards of at most 50 GB.
#   launch/preprocess_data.sh <input dir> <tokenizer dir> <output dir> [workers]
set -euo pipefail
INPUT=${1:?input directory}; TOKENIZER=${2:?tokenizer}; OUTPUT=${3:?output directory}; WORKERS=${4:-32}
python -m lm_engine_b200.data.preprocess --input "$INPUT" --tokenizer "$TOKENIZER" --append-eod \
    --output-prefix "$OUTPUT/shards" --workers "$WORKERS"
python -m lm_engine_b200.data.merge merge --input-directory "$OUTPUT/shards" --output-prefix "$OUTPUT/merged" \
    --max-size 50 --workers "$WORKERS"
python -m lm_engine_b200.data.merge list --input-directory "$OUTPUT/merged"
