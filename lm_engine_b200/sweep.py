"""``python -m lm_engine_b200.sweep``: hyper-parameter sweeps over training configs without an external service.

Reads the reference's sweep file format (``method``, ``metric``, ``parameters`` keyed by dotted config paths with
``values`` or ``distribution / min / max``; tools/wandb_sweep.py:55-441 drives the same file through a W&B sweep
controller and a Slurm agent submitter).  Here the controller is local: ``grid`` enumerates, ``random`` (and ``bayes``,
which falls back to it: there is no W&B server to ask) samples with a seeded generator.  For every trial the base
config is copied, the sampled values are written at their dotted paths, ``save_args.save_path`` and
``logging_args.experiments_tracker_name`` are made unique, and the config is written to ``<out>/trial-<i>/config.yml``.
``--launch`` is a command template run per trial (``{config}``, ``{trial}``, ``{dir}``), e.g.
``--launch "sbatch launch/slurm.sbatch {config}"``; ``collect`` reads each trial's ``metrics.jsonl`` and ranks the
trials by the sweep's metric.
"""

from __future__ import annotations

import argparse
import copy
import itertools
import json
import math
import os
import random
import shlex
import subprocess

import yaml


def deep_set(d: dict, dotpath: str, value) -> None:
    keys = dotpath.split(".")
    for key in keys[:-1]:
        d = d.setdefault(key, {})
    d[keys[-1]] = value


def _sample(spec: dict, rng: random.Random):
    if "value" in spec:
        return spec["value"]
    if "values" in spec:
        return rng.choice(spec["values"])
    dist = spec.get("distribution", "uniform")
    lo, hi = spec["min"], spec["max"]
    if dist in ("log_uniform_values", "log_uniform"):
        return math.exp(rng.uniform(math.log(lo), math.log(hi)))
    if dist == "int_uniform":
        return rng.randint(int(lo), int(hi))
    if dist == "q_uniform":
        q = spec.get("q", 1)
        return round(rng.uniform(lo, hi) / q) * q
    return rng.uniform(lo, hi)


def generate_trials(sweep: dict, count: int | None, seed: int = 0) -> list[dict]:
    params = sweep["parameters"]
    method = sweep.get("method", "random")
    if method == "grid":
        keys = list(params)
        axes = [[p["value"]] if "value" in p else p["values"] for p in (params[k] for k in keys)]
        trials = [dict(zip(keys, combo)) for combo in itertools.product(*axes)]
        return trials if count is None else trials[:count]
    rng = random.Random(seed)
    return [{k: _sample(p, rng) for k, p in params.items()} for _ in range(count or 8)]


def materialise(base: dict, trials: list[dict], out: str, name: str = "sweep") -> list[str]:
    paths = []
    for i, trial in enumerate(trials):
        cfg = copy.deepcopy(base)
        for path, value in trial.items():
            deep_set(cfg, path, value)
        d = os.path.join(out, f"trial-{i}")
        os.makedirs(d, exist_ok=True)
        deep_set(cfg, "save_args.save_path", os.path.join(d, "checkpoints"))
        if cfg.get("logging_args", {}).get("experiments_tracker_name") is not None:
            deep_set(cfg, "logging_args.experiment_name", f"{name}-{i}")
        with open(os.path.join(d, "config.yml"), "w") as f:
            yaml.safe_dump(cfg, f, sort_keys=False)
        with open(os.path.join(d, "trial.json"), "w") as f:
            json.dump(trial, f, indent=1)
        paths.append(os.path.join(d, "config.yml"))
    return paths


def collect(out: str, metric: str, goal: str = "minimize") -> list[tuple[int, float, dict]]:
    """Last logged value of ``metric`` (``context/name``, e.g. ``train/lm_loss``) per trial, best first."""
    ctx, _, key = metric.partition("/")
    rows = []
    for d in sorted(os.listdir(out)):
        if not d.startswith("trial-"):
            continue
        log = os.path.join(out, d, "metrics.jsonl")
        value = None
        if os.path.isfile(log):
            for line in open(log):
                rec = json.loads(line)
                if rec.get("context", ctx) == ctx and key in rec:
                    value = rec[key]
        if value is not None:
            rows.append((int(d.split("-")[1]), float(value), json.load(open(os.path.join(out, d, "trial.json")))))
    return sorted(rows, key=lambda r: r[1], reverse=goal == "maximize")


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m lm_engine_b200.sweep")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate")
    g.add_argument("--sweep", required=True, help="sweep description (method / metric / parameters)")
    g.add_argument("--config", required=True, help="base training config")
    g.add_argument("--out", required=True)
    g.add_argument("--count", type=int, default=None)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--launch", default=None, help="command template per trial: {config} {trial} {dir}")
    c = sub.add_parser("collect")
    c.add_argument("--sweep", required=True)
    c.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    sweep = yaml.safe_load(open(a.sweep))
    if a.cmd == "collect":
        m = sweep.get("metric", {"name": "train/lm_loss", "goal": "minimize"})
        for i, v, trial in collect(a.out, m["name"], m.get("goal", "minimize")):
            print(f"trial {i:3d}  {m['name']} = {v:.6g}  {trial}")
        return 0
    base = yaml.safe_load(open(a.config))
    trials = generate_trials(sweep, a.count, a.seed)
    paths = materialise(base, trials, a.out)
    for i, p in enumerate(paths):
        print(p)
        if a.launch:
            cmd = a.launch.format(config=p, trial=i, dir=os.path.dirname(p))
            subprocess.run(shlex.split(cmd), check=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
