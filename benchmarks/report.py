#!/usr/bin/env python
"""Markdown tables from a directory of benchmark results, and regression checks.

    python benchmarks/report.py DIR                    one table per result file in DIR
    python benchmarks/report.py --compare REF NEW      cells of NEW worse than REF by more than
                                                       --tolerance (default 10 %); exit 1 if any

A result file is what a benchmark of this directory writes with ``--out`` (one JSON object with a
``bench`` name and ``rows``), or the single JSON line of ``bench.py``.  Columns whose name says time
(``*_us``, ``*_ms``, ``ms_per_*``, ``round_us``) count as lower-is-better in ``--compare``; rates
(``*_gbs``, ``gbs``, ``*_tflops``, ``tokens_per_s``, ``value``, ``speedup``) as higher-is-better; the
rest identify a row.  Same role as the reference's experiments/bench/report.py:1-40.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

LOWER = ("_us", "_ms", "ms_per_step", "ms_per_token", "round_us", "us_per_round", "latency")
HIGHER = ("_gbs", "gbs", "_tflops", "tokens_per_s", "value", "speedup", "frac_of_roof", "busbw")


def load(path: Path) -> dict:
    text = path.read_text().strip()
    try:
        data = json.loads(text)
    except json.JSONDecodeError:
        data = json.loads(text.splitlines()[-1])   # a log whose last line is the JSON record
    if "rows" not in data:                         # bench.py: one record, no rows
        flat = {k: v for k, v in data.items() if isinstance(v, (int, float, str)) and k != "data"}
        if isinstance(data.get("e2e"), dict):
            flat["e2e_value"] = data["e2e"].get("value")
        data = {"bench": data.get("metric", path.stem), "rows": [flat]}
    return data


def direction(column: str) -> int:
    """-1 lower is better, +1 higher is better, 0 identifies the row."""
    if any(column.endswith(s) or column == s for s in LOWER):
        return -1
    if any(column.endswith(s) or column == s for s in HIGHER):
        return 1
    return 0


def cell(value) -> str:
    if isinstance(value, float):
        return f"{value:.4g}"
    if isinstance(value, (dict, list)):
        return json.dumps(value)[:40]
    return str(value)


def table(data: dict) -> str:
    rows = data["rows"]
    columns: list[str] = []
    for row in rows:
        columns += [c for c in row if c not in columns]
    out = [f"### {data.get('bench', '?')}" + (f" ({data['n_gpus']} GPUs)" if "n_gpus" in data else ""), "",
           "| " + " | ".join(columns) + " |", "|" + "---|" * len(columns)]
    out += ["| " + " | ".join(cell(row.get(c, "")) for c in columns) + " |" for row in rows]
    return "\n".join(out)


def key_of(row: dict) -> tuple:
    return tuple((k, cell(v)) for k, v in row.items() if direction(k) == 0 and not isinstance(v, (dict, list)))


def compare(ref: dict, new: dict, tolerance: float) -> list[str]:
    worse = []
    index = {key_of(r): r for r in ref["rows"]}
    for row in new["rows"]:
        base = index.get(key_of(row))
        if base is None:
            continue
        for column, value in row.items():
            sign = direction(column)
            old = base.get(column)
            if not sign or not isinstance(value, (int, float)) or not isinstance(old, (int, float)) or not old:
                continue
            change = (value - old) / abs(old) * -sign      # positive = worse
            if change > tolerance:
                label = ", ".join(f"{k}={v}" for k, v in key_of(row))
                worse.append(f"{new.get('bench', '?')} [{label}] {column}: {cell(old)} -> {cell(value)} "
                             f"({change * 100:+.1f} % worse)")
    return worse


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("paths", nargs="+")
    ap.add_argument("--compare", action="store_true")
    ap.add_argument("--tolerance", type=float, default=0.10)
    args = ap.parse_args(argv)
    if args.compare:
        if len(args.paths) != 2:
            ap.error("--compare takes REF and NEW (two files, or two directories with files of the same names)")
        ref, new = map(Path, args.paths)
        pairs = [(ref, new)] if ref.is_file() else [(p, new / p.name) for p in sorted(ref.glob("*.json"))
                                                    if (new / p.name).exists()]
        worse = [line for a, b in pairs for line in compare(load(a), load(b), args.tolerance)]
        print("\n".join(worse) if worse else f"no cell worse by more than {args.tolerance * 100:.0f} %")
        return 1 if worse else 0
    for name in args.paths:
        path = Path(name)
        for file in (sorted(path.glob("*.json")) if path.is_dir() else [path]):
            try:
                print(table(load(file)), end="\n\n")
            except (json.JSONDecodeError, KeyError, IndexError) as error:
                print(f"(skipped {file.name}: {error})", file=sys.stderr)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
