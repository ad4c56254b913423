"""Compare the running environment with a pinned one.

    python -m aboleth_b200.utils.environment --check repro/environment.json

The reference pins its software in repro/environment.json (repro/README.md:28-36, 91-112) and
ships a bootstrap script that installs it; an offline machine cannot install anything, so this
module only reports: for every pinned package whether it is present and at the pinned version,
the CUDA toolkit's nvcc, the Python minor version and (with a GPU) the device name.  Exit code 0
when everything marked ``required`` matches, 1 otherwise; mismatches of packages that only the
baselines use are printed as warnings.
"""
from __future__ import annotations

import argparse
import importlib.metadata as metadata
import json
import re
import shutil
import subprocess
import sys
from pathlib import Path


def installed(name: str):
    try:
        return metadata.version(name)
    except metadata.PackageNotFoundError:
        return None


def nvcc_version():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    try:
        text = subprocess.run([nvcc, "--version"], capture_output=True, text=True, timeout=20).stdout
    except (OSError, subprocess.TimeoutExpired):
        return None
    found = re.search(r"release \S+, V(\S+)", text)
    return found.group(1) if found else None


def compare(pins: dict) -> dict:
    """-> {"ok": bool, "rows": [(what, pinned, found, severity)]}; severity in ok / warn / fail."""
    rows = []
    required = set(pins.get("required", []))
    for name, pinned in pins.get("packages", {}).items():
        found = installed(name)
        if found == pinned:
            rows.append((name, pinned, found, "ok"))
        else:
            rows.append((name, pinned, found, "fail" if name in required else "warn"))
    python = "%d.%d" % sys.version_info[:2]
    rows.append(("python", pins.get("python"), python, "ok" if python == pins.get("python") else "warn"))
    pinned_nvcc = pins.get("cuda_toolkit", {}).get("nvcc")
    found_nvcc = nvcc_version()
    rows.append(("nvcc", pinned_nvcc, found_nvcc,
                 "ok" if found_nvcc == pinned_nvcc else ("fail" if found_nvcc is None else "warn")))
    try:
        import torch
        if torch.cuda.is_available():
            name = torch.cuda.get_device_name(0)
            wanted = pins.get("hardware", {}).get("gpu")
            rows.append(("gpu", wanted, name, "ok" if wanted and wanted in name else "warn"))
    except Exception:  # noqa: BLE001 - torch itself is reported above
        pass
    return {"ok": all(severity != "fail" for *_, severity in rows), "rows": rows}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--check", type=Path, required=True, help="the pinned environment (JSON)")
    args = ap.parse_args(argv)
    result = compare(json.loads(args.check.read_text()))
    for what, pinned, found, severity in result["rows"]:
        print(f"{severity:4s}  {what:24s} pinned {pinned!s:14s} found {found!s}")
    return 0 if result["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
