"""Puts the unmodified reference (Leon-CYL/DistEngine) under ``baseline/_ref`` so that
``bench.py --impl reference`` can run it on the GPU box.

    python baseline/install_reference.py [--source DIR]

First the offline ``pip install --target baseline/_ref`` is tried.  Its build backend (hatchling)
is not available offline, so that fails; the wheel it would build is, by the project's own
``[tool.hatch.build.targets.wheel] packages`` list (pyproject.toml:21-22), exactly four pure-Python
package folders, and installing it means copying them.  That is what happens then: the four
folders are copied file for file, nothing is changed, and ``INSTALLED.json`` records where they
came from and a digest of every file.  ``baseline/_ref`` is not committed.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")
PACKAGES = ("distengine", "models", "layers", "utils")      # src/<name> in the reference's tree


def try_pip(source: str) -> tuple[bool, str]:
    with tempfile.TemporaryDirectory() as scratch:
        copy = os.path.join(scratch, "reference")            # the build may write into its tree
        shutil.copytree(source, copy)
        proc = subprocess.run(
            [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation",
             "--no-deps", "--find-links", "/opt/wheelhouse", "--target", TARGET, copy],
            capture_output=True, text=True)
    tail = (proc.stderr or proc.stdout).strip().splitlines()[-1:] or [""]
    return proc.returncode == 0, tail[0]


def copy_packages(source: str) -> dict[str, str]:
    digests: dict[str, str] = {}
    for name in PACKAGES:
        src = os.path.join(source, "src", name)
        dst = os.path.join(TARGET, name)
        if not os.path.isdir(src):
            raise SystemExit(f"{src} is missing: not the reference's tree")
        shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__"))
        for root, _, files in os.walk(dst):
            for file in sorted(files):
                path = os.path.join(root, file)
                with open(path, "rb") as handle:
                    digests[os.path.relpath(path, TARGET)] = hashlib.sha256(
                        handle.read()).hexdigest()
    return digests


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--source", default="/root/reference")
    args = parser.parse_args()
    if os.path.isdir(TARGET):
        shutil.rmtree(TARGET)
    ok, message = try_pip(args.source)
    record = {"source": args.source, "pip": "ok" if ok else f"failed: {message}"}
    if not ok:
        if os.path.isdir(TARGET):
            shutil.rmtree(TARGET)
        os.makedirs(TARGET)
        record["how"] = "copied the wheel's package folders unmodified"
        record["files"] = copy_packages(args.source)
    with open(os.path.join(TARGET, "INSTALLED.json"), "w") as out:
        json.dump(record, out, indent=1, sort_keys=True)
    print(f"reference under {TARGET}: pip {record['pip']}; "
          f"{len(record.get('files', {}))} files copied")
    return 0


if __name__ == "__main__":
    sys.exit(main())
