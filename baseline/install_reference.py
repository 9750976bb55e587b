#!/usr/bin/env python3
"""Puts the unmodified reference engine under ``baseline/_ref`` for ``bench.py --impl reference``.

    python baseline/install_reference.py [--source DIR]

It first tries the offline install (pip with no index and no build isolation, from a copy of the
source tree, since the build may write into it). The reference's build backend (hatchling) is
not in the offline wheelhouse, so that attempt fails here; the reference is pure Python (no
native code, no generated files), so its package folder ``src/turboserve`` is then copied as it
is, which is all that a wheel of it would contain. ``baseline/_ref/INSTALL.json`` records which
of the two happened and a digest of the installed files. Nothing of this repository's own
engine is placed there.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"


def digest(folder: Path) -> tuple[str, int]:
    sha = hashlib.sha256()
    count = 0
    for path in sorted(folder.rglob("*.py")):
        sha.update(str(path.relative_to(folder)).encode())
        sha.update(path.read_bytes())
        count += 1
    return sha.hexdigest()[:16], count


def pip_install(source: Path) -> str | None:
    """Returns None on success, else the last line of pip's error."""
    with tempfile.TemporaryDirectory() as tmp:
        copy = Path(tmp) / "reference"
        shutil.copytree(source, copy, ignore=shutil.ignore_patterns(".git", "results", "docs"))
        command = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                   "--find-links", "/opt/wheelhouse", "--target", str(TARGET), str(copy)]
        done = subprocess.run(command, capture_output=True, text=True)
        if done.returncode == 0 and (TARGET / "turboserve").is_dir():
            return None
        lines = [line for line in (done.stderr or done.stdout).splitlines() if line.strip()]
        return lines[-1] if lines else f"pip exited with {done.returncode}"


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--source", default="/root/reference", help="the reference's checkout")
    args = parser.parse_args()
    source = Path(args.source)
    if not (source / "src" / "turboserve").is_dir():
        print(f"no reference checkout at {source}")
        return 1
    if TARGET.exists():
        shutil.rmtree(TARGET)
    TARGET.mkdir(parents=True)
    error = pip_install(source)
    how = "pip install --no-index --no-build-isolation --no-deps"
    if error is not None:
        if TARGET.exists():
            shutil.rmtree(TARGET)
        TARGET.mkdir(parents=True)
        shutil.copytree(source / "src" / "turboserve", TARGET / "turboserve",
                        ignore=shutil.ignore_patterns("__pycache__"))
        how = f"copied src/turboserve unchanged (pip failed: {error})"
    sha, count = digest(TARGET / "turboserve")
    source_sha, source_count = digest(source / "src" / "turboserve")
    record = {"how": how, "files": count, "sha256_16": sha, "same_as_source": sha == source_sha and count == source_count}
    (TARGET / "INSTALL.json").write_text(json.dumps(record, indent=1) + "\n")
    print(json.dumps(record))
    return 0 if record["same_as_source"] else 1


if __name__ == "__main__":
    sys.exit(main())
