"""Regenerates the golden files of this directory from the reference checkout.

Run where a checkout of the reference is available:

    python tests/golden/make_golden.py /path/to/reference

It executes the reference's own fixture generators (scripts/gen-tiny-fixture.py,
scripts/gen-tiny-moe-fixture.py) unmodified and stores their OUTPUT here, then checks each file
against the SHA-256 the reference pins in tests/fixtures/TINY_*_FIXTURE.toml. No reference source
is copied. The tests never run this script and never read the reference at run time.
"""
from __future__ import annotations

import hashlib
import json
import re
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def manifest(ref: Path, name: str) -> dict:
    text = (ref / "tests" / "fixtures" / name).read_text()
    out = {}
    for key in ("filename", "generator", "generator_args", "sha256", "size_bytes"):
        m = re.search(rf'^{key}\s*=\s*"?([^"\n]*)"?\s*$', text, re.M)
        if m:
            out[key] = m.group(1)
    return out


def main() -> int:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference")
    ref = Path(sys.argv[1])
    pinned = {}
    for toml in ("TINY_FIXTURE.toml", "TINY_F16_FIXTURE.toml", "TINY_Q8_FIXTURE.toml", "TINY_MOE_FIXTURE.toml"):
        m = manifest(ref, toml)
        dest = HERE / m["filename"]
        args = m.get("generator_args", "").split()
        subprocess.run([sys.executable, str(ref / m["generator"]), *args, str(dest)], check=True)
        digest = hashlib.sha256(dest.read_bytes()).hexdigest()
        if digest != m["sha256"] or dest.stat().st_size != int(m["size_bytes"]):
            raise SystemExit(f"{dest.name}: digest {digest} differs from the reference manifest {m['sha256']}")
        pinned[m["filename"]] = {"sha256": digest, "size_bytes": dest.stat().st_size, "manifest": f"tests/fixtures/{toml}"}
        print(dest.name, digest)
    (HERE / "fixtures.json").write_text(json.dumps(pinned, indent=2) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
