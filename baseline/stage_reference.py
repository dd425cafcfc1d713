#!/usr/bin/env python
"""Stage the reference project's Python sources for runs on a machine that has no checkout of it.

    python baseline/stage_reference.py [--reference /path/to/GeoWeave]

Copies the packages the reference's own caller of the sparse global-attention path needs (``easyvolcap``,
``geoweave``, the Pi3 model package, and the three small pure-Python helpers it imports) -- ``*.py`` and
``*.json`` only -- to ``baseline/_ref/GeoWeave``, plus a ten-line stand-in for the one import this image
lacks (``ruamel.yaml``, needed only at import time).  ``baseline/_ref/`` is not version-controlled: it is a
build product, like the compiled library, and travels with the working tree.  Nothing in ``geoweave_b200/``
reads it; ``baseline/ref_harness.py`` (tests and the benchmark's reference arm) does.
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
TREES = ["easyvolcap", "geoweave", os.path.join("aidi", "third_party", "pi3_training", "pi3"), "pdbr", "einops"]
FILES = ["ujson.py"]
KEEP = (".py", ".json")

RUAMEL_STUB = '''"""Stand-in for ruamel.yaml (absent from this image): the reference imports it at module load only."""
import yaml as _y


class YAML:
    def __init__(self, *a, **k):
        self.default_flow_style = None

    def load(self, s):
        return _y.safe_load(s)

    def dump(self, obj, stream):
        stream.write(_y.safe_dump(obj).encode())
'''


def stage(reference: str, dest: str = DEST) -> int:
    if not os.path.isdir(os.path.join(reference, "easyvolcap")):
        raise FileNotFoundError(f"{reference} is not a checkout of the reference project")
    root = os.path.join(dest, "GeoWeave")
    if os.path.isdir(root):
        shutil.rmtree(root)
    n = 0
    for tree in TREES:
        src_tree = os.path.join(reference, tree)
        if not os.path.isdir(src_tree):
            continue
        for dirpath, dirnames, filenames in os.walk(src_tree):
            dirnames[:] = [d for d in dirnames if d != "__pycache__"]
            for name in filenames:
                if name.endswith(KEEP):
                    rel = os.path.relpath(os.path.join(dirpath, name), reference)
                    out = os.path.join(root, rel)
                    os.makedirs(os.path.dirname(out), exist_ok=True)
                    shutil.copyfile(os.path.join(dirpath, name), out)
                    n += 1
    for name in FILES:
        if os.path.exists(os.path.join(reference, name)):
            shutil.copyfile(os.path.join(reference, name), os.path.join(root, name))
            n += 1
    stub = os.path.join(dest, "_stubs", "ruamel", "yaml")
    os.makedirs(stub, exist_ok=True)
    open(os.path.join(dest, "_stubs", "ruamel", "__init__.py"), "w").close()
    with open(os.path.join(stub, "__init__.py"), "w") as f:
        f.write(RUAMEL_STUB)
    with open(os.path.join(dest, "STAGED"), "w") as f:
        f.write(f"{n} files staged from a checkout of zss171999645/GeoWeave\n")
    return n


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("GEOWEAVE_REFERENCE", "/root/reference"))
    args = ap.parse_args()
    print(f"staged {stage(args.reference)} files under {DEST}")


if __name__ == "__main__":
    sys.exit(main())
