"""Builds ``oracle/_ref``: the reference's own Python files for this path, taken unmodified from a checkout of
EverMind-AI/MSA, so that tests and ``bench.py``'s reference / baseline legs can run the reference's code itself
on a machine that has no checkout.  TEST INFRASTRUCTURE ONLY: nothing under ``msa_b200/`` imports it.

    python oracle/build_ref.py [--reference /path/to/MSA]

``oracle/_ref`` is an output folder (never committed).  What is copied: ``src/__init__.py``, ``src/msa_service.py``
(``Memory._generate_slice``, ``Memory.prefill_stage2``, ``MSAService.doc_query``), ``src/prefill.py``,
``src/types.py``, and the packages they import (``src/config``, ``src/utils``, ``src/msa``).  Nothing is edited;
``oracle/ref_runner.py`` holds the two-name shim the import needs under transformers 5.
"""
import argparse
import os
import shutil

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
FILES = ["src/__init__.py", "src/msa_service.py", "src/prefill.py", "src/types.py"]
PACKAGES = ["src/config", "src/utils", "src/msa"]


def build_ref(reference: str = "/root/reference", quiet: bool = False) -> bool:
    """Copy the files; returns False (and leaves an existing ``_ref`` alone) when there is no checkout."""
    if not os.path.exists(os.path.join(reference, "src", "msa_service.py")):
        return False
    tmp = OUT + ".tmp"
    shutil.rmtree(tmp, ignore_errors=True)
    for f in FILES:
        os.makedirs(os.path.dirname(os.path.join(tmp, f)), exist_ok=True)
        shutil.copyfile(os.path.join(reference, f), os.path.join(tmp, f))
    for p in PACKAGES:
        shutil.copytree(os.path.join(reference, p), os.path.join(tmp, p),
                        ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    shutil.rmtree(OUT, ignore_errors=True)
    os.replace(tmp, OUT)
    if not quiet:
        n = sum(len(fs) for _, _, fs in os.walk(OUT))
        print(f"oracle/_ref: {n} files copied unmodified from {reference}")
    return True


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    a = ap.parse_args()
    if not build_ref(a.reference):
        raise SystemExit(f"no reference checkout at {a.reference}")
