"""Fetch the reference project's own test files, unchanged, for the acceptance run against the drop-in.

    python tests/reference_suite/fetch.py [path to the reference checkout]

(default: the directory ``reference`` beside this repository, or ``$ATTENTION_IMPL_REFERENCE``)

Copies ``<reference>/tests/*.py`` byte for byte into ``tests/reference_suite/_ref/`` and writes a
MANIFEST with their SHA-256 sums.  ``_ref/`` is listed in .gitignore: the files are fetched, not
committed.  ``tests/test_reference_suite_gpu.py`` runs them in a child process with the drop-in
modules (``attention_impl_b200/dropin``: lm_ops, attention, paged_attention, rotary_embedding) first
on the import path; nothing else of the reference is involved.
"""
import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def default_reference_root() -> str:
    env = os.environ.get("ATTENTION_IMPL_REFERENCE")
    if env:
        return env
    repo = os.path.dirname(os.path.dirname(HERE))
    return os.path.join(os.path.dirname(repo), "reference")


def fetch(reference_root: str = "") -> int:
    src = os.path.join(reference_root or default_reference_root(), "tests")
    if not os.path.isdir(src):
        return 0
    os.makedirs(DEST, exist_ok=True)
    lines = []
    for name in sorted(os.listdir(src)):
        if not name.endswith(".py"):
            continue
        shutil.copyfile(os.path.join(src, name), os.path.join(DEST, name))
        with open(os.path.join(DEST, name), "rb") as f:
            lines.append(f"{hashlib.sha256(f.read()).hexdigest()}  {name}")
    with open(os.path.join(DEST, "MANIFEST"), "w") as f:
        f.write("\n".join(lines) + "\n")
    return len(lines)


if __name__ == "__main__":
    n = fetch(*sys.argv[1:2])
    print(f"{n} files -> {DEST}")
