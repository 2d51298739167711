"""Puts a byte-for-byte copy of the reference tree under ``baseline/_ref/``.

    python baseline/setup_ref.py <path of the reference tree>   (or GTOPK_REFERENCE_DIR)

The reference has no ``setup.py``/``pyproject.toml`` (``pip install`` answers
"Neither 'setup.py' nor 'pyproject.toml' found"): it is a flat directory of
scripts that run in place, so installing it means copying it.  Nothing is
patched.  ``baseline/ref_manifest.sha256`` lists the SHA-256 of every Python
file of the copy; ``verify()`` (also called by ``baseline/ref_arm.py``) checks a
tree against it, so a benchmark box that only has the copy can still tell that
it is unmodified.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
MANIFEST = os.path.join(HERE, "ref_manifest.sha256")


def _py_files(root):
    out = []
    for d, dirs, files in os.walk(root):
        dirs[:] = sorted(x for x in dirs if x not in (".git", "__pycache__"))
        for f in sorted(files):
            if f.endswith((".py", ".sh", ".conf", ".json")):
                out.append(os.path.relpath(os.path.join(d, f), root))
    return out


def digest(root):
    lines = []
    for rel in _py_files(root):
        with open(os.path.join(root, rel), "rb") as fh:
            lines.append("%s  %s" % (hashlib.sha256(fh.read()).hexdigest(), rel))
    return lines


def verify(root=REF):
    """True when every listed file of ``root`` has the recorded hash."""
    if not os.path.isfile(MANIFEST) or not os.path.isdir(root):
        return False
    with open(MANIFEST) as fh:
        want = [l.rstrip("\n") for l in fh if l.strip()]
    return digest(root) == want


def main(argv):
    args = [a for a in argv[1:] if not a.startswith("--")]
    src = args[0] if args else os.environ.get("GTOPK_REFERENCE_DIR", "")
    if not os.path.isdir(src):
        print("reference tree not found at %s; keeping %s as it is" % (src, REF))
        return 0 if verify() else 1
    if os.path.isdir(REF):
        shutil.rmtree(REF)
    shutil.copytree(src, REF, ignore=shutil.ignore_patterns(".git", "__pycache__"))
    for d, _, files in os.walk(REF):
        os.chmod(d, 0o755)
        for f in files:
            os.chmod(os.path.join(d, f), 0o644)
    lines = digest(REF)
    if "--write-manifest" in argv or not os.path.isfile(MANIFEST):
        with open(MANIFEST, "w") as fh:
            fh.write("\n".join(lines) + "\n")
    ok = verify()
    print("copied %s -> %s (%d files hashed, manifest %s)" % (src, REF, len(lines), "matches" if ok else "DIFFERS"))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv))
