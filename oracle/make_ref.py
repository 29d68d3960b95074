"""Recipe for oracle/_ref: the reference project's own Python path, placed where it can travel.

    python oracle/make_ref.py [REFERENCE_DIR]

Test infrastructure, not product code.  Copies, unmodified, the reference files that define and drive its
PyTorch implementation of the two hot paths

    scripts/eval.py  scripts/utils.py
    scripts/problems/gemm/{reference.py, task.py, task.yml}
    scripts/problems/moe/{reference.py, task.py, task.yml}

from a checkout of kukrejayug/RadeonFlow_Kernels into oracle/_ref/scripts/ (same relative layout; the folder
is ignored by git, so no reference source enters this repository's history) and writes next to each
problem's reference.py the two-line submission.py through which the reference's harness reaches this
library (the generated submission of scripts/gen_submission.py:327-330 / :376-404 is what it replaces).

Users of the copy:
  * bench.py --impl reference: times the reference's ref_kernel (scripts/problems/gemm/reference.py:40-85) on
    the host cores;
  * tests/test_reference_harness_gpu.py: runs the reference's eval.py, unmodified, against the library.
REFERENCE_DIR defaults to $RF_REFERENCE_DIR, else a folder named "reference" beside this repository.
"""
import hashlib
import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEST = os.path.join(ROOT, "oracle", "_ref")
FILES = [
    "scripts/eval.py", "scripts/utils.py",
    "scripts/problems/gemm/reference.py", "scripts/problems/gemm/task.py", "scripts/problems/gemm/task.yml",
    "scripts/problems/moe/reference.py", "scripts/problems/moe/task.py", "scripts/problems/moe/task.yml",
]
SUBMISSION = '''# written by oracle/make_ref.py: the submission the reference's eval.py imports (`from submission import custom_kernel`)
import os, sys
sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), *[".."] * 5)))
from radeonflow_kernels_b200.{module} import custom_kernel  # noqa: E402,F401
'''


def reference_dir(argv):
    if len(argv) > 1:
        return argv[1]
    return os.environ.get("RF_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")


def available() -> bool:
    """True when oracle/_ref holds every file of the recipe."""
    return all(os.path.exists(os.path.join(DEST, f)) for f in FILES)


def make(src: str) -> bool:
    """Copies the files; returns False (and leaves DEST alone) when `src` is not a reference checkout."""
    if not all(os.path.exists(os.path.join(src, f)) for f in FILES):
        return False
    manifest = []
    for f in FILES:
        dst = os.path.join(DEST, f)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(src, f), dst)
        manifest.append(f"{hashlib.sha256(open(dst, 'rb').read()).hexdigest()}  {f}")
    for prob in ("gemm", "moe"):
        with open(os.path.join(DEST, "scripts", "problems", prob, "submission.py"), "w") as fh:
            fh.write(SUBMISSION.format(module=prob))
    with open(os.path.join(DEST, "MANIFEST.sha256"), "w") as fh:
        fh.write("\n".join(manifest) + "\n")
    return True


if __name__ == "__main__":
    src = reference_dir(sys.argv)
    if make(src):
        print("oracle/_ref written from", src)
    else:
        print("no reference checkout at", src, "- oracle/_ref left as it is", file=sys.stderr)
        sys.exit(1)
