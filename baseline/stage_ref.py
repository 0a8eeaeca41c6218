"""Stage the UNMODIFIED reference modules for timing on a GPU: copies clip_loss.py and lit_loss.py of
b0nce/MemoryEfficientCLIP from a checkout into baseline/_ref/ (git-ignored: the reference's sources
are never part of this repository's history).

    python baseline/stage_ref.py [path to the reference checkout]

bench.py then reports a `reference_gpu` block (the reference's own Triton kernels on the same GPU);
without the staged files that block says "unavailable".
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = ("clip_loss.py", "lit_loss.py")


def stage(src: str) -> bool:
    if not all(os.path.isfile(os.path.join(src, f)) for f in FILES):
        return False
    os.makedirs(DEST, exist_ok=True)
    for f in FILES:
        shutil.copyfile(os.path.join(src, f), os.path.join(DEST, f))
    return True


if __name__ == "__main__":
    source = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MECLIP_REFERENCE_DIR", "")
    ok = bool(source) and stage(source)
    print("staged" if ok else "nothing staged: give the path of a MemoryEfficientCLIP checkout")
    sys.exit(0 if ok else 1)
