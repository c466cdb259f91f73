"""Stage the reference's own Python modules for this path under ``oracle/_ref`` (TEST INFRASTRUCTURE).

    python oracle/make_ref.py --ref /path/to/HazyResearch-based

copies, unchanged, the handful of files of the reference's ``based`` package that its language
model and the three Based mixers need (``based/generation.py``, ``based/models/{gpt,block,mlp}.py``,
``based/models/mixers/{linear_attention,convolution,slide_attention}.py``,
``based/ops/triton/layer_norm.py``, ``based/utils/hf.py`` and the package ``__init__`` files) into
``oracle/_ref/based/``.  The directory is ignored by git — no reference source enters this
repository's history — but it is an ordinary directory next to the tests, so a machine that gets
a copy of the working tree (the GPU box) gets it too.  ``oracle/ref_shims.py`` imports from it.

What uses it: tests that drive the B200 mixers through the reference's own ``GPTLMHeadModel`` /
``GenerationMixin.generate``, and ``bench.py --impl reference`` / its ``cpu_baseline`` leg, which
time the reference's ``recurrent_forward`` / ``parallel_forward`` on the host cores.  Nothing
under ``based_b200`` ever imports it.
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")

# paths inside the reference tree; directories on the way get their own __init__.py copied too
FILES = [
    "based/__init__.py",
    "based/generation.py",
    "based/models/__init__.py",
    "based/models/gpt.py",
    "based/models/block.py",
    "based/models/mlp.py",
    "based/models/mixers/__init__.py",
    "based/models/mixers/linear_attention.py",
    "based/models/mixers/convolution.py",
    "based/models/mixers/slide_attention.py",
    "based/ops/__init__.py",
    "based/ops/triton/__init__.py",
    "based/ops/triton/layer_norm.py",
    "based/utils/__init__.py",
    "based/utils/hf.py",
]


def make_ref(ref_root: str, dest: str = DEST) -> str:
    """Copy the files above from ``ref_root``; returns ``dest``.  Idempotent."""
    missing = [f for f in FILES if not os.path.exists(os.path.join(ref_root, f))]
    if missing:
        raise FileNotFoundError(f"not a HazyResearch/based tree ({ref_root}): missing {missing}")
    for f in FILES:
        dst = os.path.join(dest, f)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(ref_root, f), dst)
    with open(os.path.join(dest, "SOURCE.txt"), "w") as fh:
        fh.write("Unmodified copies of files of HazyResearch/based, staged by oracle/make_ref.py.\n"
                 "Not part of this repository's history (git-ignored); test infrastructure only.\n")
    return dest


def available(dest: str = DEST) -> bool:
    return all(os.path.exists(os.path.join(dest, f)) for f in FILES)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("BASED_REFERENCE"))
    args = ap.parse_args()
    if not args.ref:
        ap.error("--ref or BASED_REFERENCE must point at the HazyResearch/based tree")
    print(make_ref(args.ref))


if __name__ == "__main__":
    sys.exit(main())
