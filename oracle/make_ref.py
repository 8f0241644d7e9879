"""Makes oracle/_ref: the reference implementation itself, where its checkout is present.

TEST AND BASELINE INFRASTRUCTURE, not product code. The reference's path for this project is pure Python (its front end
and its NumPy interpreter, anvil/interp.py), so there is nothing to compile: the recipe copies the reference's `anvil`
package from the checkout into oracle/_ref/ (git-ignored; it travels to the GPU machine with the built libraries).
`bench.py --impl reference` and the `cpu_baseline` leg then time the reference interpreter itself, and fall back to the
port in oracle/kir_interp.py where oracle/_ref is absent. Nothing under anvil_lang_b200/ imports it.

    python oracle/make_ref.py [--reference /path/to/checkout]
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def make(reference: str) -> bool:
    src = os.path.join(reference, "anvil")
    if not os.path.isdir(src):
        return False
    dst = os.path.join(REF_DIR, "anvil")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(REF_DIR, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return True


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("ANVIL_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")))
    a = ap.parse_args()
    ok = make(a.reference)
    print("oracle/_ref/anvil written" if ok else f"no reference checkout at {a.reference}: oracle/_ref not made")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
