"""Stage the reference's own operator files, UNCHANGED, under oracle/_ref/ so that they can be executed as the checker
and as the baseline on a machine that has no checkout of the reference.

    python oracle/make_ref.py /path/to/BitStack-checkout

Copies exactly the files of the linear-layer path -- bitstack/__init__.py, bitstack/modules/{__init__,BitStackLinear}.py,
bitstack/utils/{__init__,pack_utils,inference_utils}.py -- byte for byte (a manifest with their SHA-256 is written
beside them).  oracle/_ref/ is ignored by git: the copies are test / baseline infrastructure, never product code, and
nothing in the package may import them.  Users: `bench.py --impl reference` and the `cpu_baseline` leg (the reference's
`forward_l0` on the host cores) and `python -m bitstack_b200.layer_bench --ref-level {2,3,5}` (its Triton levels on the
GPU, the baseline its authors publish).
"""
import hashlib
import json
import os
import shutil
import sys

FILES = ["bitstack/__init__.py", "bitstack/modules/__init__.py", "bitstack/modules/BitStackLinear.py",
         "bitstack/utils/__init__.py", "bitstack/utils/pack_utils.py", "bitstack/utils/inference_utils.py"]
HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def main(src: str) -> None:
    manifest = {}
    for rel in FILES:
        s, d = os.path.join(src, rel), os.path.join(DEST, rel)
        if not os.path.isfile(s):
            raise SystemExit(f"{s} not found: is {src} a checkout of xinghaow99/BitStack?")
        os.makedirs(os.path.dirname(d), exist_ok=True)
        shutil.copyfile(s, d)
        manifest[rel] = hashlib.sha256(open(d, "rb").read()).hexdigest()
    with open(os.path.join(DEST, "MANIFEST.json"), "w") as f:
        json.dump({"source": os.path.abspath(src), "sha256": manifest}, f, indent=1)
    print(f"staged {len(FILES)} reference files under {DEST}")


def ref_available() -> bool:
    return os.path.isfile(os.path.join(DEST, "bitstack", "modules", "BitStackLinear.py"))


def import_reference():
    """The reference's BitStackLinear class from the staged copy (raises ImportError when it is not staged)."""
    if not ref_available():
        raise ImportError("oracle/_ref is empty: run `python oracle/make_ref.py <checkout>` first")
    if DEST not in sys.path:
        sys.path.insert(0, DEST)
    from bitstack.modules.BitStackLinear import BitStackLinear   # noqa: E402
    return BitStackLinear


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
