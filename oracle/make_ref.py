"""Stage the reference's own Python for this path under ``oracle/_ref`` (test infrastructure, not shipped).

    python oracle/make_ref.py [/path/to/NanoQuant]        (default: $NANOQUANT_REFERENCE)

Copies the two pure-Python files of the hot path, ``src/nanoquant/modules/linear.py`` (the module whose
``forward`` / ``_prepare_kernel`` the kernels sit behind, and whose PyTorch branch is the dequantise-then-matmul
oracle and CPU baseline) and ``src/nanoquant/kernel/utils.py`` (packers, operator lookup), into a small package
``oracle/_ref/nanoquant_ref`` with empty ``__init__`` files, so that they import without the reference's
``modules/__init__`` (which pulls in its hub, evaluation and training dependencies).  ``oracle/_ref`` is ignored
by git and travels to the GPU box with the working tree.  The files are used as they are: the GPU test runs the
reference's module on top of this repository's ``binary_kernels`` operators, and ``bench.py --impl reference``
times its PyTorch branch on the host cores.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DST = os.path.join(HERE, "_ref", "nanoquant_ref")
FILES = (("modules", "linear.py"), ("kernel", "utils.py"))


DEFAULT_ROOT = os.environ.get("NANOQUANT_REFERENCE", os.path.join(os.sep, "root", "reference"))


def make(ref_root: str = DEFAULT_ROOT) -> bool:
    src = os.path.join(ref_root, "src", "nanoquant")
    if not all(os.path.exists(os.path.join(src, d, f)) for d, f in FILES):
        return False
    for d, f in FILES:
        os.makedirs(os.path.join(DST, d), exist_ok=True)
        shutil.copyfile(os.path.join(src, d, f), os.path.join(DST, d, f))
        open(os.path.join(DST, d, "__init__.py"), "w").close()
    open(os.path.join(DST, "__init__.py"), "w").close()
    return True


def load():
    """The staged reference package (``nanoquant_ref``), or None when it has not been staged."""
    if not os.path.exists(os.path.join(DST, "modules", "linear.py")):
        return None
    root = os.path.dirname(DST)
    if root not in sys.path:
        sys.path.insert(0, root)
    import importlib
    return importlib.import_module("nanoquant_ref")


if __name__ == "__main__":
    ok = make(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_ROOT)
    print("staged" if ok else "reference sources not found: nothing staged", DST)
