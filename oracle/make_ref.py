"""Recipe that puts the reference (NervanaSystems/ngraph-python, pure Python) where the checker
can import it on a machine that has no checkout of it.

    python oracle/make_ref.py /path/to/ngraph-python      # -> oracle/_ref/

Test infrastructure: nothing in the product imports oracle/.  The copy under oracle/_ref/ is
git-ignored (no reference source enters the history) and is only ever imported, never edited:
  oracle/_ref/ngraph/                 the package, Python files only
  oracle/_ref/examples/resnet/        the CIFAR-10 ResNet builder (resnet.py) the benchmark names
  oracle/_ref/tests/, conftest.py     the reference's own tests (transformer_dependent, flex_tests)
  oracle/_ref/third_party/            Python wrapper the CPU transformer's generated code imports
  oracle/_ref/SOURCE                  where it came from and when
The third-party packages the reference imports and this image lacks are stood in for by the small
modules of ngraph_python_b200/ngraph_compat/ (own code) -- see oracle/ref_env.py.
"""
import os
import shutil
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")

# (source path inside the reference, keep only these suffixes or None for everything)
PARTS = (
    ("ngraph", (".py", ".json")),
    (os.path.join("examples", "resnet"), (".py",)),
    ("tests", (".py",)),
    ("third_party", (".py",)),      # imported by the CPU transformer's generated module
    ("conftest.py", None),
    ("pytest.ini", None),
)


def _copy_tree(src, dst, suffixes):
    n = 0
    for root, dirs, files in os.walk(src):
        dirs[:] = [d for d in dirs if d != "__pycache__"]
        rel = os.path.relpath(root, src)
        out = os.path.join(dst, rel) if rel != "." else dst
        for f in files:
            if suffixes is not None and not f.endswith(suffixes):
                continue
            os.makedirs(out, exist_ok=True)
            shutil.copyfile(os.path.join(root, f), os.path.join(out, f))
            n += 1
    return n


def make(reference_root, dest=DEST, force=False):
    """Returns dest; copies only when dest is absent or older than the recipe asks for."""
    reference_root = os.path.abspath(reference_root)
    if not os.path.isdir(os.path.join(reference_root, "ngraph")):
        raise FileNotFoundError("%s does not hold the ngraph package" % reference_root)
    stamp = os.path.join(dest, "SOURCE")
    if os.path.exists(stamp) and not force:
        return dest
    if os.path.isdir(dest):
        shutil.rmtree(dest)
    os.makedirs(dest)
    total = 0
    for rel, suffixes in PARTS:
        src = os.path.join(reference_root, rel)
        if os.path.isdir(src):
            total += _copy_tree(src, os.path.join(dest, rel), suffixes)
        elif os.path.isfile(src):
            shutil.copyfile(src, os.path.join(dest, rel))
            total += 1
    with open(stamp, "w") as f:
        f.write("copied from %s on %s: %d files\n" % (reference_root, time.strftime("%Y-%m-%d"),
                                                       total))
    return dest


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    print(make(sys.argv[1], force="--force" in sys.argv))
