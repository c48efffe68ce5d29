"""Place the unmodified reference package under baseline/_ref/ (git-ignored) for the hosted-model test and the
reference-kernel timing.

The reference tree has neither setup.py nor pyproject.toml, so `pip install --target baseline/_ref <tree>` stops with
"Neither 'setup.py' nor 'pyproject.toml' found"; what pip would have done for a pure-Python package -- copy the
package directory -- is done here instead.  Nothing under baseline/_ref/ is product code or is committed.

    python baseline/install_reference.py [path-of-the-reference-checkout]
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")


def install(src):
    pkg = os.path.join(src, "mathbrain")
    if not os.path.isfile(os.path.join(pkg, "model.py")):
        return False
    dst = os.path.join(TARGET, "mathbrain")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(TARGET, exist_ok=True)
    shutil.copytree(pkg, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return True


if __name__ == "__main__":
    src = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MATHBRAIN_REFERENCE", "")
    if not src:
        sys.exit("usage: install_reference.py <reference checkout>  (or set MATHBRAIN_REFERENCE)")
    ok = install(src)
    print("installed" if ok else "no mathbrain/model.py under %s" % src)
    sys.exit(0 if ok else 1)
