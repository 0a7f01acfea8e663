"""Install the UNMODIFIED reference (CESOIA/transformer-surgeon) under oracle/_ref/ (TEST INFRASTRUCTURE).

    python oracle/make_ref.py [<reference checkout>]        default: $TSB200_REFERENCE, else a `reference` directory beside this repository

oracle/_ref/ is git-ignored (no reference source enters the history) but ships with the working tree to
the GPU machine, like the built shared library.  The reference is pure Python, so "installing" it means
placing its `transformersurgeon` package there, from a temporary copy (the checkout may be read-only and
`setup.py` writes build directories next to itself).  pip does the placing when it can; dependency
resolution is skipped (`--no-deps`: torchao and a newer transformers are asked for by the reference's
setup.py and are not installed in this environment; the hot path needs neither).

Who may use oracle/_ref: the tests (the drop-in round trip on the reference's real classes, config-1 at
full size) and the CPU legs of bench.py.  Nothing in the product package imports it.

`ref_path()` returns the directory to put on sys.path, or None when the install is absent.
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
PKG = "transformersurgeon"


def ref_path():
    return DEST if os.path.isfile(os.path.join(DEST, PKG, "__init__.py")) else None


def import_reference():
    """Import the reference from oracle/_ref (raises ImportError when it is not installed)."""
    p = ref_path()
    if p is None:
        raise ImportError("oracle/_ref is absent: run `python oracle/make_ref.py <reference checkout>`")
    if p not in sys.path:
        sys.path.insert(0, p)
    import transformersurgeon
    return transformersurgeon


def make(src=None, force=False):
    src = src or os.environ.get("TSB200_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    if not os.path.isfile(os.path.join(src, PKG, "__init__.py")):
        raise FileNotFoundError(f"{src} holds no `{PKG}` package")
    if ref_path() and not force:
        return DEST
    with tempfile.TemporaryDirectory() as tmp:
        work = os.path.join(tmp, "reference")
        os.makedirs(work)
        shutil.copytree(os.path.join(src, PKG), os.path.join(work, PKG))
        shutil.copy2(os.path.join(src, "setup.py"), os.path.join(work, "setup.py"))
        if os.path.isdir(DEST):
            shutil.rmtree(DEST)
        r = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                            "--quiet", "--target", DEST, work], capture_output=True, text=True)
        if r.returncode != 0 or not os.path.isfile(os.path.join(DEST, PKG, "__init__.py")):
            # pip could not build a wheel here: the package is pure Python, place it directly
            os.makedirs(DEST, exist_ok=True)
            if os.path.isdir(os.path.join(DEST, PKG)):
                shutil.rmtree(os.path.join(DEST, PKG))
            shutil.copytree(os.path.join(work, PKG), os.path.join(DEST, PKG))
            how = "copied (pip: %s)" % (r.stderr.strip().splitlines()[-1] if r.stderr.strip() else "failed")
        else:
            how = "pip install --no-deps --target"
    with open(os.path.join(DEST, "INSTALLED_FROM.txt"), "w") as f:
        f.write(f"{src}\n{how}\n")
    return DEST


if __name__ == "__main__":
    print(make(sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("-") else None,
               force="--force" in sys.argv))
