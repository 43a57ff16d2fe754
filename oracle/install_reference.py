"""Put the reference project where the benchmark box can import it: ``baseline/_ref`` (git-ignored, travels with the repo).

    python oracle/install_reference.py --reference <checkout of Noumena-Network/NSA-Test>

First tries the regular offline install (``pip install --no-index --no-build-isolation --target baseline/_ref``).  The
reference ships neither ``setup.py`` nor ``pyproject.toml`` (its README.md:19-21 names a ``pip install -e .`` that cannot
work), so that attempt fails and the fallback does what such an install would have done for a pure-Python project: it copies
the package directory ``nsa/`` unchanged, and the project's own ``tests/`` beside it as ``reference_tests/`` (they are
the drop-in acceptance suite).  Nothing is copied into tracked paths, nothing is modified.

TEST INFRASTRUCTURE ONLY: the shipped package never imports anything from ``baseline/_ref``.
"""
import argparse
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEST = os.path.join(ROOT, "baseline", "_ref")


def install(reference: str, verbose: bool = True) -> str:
    if not os.path.exists(os.path.join(reference, "nsa", "kernels.py")):
        raise FileNotFoundError(f"{reference} is not a checkout of the reference project (no nsa/kernels.py)")
    os.makedirs(DEST, exist_ok=True)
    how = "copy"
    if os.path.exists(os.path.join(reference, "setup.py")) or os.path.exists(os.path.join(reference, "pyproject.toml")):
        tmp = "/tmp/nsa_reference_src"
        shutil.rmtree(tmp, ignore_errors=True)
        shutil.copytree(reference, tmp)
        r = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--find-links",
                            "/opt/wheelhouse", "--target", DEST, tmp], capture_output=True, text=True)
        how = "pip" if r.returncode == 0 else "copy"
    if how == "copy":
        for sub, dst in (("nsa", "nsa"), ("tests", "reference_tests")):
            target = os.path.join(DEST, dst)
            shutil.rmtree(target, ignore_errors=True)
            shutil.copytree(os.path.join(reference, sub), target, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
        for name in ("pytest.ini", "test_imports.py"):
            if os.path.exists(os.path.join(reference, name)):
                shutil.copy(os.path.join(reference, name), os.path.join(DEST, name))
    with open(os.path.join(DEST, "INSTALLED_FROM"), "w") as f:
        f.write(f"{how}: no setup.py / pyproject.toml in the reference project, package directory copied unchanged\n")
    if verbose:
        print(f"reference installed into {DEST} ({how})")
    return DEST


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    install(ap.parse_args().reference)
