#!/usr/bin/env python3
"""Run the reference project's OWN test files, unchanged, against this repository's ``nsa`` package on a GPU.

    python tests/run_reference_suite.py [--out table.md] [--files test_kernel_contracts.py ...]

The reference's tests live where ``oracle/install_reference.py`` put them (``baseline/_ref/reference_tests``).  They are
collected by a child pytest whose import path puts THIS package first, so ``import nsa`` / ``from nsa.kernels import ...``
resolve to the CUDA implementation, while ``nsa.reference`` (the slow loop implementations the tests compare against)
forwards to the reference checkout named by NSA_REFERENCE_PATH.  Prints one line per test file (passed / failed /
skipped / errors) and the failing test ids; this is the drop-in acceptance run, not part of the regular test suite.
"""
import argparse
import os
import subprocess
import sys
import xml.etree.ElementTree as ET

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
DEFAULT = ["test_kernel_contracts.py", "test_branches.py", "test_accuracy.py", "test_whitepaper_spec.py", "test_selection_reference.py",
           "test_comprehensive.py", "test_backward.py", "test_spec_blocks.py", "test_spec_algorithms.py", "test_selection_validation.py",
           "test_module_e2e.py", "test_reference.py", "test_large_scale.py"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None, help="also write the table to this file (markdown)")
    ap.add_argument("--files", nargs="*", default=DEFAULT)
    ap.add_argument("--per-test-timeout", type=int, default=300)
    args = ap.parse_args()
    tests = os.path.join(REF, "reference_tests")
    if not os.path.isdir(tests):
        sys.exit(f"{tests} is missing: run oracle/install_reference.py --reference <checkout> first")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.join(ROOT, "nsa-test_b200"), os.environ.get("PYTHONPATH", "")]),
               NSA_REFERENCE_PATH=REF)
    lines = ["| reference test file | passed | failed | errors | skipped | failing tests |", "|---|---:|---:|---:|---:|---|"]
    total = dict(passed=0, failed=0, errors=0, skipped=0)
    for name in args.files:
        path = os.path.join(tests, name)
        if not os.path.exists(path):
            lines.append(f"| {name} | - | - | - | - | file not in the reference checkout |")
            continue
        xml = os.path.join("/tmp", f"nsa_ref_{os.getpid()}_{name}.xml")
        cmd = [sys.executable, "-m", "pytest", path, "-q", "-p", "no:cacheprovider", "--rootdir", tests, f"--junitxml={xml}",
               f"--timeout={args.per_test_timeout}", "-W", "ignore"]
        r = subprocess.run(cmd, env=env, cwd=tests, capture_output=True, text=True)
        try:
            suite = ET.parse(xml).getroot()
            suite = suite if suite.tag == "testsuite" else suite.find("testsuite")
            n, f, e, s = (int(suite.get(k_, 0)) for k_ in ("tests", "failures", "errors", "skipped"))
            bad = [f"{tc.get('name')}" for tc in suite.iter("testcase") if tc.find("failure") is not None or tc.find("error") is not None]
            why = []
            for tc in suite.iter("testcase"):
                node = tc.find("failure") if tc.find("failure") is not None else tc.find("error")
                if node is not None:
                    msg = (node.get("message") or "").strip().splitlines()
                    why.append(f"{tc.get('name')}: {msg[0][:140] if msg else ''}")
            lines.append(f"| {name} | {n - f - e - s} | {f} | {e} | {s} | {'; '.join(why) if why else ''} |")
            for k_, v_ in (("passed", n - f - e - s), ("failed", f), ("errors", e), ("skipped", s)):
                total[k_] += v_
        except Exception as ex:  # collection crashed before a report was written
            tail = (r.stdout + r.stderr).strip().splitlines()[-3:]
            lines.append(f"| {name} | - | - | - | - | no report ({type(ex).__name__}); pytest said: {' / '.join(tail)[:300]} |")
        finally:
            if os.path.exists(xml):
                os.remove(xml)
    lines.append(f"| **total** | {total['passed']} | {total['failed']} | {total['errors']} | {total['skipped']} | |")
    text = "\n".join(lines)
    print(text)
    if args.out:
        with open(args.out, "w") as fh:
            fh.write(text + "\n")


if __name__ == "__main__":
    main()
