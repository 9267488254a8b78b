"""Every `path:line` or `path:first-last` citation of a reference file in the sources, headers
and tests names a file of the reference tree that has that many lines.  The
reference tree is only present where the library is developed; elsewhere the test is skipped."""
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("KQ_REFERENCE_TREE", os.path.join(os.path.dirname(ROOT), "reference"))  # a checkout beside this one
CITATION = re.compile(r"((?:packages|docs|tools|scripts|apps)/[\w/.\-]+\.(?:ts|wgsl|md|json|py|js)):(\d+)(?:-(\d+))?")


def cited_files():
    names = glob.glob(os.path.join(ROOT, "include", "*.h"))
    for sub in ("karume_b200", "oracle", "tests"):
        names += glob.glob(os.path.join(ROOT, sub, "**", "*.*"), recursive=True)
    names += glob.glob(os.path.join(ROOT, "*.py"))
    keep = (".h", ".cuh", ".cu", ".c", ".cpp", ".py")
    return [n for n in names if os.path.isfile(n) and n.endswith(keep) and os.sep + "build" + os.sep not in n]


@pytest.mark.skipif(not os.path.isdir(REFERENCE), reason="reference tree not present")
def test_cited_reference_lines_exist():
    lengths, bad, seen = {}, [], 0
    for name in cited_files():
        with open(name, errors="ignore") as fh:
            text = fh.read()
        for m in CITATION.finditer(text):
            seen += 1
            path = os.path.join(REFERENCE, m.group(1))
            if not os.path.isfile(path):
                bad.append((os.path.relpath(name, ROOT), m.group(0), "no such file"))
                continue
            if path not in lengths:
                with open(path, errors="ignore") as fh:
                    lengths[path] = sum(1 for _ in fh)
            last = int(m.group(3) or m.group(2))
            if last > lengths[path] or int(m.group(2)) < 1 or last < int(m.group(2)):
                bad.append((os.path.relpath(name, ROOT), m.group(0), f"file has {lengths[path]} lines"))
    assert seen > 50, seen
    assert not bad, bad
