"""Every ```python block of the user guide under docs/ runs on the CPU (blocks of one chapter share a namespace and
run in order, in a scratch directory); blocks marked ```python gpu or ```python ranks need a B200 or several processes
and are only compiled."""
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHAPTERS = sorted(glob.glob(os.path.join(ROOT, "docs", "*.md")))
BLOCK = re.compile(r"^```python([^\n]*)\n(.*?)^```", re.S | re.M)


def test_the_guide_has_its_chapters():
    names = [os.path.basename(c) for c in CHAPTERS]
    assert len(names) >= 12 and "01_index.md" in names, names
    index = open(os.path.join(ROOT, "docs", "01_index.md")).read()
    for n in names:
        assert n in index, n + " is not linked from the index"


@pytest.mark.parametrize("chapter", CHAPTERS, ids=[os.path.basename(c) for c in CHAPTERS])
def test_chapter_examples_run(chapter, tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    text = open(chapter).read()
    ns = {"__name__": "__docs__"}
    for i, m in enumerate(BLOCK.finditer(text)):
        tag, code = m.group(1).strip(), m.group(2)
        compiled = compile(code, "%s[block %d]" % (os.path.basename(chapter), i), "exec")
        if tag:            # "gpu", "ranks": syntax only
            continue
        exec(compiled, ns)
