"""The documents name files, modules and configuration keys that exist."""
import importlib
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = [os.path.join(ROOT, "README.md")] + sorted(
    os.path.join(ROOT, "docs", f) for f in os.listdir(os.path.join(ROOT, "docs")) if f.endswith(".md"))


@pytest.mark.parametrize("path", DOCS, ids=[os.path.relpath(p, ROOT) for p in DOCS])
def test_paths_and_modules_named_in_the_document_exist(path):
    text = open(path, encoding="utf-8").read()
    for rel in set(re.findall(r"\b((?:playground|benchmarks|steptronoss_b200|tests|profiles|docs)/[\w/.\-]+\.(?:py|md|cu|cuh|h))\b", text)):
        assert os.path.exists(os.path.join(ROOT, rel)), f"{os.path.relpath(path, ROOT)} names {rel}"
    for mod in set(re.findall(r"-m ((?:playground|steptronoss_b200|benchmarks)(?:\.\w+)+)", text)):
        if mod.endswith(".run"):      # torch.distributed.run is matched by neither prefix; guard anyway
            continue
        assert importlib.util.find_spec(mod) is not None, f"{os.path.relpath(path, ROOT)} runs python -m {mod}"


def test_environment_variables_named_in_the_documents_are_read_somewhere():
    names = set()
    for p in DOCS:
        names |= set(re.findall(r"\b(STB200_[A-Z0-9_]+)\b", open(p, encoding="utf-8").read()))
    src = ""
    for base in ("steptronoss_b200", "playground", "bench.py"):
        full = os.path.join(ROOT, base)
        files = [full] if os.path.isfile(full) else [os.path.join(d, f) for d, _, fs in os.walk(full) for f in fs if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h"))]
        for f in files:
            src += open(f, encoding="utf-8").read()
    missing = sorted(n for n in names if n not in src)
    assert not missing, missing
