"""The documents name files, tests and environment knobs; this keeps those names real."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = ["README.md"] + sorted("docs/" + f for f in os.listdir(os.path.join(ROOT, "docs")) if f.endswith(".md"))


def _text(path):
    with open(os.path.join(ROOT, path)) as fh:
        return fh.read()


def test_referenced_files_exist():
    missing = []
    pat = re.compile(r"`((?:bench|tests|docs|profiles|tridist_b200|triton_dist|pydushmem)/[\w./-]+\.(?:py|md|json|cuh|cu|cpp|h))\b")
    for doc in DOCS:
        text = _text(doc)
        for m in pat.finditer(text):
            rel = m.group(1)
            if "*" in rel or "<" in rel or "NxB200" in rel:
                continue
            if not os.path.exists(os.path.join(ROOT, rel)):
                missing.append((doc, rel))
    assert not missing, missing


def test_referenced_tests_exist():
    missing = []
    pat = re.compile(r"`(tests/[\w/]+\.py)::(\w+)`")
    for doc in DOCS:
        for m in pat.finditer(_text(doc)):
            path, name = m.group(1), m.group(2)
            full = os.path.join(ROOT, path)
            if not os.path.exists(full) or not re.search(rf"def {name}\b", _text(path)):
                missing.append((doc, path, name))
    assert not missing, missing


def test_documented_knobs_are_read_somewhere():
    knobs = set(re.findall(r"^(TRIDIST_[A-Z0-9_]+)", _text("tridist_b200/utils/config.py"), flags=re.M))
    assert len(knobs) >= 10
    sources = []
    for base in ("tridist_b200", "bench"):
        for dirpath, _, files in os.walk(os.path.join(ROOT, base)):
            for f in files:
                if f.endswith(".py") and f != "config.py":
                    sources.append(_text(os.path.relpath(os.path.join(dirpath, f), ROOT)))
    blob = "\n".join(sources)
    unread = sorted(k for k in knobs if f'"{k}"' not in blob)
    assert not unread, unread
