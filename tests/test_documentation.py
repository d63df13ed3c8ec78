"""The guides stay true to the tree: relative links resolve, JSON examples parse, every ``python -m uttt_b200...``
module a guide names can be found, every repository path a guide names exists, and the configuration catalog is the
one the checker would write now."""
import importlib.util
import json
import os
import re
from urllib.parse import unquote, urlsplit

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _documents():
    names = ["README.md", "CONTRIBUTING.md", "THIRD_PARTY_NOTICES.md"]
    docs = os.path.join(ROOT, "docs")
    return [os.path.join(ROOT, n) for n in names] + sorted(os.path.join(docs, n) for n in os.listdir(docs)
                                                           if n.endswith(".md"))


def _text(path):
    with open(path, encoding="utf-8") as fh:
        return fh.read()


def test_relative_links_resolve():
    broken = []
    for path in _documents():
        text = _text(path)
        assert "�" not in text, path
        prose = re.sub(r"```.*?```", "", text, flags=re.DOTALL)
        for dest in re.findall(r"\[[^\]]*\]\(([^\s)]+)\)", prose):
            parts = urlsplit(dest)
            if parts.scheme or not parts.path:
                continue
            if not os.path.exists(os.path.join(os.path.dirname(path), unquote(parts.path))):
                broken.append(f"{os.path.relpath(path, ROOT)} -> {dest}")
    assert not broken, "\n".join(broken)


def test_json_examples_parse():
    for path in _documents():
        for block in re.findall(r"```json\n(.*?)```", _text(path), re.DOTALL):
            json.loads(block)


def test_named_modules_exist():
    missing = []
    for path in _documents():
        for mod in set(re.findall(r"python3? -m (uttt_b200(?:\.\w+)+)", _text(path))):
            if importlib.util.find_spec(mod) is None:
                missing.append(f"{os.path.relpath(path, ROOT)}: {mod}")
    assert not missing, "\n".join(missing)


def test_named_paths_exist():
    """Paths written in code spans or commands that point into the repository (sources, configs, launchers, tests)."""
    pattern = re.compile(r"(?<![\w/.<{$])((?:uttt_b200|configs|launch|examples|tests|profiles|docs)/[\w./-]+\.\w+)")
    missing = []
    for path in _documents():
        for rel in set(pattern.findall(_text(path))):
            if any(ch in rel for ch in "*{<") or rel.endswith("datasets.yaml") or rel.endswith("api_keys.yaml"):
                continue                                    # patterns, and files the user creates from the examples
            if not os.path.exists(os.path.join(ROOT, rel)):
                missing.append(f"{os.path.relpath(path, ROOT)}: {rel}")
    assert not missing, "\n".join(sorted(missing))


def test_configuration_catalog_is_current():
    from uttt_b200.tools.check_configs import catalog
    assert _text(os.path.join(ROOT, "configs", "CATALOG.md")) == catalog()
