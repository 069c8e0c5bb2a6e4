"""The guides name files, options and environment variables: those must exist."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = ["README.md"] + [os.path.join("docs", f) for f in sorted(os.listdir(os.path.join(ROOT, "docs"))) if f.endswith(".md")] + [
    os.path.join("examples", d, "README.md") for d in ("doremi", "mamba", "moe", "mup", "custom_dataloader", "llama", "contributor_guide")]


def _text(path):
    with open(os.path.join(ROOT, path)) as f:
        return f.read()


def _alternatives(ref):
    """``a/{b,c}.py`` -> ``a/b.py``, ``a/c.py``."""
    m = re.search(r"\{([^}]*)\}", ref)
    return [ref[: m.start()] + alt + ref[m.end() :] for alt in m.group(1).split(",")] if m else [ref]


def test_paths_named_in_the_guides_exist():
    import glob

    tops = ("nanotron_b200/", "docs/", "examples/", "tests/", "tools/", "scripts/", "profiles/")
    missing = []
    measured = [os.path.join("profiles", f) for f in sorted(os.listdir(os.path.join(ROOT, "profiles"))) if f.endswith(".md")]
    for doc in DOCS + measured:
        for ref in re.findall(r"`([A-Za-z0-9_./{},*-]+)`", _text(doc)):
            if "<" in ref or not ref.startswith(tops):
                continue
            if not all(glob.glob(os.path.join(ROOT, alt.rstrip("/"))) for alt in _alternatives(ref)):
                missing.append((doc, ref))
    assert not missing, missing


def test_environment_variables_named_in_the_guides_are_read_somewhere():
    sources = []
    for root, _, files in os.walk(os.path.join(ROOT, "nanotron_b200")):
        sources += [os.path.join(root, f) for f in files if f.endswith(".py")]
    sources += [os.path.join(ROOT, f) for f in os.listdir(ROOT) if f.endswith(".py")]  # the entry points
    code = "\n".join(open(p, errors="ignore").read() for p in sources)
    unknown = []
    for doc in DOCS:
        for var in set(re.findall(r"`((?:NANOTRON|ENABLE|DEBUG)_[A-Z_]+)(?:=[^`]*)?`", _text(doc))):
            if var not in code:
                unknown.append((doc, var))
    assert not unknown, unknown
