"""Paths quoted in the documentation exist.

Every back-quoted token of a Markdown file that starts with one of the repository's own top-level
folders must name a file or folder that is there; a ``path::name`` token must also find ``name`` in
that file.  Checked: every file under ``profiles/``, ``docs/`` and ``web/`` and every Markdown file of the repository root that
carries the marker comment ``<!-- docs-links: checked -->`` (notes written by other parties quote
paths of other snapshots and carry no marker).  Paths of other projects (they start with other
folders) are not checked.  Parity: the reference's docs-link gate (tests/test_docs_links.py).
"""
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OWN = ("tilerl_b200/", "csrc/", "tests/", "profiles/", "bench/", "k8s/", ".github/")
MARKER = "<!-- docs-links: checked -->"


def _tokens(text):
    for tok in re.findall(r"`([^`\n]+)`", text):
        tok = tok.strip()
        if tok.startswith(OWN) and " " not in tok:
            yield tok


def _exists(tok: str) -> bool:
    path, _, name = tok.partition("::")
    path = re.sub(r":\d+(-\d+)?$", "", path)          # file:line or file:line-line
    if any(c in path for c in "*{<"):                  # a pattern: at least one match
        return bool(glob.glob(os.path.join(ROOT, path.replace("{", "[").replace("}", "]")))) or \
            bool(glob.glob(os.path.join(ROOT, re.sub(r"\{[^}]*\}", "*", path))))
    full = os.path.join(ROOT, path)
    if not os.path.exists(full):
        return False
    if name and os.path.isfile(full):
        first = re.split(r"[.(\[]", name)[0].rstrip("*")
        return first in open(full, errors="ignore").read()
    return True


def test_paths_quoted_in_the_markdown_files_exist():
    files = [p for p in glob.glob(os.path.join(ROOT, "*.md")) if MARKER in open(p, errors="ignore").read(2000)]
    assert len(files) >= 3, "the repository's own documents carry the marker"
    files += glob.glob(os.path.join(ROOT, "profiles", "*.md")) + glob.glob(os.path.join(ROOT, "docs", "*.md")) + \
        glob.glob(os.path.join(ROOT, "web", "*.md"))
    missing = []
    for f in files:
        for tok in _tokens(open(f, errors="ignore").read()):
            if not _exists(tok):
                missing.append((os.path.relpath(f, ROOT), tok))
    assert not missing, missing[:20]
