"""Copyright banner tool: formats per file family, idempotent stamping, check mode, exclusions."""

import os
import subprocess

from lm_engine_b200.utils import license_header as lh

HEADER = "Copyright (c) 2026, __authors__"


def _tree(tmp_path):
    (tmp_path / "a.py").write_text("import os\n")
    (tmp_path / "k.cu").write_text("__global__ void k() {}\n")
    (tmp_path / "doc.md").write_text("# title\n")
    (tmp_path / "empty.py").write_text("")
    (tmp_path / "data.bin").write_bytes(b"\x00\x01")
    (tmp_path / "skip").mkdir()
    (tmp_path / "skip" / "b.py").write_text("x = 1\n")
    return tmp_path


def test_banner_formats():
    line = "Copyright (c) 2026, A"
    stars = "*" * 50
    assert lh.style_for("x.cu").render(line) == f"// {stars}\n// {line}\n// {stars}\n\n"
    assert lh.style_for("x.py").render(line) == f"# {stars}\n# {line}\n# {stars}\n\n"
    assert lh.style_for("x.md").render(line) == f"<!-- {stars}\n{line}\n{stars} -->\n\n"
    assert lh.style_for("x.bin") is None


def test_author_substitution():
    assert lh.copyright_line(HEADER, ["B", "A"], None) == "Copyright (c) 2026, B, A"
    assert lh.copyright_line(HEADER, ["B", "A"], "A") == "Copyright (c) 2026, A, B"
    assert lh.copyright_line(HEADER, [], None) == "Copyright (c) 2026"
    assert lh.copyright_line(HEADER, [], "Z") == "Copyright (c) 2026, Z"


def test_stamp_check_and_exclude(tmp_path):
    root = _tree(tmp_path)
    skip = str(root / "skip")
    missing = lh.run(str(root), HEADER, exclude=[skip], no_contributors=True, check=True)
    assert sorted(missing) == ["a.py", "doc.md", "k.cu"]          # empty files pass, excluded and unknown files are not looked at
    assert lh.run(str(root), HEADER, exclude=[skip], extra_name="Someone", no_contributors=True) == []
    assert lh.run(str(root), HEADER, exclude=[skip], no_contributors=True, check=True) == []
    first = (root / "a.py").read_text()
    assert first.startswith("# " + "*" * 50 + "\n# Copyright (c) 2026, Someone\n") and first.endswith("import os\n")
    assert (root / "skip" / "b.py").read_text() == "x = 1\n"
    assert (root / "empty.py").read_text() == ""
    # stamping again with another name replaces the banner instead of stacking a second one
    lh.run(str(root), HEADER, exclude=[skip], extra_name="Other", no_contributors=True)
    again = (root / "a.py").read_text()
    assert again.count("Copyright") == 1 and "Other" in again and again.endswith("import os\n")
    assert lh.main(["--repo", str(root), "--header", HEADER, "--check"]) == 1          # skip/b.py is now in scope
    assert lh.main(["--repo", str(root), "--header", HEADER, "--check", "--exclude", skip]) == 0


def test_git_authors(tmp_path):
    root = _tree(tmp_path)
    env = dict(os.environ, GIT_AUTHOR_NAME="Ada", GIT_AUTHOR_EMAIL="a@x", GIT_COMMITTER_NAME="Ada",
               GIT_COMMITTER_EMAIL="a@x")
    for cmd in (["git", "init", "-q"], ["git", "add", "a.py"], ["git", "commit", "-qm", "one"]):
        subprocess.run(cmd, cwd=root, env=env, check=True)
    authors = lh.authors_by_file(str(root))
    assert authors[os.path.realpath(root / "a.py")] == ["Ada"]
    lh.run(str(root), HEADER)
    assert "# Copyright (c) 2026, Ada\n" in (root / "a.py").read_text()
    assert "// Copyright (c) 2026\n" in (root / "k.cu").read_text()       # never committed: no authors
