"""Copyright banner stamping / checking for a source tree.

``python -m lm_engine_b200.utils.license_header --repo . --header "Copyright (c) 2026, __authors__" [--check]``

Same command line and banner format as the reference's pre-commit hook (tools/copyright.py:11-182), so a tree stamped
by either is accepted by the other: a three-line banner (a row of asterisks, the copyright line, a row of asterisks)
followed by one blank line, written in the comment syntax of the file's family.  ``__authors__`` in the header is
replaced by the file's git authors (sorted, ``--extra-name`` first), or dropped with ``--no-contributors``.
"""

from __future__ import annotations

import argparse
import os
import re
import subprocess
from dataclasses import dataclass

_STARS = "*" * 50


@dataclass(frozen=True)
class BannerStyle:
    """How one family of files writes the banner: ``open_``/``close`` wrap the block, ``prefix`` starts each line."""

    suffixes: tuple[str, ...]
    prefix: str          # per-line comment leader ("" for block comments)
    open_: str           # text before the first row of asterisks
    close: str           # text after the last row of asterisks

    def render(self, line: str) -> str:
        lead = f"{self.prefix} " if self.prefix else ""
        body = "\n".join(f"{lead}{part}" for part in line.split("\n"))
        first = f"{self.open_}{lead}{_STARS}" if not self.open_ else f"{self.open_} {_STARS}"
        last = f"{lead}{_STARS}{self.close}" if not self.close else f"{_STARS} {self.close}"
        return f"{first}\n{body}\n{last}\n\n"

    def pattern(self) -> re.Pattern:
        lead = re.escape(f"{self.prefix} ") if self.prefix else ""
        first = rf"{re.escape(self.open_)} \*+" if self.open_ else rf"{lead}\*+"
        last = rf"\*+ {re.escape(self.close)}" if self.close else rf"{lead}\*+"
        return re.compile(rf"{first}\n{lead}\s*Copyright[^\n]*\n{last}\n\n")


STYLES = (
    BannerStyle((".cu", ".cuh", ".h", ".c", ".cpp"), "//", "", ""),
    BannerStyle((".py", ".yml", ".yaml", ".clang-format", "requirements-dev.txt", "requirements.txt", "setup.cfg",
                 "Makefile"), "#", "", ""),
    BannerStyle((".html", ".md"), "", "<!--", "-->"),
)


def style_for(path: str) -> BannerStyle | None:
    for style in STYLES:
        if path.endswith(style.suffixes):
            return style
    return None


def authors_by_file(repo: str) -> dict[str, list[str]]:
    """One ``git log`` over the whole history: absolute path -> sorted author names."""
    try:
        out = subprocess.run(["git", "-C", repo, "log", "--name-only", "--format=%x00%an"], capture_output=True,
                             text=True, timeout=60).stdout
    except (subprocess.TimeoutExpired, OSError):
        return {}
    seen: dict[str, set[str]] = {}
    author = None
    for row in out.splitlines():
        if row.startswith("\x00"):
            author = row[1:]
        elif row and author:
            seen.setdefault(os.path.realpath(os.path.join(repo, row)), set()).add(author)
    return {path: sorted(names) for path, names in seen.items()}


def copyright_line(header: str, authors: list[str], extra_name: str | None) -> str:
    names = list(authors)
    if extra_name:
        names = [extra_name] + [n for n in names if n != extra_name]
    if names:
        return header.replace("__authors__", ", ".join(names))
    return header.replace(", __authors__", "").replace("__authors__", "")


def has_banner(text: str, style: BannerStyle) -> bool:
    return len(text) == 0 or style.pattern().match(text) is not None


def stamp(text: str, style: BannerStyle, line: str) -> str:
    """``text`` with exactly one, current banner at the top (an older banner is replaced; empty files stay empty)."""
    if len(text) == 0:
        return text
    banner = style.render(line)
    rest = style.pattern().sub("", text, count=1) if style.pattern().match(text) else text
    return banner + rest


def walk(repo: str, excluded: list[str]):
    banned = [os.path.realpath(os.path.join(repo, ".git"))] + [os.path.realpath(e) for e in excluded]

    def skip(path: str) -> bool:
        return any(path == b or path.startswith(b + os.sep) for b in banned)

    for root, dirs, files in os.walk(repo):
        dirs[:] = sorted(d for d in dirs if not skip(os.path.join(root, d)))
        for name in sorted(files):
            path = os.path.join(root, name)
            if not skip(path) and style_for(path) is not None:
                yield path


def run(repo: str, header: str, *, exclude: list[str] = (), extra_name: str | None = None,
        no_contributors: bool = False, check: bool = False) -> list[str]:
    """Stamps (or, with ``check``, only inspects) every recognised file; returns the files without a banner."""
    repo = os.path.realpath(repo)
    authors = {} if no_contributors else authors_by_file(repo)
    missing = []
    for path in walk(repo, list(exclude)):
        style = style_for(path)
        with open(path, "r") as f:
            text = f.read()
        if check:
            if not has_banner(text, style):
                missing.append(os.path.relpath(path, repo))
            continue
        line = copyright_line(header, authors.get(os.path.realpath(path), []), extra_name)
        new = stamp(text, style, line)
        if new != text:
            with open(path, "w") as f:
                f.write(new)
    return missing


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--repo", required=True)
    ap.add_argument("--exclude", help="comma-separated paths to leave alone")
    ap.add_argument("--header", required=True, help='e.g. "Copyright (c) 2026, __authors__"')
    ap.add_argument("--extra-name")
    ap.add_argument("--no-contributors", action="store_true")
    ap.add_argument("--check", action="store_true", help="change nothing; exit 1 if a file has no banner")
    a = ap.parse_args(argv)
    exclude = [e.strip() for e in a.exclude.split(",")] if a.exclude else []
    missing = run(a.repo, a.header, exclude=exclude, extra_name=a.extra_name, no_contributors=a.no_contributors,
                  check=a.check)
    for path in sorted(missing):
        print(f"No copyright found on '{path}'.")
    return 1 if missing else 0


if __name__ == "__main__":
    raise SystemExit(main())
