"""Finding what ``use NAME`` names and joining files into one program.

A module is a ``.bux`` file found by name, never by path. Search order (behaviour
of the reference, ``src/bux/lang/modules.py``): the folder of the using file, then
every folder listed under ``[tool.bux] path`` of the nearest ``pyproject.toml``
(sub-folders included), then the folders of ``BUX_PATH``.

A `Program` is a stack of *layers* of statements: used modules first (in the order
met, depth first), then the main file, then the command line's overrides. A later
layer's definition of a name replaces earlier ones everywhere. All files are joined
into one text so that every span indexes one string; `Program.locate` maps an error
back to the file it is in.
"""

from __future__ import annotations

import difflib
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Mapping, Optional, Sequence

from . import syntax
from .syntax import BuxError, Span

COMMAND_LINE = "<command line>"
_SKIPPED_DIRS = frozenset({"__pycache__", "node_modules"})
Loader = Callable[[str, str], tuple]


def _project_path(start: Path) -> list:
    try:
        import tomllib
    except ImportError:  # pragma: no cover
        return []
    for folder in (start, *start.parents):
        pyproject = folder / "pyproject.toml"
        if pyproject.is_file():
            with pyproject.open("rb") as f:
                tool = tomllib.load(f).get("tool", {}).get("bux", {})
            return [folder / p for p in tool.get("path", [])]
    return []


def search_roots(importer: str) -> list:
    here = (Path.cwd() if importer.startswith("<") else Path(importer).parent).resolve()
    env = [Path(p) for p in os.environ.get("BUX_PATH", "").split(os.pathsep) if p]
    roots = [(here, False)]
    for root in _project_path(here) + env:
        if root.is_dir() and (root.resolve(), True) not in roots:
            roots.append((root.resolve(), True))
    return roots


def _bux_files(root: Path, recursive: bool) -> dict:
    found: dict = {}
    for folder, dirs, files in os.walk(root):
        dirs[:] = sorted(d for d in dirs if not d.startswith(".") and d not in _SKIPPED_DIRS)
        if not recursive:
            dirs.clear()
        for name in sorted(files):
            if name.endswith(".bux"):
                found.setdefault(name[:-4], []).append(Path(folder) / name)
    return found


def find(name: str, importer: str) -> tuple:
    """Return (source, filename) of module `name` used by file `importer`."""
    seen: list = []
    for root, recursive in search_roots(importer):
        files = _bux_files(root, recursive)
        seen += list(files)
        hits = files.get(name)
        if not hits:
            continue
        if len(hits) > 1:
            listed = ", ".join(str(h) for h in hits)
            raise BuxError(f"module '{name}' is ambiguous under {root}: {listed}")
        return hits[0].read_text(), str(hits[0])
    close = difflib.get_close_matches(name, sorted(set(seen)), n=1)
    raise BuxError(f"no module named '{name}'",
                   hint=f"did you mean '{close[0]}'?" if close else
                   "modules are .bux files in this folder, under [tool.bux] path, or BUX_PATH")


def from_mapping(sources: Mapping) -> Loader:
    def loader(name: str, importer: str) -> tuple:
        if name not in sources:
            raise BuxError(f"no module named '{name}'")
        return sources[name], f"{name}.bux"

    return loader


@dataclass
class _File:
    filename: str
    start: int
    stop: int


@dataclass
class Program:
    source: str = ""
    layers: list = field(default_factory=list)  # list[list[Statement]]
    files: list = field(default_factory=list)
    broken: set = field(default_factory=set)
    incomplete: bool = False
    errors: list = field(default_factory=list)

    def file_of(self, offset: int) -> _File:
        for f in self.files:
            if f.start <= offset <= f.stop:
                return f
        return self.files[0]

    def locate(self, err: BuxError) -> BuxError:
        """Attach `err` to the file its span is in, spans rebased to that file."""
        if err.source is not None or not self.files:
            return err
        if err.span is None:
            main = next((f for f in self.files if not f.filename.startswith("<command")),
                        self.files[0])
            return err.attach(self.source[main.start:main.stop], main.filename)
        f = self.file_of(err.span.start)
        err.span = Span(err.span.start - f.start, err.span.end - f.start)
        return err.attach(self.source[f.start:f.stop], f.filename)


def load(source: str, filename: str = "<string>", *, overrides: Sequence = (),
         loader: Optional[Loader] = None, recover: bool = False) -> Program:
    """Parse `source`, every module it uses (transitively) and the overrides."""
    loader = loader or find
    prog = Program()
    loaded: dict = {}
    stack: list = []

    def add_text(text: str, name: str) -> _File:
        start = len(prog.source)
        prog.source += text + "\n"
        f = _File(name, start, start + len(text))
        prog.files.append(f)
        return f

    def parse_into(text: str, name: str) -> list:
        f = add_text(text, name)
        errors: Optional[list] = [] if recover else None
        try:
            tokens = syntax.tokenize(prog.source, f.start, f.stop, errors)
            items, broken = syntax.Parser(prog.source, tokens).program(errors)
        except BuxError as err:
            raise prog.locate(err) from None
        prog.broken.update(broken)
        if errors:
            prog.errors += [prog.locate(e) for e in errors]
        return items

    def visit(text: str, name: str, into: list) -> None:
        """Depth-first: a file's modules come before the file itself."""
        items = parse_into(text, name)
        own = []
        for st in items:
            if st.use is None:
                own.append(st)
                continue
            if st.use in stack:
                raise prog.locate(BuxError(
                    f"modules use each other in a cycle: {' -> '.join([*stack, st.use])}",
                    st.name_span))
            if st.use in loaded:
                continue
            try:
                mod_src, mod_file = loader(st.use, name)
            except BuxError as err:
                err.span = err.span or st.name_span
                if recover:
                    prog.errors.append(prog.locate(err))
                    prog.incomplete = True
                    continue
                raise prog.locate(err) from None
            loaded[st.use] = mod_file
            stack.append(st.use)
            visit(mod_src, mod_file, into)
            stack.pop()
        into.extend(_split_layers(own))

    main_layers: list = []
    visit(source, filename, main_layers)
    # The main file's modules may also come from overrides (``use recipe``).
    if overrides:
        visit("\n".join(overrides), COMMAND_LINE, main_layers)
    prog.layers = main_layers
    return prog


def _split_layers(statements: list) -> list:
    """A file's plain definitions, then (one layer up) its amendments, those of one
    name merged into a single call so that ``a.x = 1`` and ``a.y = 2`` both apply."""
    from dataclasses import replace

    plain = [st for st in statements if not st.amends]
    merged: dict = {}
    for st in statements:
        if not st.amends:
            continue
        prev = merged.get(st.name)
        if prev is not None:
            body = replace(prev.body, span=prev.body.span.to(st.body.span),
                           args=prev.body.args + st.body.args)
            st = replace(prev, span=prev.span.to(st.span), body=body)
        merged[st.name] = st
    return [plain, list(merged.values())] if merged else [plain]


def extended(program: Program, statement: str, name: str = COMMAND_LINE) -> Program:
    """A copy of `program` with one more top layer holding `statement`."""
    new = Program(program.source, list(program.layers), list(program.files),
                  set(program.broken), program.incomplete, list(program.errors))
    start = len(new.source)
    new.source += statement + "\n"
    f = _File(name, start, start + len(statement))
    new.files.append(f)
    tokens = syntax.tokenize(new.source, f.start, f.stop)
    items, _ = syntax.Parser(new.source, tokens).program()
    new.layers.append(items)
    return new
