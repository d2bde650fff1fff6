"""The studio's HTTP server: Python's standard library serves the page (plain ES modules,
SVG and CSS under ``static/``) and a JSON API behind the session's token.

====== ======================= ==========================================================
GET    ``/``, ``/static/...``  the page; the token travels in the URL's query
GET    ``/api/session``        the file's path, whether it exists, the palette
GET    ``/api/file``           the text on disk and its modification time
POST   ``/api/view``           ``{source, run}`` → what the page draws (`view.view`)
POST   ``/api/inspect``        ``{source, start, end}`` → the inspector's form
POST   ``/api/edit``           ``{source, edit}`` → ``{source}`` or ``{error}``
POST   ``/api/complete``       ``{source, offset}`` → completions (as ``bux-lsp`` gives them)
POST   ``/api/hover``          ``{source, offset}`` → hover text
POST   ``/api/save``           ``{source, mtime, overwrite}`` → writes the file in one step,
                               keeping its line endings; refused (409) when the file changed
                               on disk since the page loaded it
POST   ``/api/train``          ``{action: start|stop, only}``; ``GET /api/runs`` → states, curves
====== ======================= ==========================================================

Requests without the token get 403; requests whose ``Host`` is not the address the studio
listens on get 400 (a page on another origin cannot reach the API through the browser).
Reference: ``studio/server.py``.
"""

from __future__ import annotations

import json
import os
import secrets
import tempfile
from http import HTTPStatus
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from pathlib import Path
from urllib.parse import parse_qs, urlparse

from ..lang import syntax
from ..lang.lsp import features
from . import edits, forms, palette
from . import view as drawing
from .training import Trainings

STATIC = Path(__file__).with_name("static")
KINDS = {".html": "text/html; charset=utf-8", ".js": "text/javascript; charset=utf-8", ".css": "text/css; charset=utf-8",
         ".svg": "image/svg+xml"}
TEMPLATE = """# a new file: a small model and its run
d_model = 256
vocab_size = 32768

norm = rmsnorm
attn = gqa(num_heads=4, num_kv_heads=2, rope=rope())
ffn = gated_mlp(intermediate_size=4 * d_model, activation=swish)
block = [norm attn] [norm ffn]
model = embed block^4 norm head(tied=true)

data = synthetic
optimizer = adamw(lr=3e-3)
schedule = wsd(warmup=20)
seq_len = 256
batch = 8
steps = 200
"""


class Refused(Exception):
    def __init__(self, status: int, body: dict):
        super().__init__(body.get("error", ""))
        self.status, self.body = status, body


def set_value(source: str, name: str, value: str) -> str:
    """``name = value`` replaced where the file writes it, appended when it does not."""
    return edits.set_setting(source, name, value)


class Studio:
    def __init__(self, file, out="runs"):
        self.file, self.out = Path(file), Path(out)
        self.token = secrets.token_urlsafe(16)
        self.trainings = Trainings(self.file, self.out)

    # -- the file on disk
    def mtime(self):
        try:
            return self.file.stat().st_mtime_ns
        except OSError:
            return None

    def source(self) -> str:
        """The file's text with ``\\n`` line ends (the page edits that; a save puts the file's own back)."""
        if not self.file.exists():
            return TEMPLATE
        return self.file.read_bytes().decode("utf-8").replace("\r\n", "\n")

    def newline(self) -> str:
        try:
            return "\r\n" if b"\r\n" in self.file.read_bytes() else "\n"
        except OSError:
            return "\n"

    # -- the API
    def session(self, body, query) -> dict:
        return {"file": str(self.file.resolve()), "exists": self.file.exists(), "name": self.file.name,
                "palette": palette.palette(self.source(), str(self.file))}

    def file_(self, body, query) -> dict:
        return {"source": self.source(), "mtime": self.mtime(), "exists": self.file.exists()}

    def view(self, body, query) -> dict:
        return drawing.view(_text(body, "source"), str(self.file), run=int(body.get("run") or 0))

    def inspect(self, body, query) -> dict:
        return forms.inspect(_text(body, "source"), int(body["start"]), int(body["end"]), str(self.file))

    def edit(self, body, query) -> dict:
        try:
            return {"source": edits.apply(_text(body, "source"), dict(body["edit"]), str(self.file))}
        except edits.EditError as err:
            return {"error": str(err)}
        except (KeyError, TypeError) as err:
            raise Refused(HTTPStatus.BAD_REQUEST, {"error": f"a malformed edit: {err}"}) from err

    def complete(self, body, query) -> list:
        items = features.complete(_text(body, "source"), int(body["offset"]), str(self.file))
        return [{"label": c.label, "kind": c.kind, "detail": c.detail, "doc": c.doc, "insert": c.insert or c.label} for c in items]

    def hover(self, body, query):
        h = features.hover(_text(body, "source"), int(body["offset"]), str(self.file))
        return None if h is None else {"start": h.start, "end": h.end, "text": h.text}

    def save(self, body, query) -> dict:
        """Write the file in one step (a temporary file moved into place) with its own line
        endings; refuse to write over a file that changed on disk since the page loaded it."""
        text = _text(body, "source")
        seen, now = body.get("mtime"), self.mtime()
        if now is not None and seen != now and not body.get("overwrite"):
            raise Refused(HTTPStatus.CONFLICT, {"error": "the file changed on disk since it was loaded", "mtime": now})
        nl = self.newline()
        data = text.replace("\r\n", "\n").replace("\n", nl).encode("utf-8")
        self.file.parent.mkdir(parents=True, exist_ok=True)
        fd, tmp = tempfile.mkstemp(dir=str(self.file.parent), prefix=f".{self.file.name}.")
        try:
            with os.fdopen(fd, "wb") as fh:
                fh.write(data)
            os.replace(tmp, self.file)
        except BaseException:
            Path(tmp).unlink(missing_ok=True)
            raise
        return {"mtime": self.mtime()}

    def train(self, body, query) -> dict:
        action = body.get("action", "start")
        if action == "stop":
            return self.trainings.stop()
        return self.trainings.start(body.get("only"))

    def runs(self, body, query) -> dict:
        from ..lang import compile_runs

        try:
            compiled = compile_runs(self.source(), filename=str(self.file))[:64]
        except syntax.BuxError:
            compiled = []
        return {"state": self.trainings.state(), "runs": self.trainings.runs(compiled), "log": self.trainings.tail()}

    ROUTES = {("GET", "/api/session"): session, ("GET", "/api/file"): file_, ("GET", "/api/runs"): runs,
              ("POST", "/api/view"): view, ("POST", "/api/inspect"): inspect, ("POST", "/api/edit"): edit,
              ("POST", "/api/complete"): complete, ("POST", "/api/hover"): hover, ("POST", "/api/save"): save,
              ("POST", "/api/train"): train}

    # ------------------------------------------------------------------ http
    def handler(self, hosts=None):
        studio = self

        class Handler(BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def send(self, status: int, data: bytes, kind: str) -> None:
                self.send_response(status)
                self.send_header("Content-Type", kind)
                self.send_header("Content-Length", str(len(data)))
                self.send_header("Cache-Control", "no-store")
                self.end_headers()
                self.wfile.write(data)

            def send_json(self, status: int, value) -> None:
                self.send(status, json.dumps(value, default=str).encode(), "application/json")

            def answer(self, method: str) -> None:
                url = urlparse(self.path)
                query = {k: v[-1] for k, v in parse_qs(url.query).items()}
                try:
                    host = (self.headers.get("Host") or "").rsplit(":", 1)[0]
                    if hosts is not None and host not in hosts:
                        raise Refused(HTTPStatus.BAD_REQUEST, {"error": "this is not the address the studio listens on"})
                    token = query.get("t") or query.get("token") or self.headers.get("X-Bux-Token")
                    if url.path.startswith("/api/"):
                        if token != studio.token:
                            raise Refused(HTTPStatus.FORBIDDEN, {"error": "bad token"})
                        fn = Studio.ROUTES.get((method, url.path))
                        if fn is None:
                            raise Refused(HTTPStatus.NOT_FOUND, {"error": "not found"})
                        body = {}
                        if method == "POST":
                            n = int(self.headers.get("Content-Length") or 0)
                            try:
                                body = json.loads(self.rfile.read(n) or b"{}")
                            except ValueError as err:
                                raise Refused(HTTPStatus.BAD_REQUEST, {"error": f"the body is not JSON: {err}"}) from err
                        return self.send_json(200, fn(studio, body, query))
                    if method != "GET":
                        raise Refused(HTTPStatus.METHOD_NOT_ALLOWED, {"error": "GET only"})
                    if url.path == "/":
                        if token != studio.token:
                            raise Refused(HTTPStatus.FORBIDDEN, {"error": "open the URL the studio printed: it carries the session's token"})
                        return self.send(200, (STATIC / "index.html").read_bytes(), KINDS[".html"])
                    name = url.path.removeprefix("/static/")
                    path = (STATIC / name).resolve()
                    if url.path.startswith("/static/") and path.is_file() and STATIC.resolve() in path.parents:
                        return self.send(200, path.read_bytes(), KINDS.get(path.suffix, "application/octet-stream"))
                    raise Refused(HTTPStatus.NOT_FOUND, {"error": "not found"})
                except Refused as err:
                    self.send_json(err.status, err.body)
                except Exception as err:  # noqa: BLE001 - the page shows it; the server keeps serving
                    self.send_json(500, {"error": f"{type(err).__name__}: {err}"})

            def do_GET(self):
                self.answer("GET")

            def do_POST(self):
                self.answer("POST")

        return Handler


def _text(body: dict, key: str) -> str:
    value = body.get(key)
    if not isinstance(value, str):
        raise Refused(HTTPStatus.BAD_REQUEST, {"error": f"'{key}' must be a string"})
    return value


def bind(studio: Studio, host: str, port: int, tries: int = 10) -> ThreadingHTTPServer:
    """A server on `port`, or on one of the next few when it is taken."""
    last = None
    for p in range(port, port + tries):
        try:
            return ThreadingHTTPServer((host, p), studio.handler({host, "localhost", "127.0.0.1"}))
        except OSError as err:
            last = err
    raise OSError(f"no free port in {port}..{port + tries - 1}: {last}")


def serve(file, port: int = 8765, out="runs", host: str = "127.0.0.1", browser: bool = True, echo=print) -> None:
    studio = Studio(file, out)
    server = bind(studio, host, port)
    port = server.server_address[1]
    url = f"http://{host}:{port}/?t={studio.token}"
    echo(f"bux studio: {studio.file.resolve()} at {url}")
    if os.environ.get("SSH_CONNECTION"):
        # a remote shell: no browser here; forward the port and open the URL on your machine
        echo(f"  over SSH: ssh -L {port}:127.0.0.1:{port} <this host>, then open the URL there")
    elif browser:
        import webbrowser

        try:
            webbrowser.open(url)
        except Exception:  # noqa: BLE001 - no browser is not an error
            pass
    try:
        server.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        server.server_close()
