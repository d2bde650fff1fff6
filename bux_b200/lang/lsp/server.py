"""`bux-lsp`: a language server for `.bux` files over stdio (JSON-RPC 2.0 with
Content-Length framing). It keeps the open documents' text and answers with the pure
functions of `features`: diagnostics on open / change, hover, completion, definition.
Reference: ``lang/lsp/server.py``."""

from __future__ import annotations

import json
import sys
from urllib.parse import quote, unquote

from . import features


class Server:
    def __init__(self, reader=None, writer=None):
        self.reader = reader or sys.stdin.buffer
        self.writer = writer or sys.stdout.buffer
        self.docs: dict = {}
        self.running = True

    # -- framing
    def read(self):
        length = None
        while True:
            line = self.reader.readline()
            if not line:
                return None
            line = line.decode("ascii", "replace").strip()
            if not line:
                break
            if line.lower().startswith("content-length:"):
                length = int(line.split(":", 1)[1])
        if length is None:
            return None
        return json.loads(self.reader.read(length).decode("utf-8"))

    def send(self, payload: dict) -> None:
        body = json.dumps({"jsonrpc": "2.0", **payload}).encode("utf-8")
        self.writer.write(f"Content-Length: {len(body)}\r\n\r\n".encode("ascii") + body)
        self.writer.flush()

    # -- requests
    KINDS = {"field": 5, "value": 12, "layer": 7, "setting": 10, "definition": 6, "parameter": 6, "tap": 18,
             "keyword": 14, "text": 1}

    @staticmethod
    def path_of(uri: str) -> str:
        return unquote(uri[len("file://"):]) if uri.startswith("file://") else uri

    def _range(self, text: str, start: int, end: int) -> dict:
        a, b = features.position_of(text, start), features.position_of(text, end)
        return {"start": {"line": a[0], "character": a[1]}, "end": {"line": b[0], "character": b[1]}}

    def publish(self, uri: str) -> None:
        text = self.docs[uri]
        found = [{"range": self._range(text, d.start, d.end), "severity": 1, "source": "bux", "message": d.message}
                 for d in features.diagnostics(text, self.path_of(uri))]
        self.send({"method": "textDocument/publishDiagnostics", "params": {"uri": uri, "diagnostics": found}})

    def handle(self, msg: dict) -> None:
        method, params, rid = msg.get("method"), msg.get("params") or {}, msg.get("id")
        if method == "initialize":
            self.send({"id": rid, "result": {"capabilities": {
                "textDocumentSync": 1, "hoverProvider": True, "definitionProvider": True,
                "completionProvider": {"triggerCharacters": ["(", ",", " ", "=", ".", "@", "$", '"']}},
                "serverInfo": {"name": "bux-lsp"}}})
        elif method == "shutdown":
            self.send({"id": rid, "result": None})
        elif method == "exit":
            self.running = False
        elif method == "textDocument/didOpen":
            doc = params["textDocument"]
            self.docs[doc["uri"]] = doc["text"]
            self.publish(doc["uri"])
        elif method == "textDocument/didChange":
            uri = params["textDocument"]["uri"]
            self.docs[uri] = params["contentChanges"][-1]["text"]
            self.publish(uri)
        elif method == "textDocument/didClose":
            self.docs.pop(params["textDocument"]["uri"], None)
        elif method in ("textDocument/hover", "textDocument/completion", "textDocument/definition"):
            uri = params["textDocument"]["uri"]
            text, path = self.docs.get(uri, ""), self.path_of(uri)
            at = features.offset_of(text, params["position"]["line"], params["position"]["character"])
            try:
                result = self._answer(method, uri, text, path, at)
            except Exception as err:   # a feature must not take the server down with it
                self.send({"id": rid, "error": {"code": -32603, "message": f"{type(err).__name__}: {err}"}})
                return
            self.send({"id": rid, "result": result})
        elif rid is not None:
            self.send({"id": rid, "error": {"code": -32601, "message": f"no method {method}"}})

    def _answer(self, method: str, uri: str, text: str, path: str, at: int):
        if method.endswith("hover"):
            h = features.hover(text, at, path)
            return None if h is None else {"contents": {"kind": "markdown", "value": h.text},
                                           "range": self._range(text, h.start, h.end)}
        if method.endswith("completion"):
            return {"isIncomplete": False, "items": [
                {"label": c.label, "kind": self.KINDS.get(c.kind, 1), "detail": c.detail, "sortText": c.sort + c.label,
                 **({"insertText": c.insert} if c.insert else {}),
                 **({"documentation": {"kind": "markdown", "value": c.doc}} if c.doc else {})}
                for c in features.complete(text, at, path)]}
        found = features.definition(text, at, path)
        if found is None:
            return None
        file, start, end = found
        if file == path:
            return {"uri": uri, "range": self._range(text, start, end)}
        try:
            other = open(file).read()
        except OSError:
            return None
        return {"uri": "file://" + quote(file), "range": self._range(other, start, end)}

    def serve(self) -> None:
        while self.running:
            msg = self.read()
            if msg is None:
                break
            self.handle(msg)
