"""`bux-lsp`: a language server for `.bux` files over stdio (JSON-RPC 2.0 with
Content-Length framing). It keeps the open documents' text and answers with the pure
functions of `features`: diagnostics on open / change, hover, completion, definition.
Reference: ``lang/lsp/server.py``."""

from __future__ import annotations

import json
import sys

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
    def publish(self, uri: str) -> None:
        self.send({"method": "textDocument/publishDiagnostics",
                   "params": {"uri": uri, "diagnostics": features.diagnostics(self.docs[uri], uri)}})

    def handle(self, msg: dict) -> None:
        method, params, rid = msg.get("method"), msg.get("params") or {}, msg.get("id")
        if method == "initialize":
            self.send({"id": rid, "result": {"capabilities": {
                "textDocumentSync": 1, "hoverProvider": True, "definitionProvider": True,
                "completionProvider": {"triggerCharacters": ["(", ",", " ", "="]}},
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
            text = self.docs.get(uri, "")
            pos = params["position"]
            if method.endswith("hover"):
                h = features.hover(text, pos["line"], pos["character"])
                result = None if h is None else {"contents": {"kind": "plaintext", "value": h}}
            elif method.endswith("completion"):
                result = features.completion(text, pos["line"], pos["character"])
            else:
                rng = features.definition(text, pos["line"], pos["character"])
                result = None if rng is None else {"uri": uri, "range": rng}
            self.send({"id": rid, "result": result})
        elif rid is not None:
            self.send({"id": rid, "error": {"code": -32601, "message": f"no method {method}"}})

    def serve(self) -> None:
        while self.running:
            msg = self.read()
            if msg is None:
                break
            self.handle(msg)
