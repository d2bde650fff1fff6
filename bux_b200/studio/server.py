from __future__ import annotations

import json
import re
import secrets
import subprocess
import sys
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from pathlib import Path

from ..lang import compile_runs, syntax
from ..lang.lsp import features
from ..lang.render import render

PAGE = """<!doctype html><meta charset=utf-8><title>bux studio</title>
<style>body{font:14px system-ui;margin:0;display:grid;grid-template-columns:1fr 1fr;height:100vh}
textarea{font:13px ui-monospace,monospace;border:0;padding:12px;resize:none;outline:none}
#side{overflow:auto;padding:12px;background:#f6f6f4}pre{font:12px ui-monospace,monospace}
.err{color:#b00020;white-space:pre-wrap}button{margin-right:8px}</style>
<textarea id=src spellcheck=false></textarea><div id=side><button onclick=save()>save</button>
<button onclick=train()>train</button><span id=state></span><div id=errs class=err></div>
<h3>runs</h3><pre id=runs></pre><h3>graph</h3><pre id=graph></pre><h3>metrics</h3><pre id=metrics></pre></div>
<script>const T=new URLSearchParams(location.search).get('token');
async function api(p,b){const r=await fetch(p+'?token='+T,b?{method:'POST',body:JSON.stringify(b)}:{});return r.json()}
function show(v){errs.textContent=v.diagnostics.map(d=>`line ${d.range.start.line+1}: ${d.message}`).join('\\n');
runs.textContent=v.runs.map(r=>`${r.id}  ${r.name}  ${r.params} params`).join('\\n');graph.textContent=v.graph||'';
metrics.textContent=JSON.stringify(v.metrics,null,1)}
async function load(){const v=await api('/api/view');src.value=v.source;show(v)}
async function save(){show(await api('/api/source',{source:src.value}))}
async function train(){state.textContent=(await api('/api/train',{})).state}
let t;src.oninput=()=>{clearTimeout(t);t=setTimeout(save,600)};load();setInterval(async()=>show(await api('/api/view')),5000)
</script>"""


def set_value(source: str, name: str, value: str) -> str:
    """The source with the statement ``name = ...`` replaced (continuation lines included),
    or ``name = value`` appended when the file does not set it."""
    lines = source.split("\n")
    pat = re.compile(rf"^{re.escape(name)}\s*=")
    for i, line in enumerate(lines):
        if pat.match(line):
            j = i + 1
            while j < len(lines) and lines[j][:1] in (" ", "\t") and lines[j].strip():
                j += 1
            return "\n".join([*lines[:i], f"{name} = {value}", *lines[j:]])
    return source.rstrip("\n") + f"\n{name} = {value}\n"


class Studio:
    def __init__(self, file, out="runs"):
        self.file, self.out = Path(file), Path(out)
        self.token = secrets.token_urlsafe(16)
        self.buffer = self.file.read_text()
        self.job = None

    def view(self) -> dict:
        src = self.buffer
        diags = features.diagnostics(src, str(self.file))
        runs, graph = [], None
        if not diags:
            try:
                from ..train.trainer import count_params, directory

                compiled = compile_runs(src, filename=str(self.file))
                for r in compiled[:64]:
                    runs.append({"name": r.name, "id": r.id, "params": count_params(r.arch),
                                 "folder": str(directory(r, self.out))})
                graph = render(compiled[0].arch)
            except syntax.BuxError as err:
                diags = [{"range": {"start": {"line": 0, "character": 0}, "end": {"line": 0, "character": 1}},
                          "message": err.message}]
        metrics = {}
        for r in runs:
            st = Path(r["folder"]) / "status.json"
            if st.exists():
                try:
                    s = json.loads(st.read_text())
                    metrics[r["name"]] = {"state": s.get("state"), "step": s.get("step"),
                                          "loss": s.get("metrics", {}).get("loss")}
                except ValueError:
                    pass
        state = "idle" if self.job is None else ("training" if self.job.poll() is None else f"exit {self.job.returncode}")
        return {"source": src, "diagnostics": diags, "runs": runs, "graph": graph, "metrics": metrics, "state": state}

    def set_source(self, text: str) -> dict:
        self.buffer = text
        v = self.view()
        if not v["diagnostics"]:
            self.file.write_text(text)
        return v

    def set(self, name: str, value: str) -> dict:
        return self.set_source(set_value(self.buffer, name, value))

    def train(self) -> dict:
        if self.job is not None and self.job.poll() is None:
            return {"state": "training"}
        self.job = subprocess.Popen([sys.executable, "-m", "bux_b200", "launch", str(self.file), "--out", str(self.out)],
                                    stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        return {"state": "training"}

    # ------------------------------------------------------------------ http
    def handler(self):
        studio = self

        class Handler(BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def _reply(self, code, body, kind="application/json"):
                data = body.encode() if isinstance(body, str) else json.dumps(body, default=str).encode()
                self.send_response(code)
                self.send_header("Content-Type", kind)
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

            def _allowed(self) -> bool:
                return f"token={studio.token}" in (self.path.split("?", 1) + [""])[1]

            def do_GET(self):
                path = self.path.split("?")[0]
                if path == "/":
                    return self._reply(200 if self._allowed() else 403, PAGE if self._allowed() else "forbidden", "text/html")
                if not self._allowed():
                    return self._reply(403, {"error": "bad token"})
                if path == "/api/view":
                    return self._reply(200, studio.view())
                self._reply(404, {"error": "not found"})

            def do_POST(self):
                if not self._allowed():
                    return self._reply(403, {"error": "bad token"})
                n = int(self.headers.get("Content-Length") or 0)
                body = json.loads(self.rfile.read(n) or b"{}")
                path = self.path.split("?")[0]
                if path == "/api/source":
                    return self._reply(200, studio.set_source(body["source"]))
                if path == "/api/set":
                    return self._reply(200, studio.set(body["name"], body["value"]))
                if path == "/api/train":
                    return self._reply(200, studio.train())
                self._reply(404, {"error": "not found"})

        return Handler


def serve(file, port: int = 8765, out="runs", echo=print) -> None:
    studio = Studio(file, out)
    server = ThreadingHTTPServer(("127.0.0.1", port), studio.handler())
    echo(f"bux studio: http://127.0.0.1:{port}/?token={studio.token}")
    try:
        server.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        server.server_close()
