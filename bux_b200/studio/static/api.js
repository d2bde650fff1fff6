// The studio's API: every call carries the session's token, which the page's URL holds.
const token = new URLSearchParams(location.search).get("t") || new URLSearchParams(location.search).get("token") || "";

export class Conflict extends Error {}

async function call(method, path, body) {
  const reply = await fetch(`${path}?t=${encodeURIComponent(token)}`, {
    method, headers: body ? { "Content-Type": "application/json" } : {}, body: body ? JSON.stringify(body) : undefined });
  const value = await reply.json().catch(() => ({ error: reply.statusText }));
  if (reply.status === 409) { const e = new Conflict(value.error); e.mtime = value.mtime; throw e; }
  if (!reply.ok) throw new Error(value.error || reply.statusText);
  return value;
}

export const api = {
  session: () => call("GET", "/api/session"),
  file: () => call("GET", "/api/file"),
  runs: () => call("GET", "/api/runs"),
  view: (source, run) => call("POST", "/api/view", { source, run }),
  inspect: (source, start, end) => call("POST", "/api/inspect", { source, start, end }),
  edit: (source, edit) => call("POST", "/api/edit", { source, edit }),
  complete: (source, offset) => call("POST", "/api/complete", { source, offset }),
  hover: (source, offset) => call("POST", "/api/hover", { source, offset }),
  save: (source, mtime, overwrite) => call("POST", "/api/save", { source, mtime, overwrite }),
  train: (action, only) => call("POST", "/api/train", { action, only }),
};
