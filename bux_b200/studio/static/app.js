// bux studio: the source, the model and the training of one .bux file, each editing the file's
// text. The page holds the text; every edit (typing or visual) makes a new text, which goes
// through the compiler (/api/view) before anything is drawn from it.
import { api, Conflict } from "./api.js";
import { el, clear, si } from "./dom.js";
import { Editor } from "./editor.js";
import { drawModel, nodeAt, nodes } from "./diagram.js";
import { showInspector, showTraining, showSweep } from "./panels.js";

const $ = id => document.getElementById(id);

const app = {
  source: "", saved: "", mtime: null, run: 0, view: null, picked: null, fresh: false,
  undo: [], redo: [], lastKind: null, lastAt: 0, palette: [],

  // -- the text and its history: a visual edit is one step, a burst of typing another
  setSource(text, kind) {
    if (text === this.source) return;
    const now = Date.now();
    if (!(kind === "typing" && this.lastKind === "typing" && now - this.lastAt < 1200)) { this.undo.push(this.source); this.redo = []; }
    this.lastKind = kind; this.lastAt = now;
    this.source = text;
    this.stale();
    this.refresh();
  },
  step(from, to) {
    if (!from.length) return;
    to.push(this.source);
    this.source = from.pop(); this.lastKind = null;
    editor.set(this.source); this.stale(); this.refresh();
  },
  stale() { this.fresh = false; $("diagram-scroll").classList.add("stale"); $("dirty").classList.toggle("on", this.source !== this.saved); $("undo").disabled = !this.undo.length; $("redo").disabled = !this.redo.length; },

  // -- what the compiler says the text means
  refresh() {
    clearTimeout(this.timer);
    this.timer = setTimeout(async () => {
      const text = this.source;
      let v;
      try { v = await api.view(text, this.run); } catch (err) { $("status").textContent = String(err.message); return; }
      if (text !== this.source) return;            // typed on since
      this.view = v;
      editor.show(v.errors);
      const errors = clear($("errors"));
      for (const e of v.errors) errors.append(el("div", { onclick: () => { editor.area.focus(); editor.area.setSelectionRange(e.start, e.end); } },
        `line ${text.slice(0, e.start).split("\n").length}: ${e.message}`));
      if (v.errors.length) { $("status").textContent = `${v.errors.length} error${v.errors.length > 1 ? "s" : ""}: the drawing shows the last text that compiled`; return; }
      if (!v.model) { $("status").textContent = "this file defines no model to draw"; return; }
      this.fresh = true;
      $("diagram-scroll").classList.remove("stale");
      $("status").textContent = "";
      this.run = v.run || 0;
      drawModel($("diagram"), v.model, ui);
      const c = v.card;
      clear($("card")).append(el("span", {}, el("b", {}, si(c.params)), " parameters · width ", el("b", {}, c.d_model), " · vocabulary ", el("b", {}, si(c.vocab_size)),
        ` · ${c.layers} layers: `, c.by_type.map(([t, n]) => `${t}×${n}`).join("  "), c.residual ? ` · residual ${c.residual}` : ""));
      const pick = clear($("run-pick"));
      v.runs.forEach(r => pick.append(el("option", { value: r.index, selected: r.index === this.run }, r.name)));
      pick.hidden = v.runs.length < 2;
      showTraining($("training"), this, v.training);
      showSweep($("sweep"), this, v.sweep, v.runs, this.run);
      if (this.picked) {                           // keep the selection where the text still writes it
        const again = [...nodes(v.model)].find(n => n.span && this.picked.span && n.span[0] === this.picked.span[0] && n.kind === this.picked.kind);
        ui.pick(again || null, again ? document.querySelector(`#diagram g[data-id="${again.id}"]`) : null);
      }
    }, 250);
  },

  // -- a visual edit: refused while the drawing is behind the text
  async edit(edit) {
    if (!this.fresh) { $("status").textContent = "the source has errors or the drawing has not caught up: no visual edit is made"; return; }
    let reply;
    try { reply = await api.edit(this.source, edit); } catch (err) { $("status").textContent = String(err.message); return; }
    if (reply.error) { $("status").textContent = reply.error; return; }
    editor.set(reply.source);
    this.setSource(reply.source, "visual");
  },

  pickRun(index) { this.run = index; this.stale(); this.refresh(); },

  async save(overwrite = false) {
    try {
      const r = await api.save(this.source, this.mtime, overwrite);
      this.mtime = r.mtime; this.saved = this.source; this.stale(); if (this.view && !this.view.errors.length) { this.fresh = true; $("diagram-scroll").classList.remove("stale"); }
      $("status").textContent = "saved";
    } catch (err) {
      if (!(err instanceof Conflict)) { $("status").textContent = String(err.message); return; }
      ask("The file changed on disk since the page loaded it.", { "reload from disk": () => this.load(), "overwrite it": () => this.save(true), "cancel": () => {} });
    }
  },

  async load() {
    const f = await api.file();
    this.mtime = f.mtime; this.saved = f.exists ? f.source : ""; this.source = f.source; this.undo = []; this.redo = [];
    editor.set(f.source, false); this.stale(); this.refresh();
  },

  // the file on disk is watched: reloaded when there are no unsaved edits, asked about otherwise
  async watch() {
    let f;
    try { f = await api.file(); } catch { return; }
    if (f.mtime === this.mtime || !f.exists) return;
    if (this.source === this.saved) return this.load();
    if (!this.asked || this.asked !== f.mtime) {
      this.asked = f.mtime;
      ask("The file changed on disk and the page has unsaved edits.", { "reload from disk": () => this.load(), "keep mine": () => { this.mtime = f.mtime; } });
    }
  },
};

function ask(text, choices) {
  const box = clear($("ask"));
  box.append(el("div", {}, el("p", {}, text), Object.entries(choices).map(([label, fn]) => el("button", { onclick: () => { box.hidden = true; fn(); } }, label))));
  box.hidden = false;
}

const ui = {
  pick(node, g) {
    document.querySelectorAll("#diagram .picked").forEach(x => x.classList.remove("picked"));
    app.picked = node;
    $("toolbar").hidden = true; $("palette").hidden = true;
    if (!node) { editor.select(null); return showInspector($("inspector"), app, null); }
    if (g) {
      g.classList.add("picked");
      if (node.span) {
        const box = g.getBoundingClientRect(), pane = $("model-pane").getBoundingClientRect();
        const bar = $("toolbar"); bar.hidden = false;
        bar.style.left = Math.max(4, box.left - pane.left) + "px"; bar.style.top = Math.max(44, box.top - pane.top - 34) + "px";
        bar.querySelector('[data-act="unwrap"]').hidden = node.kind !== "residual";
      }
    }
    editor.select(node.span);
    showInspector($("inspector"), app, node);
  },
  open(node) {
    // a layer's inside, drawn by the same code in an overlay; its boxes select nothing in the source
    const box = clear($("ask"));
    const picture = document.createElementNS("http://www.w3.org/2000/svg", "svg");
    picture.id = "inside";
    const close = () => { box.hidden = true; };
    box.append(el("div", { style: "max-width:90vw;max-height:90vh;overflow:auto" }, el("h3", {}, `${node.title}${node.name ? " · " + node.name : ""}`),
      picture, el("div", {}, el("button", { onclick: close }, "close"))));
    drawModel(picture, node.inside, { pick() {}, repeat() {} });
    picture.classList.add("diagram");
    box.hidden = false;
  },
  repeat(node) {
    const n = prompt("repeat how many times?", node.times);
    if (n && /^\d+$/.test(n.trim()) && node.span) app.edit({ op: "set_repeat", start: node.span[0], end: node.span[1], times: Number(n) });
  },
};

const editor = new Editor((text, kind) => app.setSource(text, kind), offset => {
  if (!app.fresh || !app.view) return;
  const node = nodeAt(app.view.model, offset);
  if (node && node !== app.picked) ui.pick(node, document.querySelector(`#diagram g[data-id="${node.id}"]`));
});

function openPalette(after) {
  const root = clear($("palette"));
  for (const group of app.palette) {
    root.append(el("h4", {}, group.group));
    for (const item of group.items) root.append(el("button", { title: item.note, onclick: () => {
      root.hidden = true;
      const n = app.picked;
      if (n && n.span) app.edit({ op: "insert", start: n.span[0], end: n.span[1], text: item.insert, after });
    } }, item.name));
  }
  root.hidden = false;
}

$("toolbar").addEventListener("click", ev => {
  const act = ev.target.dataset.act, n = app.picked;
  if (!act || !n || !n.span) return;
  const at = { start: n.span[0], end: n.span[1] };
  // the stream runs upward: "above" comes after in the text
  if (act === "above") openPalette(true);
  else if (act === "below") openPalette(false);
  else if (act === "wrap") app.edit({ op: "wrap", ...at });
  else if (act === "unwrap") app.edit({ op: "unwrap", ...at });
  else if (act === "delete") app.edit({ op: "delete", ...at });
  else if (act === "repeat") { const k = prompt("repeat how many times?", n.times || 2); if (k && /^\d+$/.test(k.trim())) app.edit({ op: "set_repeat", ...at, times: Number(k) }); }
});

document.querySelectorAll("nav button").forEach(b => b.addEventListener("click", () => {
  document.querySelectorAll("nav button").forEach(x => x.classList.toggle("on", x === b));
  for (const tab of ["inspector", "training", "sweep"]) $(tab).hidden = tab !== b.dataset.tab;
}));
$("save").addEventListener("click", () => app.save());
$("undo").addEventListener("click", () => app.step(app.undo, app.redo));
$("redo").addEventListener("click", () => app.step(app.redo, app.undo));
$("run-pick").addEventListener("change", ev => app.pickRun(Number(ev.target.value)));
$("export-svg").addEventListener("click", () => {
  const copy = $("diagram").cloneNode(true);
  const style = el("style", {}, "text{font:11px sans-serif}.title{font-weight:600}.chip{fill:#6b7280;font-size:10px}.box{stroke:#9ca3af}.frame{fill:none;stroke:#9ca3af;stroke-dasharray:4 3}.wire{stroke:#6b7280;fill:none}");
  copy.prepend(style);
  const text = new XMLSerializer().serializeToString(copy).replace(/var\(--attn\)/g, "#dbeafe").replace(/var\(--ffn\)/g, "#dcfce7").replace(/var\(--norm\)/g, "#f3f4f6").replace(/var\(--rec\)/g, "#fef3c7").replace(/var\(--ends\)/g, "#ede9fe");
  const a = el("a", { href: URL.createObjectURL(new Blob([text], { type: "image/svg+xml" })), download: ($("file-name").textContent || "model").replace(/\.bux$/, "") + ".svg" });
  a.click();
});
document.addEventListener("keydown", ev => {
  const mod = ev.ctrlKey || ev.metaKey;
  if (mod && ev.key.toLowerCase() === "s") { ev.preventDefault(); app.save(); }
  else if (mod && ev.key.toLowerCase() === "z") { ev.preventDefault(); ev.shiftKey ? app.step(app.redo, app.undo) : app.step(app.undo, app.redo); }
  else if ((ev.key === "Delete" || ev.key === "Backspace") && document.activeElement !== editor.area && !/INPUT|SELECT|TEXTAREA/.test(document.activeElement.tagName) && app.picked && app.picked.span) {
    ev.preventDefault(); app.edit({ op: "delete", start: app.picked.span[0], end: app.picked.span[1] });
  }
});
window.addEventListener("beforeunload", ev => { if (app.source !== app.saved) ev.preventDefault(); });

(async () => {
  const s = await api.session();
  $("file-name").textContent = s.name; document.title = `${s.name} · bux studio`;
  app.palette = s.palette;
  await app.load();
  setInterval(() => app.watch(), 2000);
})();
