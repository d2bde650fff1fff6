// The side panels: the inspector of the selected node, the training (budget, learning-rate
// chart, data, evals, runs started from the page) and the sweep (axes, alternatives, runs).
import { api } from "./api.js";
import { el, svg, clear, si, markdown } from "./dom.js";

// ------------------------------------------------------------------ inspector
export async function showInspector(root, app, node) {
  clear(root);
  if (!node || !node.span) {
    root.append(el("p", { class: "why" }, node ? "This node is not written in this file (a module's, or made by the compiler)." : "Select a layer in the diagram, or move the cursor onto one in the source."));
    return;
  }
  let form;
  try { form = await api.inspect(app.source, node.span[0], node.span[1]); } catch (err) { root.append(el("p", { class: "why" }, String(err.message))); return; }
  root.append(el("h3", {}, form.name || node.kind, form.type && form.type !== form.name ? el("small", {}, `  ${form.type}`) : null));
  if (form.doc) { const p = el("p"); p.innerHTML = markdown(form.doc); root.append(p); }
  if (form.module) root.append(el("p", {}, `defined in ${form.module}: a change is written as an amendment in this file`));
  if (form.why) root.append(el("p", { class: "why" }, form.why));
  for (const f of form.fields) {
    const set = value => app.edit({ op: "set_field", start: node.span[0], end: node.span[1], key: f.name, value });
    let input;
    if (f.kind === "bool" || f.kind === "choice") {
      const options = f.kind === "bool" ? ["true", "false"] : f.options;
      input = el("select", { onchange: ev => set(ev.target.value === "(default)" ? null : ev.target.value) },
        [f.required ? null : "(default)", ...options, f.optional ? "none" : null].filter(x => x != null).map(o => el("option", { selected: f.written ? o === f.value : o === "(default)" }, o)));
    } else {
      input = el("input", { value: f.written ? f.value : "", placeholder: f.required ? "required" : `${f.default}`, type: "text",
        onchange: ev => set(ev.target.value.trim() === "" ? null : ev.target.value.trim()) });
    }
    if (form.why) input.disabled = true;
    const note = el("small"); note.innerHTML = markdown(f.note || "");
    root.append(el("div", { class: "field" }, el("label", { class: f.written ? "written" : "", title: f.kind === "config" ? f.types.join(" | ") : f.kind }, f.name), input, f.note ? note : null));
  }
}

// ------------------------------------------------------------------ training
export function showTraining(root, app, t) {
  clear(root);
  if (!t) { root.append(el("p", { class: "why" }, "This file defines a model, not a run: add data, optimizer, seq_len, batch and steps to train it.")); return; }
  const number = (name, value) => el("input", { value, type: "text", onchange: ev => app.edit({ op: "set_setting", name, value: ev.target.value.trim() }) });
  root.append(el("div", { class: "budget" },
    el("span", {}, "steps"), number("steps", t.steps), el("span", {}, "batch"), number("batch", t.batch),
    el("span", {}, "seq_len"), number("seq_len", t.seq_len), el("span", {}, "tokens"), el("b", {}, si(t.tokens))));
  root.append(el("div", {}, el("b", {}, "learning rate "), el("code", {}, t.optimizer), " ",
    el("select", { onchange: ev => app.edit({ op: "set_setting", name: "schedule", value: ev.target.value }) },
      ["constant", "cosine", "linear_decay", "wsd", "power"].map(s => el("option", { selected: s === t.schedule.type }, s)))));
  root.append(lrChart(t, app));
  root.append(el("h4", {}, "data"), el("ul", {}, t.data.map(d => el("li", {}, `${(100 * d.weight).toFixed(0)}%  ${d.name}`))));
  if (t.curriculum.length) root.append(el("h4", {}, "curriculum"), el("ul", {}, t.curriculum.map(p => el("li", {}, `from ${p.at}: ${["seq_len", "batch"].filter(k => p[k]).map(k => `${k} ${p[k]}`).join(", ") || "other data"}`))));
  if (t.evals.length) root.append(el("h4", {}, "evals"), el("ul", {}, t.evals.map(e => el("li", {}, `${e.name} every ${e.every}`))));
  if (t.checkpoint) root.append(el("p", {}, `checkpoints every ${t.checkpoint.every}, keeping ${t.checkpoint.keep}`));
  root.append(el("h4", {}, "settings"), el("table", { class: "runs" }, Object.entries(t.settings).map(([k, v]) => el("tr", {}, el("td", {}, k), el("td", {}, el("code", {}, v))))));
  const runs = el("div", { id: "runs-live" });
  root.append(el("h4", {}, "runs"), el("button", { onclick: async () => { await app.save(); await api.train("start"); refreshRuns(runs); } }, "train"), " ",
    el("button", { onclick: async () => { await api.train("stop"); refreshRuns(runs); } }, "stop after the step"), runs);
  refreshRuns(runs);
}

async function refreshRuns(root) {
  let r;
  try { r = await api.runs(); } catch { return; }
  clear(root);
  root.append(el("p", {}, `state: ${r.state}`));
  root.append(el("table", { class: "runs" }, el("tr", {}, ["run", "state", "step", "loss"].map(h => el("th", {}, h))),
    r.runs.map(x => el("tr", {}, el("td", {}, x.name), el("td", {}, x.state || "-"), el("td", {}, x.step ?? "-"), el("td", {}, x.loss == null ? "-" : x.loss.toFixed(4))))));
  if (r.log) root.append(el("pre", { class: "log" }, r.log));
  if (r.state === "training" && root.isConnected) setTimeout(() => refreshRuns(root), 2000);
}

function lrChart(t, app) {
  const W = 320, H = 150, L = 8, R = 8, T = 10, B = 18, s = t.schedule, steps = Math.max(1, t.steps - 1);
  const x = step => L + (W - L - R) * step / steps, y = v => T + (H - T - B) * (1 - v);
  const chart = svg("svg", { id: "lr-chart", viewBox: `0 0 ${W} ${H}`, preserveAspectRatio: "none" });
  chart.append(svg("path", { class: "curve", d: s.steps.map((st, i) => `${i ? "L" : "M"}${x(st).toFixed(1)},${y(s.scale[i]).toFixed(1)}` ).join(" ") }));
  chart.append(svg("text", { x: L, y: H - 4, "font-size": 10 }, "0"), svg("text", { x: W - R, y: H - 4, "font-size": 10, "text-anchor": "end" }, `${t.steps} steps`),
    svg("text", { x: L, y: T + 2, "font-size": 10 }, `peak ${s.peak}`));
  const handle = (at, what) => {
    if (at == null) return;
    chart.append(svg("line", { class: "mark", x1: x(at), x2: x(at), y1: T, y2: H - B }));
    const grip = svg("line", { class: "handle", x1: x(at), x2: x(at), y1: T, y2: H - B });
    grip.append(svg("title", {}, what === "warmup" ? "drag: the end of the warm-up" : "drag: the start of the decay"));
    grip.addEventListener("pointerdown", down => {
      grip.setPointerCapture(down.pointerId);
      const box = chart.getBoundingClientRect();
      const stepAt = ev => Math.max(0, Math.min(t.steps, Math.round(((ev.clientX - box.left) / box.width * W - L) / (W - L - R) * steps)));
      grip.addEventListener("pointerup", up => {
        const at2 = stepAt(up);
        // one field of the schedule's call; its other settings (final, shape, ...) stay as written
        if (what === "warmup") app.edit({ op: "set_setting_field", name: "schedule", key: "warmup", value: String(at2), kind: s.type });
        else app.edit({ op: "set_setting_field", name: "schedule", key: "decay", value: ((t.steps - at2) / t.steps).toFixed(3), kind: s.type });
      }, { once: true });
    });
    chart.append(grip);
  };
  handle(s.warmup_end, "warmup"); handle(s.decay_start, "decay");
  return chart;
}

// ------------------------------------------------------------------ sweep
export function showSweep(root, app, sweep, runs, run) {
  clear(root);
  if (!sweep || (!sweep.axes.length && !sweep.dimensions.length)) { root.append(el("p", {}, "No sweep: write alternatives with `a | b` (or `name: a | name: b`) to train a run for each.")); return; }
  root.append(el("p", {}, `${sweep.runs} run${sweep.runs === 1 ? "" : "s"}`));
  for (const axis of sweep.axes) {
    const box = el("div", { class: "axis" }, el("b", {}, axis.where));
    for (const place of axis.places) {
      const row = el("div", {});
      place.options.forEach((o, i) => {
        const alt = el("span", { class: "alt", title: "click: pick a run that takes it; double-click: edit" }, (o.label ? o.label + ": " : "") + o.text);
        alt.addEventListener("click", () => {
          const want = o.label || o.text;
          const hit = runs.find(r => r.name.includes(want)) || runs[i];
          if (hit) app.pickRun(hit.index);
        });
        if (o.span) {
          alt.addEventListener("dblclick", () => { const text = prompt("the alternative", o.text); if (text != null && text.trim()) app.edit({ op: "alt_replace", start: o.span[0], end: o.span[1], text: text.trim() }); });
          if (place.options.length > 1) alt.append(el("i", { title: "remove", onclick: ev => { ev.stopPropagation(); app.edit({ op: "alt_remove", start: o.span[0], end: o.span[1] }); } }, "×"));
        }
        row.append(alt);
      });
      const last = place.options[place.options.length - 1];
      if (last && last.span) row.append(el("button", { onclick: () => {
        const text = prompt("a new alternative" + (last.label ? " (label: value)" : ""), last.label ? "name: " + last.text : last.text);
        if (!text) return;
        const m = last.label ? /^\s*([A-Za-z_]\w*)\s*:\s*(.+)$/.exec(text) : null;
        app.edit({ op: "alt_add", last_start: last.span[0], last_end: last.span[1], text: m ? m[2] : text.trim(), label: m ? m[1] : null });
      } }, "+"));
      box.append(row);
    }
    root.append(box);
  }
  if (sweep.dimensions.length) root.append(el("h4", {}, "search dimensions"), el("ul", {}, sweep.dimensions.map(d => el("li", {}, `${d.where}: ${d.space}`))));
  root.append(el("h4", {}, "runs"), el("ul", {}, runs.map(r => el("li", { style: r.index === run ? "font-weight:700" : "cursor:pointer", onclick: () => app.pickRun(r.index) }, r.name))));
}
