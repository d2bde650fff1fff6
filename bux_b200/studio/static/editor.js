// The source panel: a textarea over a mirror that underlines errors and highlights the selected
// node's text; completion after ( , . = @ $ " or on Ctrl-Space; hover after the pointer rests.
import { api } from "./api.js";
import { el, clear, markdown } from "./dom.js";

export class Editor {
  constructor(onChange, onCursor) {
    this.area = document.getElementById("source");
    this.marks = document.getElementById("marks");
    this.list = document.getElementById("completions");
    this.tip = document.getElementById("hover");
    this.errors = []; this.selected = null; this.items = []; this.at = 0;
    this.area.addEventListener("input", () => { this.paint(); onChange(this.area.value, "typing"); this.maybeComplete(); });
    this.area.addEventListener("scroll", () => { this.marks.scrollTop = this.area.scrollTop; this.marks.scrollLeft = this.area.scrollLeft; });
    this.area.addEventListener("keyup", ev => { if (!ev.key.startsWith("Arrow") || this.list.hidden) onCursor(this.area.selectionStart); });
    this.area.addEventListener("click", () => { this.hideList(); onCursor(this.area.selectionStart); });
    this.area.addEventListener("keydown", ev => this.keys(ev));
    this.area.addEventListener("mousemove", ev => this.restHover(ev));
    this.area.addEventListener("mouseleave", () => { clearTimeout(this.rest); this.tip.hidden = true; });
  }

  get text() { return this.area.value; }

  // the width of a character and the height of a line in the editor's own font, measured once
  get cell() {
    if (!this._cell) {
      const probe = el("span", { style: "position:absolute;visibility:hidden;white-space:pre" }, "x".repeat(50));
      this.marks.append(probe);
      const box = probe.getBoundingClientRect();
      const line = parseFloat(getComputedStyle(this.marks).lineHeight) || box.height;
      this._cell = { w: box.width / 50 || 7.5, h: line || 18.75 };
      probe.remove();
    }
    return this._cell;
  }

  set(text, keepCursor = true) {
    const at = this.area.selectionStart;
    this.area.value = text;
    if (keepCursor) this.area.setSelectionRange(Math.min(at, text.length), Math.min(at, text.length));
    this.paint();
  }

  show(errors) { this.errors = errors; this.paint(); }

  select(span) {
    this.selected = span; this.paint();
    if (span) {                                  // bring the text into view without moving the caret
      const line = this.text.slice(0, span[0]).split("\n").length;
      const y = (line - 3) * this.cell.h;
      if (y < this.area.scrollTop || y > this.area.scrollTop + this.area.clientHeight - 60) this.area.scrollTop = Math.max(0, y);
    }
  }

  paint() {
    // the mirror holds the same text, cut at the marks' borders
    const cuts = [];
    for (const e of this.errors) cuts.push([e.start, Math.max(e.end, e.start + 1), "bad"]);
    if (this.selected) cuts.push([this.selected[0], this.selected[1], "sel"]);
    cuts.sort((a, b) => a[0] - b[0]);
    clear(this.marks);
    let at = 0;
    const text = this.text;
    for (const [s, e, cls] of cuts) {
      if (s < at) continue;
      this.marks.append(text.slice(at, s), el("span", { class: cls }, text.slice(s, e)));
      at = e;
    }
    this.marks.append(text.slice(at) + "\n");
    this.marks.scrollTop = this.area.scrollTop;
  }

  // -- completion
  async maybeComplete(force = false) {
    const at = this.area.selectionStart, before = this.text.slice(0, at);
    const word = /[A-Za-z_][A-Za-z0-9_]*$/.exec(before);
    const trigger = /[(,.=@$"]\s*$/.test(before);
    if (!force && !trigger && !(word && word[0].length >= 2)) return this.hideList();
    let items;
    try { items = await api.complete(this.text, at); } catch { return this.hideList(); }
    if (at !== this.area.selectionStart || !items.length) return this.hideList();
    this.items = items.slice(0, 60); this.at = 0; this.prefix = word ? word[0].length : 0;
    clear(this.list);
    this.items.forEach((it, i) => this.list.append(el("li", { class: i === 0 ? "on" : "", title: it.doc, onmousedown: ev => { ev.preventDefault(); this.accept(i); } },
      el("span", {}, it.label), el("small", {}, it.detail || it.kind))));
    const lines = before.split("\n");
    this.list.style.left = Math.min(this.area.clientWidth - 220, 12 + this.cell.w * lines[lines.length - 1].length - this.area.scrollLeft) + "px";
    this.list.style.top = 10 + this.cell.h * lines.length - this.area.scrollTop + "px";
    this.list.hidden = false;
  }

  hideList() { this.list.hidden = true; }

  accept(i) {
    const it = this.items[i], at = this.area.selectionStart;
    this.area.setRangeText(it.insert, at - this.prefix, at, "end");
    this.hideList();
    this.area.dispatchEvent(new Event("input"));
  }

  keys(ev) {
    if ((ev.ctrlKey || ev.metaKey) && ev.key === " ") { ev.preventDefault(); return this.maybeComplete(true); }
    if (this.list.hidden) return;
    if (ev.key === "ArrowDown" || ev.key === "ArrowUp") {
      ev.preventDefault();
      this.list.children[this.at].classList.remove("on");
      this.at = (this.at + (ev.key === "ArrowDown" ? 1 : this.items.length - 1)) % this.items.length;
      this.list.children[this.at].classList.add("on");
      this.list.children[this.at].scrollIntoView({ block: "nearest" });
    } else if (ev.key === "Enter" || ev.key === "Tab") { ev.preventDefault(); this.accept(this.at); }
    else if (ev.key === "Escape") this.hideList();
  }

  // -- hover
  restHover(ev) {
    clearTimeout(this.rest);
    this.tip.hidden = true;
    this.rest = setTimeout(async () => {
      const box = this.area.getBoundingClientRect();
      const line = Math.floor((ev.clientY - box.top - 10 + this.area.scrollTop) / this.cell.h);
      const col = Math.round((ev.clientX - box.left - 12 + this.area.scrollLeft) / this.cell.w);
      const lines = this.text.split("\n");
      if (line < 0 || line >= lines.length || col > lines[line].length) return;
      const offset = lines.slice(0, line).reduce((a, l) => a + l.length + 1, 0) + Math.max(0, col);
      let h;
      try { h = await api.hover(this.text, offset); } catch { return; }
      if (!h) return;
      this.tip.innerHTML = markdown(h.text);
      this.tip.style.left = Math.min(ev.clientX - box.left, box.width - 300) + "px";
      this.tip.style.top = ev.clientY - box.top + 16 + "px";
      this.tip.hidden = false;
    }, 500);
  }
}
