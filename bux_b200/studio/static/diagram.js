// The model as a diagram: tokens enter at the bottom, logits leave at the top. Every node of
// the view's tree is laid out as a box of (w, h); a sequence stacks its items upward, `[f]`
// is a ⊕ above `f` with its skip wire beside it, sums and products are columns merged in ⊕ / ⊗,
// a repeat is a dashed container marked ×n, a named block a container captioned with its name.
import { svg, clear } from "./dom.js";

const PAD = 10, GAP = 14, BOX_W = 190, SKIP = 18;
const FILL = { gqa: "var(--attn)", mla: "var(--attn)", csa: "var(--attn)", mlp: "var(--ffn)", gated_mlp: "var(--ffn)", moe: "var(--ffn)",
  rmsnorm: "var(--norm)", layernorm: "var(--norm)", dyt: "var(--norm)", embed: "var(--ends)", head: "var(--ends)", nextn: "var(--ends)" };
const RECURRENT = new Set(["deltanet", "gdn", "gdn2", "kda", "gla", "lightning", "rwkv7", "mamba", "mamba2", "conv", "short_conv"]);

function size(n) {
  // returns {w, h} and stores the layout on the node as n._
  let w, h;
  if (n.kind === "layer") { w = BOX_W; h = 30 + (n.chips.length ? 14 : 0) + (n.name ? 12 : 0); }
  else if (n.kind === "seq") {
    const kids = n.items.map(size);
    w = Math.max(60, ...kids.map(k => k.w)); h = kids.reduce((a, k) => a + k.h, 0) + GAP * Math.max(0, kids.length - 1);
    if (n.name) { w += 2 * PAD; h += 2 * PAD + 12; }
  } else if (n.kind === "residual") { const b = size(n.body); w = b.w + SKIP + PAD; h = b.h + GAP + 18; }
  else if (n.kind === "sum" || n.kind === "prod") {
    const kids = (n.terms || n.factors).map(size);
    w = kids.reduce((a, k) => a + k.w, 0) + GAP * (kids.length - 1); h = Math.max(...kids.map(k => k.h)) + 2 * GAP + 18;
  } else if (n.kind === "repeat") { const b = size(n.body); w = b.w + 2 * PAD; h = b.h + 2 * PAD + 12; }
  else if (n.kind === "neg") { const b = size(n.body); w = b.w; h = b.h + GAP + 16; }
  else { w = 70; h = 22; }                       // tap, ref, const, identity
  n._ = { w, h };
  return n._;
}

function wire(x1, y1, x2, y2) { return svg("path", { class: "wire", d: `M${x1},${y1} L${x2},${y2}` }); }

function circle(x, y, mark) {
  return svg("g", {}, svg("circle", { cx: x, cy: y, r: 8, fill: "white", stroke: "#6b7280" }),
    svg("text", { x, y: y + 4, "text-anchor": "middle" }, mark));
}

// draw node `n` with its bottom-centre at (cx, bottom); the stream enters there and leaves at the top centre
function draw(n, cx, bottom, ui) {
  const { w, h } = n._;
  const g = svg("g", { class: "node", "data-id": n.id });
  g.addEventListener("click", ev => { ev.stopPropagation(); ui.pick(n, g); });
  g.addEventListener("dblclick", ev => {
    if (n.kind === "repeat") { ev.stopPropagation(); ui.repeat(n); }
    else if (n.inside && ui.open) { ev.stopPropagation(); ui.open(n); }     // what the layer is made of
  });
  const top = bottom - h, left = cx - w / 2;
  if (n.kind === "layer") {
    g.append(svg("rect", { class: "box", x: left, y: top, width: w, height: h, fill: FILL[n.type] || (RECURRENT.has(n.type) ? "var(--rec)" : "white") }));
    g.append(svg("text", { class: "title", x: cx, y: top + 18, "text-anchor": "middle" }, n.title + (n.opens ? " ▸" : "")));
    let y = top + 31;
    if (n.chips.length) { g.append(svg("text", { class: "chip", x: cx, y, "text-anchor": "middle" }, n.chips.join(" · "))); y += 13; }
    if (n.name) g.append(svg("text", { class: "chip", x: cx, y, "text-anchor": "middle" }, n.name));
    for (const p of n.ports) g.append(svg("text", { class: "chip", x: left + w + 4, y: top + 14 }, `${p.name}${p.mode === "write" ? "→@" : "←$"}${p.tap}`));
  } else if (n.kind === "seq") {
    let inner = bottom, innerCx = cx;
    if (n.name) {
      g.append(svg("rect", { class: "frame", x: left, y: top, width: w, height: h }));
      g.append(svg("text", { class: "chip", x: left + 8, y: top + 13 }, n.name));
      inner = bottom - PAD;
    }
    let y = inner;
    n.items.forEach((k, i) => {
      g.append(draw(k, innerCx, y, ui));
      y -= k._.h;
      if (i < n.items.length - 1) { g.append(wire(innerCx, y, innerCx, y - GAP)); y -= GAP; }
    });
  } else if (n.kind === "residual") {
    const bx = cx + (SKIP + PAD) / 2 - PAD / 2;
    g.append(draw(n.body, bx, bottom - GAP / 2, ui));
    const join = top + 9, skipX = left + 6;
    g.append(svg("path", { class: "wire", d: `M${bx},${bottom} L${bx},${bottom - GAP / 2}` }));
    g.append(svg("path", { class: "wire", d: `M${bx},${bottom} L${skipX},${bottom} L${skipX},${join} L${bx - 8},${join}` }));
    g.append(wire(bx, bottom - GAP / 2 - n.body._.h, bx, join + 8));
    g.append(circle(bx, join, "+"));
    n._.out = bx;
  } else if (n.kind === "sum" || n.kind === "prod") {
    const kids = n.terms || n.factors, join = top + 9;
    let x = left;
    g.append(circle(cx, join, n.kind === "sum" ? "+" : "×"));
    for (const k of kids) {
      const kx = x + k._.w / 2, kb = bottom - GAP;
      g.append(draw(k, kx, kb, ui));
      g.append(svg("path", { class: "wire", d: `M${cx},${bottom} L${kx},${bottom} L${kx},${kb}` }));
      g.append(svg("path", { class: "wire", d: `M${kx},${kb - k._.h} L${kx},${join} L${cx + (kx < cx ? -8 : 8)},${join}` }));
      x += k._.w + GAP;
    }
  } else if (n.kind === "repeat") {
    g.append(svg("rect", { class: "frame", x: left, y: top, width: w, height: h }));
    g.append(svg("text", { class: "title", x: left + w - 8, y: top + 14, "text-anchor": "end" }, `×${n.times}`));
    g.append(draw(n.body, cx, bottom - PAD, ui));
  } else if (n.kind === "neg") {
    g.append(draw(n.body, cx, bottom, ui));
    g.append(circle(cx, top + 8, "−"));
  } else {
    const label = n.kind === "tap" ? `@${n.tap}` : n.kind === "ref" ? `$${n.tap}${n.pop ? "!" : ""}` : n.kind === "const" ? String(n.value) : "·";
    g.append(svg("rect", { class: "box", x: left, y: top, width: w, height: h, fill: "white", "stroke-dasharray": "2 2" }));
    g.append(svg("text", { x: cx, y: top + 15, "text-anchor": "middle" }, label));
  }
  return g;
}

export function drawModel(root, tree, ui) {
  clear(root);
  if (!tree) return;
  const { w, h } = size(tree);
  const W = w + 80, H = h + 70;
  root.setAttribute("width", W); root.setAttribute("height", H); root.setAttribute("viewBox", `0 0 ${W} ${H}`);
  const cx = W / 2, bottom = H - 30;
  root.append(svg("text", { class: "chip", x: cx, y: H - 8, "text-anchor": "middle" }, "tokens"));
  root.append(wire(cx, H - 20, cx, bottom));
  root.append(draw(tree, cx, bottom, ui));
  root.append(wire(cx, bottom - h, cx, 22));
  root.append(svg("text", { class: "chip", x: cx, y: 14, "text-anchor": "middle" }, "logits"));
  root.onclick = () => ui.pick(null, null);
}

// every node of the tree, depth first
export function* nodes(n) {
  if (!n) return;
  yield n;
  for (const k of n.items || n.terms || n.factors || []) yield* nodes(k);
  if (n.body) yield* nodes(n.body);
}

// the smallest node whose span holds the offset
export function nodeAt(tree, offset) {
  let best = null;
  for (const n of nodes(tree)) {
    if (n.span && n.span[0] <= offset && offset <= n.span[1]) {
      if (!best || n.span[1] - n.span[0] <= best.span[1] - best.span[0]) best = n;
    }
  }
  return best;
}
