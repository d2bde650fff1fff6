// Small helpers for building DOM and SVG without a framework.
export function el(tag, attrs = {}, ...kids) {
  const node = document.createElement(tag);
  for (const [k, v] of Object.entries(attrs)) {
    if (k === "class") node.className = v;
    else if (k.startsWith("on")) node.addEventListener(k.slice(2), v);
    else if (v === true) node.setAttribute(k, "");
    else if (v !== false && v != null) node.setAttribute(k, v);
  }
  for (const kid of kids.flat()) if (kid != null) node.append(kid);
  return node;
}

const SVG = "http://www.w3.org/2000/svg";
export function svg(tag, attrs = {}, ...kids) {
  const node = document.createElementNS(SVG, tag);
  for (const [k, v] of Object.entries(attrs)) {
    if (k.startsWith("on")) node.addEventListener(k.slice(2), v);
    else if (v != null) node.setAttribute(k, v);
  }
  for (const kid of kids.flat()) if (kid != null) node.append(kid);
  return node;
}

export function clear(node) { while (node.firstChild) node.firstChild.remove(); return node; }

export function si(n) {
  if (n == null) return "?";
  for (const [unit, size] of [["T", 1e12], ["B", 1e9], ["M", 1e6], ["k", 1e3]]) if (n >= size) return (n / size).toFixed(n / size >= 100 ? 0 : 1).replace(/\.0$/, "") + unit;
  return String(n);
}

// Minimal Markdown for hovers and notes: code spans, bold, line breaks. Text is escaped first.
export function markdown(text) {
  const esc = text.replace(/&/g, "&amp;").replace(/</g, "&lt;").replace(/>/g, "&gt;");
  return esc.replace(/```bux\n([\s\S]*?)\n```/g, "<code>$1</code>").replace(/`([^`]+)`/g, "<code>$1</code>")
            .replace(/\*\*([^*]+)\*\*/g, "<b>$1</b>");
}
