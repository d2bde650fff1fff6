"""Chat templates: a conversation rendered the way the tokenizer's model reads it, and which of
its characters a run trains on.

A template is Jinja source in the Hugging Face convention (``messages``, ``add_generation_prompt``,
the special tokens by name, ``raise_exception``, ``strftime_now``), rendered in a sandbox with the
whitespace rules transformers uses. It comes from a folder (its ``chat_template.jinja``, else the
``chat_template`` of its ``tokenizer_config.json``, which also names ``bos_token`` / ``eos_token``),
from a ``.jinja`` file, from a built-in name (``chatml``) or inline.

`ChatTemplate.pieces` cuts a rendered conversation into (text, role, trained) runs by rendering
its prefixes: what message i adds is the render of the first i + 1 messages minus the render of
the first i, so templates that look at a message's index (a system prompt injected once, a
beginning-of-text token) come out as the model sees them. Of an assistant's piece the reply's
header (what ``add_generation_prompt`` writes) is not trained on, the reply and its end token are.
Reference: ``data/templates.py`` (its `load`, `ChatTemplate.render`).
"""

from __future__ import annotations

import datetime
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

CHATML = ("{% for m in messages %}<|im_start|>{{ m.role }}\n{{ m.content }}<|im_end|>\n{% endfor %}"
          "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}")
BUILT_IN = {"chatml": CHATML}
NAMED = ("bos_token", "eos_token", "unk_token", "sep_token", "pad_token", "cls_token", "mask_token")


def _environment():
    import jinja2
    from jinja2.sandbox import ImmutableSandboxedEnvironment

    def raise_exception(message: str):
        raise jinja2.exceptions.TemplateError(message)

    def strftime_now(fmt: str) -> str:
        return datetime.datetime.now().strftime(fmt)

    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True,
                                        extensions=["jinja2.ext.loopcontrols"])
    env.globals.update(raise_exception=raise_exception, strftime_now=strftime_now)
    env.filters["tojson"] = lambda value, **kw: json.dumps(value, ensure_ascii=False, **{k: v for k, v in kw.items() if k == "indent"})
    return env


@dataclass
class ChatTemplate:
    source: str
    tokens: dict = field(default_factory=dict)    # bos_token, eos_token, ... by name
    _compiled: object = None

    def _template(self):
        if self._compiled is None:
            self._compiled = _environment().from_string(self.source)
        return self._compiled

    def render(self, messages: list, prompt: bool = False) -> str:
        """The conversation as text; with `prompt`, followed by the header of the reply to come."""
        return self._template().render(messages=messages, add_generation_prompt=prompt, **self.tokens)

    def pieces(self, messages: list) -> list:
        """[(text, role, trained_from)] in order: `text` is what the message adds to the render,
        `trained_from` the offset in it where an assistant's own words start (after its header)."""
        out, before = [], ""
        for i, m in enumerate(messages):
            now = self.render(messages[: i + 1])
            if now.startswith(before):
                piece = now[len(before):]
            else:   # a template that rewrites what came before: the message alone
                piece, now = self.render([m]), before + self.render([m])
            start = 0
            if m.get("role") == "assistant":
                try:
                    header = self.render(messages[:i], prompt=True)[len(before):] if i else self.render([], prompt=True)
                except Exception:   # noqa: BLE001 - a template that refuses an empty or odd prefix
                    header = ""
                if header and piece.startswith(header):
                    start = len(header)
            out.append((piece, m.get("role", ""), start))
            before = now
        return out


def load(spec: Optional[str]) -> ChatTemplate:
    """`spec`: None or a built-in name, a folder of a tokenizer, a ``.jinja`` file, or Jinja source."""
    if spec is None:
        return ChatTemplate(CHATML)
    if spec in BUILT_IN:
        return ChatTemplate(BUILT_IN[spec])
    path = Path(spec)
    if "{" not in spec and path.is_dir():
        tokens, source = {}, None
        cfg = path / "tokenizer_config.json"
        if cfg.exists():
            data = json.loads(cfg.read_text())
            for name in NAMED:
                value = data.get(name)
                if isinstance(value, dict):
                    value = value.get("content")
                if isinstance(value, str):
                    tokens[name] = value
            source = data.get("chat_template")
            if isinstance(source, list):   # several named templates: the default one
                source = next((t.get("template") for t in source if t.get("name") == "default"), None)
        jinja_file = path / "chat_template.jinja"
        if jinja_file.exists():
            source = jinja_file.read_text()
        if not source:
            raise ValueError(f"{spec}: no chat_template.jinja and no chat_template in tokenizer_config.json")
        return ChatTemplate(source, tokens)
    if "{" not in spec and path.is_file():
        return ChatTemplate(path.read_text())
    if "{" not in spec:
        raise ValueError(f"chat(template={spec!r}): not a built-in template ({', '.join(BUILT_IN)}), a folder, a file or Jinja source")
    return ChatTemplate(spec)
