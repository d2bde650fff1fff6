"""`bux studio FILE`: a page in the browser that shows a ``.bux`` file three ways at once (its
source, its model as a diagram, its training and sweep) and edits the file's text from any of
them. `server` serves the page and the JSON API, `view` says what to draw, `edits` turns a
visual edit into a splice of the text, `forms` is the inspector, `palette` what can be
inserted, `training` runs the file from the page; ``static/`` is the page (ES modules, SVG,
CSS: no build step, no network). Reference: ``studio/*.py``."""

from .server import Studio, serve  # noqa: F401
