"""`bux studio FILE`: a local page to edit a `.bux` file and watch what it compiles to.

A stdlib HTTP server with a small JSON API behind a per-session token:

* ``GET  /``                the page (one HTML file, no build step);
* ``GET  /api/view``        the file's source, its diagnostics, runs (name, id, parameters,
                            FLOPs per token), the rendered graph of the first run and the
                            latest metrics of runs found under ``--out``;
* ``POST /api/source``      replace the file's text (checked first; a text with errors is
                            kept in memory and reported, the file on disk stays);
* ``POST /api/set``         a structural edit: set ``name = value`` (appends the setting or
                            rewrites its statement);
* ``POST /api/train``       launch the file's runs in a background process (``bux launch``).

Reference: ``studio/server.py``, ``studio/view.py``, ``studio/edits.py``, ``studio/training.py``.
"""

from .server import Studio, serve  # noqa: F401
