"""Read-only terminal viewer for job logs with a client-side cache (no terminal-UI toolkit needed).

``log_cache`` keeps, per job and log source, the entries already fetched and the cursor to resume from; ``format``
turns entries and job records into lines; ``viewer`` ties them to a ``NeutrinoClient`` and a terminal.
Counterpart of cortex-client/dss_client/tui/ (a Textual application there; plain ANSI output here)."""
from .log_cache import LogCache, cache_root, cached_pages, safe_source_name, unsafe_source_name  # noqa: F401
from .viewer import LogViewer  # noqa: F401
