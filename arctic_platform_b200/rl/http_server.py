"""``python -m arctic_platform_b200.rl.http_server --host 0.0.0.0 --port 7000`` -- the module path the HTTP client
launches for a local server (arctic_platform/rl/http_server.py in the reference).  The application lives in
:mod:`arctic_platform_b200.common.http_server`."""
from ..common.http_server import create_app, main  # noqa: F401

if __name__ == "__main__":
    main()
