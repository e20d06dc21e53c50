"""SFT over HTTP with the server as a child of the client -- the smallest two-process deployment.

    CUDA_VISIBLE_DEVICES= python -m arctic_platform_b200.sft.examples.run_sft_http_demo \
        --launch-local-server --server-cuda-visible-devices 0,1 --training-gpus 2 --model /models/Qwen3-1.7B

The client process needs no GPU (blank ``CUDA_VISIBLE_DEVICES`` for it if you like); the server child gets
``--server-cuda-visible-devices``.  Without ``--launch-local-server`` the demo connects to ``--host:--port``.
Prints the loss per step and, at the end, whether the loss fell.
Counterpart of arctic_platform/sft/examples/run_sft_http_demo.py in the reference.
"""
from __future__ import annotations

import json
import socket
from typing import List, Optional

from . import sft_example


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def main(argv: Optional[List[str]] = None, log=print) -> int:
    ap = sft_example.parser()
    ap.set_defaults(comm_protocol="http", steps=12)
    a = ap.parse_args(argv)
    if a.launch_local_server and a.port == 8765:
        a.port = free_port()                      # a private port: several demos can run on one machine
    a.host = "127.0.0.1" if a.launch_local_server else a.host
    hist = sft_example.run(a, log=log)
    first, last = hist[0]["loss"], hist[-1]["loss"]
    log(json.dumps({"first_loss": first, "last_loss": last, "improved": last < first}))
    return 0 if last < first else 1


if __name__ == "__main__":
    raise SystemExit(main())
