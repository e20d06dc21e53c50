"""``dss_client`` -- the import name the reference's stand-alone client installs -- resolves to this build's client
package with the SAME module objects, and the helper names a reference program takes from it exist."""
import importlib

import pytest


def test_top_level_names_and_redirected_modules_are_the_same_objects():
    import dss_client
    from dss_client import NeutrinoClient, NeutrinoTrainingEngine, SubJobConfig, wire  # noqa: F401
    import arctic_platform_b200.wire as platform_wire
    import cortex_client.dss_client.engines as engines
    import cortex_client.dss_client.neutrino_client as nc

    assert importlib.import_module("dss_client.neutrino_client") is nc and NeutrinoClient is nc.NeutrinoClient
    assert wire is platform_wire and importlib.import_module("dss_client.wire") is platform_wire
    for path in ("client", "engine"):
        assert importlib.import_module(f"dss_client.{path}") is engines
    for path in ("neutrino_engine", "common"):
        assert importlib.import_module(f"dss_client.{path}") is nc
    from dss_client.client import ArcticInferenceClient, DSSClient, DSSTrainingClient  # noqa: F401
    from dss_client.common import JobType
    from dss_client.engine import ArcticInferenceEngine, DSSTrainingEngine  # noqa: F401
    from dss_client.neutrino_client import build_forward_backward_kwargs, build_forward_backward_payload  # noqa: F401
    assert JobType is nc.JobType and "NeutrinoClient" in dss_client.__all__ and dss_client.__version__
    with pytest.raises(ImportError):
        importlib.import_module("dss_client.no_such_module")
    with pytest.raises(AttributeError):
        nc.no_such_name


def test_source_labels():
    from dss_client.tui.format import source_label

    assert source_label("0f3a:training:2") == "training #2"
    assert source_label({"sub_job_id": "0f3a:sampling:0"}) == "sampling #0"
    assert source_label({"sub_job_id": "0f3a:x:1", "job_type": "log_prob"}) == "log_prob #1"
    assert source_label("plain") == "plain" and source_label({}) == "?"


class _Logs:
    def __init__(self):
        self.calls = []
        self.pages = [{"entries": ["a", "b"], "next_cursor": "c1", "eof": False},
                      {"entries": ["c"], "next_cursor": "c2", "eof": True}]

    def tail_logs(self, job_id, cursor=None, max_lines=None, sub_job_id=None):
        self.calls.append({"job": job_id, "cursor": cursor, "max_lines": max_lines, "sub": sub_job_id})
        return self.pages.pop(0) if self.pages else {"entries": [], "next_cursor": cursor, "eof": True}


def test_cached_log_pages_tails_on_first_open_and_resumes_from_the_cursor(tmp_path):
    from dss_client.tui.log_cache import LogCache, cached_log_pages

    client = _Logs()
    cache = LogCache("job-1", root=tmp_path)
    pages = list(cached_log_pages(cache, client, "job-1", "job-1:training:0", follow=False, tail_lines=50, sleep=lambda s: None))
    assert pages == [["a", "b"], ["c"]]
    assert client.calls[0] == {"job": "job-1", "cursor": None, "max_lines": 50, "sub": "job-1:training:0"}
    assert client.calls[1]["cursor"] == "c1" and client.calls[1]["max_lines"] is None

    # a second open replays the cache, then asks from the saved cursor without a line limit
    again = list(cached_log_pages(cache, client, "job-1", "job-1:training:0", follow=False, sleep=lambda s: None))
    assert again[0] == ["a", "b", "c"]
    assert client.calls[-1]["cursor"] == "c2" and client.calls[-1]["max_lines"] is None
