"""Batch-level record / replay (``RecordReplay``) and the ``load`` spelling of the replay mode."""
import pytest
import torch

from arctic_platform_b200.utils.record_replay import RecordReplay, ReplayMiss, record_replay_generation


def test_batches_are_taped_as_frames_and_replayed(tmp_path, monkeypatch):
    for k in ("REPLAY_GENERATION", "REPLAY_GENERATION_DIR", "REPLAY_GENERATION_MODE", "REPLAY_START_RECORD"):
        monkeypatch.delenv(k, raising=False)
    off = RecordReplay()
    assert not off.is_enabled() and not off.is_record_mode() and off.load_record(1) is None
    off.save_record(1, {"x": 1})                                           # silently nothing
    monkeypatch.setenv("REPLAY_GENERATION", "1")
    monkeypatch.setenv("REPLAY_GENERATION_DIR", str(tmp_path / "tape"))
    rec = RecordReplay()
    assert rec.is_record_mode() and not rec.is_replay_mode() and (tmp_path / "tape").is_dir()
    batch = {"input_ids": torch.arange(6).view(2, 3), "rewards": torch.tensor([0.5, 1.0]), "meta": {"step": 3, "tags": ["a"]}}
    rec.save_record(1, batch)
    rec.save_record(2, {"input_ids": torch.zeros(1, 1, dtype=torch.long)})
    monkeypatch.setenv("REPLAY_GENERATION_MODE", "load")
    monkeypatch.setenv("REPLAY_START_RECORD", "1")
    rep = RecordReplay()
    assert rep.is_replay_mode() and rep.skip_record(1) and not rep.skip_record(2)
    got = rep.load_record(1)
    assert torch.equal(got["input_ids"], batch["input_ids"]) and got["meta"] == batch["meta"]
    assert got["rewards"].dtype == torch.float32
    with pytest.raises(FileNotFoundError):
        rep.load_record(9)
    rep.save_record(5, batch)                                              # load mode never writes
    assert not (tmp_path / "tape" / "generate-5.dssst1").exists()
    monkeypatch.setenv("REPLAY_GENERATION_MODE", "rewind")
    with pytest.raises(ValueError):
        RecordReplay()
    monkeypatch.setenv("REPLAY_GENERATION_MODE", "load")
    monkeypatch.setenv("REPLAY_GENERATION_DIR", str(tmp_path / "absent"))
    with pytest.raises(FileNotFoundError):
        RecordReplay()


def test_generation_decorator_accepts_the_load_spelling(tmp_path, monkeypatch):
    calls = []

    @record_replay_generation
    def generate(prompts):
        calls.append(prompts)
        return [{"token_ids": [len(p)]} for p in prompts]

    monkeypatch.setenv("REPLAY_GENERATION_DIR", str(tmp_path))
    monkeypatch.setenv("REPLAY_GENERATION_MODE", "record")
    assert generate([[1, 2]]) == [{"token_ids": [2]}]
    generate._replay_counter["i"] = 0
    monkeypatch.setenv("REPLAY_GENERATION_MODE", "load")
    assert generate([[9, 9, 9]]) == [{"token_ids": [2]}] and len(calls) == 1      # from the tape, not computed
    with pytest.raises(ReplayMiss):
        generate([[1]])
