import json

from arctic_platform_b200.cli import check_license, flops_estimator


def test_flops_estimator(capsys):
    assert abs(flops_estimator.active_fraction(0.9, 128, 8, None) - (0.1 + 0.9 * 8 / 128)) < 1e-12
    assert flops_estimator.active_fraction(None, None, None, 0.25) == 0.25
    r = flops_estimator.estimate(10, 1e12, 6, 0.25, gpu_tflops=1000, num_gpus=10, mfu=0.5)
    assert r["total_flops"] == 6 * 2.5e9 * 1e12 and abs(r["seconds"] - 1.5e22 / (1e15 * 10 * 0.5)) < 1
    flops_estimator.main(["--params", "4", "--tokens", "1e9", "--json"])
    out = json.loads(capsys.readouterr().out)
    assert out["active_fraction"] == 1.0 and out["total_flops"] == 6 * 4e9 * 1e9
    assert flops_estimator.human(2.5e15) == "2.5P"


def test_check_license(tmp_path):
    a = tmp_path / "a.py"
    a.write_text("#!/usr/bin/env python\nprint(1)\n")
    b = tmp_path / "b.cu"
    b.write_text("// SPDX-License-Identifier: Apache-2.0\nint x;\n")
    assert check_license.missing([tmp_path]) == [a] and check_license.main([str(tmp_path)]) == 1
    assert check_license.main(["--fix", str(tmp_path)]) == 0
    assert a.read_text().splitlines()[:2] == ["#!/usr/bin/env python", "# SPDX-License-Identifier: Apache-2.0"]
    assert check_license.main([str(tmp_path)]) == 0


def test_install_groups_follows_references_to_the_projects_own_groups(tmp_path, capsys):
    from arctic_platform_b200.cli import install_groups
    py = tmp_path / "pyproject.toml"
    py.write_text('[project]\nname = "demo-pkg"\n[project.optional-dependencies]\n'
                  'a = ["x>=1", "demo_pkg[b]"]\nb = ["y", "demo-pkg[a,c]"]\nc = ["z", "other[extra]"]\n')
    groups = install_groups.load_groups(py)
    assert install_groups.resolve(["a"], groups) == ["other[extra]", "x>=1", "y", "z"]     # cycle a <-> b is harmless
    assert install_groups.resolve(["c"], groups) == ["other[extra]", "z"]
    import pytest
    with pytest.raises(ValueError, match="no optional dependency group 'nope'"):
        install_groups.resolve(["nope"], groups)
    assert install_groups.main(["a", "--pyproject", str(py), "--dry-run"]) == 0
    assert "pip install other[extra] x>=1 y z" in capsys.readouterr().out
    # the project's own file parses and its groups resolve
    own = install_groups.load_groups(install_groups.Path(install_groups.__file__).resolve().parents[2] / "pyproject.toml")
    assert "fastapi" in install_groups.resolve(["http"], own)


def test_fetch_assets_reads_sources_and_calls_the_loaders():
    from arctic_platform_b200.cli import fetch_assets
    cfg = {"data": {"sources": ["org/set-a", {"name_or_path": "/data/b", "split": "train[:10]", "kwargs": {"name": "v2"}}]},
           "model": {"name_or_path": "org/model"}}
    calls = []
    assert fetch_assets.fetch_data(cfg, load=lambda **kw: calls.append(kw)) == 2
    assert calls == [{"path": "org/set-a", "split": None}, {"path": "/data/b", "split": "train[:10]", "name": "v2"}]
    got = []
    assert fetch_assets.fetch_model(cfg, got.append, got.append) == "org/model" and got == ["org/model"] * 2
    import pytest
    with pytest.raises(ValueError, match="names no model"):
        fetch_assets.fetch_model({}, got.append, got.append)
    with pytest.raises(ValueError, match="without name_or_path"):
        fetch_assets.data_sources({"data": {"sources": [{"split": "x"}]}})


def test_upgrade_user_code_rewrites_type_attributes(tmp_path):
    from arctic_platform_b200.cli import upgrade_user_code as up
    src = ('"""doc"""\nimport os\n\n\nclass T(Base):\n    name = "t"\n    config_type = MyConfig\n'
           '    data_factory_type = [A, pkg.B]\n    model_factory_type = [Only]\n    other_type = Keep\n')
    new, union = up.upgrade_source(src)
    assert union
    assert "    config: MyConfig\n" in new and "    data_factory: Union[A, pkg.B]\n" in new
    assert "    model_factory: Only\n" in new and "    other_type = Keep\n" in new and "from typing import Union" in new
    assert up.upgrade_source(new)[0] == new                                     # idempotent
    f = tmp_path / "user.py"
    f.write_text(src)
    assert up.main([str(f), "--check"]) == 1 and f.read_text() == src
    assert up.main([str(f)]) == 0 and f.read_text() == new and up.main([str(f), "--check"]) == 0
    compile(new, "user.py", "exec")                                             # still valid Python


def test_release_refuses_untagged_or_dirty_trees():
    from arctic_platform_b200.cli import release

    class R:
        def __init__(self, out):
            self.stdout = out

    def fake(outputs):
        it = iter(outputs)
        return lambda *a, **k: R(next(it))

    assert "uncommitted" in release.check_tree("1.2", fake([" M file.py\n"]))
    assert "not tagged v1.2" in release.check_tree("1.2", fake(["", "v1.1\n"]))
    assert release.check_tree("1.2", fake(["", "v1.1\nv1.2\n"])) == ""
    assert release.release_commands(True)[-1][-3:] == ["twine", "upload", "dist/*"]
    assert release.project_version()
