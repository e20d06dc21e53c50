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
