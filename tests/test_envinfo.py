"""The record of what a measurement ran on (no GPU needed: missing tools give None)."""

import json

from dli_b200 import cli, envinfo


def test_collect_is_best_effort_and_serialisable(tmp_path, monkeypatch):
    env = envinfo.collect()
    assert {"time_utc", "package", "python", "platform", "cpu", "gpus", "torch", "nvcc", "kernels_built", "argv"} <= set(env)
    assert env["package"]["name"] == "dli_b200" and env["torch"]["tf32_matmul"] is False
    json.dumps(env)
    monkeypatch.setattr(envinfo.shutil, "which", lambda name: None)  # a machine without nvidia-smi, git or nvcc on PATH
    bare = envinfo.collect(revision_override="abc")
    assert bare["gpus"] is None and bare["package"]["revision"] == "abc"


def test_env_command_writes_the_file(tmp_path):
    out = tmp_path / "results" / "env.json"
    assert cli.main(["env", "--out", str(out)]) == 0
    assert json.loads(out.read_text())["python"]
