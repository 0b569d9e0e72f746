"""The kernel build helper's host side (no GPU, nothing is compiled)."""

import threading

from dli_b200.csrc import build


def test_build_dir_is_one_place_whoever_asks(monkeypatch, tmp_path):
    """Threads that ask at the same time all get the folder beside the sources (a probe file named
    after the process alone once sent some of them to the fallback under the temporary folder)."""
    monkeypatch.setattr(build, "_build_dir", None)
    monkeypatch.setenv("DLI_B200_BUILD_DIR", str(tmp_path / "libs"))
    got = []
    barrier = threading.Barrier(16)

    def ask():
        barrier.wait()
        got.append(build.build_dir())

    threads = [threading.Thread(target=ask) for _ in range(16)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert set(got) == {tmp_path / "libs"} and not list((tmp_path / "libs").iterdir())


def test_library_names_carry_source_defines_and_hash(monkeypatch, tmp_path):
    monkeypatch.setattr(build, "_build_dir", tmp_path)
    a = build.library_path("attention_mma.cu", {"HEAD_DIM": 64})
    b = build.library_path("attention_mma.cu", {"HEAD_DIM": 80})
    assert a.parent == tmp_path and a.name.startswith("dli_attention_mma_head_dim64_") and a.name != b.name
    assert build.library_path("attention_mma.cu", {"HEAD_DIM": 64}) == a  # stable for the same sources
