"""What a measurement ran on: hardware, driver, libraries and the revision of the code.

``collect()`` returns one dictionary meant to be stored as ``env.json`` beside a result, so that a
number can be traced to the machine and the code that produced it (the purpose of
src/dli/envinfo.py:1-10,202-228).  Every field is best effort: a tool that is missing
(``nvidia-smi`` on a machine without a GPU, ``git`` outside a checkout) gives ``None`` instead of
an error, because a partial record is still a record.  Settings of the GPU are only read.

    python -m dli_b200.envinfo [out.json]        bin/dli env [--out out.json]
"""

from __future__ import annotations

import json
import os
import platform
import shutil
import subprocess
import sys
from datetime import datetime, timezone
from pathlib import Path
from typing import Any

GPU_FIELDS = ("name", "uuid", "memory.total", "compute_cap", "driver_version", "clocks.max.sm", "clocks.max.memory", "power.limit")


def _run(cmd: list[str], timeout: float = 20.0) -> str | None:
    """What ``cmd`` prints, or None if the tool is not there, fails, or takes longer than ``timeout``."""
    tool = shutil.which(cmd[0])
    if tool is None:
        return None
    try:
        done = subprocess.run([tool, *cmd[1:]], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, timeout=timeout)
    except (subprocess.TimeoutExpired, OSError):
        return None
    return done.stdout.strip() if done.returncode == 0 else None


def _proc_field(path: str, key: str) -> str | None:
    """The value behind ``key`` in a /proc file of ``key : value`` lines."""
    try:
        with open(path) as lines:
            for line in lines:
                if line.startswith(key):
                    return line.partition(":")[2].strip()
    except OSError:
        pass
    return None


def gpus() -> list[dict[str, str]] | None:
    out = _run(["nvidia-smi", f"--query-gpu={','.join(GPU_FIELDS)}", "--format=csv,noheader,nounits"])
    if not out:
        return None
    return [dict(zip(GPU_FIELDS, (v.strip() for v in line.split(",")))) for line in out.splitlines() if line.strip()]


def cpu() -> dict[str, Any]:
    total = _proc_field("/proc/meminfo", "MemTotal")  # "<n> kB"
    try:
        mem = round(int(total.split()[0]) / 2**20, 1) if total else None
    except (ValueError, IndexError):
        mem = None
    return {"model": _proc_field("/proc/cpuinfo", "model name"), "logical_cores": os.cpu_count(), "memory_gib": mem}


def torch_info() -> dict[str, Any] | None:
    try:
        import torch
    except Exception:
        return None
    info: dict[str, Any] = {"version": torch.__version__, "cuda": torch.version.cuda, "cuda_available": torch.cuda.is_available()}
    try:
        info["tf32_matmul"] = bool(torch.backends.cuda.matmul.allow_tf32)
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(0)
            info["device0"] = {"name": p.name, "sms": p.multi_processor_count, "memory_gib": round(p.total_memory / 2**30, 1),
                               "capability": f"{p.major}.{p.minor}"}
    except Exception:
        pass
    return info


def nvcc_version() -> str | None:
    out = _run([os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc", "--version"])
    if not out:
        return None
    return next((line.strip() for line in out.splitlines() if "release" in line), out.splitlines()[-1])


def revision(root: Path | None = None) -> str | None:
    """The commit of the checkout the package lives in, with ``+dirty`` if files differ from it."""
    root = root or Path(__file__).resolve().parents[1]
    head = _run(["git", "-C", str(root), "rev-parse", "HEAD"])
    if not head:
        return None
    dirty = _run(["git", "-C", str(root), "status", "--porcelain", "--untracked-files=no"])
    return head + ("+dirty" if dirty else "")


def built_kernels() -> list[str]:
    """The kernel libraries compiled so far (their names carry the hash of their sources)."""
    try:
        from .csrc.build import build_dir

        return sorted(p.name for p in build_dir().glob("dli_*.so"))
    except Exception:
        return []


def collect(revision_override: str | None = None) -> dict[str, Any]:
    from . import __version__

    return {
        "time_utc": datetime.now(timezone.utc).isoformat(timespec="seconds"),
        "package": {"name": "dli_b200", "version": __version__, "revision": revision_override or revision()},
        "python": sys.version.split()[0],
        "platform": platform.platform(),
        "cpu": cpu(),
        "gpus": gpus(),
        "torch": torch_info(),
        "nvcc": nvcc_version(),
        "kernels_built": built_kernels(),
        "argv": sys.argv,
    }


def write(path: str | Path, revision_override: str | None = None) -> dict[str, Any]:
    env = collect(revision_override)
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    Path(path).write_text(json.dumps(env, indent=1) + "\n")
    return env


def main(argv: list[str] | None = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if argv:
        write(argv[0])
    else:
        print(json.dumps(collect(), indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
