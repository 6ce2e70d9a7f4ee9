"""What a report says about the machine it was made on, after the reference's record
(src/environment.rs:15-41): hardware, software, the source's revision and whether it had
uncommitted changes, and what else the GPU was doing (clocks, throttle reasons, temperature,
other processes on it), with the time of capture.  A field that cannot be had reads
"unavailable", as in the reference.
"""
from __future__ import annotations

import hashlib
import os
import platform
import subprocess
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _command(args: list, cwd: str | None = None) -> str:
    try:
        out = subprocess.run(args, capture_output=True, text=True, timeout=20, cwd=cwd)
    except (OSError, subprocess.SubprocessError):
        return "unavailable"
    return out.stdout.strip() if out.returncode == 0 else "unavailable"


def _smi(fields: str) -> list:
    raw = _command(["nvidia-smi", "-i", "0", f"--query-gpu={fields}", "--format=csv,noheader,nounits"])
    return [c.strip() for c in raw.split(",")] if raw != "unavailable" else []


def capture() -> dict:
    import torch
    hardware = {"machine": platform.machine(), "cpu_count": os.cpu_count()}
    workload = {}
    if torch.cuda.is_available():
        props = torch.cuda.get_device_properties(0)
        hardware.update(gpu=props.name, sm=f"{props.major}.{props.minor}", sms=props.multi_processor_count,
                        memory_bytes=props.total_memory)
        row = _smi("clocks.sm,clocks.max.sm,clocks.mem,temperature.gpu,power.draw,power.limit,"
                   "clocks_event_reasons.active,utilization.gpu")
        if len(row) == 8:
            workload = {"sm_mhz": row[0], "sm_max_mhz": row[1], "mem_mhz": row[2], "temperature_c": row[3],
                        "power_w": row[4], "power_limit_w": row[5], "clock_event_reasons": row[6], "utilization": row[7]}
        else:
            workload = {"clocks": "unavailable"}
        workload["other_gpu_processes"] = [ln for ln in _command(
            ["nvidia-smi", "--query-compute-apps=pid,used_memory", "--format=csv,noheader"]).splitlines()
            if ln and ln != "unavailable" and not ln.startswith(str(os.getpid()))]
    software = {"python": platform.python_version(), "torch": torch.__version__, "cuda": torch.version.cuda,
                "driver": (_smi("driver_version") or ["unavailable"])[0], "nvcc": _command(["nvcc", "--version"]).splitlines()[-1:],
                "os": platform.platform()}
    from .. import __version__
    software["package_version"] = __version__
    lib = os.path.join(ROOT, "rust-mlx_b200", "csrc", "_build", "librmx_kernels.so")
    if os.path.exists(lib):
        with open(lib, "rb") as fh:
            software["kernels_sha256"] = hashlib.sha256(fh.read()).hexdigest()
    commit = _command(["git", "rev-parse", "HEAD"], cwd=ROOT)
    status = _command(["git", "status", "--porcelain"], cwd=ROOT)
    revision = {"commit": commit, "dirty": None if status == "unavailable" else bool(status)}
    return {"hardware": hardware, "software": software, "revision": revision, "workload": workload,
            "captured_unix_seconds": int(time.time())}
