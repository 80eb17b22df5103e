"""Runs a rank script under ``torch.distributed.run`` with the gloo backend on CPU.

Rank scripts print ``RESULT key value`` marker lines; the parent parses them.
Every rank arms ``faulthandler.dump_traceback_later`` so that a deadlock shows
up as stack dumps instead of a silent timeout.
"""
from __future__ import annotations

import os
import re
import socket
import subprocess
import sys
from pathlib import Path
from typing import Dict, List

ROOT = Path(__file__).resolve().parents[2]


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def torchrun_gloo(script: str, nproc: int = 2, args: List[str] = (), timeout: int = 240, env: Dict[str, str] = None):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), str(script), *args]
    e = dict(os.environ)
    e.update({"CUDA_VISIBLE_DEVICES": "", "PYTHONPATH": f"{ROOT}:{e.get('PYTHONPATH', '')}", "OMP_NUM_THREADS": "2",
              "SCAFFOLD_TEST_FAULT_TIMEOUT": str(timeout - 20)})
    e.update(env or {})
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e, cwd=str(ROOT))
    return proc


def results(stdout: str) -> Dict[str, List[str]]:
    out: Dict[str, List[str]] = {}
    for m in re.finditer(r"^RESULT (\S+) (.*)$", stdout, flags=re.M):
        out.setdefault(m.group(1), []).append(m.group(2).strip())
    return out
