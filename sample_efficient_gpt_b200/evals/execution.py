"""Guarded execution of model-written Python (HumanEval / MBPP scoring).

Same contract as evals/execution.py:39-357 of the reference - ``execute_code(code, timeout, maximum_memory_bytes) ->
ExecutionResult(success, stdout, stderr, error, timeout, memory_exceeded)`` - but every program runs in a *fresh
interpreter* (``python -I``) instead of a forked copy of the caller: the evaluating process holds a CUDA context and
forking it is not safe.  The child

  * sets address-space / data / CPU-time limits (``resource``), and a wall-clock alarm;
  * works in a throw-away directory;
  * has the destructive entry points of ``os``, ``shutil``, ``subprocess`` and ``builtins.exit/quit`` replaced by
    ``None`` and reading from stdin disabled;
  * reports its outcome as one JSON line on a dedicated pipe, so anything the program prints stays in ``stdout``.

The parent kills the whole process group when the wall-clock limit (+1 s) passes.  This protects against accidents
(endless loops, runaway allocation, ``rm -rf``), not against an adversary: there is no kernel-level isolation and the
network stays reachable.
"""

from __future__ import annotations

import json
import os
import signal
import subprocess
import sys
import tempfile
from dataclasses import dataclass

_CHILD = r"""
import sys, os, json, io, signal, contextlib, faulthandler
report_fd, timeout, mem = int(sys.argv[1]), float(sys.argv[2]), int(sys.argv[3])
code = sys.stdin.read()
sys.stdin = open(os.devnull)
out = {"success": False, "error": None, "timeout": False, "memory_exceeded": False}
def _limits():
    import resource
    if mem > 0:
        for what in (resource.RLIMIT_AS, resource.RLIMIT_DATA):
            resource.setrlimit(what, (mem, mem))
    cpu = int(timeout) + 2
    resource.setrlimit(resource.RLIMIT_CPU, (cpu, cpu + 1))
def _disarm():
    import builtins, shutil, subprocess
    faulthandler.disable()
    builtins.exit = builtins.quit = None
    os.environ["OMP_NUM_THREADS"] = "1"
    for name in ("kill", "system", "putenv", "remove", "removedirs", "rmdir", "fchdir", "setuid", "fork", "forkpty",
                 "killpg", "rename", "renames", "truncate", "replace", "unlink", "fchmod", "fchown", "chmod", "chown",
                 "chroot", "lchflags", "lchmod", "lchown", "getcwd", "chdir", "execv", "execve", "execl", "spawnl",
                 "spawnv", "popen"):
        if hasattr(os, name):
            setattr(os, name, None)
    shutil.rmtree = shutil.move = shutil.chown = None
    subprocess.Popen = None
    for mod in ("ipdb", "joblib", "resource", "psutil", "tkinter"):
        sys.modules[mod] = None
class _Timeout(BaseException):
    pass
def _alarm(signum, frame):
    raise _Timeout()
report = os.fdopen(report_fd, "w")
try:
    _limits()
    _disarm()
    signal.signal(signal.SIGALRM, _alarm)
    signal.setitimer(signal.ITIMER_REAL, timeout)
    try:
        exec(compile(code, "<candidate>", "exec"), {"__name__": "__main__"})
        out["success"] = True
    finally:
        signal.setitimer(signal.ITIMER_REAL, 0)
except _Timeout:
    out.update(timeout=True, error="Execution timed out")
except MemoryError as e:
    out.update(memory_exceeded=True, error=f"Memory limit exceeded: {e}")
except BaseException as e:
    out.update(error=f"{type(e).__name__}: {e}")
sys.stdout.flush(); sys.stderr.flush()
report.write(json.dumps(out)); report.flush()
os._exit(0)
"""


@dataclass
class ExecutionResult:
    success: bool
    stdout: str
    stderr: str
    error: str | None = None
    timeout: bool = False
    memory_exceeded: bool = False

    def __repr__(self) -> str:
        shown = [f"success={self.success}"]
        shown += [f"{k}=True" for k in ("timeout", "memory_exceeded") if getattr(self, k)]
        shown += [f"{k}={getattr(self, k)!r}" for k in ("error", "stdout", "stderr") if getattr(self, k)]
        return f"ExecutionResult({', '.join(shown)})"


def execute_code(code: str, timeout: float = 5.0, maximum_memory_bytes: int | None = 256 * 1024 * 1024) -> ExecutionResult:
    r, w = os.pipe()
    with tempfile.TemporaryDirectory() as tmp:
        proc = subprocess.Popen(
            [sys.executable, "-I", "-c", _CHILD, str(w), str(timeout), str(maximum_memory_bytes or 0)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, cwd=tmp, pass_fds=(w,),
            start_new_session=True, text=True,
        )
        os.close(w)
        try:
            stdout, stderr = proc.communicate(code, timeout=timeout + 1.0)
        except subprocess.TimeoutExpired:
            try:
                os.killpg(proc.pid, signal.SIGKILL)
            except ProcessLookupError:
                pass
            proc.communicate()
            os.close(r)
            return ExecutionResult(False, "", "", "Execution timed out (process killed)", timeout=True)
    with os.fdopen(r) as f:
        raw = f.read()
    if not raw:
        return ExecutionResult(False, stdout, stderr, "Execution failed (no result returned)", timeout=True)
    o = json.loads(raw)
    return ExecutionResult(o["success"], stdout, stderr, o["error"], o["timeout"], o["memory_exceeded"])
