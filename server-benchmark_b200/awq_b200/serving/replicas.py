"""Replica topology and launch: instance ``i`` of ``g`` GPUs each gets GPUs ``i*g .. i*g+g-1``
(reference utils/generate_compose.py:191-194) and runs vLLM's OpenAI server with the reference's
argument list (utils/generate_compose.py:85-93), one process tree per instance in place of one
container."""
from __future__ import annotations

import os
import signal
import subprocess
import sys
import time
import urllib.request

PACKAGE_PARENT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def replica_gpu_list(instance_id: int, gpus_per_instance: int) -> str:
    """Comma-separated contiguous GPU slice of one instance."""
    start = instance_id * gpus_per_instance
    return ",".join(str(g) for g in range(start, start + gpus_per_instance))


def serve_command(model_dir: str, served_name: str, port: int, tensor_parallel_size: int = 1,
                  pipeline_parallel_size: int = 1, extra_args: str = "") -> list[str]:
    """The reference's server arguments, plus the two an offline random-init run needs:
    ``--dtype half`` (AWQ computes in fp16) and ``--load-format dummy`` (no checkpoint)."""
    cmd = [sys.executable, "-m", "vllm.entrypoints.openai.api_server",
           "--trust-remote-code", "--gpu-memory-utilization=0.9", "--host", "127.0.0.1",
           "--port", str(port), "--tensor-parallel-size", str(tensor_parallel_size),
           "--pipeline-parallel-size", str(pipeline_parallel_size), "--model", model_dir,
           "--served-model-name", served_name, "--dtype", "half", "--load-format", "dummy"]
    return cmd + extra_args.split()


def replica_env(instance_id: int, gpus_per_instance: int, plugin: str = "on",
                dummy_fill: int = 0, options: dict | None = None) -> dict:
    """Environment of one instance.  ``plugin``: "on" (this package's kernels), "fill" (stock
    vLLM kernels, but the same seeded parameter fill, so both columns compute on the same
    weights) or "off" (vLLM untouched)."""
    env = dict(os.environ)
    env["CUDA_VISIBLE_DEVICES"] = replica_gpu_list(instance_id, gpus_per_instance)
    env.update({"HF_HUB_OFFLINE": "1", "TRANSFORMERS_OFFLINE": "1", "VLLM_NO_USAGE_STATS": "1",
                "DO_NOT_TRACK": "1", "TOKENIZERS_PARALLELISM": "false"})
    if plugin in ("on", "fill"):
        env["PYTHONPATH"] = PACKAGE_PARENT + os.pathsep + env.get("PYTHONPATH", "")
        env["AWQ_B200_DUMMY_FILL"] = str(dummy_fill)
        env["AWQ_B200_MODE"] = "kernels" if plugin == "on" else "fill_only"
        for key, val in (options or {}).items():
            env[key] = str(val)
    elif plugin != "off":
        raise ValueError("plugin is 'on', 'fill' or 'off'")
    return env


class Replicas:
    """N server process groups; ``wait_ready`` polls the reference's health check
    (/health and /v1/models, utils/generate_compose.py:94-99)."""

    def __init__(self) -> None:
        self.procs: list[subprocess.Popen] = []
        self.ports: list[int] = []
        self.logs: list[str] = []

    def launch(self, cmd: list[str], env: dict, port: int, log_path: str) -> None:
        log = open(log_path, "w")
        self.procs.append(subprocess.Popen(cmd, env=env, stdout=log, stderr=subprocess.STDOUT,
                                           start_new_session=True))
        self.ports.append(port)
        self.logs.append(log_path)

    def wait_ready(self, timeout_s: float = 1800.0) -> None:
        deadline = time.time() + timeout_s
        pending = set(range(len(self.procs)))
        while pending:
            for i in sorted(pending):
                if self.procs[i].poll() is not None:
                    raise RuntimeError(f"replica {i} exited with {self.procs[i].returncode}; "
                                       f"log: {self.logs[i]}")
                try:
                    base = f"http://127.0.0.1:{self.ports[i]}"
                    urllib.request.urlopen(base + "/health", timeout=5).read()
                    body = urllib.request.urlopen(base + "/v1/models", timeout=5).read()
                    if b"list" in body:
                        pending.discard(i)
                except Exception:
                    pass
            if pending:
                if time.time() > deadline:
                    raise TimeoutError(f"replicas {sorted(pending)} not ready after {timeout_s} s")
                time.sleep(2.0)

    def stop(self) -> None:
        """Ends exactly the process groups started here."""
        for p in self.procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)
                except ProcessLookupError:
                    pass
        deadline = time.time() + 30
        for p in self.procs:
            try:
                p.wait(timeout=max(0.1, deadline - time.time()))
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
        self.procs.clear()
