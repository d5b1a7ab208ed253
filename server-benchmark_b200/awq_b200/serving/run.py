"""One serving measurement from start to finish, the job of the reference's
benchmarks/3_vllm_benchmark.sh on one box without containers:

  1. write the random-init model directory (model_dir),
  2. start N vLLM servers on contiguous GPU slices (replicas) and, for N > 1, the front,
  3. wait for the health check, run ``vllm bench serve`` with the reference's flags (client),
  4. write ``<results>/<gpu>_x_<count>_<model>_vllm_benchmark.txt`` in the reference's layout and
     print one JSON line with the parsed figures; a result file that exists is not re-run
     (run_remote_benchmark.py:186-195,307-310) unless --force.

    python -m awq_b200.serving.run --arch qwen3-30b-a3b --instances 8 \
        --concurrency 1,16,64,256 --num-prompts 8,64,256,1024 --plugin on
"""
from __future__ import annotations

import argparse
import json
import os
import shlex
import socket
import subprocess
import sys
import tempfile
import time

from . import client, model_dir, replicas


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _wait_for_front(proc, base: str, timeout_s: float = 120.0) -> None:
    """The front answers /front/stats once it listens."""
    import urllib.request
    deadline = time.time() + timeout_s
    while True:
        if proc.poll() is not None:
            raise RuntimeError(f"the front exited with {proc.returncode}")
        try:
            urllib.request.urlopen(base + "/front/stats", timeout=5).read()
            return
        except Exception:
            if time.time() > deadline:
                raise TimeoutError("the front did not come up")
            time.sleep(0.5)


def topology_text(args, ports: list[int], cmds: list[list[str]], envs: list[dict]) -> str:
    """What the compose file says in the reference: one entry per instance with its GPUs, port
    and command, then the front."""
    lines = ["services:"]
    for i, (port, cmd, env) in enumerate(zip(ports, cmds, envs)):
        lines += [f"  vllm_{i}:",
                  f"    device_ids: [{', '.join(repr(g) for g in env['CUDA_VISIBLE_DEVICES'].split(','))}]",
                  f"    port: {port}",
                  f"    plugin: {args.plugin}",
                  f"    command: {' '.join(shlex.quote(c) for c in cmd[3:])}"]
    if len(ports) > 1:
        lines += ["  front:", f"    policy: {args.policy}",
                  "    backends: [" + ", ".join(f"vllm_{i}" for i in range(len(ports))) + "]"]
    return "\n".join(lines)


def _pairs(args) -> list[tuple[int, int]]:
    """(concurrency, prompts) of every client run against one set of servers."""
    conc = [int(c) for c in str(args.concurrency).split(",")]
    prompts = [int(n) for n in str(args.num_prompts).split(",")]
    if len(prompts) == 1:
        prompts = prompts * len(conc)
    if len(prompts) != len(conc):
        raise ValueError("--num-prompts has one value or one per --concurrency value")
    return list(zip(conc, prompts))


def run(args) -> dict:
    served = args.model_name
    gpus = args.instances * args.tensor_parallel_size * args.pipeline_parallel_size
    server_name = f"{args.gpu_name}_x_{gpus}"
    os.makedirs(args.results_dir, exist_ok=True)
    suffix = "" if args.plugin == "on" else f"-stock-{args.plugin}"
    pairs = _pairs(args)

    def out_path(conc: int) -> str:
        tag = args.tag + (f"-c{conc}" if len(pairs) > 1 else "")
        return os.path.join(args.results_dir,
                            client.result_file_name(server_name, served + suffix + tag))

    runs, todo = [], []
    for conc, prompts in pairs:
        path = out_path(conc)
        if os.path.exists(path) and not args.force:
            with open(path) as f:
                runs.append({"result_file": path, "skipped": "result exists",
                             "concurrency": conc, **client.parse_result_block(f.read())})
        else:
            todo.append((conc, prompts))
    summary = {"server": server_name, "model": served, "plugin": args.plugin,
               "instances": args.instances, "runs": runs}
    if not todo:
        return summary

    work = args.work_dir or tempfile.mkdtemp(prefix="awq_b200_serving_")
    mdir = model_dir.write_model_dir(os.path.join(work, "model"), args.arch,
                                     num_layers=args.num_layers)
    group = replicas.Replicas()
    front = None
    t0 = time.time()
    try:
        ports, cmds, envs = [], [], []
        per = args.tensor_parallel_size * args.pipeline_parallel_size
        for i in range(args.instances):
            port = _free_port()
            cmd = replicas.serve_command(mdir, served, port, args.tensor_parallel_size,
                                         args.pipeline_parallel_size, args.extra_args)
            env = replicas.replica_env(i, per, args.plugin, args.seed, {
                "AWQ_B200_REPACK_DECODE": int(args.repack_decode),
                "AWQ_B200_DECODE_KMAJOR": int(args.decode_kmajor)})
            group.launch(cmd, env, port, os.path.join(work, f"vllm_{i}.log"))
            ports.append(port), cmds.append(cmd), envs.append(env)
        group.wait_ready(args.startup_timeout)
        summary["startup_s"] = round(time.time() - t0, 1)
        if args.instances > 1:
            fport = _free_port()
            fcmd = [sys.executable, "-m", "awq_b200.serving.front", "--port", str(fport),
                    "--policy", args.policy]
            for p in ports:
                fcmd += ["--backend", f"http://127.0.0.1:{p}"]
            fenv = dict(os.environ, PYTHONPATH=replicas.PACKAGE_PARENT + os.pathsep +
                        os.environ.get("PYTHONPATH", ""))
            front = subprocess.Popen(fcmd, env=fenv, start_new_session=True)
            base = f"http://127.0.0.1:{fport}"
            _wait_for_front(front, base)
        else:
            base = f"http://127.0.0.1:{ports[0]}"
        benv = dict(os.environ, CUDA_VISIBLE_DEVICES="", HF_HUB_OFFLINE="1",
                    TRANSFORMERS_OFFLINE="1")
        for conc, prompts in todo:
            bcmd = client.benchmark_command(served, base, args.random_input_len,
                                            args.random_output_len, conc, prompts,
                                            tokenizer=mdir)
            t1 = time.time()
            res = subprocess.run(bcmd, env=benv, capture_output=True, text=True,
                                 timeout=args.client_timeout)
            if res.returncode != 0:
                raise RuntimeError("benchmark client failed:\n" +
                                   (res.stdout + res.stderr)[-4000:])
            block = client.legacy_result_block(
                res.stdout, topology_text(args, ports, cmds, envs),
                " ".join(shlex.quote(c) for c in bcmd[3:]))
            path = out_path(conc)
            with open(path, "w") as f:
                f.write(block)
            runs.append({"result_file": path, "concurrency": conc, "num_prompts": prompts,
                         "client_s": round(time.time() - t1, 1),
                         **client.parse_result_block(block)})
        return summary
    except Exception:
        for i, log in enumerate(group.logs):
            try:
                with open(log) as f:
                    tail = f.read()[-6000:]
                sys.stderr.write(f"---- vllm_{i} log tail ----\n{tail}\n")
            except OSError:
                pass
        raise
    finally:
        if front is not None and front.poll() is None:
            front.terminate()
        group.stop()


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--arch", default="qwen3-30b-a3b", choices=sorted(model_dir.ARCHITECTURES))
    ap.add_argument("--model-name", default="synthetic/Qwen3-30B-A3B-AWQ-random")
    ap.add_argument("--num-layers", type=int, default=None)
    ap.add_argument("--instances", type=int, default=1)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--pipeline-parallel-size", type=int, default=1)
    ap.add_argument("--extra-args", default="--max-model-len 8192")
    ap.add_argument("--plugin", default="on", choices=["on", "fill", "off"])
    ap.add_argument("--repack-decode", action="store_true")
    ap.add_argument("--decode-kmajor", action="store_true")
    ap.add_argument("--policy", default="round_robin", choices=["round_robin", "least_conn"])
    ap.add_argument("--concurrency", default="1", help="one value or a comma-separated list")
    ap.add_argument("--num-prompts", default="100", help="one value, or one per concurrency")
    ap.add_argument("--random-input-len", type=int, default=1000)
    ap.add_argument("--random-output-len", type=int, default=1000)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--gpu-name", default="b200")
    ap.add_argument("--results-dir", default="results")
    ap.add_argument("--tag", default="", help="appended to the model part of the file name")
    ap.add_argument("--work-dir", default=None)
    ap.add_argument("--startup-timeout", type=float, default=1800.0)
    ap.add_argument("--client-timeout", type=float, default=3600.0)
    ap.add_argument("--force", action="store_true")
    return ap


def main() -> None:
    print(json.dumps(run(parser().parse_args())), flush=True)


if __name__ == "__main__":
    main()
