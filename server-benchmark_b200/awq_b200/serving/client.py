"""The client side of the reference's measurement: the ``vllm bench serve`` command line with the
reference's flags (benchmarks/3_vllm_benchmark.sh:151-162), the result file in the layout the
reference writes (result block, topology, command: :177-187) and a parser with the labels the
reference's report reads (generate_benchmark_report.py:58-85)."""
from __future__ import annotations

import re
import sys

RESULT_HEADER = "============ Serving Benchmark Result ============"

# label -> key, the five the reference's report extracts
LEGACY_LABELS = {
    "Total Token throughput (tok/s):": "total_token_throughput",
    "Request throughput (req/s):": "request_throughput",
    "Output token throughput (tok/s):": "output_throughput",
    "Mean TTFT (ms):": "mean_ttft_ms",
    "Mean TPOT (ms):": "mean_tpot_ms",
}


def benchmark_command(model_name: str, base_url: str, random_input_len: int = 1000,
                      random_output_len: int = 1000, max_concurrency: int = 1,
                      num_prompts: int = 100, tokenizer: str | None = None) -> list[str]:
    cmd = [sys.executable, "-m", "vllm.entrypoints.cli.main", "bench", "serve",
           "--model", model_name, "--dataset-name", "random",
           "--random-input-len", str(random_input_len),
           "--random-output-len", str(random_output_len),
           "--max-concurrency", str(max_concurrency), "--num-prompts", str(num_prompts),
           "--ignore-eos", "--backend", "openai-chat", "--endpoint", "/v1/chat/completions",
           "--percentile-metrics", "ttft,tpot,itl,e2el", "--base-url", base_url]
    if tokenizer is not None:   # the served name is not a path: say where the tokenizer is
        cmd += ["--tokenizer", tokenizer]
    return cmd


def legacy_result_block(client_output: str, topology: str, command: str) -> str:
    """From the client's console output to the reference's result file: everything from the
    result header on, with the total-throughput label in the spelling the reference's report
    expects (newer vLLM prints it with a lower-case t), then the topology and the command."""
    at = client_output.find(RESULT_HEADER)
    if at < 0:
        raise ValueError("the client output holds no result block")
    block = client_output[at:].rstrip("\n")
    block = re.sub(r"Total token throughput \(tok/s\):", "Total Token throughput (tok/s):", block)
    return (block + "\n\n============ Docker Compose Configuration ============\n" +
            topology.rstrip("\n") + "\n\n============ Benchmark Command ============\n" +
            command + "\n==================================================\n")


def parse_result_block(text: str) -> dict:
    """The five figures of the reference's report, by its labels; {} when the total-throughput
    line is missing (the reference then drops the file)."""
    out = {}
    for label, key in LEGACY_LABELS.items():
        m = re.search(re.escape(label) + r"\s+([\d.]+)", text)
        if m:
            out[key] = float(m.group(1))
    return out if "total_token_throughput" in out else {}


def result_file_name(server_name: str, model_name: str) -> str:
    """``<server>_<model with / as _>_vllm_benchmark.txt`` (run_remote_benchmark.py:186-195);
    the report wants the server part as ``<gpu>_x_<count>``
    (generate_benchmark_report.py:158)."""
    if not re.fullmatch(r"[^_]+_x_\d+", server_name):
        raise ValueError("server name must look like b200_x_8")
    return f"{server_name}_{model_name.replace('/', '_')}_vllm_benchmark.txt"
