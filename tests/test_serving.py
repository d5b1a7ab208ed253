"""Host side of the serving measurement, on the CPU: model directory + tokenizer, replica
topology and command line, the load-balancing front (with real sockets on 127.0.0.1), the client
command and the legacy result block read back with the reference report's own patterns."""
import asyncio
import json
import re
import socket

import numpy as np
import pytest

from awq_b200 import serving
from awq_b200.serving import client, front, model_dir, replicas, run

# the patterns of the reference's report generator (generate_benchmark_report.py:58-85,158)
REFERENCE_PATTERNS = {
    "total": r"Total Token throughput \(tok/s\):\s+([\d.]+)",
    "request": r"Request throughput \(req/s\):\s+([\d.]+)",
    "output": r"Output token throughput \(tok/s\):\s+([\d.]+)",
    "ttft": r"Mean TTFT \(ms\):\s+([\d.]+)",
    "tpot": r"Mean TPOT \(ms\):\s+([\d.]+)",
}
REFERENCE_FILENAME = r"([^_]+_x_\d+)_(.+)"

# what a current `vllm bench serve` prints (labels only; note the lower-case "token")
CLIENT_OUTPUT = """INFO starting
Traffic request rate: inf
============ Serving Benchmark Result ============
Successful requests:                     64
Maximum request concurrency:             16
Benchmark duration (s):                  31.25
Total input tokens:                      64000
Total generated tokens:                  64000
Request throughput (req/s):              2.05
Output token throughput (tok/s):         2048.00
Peak output token throughput (tok/s):    2300.00
Total token throughput (tok/s):          4096.00
---------------Time to First Token----------------
Mean TTFT (ms):                          120.50
Median TTFT (ms):                        110.00
P99 TTFT (ms):                           300.00
-----Time per Output Token (excl. 1st token)------
Mean TPOT (ms):                          7.25
Median TPOT (ms):                        7.20
P99 TPOT (ms):                           8.00
==================================================
"""


def test_model_dir_tokenizer_round_trips_and_config_loads(tmp_path):
    from transformers import AutoConfig, AutoTokenizer
    path = model_dir.write_model_dir(str(tmp_path / "m"), "qwen3-30b-a3b")
    cfg = AutoConfig.from_pretrained(path)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_experts, cfg.num_experts_per_tok,
            cfg.moe_intermediate_size, cfg.vocab_size) == (48, 2048, 128, 8, 768, 151936)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (32, 4, 128)
    assert cfg.quantization_config["quant_method"] == "awq"
    assert cfg.quantization_config["group_size"] == 128
    tok = AutoTokenizer.from_pretrained(path)
    assert tok.vocab_size == 151936
    ids = np.random.default_rng(0).integers(0, tok.vocab_size, 1000).tolist()
    text = tok.decode(ids)
    assert tok.encode(text, add_special_tokens=False) == ids      # length-preserving, exact
    chat = tok.apply_chat_template([{"role": "user", "content": text}], tokenize=True)
    chat = chat["input_ids"] if isinstance(chat, dict) or hasattr(chat, "keys") else chat
    assert len(chat) == 1000


def test_model_dir_dense_variants(tmp_path):
    path = model_dir.write_model_dir(str(tmp_path / "d"), "qwen2.5-72b-tp", num_layers=2)
    cfg = json.load(open(path + "/config.json"))
    assert cfg["intermediate_size"] == 29696 and cfg["num_hidden_layers"] == 2
    for tp in (2, 4, 8):
        assert (cfg["intermediate_size"] // tp) % 128 == 0        # whole groups on every rank
    assert model_dir.ARCHITECTURES["qwen2.5-72b"]["intermediate_size"] == 29568
    with pytest.raises(ValueError):
        model_dir.write_model_dir(str(tmp_path / "x"), "nope")


def test_replica_slices_and_command():
    assert [replicas.replica_gpu_list(i, 1) for i in range(8)] == [str(i) for i in range(8)]
    assert [replicas.replica_gpu_list(i, 2) for i in range(4)] == ["0,1", "2,3", "4,5", "6,7"]
    assert replicas.replica_gpu_list(1, 4) == "4,5,6,7"
    cmd = replicas.serve_command("/m", "org/name", 8000, 2, 1, "--max-model-len 8192")
    joined = " ".join(cmd)
    for piece in ("--trust-remote-code", "--gpu-memory-utilization=0.9", "--port 8000",
                  "--tensor-parallel-size 2", "--pipeline-parallel-size 1", "--model /m",
                  "--served-model-name org/name", "--max-model-len 8192", "--dtype half",
                  "--load-format dummy"):
        assert piece in joined
    assert "--quantization" not in joined          # the reference passes none
    env = replicas.replica_env(3, 2, "on", dummy_fill=5)
    assert env["CUDA_VISIBLE_DEVICES"] == "6,7" and env["AWQ_B200_DUMMY_FILL"] == "5"
    assert env["AWQ_B200_MODE"] == "kernels" and replicas.PACKAGE_PARENT in env["PYTHONPATH"]
    assert replicas.replica_env(0, 1, "fill")["AWQ_B200_MODE"] == "fill_only"
    assert "AWQ_B200_MODE" not in replicas.replica_env(0, 1, "off")


def test_plugin_entry_point_is_discoverable_from_the_source_tree():
    import subprocess
    import sys
    code = ("from importlib.metadata import entry_points;"
            "print([e.value for e in entry_points(group='vllm.general_plugins')"
            " if e.name == 'awq_b200'])")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True,
                         env=replicas.replica_env(0, 1, "on")).stdout
    assert "awq_b200.vllm_plugin:register" in out


def test_balancer_policies():
    b = front.Balancer(["a", "b", "c"], "round_robin")
    picks = [b.acquire() for _ in range(7)]
    assert picks == [0, 1, 2, 0, 1, 2, 0]
    lc = front.Balancer(["a", "b", "c"], "least_conn")
    first = [lc.acquire() for _ in range(3)]
    assert sorted(first) == [0, 1, 2]              # an idle pool still spreads
    lc.release(1)
    assert lc.acquire() == 1                       # the only back end with a free slot
    with pytest.raises(ValueError):
        front.Balancer([], "round_robin")
    with pytest.raises(ValueError):
        front.Balancer(["a"], "random")


def _port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_front_spreads_requests_and_streams_through():
    import aiohttp
    from aiohttp import web

    async def scenario():
        runners, ports = [], []
        for name in ("r0", "r1"):
            async def chat(request, name=name):
                body = await request.json()
                resp = web.StreamResponse(headers={"Content-Type": "text/event-stream"})
                await resp.prepare(request)
                for i in range(3):
                    await resp.write(f"data: {name}:{body['n']}:{i}\n\n".encode())
                    await asyncio.sleep(0.01)
                await resp.write_eof()
                return resp

            async def models(request):
                return web.json_response({"object": "list", "data": []})

            app = web.Application()
            app.router.add_post("/v1/chat/completions", chat)
            app.router.add_get("/v1/models", models)
            runner = web.AppRunner(app)
            await runner.setup()
            port = _port()
            await web.TCPSite(runner, "127.0.0.1", port).start()
            runners.append(runner), ports.append(port)
        fapp = front.make_app([f"http://127.0.0.1:{p}" for p in ports], "round_robin")
        frunner = web.AppRunner(fapp)
        await frunner.setup()
        fport = _port()
        await web.TCPSite(frunner, "127.0.0.1", fport).start()
        seen = []
        async with aiohttp.ClientSession() as s:
            for n in range(4):
                async with s.post(f"http://127.0.0.1:{fport}/v1/chat/completions",
                                  json={"n": n}) as r:
                    assert r.status == 200
                    text = (await r.read()).decode()
                    assert text.count("data: ") == 3
                    seen.append(text.split(":")[1].strip())
            async with s.get(f"http://127.0.0.1:{fport}/v1/models") as r:
                assert (await r.json())["object"] == "list"
            async with s.get(f"http://127.0.0.1:{fport}/front/stats") as r:
                stats = await r.json()
        await frunner.cleanup()
        for r in runners:
            await r.cleanup()
        return seen, stats

    seen, stats = asyncio.run(scenario())
    assert seen == ["r0", "r1", "r0", "r1"]
    assert stats["served"] == [3, 2] and stats["active"] == [0, 0]


def test_client_command_carries_the_reference_flags():
    cmd = " ".join(client.benchmark_command("org/m", "http://127.0.0.1:8080", 1000, 1000, 16, 64,
                                            tokenizer="/m"))
    for piece in ("bench serve", "--model org/m", "--dataset-name random",
                  "--random-input-len 1000", "--random-output-len 1000", "--max-concurrency 16",
                  "--num-prompts 64", "--ignore-eos", "--backend openai-chat",
                  "--endpoint /v1/chat/completions", "--percentile-metrics ttft,tpot,itl,e2el",
                  "--base-url http://127.0.0.1:8080", "--tokenizer /m"):
        assert piece in cmd


def test_legacy_block_parses_with_the_reference_patterns():
    block = client.legacy_result_block(CLIENT_OUTPUT, "services:\n  vllm_0:\n    port: 1",
                                       "vllm bench serve --model m")
    assert block.startswith(client.RESULT_HEADER)
    assert "INFO starting" not in block
    got = {k: float(re.search(p, block).group(1)) for k, p in REFERENCE_PATTERNS.items()}
    assert got == {"total": 4096.0, "request": 2.05, "output": 2048.0, "ttft": 120.5,
                   "tpot": 7.25}
    assert re.search(REFERENCE_PATTERNS["total"], CLIENT_OUTPUT) is None   # the label drift
    assert "============ Docker Compose Configuration ============" in block
    assert "============ Benchmark Command ============" in block
    parsed = client.parse_result_block(block)
    assert parsed["total_token_throughput"] == 4096.0 and parsed["mean_tpot_ms"] == 7.25
    assert client.parse_result_block("nothing here") == {}
    with pytest.raises(ValueError):
        client.legacy_result_block("no block", "", "")


def test_result_file_name_matches_the_report_pattern():
    name = client.result_file_name("b200_x_8", "synthetic/Qwen3-30B-A3B-AWQ-random")
    assert name == "b200_x_8_synthetic_Qwen3-30B-A3B-AWQ-random_vllm_benchmark.txt"
    stem = name[:-len(".txt")].rsplit("_vllm_benchmark", 1)[0]
    m = re.match(REFERENCE_FILENAME, stem)
    assert m.group(1) == "b200_x_8" and m.group(2).replace("_", "/").startswith("synthetic/")
    with pytest.raises(ValueError):
        client.result_file_name("b200", "m")


def test_existing_result_is_not_rerun(tmp_path):
    args = run.parser().parse_args(["--results-dir", str(tmp_path), "--instances", "8"])
    name = client.result_file_name("b200_x_8", args.model_name)
    (tmp_path / name).write_text(client.legacy_result_block(CLIENT_OUTPUT, "services:", "cmd"))
    out = run.run(args)                            # no server is started: the file is there
    assert len(out["runs"]) == 1
    assert out["runs"][0]["skipped"] == "result exists"
    assert out["runs"][0]["total_token_throughput"] == 4096.0
    many = run.parser().parse_args(["--concurrency", "1,16", "--num-prompts", "8,64"])
    assert run._pairs(many) == [(1, 8), (16, 64)]
    assert run._pairs(run.parser().parse_args(["--concurrency", "1,16"])) == [(1, 100), (16, 100)]


def test_topology_text_lists_slices(tmp_path):
    args = run.parser().parse_args(["--instances", "2", "--tensor-parallel-size", "2"])
    envs = [replicas.replica_env(i, 2, "on") for i in range(2)]
    cmds = [replicas.serve_command("/m", "n", 8000 + i, 2) for i in range(2)]
    text = run.topology_text(args, [8000, 8001], cmds, envs)
    assert "device_ids: ['0', '1']" in text and "device_ids: ['2', '3']" in text
    assert "front:" in text and "policy: round_robin" in text
    assert serving.replica_gpu_list(1, 2) == "2,3"


def test_plugin_classes_pickle_by_reference():
    """vLLM pickles its config, quantization config object included, for every engine process it
    spawns: the plug-in's classes must be importable by name."""
    import pickle
    try:
        from awq_b200 import vllm_methods
    except Exception as e:  # pragma: no cover
        pytest.skip(f"vllm layer modules do not import here: {e}")
    for cls in (vllm_methods.B200AWQConfig, vllm_methods.B200AWQMarlinConfig,
                vllm_methods.B200AWQLinearMethod, vllm_methods.B200AWQMoEMethod):
        assert pickle.loads(pickle.dumps(cls)) is cls
    cfg = vllm_methods.B200AWQConfig(4, 128, True)
    back = pickle.loads(pickle.dumps(cfg))
    assert type(back) is vllm_methods.B200AWQConfig and back.group_size == 128


FAKE_SERVER = r'''
import sys
from aiohttp import web
port = int(sys.argv[sys.argv.index("--port") + 1])
async def health(r): return web.Response(text="ok")
async def models(r): return web.json_response({"object": "list", "data": [{"id": "m"}]})
async def chat(r):
    body = await r.json()
    return web.json_response({"choices": [{"message": {"content": "w1 w2"}}], "echo": body.get("n")})
app = web.Application()
app.router.add_get("/health", health); app.router.add_get("/v1/models", models)
app.router.add_post("/v1/chat/completions", chat)
web.run_app(app, host="127.0.0.1", port=port, print=None, access_log=None)
'''

FAKE_CLIENT = r'''
import sys, json, urllib.request
base = sys.argv[sys.argv.index("--base-url") + 1]
conc = sys.argv[sys.argv.index("--max-concurrency") + 1]
for n in range(4):      # really goes through the endpoint (and the front, when there is one)
    req = urllib.request.Request(base + "/v1/chat/completions", data=json.dumps({"n": n}).encode(),
                                 headers={"Content-Type": "application/json"})
    assert json.loads(urllib.request.urlopen(req, timeout=20).read())["echo"] == n
print("noise before the block")
print("============ Serving Benchmark Result ============")
print("Successful requests:                     4")
print("Maximum request concurrency:             " + conc)
print("Request throughput (req/s):              1.50")
print("Output token throughput (tok/s):         100.00")
print("Total token throughput (tok/s):          " + str(200 + int(conc)) + ".00")
print("Mean TTFT (ms):                          10.00")
print("Mean TPOT (ms):                          5.00")
print("==================================================")
'''


def test_run_orchestrates_replicas_front_and_client(tmp_path, monkeypatch):
    """serving.run.run from start to finish with stand-ins for the two vLLM programs: two fake
    servers on their GPU slices, the real front, a fake client that talks through it; the result
    files come out in the reference's layout and a second run skips them."""
    import sys
    server = tmp_path / "fake_server.py"
    server.write_text(FAKE_SERVER)
    fake_client = tmp_path / "fake_client.py"
    fake_client.write_text(FAKE_CLIENT)
    seen_env = []

    def fake_serve_command(model_dir_, served, port, tp_, pp_, extra):
        return [sys.executable, str(server), "x", "--port", str(port), "--model", model_dir_]

    real_env = replicas.replica_env

    def spy_env(i, per, plugin, seed, options=None):
        env = real_env(i, per, plugin, seed, options)
        seen_env.append((i, env["CUDA_VISIBLE_DEVICES"], env.get("AWQ_B200_DUMMY_FILL")))
        return env

    def fake_benchmark_command(model, base, inp, out, conc, prompts, tokenizer=None):
        return [sys.executable, str(fake_client), "x", "--base-url", base, "--max-concurrency",
                str(conc), "--num-prompts", str(prompts)]

    monkeypatch.setattr(replicas, "serve_command", fake_serve_command)
    monkeypatch.setattr(replicas, "replica_env", spy_env)
    monkeypatch.setattr(client, "benchmark_command", fake_benchmark_command)
    args = run.parser().parse_args([
        "--instances", "2", "--concurrency", "4,8", "--num-prompts", "4", "--num-layers", "1",
        "--results-dir", str(tmp_path / "results"), "--work-dir", str(tmp_path / "work"),
        "--startup-timeout", "60", "--client-timeout", "60", "--seed", "3"])
    out = run.run(args)
    assert out["server"] == "b200_x_2" and len(out["runs"]) == 2
    assert [r["concurrency"] for r in out["runs"]] == [4, 8]
    assert [r["total_token_throughput"] for r in out["runs"]] == [204.0, 208.0]
    assert sorted(seen_env) == [(0, "0", "3"), (1, "1", "3")]
    for r in out["runs"]:
        text = open(r["result_file"]).read()
        assert text.startswith(client.RESULT_HEADER) and "noise before" not in text
        assert re.search(REFERENCE_PATTERNS["total"], text)
        assert "vllm_0:" in text and "vllm_1:" in text and "front:" in text
        assert "============ Benchmark Command ============" in text
        name = r["result_file"].rsplit("/", 1)[1]
        assert re.match(REFERENCE_FILENAME, name[:-len(".txt")].rsplit("_vllm_benchmark", 1)[0])
    again = run.run(args)
    assert all(r.get("skipped") == "result exists" for r in again["runs"])
