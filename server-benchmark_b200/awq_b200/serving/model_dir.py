"""Random-init AWQ model directories that an unmodified ``vllm serve --load-format dummy`` can
load with no network: ``config.json`` of the architecture (with the ``quantization_config`` an
AutoAWQ export carries, so vLLM's own detection picks the AWQ route with no --quantization flag,
reference utils/generate_compose.py:85-93), a synthetic WordLevel tokenizer and a one-line chat
template (the client posts to /v1/chat/completions, reference
benchmarks/3_vllm_benchmark.sh:151-162).

The tokenizer has one whitespace-separated word per id, so decoding random ids and encoding the
text again preserves the token count, which is what ``vllm bench serve --dataset-name random``
relies on (vllm/benchmarks/datasets/datasets.py:470-524).
"""
from __future__ import annotations

import json
import os

AWQ_QUANT = {"quant_method": "awq", "bits": 4, "group_size": 128, "zero_point": True,
             "version": "gemm"}

EOS = "<|endoftext|>"

ARCHITECTURES = {
    # Qwen3-30B-A3B: 48 layers, hidden 2048, 32 q / 4 kv heads of 128, 128 experts top-8,
    # expert intermediate 768, vocab 151936
    "qwen3-30b-a3b": {
        "architectures": ["Qwen3MoeForCausalLM"], "model_type": "qwen3_moe",
        "hidden_size": 2048, "num_hidden_layers": 48, "num_attention_heads": 32,
        "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 6144,
        "moe_intermediate_size": 768, "num_experts": 128, "num_experts_per_tok": 8,
        "norm_topk_prob": True, "decoder_sparse_step": 1, "mlp_only_layers": [],
        "vocab_size": 151936, "max_position_embeddings": 40960, "rope_theta": 1000000.0,
        "rms_norm_eps": 1e-6, "hidden_act": "silu", "attention_bias": False,
        "tie_word_embeddings": False, "router_aux_loss_coef": 0.001,
        "output_router_logits": False, "use_sliding_window": False, "sliding_window": None,
    },
    # Qwen2.5-72B: 80 layers, hidden 8192, 64 q / 8 kv heads of 128, vocab 152064.  The
    # intermediate size is 29568 = 231 groups of 128; the tensor-parallel variant below pads it to
    # 232 groups so that every rank of TP 2/4/8 holds whole groups (vLLM's AWQ create_weights
    # refuses partial groups, awq.py:198-203).
    "qwen2.5-72b": {
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
        "hidden_size": 8192, "num_hidden_layers": 80, "num_attention_heads": 64,
        "num_key_value_heads": 8, "intermediate_size": 29568, "vocab_size": 152064,
        "max_position_embeddings": 32768, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
        "hidden_act": "silu", "tie_word_embeddings": False, "use_sliding_window": False,
        "sliding_window": None,
    },
}
ARCHITECTURES["qwen2.5-72b-tp"] = dict(ARCHITECTURES["qwen2.5-72b"], intermediate_size=29696)


def _tokenizer_json(vocab_size: int) -> dict:
    vocab = {EOS: 0}
    for i in range(1, vocab_size):
        vocab[f"w{i}"] = i
    return {
        "version": "1.0", "truncation": None, "padding": None,
        "added_tokens": [{"id": 0, "content": EOS, "single_word": False, "lstrip": False,
                          "rstrip": False, "normalized": False, "special": True}],
        "normalizer": None,
        "pre_tokenizer": {"type": "WhitespaceSplit"},
        "post_processor": None, "decoder": None,
        "model": {"type": "WordLevel", "vocab": vocab, "unk_token": EOS},
    }


def write_model_dir(path: str, arch: str = "qwen3-30b-a3b", num_layers: int | None = None,
                    max_model_len: int | None = None) -> str:
    """Write config.json, generation_config.json, tokenizer.json and tokenizer_config.json under
    ``path`` (created if needed; files that exist are overwritten).  ``num_layers`` shortens the
    stack (for tests); the benchmark uses the architecture's own depth."""
    if arch not in ARCHITECTURES:
        raise ValueError(f"unknown architecture {arch!r}; known: {sorted(ARCHITECTURES)}")
    cfg = dict(ARCHITECTURES[arch])
    if num_layers is not None:
        cfg["num_hidden_layers"] = int(num_layers)
    if max_model_len is not None:
        cfg["max_position_embeddings"] = int(max_model_len)
    cfg.update({"torch_dtype": "float16", "bos_token_id": 0, "eos_token_id": 0,
                "quantization_config": dict(AWQ_QUANT), "use_cache": True})
    os.makedirs(path, exist_ok=True)

    def dump(name, obj):
        with open(os.path.join(path, name), "w") as f:
            json.dump(obj, f)

    dump("config.json", cfg)
    dump("generation_config.json", {"bos_token_id": 0, "eos_token_id": 0, "do_sample": False})
    dump("tokenizer.json", _tokenizer_json(cfg["vocab_size"]))
    dump("tokenizer_config.json", {
        "tokenizer_class": "PreTrainedTokenizerFast", "eos_token": EOS, "pad_token": EOS,
        "unk_token": EOS, "model_max_length": cfg["max_position_embeddings"],
        "clean_up_tokenization_spaces": False,
        "chat_template": "{% for message in messages %}{{ message['content'] }} {% endfor %}",
    })
    return path
