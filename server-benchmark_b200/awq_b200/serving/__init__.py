"""End-to-end serving measurement, the harness side of the reference: random-init AWQ model
directories with a synthetic tokenizer (model_dir), replica launch on contiguous GPU slices with
a load-balancing front (replicas, front) and the OpenAI-endpoint client run with the legacy
result block (client)."""
from .client import (benchmark_command, legacy_result_block, parse_result_block,  # noqa: F401
                     result_file_name)
from .model_dir import ARCHITECTURES, write_model_dir  # noqa: F401
from .replicas import replica_gpu_list, serve_command  # noqa: F401
