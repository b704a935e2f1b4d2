"""Options of an engine instance, filled by the command line or the Python entry point.

The reference keeps these as globals set by its flag loop (src/main.c:4491-4850) and as
environment variables read at the point of use; here they are one typed record and no
kernel reads the environment.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class EngineOptions:
    dtype: str = "bfloat16"          # "bfloat16" (serving kernels) or "float32" (true 32-bit path)
    page_size: int = 16              # tokens per cache page
    num_pages: int = 0               # pages per cache group; 0 = derive from max_tokens
    max_tokens: int = 0              # tokens all live requests may hold; 0 = what fits the device's free memory, at most batch_max * max_model_len
    memory_fraction: float = 0.9     # share of the free device memory the cache may take when its size is derived
    batch_max: int = 32              # live requests (the reference's --batch-max, vllm_batch.c:29)
    max_step_tokens: int = 2048      # token budget of one step
    prefill_batch: int = 512         # largest prompt portion (the reference's --prefill-batch)
    max_model_len: int = 0           # longest request; 0 = max_position_embeddings
    max_queued: int = 1 << 30        # waiting requests before admission refuses (--max-queued)
    seed: int = 0
    cuda_graphs: bool = True         # capture decode-only steps per batch-size bucket
    native_step: bool = True         # run steps from the model's step program through the native runner where every part offers one
    profile: bool = False            # time the phases of every step with CUDA events and print them in the reference's formats
    debug_guards: bool = False       # check every step's description on the device and guard words behind every activation
    device: str = "cuda:0"

    def normalised_dtype(self) -> str:
        d = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp32": "float32", "float32": "float32",
             "f32": "float32"}.get(self.dtype)
        if d is None:
            raise ValueError(f"dtype '{self.dtype}' is not one of bfloat16, float32")
        return d
