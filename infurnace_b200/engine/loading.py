"""From a model folder to a runner: configuration, plan, weights, parts, cache."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..cache import CacheManager
from ..errors import ModelConfigError
from ..models import plan_for, read_config
from ..parts import DecoderModel, Runtime
from ..weights.loader import load_weights
from .runner import ModelRunner

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


@dataclass
class EngineOptions:
    """How much of the device an engine may use; none of these is a property of the model."""
    dtype: str = "bfloat16"
    device: str = "cuda"
    page_size: int = 16
    num_pages: Optional[int] = None            # pages of each key/value group
    max_num_seqs: int = 8                      # live requests (state slots)
    max_num_batched_tokens: int = 2048         # tokens of one step
    max_model_len: Optional[int] = None        # longest sequence; default: the model's limit
    memory_fraction: float = 0.8               # of free device memory, when num_pages is None


def parse_dtype(name):
    if isinstance(name, torch.dtype):
        return name
    try:
        return DTYPES[name]
    except KeyError:
        raise ModelConfigError(f"dtype {name!r}: choose bfloat16 or float32") from None


def build_runner(model_dir: Optional[str], options: EngineOptions, kernels=None, progress=None, random=None):
    """(config, plan, runner) for the model folder.  ``kernels`` None loads the CUDA kernel
    set, which fails loudly without a GPU or a compiler; tests may pass a stand-in.

    ``random`` = (config, seed, store_dtype name): no folder is read; the tensors are drawn on the
    device as the parts ask for them (weights/random_init.py), which is how models too large to pass
    through a file get their random weights."""
    dtype = parse_dtype(options.dtype)
    config = read_config(model_dir) if random is None else random[0]
    plan = plan_for(config)
    if kernels is None:
        from ..kernels import load_cuda_kernels
        kernels = load_cuda_kernels(progress=progress)
    runtime = Runtime(device=torch.device(options.device), act_dtype=dtype, kernels=kernels)
    if random is None:
        weights = load_weights(model_dir, plan, dtype, runtime.device, progress=progress)
    else:
        from ..weights.random_init import DeviceRandomWeights
        weights = DeviceRandomWeights(plan, random[1], dtype, runtime.device, kernels, store_dtype=parse_dtype(random[2]))
    model = DecoderModel(plan, weights, runtime)
    del weights
    max_len = min(options.max_model_len or plan.max_positions, plan.max_positions)
    num_pages = options.num_pages
    if num_pages is None:
        num_pages = default_num_pages(plan, options, dtype, runtime.device, max_len)
    cache = CacheManager(plan, options.page_size, num_pages, options.max_num_seqs, dtype=dtype, device=runtime.device)
    runner = ModelRunner(model, cache, runtime, options.max_num_batched_tokens, max_len)
    return config, plan, runner


def default_num_pages(plan, options, dtype, device, max_len) -> int:
    """Pages for ``max_num_seqs`` sequences of ``max_model_len``, capped by the share of
    free device memory that ``memory_fraction`` allows."""
    from ..cache import CacheLayout
    layout = CacheLayout(plan)
    per_page = 0
    esize = torch.empty((), dtype=dtype).element_size()
    for need, ids in layout.kv.values():
        per_page += len(ids) * sum(x.heads * x.width for x in need.streams) * options.page_size * esize
    want = options.max_num_seqs * (-(-max_len // options.page_size)) + 1
    if per_page == 0:
        return 1
    if device.type == "cuda":
        free, _ = torch.cuda.mem_get_info(device)
        fit = int(free * options.memory_fraction) // per_page
        want = max(1, min(want, fit))
    return want
