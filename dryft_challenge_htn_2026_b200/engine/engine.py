"""The Python entry point, in the manner of the reference's ``Engine`` (engine/engine.py:247-279,
683-732): ``Engine(model_path, dtype)`` and ``Engine.generate(input_ids, max_new_tokens)``, a
generator that yields one token per sequence per step. Beyond the reference: prompts of unequal
lengths run as one batch, sampling takes a temperature and a seed, sequences may end at stop
tokens, and ``generate_all`` runs as many batches one after another as there are requests.
"""
import torch

from ..csrc.api import PAGE
from ..registry import config_from_folder
from ..sampling import SamplingParams, request_seed
from ..weights import bind_random, load_weights
from .generate import GpuBackend, plan_batches, run_batch
from .model import CausalLM
from .runner import Runner


def _dtype(dtype):
    if isinstance(dtype, str):
        try:
            return {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}[dtype]
        except KeyError:
            raise ValueError(f"dtype must be bfloat16 or float32, not {dtype!r}") from None
    return dtype


def load_model(model_path, dtype=torch.bfloat16, device="cuda"):
    """The model class is chosen by config.json's ``architectures``; weights by tensor name."""
    config = config_from_folder(model_path)
    model = CausalLM(config.to_spec(), _dtype(dtype), device)
    load_weights(model, model_path)
    return model


def random_model(config, seed=0, dtype=torch.bfloat16, device="cuda"):
    """A model of ``config`` with seeded random weights drawn on the device."""
    return bind_random(CausalLM(config.to_spec(), _dtype(dtype), device), seed)


class Engine:
    def __init__(self, model_path=None, dtype=torch.bfloat16, model=None, max_tokens=None, use_graph=True,
                 max_prefill_tokens=32768):
        """``model_path``: folder with config.json and safetensors (or pass a built ``model``).
        ``max_tokens``: cache size in tokens; by default the cache is sized by each call.
        ``max_prefill_tokens``: most prompt tokens one step runs; a batch of prompts beyond it is
        prefilled in several steps (whole sequences, a longer one in chunks), with equal results."""
        self.model = model if model is not None else load_model(model_path, dtype)
        self.use_graph = use_graph
        self.max_prefill_tokens = max_prefill_tokens
        self.runner = None
        self.backend = None
        self._fixed_tokens = max_tokens
        if max_tokens is not None:
            self._resize(max_tokens, 1024)

    def _resize(self, tokens, slots):
        self.backend = self.runner = None   # drop the old cache before the new one is allocated
        torch.cuda.empty_cache()
        self.runner = Runner(self.model, tokens, slots)
        self.backend = GpuBackend(self.runner, self.use_graph, self.max_prefill_tokens)

    def _ensure(self, prompts, max_new_tokens):
        need = sum((len(p) + max_new_tokens + PAGE - 1) // PAGE * PAGE for p in prompts)
        if self.runner is None or self.runner.cache.num_pages * PAGE < need or self.runner.cache.max_slots < len(prompts):
            if self._fixed_tokens is not None:
                raise ValueError(f"batch needs {need} cache tokens, engine was built with max_tokens={self._fixed_tokens}")
            self._resize(need, max(len(prompts), 64))

    def generate(self, input_ids, max_new_tokens, temperature=0.0, seed=0, stop_token_ids=(), first_index=0):
        """Yields, ``max_new_tokens`` times at most, a list with the next token of every sequence
        (None once a sequence has ended at a stop token). All sequences start together; their
        prompts may have different lengths. Greedy unless ``temperature`` > 0."""
        if max_new_tokens <= 0 or not input_ids:
            return
        if any(len(p) == 0 for p in input_ids):
            raise ValueError("every prompt needs at least one token")
        params = SamplingParams(max_new_tokens, float(temperature), int(seed), tuple(stop_token_ids))
        self._ensure(input_ids, max_new_tokens)
        seeds = [request_seed(seed, first_index + i) for i in range(len(input_ids))]
        yield from run_batch(self.backend, [list(p) for p in input_ids], params, seeds)

    def generate_all(self, prompts, max_new_tokens, temperature=0.0, seed=0, stop_token_ids=(), batch_size=64):
        """Token lists for any number of requests, run ``batch_size`` at a time, one batch after
        another; a request's tokens do not depend on which batch it lands in."""
        out = [None] * len(prompts)
        for idx in plan_batches(len(prompts), batch_size):
            seqs = [[] for _ in idx]
            for row in self.generate([prompts[i] for i in idx], max_new_tokens, temperature, seed, stop_token_ids,
                                     first_index=idx.start):
                for k, t in enumerate(row):
                    if t is not None:
                        seqs[k].append(t)
            for k, i in enumerate(idx):
                out[i] = seqs[k]
        return out
