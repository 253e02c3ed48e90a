"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a config and
a seed. Matrices and embeddings N(0, 0.02), norm weights 1 + N(0, 0.1); drawn in float32 from a
seeded CPU generator, one tensor at a time in name order, then stored in the asked dtype. The
folder loads like any checkpoint (also by the reference engine: same tensor names)."""
import os

import torch
from safetensors.torch import save_file

from ..engine.model import CausalLM


def random_tensors(config, seed, dtype=torch.bfloat16, matrix_std=0.02, norm_std=0.1):
    spec = config.to_spec()
    tied = bool(spec.tie_embeddings)
    shell = CausalLM(spec, dtype=torch.float32, device="cpu")   # parts only; nothing runs on it
    gen = torch.Generator().manual_seed(int(seed))
    out = {}
    for name, decl in sorted(shell.param_decls(tied).items()):
        x = torch.randn(decl.shape, generator=gen, dtype=torch.float32)
        x = 1.0 + norm_std * x if decl.init == "norm" else matrix_std * x
        out[name] = x.to(dtype).contiguous()
    return out


def write_random_model(config, folder, seed=0, dtype=torch.bfloat16, matrix_std=0.02, norm_std=0.1):
    """Returns ``folder`` holding config.json and model.safetensors for ``config``."""
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    save_file(random_tensors(config, seed, dtype, matrix_std, norm_std), os.path.join(folder, "model.safetensors"))
    return folder


def bind_random(model, seed=0, matrix_std=0.02, norm_std=0.1):
    """Fills ``model`` with random weights drawn on its own device (no folder, no host copy):
    for sizes where writing and re-reading a checkpoint would only cost time."""
    spec = model.spec
    tied = bool(spec.tie_embeddings)
    gen = torch.Generator(device=model.rt.device).manual_seed(int(seed))
    tensors = {}
    for name, decl in sorted(model.param_decls(tied).items()):
        x = torch.randn(decl.shape, generator=gen, dtype=torch.float32, device=model.rt.device)
        x = 1.0 + norm_std * x if decl.init == "norm" else matrix_std * x
        tensors[name] = x if decl.keep_float32 else x.to(model.rt.dtype)
    model.bind(tensors, tied)
    return model
