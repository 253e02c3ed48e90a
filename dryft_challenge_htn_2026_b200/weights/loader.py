"""Fills a model's parameters from safetensors files, by tensor name.

The model says which names and shapes it wants (``CausalLM.param_decls``); the files say what
they hold. Every difference — missing, unexpected, wrong shape — is collected and raised as ONE
``WeightError``. Matrices are cast to the compute dtype (bfloat16 stays bfloat16); parameters a
part declares ``keep_float32`` (norm weights) are held in float32 whatever the file stores; integer
tensors would be held as int32. The reference loads every ``*.safetensors`` of the folder into one
dict and pops names from it (engine/engine.py:282-309), raising a bare KeyError on a missing name
and ignoring leftovers.
"""
import glob
import json
import os

import torch
from safetensors import safe_open


class WeightError(ValueError):
    def __init__(self, folder, missing, unexpected, wrong_shape):
        self.missing, self.unexpected, self.wrong_shape = sorted(missing), sorted(unexpected), sorted(wrong_shape)
        lines = [f"weights in {folder} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " +
                         ", ".join(f"{n} is {list(got)}, expected {list(exp)}" for n, got, exp in self.wrong_shape))
        super().__init__("\n".join(lines))


def _files(folder):
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            names = sorted(set(json.load(f)["weight_map"].values()))
        return [os.path.join(folder, n) for n in names]
    files = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no .safetensors file in {folder}")
    return files


def list_tensors(folder):
    """name -> (file, shape) for every tensor in the folder's safetensors files."""
    out = {}
    for fn in _files(folder):
        with safe_open(fn, framework="pt") as f:
            for k in f.keys():
                out[k] = (fn, tuple(f.get_slice(k).get_shape()))
    return out


def load_weights(model, folder):
    """Checks the folder against ``model`` and binds the tensors. Ties the head to the embedding
    when the spec says so, or, when the spec leaves it open, when the files have no head tensor
    (as the reference decides it, engine/engine.py:290). A head tensor in the files of a model whose
    config ties the head is accepted (published checkpoints of tied models ship one): its shape is
    checked, and it is bound as the head, as the reference does with a head tensor it finds."""
    have = list_tensors(folder)
    spec = model.spec
    if spec.tie_embeddings and spec.head_name in have:
        tied = False
    else:
        tied = spec.tie_embeddings if spec.tie_embeddings is not None else spec.head_name not in have
    decls = model.param_decls(tied)
    missing = [n for n in decls if n not in have]
    unexpected = [n for n in have if n not in decls]
    wrong = [(n, have[n][1], decls[n].shape) for n in decls if n in have and tuple(have[n][1]) != tuple(decls[n].shape)]
    if missing or unexpected or wrong:
        raise WeightError(folder, missing, unexpected, wrong)
    by_file = {}
    for n in decls:
        by_file.setdefault(have[n][0], []).append(n)
    tensors = {}
    dev, dtype = model.rt.device, model.rt.dtype
    for fn, names in by_file.items():
        with safe_open(fn, framework="pt") as f:
            for n in names:
                t = f.get_tensor(n)
                if not t.dtype.is_floating_point:
                    t = t.to(torch.int32)
                elif decls[n].keep_float32:
                    t = t.to(torch.float32)
                else:
                    t = t.to(dtype)
                tensors[n] = t.to(dev)
    model.bind(tensors, tied)
    return model
