"""Checkpoint loading in the reference's formats (reference: utils/loader.py:13-138).

The reference copies a checkpoint into an ``nn.Module``; the engine here is built from a plain
``{parameter name: tensor}`` dict with the reference's parameter names (``model.weights``), so the
loaders return that dict.  Accepted inputs, with the reference's resolution rules:

* a ``.pt`` file written by the training code (``{"model_state_dict", "optimizer_state_dict",
  "iteration"}``), a ``{"state_dict": ...}`` wrapper, or a bare state dict; a ``_orig_mod.``
  prefix left by ``torch.compile`` is stripped (loader.py:80-97);
* a directory: ``best_model.pt``, then ``final_model.pt``, then the highest
  ``checkpoint_iter_*.pt`` (loader.py:48-66); if it holds no ``.pt`` file, every ``*.safetensors``
  file in it (loader.py:13-36);
* a path without extension that exists with ``.pt`` appended (loader.py:133-136).
"""
from __future__ import annotations

import os
from glob import glob

import torch


def _strip_compile_prefix(state: dict) -> dict:
    if any(k.startswith("_orig_mod.") for k in state):
        return {k.replace("_orig_mod.", ""): v for k, v in state.items()}
    return dict(state)


def load_checkpoint(path: str) -> tuple[dict, int]:
    """(state dict, iteration) of a ``.pt`` checkpoint file or checkpoint directory."""
    checkpoint_path = path
    if os.path.isdir(path):
        candidates = [os.path.join(path, "best_model.pt"), os.path.join(path, "final_model.pt")]
        numbered = sorted(glob(os.path.join(path, "checkpoint_iter_*.pt")))
        if numbered:
            candidates.append(numbered[-1])
        for c in candidates:
            if os.path.exists(c):
                checkpoint_path = c
                break
        else:
            raise FileNotFoundError(f"No checkpoint file found in {path}")
    if not checkpoint_path.endswith(".pt"):
        checkpoint_path += ".pt"
    if not os.path.exists(checkpoint_path):
        raise FileNotFoundError(f"Checkpoint not found: {checkpoint_path}")
    # the training code pickles optimizer state next to the weights, hence weights_only=False as in
    # the reference; only load checkpoints you trust
    ckpt = torch.load(checkpoint_path, map_location="cpu", weights_only=False)
    iteration = 0
    if isinstance(ckpt, dict) and "model_state_dict" in ckpt:
        state, iteration = ckpt["model_state_dict"], ckpt.get("iteration", 0)
    elif isinstance(ckpt, dict) and "state_dict" in ckpt:
        state, iteration = ckpt["state_dict"], ckpt.get("iteration", 0)
    else:
        state = ckpt
    return _strip_compile_prefix(state), int(iteration)


def load_safetensors(path: str) -> dict:
    """All tensors of every ``*.safetensors`` file in a directory (or of one file)."""
    from safetensors import safe_open
    files = [path] if os.path.isfile(path) else sorted(glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"No safetensors files found in {path}")
    state = {}
    for file in files:
        with safe_open(file, "pt", "cpu") as f:
            for name in f.keys():
                state[name] = f.get_tensor(name)
    return _strip_compile_prefix(state)


def load_weights(path: str) -> dict:
    """Format detection of the reference's ``load_model`` (loader.py:109-138)."""
    if os.path.isfile(path) and path.endswith(".pt"):
        return load_checkpoint(path)[0]
    if os.path.isfile(path) and path.endswith(".safetensors"):
        return load_safetensors(path)
    if os.path.isdir(path):
        if glob(os.path.join(path, "*.pt")):          # .pt files win when both exist
            return load_checkpoint(path)[0]
        if glob(os.path.join(path, "*.safetensors")):
            return load_safetensors(path)
        raise FileNotFoundError(f"No checkpoint files found in {path}")
    if os.path.exists(path + ".pt"):
        return load_checkpoint(path + ".pt")[0]
    raise FileNotFoundError(f"Checkpoint not found: {path}")


def check_names(state: dict, expected: dict, strict: bool = True) -> tuple[list[str], list[str]]:
    """(missing, unexpected) parameter names of ``state`` against ``expected`` (e.g. the dict of
    ``init_reference_order`` for the same config), with a shape check on the common ones.  The
    reference loads with ``strict=False`` and only prints; the engine cannot run with missing
    weights, so ``strict`` raises."""
    missing = sorted(k for k in expected if k not in state)
    unexpected = sorted(k for k in state if k not in expected)
    bad = [k for k in expected if k in state and tuple(state[k].shape) != tuple(expected[k].shape)]
    if bad:
        k = bad[0]
        raise ValueError(f"shape mismatch for {k}: checkpoint {tuple(state[k].shape)}, model {tuple(expected[k].shape)}")
    if strict and missing:
        raise KeyError(f"checkpoint lacks {len(missing)} parameters, first: {missing[0]}")
    return missing, unexpected
