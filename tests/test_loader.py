"""Checkpoint formats of the reference's loader (utils/loader.py): what a user switching from the
reference has on disk must load into the engine's weight dict."""
import os

import pytest
import torch

from llm_from_scratch_b200.model import ModelConfig, init_reference_order
from llm_from_scratch_b200.utils import loader


@pytest.fixture(scope="module")
def weights():
    cfg = ModelConfig(vocab_size=50, context_length=16, d_model=32, num_layers=1, num_heads=4, num_kv_heads=2,
                      d_ff=48)
    return init_reference_order(cfg, 0)


def _same(a, b):
    assert a.keys() == b.keys()
    assert all(torch.equal(a[k], b[k]) for k in a)


def test_training_checkpoint_file_and_compile_prefix(tmp_path, weights):
    p = tmp_path / "ckpt.pt"
    torch.save({"model_state_dict": {"_orig_mod." + k: v for k, v in weights.items()},
                "optimizer_state_dict": {"state": {}}, "iteration": 1234}, p)
    state, it = loader.load_checkpoint(str(p))
    assert it == 1234
    _same(state, weights)
    _same(loader.load_weights(str(p)), weights)
    _same(loader.load_weights(str(tmp_path / "ckpt")), weights)      # extension appended


def test_bare_state_dict_and_state_dict_wrapper(tmp_path, weights):
    torch.save(dict(weights), tmp_path / "a.pt")
    torch.save({"state_dict": dict(weights), "iteration": 7}, tmp_path / "b.pt")
    _same(loader.load_weights(str(tmp_path / "a.pt")), weights)
    state, it = loader.load_checkpoint(str(tmp_path / "b.pt"))
    assert it == 7
    _same(state, weights)


def test_directory_resolution_order(tmp_path, weights):
    marked = {k: v.clone() for k, v in weights.items()}
    first = next(iter(marked))
    for name, mark in (("checkpoint_iter_100.pt", 1.0), ("checkpoint_iter_900.pt", 2.0), ("final_model.pt", 3.0)):
        marked[first] = torch.full_like(weights[first], mark)
        torch.save({"model_state_dict": dict(marked)}, tmp_path / name)
    assert loader.load_weights(str(tmp_path))[first].flatten()[0].item() == 3.0     # final_model.pt
    marked[first] = torch.full_like(weights[first], 4.0)
    torch.save({"model_state_dict": dict(marked)}, tmp_path / "best_model.pt")
    assert loader.load_weights(str(tmp_path))[first].flatten()[0].item() == 4.0     # best_model.pt wins
    os.remove(tmp_path / "best_model.pt")
    os.remove(tmp_path / "final_model.pt")
    assert loader.load_weights(str(tmp_path))[first].flatten()[0].item() == 2.0     # highest iteration


def test_safetensors_directory(tmp_path, weights):
    from safetensors.torch import save_file
    names = sorted(weights)
    half = len(names) // 2
    save_file({k: weights[k].contiguous() for k in names[:half]}, str(tmp_path / "model-00001.safetensors"))
    save_file({k: weights[k].contiguous() for k in names[half:]}, str(tmp_path / "model-00002.safetensors"))
    _same(loader.load_weights(str(tmp_path)), weights)


def test_missing_paths_and_name_check(tmp_path, weights):
    with pytest.raises(FileNotFoundError):
        loader.load_weights(str(tmp_path / "nothing"))
    with pytest.raises(FileNotFoundError):
        loader.load_weights(str(tmp_path))
    partial = dict(weights)
    dropped = sorted(partial)[0]
    del partial[dropped]
    partial["extra.weight"] = torch.zeros(1)
    missing, unexpected = loader.check_names(partial, weights, strict=False)
    assert missing == [dropped] and unexpected == ["extra.weight"]
    with pytest.raises(KeyError):
        loader.check_names(partial, weights)
    wrong = dict(weights)
    wrong[dropped] = torch.zeros(3, 3, 3)
    with pytest.raises(ValueError):
        loader.check_names(wrong, weights)
