"""User-facing scripts: sampling helpers, loss-log parsing / comparison, checkpoint conversion round trip, asset selection."""

import dataclasses
import os

import torch


def test_generate_greedy_and_top_k():
    from torchtitan_b200.models.llama3 import llama3_configs
    from torchtitan_b200.scripts.generate._generation import generate, top_k_filter

    torch.manual_seed(0)
    model = dataclasses.replace(llama3_configs["debugmodel"], n_layers=1).build()
    model.init_weights()
    ids = torch.tensor([[1, 2, 3]])
    a = generate(model, ids, max_new_tokens=4, temperature=0)
    b = generate(model, ids, max_new_tokens=4, temperature=0)
    assert a.shape == (1, 7) and torch.equal(a, b) and torch.equal(a[:, :3], ids)
    c = generate(model, ids, max_new_tokens=4, temperature=1.0, top_k=5, seed=3)
    d = generate(model, ids, max_new_tokens=4, temperature=1.0, top_k=5, seed=3)
    assert torch.equal(c, d)
    f = top_k_filter(torch.tensor([[1.0, 2.0, 3.0, 4.0]]), 2)
    assert torch.isinf(f[0, :2]).all() and f[0, 2:].tolist() == [3.0, 4.0]
    # top-k restricts what can be drawn; nucleus sampling with a tiny p is greedy
    e = generate(model, ids, max_new_tokens=3, temperature=1.0, top_p=1e-6, seed=1)
    assert torch.equal(e, generate(model, ids, max_new_tokens=3, temperature=0))


def test_loss_compare_parsing_and_compare(tmp_path):
    from torchtitan_b200.scripts import loss_compare as lc

    text = "\x1b[31mstep:  1  \x1b[32mloss:  7.12345  grad_norm: 1.0\nnoise\nstep:  2  loss:  6.50000  x\nvalidate step:  2  loss: 9.0\n"
    losses = lc.parse_losses_from_log(text)
    assert losses == {1: 7.12345, 2: 6.5}
    assert lc.compare(losses, dict(losses), True)
    assert not lc.compare(losses, {1: 7.12345, 2: 6.5001}, True)
    f = tmp_path / "golden.txt"
    lc.export_losses(str(f), losses)
    assert lc.import_losses(str(f)) == losses
    cmd = lc.build_command("llama3", "llama3_debugmodel", 2, 5, "--training.seq_len 64", "out", None)
    assert "--debug.deterministic" in cmd and "--training.steps=5" in cmd and "--nproc-per-node=2" in cmd


def test_checkpoint_conversion_round_trip(tmp_path):
    """native -> HF safetensors -> native DCP, weights unchanged."""
    import torch.distributed.checkpoint as dcp

    from torchtitan_b200.models import llama3
    from torchtitan_b200.scripts.checkpoint_conversion.convert_from_hf import convert_from_hf
    from torchtitan_b200.scripts.checkpoint_conversion.convert_to_hf import convert_to_hf

    cfg = llama3.llama3_configs["debugmodel"]
    torch.manual_seed(0)
    model = cfg.build()
    model.init_weights()
    src = {k: v.clone() for k, v in model.state_dict().items()}
    dcp.save(src, checkpoint_id=str(tmp_path / "dcp0"))
    convert_to_hf(tmp_path / "dcp0", tmp_path / "hf", "llama3", "debugmodel", None, "float32")
    assert any(f.endswith(".safetensors") for f in os.listdir(tmp_path / "hf"))
    convert_from_hf(tmp_path / "hf", tmp_path / "dcp1", "llama3", "debugmodel")
    back = {k: torch.empty_like(v) for k, v in src.items()}
    dcp.load(back, checkpoint_id=str(tmp_path / "dcp1"))
    for k in src:
        assert torch.equal(src[k], back[k]), k


def test_download_asset_selection():
    from torchtitan_b200.scripts.download_hf_assets import select_files

    files = ["tokenizer.json", "config.json", "model-00001-of-00002.safetensors", "model.safetensors.index.json", "README.md",
             "original/tokenizer.model"]
    assert select_files(files, ["tokenizer"]) == ["tokenizer.json", "original/tokenizer.model"]
    assert select_files(files, ["index"]) == ["model.safetensors.index.json"]
    assert set(select_files(files, ["safetensors", "config"])) == {"config.json", "model-00001-of-00002.safetensors",
                                                                    "model.safetensors.index.json"}
    assert select_files(files, [], download_all=True) == files
    assert select_files(files, ["config"], additional_patterns=["*.md"]) == ["config.json", "README.md"]
