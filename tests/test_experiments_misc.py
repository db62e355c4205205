"""graph_trainer plan passes / bucketing / CUDA-graph wrapper plumbing and the forge engine, on CPU."""

import dataclasses

import pytest
import torch


def test_graph_trainer_passes_build_a_plan():
    from torchtitan_b200.experiments.graph_trainer.passes import build_plan

    p = build_plan(["auto_bucketing", "cudagraph"], ["apply_sac", "fsdp_reshard_after_fwd"])
    assert p.bucketing == "auto" and p.cudagraph and p.reshard_after_forward == "always" and p.prefetch_depth >= 2
    assert "tt_b200::gemm" in p.sac_save_ops
    with pytest.raises(ValueError, match="same time"):
        build_plan(["auto_bucketing", "transformer_block_bucketing"])
    with pytest.raises(ValueError, match="last pass"):
        build_plan(["cudagraph", "auto_bucketing"])
    with pytest.raises(ValueError, match="Unknown pass"):
        build_plan(["nope"])
    with pytest.raises(NotImplementedError, match="Inductor"):
        build_plan(["full_inductor_compilation"])


def test_graph_trainer_buckets():
    from torchtitan_b200.experiments.graph_trainer.simple_fsdp import auto_buckets, get_transformer_block_buckets
    from torchtitan_b200.models.llama3 import llama3_configs

    with torch.device("meta"):
        model = dataclasses.replace(llama3_configs["debugmodel"], n_layers=4).build()
    b = get_transformer_block_buckets(model)
    assert b == ["tok_embeddings", "layers.0", "layers.1", "layers.2", "layers.3", ["norm", "output"]]
    per_block = sum(p.numel() for p in model.layers["0"].parameters()) * 2
    a = auto_buckets(model, bucket_bytes=2 * per_block)
    assert a == ["tok_embeddings", ["layers.0", "layers.1"], ["layers.2", "layers.3"], ["norm", "output"]]


def test_cudagraph_wrapper_passthrough_and_checks():
    from torchtitan_b200.experiments.graph_trainer import CUDAGraphWrapper

    calls = []
    w = CUDAGraphWrapper(lambda a, b: calls.append(1) or a + b, enabled=False)
    assert torch.equal(w(torch.ones(2), torch.ones(2)), torch.full((2,), 2.0)) and len(calls) == 1
    w2 = CUDAGraphWrapper(lambda a: a, enabled=True, warmup=1)
    with pytest.raises(TypeError, match="args must be tensor"):
        w2("text")


def test_graph_trainer_config_conversion():
    from torchtitan_b200.experiments.graph_trainer import GraphTrainer
    from torchtitan_b200.experiments.graph_trainer.llama3.config_registry import graph_trainer_llama3_debugmodel_cudagraph

    cfg = graph_trainer_llama3_debugmodel_cudagraph()
    assert isinstance(cfg, GraphTrainer.Config) and cfg.compile.passes[-1] == "cudagraph" and cfg.compile.joint_passes == ["apply_sac"]
    assert cfg.model_spec.name == "llama3"


def test_forge_engine_trains_on_cpu(tmp_path, monkeypatch):
    from torchtitan_b200.components.dataloader import SyntheticDataLoader
    from torchtitan_b200.config import TrainingConfig
    from torchtitan_b200.experiments.forge import ForgeEngine
    from torchtitan_b200.experiments.forge.example_train import ExampleTrainer
    from torchtitan_b200.models.llama3 import model_registry

    monkeypatch.setenv("LOCAL_RANK", "0")
    spec = model_registry("debugmodel")
    spec.model = dataclasses.replace(spec.model, n_layers=2)
    cfg = ForgeEngine.Config(model_spec=spec, dump_folder=str(tmp_path),
                             training=TrainingConfig(local_batch_size=2, seq_len=32, steps=3, dtype="float32"))
    cfg.optimizer.lr = 1e-2
    t = ExampleTrainer(cfg, dataloader_config=SyntheticDataLoader.Config())
    losses = t.train()
    t.close()
    assert len(losses) == 3 and t.step == 3 and all(l == l for l in losses)
    assert t.dp_degree == 1 and t.model_param_count > 0 and t.num_flops_per_token > 0
