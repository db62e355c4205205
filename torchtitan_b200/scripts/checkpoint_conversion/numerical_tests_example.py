"""Numerical check of a converted checkpoint: KL divergence between the logits of the Hugging Face model and of the
native model loaded from the converted DCP checkpoint, on random token batches.
``python -m torchtitan_b200.scripts.checkpoint_conversion.numerical_tests_example <hf_dir> <dcp_dir> --model_name llama3
--model_flavor 8B``. Parity: scripts/checkpoint_conversion/numerical_tests_example.py."""

import argparse
import importlib

import torch
import torch.distributed.checkpoint as dcp
import torch.nn.functional as F


def loss_fn(logits_a: torch.Tensor, logits_b: torch.Tensor) -> torch.Tensor:
    """KL(softmax(a) || softmax(b)) averaged over tokens."""
    pa = F.log_softmax(logits_a.float().flatten(0, 1), dim=-1)
    pb = F.log_softmax(logits_b.float().flatten(0, 1), dim=-1)
    return F.kl_div(pb, pa, log_target=True, reduction="batchmean")


@torch.no_grad()
def forward_hf(hf_dir: str, batches):
    from transformers import AutoModelForCausalLM

    model = AutoModelForCausalLM.from_pretrained(hf_dir, torch_dtype=torch.float32).eval()
    return [model(input_ids=b).logits for b in batches]


@torch.no_grad()
def forward_native(dcp_dir: str, model_name: str, flavor: str, batches):
    spec = importlib.import_module(f"torchtitan_b200.models.{model_name}").model_registry(flavor)
    model = spec.model.build()
    model.init_weights()
    sd = model.state_dict()
    dcp.load(sd, checkpoint_id=dcp_dir)
    model.load_state_dict(sd, strict=False)
    model.eval()
    return [model(b) for b in batches]


def main(argv=None) -> float:
    p = argparse.ArgumentParser()
    p.add_argument("hf_dir")
    p.add_argument("dcp_dir")
    p.add_argument("--model_name", default="llama3")
    p.add_argument("--model_flavor", default="8B")
    p.add_argument("--vocab", type=int, default=2000)
    p.add_argument("--batches", type=int, default=4)
    a = p.parse_args(argv)
    g = torch.Generator().manual_seed(0)
    batches = [torch.randint(0, a.vocab, (1, 128), generator=g) for _ in range(a.batches)]
    kl = torch.stack([loss_fn(x, y) for x, y in zip(forward_hf(a.hf_dir, batches), forward_native(a.dcp_dir, a.model_name, a.model_flavor, batches))])
    print(f"average KL divergence: {kl.mean().item():.3e}")
    return kl.mean().item()


if __name__ == "__main__":
    main()
